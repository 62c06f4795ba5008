"""Writes the golden fixtures of this directory.

Run where the reference checkout is present (`make -C oracle` must have built
oracle/_ref/libref_flashattn.so from the reference's own emitted C,
ilang-python/annotated-flashattn.c).  Each fixture stores seeded inputs and the
output of the reference's `exec` on them, so parity can be checked on machines
that have neither the reference nor its build.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402


def attention_case(name, seed, nq, nk, d, dv, scale=True):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((nq, d), dtype=np.float32)
    k = rng.standard_normal((nk, d), dtype=np.float32)
    v = rng.standard_normal((nk, dv), dtype=np.float32)
    if scale:
        q *= np.float32(1.0 / np.sqrt(d))
    o = oracle.reference_attention(q, k, v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), q=q, k=k, v=v, o=o)
    print(name, o.shape, float(np.abs(o).max()))


def main():
    if not oracle.have_reference():
        raise SystemExit("oracle/_ref is not built; run `make -C oracle` with the reference present")
    # The reference README attention, 128x64, seed 0, Q pre-scaled by 1/sqrt(64).
    attention_case("attention_cfg1_128x64_seed0", 0, 128, 128, 64, 64)
    # Ragged in every extent (tail guards of the 16-wide tiles).
    attention_case("attention_ragged_100x40_seed5", 5, 100, 77, 40, 24)
    # The reference demo's shape class: few rows, very wide features
    # (ilang-python/flash-attn.py:31-36 uses 32x32x2048; 32x32x256 keeps the file small).
    attention_case("attention_wide_32x32x256_seed1", 1, 32, 32, 256, 256, scale=False)


if __name__ == "__main__":
    main()
