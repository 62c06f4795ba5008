"""CPU checks of the oracle itself (no GPU, no shipped code involved).

The oracle is pinned three ways: bit-for-bit against the reference's own emitted
C where that is built (oracle/_ref, from ilang-python/annotated-flashattn.c),
bit-for-bit against golden outputs of that same program committed under
tests/golden/, and against float64 NumPy on the reference's own test cases
(ilang-python/test.py:40-128, ilang-python/flash-attn.py:31-77).
"""
import glob
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def rand(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "attention_*.npz"))))
def test_fused_attention_matches_golden_bitwise(oracle, path):
    g = np.load(path)
    got = oracle.attention_fused(g["q"], g["k"], g["v"])
    assert got.shape == g["o"].shape
    assert np.array_equal(got, g["o"]), "restated oracle differs from the reference's emitted C"


@pytest.mark.parametrize("shape", [(128, 128, 64, 64), (100, 40, 24, 40), (17, 33, 7, 5),
                                   (1, 1, 1, 1), (33, 100, 128, 128), (16, 16, 8, 8)])
def test_fused_attention_matches_reference_build_bitwise(oracle, shape):
    if not oracle.have_reference():
        pytest.skip("oracle/_ref not built (reference checkout absent)")
    nq, nk, d, dv = shape
    q, k, v = rand((nq, d), 1), rand((nk, d), 2), rand((nk, dv), 3)
    assert np.array_equal(oracle.attention_fused(q, k, v), oracle.reference_attention(q, k, v))


def test_row_slices_reproduce_full_run(oracle):
    q, k, v = rand((96, 32), 1), rand((80, 32), 2), rand((80, 16), 3)
    full = oracle.attention_fused(q, k, v)
    part = oracle.attention_fused(q[32:64], k, v)
    assert np.array_equal(full[32:64], part)


def test_demo_attention_close_to_numpy(oracle):
    # ilang-python/flash-attn.py:31-36, 67-77 — rtol 3e-4, atol 5e-5.
    q, k, v = rand((32, 2048), 1), rand((32, 2048), 2), rand((32, 2048), 3)
    ref = oracle.numpy_attention(q, k, v)
    for fn in (oracle.attention_fused, oracle.attention_naive):
        np.testing.assert_allclose(fn(q, k, v), ref, rtol=3e-4, atol=5e-5)


def test_matmul_case(oracle):
    # ilang-python/test.py:40-59 — 8x16 @ 16x7, rtol 1e-5 / atol 1e-6.
    a, b = rand((8, 16), 1), rand((16, 7), 2)
    got = oracle.contract(a, b, a_kmajor=True, b_kmajor=False)
    np.testing.assert_allclose(got, a.astype(np.float64) @ b.astype(np.float64), rtol=1e-5, atol=1e-6)
    got_t = oracle.contract(a, np.ascontiguousarray(b.T), True, True)
    assert np.array_equal(got, got_t)


def test_row_reductions(oracle):
    # ilang-python/test.py:103-128 — rowmax / rowmin / rowsum on 16x8.
    x = rand((16, 8), 1)
    assert np.array_equal(oracle.reduce_rows(">", x), x.max(axis=1))
    assert np.array_equal(oracle.reduce_rows("<", x), x.min(axis=1))
    np.testing.assert_allclose(oracle.reduce_rows("+", x), x.astype(np.float64).sum(axis=1),
                               rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(oracle.reduce_rows("*", x), x.astype(np.float64).prod(axis=1),
                               rtol=1e-5, atol=1e-6)
    empty = np.zeros((3, 0), dtype=np.float32)
    assert np.array_equal(oracle.reduce_rows("+", empty), np.zeros(3, np.float32))
    assert np.all(np.isneginf(oracle.reduce_rows(">", empty)))


def test_unary_defaults(oracle):
    # compiler/src/lower/exec_plan_to_module.rs:605-640, 1216-1241.
    x = np.array([-2.0, -0.5, 0.0, 0.5, 3.0], dtype=np.float32)
    assert np.array_equal(oracle.map_unary("-", x), -x)
    assert np.array_equal(oracle.map_unary("/", x[[0, 1, 3, 4]]), 1.0 / x[[0, 1, 3, 4]])
    assert np.array_equal(oracle.map_unary(">", x), np.maximum(x, 0))     # ReLU, not -inf
    assert np.array_equal(oracle.map_unary("<", x), np.minimum(x, 0))
    assert np.array_equal(oracle.map_unary("+", x), x)
    np.testing.assert_allclose(oracle.map_unary("^", x), np.exp(x.astype(np.float64)), rtol=3e-7)
    np.testing.assert_allclose(oracle.map_unary("$", x[3:]), np.log(x[3:].astype(np.float64)), rtol=2e-7)


LOGIC_VALUES = np.array([-2.0, -0.0, 0.0, 0.5, 3.0, np.nan, np.inf, -np.inf], dtype=np.float32)


def test_comparisons_and_logic(oracle):
    # C operators on floats, result stored as 0.0f / 1.0f (compiler/src/backends/c/expr.rs:136-146,
    # xor :331-339); unary forms compiler/src/lower/exec_plan_to_module.rs:613-637.
    a = np.repeat(LOGIC_VALUES, LOGIC_VALUES.size).reshape(LOGIC_VALUES.size, -1)
    b = np.ascontiguousarray(a.T)
    ta, tb = a != 0, b != 0                    # NaN is true
    with np.errstate(invalid="ignore"):
        expect = {">>": a > b, ">=": a >= b, "<<": a < b, "<=": a <= b, "==": a == b, "!=": a != b,
                  "&&": ta & tb, "||": ta | tb, "^^": ta ^ tb}
        for op, want in expect.items():
            assert np.array_equal(oracle.map_binary(op, a, b), want.astype(np.float32)), op
        x = LOGIC_VALUES
        unary = {">>": x > 0, ">=": x >= 0, "<<": x < 0, "<=": x <= 0, "==": x == 0, "!=": x != 0,
                 "!!": x == 0}
        for op, want in unary.items():
            assert np.array_equal(oracle.map_unary(op, x), want.astype(np.float32)), op
    for op in ("&&", "||", "^^"):              # unary logic copies its operand
        assert np.array_equal(oracle.map_unary(op, x), x, equal_nan=True), op


def test_logic_reductions(oracle):
    # identities 1, 0, 0 (exec_plan_to_module.rs:592-603); dst = dst OP x over ascending columns.
    x = (rand((32, 9), 5) > 0.3).astype(np.float32) * rand((32, 9), 6)
    t = x != 0
    assert np.array_equal(oracle.reduce_rows("&&", x), t.all(axis=1).astype(np.float32))
    assert np.array_equal(oracle.reduce_rows("||", x), t.any(axis=1).astype(np.float32))
    assert np.array_equal(oracle.reduce_rows("^^", x), (t.sum(axis=1) % 2).astype(np.float32))
    empty = np.zeros((3, 0), dtype=np.float32)
    assert np.array_equal(oracle.reduce_rows("&&", empty), np.ones(3, np.float32))
    assert np.array_equal(oracle.reduce_rows("||", empty), np.zeros(3, np.float32))
    assert np.array_equal(oracle.reduce_rows("^^", empty), np.zeros(3, np.float32))
    one = np.array([[2.5], [0.0]], dtype=np.float32)      # a single element still becomes 0 / 1
    assert np.array_equal(oracle.reduce_rows("&&", one), np.array([1, 0], np.float32))
    assert np.array_equal(oracle.reduce_rows("^^", one), np.array([1, 0], np.float32))


def test_binary_log_drops_second_operand(oracle):
    # compiler/src/backends/c/expr.rs:136, 319-321.
    a = np.array([[1.0, 2.0], [3.0, 4.0]], dtype=np.float32)
    b = np.full((2, 2), 7.0, dtype=np.float32)
    assert np.array_equal(oracle.map_binary("$", a, b), oracle.map_unary("$", a))


def test_row_softmax_close_to_numpy(oracle):
    x = 2.0 * rand((64, 1000), 1)
    ref = np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True))
    ref /= ref.sum(axis=1, keepdims=True)
    got = oracle.row_softmax(x)
    assert float((np.abs(got - ref) / ref).max()) < 2e-5
    np.testing.assert_allclose(got.sum(axis=1), 1.0, rtol=1e-5)


def test_broadcast_modes(oracle):
    a, r, c = rand((5, 7), 1), rand((5,), 2), rand((7,), 3)
    assert np.array_equal(oracle.map_binary("-", a, r, mode=1), a - r[:, None])
    assert np.array_equal(oracle.map_binary("-", r, a, mode=2), r[:, None] - a)
    assert np.array_equal(oracle.map_binary("*", a, c, mode=3), a * c[None, :])
    assert np.array_equal(oracle.map_binary("/", c, a, mode=4), c[None, :] / a)
