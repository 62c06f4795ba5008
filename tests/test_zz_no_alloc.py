"""ib_attention_static: the entry point for callers that cannot allocate device
memory when they call (memory owned by another allocator, latency-critical
loops, frameworks that forbid allocation in the calling context).  Its scratch
is a fixed array inside the library, so the test checks three things through
the C ABI: the result equals ib_attention's fp32 arm on the same inputs, a
second call right after the first (other shapes, stale scratch in place) is
still right, and a problem larger than the array is refused with a message
instead of overrunning it.

Collected last on purpose (file name), so a run that stops at the first failure
has already run every other test."""
import ctypes

import numpy as np
import pytest

from conftest import last_error, max_rel_to_peak

pytestmark = pytest.mark.gpu

FP32 = 1
STATIC_BYTES = 32 << 20          # IB_ATTENTION_STATIC_BYTES in include/i_b200.h


def declare(lib):
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.ib_attention_static.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, ci, vp]
    lib.ib_attention_static.restype = ci


def run_both(lib, torch, batch, nq, nk, d, dv, seed):
    rng = np.random.default_rng(seed)
    q = torch.from_numpy(rng.standard_normal((batch, nq, d), dtype=np.float32) * d ** -0.5).cuda()
    k = torch.from_numpy(rng.standard_normal((batch, nk, d), dtype=np.float32)).cuda()
    v = torch.from_numpy(rng.standard_normal((batch, nk, dv), dtype=np.float32)).cuda()
    stream = torch.cuda.current_stream().cuda_stream

    o_static = torch.full((batch, nq, dv), float("nan"), device="cuda")
    rc = lib.ib_attention_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_static.data_ptr(),
                                 batch, nq, nk, d, dv, 0, stream)
    assert rc == 0, last_error(lib)

    ws_bytes = lib.ib_attention_workspace_bytes(batch, nq, nk, d, dv, 0, FP32)
    ws = torch.empty(max(ws_bytes, 256), dtype=torch.uint8, device="cuda")
    o_ref = torch.full((batch, nq, dv), float("nan"), device="cuda")
    rc = lib.ib_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_ref.data_ptr(), batch, nq, nk,
                          d, dv, 0, FP32, 0, ws.data_ptr(), ws_bytes, stream)
    assert rc == 0, last_error(lib)
    torch.cuda.synchronize()
    return o_static.cpu().numpy(), o_ref.cpu().numpy(), (q, k, v)


def test_static_scratch_attention_matches_workspace_attention(lib, oracle):
    import torch
    declare(lib)

    # Two calls in a row on one stream: the second sees the first one's scores
    # still sitting in the shared array and must not be affected by them.
    first, first_ref, (q, k, v) = run_both(lib, torch, 2, 300, 500, 64, 48, seed=31)
    second, second_ref, _ = run_both(lib, torch, 1, 128, 1000, 40, 24, seed=32)
    for got, ref in ((first, first_ref), (second, second_ref)):
        assert np.isfinite(got).all()
        assert max_rel_to_peak(got, ref) <= 1e-5          # the fp32 arm's tolerance
    # And against the CPU oracle, like the other fp32 attention tests.
    want = oracle.attention_fused(q[0].cpu().numpy(), k[0].cpu().numpy(), v[0].cpu().numpy())
    assert max_rel_to_peak(first[0], want) <= 2e-5


def test_static_scratch_attention_refuses_oversize(lib):
    import torch
    declare(lib)
    cap = STATIC_BYTES
    nq = nk = 4096                       # 64 MiB of scores: twice the array
    assert nq * nk * 4 > cap
    q = torch.zeros(1, nq, 8, device="cuda")
    o = torch.zeros(1, nq, 8, device="cuda")
    rc = lib.ib_attention_static(q.data_ptr(), q.data_ptr(), q.data_ptr(), o.data_ptr(), 1, nq, nk,
                                 8, 8, 0, None)
    assert rc == -1
    msg = last_error(lib)
    assert "built-in array holds 33554432" in msg and "use ib_attention" in msg


def test_static_scratch_attention_allocates_nothing_once_set_up(lib):
    """After the first call on a device (which loads the module that holds the array and may
    reserve it then), a call leaves the device's free memory exactly where it was."""
    import torch
    declare(lib)
    q = torch.randn(1, 256, 64, device="cuda")
    k = torch.randn(1, 512, 64, device="cuda")
    v = torch.randn(1, 512, 32, device="cuda")
    o = torch.empty(1, 256, 32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = lib.ib_attention_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), 1, 256, 512,
                                     64, 32, 0, stream)
        assert rc == 0, last_error(lib)
        torch.cuda.synchronize()

    call()                                   # set-up call
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
