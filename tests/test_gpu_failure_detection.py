"""Failure detection on the GPU, exercised without a fault: a device-side wait that can never be
satisfied must run out, leave its code in the status word, and surface on the host as -1 with a
message; the context must stay usable.  Nothing here traps, faults or waits without a limit."""
import ctypes

import numpy as np
import pytest

from conftest import last_error

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_next_launch_succeeds(lib, oracle):
    import torch
    lib.ib_selftest_wait_timeout.argtypes = [ctypes.c_ulonglong, ctypes.c_void_p]
    lib.ib_selftest_wait_timeout.restype = ctypes.c_int
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.ib_selftest_wait_timeout(1_000_000, stream)          # one millisecond
    assert rc == -1
    message = last_error(lib)
    assert "a device-side wait timed out (code 250)" in message, message
    # The status word was cleared by the report: a second look finds nothing, an ordinary kernel
    # runs, and a fused tcgen05 attention (which uses the same status word and bounded waits) is
    # correct.
    x = np.random.default_rng(0).standard_normal((64, 300), dtype=np.float32)
    d = torch.from_numpy(x).cuda()
    y = torch.empty_like(d)
    assert lib.ib_row_softmax(d.data_ptr(), y.data_ptr(), 64, 300, stream) == 0, last_error(lib)
    torch.cuda.synchronize()
    ref = oracle.row_softmax(x)
    assert np.abs(y.cpu().numpy() - ref).max() <= 1e-5 * np.abs(ref).max()
    q = np.random.default_rng(1).standard_normal((256, 64), dtype=np.float32) * np.float32(0.125)
    k = np.random.default_rng(2).standard_normal((512, 64), dtype=np.float32)
    v = np.random.default_rng(3).standard_normal((512, 64), dtype=np.float32)
    dq, dk, dv = (torch.from_numpy(a).cuda() for a in (q, k, v))
    o = torch.empty(256, 64, device="cuda")
    wb = lib.ib_attention_workspace_bytes(1, 256, 512, 64, 64, 0, 5)
    ws = torch.empty(max(wb, 256), dtype=torch.uint8, device="cuda")
    assert lib.ib_attention(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), o.data_ptr(), 1, 256, 512, 64,
                            64, 0, 5, 0, ws.data_ptr(), wb, stream) == 0, last_error(lib)
    torch.cuda.synchronize()
    ref = oracle.attention_fused(q, k, v)
    assert np.abs(o.cpu().numpy() - ref).max() <= 5e-3 * np.abs(ref).max()
    # Repeating the self-test gives the same report.
    assert lib.ib_selftest_wait_timeout(200_000, stream) == -1
    assert "timed out" in last_error(lib)
