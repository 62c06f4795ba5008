"""ib_peer_publish on one GPU: the destinations are other buffers of the same device, which takes
the same path (event wait, one asynchronous device-to-device copy per destination, event record)
as peer-mapped buffers of other GPUs do."""
import ctypes

import pytest

from conftest import last_error

pytestmark = pytest.mark.gpu


def declare(lib):
    lib.ib_peer_publish.restype = ctypes.c_int
    lib.ib_peer_publish.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p), ctypes.c_int,
                                    ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]


def test_copies_follow_the_producer_and_precede_the_done_event(lib):
    import torch
    declare(lib)
    n = 1 << 22
    src = torch.zeros(n, device="cuda")
    dsts = [torch.full((n,), -1.0, device="cuda") for _ in range(3)]
    side = torch.cuda.Stream()
    produced, done = torch.cuda.Event(), torch.cuda.Event()
    done.record(side)                      # an event's handle exists once it has been recorded
    main = torch.cuda.current_stream()
    big = torch.randn(4096, 4096, device="cuda")
    for _ in range(8):                     # keep the producer's stream busy before it writes src
        big = big @ big * 1e-3
    src.copy_(torch.arange(n, device="cuda", dtype=torch.float32))
    produced.record(main)
    ptrs = (ctypes.c_void_p * 3)(*[d.data_ptr() for d in dsts])
    rc = lib.ib_peer_publish(src.data_ptr(), ptrs, 3, n * 4, produced.cuda_event, done.cuda_event,
                             side.cuda_stream)
    assert rc == 0, last_error(lib)
    done.synchronize()
    expect = torch.arange(n, device="cuda", dtype=torch.float32)
    for d in dsts:
        assert torch.equal(d, expect)


def test_part_of_a_buffer_and_no_destinations(lib):
    import torch
    declare(lib)
    src = torch.arange(1024, device="cuda", dtype=torch.float32)
    dst = torch.zeros(1024, device="cuda")
    torch.cuda.synchronize()
    ptrs = (ctypes.c_void_p * 1)(dst.data_ptr() + 256 * 4)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.ib_peer_publish(src.data_ptr() + 256 * 4, ptrs, 1, 512 * 4, None, None, stream) == 0
    assert lib.ib_peer_publish(src.data_ptr(), ptrs, 0, 512 * 4, None, None, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(dst[256:768], src[256:768])
    assert dst[:256].abs().sum().item() == 0 and dst[768:].abs().sum().item() == 0


def test_bad_arguments_are_refused(lib):
    import torch
    declare(lib)
    src = torch.zeros(16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.ib_peer_publish(src.data_ptr(), None, 2, 64, None, None, stream) == -1
    assert "no destinations" in last_error(lib)
    ptrs = (ctypes.c_void_p * 2)(src.data_ptr(), None)
    assert lib.ib_peer_publish(src.data_ptr(), ptrs, 2, 0, None, None, stream) == -1
    assert "null destination" in last_error(lib)
