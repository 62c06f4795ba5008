"""Three calls of the fp16 contraction arm on BASELINE config 3 (mm_t 8192 x 8192 x 4096) for a
profiler to capture: two row-conversion launches and one GEMM launch per call.

    python tests/profile_contract_f16.py
"""
import ctypes
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from i_b200 import ilang  # noqa: E402

F16 = 5


def main():
    lib = ilang.core()
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.ib_contract.argtypes = [vp, vp, vp, sz, sz, sz, sz, ci, ci, ci, vp, sz, vp]
    lib.ib_contract_workspace_bytes.argtypes = [sz] * 4 + [ci] * 3
    lib.ib_contract_workspace_bytes.restype = sz
    m = n = 8192
    k = 4096
    g = torch.Generator(device="cuda")
    g.manual_seed(2)
    a = 2 * torch.rand(m, k, device="cuda", generator=g) - 1
    b = 2 * torch.rand(n, k, device="cuda", generator=g) - 1
    c = torch.empty(m, n, device="cuda")
    wb = lib.ib_contract_workspace_bytes(1, m, n, k, 1, 1, F16)
    ws = torch.empty(wb, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        rc = lib.ib_contract(a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, m, n, k, 1, 1, F16,
                             ws.data_ptr(), wb, None)
        assert rc == 0
    torch.cuda.synchronize()
    rows = torch.arange(0, m, 512, device="cuda")
    ref = a[rows].double() @ b.double().t()
    err = ((c[rows].double() - ref).abs().max() / ref.abs().max()).item()
    print("max error relative to peak on %d sampled rows: %.2e" % (rows.numel(), err))
    assert err <= 5e-3


if __name__ == "__main__":
    main()
