"""One launch of the pointwise-chain kernel at 8192 x 8192 for a profiler to capture:
`ij-i`, `^ij`, `ij/i` (a softmax's two pointwise halves with the statistics supplied).

    python tests/profile_map_chain.py
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from i_b200 import ilang  # noqa: E402


def main():
    i = ilang.i
    rows = cols = 8192
    g = torch.Generator(device="cuda")
    g.manual_seed(1)
    x = torch.randn(rows, cols, device="cuda", generator=g)
    m = torch.randn(rows, device="cuda", generator=g)
    s = torch.rand(rows, device="cuda", generator=g) + 0.5
    out = torch.empty_like(x)
    chain = i("ij-i~ij") >> i("^ij~ij") >> i("ij/i~ij")
    assert "map_chain" in chain._code()
    for _ in range(3):
        chain.into(out, x, m, s)
    torch.cuda.synchronize()
    ref = torch.exp(x - m[:, None]) / s[:, None]
    err = ((out - ref).abs() / ref.abs().clamp_min(1e-30)).max().item()
    print("max relative difference to torch:", err)
    assert err < 1e-5


if __name__ == "__main__":
    main()
