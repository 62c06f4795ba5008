"""The schedule segment chooses the tensor-core kernels' geometry: the same component under
different splits and loop orders compiles to different plans (i_code says which), launches a
different set of kernels, and gives the same results."""
import re

import numpy as np
import pytest

from conftest import max_rel_to_peak

pytestmark = pytest.mark.gpu


def attention(ilang, split, row_outer):
    """The README attention chain under a given split, with the key axis (README) or the row axis
    outermost in every node's loop order."""
    i, I = ilang.i, ilang.I
    if row_outer:
        o = {"qk": "ijj'i'k", "red": "ij0j'i'", "map": "ij01j'i'", "pv": "ij0j'ki'", "pvr": "ijj'ki'0"}
    else:
        o = {"qk": "jii'j'k", "red": "ji0i'j'", "map": "ji01i'j'", "pv": "ji0i'kj'", "pvr": "jii'kj'0"}
    mm_t = i("ik*jk~ijk | %s | %s" % (split, o["qk"])) >> i("+ijk~ij | %s | %s0" % (split, o["qk"]))
    shift = (I & i(">ij~i | %s | %s" % (split, o["red"]))) >> i("ij-i~ij | %s | %s" % (split, o["map"]))
    ex = i("^ij~ij | %s | %s" % (split, o["red"]))
    norm = (I & i("+ij~i | %s | %s" % (split, o["red"]))) >> i("ij/i~ij | %s | %s" % (split, o["map"]))
    mm = i("ij*jk~ikj | %s | %s" % (split, o["pv"])) >> i("+ikj~ik | %s | %s" % (split, o["pvr"]))
    return mm_t >> shift >> ex >> norm >> mm


def geometry_line(component):
    return re.search(r"^\s*geometry: (.*)$", component._code(), re.M).group(1)


def launches_of(ilang, fn):
    import torch
    torch.cuda.synchronize()
    before = ilang.launch_count()
    out = fn()
    torch.cuda.synchronize()
    return out, ilang.launch_count() - before


def test_attention_key_split_and_loop_order_select_the_work_split(ilang, oracle):
    import torch
    rng = np.random.default_rng(21)
    # 16 blocks of 128 query rows for 148 SMs: whether a block's keys are divided matters here.
    q = rng.standard_normal((2048, 128), dtype=np.float32) * np.float32(128 ** -0.5)
    k = rng.standard_normal((8192, 128), dtype=np.float32)
    v = rng.standard_normal((8192, 128), dtype=np.float32)
    dq, dk, dv = (torch.from_numpy(x).cuda() for x in (q, k, v))
    variants = {
        "readme": attention(ilang, "i:16,j:16", row_outer=False),
        "key split 1024": attention(ilang, "i:16,j:1024", row_outer=False),
        "row axis outermost": attention(ilang, "i:16,j:16", row_outer=True),
    }
    lines = {name: geometry_line(c) for name, c in variants.items()}
    assert "multiples of 128 keys" in lines["readme"]
    assert "multiples of 1024 keys" in lines["key split 1024"]
    assert "stays on one SM" in lines["row axis outermost"] and "no merge kernel" in lines["row axis outermost"]
    assert len(set(lines.values())) == 3

    rows = np.arange(0, 2048, 16)
    ref = oracle.attention_fused(q[rows], k, v)
    results, counts = {}, {}
    for name, c in variants.items():
        c.exec_torch(dq, dk, dv)                                  # compile, first-call set-up
        out, counts[name] = launches_of(ilang, lambda c=c: c.exec_torch(dq, dk, dv))
        results[name] = out.cpu().numpy()
        assert max_rel_to_peak(results[name][rows], ref) <= 5e-3, name
    # Divided key ranges are merged by one more kernel; undivided ones are not.
    assert counts["readme"] == counts["key split 1024"] == counts["row axis outermost"] + 1, counts
    for name in ("key split 1024", "row axis outermost"):
        assert max_rel_to_peak(results[name], results["readme"]) <= 2e-3, name


def test_contraction_column_split_and_loop_order_select_the_tiles(ilang, oracle):
    import torch
    i = ilang.i
    rng = np.random.default_rng(22)
    a = 2 * rng.random((1024, 512), dtype=np.float32) - 1
    b = 2 * rng.random((1536, 512), dtype=np.float32) - 1
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()

    def mm_t(split, order):
        return (i("ik*jk~ijk | %s | %s" % (split, order)) >> i("+ijk~ij | %s | %s0" % (split, order))
                ).set_precision("tf32")

    variants = {
        "readme": mm_t("i:16,j:16", "jii'j'k"),
        "128 columns, row by row": mm_t("i:128,j:128", "ijj'i'k"),
        "256 columns": mm_t("i:128,j:256", "jii'j'k"),
    }
    lines = {name: geometry_line(c) for name, c in variants.items()}
    assert "128 or 256 columns by the output's width" in lines["readme"] and "groups of 12" in lines["readme"]
    assert "128 columns (the schedule's column split)" in lines["128 columns, row by row"]
    assert "row by row" in lines["128 columns, row by row"]
    assert "256 columns (the schedule's column split)" in lines["256 columns"]
    rows = np.arange(0, 1024, 8)
    ref = np.concatenate(oracle.contract_rows(a[rows], b))
    outs = {name: c.exec_torch(da, db).cpu().numpy() for name, c in variants.items()}
    for name, got in outs.items():
        assert max_rel_to_peak(got[rows], ref) <= 2e-3, name
    # The tile shape and the walk change which SM computes what, not the arithmetic of an element.
    assert np.array_equal(outs["readme"], outs["128 columns, row by row"])
    assert np.array_equal(outs["readme"], outs["256 columns"])


@pytest.mark.parametrize("batch,m,n,k", [(1, 256, 256, 32), (1, 257, 259, 36), (1, 300, 700, 100),
                                         (3, 384, 512, 128), (2, 1000, 1300, 260), (1, 4096, 256, 64),
                                         (1, 256, 4096, 4), (5, 511, 513, 68)])
@pytest.mark.parametrize("precision", [2, 3, 5])          # TF32, BF16, scaled fp16
def test_pair_kernel_matches_the_single_cta_kernel_bit_for_bit(lib, batch, m, n, k, precision):
    """Outputs of at least 256 x 256 run on CTA pairs (M = 256 MMAs over 256 x 256 tiles) unless the
    caller fixes the column tile; a fixed tile of 256 runs the single-CTA kernel.  Same products,
    same order of accumulation over K: the results have to be identical, ragged edges included."""
    import ctypes
    import torch
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    lib.ib_contract_tiled.argtypes = [vp, vp, vp, sz, sz, sz, sz, ci, ci, ci, sz, sz, vp, sz, vp]
    lib.ib_contract_tiled.restype = ci
    lib.ib_contract_workspace_bytes.restype = sz
    lib.ib_contract_workspace_bytes.argtypes = [sz] * 4 + [ci] * 3
    g = torch.Generator(device="cuda")
    g.manual_seed(m * 3 + n * 5 + k)
    a = 2 * torch.rand(batch, m, k, device="cuda", generator=g) - 1
    b = 2 * torch.rand(batch, n, k, device="cuda", generator=g) - 1
    wb = lib.ib_contract_workspace_bytes(batch, m, n, k, 1, 1, precision)
    ws = torch.empty(max(wb, 256), dtype=torch.uint8, device="cuda")
    outs = []
    for tile in (0, 256):
        c = torch.full((batch, m, n), float("nan"), device="cuda")
        rc = lib.ib_contract_tiled(a.data_ptr(), b.data_ptr(), c.data_ptr(), batch, m, n, k, 1, 1, precision,
                                   tile, 0, ws.data_ptr(), wb, None)
        assert rc == 0
        torch.cuda.synchronize()
        outs.append(c)
    assert torch.isfinite(outs[0]).all()
    assert torch.equal(outs[0], outs[1])
    ref = (a.double() @ b.double().transpose(1, 2)).float()
    tol = 2e-2 if precision == 3 else 5e-3
    assert ((outs[0] - ref).abs().max() / ref.abs().max()).item() <= tol
