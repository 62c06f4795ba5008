"""Parity of every arithmetic arm on the benchmark workloads themselves, called through the C ABI.

* fused attention, one head of 16384 x 16384 x 128 (seed 3): every precision, 1024 rows spread
  over all 128 row tiles, against the reference's own emitted C (oracle/_ref, one slice per
  host core; rows are independent given K and V, ilang-python/annotated-flashattn.c:92-127, 240-307);
* 64 heads of 32768 x 32768 x 128 (seed 4) as one batched invocation: 1024 rows over 16 heads;
* `mm_t` 8192 x 8192 x 4096 (seed 2) under AUTO (the scaled-fp16 arm at that shape) and TF32:
  256 sampled rows against the restated loop nest (oracle.contract);
* adversarial logits for the arms that hold P in fp16: one key at logit 0 and nk - 1 keys at
  about -L ln 2, where P is an fp16 subnormal (L >= 15) or flushes to zero (L >= 25).

Bounds: 5e-3 of the output's peak for the TF32-class arms (TF32, TF32 x fp16, fp16 over powers
of two, AUTO), 2e-2 for BF16.
"""
import os

import numpy as np
import pytest

from conftest import last_error, max_rel_to_peak

pytestmark = pytest.mark.gpu

AUTO, FP32, TF32, BF16, TF32_F16, F16 = 0, 1, 2, 3, 4, 5
TOL_TF32 = 5e-3
TOL_BF16 = 2e-2
ARMS = [("auto", AUTO, TOL_TF32), ("f16", F16, TOL_TF32), ("tf32_f16", TF32_F16, TOL_TF32),
        ("tf32", TF32, TOL_TF32), ("bf16", BF16, TOL_BF16)]


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


def attention(lib, torch, q, k, v, precision):
    """ib_attention on device tensors [batch, n, d]; returns the output tensor (on the device)."""
    batch, nq, d = q.shape
    nk, dv = k.shape[1], v.shape[2]
    o = torch.full((batch, nq, dv), float("nan"), device="cuda")
    wb = lib.ib_attention_workspace_bytes(batch, nq, nk, d, dv, 0, precision)
    ws = torch.empty(max(wb, 256), dtype=torch.uint8, device="cuda")
    rc = lib.ib_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), batch, nq, nk, d, dv,
                          0, precision, 0, ws.data_ptr(), wb, None)
    assert rc == 0, last_error(lib)
    torch.cuda.synchronize()
    return o


def reference_rows(oracle, q_rows, k, v):
    """Rows of the reference's emitted C on all host cores (the restated port if _ref is absent)."""
    fn = oracle.reference_attention if oracle.have_reference() else oracle.attention_fused
    cores = os.cpu_count() or 1
    n = q_rows.shape[0]
    cuts = np.linspace(0, n, min(cores, n) + 1).astype(int)
    blocks = [(a, b) for a, b in zip(cuts[:-1], cuts[1:]) if b > a]
    return np.concatenate(oracle.reference_attention_rows(q_rows, k, v, blocks, fn=fn))


# ---- one head of 16384 ------------------------------------------------------------------------

@pytest.fixture(scope="module")
def config4(oracle):
    rng = np.random.default_rng(3)
    q = rng.standard_normal((16384, 128), dtype=np.float32)
    k = rng.standard_normal((16384, 128), dtype=np.float32)
    v = rng.standard_normal((16384, 128), dtype=np.float32)
    q *= np.float32(1.0 / np.sqrt(128))
    # Eight rows of every 128-row tile, at offsets that differ from tile to tile.
    tiles = np.arange(128)
    rows = np.sort(np.concatenate([tiles * 128 + (17 * j + 5 * tiles) % 128 for j in range(8)]))
    assert rows.size == 1024 and np.unique(rows // 128).size == 128
    return q, k, v, rows, reference_rows(oracle, q[rows], k, v)


@pytest.mark.parametrize("name,precision,tol", ARMS)
def test_attention_seq16384_every_arm_against_reference(lib, torch, config4, name, precision, tol):
    q, k, v, rows, ref = config4
    dq, dk, dv_ = (torch.from_numpy(x).cuda()[None] for x in (q, k, v))
    o = attention(lib, torch, dq, dk, dv_, precision)[0]
    assert torch.isfinite(o).all()
    got = o[torch.from_numpy(rows).cuda()].cpu().numpy()
    err = max_rel_to_peak(got, ref)
    print("seq16384 %s: max error %.2e of peak" % (name, err))
    assert err <= tol, (name, err)
    # Size-independent property: with V = 1 every output is the row sum of the softmax, 1.
    o1 = attention(lib, torch, dq, dk, torch.ones_like(dv_), precision)[0]
    assert (o1 - 1.0).abs().max().item() < (2e-3 if precision != BF16 else 8e-3)


# ---- 64 heads of 32768 ------------------------------------------------------------------------

def test_attention_64_heads_seq32768_one_invocation(lib, oracle, torch):
    heads, n, d = 64, 32768, 128
    rng = np.random.default_rng(4)
    q = rng.standard_normal((heads, n, d), dtype=np.float32)
    k = rng.standard_normal((heads, n, d), dtype=np.float32)
    v = rng.standard_normal((heads, n, d), dtype=np.float32)
    q *= np.float32(1.0 / np.sqrt(d))
    dq, dk, dv_ = torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    o = attention(lib, torch, dq, dk, dv_, AUTO)
    assert torch.isfinite(o).all()
    # 64 rows in each of 16 heads (every fourth head), spread over the head's 256 row tiles.
    worst = 0.0
    for h in range(0, heads, 4):
        rows = (np.arange(64) * 512 + (37 * h + 129 * np.arange(64)) % 512).astype(np.int64)
        ref = reference_rows(oracle, q[h][rows], k[h], v[h])
        got = o[h][torch.from_numpy(rows).cuda()].cpu().numpy()
        worst = max(worst, max_rel_to_peak(got, ref))
    print("64 x 32768: max error %.2e of peak over 1024 rows of 16 heads" % worst)
    assert worst <= TOL_TF32
    # Heads are independent: head 5 alone gives the same rows as head 5 of the batch, up to the
    # rounding of a different split of the key range (alone, the head's 256 row tiles are cut
    # over the 148 SMs differently, so other rows are summed in two pieces).
    alone = attention(lib, torch, dq[5:6], dk[5:6], dv_[5:6], AUTO)[0]
    gap = (alone - o[5]).abs().max().item() / o[5].abs().max().item()
    print("head 5 alone against head 5 of the batch: %.2e of peak" % gap)
    assert gap <= 2e-3


# ---- mm_t 8192 x 8192 x 4096 --------------------------------------------------------------------

@pytest.mark.parametrize("name,precision", [("auto", AUTO), ("tf32", TF32), ("f16", F16)])
def test_mm_t_8192_sampled_rows_against_oracle(lib, oracle, torch, name, precision):
    rng = np.random.default_rng(2)
    a = 2 * rng.random((8192, 4096), dtype=np.float32) - 1
    b = 2 * rng.random((8192, 4096), dtype=np.float32) - 1
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    c = torch.full((8192, 8192), float("nan"), device="cuda")
    wb = lib.ib_contract_workspace_bytes(1, 8192, 8192, 4096, 1, 1, precision)
    ws = torch.empty(max(wb, 256), dtype=torch.uint8, device="cuda")
    rc = lib.ib_contract(da.data_ptr(), db.data_ptr(), c.data_ptr(), 1, 8192, 8192, 4096, 1, 1, precision,
                         ws.data_ptr() if wb else None, wb, None)
    assert rc == 0, last_error(lib)
    torch.cuda.synchronize()
    assert torch.isfinite(c).all()
    rows = np.sort((np.arange(256) * 32 + (13 * np.arange(256)) % 32).astype(np.int64))
    ref = np.concatenate(oracle.contract_rows(a[rows], b))
    err = max_rel_to_peak(c[torch.from_numpy(rows).cuda()].cpu().numpy(), ref)
    print("mm_t 8192x8192x4096 %s: max error %.2e of peak" % (name, err))
    assert err <= TOL_TF32, (name, err)
    # Size-independent property: row sums of C equal A (B^T 1), computed in float64.
    want = da.double() @ db.double().sum(dim=0)
    scale = (da.double().abs() @ db.double().abs().sum(dim=0)).max().item()
    assert (c.double().sum(dim=1) - want).abs().max().item() / scale < 1e-3


# ---- adversarial logits for the fp16-P arms -----------------------------------------------------

@pytest.mark.parametrize("nk", [4096, 32768])
@pytest.mark.parametrize("where", ["first", "last"])
@pytest.mark.parametrize("values", ["ones", "normal"])
@pytest.mark.parametrize("name,precision", [("auto", AUTO), ("f16", F16), ("tf32_f16", TF32_F16)])
def test_attention_one_dominant_key_and_a_far_tail(lib, oracle, torch, nk, where, values, name, precision):
    """Row i has one key at logit 0 and nk - 1 keys at -L_i * 0.693359375 (about 2^-L_i of the
    dominant weight), L_i in {10, 14, 16, 20, 24, 26}: the tail's probabilities are fp16
    subnormals from L = 15 and flush to zero from L = 25, while its total mass (up to nk * 2^-L)
    is not negligible.  Every product is exact in fp16 and TF32 (q = L, a small integer; k =
    -0.693359375 = -710/1024), so what is compared is the softmax and the second contraction."""
    d, dv, nq = 64, 64, 768
    levels = np.array([10, 14, 16, 20, 24, 26], dtype=np.float32)
    q = np.zeros((nq, d), dtype=np.float32)
    q[:, 0] = levels[np.arange(nq) % levels.size]
    k = np.zeros((nk, d), dtype=np.float32)
    k[:, 0] = np.float32(-0.693359375)
    dominant = 3 if where == "first" else nk - 2
    k[dominant, 0] = 0.0
    rng = np.random.default_rng(11)
    v = np.ones((nk, dv), dtype=np.float32) if values == "ones" else rng.standard_normal((nk, dv), dtype=np.float32)
    dq, dk, dv_ = (torch.from_numpy(x).cuda()[None] for x in (q, k, v))
    # AUTO only takes a tensor arm above its size threshold; ask for the tensor arm it would take.
    prec = F16 if precision == AUTO and not lib.ib_attention_uses_tensor_arm(1, nq, nk, d, dv, AUTO) else precision
    o = attention(lib, torch, dq, dk, dv_, prec)[0].cpu().numpy()
    assert np.isfinite(o).all()
    ref = reference_rows(oracle, q, k, v)
    for li, level in enumerate(levels):
        rows = np.arange(nq) % levels.size == li
        err = max_rel_to_peak(o[rows], ref[rows])
        assert err <= TOL_TF32, (name, nk, where, values, float(level), err)
