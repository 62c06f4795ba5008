"""GPU parity of every ib_* kernel, called through the C ABI on device buffers
and compared with the CPU oracle on the same seeded inputs.

Tolerances (max relative error against the reference C backend's arithmetic):
  maps, reductions, row softmax: 1e-5 element-wise (exact for max/min/copy);
  fp32 contraction arm: 1e-5 of the output's peak magnitude;
  TF32 tensor-core arm (contraction and fused attention): 5e-3 of the peak.
"""
import ctypes
import glob
import os

import numpy as np
import pytest

from conftest import last_error, max_rel_elementwise, max_rel_to_peak

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FP32, TF32, BF16, TF32_F16, F16 = 1, 2, 3, 4, 5
TOL_MAP = 1e-5
TOL_FP32 = 1e-5
TOL_TF32 = 5e-3
TOL_BF16 = 2e-2


@pytest.fixture(scope="module")
def torch():
    import torch
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def rand(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


def ok(lib, rc):
    assert rc == 0, last_error(lib)


# ---- maps -----------------------------------------------------------------

@pytest.mark.parametrize("op", list("+*-/><^$"))
@pytest.mark.parametrize("n", [1, 7, 1024, 100003])
def test_map_unary(lib, oracle, torch, op, n):
    x = rand((n,), 1)
    if op == "$":
        x = np.abs(x) + 0.05
    d = dev(torch, x)
    y = torch.empty_like(d)
    ok(lib, lib.ib_map_unary(oracle.OPS[op], d.data_ptr(), y.data_ptr(), n, None))
    ref = oracle.map_unary(op, x)
    got = y.cpu().numpy()
    if op in "+*-><":
        assert np.array_equal(got, ref)
    else:
        assert max_rel_elementwise(got, ref) <= TOL_MAP


def test_map_unary_misaligned_and_special_values(lib, oracle, torch):
    x = np.concatenate([rand((1001,), 2), [np.inf, -np.inf, 0.0, -0.0, 88.0, -104.0, -200.0]]).astype(np.float32)
    buf = torch.zeros(x.size + 1, device="cuda")
    buf[1:] = dev(torch, x)
    out = torch.zeros(x.size + 1, device="cuda")
    src, dst = buf[1:], out[1:]                      # 4-byte aligned only
    ok(lib, lib.ib_map_unary(oracle.OPS["^"], src.data_ptr(), dst.data_ptr(), x.size, None))
    ref = oracle.map_unary("^", x)
    got = dst.cpu().numpy()
    finite = np.isfinite(ref) & (ref > 1e-30)
    assert max_rel_elementwise(got[finite], ref[finite]) <= TOL_MAP
    assert np.array_equal(np.isinf(got), np.isinf(ref))
    assert np.all(got[ref == 0] == 0)


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("op", list("+*-/><^$"))
def test_map_binary_modes(lib, oracle, torch, mode, op):
    rows, cols = 37, 52 if mode % 2 == 0 else 51
    full = rand((rows, cols), 3)
    row_v, col_v = rand((rows,), 4), rand((cols,), 5)
    a = full if mode in (0, 1, 3) else (row_v if mode == 2 else col_v)
    b = rand((rows, cols), 6) if mode in (0, 2, 4) else (row_v if mode == 1 else col_v)
    if op in "^$":
        a = np.abs(a) + 0.1
    if op == "/":
        b = np.abs(b) + 0.1
    da, db = dev(torch, a), dev(torch, b)
    y = torch.empty(rows, cols, device="cuda")
    ok(lib, lib.ib_map_binary(oracle.OPS[op], mode, da.data_ptr(), db.data_ptr(), y.data_ptr(),
                              rows, cols, None))
    ref = oracle.map_binary(op, a, b, mode)
    assert max_rel_elementwise(y.cpu().numpy(), ref) <= TOL_MAP


NONE, PREV = -1, -2


def run_chain(lib, oracle, torch, ops, operands, modes, rows, cols, misalign=False, fold=None):
    """ops: (token, lhs, rhs) with lhs/rhs an operand index, PREV or NONE.  Returns (got, ref):
    the kernel's result and the same operators applied one at a time by the oracle; with `fold`
    (an operator token) both are folded along each row."""
    devs = []
    for a in operands:
        if misalign:                                   # 4-byte aligned only
            buf = torch.zeros(a.size + 1, device="cuda")
            buf[1:] = dev(torch, a).reshape(-1)
            devs.append(buf[1:])
        else:
            devs.append(dev(torch, a))
    n_out = rows if fold else rows * cols
    y = torch.empty(n_out + 1, device="cuda")[1 if misalign else 0:][:n_out]
    flat = (ctypes.c_int * (3 * len(ops)))(*[v for tok, l, r in ops for v in (oracle.OPS[tok], l, r)])
    ptrs = (ctypes.c_void_p * len(devs))(*[d.data_ptr() for d in devs])
    md = (ctypes.c_int * len(modes))(*modes)
    if fold:
        ok(lib, lib.ib_reduce_rows_chain(oracle.OPS[fold], len(ops), flat, len(devs), ptrs, md,
                                         y.data_ptr(), rows, cols, None))
    else:
        ok(lib, lib.ib_map_chain(len(ops), flat, len(devs), ptrs, md, y.data_ptr(), rows, cols, None))

    def full(code, prev):
        if code == PREV:
            return prev
        a, m = operands[code], modes[code]
        shaped = {0: lambda: a.reshape(rows, cols), 1: lambda: a.reshape(rows, 1),
                  2: lambda: a.reshape(1, cols), 3: lambda: a.reshape(1, 1)}[m]()
        return np.ascontiguousarray(np.broadcast_to(shaped, (rows, cols)))
    prev = None
    for tok, l, r in ops:
        prev = (oracle.map_unary(tok, full(l, prev)) if r == NONE
                else oracle.map_binary(tok, full(l, prev), full(r, prev)))
    if fold:
        return y.cpu().numpy(), oracle.reduce_rows(fold, prev)
    return y.cpu().numpy().reshape(rows, cols), prev


@pytest.mark.parametrize("rows,cols,misalign", [(37, 52, False), (37, 51, False), (64, 128, True),
                                                (1, 100003, False), (300, 4, False)])
def test_map_chain_softmax_like(lib, oracle, torch, rows, cols, misalign):
    # (x - m[r]) -> exp -> / s[r] -> * g[c] -> + scalar: every operand mode in one chain.
    x, m = rand((rows, cols), 1), rand((rows,), 2)
    s_, g, c0 = np.abs(rand((rows,), 3)) + 0.5, rand((cols,), 4), rand((1,), 5)
    ops = [("-", 0, 1), ("^", PREV, NONE), ("/", PREV, 2), ("*", 3, PREV), ("+", PREV, 4)]
    # Five operands is one too many for one call: fold the scalar in a second chain.
    got, ref = run_chain(lib, oracle, torch, ops[:4], [x, m, s_, g], [0, 1, 1, 2], rows, cols, misalign)
    assert max_rel_elementwise(got, ref) <= TOL_MAP
    got2, ref2 = run_chain(lib, oracle, torch, [("+", 0, 1), ("-", PREV, NONE)], [ref, c0], [0, 3],
                           rows, cols, misalign)
    assert np.array_equal(got2, ref2)


def test_map_chain_exact_ops_and_reuse(lib, oracle, torch):
    # Select by a comparison: (x > t[c]) * x, then clamp at a per-row ceiling; x appears twice.
    rows, cols = 129, 260
    x, t, hi = rand((rows, cols), 6), rand((cols,), 7), np.abs(rand((rows,), 8))
    ops = [(">>", 0, 1), ("*", PREV, 0), ("<", PREV, 2), ("!!", PREV, NONE)]
    got, ref = run_chain(lib, oracle, torch, ops[:3], [x, t, hi], [0, 2, 1], rows, cols)
    assert np.array_equal(got, ref)
    assert np.array_equal(ref, np.minimum(np.where(x > t[None, :], x, 0.0), hi[:, None]).astype(np.float32))
    got, ref = run_chain(lib, oracle, torch, ops, [x, t, hi], [0, 2, 1], rows, cols)
    assert np.array_equal(got, ref)


def test_map_chain_larger_than_l2(lib, oracle, torch):
    rows, cols = 4096, 8192 + 4
    x, b = rand((rows, cols), 9), rand((cols,), 10)
    got, ref = run_chain(lib, oracle, torch, [("+", 0, 1), (">", PREV, NONE), ("*", PREV, PREV)],
                         [x, b], [0, 2], rows, cols)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("seed", range(24))
def test_map_chain_random_programs(lib, oracle, torch, seed):
    # Random operator lists over random shapes and operand modes.  Every operator used here is
    # exactly rounded on both sides, so the results must agree bit for bit (NaN and inf included:
    # differences and quotients of random values produce them).
    rng = np.random.default_rng(1000 + seed)
    rows = int(rng.choice([1, 3, 17, 64, 257]))
    cols = int(rng.choice([1, 4, 5, 60, 128, 1001, 4096]))
    n_operands = int(rng.integers(1, 5))
    modes = [0] + [int(rng.integers(0, 4)) for _ in range(n_operands - 1)]
    rng.shuffle(modes)
    if 0 not in modes:
        modes[0] = 0
    shape = {0: (rows, cols), 1: (rows,), 2: (cols,), 3: (1,)}
    operands = [rng.choice([-2.0, -1.0, 0.0, 0.5, 1.0, 3.0], size=shape[m]).astype(np.float32)
                + (rng.standard_normal(shape[m]).astype(np.float32) if rng.random() < 0.7 else 0)
                for m in modes]
    binary = ["+", "*", "-", "/", ">", "<", ">>", ">=", "<<", "<=", "==", "!=", "&&", "||", "^^"]
    unary = ["-", "/", ">", "<", "!!", ">>", "=="]
    ops = []
    for k in range(int(rng.integers(1, 9))):
        if rng.random() < 0.3:
            ops.append((str(rng.choice(unary)), PREV if k else int(rng.integers(n_operands)), NONE))
            continue
        other = int(rng.integers(n_operands)) if rng.random() < 0.85 or k == 0 else PREV
        mine = PREV if k else int(rng.integers(n_operands))
        ops.append((str(rng.choice(binary)),) + ((mine, other) if rng.random() < 0.6 or k == 0 else (other, mine)))
    got, ref = run_chain(lib, oracle, torch, ops, operands, modes, rows, cols, misalign=bool(seed % 5 == 4))
    assert np.array_equal(got, ref, equal_nan=True), (ops, modes, rows, cols)


@pytest.mark.parametrize("rows,cols,misalign", [(37, 52, False), (37, 51, False), (9, 8192, False),
                                                (5, 4096 + 4, True), (300, 4, False), (2, 20000, False),
                                                (1, 1, False), (1000, 128, False)])
def test_reduce_rows_chain_softmax_denominator(lib, oracle, torch, rows, cols, misalign):
    # sum_c exp(x[r][c] - m[r]) and max_c (x[r][c] - m[r]) * g[c]: warp-per-row, block-per-row and
    # element-wise paths.
    x, m, g = rand((rows, cols), 1), rand((rows,), 2) + 2.0, rand((cols,), 3)
    got, ref = run_chain(lib, oracle, torch, [("-", 0, 1), ("^", PREV, NONE)], [x, m], [0, 1], rows, cols,
                         misalign, fold="+")
    assert max_rel_elementwise(got, ref) <= TOL_MAP
    got, ref = run_chain(lib, oracle, torch, [("-", 0, 1), ("*", 2, PREV)], [x, m, g], [0, 1, 2], rows, cols,
                         misalign, fold=">")
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("fold", ["+", "*", ">", "<", "&&", "||", "^^"])
def test_reduce_rows_chain_every_fold(lib, oracle, torch, fold):
    rows, cols = 67, 1028
    x, t = rand((rows, cols), 4), rand((cols,), 5)
    if fold == "*":
        ops, operands, modes = [("*", 0, 1), ("+", PREV, 2)], [x, np.float32([0.01]), np.float32([1.0])], [0, 3, 3]
    elif fold in ("&&", "||", "^^"):
        x[3] = 5.0                                     # a row that is above every threshold
        x[4] = -5.0                                    # and one below
        ops, operands, modes = [(">>", 0, 1)], [x, t], [0, 2]
    else:
        ops, operands, modes = [("-", 0, 1), ("*", PREV, PREV)], [x, t], [0, 2]
    got, ref = run_chain(lib, oracle, torch, ops, operands, modes, rows, cols, fold=fold)
    if fold in "+*":
        assert max_rel_elementwise(got, ref) <= TOL_MAP
    else:
        assert np.array_equal(got, ref)


def test_reduce_rows_chain_rejects_bad_calls(lib, oracle, torch):
    x = dev(torch, rand((4, 4), 1))
    y = torch.empty(4, device="cuda")
    ptrs = (ctypes.c_void_p * 1)(x.data_ptr())
    md = (ctypes.c_int * 1)(0)
    one = (ctypes.c_int * 3)(oracle.OPS["-"], 0, NONE)
    assert lib.ib_reduce_rows_chain(oracle.OPS["-"], 1, one, 1, ptrs, md, y.data_ptr(), 4, 4, None) != 0
    assert "not reducible" in last_error(lib)
    bad = (ctypes.c_int * 3)(oracle.OPS["-"], PREV, NONE)
    assert lib.ib_reduce_rows_chain(oracle.OPS["+"], 1, bad, 1, ptrs, md, y.data_ptr(), 4, 4, None) != 0
    ok(lib, lib.ib_reduce_rows_chain(oracle.OPS["+"], 1, one, 1, ptrs, md, y.data_ptr(), 4, 4, None))
    # No columns: every row is the fold's identity.
    ok(lib, lib.ib_reduce_rows_chain(oracle.OPS[">"], 1, one, 1, ptrs, md, y.data_ptr(), 4, 0, None))
    assert np.all(np.isneginf(y.cpu().numpy()))


def test_map_chain_rejects_bad_programs(lib, oracle, torch):
    x = dev(torch, rand((4, 4), 1))
    y = torch.empty_like(x)
    ptrs = (ctypes.c_void_p * 1)(x.data_ptr())
    md = (ctypes.c_int * 1)(0)

    def call(triples, n_operands=1, modes=md):
        flat = (ctypes.c_int * len(triples))(*triples)
        return lib.ib_map_chain(len(triples) // 3, flat, n_operands, ptrs, modes, y.data_ptr(), 4, 4, None)
    add = oracle.OPS["+"]
    assert call([add, PREV, NONE]) != 0 and "operand code" in last_error(lib)     # nothing before the first
    assert call([add, 0, 1]) != 0                                                  # operand 1 does not exist
    assert call([add, NONE, 0]) != 0                                               # lhs is mandatory
    assert call([99, 0, NONE]) != 0 and "unknown operator" in last_error(lib)
    assert call([oracle.OPS["!!"], 0, 0]) != 0 and "one operand" in last_error(lib)
    assert call([add, 0, NONE] * 9) != 0                                           # nine operators
    assert call([add, 0, NONE], modes=(ctypes.c_int * 1)(4)) != 0
    assert call([add, 0, NONE]) == 0


def test_map_strided_transpose(lib, oracle, torch):
    x = rand((19, 33), 7)
    d = dev(torch, x)
    y = torch.empty(33, 19, device="cuda")
    extent = (ctypes.c_size_t * 2)(33, 19)
    stride = (ctypes.c_ssize_t * 2)(1, 33)           # y[j][i] = -x[i][j]
    ok(lib, lib.ib_map_strided(oracle.OPS["-"], d.data_ptr(), None, y.data_ptr(), 2, extent, stride,
                               None, None))
    assert np.array_equal(y.cpu().numpy(), -x.T)


LOGIC_BINARY = [">>", ">=", "<<", "<=", "==", "!=", "&&", "||", "^^"]


def logic_values(shape, seed):
    """Mostly small integers (so equal and zero operands are common), some NaN, inf and -0."""
    rng = np.random.default_rng(seed)
    x = rng.integers(-2, 3, size=shape).astype(np.float32)
    special = rng.random(shape)
    x[special < 0.03] = np.nan
    x[(special >= 0.03) & (special < 0.05)] = np.inf
    x[(special >= 0.05) & (special < 0.07)] = -0.0
    return x


@pytest.mark.parametrize("op", LOGIC_BINARY + ["!!"])
@pytest.mark.parametrize("n", [1, 1024, 100003])
def test_map_unary_comparisons_and_logic(lib, oracle, torch, op, n):
    x = logic_values((n,), 11)
    d = dev(torch, x)
    y = torch.empty_like(d)
    ok(lib, lib.ib_map_unary(oracle.OPS[op], d.data_ptr(), y.data_ptr(), n, None))
    assert np.array_equal(y.cpu().numpy(), oracle.map_unary(op, x), equal_nan=True)


@pytest.mark.parametrize("mode", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("op", LOGIC_BINARY)
def test_map_binary_comparisons_and_logic(lib, oracle, torch, mode, op):
    rows, cols = 37, 52 if mode % 2 == 0 else 51
    full = logic_values((rows, cols), 12)
    row_v, col_v = logic_values((rows,), 13), logic_values((cols,), 14)
    a = full if mode in (0, 1, 3) else (row_v if mode == 2 else col_v)
    b = logic_values((rows, cols), 15) if mode in (0, 2, 4) else (row_v if mode == 1 else col_v)
    da, db = dev(torch, a), dev(torch, b)
    y = torch.empty(rows, cols, device="cuda")
    ok(lib, lib.ib_map_binary(oracle.OPS[op], mode, da.data_ptr(), db.data_ptr(), y.data_ptr(),
                              rows, cols, None))
    assert np.array_equal(y.cpu().numpy(), oracle.map_binary(op, a, b, mode))


def test_map_binary_rejects_not(lib, oracle, torch):
    x = torch.zeros(4, device="cuda")
    assert lib.ib_map_binary(oracle.OPS["!!"], 0, x.data_ptr(), x.data_ptr(), x.data_ptr(), 1, 4,
                             None) == -1
    assert "one operand" in last_error(lib)


@pytest.mark.parametrize("op", ["&&", "||", "^^"])
@pytest.mark.parametrize("shape", [(16, 8), (100, 257), (7, 5000), (3, 4096), (5, 1), (4, 0)])
def test_reduce_rows_logic(lib, oracle, torch, op, shape):
    rng = np.random.default_rng(16)
    x = logic_values(shape, 17)
    # rows that are all true, all false, and mixed
    x[rng.random(shape) < (0.9 if op == "&&" else 0.0)] = 3.0
    if op == "||":
        x[rng.random(shape) < 0.98] = 0.0
    d = dev(torch, x) if x.size else torch.empty(shape, device="cuda")
    y = torch.empty(shape[0], device="cuda")
    ptr = d.data_ptr() if x.size else None
    ok(lib, lib.ib_reduce_rows(oracle.OPS[op], ptr, y.data_ptr(), shape[0], shape[1], None))
    assert np.array_equal(y.cpu().numpy(), oracle.reduce_rows(op, x))


# ---- reductions -----------------------------------------------------------

@pytest.mark.parametrize("op", list("+*><"))
@pytest.mark.parametrize("shape", [(16, 8), (100, 257), (7, 5000), (3, 4096), (1, 1), (2049, 33)])
def test_reduce_rows(lib, oracle, torch, op, shape):
    x = rand(shape, 8)
    if op == "*":
        x = (1.0 + 0.01 * x).astype(np.float32)
    if op == "+":
        x = np.abs(x)                                 # well-conditioned sum
    d = dev(torch, x)
    y = torch.empty(shape[0], device="cuda")
    ok(lib, lib.ib_reduce_rows(oracle.OPS[op], d.data_ptr(), y.data_ptr(), shape[0], shape[1], None))
    ref = oracle.reduce_rows(op, x)
    got = y.cpu().numpy()
    if op in "><":
        assert np.array_equal(got, ref)
    else:
        assert max_rel_elementwise(got, ref) <= TOL_MAP


def test_reduce_signed_sum_against_magnitude(lib, oracle, torch):
    # test.py:120-128 sums N(0,1) rows; the error is judged against sum|x|.
    x = rand((16, 8), 1)
    d = dev(torch, x)
    y = torch.empty(16, device="cuda")
    ok(lib, lib.ib_reduce_rows(oracle.OPS["+"], d.data_ptr(), y.data_ptr(), 16, 8, None))
    err = np.abs(y.cpu().numpy() - oracle.reduce_rows("+", x))
    assert np.all(err <= 1e-6 * np.abs(x).sum(axis=1))


def test_reduce_empty_rows_give_identity(lib, oracle, torch):
    x = torch.empty(4, 0, device="cuda")
    y = torch.full((4,), 7.0, device="cuda")
    ok(lib, lib.ib_reduce_rows(oracle.OPS[">"], x.data_ptr(), y.data_ptr(), 4, 0, None))
    assert np.all(np.isneginf(y.cpu().numpy()))
    ok(lib, lib.ib_reduce_rows(oracle.OPS["+"], x.data_ptr(), y.data_ptr(), 4, 0, None))
    assert np.all(y.cpu().numpy() == 0)


def test_reduce_strided_columns(lib, oracle, torch):
    x = np.abs(rand((50, 21), 9))
    d = dev(torch, x)
    y = torch.empty(21, device="cuda")
    ke, ks = (ctypes.c_size_t * 1)(21), (ctypes.c_ssize_t * 1)(1)
    re_, rs = (ctypes.c_size_t * 1)(50), (ctypes.c_ssize_t * 1)(21)
    ok(lib, lib.ib_reduce_strided(oracle.OPS["+"], d.data_ptr(), y.data_ptr(), 1, ke, ks, 1, re_, rs, None))
    ref = oracle.reduce_rows("+", np.ascontiguousarray(x.T))
    assert max_rel_elementwise(y.cpu().numpy(), ref) <= TOL_MAP


def test_reduce_rejects_non_reducible(lib, oracle, torch):
    x = torch.ones(2, 2, device="cuda")
    y = torch.ones(2, device="cuda")
    assert lib.ib_reduce_rows(oracle.OPS["-"], x.data_ptr(), y.data_ptr(), 2, 2, None) == -1
    assert "not reducible" in last_error(lib)


# ---- row softmax ----------------------------------------------------------

@pytest.mark.parametrize("shape", [(64, 16), (1000, 30), (777, 50), (33, 64), (9, 3), (100, 257), (33, 1000), (5, 1023), (16, 4096),
                                   (8, 8192), (3, 16384), (2, 20001), (1, 1), (5, 12000), (3, 20000),
                                   (2, 32768), (2, 40000),
                                   # rows held by a cluster of 2, 4 and 8 CTAs (whole and ragged
                                   # slices, widths not a multiple of four, more rows than clusters),
                                   # and one beyond what a cluster holds
                                   (3, 65536), (2, 100000), (80, 50001), (2, 200002), (40, 131073),
                                   (1, 262144), (2, 300000)])
def test_row_softmax(lib, oracle, torch, shape):
    x = 2.0 * rand(shape, 10)                        # N(0, 4), the published row-softmax case
    d = dev(torch, x)
    y = torch.empty_like(d)
    ok(lib, lib.ib_row_softmax(d.data_ptr(), y.data_ptr(), shape[0], shape[1], None))
    if shape[1] <= 32768:
        ref = oracle.row_softmax(x)
    else:
        # The oracle adds a row's exponentials one after another in fp32, as the reference does;
        # over tens of thousands of terms that sum is itself off by about 1e-5 (one row of
        # 80 x 50001 differs from the float64 value by 1.0e-5), which is the whole bound.  Long rows
        # are therefore held against the same arithmetic in float64.
        z = x.astype(np.float64)
        e = np.exp((z - z.max(axis=1, keepdims=True)) * np.log(np.float64(np.float32(2.71828175))))
        ref = e / e.sum(axis=1, keepdims=True)
    assert max_rel_elementwise(y.cpu().numpy(), ref) <= TOL_MAP


def test_row_softmax_config2_sample_and_checksum(lib, oracle, torch):
    # 8192 x 8192 N(0,4), seed 1: every row sums to 1; 48 sampled rows against the oracle.
    rng = np.random.default_rng(1)
    x = 2.0 * rng.standard_normal((8192, 8192), dtype=np.float32)
    d = dev(torch, x)
    y = torch.empty_like(d)
    ok(lib, lib.ib_row_softmax(d.data_ptr(), y.data_ptr(), 8192, 8192, None))
    sums = y.double().sum(dim=1).cpu().numpy()
    assert np.abs(sums - 1.0).max() < 1e-5
    rows = np.linspace(0, 8191, 48).astype(int)
    ref = oracle.row_softmax(x[rows])
    assert max_rel_elementwise(y[torch.from_numpy(rows).cuda()].cpu().numpy(), ref) <= TOL_MAP


# ---- contraction ----------------------------------------------------------

def run_contract(lib, torch, a, b, akm, bkm, precision, batch=None):
    nb = 1 if batch is None else batch
    sa = a.shape[-2:] if akm else a.shape[-2:][::-1]
    m, k = sa
    n = b.shape[-2] if bkm else b.shape[-1]
    da, db = dev(torch, a), dev(torch, b)
    c = torch.full((nb, m, n), float("nan"), device="cuda")
    ws_bytes = lib.ib_contract_workspace_bytes(nb, m, n, k, int(akm), int(bkm), precision)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    ok(lib, lib.ib_contract(da.data_ptr(), db.data_ptr(), c.data_ptr(), nb, m, n, k, int(akm),
                            int(bkm), precision, ws.data_ptr(), ws_bytes, None))
    torch.cuda.synchronize()
    out = c.cpu().numpy()
    return out[0] if batch is None else out


@pytest.mark.parametrize("m,n,k,akm,bkm", [
    (8, 7, 16, True, False),      # ilang-python/test.py:40-59
    (100, 40, 33, True, True), (65, 130, 17, False, True), (64, 64, 64, False, False),
    (1, 1, 1, True, True), (16, 1, 8, True, True),
])
def test_contract_fp32_arm(lib, oracle, torch, m, n, k, akm, bkm):
    a = rand((m, k) if akm else (k, m), 11)
    b = rand((n, k) if bkm else (k, n), 12)
    got = run_contract(lib, torch, a, b, akm, bkm, FP32)
    assert max_rel_to_peak(got, oracle.contract(a, b, akm, bkm)) <= TOL_FP32


@pytest.mark.parametrize("m,n,k,akm,bkm", [
    (128, 128, 32, True, True), (128, 128, 64, True, True), (256, 512, 256, True, True),
    (200, 300, 100, True, True),       # ragged tiles and K tail
    (130, 70, 36, True, True), (1, 5, 8, True, True),
    (256, 256, 128, True, False),      # `ik*kj~ijk`: B needs the K-major copy
    (192, 160, 96, False, True), (96, 200, 64, False, False),
    (512, 1024, 512, True, True),
])
def test_contract_tf32_arm(lib, oracle, torch, m, n, k, akm, bkm):
    rng = np.random.default_rng(2)
    a = (2 * rng.random((m, k) if akm else (k, m), dtype=np.float32) - 1)
    b = (2 * rng.random((n, k) if bkm else (k, n), dtype=np.float32) - 1)
    got = run_contract(lib, torch, a, b, akm, bkm, TF32)
    assert not np.isnan(got).any()
    assert max_rel_to_peak(got, oracle.contract(a, b, akm, bkm)) <= TOL_TF32


@pytest.mark.parametrize("m,n,k,akm,bkm", [
    (128, 128, 64, True, True), (256, 512, 256, True, True), (200, 300, 100, True, True),
    (130, 70, 36, True, True), (3, 5, 7, True, True),      # K not a multiple of 8: padded copy
    (256, 256, 128, True, False), (96, 200, 64, False, False),
])
def test_contract_bf16_arm(lib, oracle, torch, m, n, k, akm, bkm):
    rng = np.random.default_rng(2)
    a = (2 * rng.random((m, k) if akm else (k, m), dtype=np.float32) - 1)
    b = (2 * rng.random((n, k) if bkm else (k, n), dtype=np.float32) - 1)
    got = run_contract(lib, torch, a, b, akm, bkm, BF16)
    assert not np.isnan(got).any()
    err = max_rel_to_peak(got, oracle.contract(a, b, akm, bkm))
    assert err <= TOL_BF16
    assert err > 1e-6 or k < 8          # really bf16 arithmetic, not the fp32 arm


@pytest.mark.parametrize("m,n,k,akm,bkm", [
    (128, 128, 64, True, True), (256, 512, 256, True, True), (200, 300, 100, True, True),
    (130, 70, 36, True, True), (3, 5, 7, True, True), (1, 1, 1, True, True),
    (256, 256, 128, True, False), (96, 200, 64, False, False), (512, 1024, 512, True, True),
])
def test_contract_f16_arm(lib, oracle, torch, m, n, k, akm, bkm):
    # fp16 operands over one power of two per row: TF32's mantissa, held to the TF32 bound.
    rng = np.random.default_rng(2)
    a = (2 * rng.random((m, k) if akm else (k, m), dtype=np.float32) - 1)
    b = (2 * rng.random((n, k) if bkm else (k, n), dtype=np.float32) - 1)
    got = run_contract(lib, torch, a, b, akm, bkm, F16)
    assert not np.isnan(got).any()
    assert max_rel_to_peak(got, oracle.contract(a, b, akm, bkm)) <= TOL_TF32


def test_contract_f16_is_as_accurate_as_tf32_at_any_magnitude(lib, oracle, torch):
    # Rows of A eight decades apart, B at 1e-20 (far below fp16's range), batched: every row of C
    # must come out as accurately, relative to its own peak, as from the TF32 arm.
    rng = np.random.default_rng(3)
    batch, m, n, k = 2, 300, 260, 512
    a = rng.standard_normal((batch, m, k), dtype=np.float32)
    a *= (np.float32(10.0) ** np.linspace(-4, 4, m).astype(np.float32))[None, :, None]
    b = rng.standard_normal((batch, n, k), dtype=np.float32) * np.float32(1e-20)
    b[1] *= np.float32(1e25)
    got = run_contract(lib, torch, a, b, True, True, F16, batch=batch)
    tf32 = run_contract(lib, torch, a, b, True, True, TF32, batch=batch)
    assert np.isfinite(got).all()
    for i in range(batch):
        ref = a[i].astype(np.float64) @ b[i].astype(np.float64).T
        peak = np.abs(ref).max(axis=1)
        err = (np.abs(got[i] - ref).max(axis=1) / peak).max()
        err_tf32 = (np.abs(tf32[i] - ref).max(axis=1) / peak).max()
        assert err <= TOL_TF32 and err <= 1.5 * err_tf32 + 1e-6, (i, err, err_tf32)


def test_contract_auto_large_deep_shape(lib, torch):
    # Large enough for AUTO to take the fp16 arm (both extents >= 4096, depth >= 2048) when the
    # caller brings the workspace ib_contract_workspace_bytes asks for; checked against float64 on
    # the device (the CPU oracle would need minutes here), with and without that workspace.
    m, n, k = 4096, 4224, 2048
    g = torch.Generator(device="cuda")
    g.manual_seed(7)
    a = torch.randn(m, k, device="cuda", generator=g) * 1e-3
    b = torch.randn(n, k, device="cuda", generator=g) * 1e4
    ref = a.double() @ b.double().t()
    peak = ref.abs().max().item()
    for with_ws in (True, False):
        c = torch.full((m, n), float("nan"), device="cuda")
        wb = lib.ib_contract_workspace_bytes(1, m, n, k, 1, 1, 0) if with_ws else 0
        assert (wb > 0) == with_ws
        ws = torch.empty(max(wb, 256), dtype=torch.uint8, device="cuda")
        ok(lib, lib.ib_contract(a.data_ptr(), b.data_ptr(), c.data_ptr(), 1, m, n, k, 1, 1, 0,
                                ws.data_ptr() if with_ws else None, wb, None))
        err = ((c.double() - ref).abs().max() / peak).item()
        assert err <= TOL_TF32, (with_ws, err)


def test_contract_tf32_batched(lib, oracle, torch):
    a, b = rand((3, 150, 64), 13), rand((3, 90, 64), 14)
    got = run_contract(lib, torch, a, b, True, True, TF32, batch=3)
    for i in range(3):
        assert max_rel_to_peak(got[i], oracle.contract(a[i], b[i])) <= TOL_TF32


def test_contract_config3_sample_and_checksum(lib, oracle, torch):
    # The published mm_t case: A, B 8192x4096 U(-1,1) seed 2 -> C 8192x8192 on the TF32 arm.
    rng = np.random.default_rng(2)
    a = 2 * rng.random((8192, 4096), dtype=np.float32) - 1
    b = 2 * rng.random((8192, 4096), dtype=np.float32) - 1
    da, db = dev(torch, a), dev(torch, b)
    c = torch.empty(8192, 8192, device="cuda")
    ok(lib, lib.ib_contract(da.data_ptr(), db.data_ptr(), c.data_ptr(), 1, 8192, 8192, 4096, 1, 1,
                            TF32, None, 0, None))
    torch.cuda.synchronize()
    # Size-independent property: row sums of C equal A (B^T 1), computed in float64.
    want = da.double() @ db.double().sum(dim=0)
    got = c.double().sum(dim=1)
    scale = (da.double().abs() @ db.double().abs().sum(dim=0)).max().item()
    assert ((got - want).abs().max().item()) / scale < 1e-3
    rows = np.array([0, 1, 127, 128, 4095, 4096, 8190, 8191])
    ref = oracle.contract(a[rows], b)
    assert max_rel_to_peak(c[torch.from_numpy(rows).cuda()].cpu().numpy(), ref) <= TOL_TF32


# ---- attention ------------------------------------------------------------

def run_attention(lib, torch, q, k, v, precision, v_kmajor=False):
    batch = q.shape[0] if q.ndim == 3 else 1
    nq, d = q.shape[-2:]
    nk = k.shape[-2]
    dv = v.shape[-2] if v_kmajor else v.shape[-1]
    dq, dk, dvv = dev(torch, q), dev(torch, k), dev(torch, v)
    o = torch.full((batch, nq, dv), float("nan"), device="cuda")
    ws_bytes = lib.ib_attention_workspace_bytes(batch, nq, nk, d, dv, int(v_kmajor), precision)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    ok(lib, lib.ib_attention(dq.data_ptr(), dk.data_ptr(), dvv.data_ptr(), o.data_ptr(), batch, nq,
                             nk, d, dv, int(v_kmajor), precision, 0, ws.data_ptr(), ws_bytes, None))
    torch.cuda.synchronize()
    out = o.cpu().numpy()
    return out if q.ndim == 3 else out[0]


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "attention_*.npz"))))
@pytest.mark.parametrize("precision,tol", [(FP32, 2e-5), (TF32, TOL_TF32), (BF16, TOL_BF16),
                                           (TF32_F16, TOL_TF32), (F16, TOL_TF32)])
def test_attention_golden(lib, torch, path, precision, tol):
    g = np.load(path)
    got = run_attention(lib, torch, g["q"], g["k"], g["v"], precision)
    assert not np.isnan(got).any()
    assert max_rel_to_peak(got, g["o"]) <= tol


@pytest.mark.parametrize("nq,nk,d,dv", [
    (256, 64, 64, 64), (256, 128, 64, 64), (512, 512, 128, 128), (300, 200, 40, 24),
    (1, 1, 4, 1), (129, 65, 8, 100), (1000, 3000, 128, 128), (64, 4096, 32, 16),
])
def test_attention_tf32_shapes(lib, oracle, torch, nq, nk, d, dv):
    q = rand((nq, d), 15) * np.float32(d ** -0.5)
    k, v = rand((nk, d), 16), rand((nk, dv), 17)
    got = run_attention(lib, torch, q, k, v, TF32)
    assert not np.isnan(got).any()
    assert max_rel_to_peak(got, oracle.attention_fused(q, k, v)) <= TOL_TF32


def test_attention_tf32_random_shapes(lib, oracle, torch):
    # Seeded sweep over ragged shapes (rows, keys, both head dimensions, heads): every way a row
    # tile, a key tile or a feature chunk can be partial, and every split of the work over CTAs
    # that small and medium problems produce.  Each head is checked against the oracle.
    rng = np.random.default_rng(2024)
    for case in range(40):
        batch = int(rng.integers(1, 4))
        nq = int(rng.integers(1, 700))
        nk = int(rng.integers(1, 900))
        d = 4 * int(rng.integers(1, 33))
        dv = int(rng.integers(1, 129))
        q = rand((batch, nq, d), 100 + case) * np.float32(d ** -0.5)
        k, v = rand((batch, nk, d), 200 + case), rand((batch, nk, dv), 300 + case)
        got = run_attention(lib, torch, q, k, v, TF32)
        assert not np.isnan(got).any(), (batch, nq, nk, d, dv)
        for b in range(batch):
            err = max_rel_to_peak(got[b], oracle.attention_fused(q[b], k[b], v[b]))
            assert err <= TOL_TF32, (batch, nq, nk, d, dv, b, err)


@pytest.mark.parametrize("nq,nk,d,dv", [
    (256, 64, 64, 64), (512, 512, 128, 128), (300, 200, 40, 24), (1, 1, 4, 1), (129, 65, 8, 100),
    (1000, 3000, 128, 128), (64, 4096, 32, 16),
])
@pytest.mark.parametrize("precision", [TF32_F16, F16])
def test_attention_tf32_f16_shapes(lib, oracle, torch, nq, nk, d, dv, precision):
    # S = Q K^T in TF32 (or fp16 over per-row / per-tile scales), O += P V in fp16 (same
    # mantissa): held to the TF32 bound.
    q = rand((nq, d), 15) * np.float32(d ** -0.5)
    k, v = rand((nk, d), 16), rand((nk, dv), 17)
    got = run_attention(lib, torch, q, k, v, precision)
    assert not np.isnan(got).any()
    assert max_rel_to_peak(got, oracle.attention_fused(q, k, v)) <= TOL_TF32


def test_attention_f16_is_as_accurate_as_tf32(lib, oracle, torch):
    # fp16 operands carry TF32's 10-bit mantissa: against an exact reference the fp16 arm's error
    # must sit where the TF32 arm's does, not where bf16's (8 bits) does.
    nq, nk, d, dv = 512, 2048, 128, 128
    q = rand((nq, d), 81) * np.float32(d ** -0.5)
    k, v = rand((nk, d), 82), rand((nk, dv), 83)
    ref = oracle.attention_fused(q, k, v)
    err = {name: max_rel_to_peak(run_attention(lib, torch, q, k, v, prec), ref)
           for name, prec in (("tf32", TF32), ("f16", F16), ("bf16", BF16))}
    assert err["f16"] <= 1.5 * err["tf32"] + 1e-5, err
    assert err["f16"] < 0.5 * err["bf16"], err


@pytest.mark.parametrize("q_mag,k_mag", [(1e-20, 1e20), (1e15, 1e-15), (3e4, 1.0), (1.0, 7e4), (1e-6, 1e6)])
def test_attention_f16_operand_magnitudes(lib, oracle, torch, q_mag, k_mag):
    # Q and K far outside fp16's range in opposite directions (their product stays O(1)): the
    # per-row and per-tile powers of two must bring both into range and come back out exactly.
    nq, nk, d, dv = 260, 700, 64, 40
    q = rand((nq, d), 84) * np.float32(d ** -0.5) * np.float32(q_mag)
    k, v = rand((nk, d), 85) * np.float32(k_mag), rand((nk, dv), 86)
    got = run_attention(lib, torch, q, k, v, F16)
    assert np.isfinite(got).all()
    assert max_rel_to_peak(got, oracle.attention_fused(q, k, v)) <= TOL_TF32


def test_attention_f16_rows_and_key_tiles_of_different_magnitude(lib, oracle, torch):
    # Every query row has its own scale, every tile of 128 keys its own: rows six decades apart
    # and key tiles three decades apart each keep full precision.  (Keys that large make the
    # softmax pick single keys; the check is against the oracle on the same inputs.)
    nq, nk, d, dv = 300, 1024, 64, 32
    q = rand((nq, d), 87) * np.float32(d ** -0.5)
    q *= (np.float32(10.0) ** np.linspace(-3, 3, nq).astype(np.float32))[:, None]
    k, v = rand((nk, d), 88), rand((nk, dv), 89)
    k[256:384] *= np.float32(1e-3)
    k[512:640] *= np.float32(30.0)
    q[:, :] /= np.float32(30.0)
    got = run_attention(lib, torch, q, k, v, F16)
    assert np.isfinite(got).all()
    ref = oracle.attention_fused(q, k, v)
    tf32 = run_attention(lib, torch, q, k, v, TF32)
    assert max_rel_to_peak(got, ref) <= max(TOL_TF32, 1.5 * max_rel_to_peak(tf32, ref))


@pytest.mark.parametrize("precision,tol", [(FP32, 2e-5), (TF32, TOL_TF32), (BF16, TOL_BF16),
                                           (TF32_F16, TOL_TF32), (F16, TOL_TF32)])
@pytest.mark.parametrize("c,divide", [(0.125, False), (8.0, True), (-0.25, False), (-5.0, True)])
@pytest.mark.parametrize("nq,nk,d,dv", [(300, 517, 64, 40), (2, 130, 128, 128)])
def test_attention_scaled_logits(lib, oracle, torch, precision, tol, c, divide, nq, nk, d, dv):
    # softmax(c Q K^T) V or softmax(Q K^T / c) V against the oracle's chain with the scale applied
    # to the scores (a negative scale turns the row maximum into the row minimum).
    q, k, v = rand((2, nq, d), 71), rand((2, nk, d), 72), rand((2, nk, dv), 73)
    dq, dk, dvv = dev(torch, q), dev(torch, k), dev(torch, v)
    dc = dev(torch, np.float32([c]))
    o = torch.full((2, nq, dv), float("nan"), device="cuda")
    ws_bytes = lib.ib_attention_workspace_bytes(2, nq, nk, d, dv, 0, precision)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    ok(lib, lib.ib_attention_scaled(dq.data_ptr(), dk.data_ptr(), dvv.data_ptr(), o.data_ptr(), 2, nq,
                                    nk, d, dv, 0, precision, 0, dc.data_ptr(), int(divide),
                                    ws.data_ptr(), ws_bytes, None))
    got = o.cpu().numpy()
    assert not np.isnan(got).any()
    for b in range(2):
        s_ = oracle.contract(q[b], k[b])
        s_ = oracle.map_binary("/" if divide else "*", s_, np.full_like(s_, c))
        ref = oracle.contract(oracle.row_softmax(s_), v[b], b_kmajor=False)
        assert max_rel_to_peak(got[b], ref) <= tol


@pytest.mark.parametrize("scale", [1e-30, 1e-6, 1.0, 3.0e4, 7.0e4, 1e9, 1e30])
@pytest.mark.parametrize("v_kmajor", [False, True])
@pytest.mark.parametrize("precision", [TF32_F16, F16])
def test_attention_tf32_f16_value_range(lib, oracle, torch, scale, v_kmajor, precision):
    # V is scaled per head by a power of two so that its largest magnitude sits just under 2^15:
    # magnitudes far outside fp16's range (6e-5 .. 65504) in either direction must come out as
    # accurately as ordinary ones, and heads with different magnitudes must not affect each other.
    nq, nk, d, dv = 200, 333, 64, 40
    q = rand((2, nq, d), 61) * np.float32(d ** -0.5)
    k = rand((2, nk, d), 62)
    v = rand((2, nk, dv), 63)
    v[0] *= np.float32(scale)
    v[0, 5, 3] = np.float32(scale) * 20           # one outlier sets the head's scale
    ref = [oracle.attention_fused(q[b], k[b], v[b]) for b in range(2)]
    vin = np.ascontiguousarray(np.swapaxes(v, 1, 2)) if v_kmajor else v
    got = run_attention(lib, torch, q, k, vin, precision, v_kmajor=v_kmajor)
    assert np.isfinite(got).all()
    for b in range(2):
        assert max_rel_to_peak(got[b], ref[b]) <= TOL_TF32, (b, scale)


@pytest.mark.parametrize("v_kmajor", [False, True])
def test_attention_tf32_f16_columns_of_different_magnitude(lib, oracle, torch, v_kmajor):
    # The fp16 scaling of V is one power of two per head, chosen from the head's largest magnitude;
    # fp16 then keeps full precision for values down to 2^-29 of that.  Columns whose magnitudes
    # differ by six decades must each come out within the TF32 bound of their own peak.
    nq, nk, d, dv = 300, 500, 64, 37
    q = rand((nq, d), 64) * np.float32(d ** -0.5)
    k, v = rand((nk, d), 65), rand((nk, dv), 66)
    mags = np.float32(10.0) ** np.linspace(-3, 3, dv).astype(np.float32)
    v = v * mags[None, :]
    ref = oracle.attention_fused(q, k, v)
    vin = np.ascontiguousarray(v.T) if v_kmajor else v
    got = run_attention(lib, torch, q, k, vin, TF32_F16, v_kmajor=v_kmajor)
    assert np.isfinite(got).all()
    for c in range(dv):
        err = np.abs(got[:, c] - ref[:, c]).max() / np.abs(ref[:, c]).max()
        assert err <= TOL_TF32, (c, float(mags[c]), float(err))


@pytest.mark.parametrize("nq,nk,d,dv", [
    (256, 128, 64, 64), (512, 512, 128, 128), (300, 200, 40, 24), (129, 65, 8, 100),
    (1000, 3000, 128, 128),
])
def test_attention_bf16_shapes(lib, oracle, torch, nq, nk, d, dv):
    q = rand((nq, d), 15) * np.float32(d ** -0.5)
    k, v = rand((nk, d), 16), rand((nk, dv), 17)
    got = run_attention(lib, torch, q, k, v, BF16)
    assert not np.isnan(got).any()
    err = max_rel_to_peak(got, oracle.attention_fused(q, k, v))
    assert 1e-5 < err <= TOL_BF16          # bf16 arithmetic, within the opt-in bound


def test_attention_tf32_batched_and_transposed_v(lib, oracle, torch):
    q = rand((3, 260, 64), 18) * np.float32(0.125)
    k, v = rand((3, 333, 64), 19), rand((3, 333, 48), 20)
    got = run_attention(lib, torch, q, k, v, TF32)
    vt = np.ascontiguousarray(v.transpose(0, 2, 1))
    got_t = run_attention(lib, torch, q, k, vt, TF32, v_kmajor=True)
    got_b = run_attention(lib, torch, q, k, v, BF16)
    got_bt = run_attention(lib, torch, q, k, vt, BF16, v_kmajor=True)
    for i in range(3):
        ref = oracle.attention_fused(q[i], k[i], v[i])
        assert max_rel_to_peak(got[i], ref) <= TOL_TF32
        assert max_rel_to_peak(got_t[i], ref) <= TOL_TF32
        assert max_rel_to_peak(got_b[i], ref) <= TOL_BF16
        assert max_rel_to_peak(got_bt[i], ref) <= TOL_BF16


@pytest.mark.parametrize("precision,tol", [(TF32, TOL_TF32), (BF16, TOL_BF16), (TF32_F16, TOL_TF32),
                                           (F16, TOL_TF32)])
@pytest.mark.parametrize("v_kmajor", [False, True])
def test_attention_two_phase_matches_one_call(lib, oracle, torch, precision, tol, v_kmajor):
    # K and V prepared once, query rows attended in ragged blocks: same rows as one ib_attention.
    batch, nq, nk, d, dv = 2, 1000, 700, 64, 48
    q = rand((batch, nq, d), 31) * np.float32(d ** -0.5)
    k = rand((batch, nk, d), 32)
    v = rand((batch, dv, nk) if v_kmajor else (batch, nk, dv), 33)
    whole = run_attention(lib, torch, q, k, v, precision, v_kmajor=v_kmajor)
    dk, dvv = dev(torch, k), dev(torch, v)
    pb = lib.ib_attention_prepare_bytes(batch, nk, d, dv, precision)
    prepared = torch.empty(pb, dtype=torch.uint8, device="cuda")
    ok(lib, lib.ib_attention_prepare(dk.data_ptr(), dvv.data_ptr(), batch, nk, d, dv, int(v_kmajor),
                                     precision, prepared.data_ptr(), pb, None))
    got = np.empty_like(whole)
    for r0, r1 in ((0, 1), (1, 300), (300, 1000)):
        rows = r1 - r0
        dq = dev(torch, np.ascontiguousarray(q[:, r0:r1]))
        o = torch.full((batch, rows, dv), float("nan"), device="cuda")
        wb = lib.ib_attention_run_workspace_bytes(batch, rows, nk, dv)
        ws = torch.empty(max(wb, 16), dtype=torch.uint8, device="cuda")
        ok(lib, lib.ib_attention_run(dq.data_ptr(), prepared.data_ptr(), o.data_ptr(), batch, rows,
                                     nk, d, dv, precision, ws.data_ptr(), wb, None))
        torch.cuda.synchronize()
        got[:, r0:r1] = o.cpu().numpy()
    assert not np.isnan(got).any()
    assert max_rel_to_peak(got, whole) <= 1e-5           # same operands, same arithmetic per row
    for b in range(batch):
        vb = np.ascontiguousarray(v[b].T) if v_kmajor else v[b]
        assert max_rel_to_peak(got[b], oracle.attention_fused(q[b], k[b], vb)) <= tol


def test_attention_two_phase_rejects_fp32_arm(lib, torch):
    x = torch.zeros(1 << 16, device="cuda")
    assert lib.ib_attention_prepare(x.data_ptr(), x.data_ptr(), 1, 64, 64, 64, 0, FP32,
                                    x.data_ptr(), 1 << 18, None) == -1
    assert "tensor arms" in last_error(lib)
    assert lib.ib_attention_uses_tensor_arm(1, 16384, 16384, 128, 128, 0) == 1
    assert lib.ib_attention_uses_tensor_arm(1, 16, 16, 128, 128, 0) == 0      # too small under AUTO
    assert lib.ib_attention_uses_tensor_arm(1, 16384, 16384, 130, 128, TF32) == 0


def round_to_tf32(x):
    """fp32 -> nearest value with a 10-bit mantissa (ties to even), as the tensor arms store Q and K."""
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0xFFF + ((bits >> 13) & 1)) & ~np.uint64(0x1FFF)
    return bits.astype(np.uint32).view(np.float32).reshape(np.shape(x))


@pytest.mark.parametrize("precision", [TF32, TF32_F16, F16])
def test_attention_large_scores_stay_finite(lib, oracle, torch, precision):
    # Unscaled Q: logits up to ~ +-130, a peaky softmax whose running maximum moves a lot.  Two
    # comparisons.  Against the reference arithmetic on the operands the tensor cores see (Q and K
    # rounded to a 10-bit mantissa) the kernel has to meet the ordinary bound: what is left is its
    # own work (fp32 accumulation order, P and V rounding, the exponential).  Against the reference
    # on the unrounded operands the distance is dominated by the rounding of Q and K itself: a logit
    # of magnitude 100 moves by up to 100 * 2^-11 = 0.05, i.e. its probability by 5 %, whatever the
    # kernel does afterwards; measured 5.5e-3 of the output's peak on every arm, bound 1e-2.
    q, k, v = rand((256, 128), 21) * 3, rand((1024, 128), 22), rand((1024, 128), 23)
    got = run_attention(lib, torch, q, k, v, precision)
    assert np.isfinite(got).all()
    same_operands = max_rel_to_peak(got, oracle.attention_fused(round_to_tf32(q), round_to_tf32(k), v))
    unrounded = max_rel_to_peak(got, oracle.attention_fused(q, k, v))
    print("large scores, precision %d: %.2e against rounded operands, %.2e against unrounded"
          % (precision, same_operands, unrounded))
    assert same_operands <= TOL_TF32
    assert unrounded <= 1e-2


def test_attention_config4_sample_and_checksum(lib, oracle, torch):
    # The headline attention case: seq 16384, d 128, N(0,1) seed 3, Q scaled by 1/sqrt(128).
    rng = np.random.default_rng(3)
    q = rng.standard_normal((16384, 128), dtype=np.float32)
    k = rng.standard_normal((16384, 128), dtype=np.float32)
    v = rng.standard_normal((16384, 128), dtype=np.float32)
    q *= np.float32(1.0 / np.sqrt(128))
    got = run_attention(lib, torch, q, k, v, TF32)
    assert np.isfinite(got).all()
    rows = np.concatenate([np.arange(0, 16384, 1024), np.arange(255, 16384, 1024), [16383]])
    ref = oracle.attention_fused(q[rows], k, v)
    assert max_rel_to_peak(got[rows], ref) <= TOL_TF32
    # Size-independent property: with V = 1 every output element is the row sum of softmax = 1.
    ones = np.ones_like(v)
    got1 = run_attention(lib, torch, q, k, ones, TF32)
    assert np.abs(got1 - 1.0).max() < 2e-3


@pytest.mark.parametrize("batch,nq,nk", [(40, 640, 100), (40, 640, 256), (37, 700, 300), (3, 8192, 130),
                                         (150, 128, 128), (300, 100, 1), (2, 19000, 384)])
@pytest.mark.parametrize("precision,tol", [(F16, TOL_TF32), (BF16, TOL_BF16)])
def test_attention_many_row_blocks_of_few_key_tiles(lib, torch, batch, nq, nk, precision, tol):
    # More row blocks than SMs and one to three key tiles each: every CTA walks several pieces, and
    # the next block's Q is staged from inside the first (or only) tile of the current one.
    d, dv = 64, 48
    g = torch.Generator(device="cuda")
    g.manual_seed(batch * 7 + nk)
    q = torch.randn(batch, nq, d, device="cuda", generator=g) * d ** -0.5
    k = torch.randn(batch, nk, d, device="cuda", generator=g)
    v = torch.randn(batch, nk, dv, device="cuda", generator=g)
    o = torch.full((batch, nq, dv), float("nan"), device="cuda")
    ws_bytes = lib.ib_attention_workspace_bytes(batch, nq, nk, d, dv, 0, precision)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device="cuda")
    ok(lib, lib.ib_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), batch, nq, nk, d, dv,
                             0, precision, 0, ws.data_ptr(), ws_bytes, None))
    torch.cuda.synchronize()
    assert lib.ib_attention_uses_tensor_arm(batch, nq, nk, d, dv, precision) == 1
    # Same operator in plain fp32 PyTorch (the CPU oracle would take minutes at these sizes; it
    # pins the kernels on the other attention tests).
    torch.backends.cuda.matmul.allow_tf32 = False
    ref = torch.softmax(q @ k.transpose(1, 2), dim=-1) @ v
    assert torch.isfinite(o).all()
    assert ((o - ref).abs().max() / ref.abs().max()).item() <= tol
