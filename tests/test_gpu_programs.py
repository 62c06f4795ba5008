"""GPU end-to-end tests through the front-end: the reference's own acceptance
cases (ilang-python/test.py:40-128, ilang-python/flash-attn.py:31-77) with the
reference's tolerances, plus the boundary behaviours of include/i.h."""
import numpy as np
import pytest

from conftest import max_rel_elementwise, max_rel_to_peak
from test_front import deferred_attention, naive_attention, readme_attention, scaled_attention

pytestmark = pytest.mark.gpu


def rand(shape, seed):
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


def as_numpy(t):
    return np.asarray(t.data, dtype=np.float32).reshape(t.shape)


def np_attention(q, k, v):
    s = q.astype(np.float64) @ np.swapaxes(k.astype(np.float64), -1, -2)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    w = w / w.sum(axis=-1, keepdims=True)
    return w @ v.astype(np.float64)


def test_matmul_with_bang_init(ilang):
    # test.py:40-59, nested-list Tensors through i_exec.
    a, b = rand((8, 16), 1), rand((16, 7), 2)
    f = ilang.i("ik*kj~ijk|i:2,k:2|ii'jkk'") >> ilang.i("+ijk~ij|i:2,k:2|ii'j!kk'0")
    got = as_numpy(f.exec(ilang.Tensor(a.tolist()), ilang.Tensor(b.tolist())))
    np.testing.assert_allclose(got, a.astype(np.float64) @ b.astype(np.float64), rtol=1e-5, atol=1e-6)


def test_batched_attention_naive_schedule(ilang):
    # test.py:61-82: b2 h3 q4 k4 d8.
    i, I = ilang.i, ilang.I
    q, k, v = rand((2, 3, 4, 8), 1), rand((2, 3, 4, 8), 2), rand((2, 3, 4, 8), 3)
    mm_t = i("bhij*bhkj~bhikj | i:16,k:16 | bhkii'k'j") >> i("+bhikj~bhik | i:16,k:16 | bhkii'k'j0")
    rms = (I & i(">bhik~bhi | i:16,k:16 | bhkii'k'")) >> i("bhik-bhi~bhik | i:16,k:16 | bh1kii'k'")
    exp = i("^bhik~bhik | i:16,k:16 | bhkii'k'")
    rn = (I & i("+bhik~bhi | i:16,k:16 | bhkii'k'")) >> i("bhik/bhi~bhik | i:16,k:16 | bh1kii'k'")
    mm = i("bhik*bhkj~bhijk | i:16,k:16 | bhkii'jk'") >> i("+bhijk~bhij | i:16,k:16 | bhkii'jk'0")
    attn = mm_t >> rms >> exp >> rn >> mm
    got = as_numpy(attn.exec(*(ilang.Tensor(x.tolist()) for x in (q, k, v))))
    np.testing.assert_allclose(got, np_attention(q, k, v), rtol=1e-5, atol=1e-6)


def test_mlp_intent(ilang):
    # test.py:84-98 means w2 @ relu(w1 @ x); written with the combinators that exist.
    i = ilang.i
    x, w1, w2 = rand((8,), 1), rand((16, 8), 2), rand((7, 16), 3)
    mvp = i("ij*j~ij") >> i("+ij~i")
    hidden = mvp >> i(">i~i")
    f = (ilang.I | hidden) >> (i("ij*j~ij") >> i("+ij~i"))
    got = f.exec_numpy(w2, w1, x)
    ref = w2.astype(np.float64) @ np.maximum(w1.astype(np.float64) @ x, 0)
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-5)


def test_comparison_and_logic_components(ilang):
    # Operators of compiler/src/front/parser.rs:270-279 through whole components: a causal-style
    # mask built from comparisons, a column-wise "any", and not-of-a-reduction.
    i = ilang.i
    x = rand((33, 20), 1)
    x[x < -1.0] = 0.0
    thr = rand((20,), 2)
    mask = i("ij>>j~ij").exec_numpy(x, thr)                       # 1 where x > thr[j]
    assert np.array_equal(mask, (x > thr[None, :]).astype(np.float32))
    sel = i("ij*ij~ij").exec_numpy(mask, x)                       # select by mask
    assert np.array_equal(sel, np.where(x > thr[None, :], x, 0.0).astype(np.float32))
    any_col = i("||ij~j").exec_numpy(x)
    assert np.array_equal(any_col, (x != 0).any(axis=0).astype(np.float32))
    none_row = (i("||ij~i") >> i("!!i~i")).exec_numpy(x)
    assert np.array_equal(none_row, (~(x != 0).any(axis=1)).astype(np.float32))
    parity = i("^^ij~i").exec_numpy(x)
    assert np.array_equal(parity, ((x != 0).sum(axis=1) % 2).astype(np.float32))
    both = i("ij&&ij~ij").exec_numpy(x, mask)
    assert np.array_equal(both, ((x != 0) & (mask != 0)).astype(np.float32))


def test_pointwise_chain_components(ilang, oracle):
    # Consecutive maps over one index space run as one kernel; results are those of the maps one
    # after another (each rounded to fp32), which is what the oracle computes here.
    i = ilang.i
    x, b, g = rand((130, 72), 1), rand((72,), 2), rand((130, 72), 3)
    f = i("ij+j~ij") >> i(">ij~ij") >> i("ij*ij~ij")
    assert "map_chain" in f._code()
    ref = oracle.map_binary("*", oracle.map_unary(">", oracle.map_binary("+", x, b, 3)), g)
    assert np.array_equal(f.exec_numpy(x, b, g), ref)
    # Batched, per-row operands (the two halves of a softmax whose statistics come from elsewhere).
    y, m, l = rand((3, 50, 41), 4), rand((3, 50), 5), np.abs(rand((3, 50), 6)) + 0.5
    h = i("bij-bi~bij") >> i("^bij~bij") >> i("bij/bi~bij")
    ref = oracle.map_binary("/", oracle.map_unary("^", oracle.map_binary("-", y, m, 1)), l, 1)
    got = h.exec_numpy(y, m, l)
    assert got.shape == (3, 50, 41) and max_rel_elementwise(got, ref) <= 1e-5
    # Rank 1 with a scalar, and a chain feeding a reduction.
    two = np.array(2.0, dtype=np.float32)
    v = rand((1000,), 7)
    assert np.array_equal((i(".*i~i") >> i("-i~i")).exec_numpy(two, v), -(2 * v))
    norm = i("ij*ij~ij") >> i("-ij~ij") >> i("+ij~i")
    ref = oracle.reduce_rows("+", oracle.map_unary("-", oracle.map_binary("*", x, x)))
    assert max_rel_elementwise(norm.exec_numpy(x, x), ref) <= 1e-5


def test_chain_reduction_components(ilang, oracle):
    i, I = ilang.i, ilang.I
    x, m = rand((70, 130), 1), rand((70,), 2) + 2.0
    denom = i("ij-i~ij") >> i("^ij~ij") >> i("+ij~i")
    assert "chain_reduce" in denom._code()
    ref = oracle.reduce_rows("+", oracle.map_unary("^", oracle.map_binary("-", x, m, 1)))
    assert max_rel_elementwise(denom.exec_numpy(x, m), ref) <= 1e-5
    # log-sum-exp with the maximum taken by the program itself: fan-out, two folds, two chains.
    lse = (I & i(">ij~i")) >> (i("ij-i~ij") >> i("^ij~ij") >> i("+ij~i") >> i("$i~i"))
    got = lse.exec_numpy(x)
    want = np.log(np.exp(x.astype(np.float64) - x.max(axis=1, keepdims=True)).sum(axis=1))
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    # Batched "any above the column's threshold", exact.
    y, t = rand((3, 40, 33), 3), rand((33,), 4) + 1.5
    any_above = i("bij>>j~bij") >> i("||bij~bi")
    assert np.array_equal(any_above.exec_numpy(y, t), (y > t).any(axis=2).astype(np.float32))
    # Rank 1 to a scalar.
    v = rand((1000,), 5)
    got = (i("-i~i") >> i(">i~.")).exec_numpy(v)
    assert got.shape == () and got == np.max(-v)


@pytest.mark.parametrize("src,fn", [(">ij~i", np.max), ("<ij~i", np.min), ("+ij~i", np.sum)])
def test_row_reductions(ilang, src, fn):
    # test.py:103-128
    x = rand((16, 8), 1)
    got = as_numpy(ilang.i(src).exec(ilang.Tensor(x.tolist())))
    np.testing.assert_allclose(got, fn(x.astype(np.float64), axis=1), rtol=1e-5, atol=1e-6)


def test_flash_attention_demo(ilang):
    # flash-attn.py:31-77: 32 x 32 x 2048, fused and naive schedules, rtol 3e-4 / atol 5e-5.
    q, k, v = rand((32, 2048), 1), rand((32, 2048), 2), rand((32, 2048), 3)
    ref = np_attention(q, k, v)
    for attn in (readme_attention(ilang), naive_attention(ilang)):
        assert isinstance(attn._code(), str)
        np.testing.assert_allclose(attn.exec_numpy(q, k, v), ref, rtol=3e-4, atol=5e-5)


def test_config1_through_the_front_end(ilang, oracle):
    rng = np.random.default_rng(0)
    q, k, v = (rng.standard_normal((128, 64), dtype=np.float32) for _ in range(3))
    q *= np.float32(1 / 8)
    ref = oracle.attention_fused(q, k, v)
    attn = readme_attention(ilang)
    assert max_rel_to_peak(attn.exec_numpy(q, k, v), ref) <= 2e-5       # auto -> fp32 arm
    attn.set_precision("tf32")
    assert max_rel_to_peak(attn.exec_numpy(q, k, v), ref) <= 5e-3       # fused tcgen05 kernel


@pytest.mark.parametrize("shift", [False, True])
def test_deferred_normalisation_attention(ilang, shift):
    # exp >> (mm & row_sum) >> row_div (stage_to_kernel_program.rs:2705-2780), fused and unfused.
    q = rand((300, 64), 51) * np.float32(64 ** -0.5)
    k, v = rand((500, 64), 52), rand((500, 48), 53)
    ref = np_attention(q, k, v)
    for staged in (True, False):
        attn = deferred_attention(ilang, shift=shift, staged=staged)
        np.testing.assert_allclose(attn.exec_numpy(q, k, v), ref, rtol=3e-4, atol=5e-5)   # fp32 arm
        attn.set_precision("tf32")
        assert max_rel_to_peak(attn.exec_numpy(q, k, v), ref) <= 5e-3
    # Logits beyond exp's range (|S| up to ~150): the fused step works relative to the row maximum,
    # so the unshifted form stays finite too.  Exact arm for the values, tensor arm for finiteness
    # (TF32 rounding of logits this large moves the probabilities themselves).
    big = deferred_attention(ilang, shift=False)
    qb = q * np.float32(40.0)
    assert max_rel_to_peak(big.exec_numpy(qb, k, v), np_attention(qb, k, v)) <= 1e-4
    big.set_precision("tf32")
    assert np.isfinite(big.exec_numpy(qb, k, v)).all()


@pytest.mark.parametrize("kind", ["mul_right", "mul_left", "div"])
def test_scaled_dot_product_attention(ilang, kind):
    # The 1/sqrt(d) of scaled-dot-product attention written into the component: one fused kernel,
    # on the tensor arm (large case) and on the exact arm (small case).
    attn = scaled_attention(ilang, kind)
    assert "step 0: attention" in attn._code()
    for (nq, nk, d, dv), tol in (((700, 900, 64, 64), 5e-3), ((40, 50, 16, 8), 1e-5)):
        q, k, v = rand((nq, d), 1), rand((nk, d), 2), rand((nk, dv), 3)
        c = np.float32(d ** 0.5 if kind == "div" else d ** -0.5)
        args = (c, q, k, v) if kind == "mul_left" else (q, k, c, v)
        attn.set_precision("auto" if tol > 1e-4 else "fp32")
        got = attn.exec_numpy(*args)
        ref = np_attention(q * np.float32(d ** -0.5), k, v)
        assert max_rel_to_peak(got, ref) <= tol


def test_scaled_attention_batched_on_device(ilang):
    import torch
    attn = scaled_attention(ilang, "div", batched=True)
    q, k, v = rand((2, 3, 260, 64), 4), rand((2, 3, 300, 64), 5), rand((2, 3, 300, 32), 6)
    c = torch.tensor(8.0, device="cuda")
    got = attn.exec_torch(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), c,
                          torch.from_numpy(v).cuda()).cpu().numpy()
    assert max_rel_to_peak(got, np_attention(q / 8.0, k, v)) <= 5e-3


def batched_readme_attention(ilang):
    """README attention with a leading head axis: one invocation for all heads."""
    i, I = ilang.i, ilang.I
    mm_t = i("hik*hjk~hijk | i:16,j:16 | hjii'j'k") >> i("+hijk~hij | i:16,j:16 | hjii'j'k0")
    row_max_shift = (I & i(">hij~hi | i:16,j:16 | hji0i'j'")) >> i("hij-hi~hij | i:16,j:16 | hji01i'j'")
    exp = i("^hij~hij | i:16,j:16 | hji0i'j'")
    row_normalize = (I & i("+hij~hi | i:16,j:16 | hji0i'j'")) >> i("hij/hi~hij | i:16,j:16 | hji01i'j'")
    mm = i("hij*hjk~hikj | i:16,j:16 | hji0i'kj'") >> i("+hikj~hik | i:16,j:16 | hjii'kj'0")
    return mm_t >> row_max_shift >> exp >> row_normalize >> mm


def test_host_buffers_one_head_pipelined_by_query_rows(ilang, oracle):
    # Large enough that i_exec_into overlaps its copies with the kernels, block by block of
    # query rows (ragged last block: 8100 rows).  Rows are checked against the reference's
    # emitted C where it was built, else the restated oracle.
    nq, nk, d = 8100, 2048, 128
    q = rand((nq, d), 41) * np.float32(d ** -0.5)
    k, v = rand((nk, d), 42), rand((nk, d), 43)
    attn = readme_attention(ilang)
    launches = ilang.launch_count()
    got = attn.exec_numpy(q, k, v)
    assert ilang.launch_count() - launches >= 5          # one preparation, several row blocks
    assert got.shape == (nq, d) and not np.isnan(got).any()
    rows = np.r_[0:64, 2000:2064, 4090:4110, nq - 36:nq]
    ref = oracle.attention_fused(q[rows], k, v)
    assert max_rel_to_peak(got[rows], ref) <= 5e-3
    assert max_rel_to_peak(got, np_attention(q, k, v)) <= 5e-3
    out = np.full((nq, d), np.nan, dtype=np.float32)      # same through `into`
    attn.into(out, q, k, v)
    assert np.array_equal(out, got)


def test_host_buffers_many_heads_pipelined_by_heads(ilang, oracle):
    heads, n, d = 20, 512, 64                              # blocks of 3 heads, the last of 2
    q = rand((heads, n, d), 44) * np.float32(d ** -0.5)
    k, v = rand((heads, n, d), 45), rand((heads, n, d), 46)
    attn = batched_readme_attention(ilang)
    assert "attention" in attn._code()
    got = attn.exec_numpy(q, k, v)
    assert got.shape == (heads, n, d) and not np.isnan(got).any()
    assert max_rel_to_peak(got, np_attention(q, k, v)) <= 5e-3
    for h in (0, 7, 19):
        assert max_rel_to_peak(got[h], oracle.attention_fused(q[h], k[h], v[h])) <= 5e-3


def test_softmax_component_config2_slice(ilang, oracle):
    i, I = ilang.i, ilang.I
    sm = ((I & i(">ij~i | i:16,j:16 | jii'j'")) >> i("ij-i~ij | i:16,j:16 | 1jii'j'")) \
        >> i("^ij~ij | i:16,j:16 | jii'j'") \
        >> ((I & i("+ij~i | i:16,j:16 | jii'j'")) >> i("ij/i~ij | i:16,j:16 | 1jii'j'"))
    x = 2.0 * np.random.default_rng(1).standard_normal((256, 8192), dtype=np.float32)
    assert max_rel_elementwise(sm.exec_numpy(x), oracle.row_softmax(x)) <= 1e-5


def test_mm_t_component_tf32(ilang, oracle):
    i = ilang.i
    mm_t = i("ik*jk~ijk | i:16,j:16 | jii'j'k") >> i("+ijk~ij | i:16,j:16 | jii'j'k0")
    rng = np.random.default_rng(2)
    a = 2 * rng.random((512, 1024), dtype=np.float32) - 1
    b = 2 * rng.random((384, 1024), dtype=np.float32) - 1
    got = mm_t.exec_numpy(a, b)                                        # auto -> tensor arm
    assert max_rel_to_peak(got, oracle.contract(a, b)) <= 5e-3
    mm_t.set_precision("fp32")
    assert max_rel_to_peak(mm_t.exec_numpy(a, b), oracle.contract(a, b)) <= 1e-5
    mm_t.set_precision("bf16")                                         # opt-in BF16 arm
    assert max_rel_to_peak(mm_t.exec_numpy(a, b), oracle.contract(a, b)) <= 2e-2


@pytest.mark.parametrize("precision", ["fp32", "tf32", "bf16", "f16"])
def test_pointwise_operators_in_the_contraction_epilogue(ilang, oracle, precision):
    # A layer (product, bias, rectifier) and a gated form compile to one contraction step.  On
    # every arm the result must be, bit for bit, the arm's contraction followed by the pointwise
    # kernels (the product of the fp32 arm is the oracle's, so there the whole layer is pinned).
    i, I = ilang.i, ilang.I
    rng = np.random.default_rng(31)
    mm_t = i("ik*jk~ijk") >> i("+ijk~ij")
    layer = mm_t >> i("ij+j~ij") >> i(">ij~ij")
    gated = (I | mm_t | I) >> (i("i-ij~ij") | I) >> i("ij*ij~ij") >> i("<ij~ij")
    assert steps_of_code(layer._code()) == ["contract"] and steps_of_code(gated._code()) == ["contract"]
    for comp in (mm_t, layer, gated):
        comp.set_precision(precision)
    # Ragged against every tile (300 x 260), the CTA-pair kernel (512 x 768), and a shape whose
    # rows are not a multiple of four floats wide (scalar loads and stores in the epilogue).
    for m, n, k in ((300, 260, 96), (512, 768, 256), (130, 131, 64)):
        a = 2 * rng.random((m, k), dtype=np.float32) - 1
        b = 2 * rng.random((n, k), dtype=np.float32) - 1
        bias, row = rand((n,), 5), rand((m,), 6)
        gate = rand((m, n), 7)
        product = mm_t.exec_numpy(a, b)
        want = oracle.map_unary(">", oracle.map_binary("+", product, bias, 3))
        assert np.array_equal(layer.exec_numpy(a, b, bias), want), (precision, m, n, k)
        want = oracle.map_unary("<", oracle.map_binary("*", oracle.map_binary("-", row, product, 2), gate))
        assert np.array_equal(gated.exec_numpy(row, a, b, gate), want), (precision, m, n, k)
        if precision == "fp32":
            assert max_rel_to_peak(product, oracle.contract(a, b)) <= 1e-5
    # Batch axes: the per-row operand is indexed by (batch, row).
    batched = (i("bik*bjk~bijk") >> i("+bijk~bij")) >> i("bij+bi~bij")
    batched.set_precision(precision)
    plain = i("bik*bjk~bijk") >> i("+bijk~bij")
    plain.set_precision(precision)
    a, b, shift = rand((3, 140, 64), 8), rand((3, 150, 64), 9), rand((3, 140), 10)
    want = oracle.map_binary("+", plain.exec_numpy(a, b), shift, 1)
    assert np.array_equal(batched.exec_numpy(a, b, shift), want)


@pytest.mark.parametrize("precision", ["auto", "fp32", "tf32"])
def test_matrix_vector_and_row_dot_contractions(ilang, precision):
    # Contractions with one output axis (or none) per batch entry are passes over memory: they run
    # as a weighted row fold in fp32 under every precision.  Short rows (a warp per row), long rows
    # (a block per row), widths that are not a multiple of four, batch entries with their own
    # vector, the vector on either side.
    i = ilang.i

    def check(comp, args, want):
        comp.set_precision(precision)
        got = comp.exec_numpy(*args)
        assert got.shape == want.shape
        assert max_rel_to_peak(got, want) <= 2e-6, (precision, [a.shape for a in args])

    for rows, k in ((300, 1000), (70, 4100), (129, 1001), (5, 3)):
        a, b, x = rand((rows, k), 11), rand((rows, k), 12), rand((k,), 13)
        a64, b64, x64 = (t.astype(np.float64) for t in (a, b, x))
        check(i("ij*j~ij") >> i("+ij~i"), (a, x), a64 @ x64)                    # matrix times vector
        check(i("j*ij~ij") >> i("+ij~i"), (x, a), a64 @ x64)                    # vector on the left
        check(i("ij*ij~ij") >> i("+ij~i"), (a, b), (a64 * b64).sum(axis=1))     # row-wise dot products
        # The matrix stored the other way round, [k][rows]: a weighted fold down its columns.
        at = np.ascontiguousarray(a.T)
        check(i("j*ji~ji") >> i("+ji~i"), (x, at), a64 @ x64)
        check(i("ji*j~ji") >> i("+ji~i"), (at, x), a64 @ x64)
    a, x = rand((3, 40, 260), 14), rand((3, 260), 15)
    check(i("bij*bj~bij") >> i("+bij~bi"), (a, x), np.einsum("bij,bj->bi", a.astype(np.float64), x.astype(np.float64)))
    y = rand((3, 40), 21)
    check(i("bi*bij~bij") >> i("+bij~bj"), (y, a), np.einsum("bi,bij->bj", y.astype(np.float64), a.astype(np.float64)))
    u, v = rand((2048,), 16), rand((2048,), 17)
    check(i("i*i~i") >> i("+i~."), (u, v), np.asarray(u.astype(np.float64) @ v.astype(np.float64)))
    # A layer on a vector: product, bias, rectifier (the operators after the product are a pass of
    # their own here: there is no tile epilogue to put them in).
    w, x, bias = rand((96, 512), 18), rand((512,), 19), rand((96,), 20)
    layer = i("ij*j~ij") >> i("+ij~i") >> i("i+i~i") >> i(">i~i")
    want = np.maximum(w.astype(np.float64) @ x.astype(np.float64) + bias, 0)
    check(layer, (w, x, bias), want)


def test_folds_of_leading_axes(ilang, oracle):
    # `+ij~j`, `>bij~ij`, `+bij~j`: the kept axes trail, the folded ones lead; rows are folded in
    # slabs and the slabs' results once more.  Maxima and the logic folds are exact, sums differ
    # from a serial sum by rounding only, and repeat from run to run.
    i = ilang.i
    for rows, cols in ((5000, 260), (33, 4100), (1001, 129), (7, 1), (100000, 8)):
        x = rand((rows, cols), 22)
        got = i("+ij~j").exec_numpy(x)
        assert got.shape == (cols,)
        assert max_rel_to_peak(got, x.astype(np.float64).sum(axis=0)) <= 2e-6, (rows, cols)
        assert np.array_equal(got, i("+ij~j").exec_numpy(x))
        assert np.array_equal(i(">ij~j").exec_numpy(x), x.max(axis=0))
        assert np.array_equal(i("<ij~j").exec_numpy(x), x.min(axis=0))
        truth = (x > 0.5).astype(np.float32)
        assert np.array_equal(i("||ij~j").exec_numpy(truth), truth.max(axis=0))
        assert np.array_equal(i("^^ij~j").exec_numpy(truth), truth.sum(axis=0) % 2)
    x = rand((6, 300, 44), 23)
    assert np.array_equal(i(">bij~ij").exec_numpy(x), x.max(axis=0))
    assert max_rel_to_peak(i("+bij~j").exec_numpy(x), x.astype(np.float64).sum(axis=(0, 1))) <= 2e-6
    # A fold of the middle axis: one such array per leading entry.
    assert np.array_equal(i(">bij~bj").exec_numpy(x), x.max(axis=1))
    assert max_rel_to_peak(i("+bij~bj").exec_numpy(x), x.astype(np.float64).sum(axis=1)) <= 2e-6
    y = rand((3, 4, 700, 36), 27)
    assert np.array_equal(i("<abij~abj").exec_numpy(y), y.min(axis=2))
    assert np.array_equal(i(">abij~aj").exec_numpy(y), y.max(axis=(1, 2)))
    # More leading entries than the kernel's grid has room for: the strided fold takes over.
    many = rand((70000, 3, 4), 34)
    assert np.array_equal(i(">bij~bj").exec_numpy(many), many.max(axis=1))
    # Kept axes that change places, or folded axes apart from each other, stay with the strided fold.
    assert np.array_equal(i(">bij~jb").exec_numpy(x), x.max(axis=1).T)
    assert np.array_equal(i(">abij~bj").exec_numpy(y), y.max(axis=(0, 2)))


def test_permutations_and_broadcasts_move_whole_lines(ilang):
    # Copies with the last two axes exchanged go through the tiled transpose; maps whose operands
    # are contiguous or constant along the innermost axis run four results at a time.  Results
    # are exact either way; shapes with and without a multiple of four innermost.
    i = ilang.i
    for shape in ((300, 520), (33, 77), (1, 64), (2048, 4)):
        x = rand(shape, 28)
        assert np.array_equal(i("ij~ji").exec_numpy(x), x.T)
    tall = rand((4200000, 2), 36)                      # more row tiles than the tile kernel's grid: element by element
    assert np.array_equal(i("ij~ji").exec_numpy(tall), tall.T)
    t = rand((5, 130, 72), 29)
    assert np.array_equal(i("bij~bji").exec_numpy(t), t.transpose(0, 2, 1))
    assert np.array_equal(i("bij~ibj").exec_numpy(t), t.transpose(1, 0, 2))
    assert np.array_equal(i("bij~jib").exec_numpy(t), t.transpose(2, 1, 0))
    assert np.array_equal(i("-bij~bji").exec_numpy(t), -t.transpose(0, 2, 1))
    for last in (72, 70):
        t = rand((5, 130, last), 30)
        m, r, c = rand((5, last), 31), rand((130,), 32), rand((last,), 33)
        assert np.array_equal(i("bij*bj~bij").exec_numpy(t, m), t * m[:, None, :])
        assert np.array_equal(i("bj-bij~bij").exec_numpy(m, t), m[:, None, :] - t)
        assert np.array_equal(i("bij+i~bij").exec_numpy(t, r), t + r[None, :, None])
        assert np.array_equal(i("i*j~ij").exec_numpy(r, c), np.outer(r, c))
        assert np.array_equal(i("j*i~ij").exec_numpy(c, r), np.outer(r, c))


@pytest.mark.parametrize("precision,bound", [("fp32", 1e-5), ("auto", 5e-3), ("tf32", 5e-3)])
def test_contractions_with_few_output_tiles_and_a_long_sum(ilang, precision, bound):
    # A small output over a long k (a Gram matrix of few features, one block of logits) has too few
    # tiles for the machine: its k range is cut into parts, each summed into a copy of the result,
    # and the copies are added.  Every operand layout, batch entries, ragged shapes, and operators
    # on the sum.
    i = ilang.i
    rng = np.random.default_rng(35)

    def draw(*shape):
        return (2 * rng.random(shape, dtype=np.float32) - 1)

    forms = {"ik*jk~ijk": "ik,jk->ij", "ik*kj~ijk": "ik,kj->ij", "ki*jk~ijk": "ki,jk->ij", "ki*kj~ijk": "ki,kj->ij"}
    for m, n, k in ((128, 128, 4096), (100, 60, 5000), (30, 257, 12288)):
        for src, ein in forms.items():
            a = draw(*((m, k) if src[:2] == "ik" else (k, m)))
            b = draw(*((n, k) if src[3:5] == "jk" else (k, n)))
            comp = (i(src) >> i("+ijk~ij")).set_precision(precision)
            want = np.einsum(ein, a.astype(np.float64), b.astype(np.float64))
            assert max_rel_to_peak(comp.exec_numpy(a, b), want) <= bound, (precision, src, m, n, k)
    a, b, bias = draw(3, 70, 6000), draw(3, 50, 6000), draw(50)
    comp = (i("bik*bjk~bijk") >> i("+bijk~bij") >> i("bij+j~bij") >> i(">bij~bij")).set_precision(precision)
    want = np.maximum(np.einsum("bik,bjk->bij", a.astype(np.float64), b.astype(np.float64)) + bias, 0)
    assert max_rel_to_peak(comp.exec_numpy(a, b, bias), want) <= bound


def test_folds_of_few_very_long_rows(ilang):
    # A fold of a whole array is one row of millions of columns: it is cut into segments, one CTA
    # each, and the segments' results are folded once more.  Also the dot product of two long
    # vectors, and widths that are not a multiple of four.
    i = ilang.i
    for shape in ((3000, 3000), (5, 1000003), (40, 70001)):
        x = rand(shape, 24)
        x64 = x.astype(np.float64)
        assert max_rel_to_peak(i("+ij~.").exec_numpy(x), np.asarray(x64.sum())) <= 2e-6 * np.sqrt(x.size), shape
        assert np.array_equal(i(">ij~.").exec_numpy(x), np.asarray(x.max()))
        got = i("+ij~i").exec_numpy(x)
        assert max_rel_to_peak(got, x64.sum(axis=1)) <= 2e-6, shape
        assert np.array_equal(got, i("+ij~i").exec_numpy(x))
        assert np.array_equal(i("<ij~i").exec_numpy(x), x.min(axis=1))
    u, v = rand((5000001,), 25), rand((5000001,), 26)
    want = np.asarray(u.astype(np.float64) @ v.astype(np.float64))
    got = (i("i*i~i") >> i("+i~.")).exec_numpy(u, v)
    assert abs(got - want) <= 1e-6 * np.abs(u.astype(np.float64) * v).sum()


def steps_of_code(code):
    return [line.split()[2] for line in code.splitlines() if line.startswith("step ")]


def test_multiple_outputs_identity_and_swap(ilang):
    i, I = ilang.i, ilang.I
    x = rand((6, 5), 4)
    both = ~(i("+ij~i") & i(">ij~i"))
    mx, sm = both.exec_numpy(x)
    assert np.array_equal(mx, x.max(axis=1))
    np.testing.assert_allclose(sm, x.sum(axis=1), rtol=1e-5, atol=1e-6)
    same, neg = (I & i("-ij~ij")).exec_numpy(x)
    assert np.array_equal(same, x) and np.array_equal(neg, -x)
    t = i("ij~ji").exec_numpy(x)
    assert np.array_equal(t, x.T)
    total = i("+ij~.").exec_numpy(np.abs(x))
    np.testing.assert_allclose(total, np.abs(x).sum(), rtol=1e-5)


def test_scalar_operand_and_column_broadcast(ilang):
    i = ilang.i
    x, c = rand((4, 9), 5), rand((9,), 6)
    assert np.array_equal(i("ij*j~ij").exec_numpy(x, c), x * c[None, :])
    two = np.array(2.0, dtype=np.float32)
    assert np.array_equal(i(".*ij~ij").exec_numpy(two, x), 2 * x)


def test_torch_cuda_tensors_run_in_place(ilang, oracle):
    import torch
    attn = readme_attention(ilang).set_precision("tf32")
    q, k, v = (torch.randn(512, 64, device="cuda") for _ in range(3))
    q *= 0.125
    before = ilang.launch_count()
    o = attn.exec_torch(q, k, v)
    torch.cuda.synchronize()
    assert o.is_cuda and ilang.launch_count() > before
    ref = oracle.attention_fused(q.cpu().numpy(), k.cpu().numpy(), v.cpu().numpy())
    assert max_rel_to_peak(o.cpu().numpy(), ref) <= 5e-3


def test_shape_errors_are_reported_not_crashes(ilang):
    attn = readme_attention(ilang)
    with pytest.raises(RuntimeError):
        attn.exec_numpy(rand((8, 4), 1), rand((8, 5), 2), rand((8, 4), 3))
    with pytest.raises(RuntimeError):
        ilang.i("+ij~i").exec_numpy(rand((8,), 1))


def test_concurrent_exec_from_threads(ilang, oracle):
    # One program, several host threads (legal in the reference: exec uses only locals).
    from concurrent.futures import ThreadPoolExecutor
    sm = ((ilang.I & ilang.i(">ij~i")) >> ilang.i("ij-i~ij")) >> ilang.i("^ij~ij") \
        >> ((ilang.I & ilang.i("+ij~i")) >> ilang.i("ij/i~ij"))
    xs = [2 * rand((64, 300), s) for s in range(8)]
    with ThreadPoolExecutor(4) as pool:
        outs = list(pool.map(sm.exec_numpy, xs))
    for x, o in zip(xs, outs):
        assert max_rel_elementwise(o, oracle.row_softmax(x)) <= 1e-5


def test_concurrent_pipelined_attention_from_threads(ilang):
    # Several host threads run the copy/compute pipeline of host-buffer attention at once (each
    # thread has its own three streams); results must not mix.
    from concurrent.futures import ThreadPoolExecutor
    attn = readme_attention(ilang)
    cases = []
    for s in range(6):
        q = rand((4096, 128), 70 + s) * np.float32(128 ** -0.5)
        cases.append((q, rand((2048, 128), 80 + s), rand((2048, 128), 90 + s)))
    with ThreadPoolExecutor(3) as pool:
        outs = list(pool.map(lambda c: attn.exec_numpy(*c), cases))
    for (q, k, v), o in zip(cases, outs):
        assert max_rel_to_peak(o, np_attention(q, k, v)) <= 5e-3

