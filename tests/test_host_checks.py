"""Host-side checks of the kernel library that need no GPU: extents whose element counts do not
fit size_t are refused before anything is launched, and kernel attributes are set once per device."""
import ctypes

import pytest

from conftest import last_error

SIZE_MAX = ctypes.c_size_t(-1).value
FP32, AUTO, TF32 = 1, 0, 2


def declare(lib):
    sz, ci, vp = ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p
    lib.ib_attention_workspace_bytes.restype = sz
    lib.ib_attention_workspace_bytes.argtypes = [sz, sz, sz, sz, sz, ci, ci]
    lib.ib_contract_workspace_bytes.restype = sz
    lib.ib_contract_workspace_bytes.argtypes = [sz] * 4 + [ci] * 3
    lib.ib_attention.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, ci, ci, sz, vp, sz, vp]
    lib.ib_attention_static.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, ci, vp]
    lib.ib_contract.argtypes = [vp, vp, vp, sz, sz, sz, sz, ci, ci, ci, vp, sz, vp]
    lib.ib_attention_run_workspace_bytes.restype = sz
    lib.ib_attention_run_workspace_bytes.argtypes = [sz] * 4
    lib.ib_selftest_once_per_device.restype = ci
    lib.ib_selftest_once_per_device.argtypes = [ci, ci, ci]


# batch * nq * nk = 2^62 floats: times four bytes that wraps to zero.
WRAPPING = (2048, 1 << 21, 1 << 30, 1, 1)


@pytest.mark.parametrize("precision", [FP32, AUTO, TF32])
def test_workspace_size_of_wrapping_extents_is_unsatisfiable(lib, precision):
    declare(lib)
    batch, nq, nk, d, dv = WRAPPING
    assert lib.ib_attention_workspace_bytes(batch, nq, nk, d, dv, 0, precision) == SIZE_MAX
    assert lib.ib_attention_run_workspace_bytes(batch, nq, nk, dv) == SIZE_MAX
    assert lib.ib_contract_workspace_bytes(1 << 22, 1 << 21, 1 << 21, 4, 0, 0, precision) == SIZE_MAX
    # Ordinary extents are unaffected.
    assert 0 < lib.ib_attention_workspace_bytes(1, 16384, 16384, 128, 128, 0, AUTO) < 1 << 30


def test_entry_points_refuse_wrapping_extents_before_touching_the_gpu(lib):
    declare(lib)
    batch, nq, nk, d, dv = WRAPPING
    fake = ctypes.c_void_p(256)            # never dereferenced: the refusal comes first
    rc = lib.ib_attention(fake, fake, fake, fake, batch, nq, nk, d, dv, 0, FP32, 0, fake, 1 << 25, None)
    assert rc == -1 and "extents too large" in last_error(lib)
    rc = lib.ib_attention_static(fake, fake, fake, fake, batch, nq, nk, d, dv, 0, None)
    assert rc == -1 and "extents too large" in last_error(lib)
    rc = lib.ib_contract(fake, fake, fake, 1 << 22, 1 << 21, 1 << 21, 4, 1, 1, FP32, None, 0, None)
    assert rc == -1 and "extents too large" in last_error(lib)


def test_kernel_attributes_are_set_once_per_device(lib):
    declare(lib)
    assert lib.ib_selftest_once_per_device(4, 5, 0) == 4          # once each, however many calls
    assert lib.ib_selftest_once_per_device(8, 3, 0) == 8
    assert lib.ib_selftest_once_per_device(4, 5, 2) == 12         # two failures are retried, then once
    assert lib.ib_selftest_once_per_device(3, 1, 2) == 3          # a failure is not remembered as done


def test_operators_after_a_contraction_are_checked_before_anything_is_launched(lib):
    declare(lib)
    sz, ci, vp = ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p
    lib.ib_contract_chain.argtypes = [vp, vp, vp, sz, sz, sz, sz, ci, ci, ci, sz, sz, ci,
                                      ctypes.POINTER(ci), ci, ctypes.POINTER(vp), ctypes.POINTER(ci),
                                      vp, sz, vp]
    fake = ctypes.c_void_p(256)            # never dereferenced: the refusals come first
    ADD, DIV, PREV, NONE = 0, 3, -2, -1

    def call(ops, n_operands=1, modes=(2,)):
        flat = (ci * len(ops))(*ops)
        ptrs = (vp * 3)(256, 256, 256)
        return lib.ib_contract_chain(fake, fake, fake, 1, 64, 64, 64, 1, 1, FP32, 0, 0, len(ops) // 3, flat,
                                     n_operands, ptrs, (ci * 3)(*modes, *([0] * (3 - len(modes)))), None, 0,
                                     None)

    assert call([DIV, PREV, 0]) == -1 and "only + - * > <" in last_error(lib)
    assert call([ADD, 0, 0]) == -1 and "exactly one side" in last_error(lib)
    assert call([ADD, PREV, PREV]) == -1 and "exactly one side" in last_error(lib)
    assert call([ADD, PREV, 1]) == -1 and "out of range" in last_error(lib)
    assert call([ADD, NONE, PREV]) == -1
    assert call([ADD, PREV, 0], modes=(7,)) == -1 and "mode" in last_error(lib)
    assert call([ADD, PREV, 0] * 9) == -1 and "operators" in last_error(lib)
    assert call([ADD, PREV, 0], n_operands=4) == -1 and "operands" in last_error(lib)


def test_workspace_sizes_of_folds_and_split_contractions(lib):
    declare(lib)
    sz = ctypes.c_size_t
    lib.ib_reduce_rows_workspace_bytes.restype = sz
    lib.ib_reduce_rows_workspace_bytes.argtypes = [sz, sz]
    lib.ib_reduce_leading_workspace_bytes.restype = sz
    lib.ib_reduce_leading_workspace_bytes.argtypes = [sz, sz, sz]
    # Many rows, or short ones, are folded whole; a handful of very long rows in segments of at
    # least 8192 columns, one partial result per segment.
    assert lib.ib_reduce_rows_workspace_bytes(8192, 8192) == 0
    assert lib.ib_reduce_rows_workspace_bytes(1, 20000) == 0
    whole_array = lib.ib_reduce_rows_workspace_bytes(1, 8192 * 8192)
    assert 0 < whole_array <= 4 * 8192 and whole_array % 4 == 0
    assert lib.ib_reduce_rows_workspace_bytes(64, 1 << 20) >= 64 * 2 * 4
    # Folds of leading axes: slabs x columns partial results per array; none for a few rows.
    assert lib.ib_reduce_leading_workspace_bytes(1, 8, 4096) == 0
    tall = lib.ib_reduce_leading_workspace_bytes(1, 1 << 20, 64)
    assert tall > 0 and tall % (64 * 4) == 0
    assert lib.ib_reduce_leading_workspace_bytes(3, 1 << 16, 256) % (3 * 256 * 4) == 0
    assert lib.ib_reduce_leading_workspace_bytes(0, 5, 5) == 0
    assert lib.ib_reduce_leading_workspace_bytes(1 << 30, 1 << 30, 1 << 30) == SIZE_MAX
    # A contraction with few output tiles and a long sum asks for room for the copies it adds up;
    # one with plenty of tiles, or on the vector routes, does not.
    assert lib.ib_contract_workspace_bytes(1, 128, 128, 4096, 1, 1, FP32) >= 2 * 128 * 128 * 4
    assert lib.ib_contract_workspace_bytes(1, 2048, 2048, 4096, 1, 1, FP32) == 0
    assert lib.ib_contract_workspace_bytes(1, 8192, 1, 8192, 1, 1, AUTO) == 0
    assert lib.ib_contract_workspace_bytes(1, 8192, 1, 8192, 0, 1, AUTO) > 0      # [k][rows]: slabs' partial sums
