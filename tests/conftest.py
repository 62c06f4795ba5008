import ctypes
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def _have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


HAVE_GPU = _have_gpu()


def pytest_collection_modifyitems(config, items):
    if HAVE_GPU:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def ilang():
    """The repo's front-end, with the library built on demand."""
    from i_b200 import build
    build.build()
    from i_b200 import ilang as mod
    return mod


@pytest.fixture(scope="session")
def lib(ilang):
    """libi_core.so with the ib_* kernel signatures declared."""
    lib = ilang.core()
    vp, sz, ci = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    pd = ctypes.POINTER(ctypes.c_ssize_t)
    ps = ctypes.POINTER(sz)
    lib.ib_map_unary.argtypes = [ci, vp, vp, sz, vp]
    lib.ib_map_binary.argtypes = [ci, ci, vp, vp, vp, sz, sz, vp]
    lib.ib_map_strided.argtypes = [ci, vp, vp, vp, ci, ps, pd, pd, vp]
    lib.ib_map_chain.argtypes = [ci, ctypes.POINTER(ci), ci, ctypes.POINTER(vp), ctypes.POINTER(ci),
                                 vp, sz, sz, vp]
    lib.ib_reduce_rows.argtypes = [ci, vp, vp, sz, sz, vp]
    lib.ib_reduce_rows_chain.argtypes = [ci, ci, ctypes.POINTER(ci), ci, ctypes.POINTER(vp),
                                         ctypes.POINTER(ci), vp, sz, sz, vp]
    lib.ib_reduce_strided.argtypes = [ci, vp, vp, ci, ps, pd, ci, ps, pd, vp]
    lib.ib_row_softmax.argtypes = [vp, vp, sz, sz, vp]
    lib.ib_contract.argtypes = [vp, vp, vp, sz, sz, sz, sz, ci, ci, ci, vp, sz, vp]
    lib.ib_contract_workspace_bytes.argtypes = [sz, sz, sz, sz, ci, ci, ci]
    lib.ib_contract_workspace_bytes.restype = sz
    lib.ib_attention.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, ci, ci, sz, vp, sz, vp]
    lib.ib_attention_scaled.argtypes = [vp, vp, vp, vp, sz, sz, sz, sz, sz, ci, ci, sz, vp, ci, vp, sz, vp]
    lib.ib_attention_scaled.restype = ci
    lib.ib_attention_workspace_bytes.argtypes = [sz, sz, sz, sz, sz, ci, ci]
    lib.ib_attention_workspace_bytes.restype = sz
    lib.ib_attention_prepare_bytes.argtypes = [sz, sz, sz, sz, ci]
    lib.ib_attention_prepare_bytes.restype = sz
    lib.ib_attention_prepare.argtypes = [vp, vp, sz, sz, sz, sz, ci, ci, vp, sz, vp]
    lib.ib_attention_prepare.restype = ci
    lib.ib_attention_run_workspace_bytes.argtypes = [sz, sz, sz, sz]
    lib.ib_attention_run_workspace_bytes.restype = sz
    lib.ib_attention_run.argtypes = [vp, vp, vp, sz, sz, sz, sz, sz, ci, vp, sz, vp]
    lib.ib_attention_run.restype = ci
    lib.ib_attention_uses_tensor_arm.argtypes = [sz, sz, sz, sz, sz, ci]
    lib.ib_attention_uses_tensor_arm.restype = ci
    for name in ("ib_map_unary", "ib_map_binary", "ib_map_strided", "ib_map_chain", "ib_reduce_rows",
                 "ib_reduce_rows_chain",
                 "ib_reduce_strided", "ib_row_softmax", "ib_contract", "ib_attention"):
        getattr(lib, name).restype = ci
    return lib


@pytest.fixture(scope="session")
def oracle():
    import oracle as mod
    mod.build()
    return mod


def last_error(lib):
    err = lib.i_error()
    return err.decode() if err else None


def max_rel_to_peak(got, ref):
    """max|got - ref| / max|ref|: the contraction/attention error metric."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-300))


def max_rel_elementwise(got, ref):
    """max over elements of |got - ref| / |ref|: the map/reduce error metric."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    denom = np.maximum(np.abs(ref), 1e-300)
    return float((np.abs(got - ref) / denom).max())
