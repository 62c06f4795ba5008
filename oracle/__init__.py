"""ctypes driver for the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this package; the shipped library never does.  `restated` wraps
`libi_oracle.so` (oracle/i_oracle.c, a restatement of what the reference's C
backend emits).  `reference_attention` wraps `_ref/libref_flashattn.so`, the
reference's own emitted C for the README attention component
(ilang-python/annotated-flashattn.c) compiled by oracle/Makefile, through the
generated-module ABI (ABI.md:5-10: count / ranks / shapes / exec).
"""
import ctypes
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libi_oracle.so")
_REF = os.path.join(_HERE, "_ref", "libref_flashattn.so")

OPS = {"+": 0, "*": 1, "-": 2, "/": 3, ">": 4, "<": 5, "^": 6, "$": 7,
       ">>": 8, ">=": 9, "<<": 10, "<=": 11, "==": 12, "!=": 13,
       "&&": 14, "||": 15, "^^": 16, "!!": 17}

_fp = ctypes.POINTER(ctypes.c_float)
_sz = ctypes.c_size_t


def build():
    """Compile the oracle (and `_ref` when the reference checkout is present)."""
    subprocess.run(["make", "-C", _HERE, "-s"], check=True, stdout=subprocess.DEVNULL)


def _load(path):
    if not os.path.exists(path):
        build()
    return ctypes.CDLL(path)


class _Restated:
    def __init__(self):
        self._lib = None

    @property
    def lib(self):
        if self._lib is None:
            lib = _load(_LIB)
            lib.io_map_unary.argtypes = [ctypes.c_int, _fp, _fp, _sz]
            lib.io_map_binary.argtypes = [ctypes.c_int, ctypes.c_int, _fp, _fp, _fp, _sz, _sz]
            lib.io_reduce_rows.argtypes = [ctypes.c_int, _fp, _fp, _sz, _sz]
            lib.io_contract.argtypes = [_fp, _fp, _fp, _sz, _sz, _sz, ctypes.c_int, ctypes.c_int]
            lib.io_row_softmax.argtypes = [_fp, _fp, _sz, _sz]
            lib.io_attention_fused.argtypes = [_fp, _fp, _fp, _fp, _sz, _sz, _sz, _sz]
            lib.io_attention_naive.argtypes = [_fp, _fp, _fp, _fp, _fp, _sz, _sz, _sz, _sz]
            for name in ("io_map_unary", "io_map_binary", "io_reduce_rows", "io_contract",
                         "io_row_softmax", "io_attention_fused", "io_attention_naive"):
                getattr(lib, name).restype = None
            self._lib = lib
        return self._lib


_restated = _Restated()


def _f32(x):
    return np.ascontiguousarray(x, dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(_fp)


def map_unary(op, x):
    x = _f32(x)
    y = np.empty_like(x)
    _restated.lib.io_map_unary(OPS[op], _p(x), _p(y), x.size)
    return y


def map_binary(op, a, b, mode=0):
    """mode: 0 a[r,c]·b[r,c]; 1 a[r,c]·b[r]; 2 a[r]·b[r,c]; 3 a[r,c]·b[c]; 4 a[c]·b[r,c]."""
    a, b = _f32(a), _f32(b)
    full = a if mode in (0, 1, 3) else b
    rows = int(np.prod(full.shape[:-1])) if full.ndim > 1 else 1
    cols = full.shape[-1]
    y = np.empty_like(full)
    _restated.lib.io_map_binary(OPS[op], mode, _p(a), _p(b), _p(y), rows, cols)
    return y


def reduce_rows(op, x):
    x = _f32(x)
    rows = int(np.prod(x.shape[:-1]))
    y = np.empty(x.shape[:-1], dtype=np.float32)
    _restated.lib.io_reduce_rows(OPS[op], _p(x), _p(y), rows, x.shape[-1])
    return y


def contract(a, b, a_kmajor=True, b_kmajor=True):
    """C[i,j] = sum_k A(i,k) B(j,k); *_kmajor False means the operand is stored [k][row]."""
    a, b = _f32(a), _f32(b)
    ni, nk = (a.shape if a_kmajor else a.shape[::-1])
    nj = b.shape[0] if b_kmajor else b.shape[1]
    c = np.empty((ni, nj), dtype=np.float32)
    _restated.lib.io_contract(_p(a), _p(b), _p(c), ni, nj, nk, int(a_kmajor), int(b_kmajor))
    return c


def contract_rows(a_rows, b, threads=None):
    """`contract` on slices of A's rows, one slice per task, on `threads` host cores (rows of C
    are independent, and ctypes releases the GIL).  Returns the list of output slices in order."""
    threads = threads or os.cpu_count() or 1
    n = a_rows.shape[0]
    cuts = np.linspace(0, n, min(threads, n) + 1).astype(int)
    with ThreadPoolExecutor(max_workers=threads) as pool:
        futs = [pool.submit(contract, a_rows[lo:hi], b) for lo, hi in zip(cuts[:-1], cuts[1:]) if hi > lo]
        return [f.result() for f in futs]


def row_softmax(x):
    x = _f32(x)
    rows = int(np.prod(x.shape[:-1]))
    y = np.empty_like(x)
    _restated.lib.io_row_softmax(_p(x), _p(y), rows, x.shape[-1])
    return y


def attention_fused(q, k, v):
    q, k, v = _f32(q), _f32(k), _f32(v)
    o = np.empty((q.shape[0], v.shape[1]), dtype=np.float32)
    _restated.lib.io_attention_fused(_p(q), _p(k), _p(v), _p(o), q.shape[0], k.shape[0],
                                     q.shape[1], v.shape[1])
    return o


def attention_naive(q, k, v):
    q, k, v = _f32(q), _f32(k), _f32(v)
    o = np.empty((q.shape[0], v.shape[1]), dtype=np.float32)
    s = np.empty((q.shape[0], k.shape[0]), dtype=np.float32)
    _restated.lib.io_attention_naive(_p(q), _p(k), _p(v), _p(o), _p(s), q.shape[0], k.shape[0],
                                     q.shape[1], v.shape[1])
    return o


# ---------------------------------------------------------------------------
# The reference's own emitted C (when built).
# ---------------------------------------------------------------------------

class _Tensor(ctypes.Structure):
    _fields_ = [("data", _fp), ("shape", ctypes.POINTER(_sz)), ("rank", _sz)]


_ref_lib = None


def have_reference():
    return os.path.exists(_REF)


def _ref():
    global _ref_lib
    if _ref_lib is None:
        lib = ctypes.CDLL(_REF)
        lib.exec.argtypes = [ctypes.POINTER(_Tensor), ctypes.POINTER(_Tensor)]
        lib.exec.restype = None
        lib.shapes.argtypes = [ctypes.POINTER(_Tensor), ctypes.POINTER(ctypes.POINTER(_sz))]
        lib.shapes.restype = None
        lib.count.restype = _sz
        _ref_lib = lib
    return _ref_lib


def _view(a):
    shape = (_sz * a.ndim)(*a.shape)
    return _Tensor(_p(a), shape, a.ndim), shape


def reference_attention(q, k, v):
    """Run the reference's emitted `exec` (single thread) on host arrays."""
    lib = _ref()
    q, k, v = _f32(q), _f32(k), _f32(v)
    views = [_view(x) for x in (q, k, v)]
    ins = (_Tensor * 3)(*(t for t, _ in views))
    out_shape = (_sz * 2)()
    rows = (ctypes.POINTER(_sz) * 1)(ctypes.cast(out_shape, ctypes.POINTER(_sz)))
    lib.shapes(ins, rows)
    o = np.empty((out_shape[0], out_shape[1]), dtype=np.float32)
    ov, keep = _view(o)
    outs = (_Tensor * 1)(ov)
    lib.exec(ins, outs)
    return o


def reference_attention_rows(q, k, v, row_blocks, threads=None, fn=None):
    """Run attention on several Q row-slices concurrently (one slice per task).

    Rows of the fused kernel are independent given full K/V, so slices reproduce
    the corresponding rows of a full run bit for bit.  ctypes releases the GIL,
    so a thread pool uses that many host cores.  Returns the list of outputs.
    """
    fn = fn or reference_attention
    threads = threads or os.cpu_count() or 1
    with ThreadPoolExecutor(max_workers=threads) as pool:
        futs = [pool.submit(fn, q[a:b], k, v) for a, b in row_blocks]
        return [f.result() for f in futs]


def numpy_attention(q, k, v):
    """float64 NumPy attention, the secondary check (ilang-python/flash-attn.py:38-43)."""
    q, k, v = (np.asarray(x, dtype=np.float64) for x in (q, k, v))
    s = q @ np.swapaxes(k, -1, -2)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    w = w / w.sum(axis=-1, keepdims=True)
    return w @ v
