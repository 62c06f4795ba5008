"""Python front-end for the B200 `i` runtime.

Same surface as the reference binding (ilang-python/ilang.py): `i("...")` /
`Component` with the `>>` `<<` `&` `|` `~` combinators (ilang.py:278-291), the
identity component `I` (ilang.py:389), `Tensor` for nested lists
(ilang.py:148-186), and `exec`, `exec_numpy`, `exec_torch`, `into`,
`output_shapes`, `_code` (ilang.py:293-360).  It binds the same 19 C symbols
(ilang.py:66-106), so a script written for the reference runs unchanged with
`from i_b200.ilang import ...`.

Extensions, all additive:
  * torch CUDA tensors are accepted as inputs and outputs and are used in place
    (the reference rejects non-CPU tensors, ilang.py:219-228, 376-385);
    `exec_torch` returns CUDA tensors when its inputs are CUDA tensors and the
    work is queued on torch's current stream without synchronising;
  * `Component.set_precision("auto" | "fp32" | "tf32" | "bf16" | "tf32_f16" | "f16")`.

The library is found through ILANG_CORE_LIB (as in the reference, ilang.py:6-9)
or in-tree at i_b200/lib/libi_core.so.  Nothing here computes on the CPU: with
no usable GPU every exec raises RuntimeError with the runtime's message.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_HERE, "lib", "libi_core.so")

PRECISIONS = {"auto": 0, "fp32": 1, "tf32": 2, "bf16": 3, "tf32_f16": 4, "f16": 5}


class _CTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p),
                ("shape", ctypes.POINTER(ctypes.c_size_t)),
                ("rank", ctypes.c_size_t)]


class _COwnedTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.POINTER(ctypes.c_float)),
                ("shape", ctypes.POINTER(ctypes.c_size_t)),
                ("rank", ctypes.c_size_t),
                ("len", ctypes.c_size_t)]


class _COutputs(ctypes.Structure):
    _fields_ = [("tensors", ctypes.POINTER(_COwnedTensor)), ("count", ctypes.c_size_t)]


def load_core(path=None):
    """Load libi_core.so and declare the C signatures (include/i.h, include/i_b200.h)."""
    path = path or os.environ.get("ILANG_CORE_LIB") or DEFAULT_LIB
    if not os.path.exists(path):
        raise RuntimeError(
            "could not find %s; build it with `python -m i_b200.build`" % path)
    lib = ctypes.CDLL(path)
    vp, sz = ctypes.c_void_p, ctypes.c_size_t
    lib.i_parse.argtypes = [ctypes.c_char_p]
    lib.i_parse.restype = vp
    lib.i_identity.argtypes = []
    lib.i_identity.restype = vp
    for name in ("i_chain", "i_compose", "i_fanout", "i_pair"):
        fn = getattr(lib, name)
        fn.argtypes = [vp, vp]
        fn.restype = vp
    lib.i_swap.argtypes = [vp]
    lib.i_swap.restype = vp
    lib.i_code.argtypes = [vp]
    lib.i_code.restype = vp
    lib.i_compile.argtypes = [vp]
    lib.i_compile.restype = vp
    lib.i_output_count.argtypes = [vp]
    lib.i_output_count.restype = sz
    lib.i_output_ranks.argtypes = [vp, ctypes.POINTER(sz)]
    lib.i_output_ranks.restype = ctypes.c_int
    lib.i_output_shapes.argtypes = [vp, ctypes.POINTER(_CTensor), sz,
                                    ctypes.POINTER(ctypes.POINTER(sz))]
    lib.i_output_shapes.restype = ctypes.c_int
    lib.i_exec_into.argtypes = [vp, ctypes.POINTER(_CTensor), sz, ctypes.POINTER(_CTensor), sz]
    lib.i_exec_into.restype = ctypes.c_int
    lib.i_exec.argtypes = [vp, ctypes.POINTER(_CTensor), sz]
    lib.i_exec.restype = _COutputs
    lib.i_error.argtypes = []
    lib.i_error.restype = ctypes.c_char_p
    lib.i_component_free.argtypes = [vp]
    lib.i_program_free.argtypes = [vp]
    lib.i_outputs_free.argtypes = [_COutputs]
    lib.i_string_free.argtypes = [vp]
    lib.i_b200_exec_into.argtypes = [vp, ctypes.POINTER(_CTensor), sz, ctypes.POINTER(_CTensor),
                                     sz, vp]
    lib.i_b200_exec_into.restype = ctypes.c_int
    lib.i_b200_program_set_precision.argtypes = [vp, ctypes.c_int]
    lib.i_b200_program_set_precision.restype = ctypes.c_int
    lib.i_b200_program_precision.argtypes = [vp]
    lib.i_b200_program_precision.restype = ctypes.c_int
    lib.i_b200_device_count.argtypes = []
    lib.i_b200_device_count.restype = ctypes.c_int
    lib.i_b200_set_reserved_sms.argtypes = [ctypes.c_int]
    lib.i_b200_set_reserved_sms.restype = ctypes.c_int
    lib.i_b200_launch_count.argtypes = []
    lib.i_b200_launch_count.restype = sz
    return lib


_core = load_core()


def core():
    """The loaded ctypes library (for callers that use the C ABI directly)."""
    return _core


def launch_count():
    """Kernels launched by the library in this process so far."""
    return int(_core.i_b200_launch_count())


def set_reserved_sms(n):
    """Leave n SMs free next to the persistent attention kernel (for collectives)."""
    _check(_core.i_b200_set_reserved_sms(int(n)))


def _raise_last():
    err = _core.i_error()
    raise RuntimeError(err.decode() if err else "i-core error")


def _check_ptr(ptr):
    if not ptr:
        _raise_last()
    return ptr


def _check(code):
    if code != 0:
        _raise_last()


def _shape_array(shape):
    shape = tuple(int(d) for d in shape)
    return shape, (ctypes.c_size_t * max(len(shape), 1))(*shape)


def _flatten(x):
    if isinstance(x, (int, float)):
        return (), [float(x)]
    if not isinstance(x, (list, tuple)):
        raise TypeError("Tensor expects a scalar or nested Python lists")
    if not x:
        return (0,), []
    child_shape, _ = _flatten(x[0])
    out = []
    for item in x:
        item_shape, item_data = _flatten(item)
        if item_shape != child_shape:
            raise ValueError("ragged Tensor input")
        out.extend(item_data)
    return (len(x),) + child_shape, out


class Tensor:
    """Host tensor built from nested lists, or a view of runtime-owned output."""

    def __init__(self, x, shape=None):
        if shape is None:
            shape, data = _flatten(x)
        else:
            shape = tuple(int(d) for d in shape)
            data = [float(v) for v in x]
        self.shape = tuple(shape)
        self._len = len(data)
        self._data = (ctypes.c_float * max(self._len, 1))(*data)
        self._shape, self._shape_buf = _shape_array(self.shape)
        self._owner = None

    @classmethod
    def _from_owned(cls, owner, index):
        raw = owner.outputs.tensors[index]
        self = cls.__new__(cls)
        self.shape = tuple(raw.shape[i] for i in range(raw.rank))
        self._len = raw.len
        self._data = raw.data
        self._shape, self._shape_buf = _shape_array(self.shape)
        self._owner = owner
        return self

    @property
    def data(self):
        return [self._data[i] for i in range(self._len)]

    def numpy(self):
        import numpy as np
        return np.ctypeslib.as_array(self._data, shape=(self._len,))[: self._len].reshape(
            self.shape).copy()

    def _view(self):
        return _CTensor(ctypes.cast(self._data, ctypes.c_void_p), self._shape_buf, len(self.shape))

    def __repr__(self):
        return "Tensor(shape=%s, data=%s)" % (self.shape, self.data)


class _OwnedOutputs:
    def __init__(self, outputs):
        self.outputs = outputs

    def __del__(self):
        outputs = getattr(self, "outputs", None)
        if outputs is not None:
            self.outputs = None
            _core.i_outputs_free(outputs)


def _is_torch(x):
    return hasattr(x, "data_ptr") and hasattr(x, "shape") and hasattr(x, "device")


def _on_cuda(x):
    return _is_torch(x) and x.device.type == "cuda"


def _view_of(x, writable):
    """(_CTensor, keepalive, is_cuda) for one argument."""
    if isinstance(x, Tensor):
        if writable:
            raise TypeError("outputs must be NumPy arrays or Torch tensors")
        return x._view(), x, False
    try:
        import numpy as np
    except ImportError:  # pragma: no cover
        np = None
    if np is not None and isinstance(x, np.generic) and not writable:
        x = np.asarray(x, dtype=np.float32)             # a NumPy scalar is a rank-0 tensor
    if np is not None and isinstance(x, np.ndarray):
        arr = x
        if arr.dtype != np.float32 or not arr.flags.c_contiguous:
            if writable:
                raise TypeError("NumPy outputs must be float32 and C-contiguous")
            arr = np.ascontiguousarray(arr, dtype=np.float32)
        shape, buf = _shape_array(arr.shape)
        return _CTensor(arr.ctypes.data, buf, len(shape)), (arr, buf), False
    if _is_torch(x):
        if str(x.dtype) != "torch.float32":
            raise TypeError("Torch tensors must be float32")
        if not x.is_contiguous():
            if writable:
                raise TypeError("Torch outputs must be contiguous")
            x = x.contiguous()
        shape, buf = _shape_array(tuple(x.shape))
        return _CTensor(x.data_ptr(), buf, len(shape)), (x, buf), x.device.type == "cuda"
    if writable:
        raise TypeError("outputs must be NumPy arrays or Torch tensors")
    return _view_of(Tensor(x), False)


def _views(xs, writable=False):
    items = [_view_of(x, writable) for x in xs]
    arr = (_CTensor * max(len(items), 1))(*(v for v, _, _ in items))
    return arr, [k for _, k, _ in items], [c for _, _, c in items]


class Component:
    def __init__(self, src=None, _ptr=None):
        if _ptr is None:
            if src is None:
                raise TypeError("Component needs source")
            _ptr = _core.i_parse(src.encode())
        self._ptr = _check_ptr(_ptr)
        self._program = None
        self._precision = None

    def __del__(self):
        program = getattr(self, "_program", None)
        ptr = getattr(self, "_ptr", None)
        if _core is None:          # interpreter shutdown: the library is already gone
            return
        if program:
            _core.i_program_free(program)
            self._program = None
        if ptr:
            _core.i_component_free(ptr)
            self._ptr = None

    def _bin(self, other, fn):
        if not isinstance(other, Component):
            other = Component(other)
        return Component(_ptr=_check_ptr(fn(self._ptr, other._ptr)))

    def chain(self, other):
        return self._bin(other, _core.i_chain)

    def compose(self, other):
        return self._bin(other, _core.i_compose)

    def fanout(self, other):
        return self._bin(other, _core.i_fanout)

    def pair(self, other):
        return self._bin(other, _core.i_pair)

    def swap(self):
        return Component(_ptr=_check_ptr(_core.i_swap(self._ptr)))

    __rshift__ = chain
    __lshift__ = compose
    __and__ = fanout
    __or__ = pair

    def __invert__(self):
        return self.swap()

    def _compile(self):
        if self._program is None:
            self._program = _check_ptr(_core.i_compile(self._ptr))
            if self._precision is not None:
                _check(_core.i_b200_program_set_precision(self._program, self._precision))
        return self._program

    def set_precision(self, name):
        """Arithmetic of this component's contractions: auto, fp32, tf32 or bf16."""
        self._precision = PRECISIONS[name]
        if self._program is not None:
            _check(_core.i_b200_program_set_precision(self._program, self._precision))
        return self

    def _code(self):
        s = _check_ptr(_core.i_code(self._ptr))
        try:
            return ctypes.cast(s, ctypes.c_char_p).value.decode()
        finally:
            _core.i_string_free(s)

    def output_shapes(self, *inputs):
        program = self._compile()
        input_arr, keep, _ = _views(inputs)
        count = _core.i_output_count(program)
        ranks = (ctypes.c_size_t * max(count, 1))()
        _check(_core.i_output_ranks(program, ranks))
        bufs = [(ctypes.c_size_t * max(ranks[i], 1))() for i in range(count)]
        ptrs = (ctypes.POINTER(ctypes.c_size_t) * max(count, 1))(
            *(ctypes.cast(b, ctypes.POINTER(ctypes.c_size_t)) for b in bufs))
        _check(_core.i_output_shapes(program, input_arr, len(inputs), ptrs))
        return [tuple(b[j] for j in range(ranks[i])) for i, b in enumerate(bufs)]

    def exec(self, *inputs):
        program = self._compile()
        input_arr, keep, _ = _views(inputs)
        outputs = _core.i_exec(program, input_arr, len(inputs))
        if outputs.count == 0:
            _check(-1)
        owner = _OwnedOutputs(outputs)
        tensors = [Tensor._from_owned(owner, i) for i in range(outputs.count)]
        return tensors[0] if len(tensors) == 1 else tuple(tensors)

    def exec_numpy(self, *inputs):
        import numpy as np
        outs = [np.empty(s, dtype=np.float32) for s in self.output_shapes(*inputs)]
        self.into(outs if len(outs) != 1 else outs[0], *inputs)
        return outs[0] if len(outs) == 1 else tuple(outs)

    def exec_torch(self, *inputs):
        import torch
        device = "cpu"
        for x in inputs:
            if _on_cuda(x):
                device = x.device
                break
        outs = [torch.empty(s, dtype=torch.float32, device=device)
                for s in self.output_shapes(*inputs)]
        self.into(outs if len(outs) != 1 else outs[0], *inputs)
        return outs[0] if len(outs) == 1 else tuple(outs)

    def into(self, outputs, *inputs):
        """Run into caller-provided outputs.

        With every tensor on one CUDA device the call is asynchronous on torch's
        current stream; otherwise it copies host tensors through the GPU and
        returns when the outputs are complete (reference: ilang.py:346-360).
        """
        program = self._compile()
        if not isinstance(outputs, (tuple, list)):
            outputs = (outputs,)
        input_arr, keep_in, cuda_in = _views(inputs)
        output_arr, keep_out, cuda_out = _views(outputs, writable=True)
        flags = cuda_in + cuda_out
        if flags and all(flags):
            import torch
            dev = next(x for x in list(inputs) + list(outputs) if _on_cuda(x)).device
            with torch.cuda.device(dev):
                stream = torch.cuda.current_stream().cuda_stream
                _check(_core.i_b200_exec_into(program, input_arr, len(inputs), output_arr,
                                              len(outputs), ctypes.c_void_p(stream)))
        else:
            _check(_core.i_exec_into(program, input_arr, len(inputs), output_arr, len(outputs)))
        return outputs[0] if len(outputs) == 1 else tuple(outputs)


I = Component(_ptr=_core.i_identity())


def i(src):
    return Component(src)
