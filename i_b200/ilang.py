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
import array
import ctypes
import os
import weakref

_HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_LIB = os.path.join(_HERE, "lib", "libi_core.so")

PRECISIONS = {"auto": 0, "fp32": 1, "tf32": 2, "bf16": 3, "tf32_f16": 4, "f16": 5}

_VOIDP, _SIZE, _INT = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
_SIZE_P = ctypes.POINTER(_SIZE)


class _CTensor(ctypes.Structure):
    """ITensor of include/i.h: a borrowed float buffer with its extents."""
    _fields_ = [("data", _VOIDP), ("shape", _SIZE_P), ("rank", _SIZE)]


class _COwnedTensor(ctypes.Structure):
    """IOwnedTensor: one output of i_exec, owned by the runtime until i_outputs_free."""
    _fields_ = [("data", ctypes.POINTER(ctypes.c_float)), ("shape", _SIZE_P), ("rank", _SIZE),
                ("len", _SIZE)]


class _COutputs(ctypes.Structure):
    _fields_ = [("tensors", ctypes.POINTER(_COwnedTensor)), ("count", _SIZE)]


_CTENSOR_P = ctypes.POINTER(_CTensor)

# symbol -> (result type, argument types); include/i.h first, then include/i_b200.h.
_SIGNATURES = {
    "i_parse": (_VOIDP, [ctypes.c_char_p]),
    "i_identity": (_VOIDP, []),
    "i_chain": (_VOIDP, [_VOIDP, _VOIDP]),
    "i_compose": (_VOIDP, [_VOIDP, _VOIDP]),
    "i_fanout": (_VOIDP, [_VOIDP, _VOIDP]),
    "i_pair": (_VOIDP, [_VOIDP, _VOIDP]),
    "i_swap": (_VOIDP, [_VOIDP]),
    "i_code": (_VOIDP, [_VOIDP]),
    "i_compile": (_VOIDP, [_VOIDP]),
    "i_output_count": (_SIZE, [_VOIDP]),
    "i_output_ranks": (_INT, [_VOIDP, _SIZE_P]),
    "i_output_shapes": (_INT, [_VOIDP, _CTENSOR_P, _SIZE, ctypes.POINTER(_SIZE_P)]),
    "i_exec_into": (_INT, [_VOIDP, _CTENSOR_P, _SIZE, _CTENSOR_P, _SIZE]),
    "i_exec": (_COutputs, [_VOIDP, _CTENSOR_P, _SIZE]),
    "i_error": (ctypes.c_char_p, []),
    "i_component_free": (None, [_VOIDP]),
    "i_program_free": (None, [_VOIDP]),
    "i_outputs_free": (None, [_COutputs]),
    "i_string_free": (None, [_VOIDP]),
    "i_b200_exec_into": (_INT, [_VOIDP, _CTENSOR_P, _SIZE, _CTENSOR_P, _SIZE, _VOIDP]),
    "i_b200_program_set_precision": (_INT, [_VOIDP, _INT]),
    "i_b200_program_precision": (_INT, [_VOIDP]),
    "i_b200_device_count": (_INT, []),
    "i_b200_set_reserved_sms": (_INT, [_INT]),
    "i_b200_launch_count": (_SIZE, []),
}


def load_core(path=None):
    """Load libi_core.so and declare the C signatures (include/i.h, include/i_b200.h)."""
    path = path or os.environ.get("ILANG_CORE_LIB") or DEFAULT_LIB
    if not os.path.exists(path):
        raise RuntimeError("could not find %s; build it with `python -m i_b200.build`" % path)
    lib = ctypes.CDLL(path)
    for symbol, (result, arguments) in _SIGNATURES.items():
        fn = getattr(lib, symbol)
        fn.restype, fn.argtypes = result, arguments
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
    _ok(_core.i_b200_set_reserved_sms(int(n)))


def _fail():
    message = _core.i_error()
    raise RuntimeError(message.decode() if message else "i-core error")


def _ok(status):
    """int-returning calls: 0 is success, anything else carries a message in i_error()."""
    if status:
        _fail()


def _handle(pointer):
    """pointer-returning calls: NULL is failure."""
    if pointer is None or pointer == 0:
        _fail()
    return pointer


class _Extents:
    """A size_t array for a shape (at least one slot, so rank 0 still has an address)."""

    def __init__(self, shape):
        self.shape = tuple(int(n) for n in shape)
        self.buffer = (_SIZE * (len(self.shape) or 1))(*self.shape)

    def describe(self, address):
        return _CTensor(address, self.buffer, len(self.shape))


def _nested_extents(value):
    """Extents of nested lists, read along the first element of every level."""
    extents = []
    while isinstance(value, (list, tuple)):
        extents.append(len(value))
        if not value:
            break
        value = value[0]
    return tuple(extents)


def _pour(value, extents, level, sink):
    """Append the numbers of nested lists to `sink`, checking every level against `extents`."""
    if level == len(extents):
        if isinstance(value, (list, tuple)) or not isinstance(value, (int, float)):
            raise (ValueError("ragged Tensor input") if isinstance(value, (list, tuple))
                   else TypeError("Tensor expects a scalar or nested Python lists"))
        sink.append(float(value))
        return
    if not isinstance(value, (list, tuple)) or len(value) != extents[level]:
        raise ValueError("ragged Tensor input")
    for item in value:
        _pour(item, extents, level + 1, sink)


_EMPTY = array.array("f", [0.0])


class Tensor:
    """A host tensor of floats: from a number, from nested lists, or from flat values plus a
    shape.  The values live in a Python-owned float array whose address is handed to the runtime."""

    def __init__(self, x, shape=None):
        values = array.array("f")
        if shape is not None:
            shape = tuple(int(n) for n in shape)
            values.extend(float(v) for v in x)
        elif isinstance(x, (int, float)):
            shape = ()
            values.append(float(x))
        elif isinstance(x, (list, tuple)):
            shape = _nested_extents(x)
            if 0 not in shape:
                _pour(x, shape, 0, values)
        else:
            raise TypeError("Tensor expects a scalar or nested Python lists")
        self._adopt(shape, values)

    def _adopt(self, shape, values):
        self.shape = shape
        self._values = values
        self._extents = _Extents(shape)

    @classmethod
    def _copied_from(cls, raw):
        """A Tensor holding a copy of one runtime-owned output (the caller frees the original)."""
        count = int(raw.len)
        values = array.array("f", bytes(4 * count))
        if count:
            ctypes.memmove(values.buffer_info()[0], raw.data, 4 * count)
        made = cls.__new__(cls)
        made._adopt(tuple(int(raw.shape[n]) for n in range(raw.rank)), values)
        return made

    @property
    def data(self):
        return self._values.tolist()

    def numpy(self):
        import numpy as np
        return np.array(self._values, dtype=np.float32).reshape(self.shape)

    def _view(self):
        # An empty tensor still hands over a valid address.
        backing = self._values if len(self._values) else _EMPTY
        return self._extents.describe(backing.buffer_info()[0])

    def __repr__(self):
        return "Tensor(shape=%s, data=%s)" % (self.shape, self.data)


def _is_torch(x):
    return hasattr(x, "data_ptr") and hasattr(x, "shape") and hasattr(x, "device")


def _on_cuda(x):
    return _is_torch(x) and x.device.type == "cuda"


class _Arguments:
    """The ITensor array for a call, the Python objects that must outlive it, and where each
    argument lives."""

    def __init__(self, values, writable):
        self.keep = []
        self.cuda = []
        described = [self._describe(v, writable) for v in values]
        self.count = len(described)
        self.array = (_CTensor * (self.count or 1))(*described)

    def _describe(self, x, writable):
        import numpy as np
        if isinstance(x, np.generic) and not writable:
            x = np.asarray(x, dtype=np.float32)                 # a NumPy scalar is a rank-0 tensor
        if isinstance(x, np.ndarray):
            if x.dtype != np.float32 or not x.flags.c_contiguous:
                if writable:
                    raise TypeError("NumPy outputs must be float32 and C-contiguous")
                x = np.ascontiguousarray(x, dtype=np.float32)
            return self._borrow(x, x.shape, x.ctypes.data, False)
        if _is_torch(x):
            if str(x.dtype) != "torch.float32":
                raise TypeError("Torch tensors must be float32")
            if not x.is_contiguous():
                if writable:
                    raise TypeError("Torch outputs must be contiguous")
                x = x.contiguous()
            return self._borrow(x, tuple(x.shape), x.data_ptr(), x.device.type == "cuda")
        if writable:
            raise TypeError("outputs must be NumPy arrays or Torch tensors")
        if not isinstance(x, Tensor):
            x = Tensor(x)
        self.keep.append(x)
        self.cuda.append(False)
        return x._view()

    def _borrow(self, owner, shape, address, on_cuda):
        extents = _Extents(shape)
        self.keep.append((owner, extents))
        self.cuda.append(on_cuda)
        return extents.describe(address)


def _release(pointer, program_box):
    """Finaliser of a Component: frees the compiled program, then the component."""
    if _core is None:                      # interpreter shutdown: the library is already gone
        return
    if program_box[0]:
        _core.i_program_free(program_box[0])
        program_box[0] = None
    _core.i_component_free(pointer)


def _combinator(symbol, doc):
    def combine(self, other):
        if not isinstance(other, Component):
            other = Component(other)
        return Component(_ptr=getattr(_core, symbol)(self._ptr, other._ptr))
    combine.__name__ = symbol[2:]
    combine.__doc__ = doc
    return combine


class Component:
    """An `i` component: parsed source, or a combination of components.  Compiled on first use."""

    def __init__(self, src=None, _ptr=None):
        if _ptr is None:
            if src is None:
                raise TypeError("Component needs source")
            _ptr = _core.i_parse(src.encode())
        self._ptr = _handle(_ptr)
        self._compiled = [None]            # boxed so the finaliser sees a later compilation
        self._precision = None
        weakref.finalize(self, _release, self._ptr, self._compiled)

    chain = _combinator("i_chain", "self >> other: other consumes this component's outputs.")
    compose = _combinator("i_compose", "self << other: this component consumes other's outputs.")
    fanout = _combinator("i_fanout", "self & other: both read the same inputs.")
    pair = _combinator("i_pair", "self | other: side by side, each on its own inputs.")
    __rshift__, __lshift__, __and__, __or__ = chain, compose, fanout, pair

    def swap(self):
        return Component(_ptr=_core.i_swap(self._ptr))

    __invert__ = swap

    @property
    def _program(self):
        return self._compiled[0]

    def _compile(self):
        if self._compiled[0] is None:
            self._compiled[0] = _handle(_core.i_compile(self._ptr))
            self._apply_precision()
        return self._compiled[0]

    def _apply_precision(self):
        if self._precision is not None and self._compiled[0] is not None:
            _ok(_core.i_b200_program_set_precision(self._compiled[0], self._precision))

    def set_precision(self, name):
        """Arithmetic of this component's contractions: one of PRECISIONS."""
        self._precision = PRECISIONS[name]
        self._apply_precision()
        return self

    def _code(self):
        text = _handle(_core.i_code(self._ptr))
        try:
            return ctypes.string_at(text).decode()
        finally:
            _core.i_string_free(text)

    def output_shapes(self, *inputs):
        program = self._compile()
        given = _Arguments(inputs, writable=False)
        count = int(_core.i_output_count(program))
        ranks = (_SIZE * (count or 1))()
        _ok(_core.i_output_ranks(program, ranks))
        # One flat buffer of extents; output n starts at the sum of the ranks before it.
        starts = [sum(ranks[:n]) for n in range(count)]
        flat = (_SIZE * (sum(ranks[:count]) + 1))()
        width = ctypes.sizeof(_SIZE)
        rows = (_SIZE_P * (count or 1))(*(
            ctypes.cast(ctypes.addressof(flat) + width * start, _SIZE_P) for start in starts))
        _ok(_core.i_output_shapes(program, given.array, given.count, rows))
        return [tuple(flat[start:start + ranks[n]]) for n, start in enumerate(starts)]

    def exec(self, *inputs):
        program = self._compile()
        given = _Arguments(inputs, writable=False)
        produced = _core.i_exec(program, given.array, given.count)
        if not produced.count:
            _fail()
        try:
            results = [Tensor._copied_from(produced.tensors[n]) for n in range(produced.count)]
        finally:
            _core.i_outputs_free(produced)
        return results[0] if len(results) == 1 else tuple(results)

    def _run_into_new(self, allocate, inputs):
        outputs = [allocate(shape) for shape in self.output_shapes(*inputs)]
        self.into(outputs, *inputs)
        return outputs[0] if len(outputs) == 1 else tuple(outputs)

    def exec_numpy(self, *inputs):
        import numpy as np
        return self._run_into_new(lambda shape: np.empty(shape, dtype=np.float32), inputs)

    def exec_torch(self, *inputs):
        import torch
        device = next((x.device for x in inputs if _on_cuda(x)), "cpu")
        return self._run_into_new(lambda shape: torch.empty(shape, dtype=torch.float32, device=device),
                                  inputs)

    def into(self, outputs, *inputs):
        """Run into caller-provided outputs.

        With every tensor on one CUDA device the call is asynchronous on torch's
        current stream; otherwise it copies host tensors through the GPU and
        returns when the outputs are complete (reference: ilang.py:346-360).  In
        the mixed case the CUDA tensors among the arguments are used in place, so
        torch's current stream is synchronised first: the runtime's own stream is
        not ordered behind work that is still producing them.
        """
        program = self._compile()
        single = not isinstance(outputs, (tuple, list))
        if single:
            outputs = (outputs,)
        given = _Arguments(inputs, writable=False)
        wanted = _Arguments(outputs, writable=True)
        where = given.cuda + wanted.cuda
        if where and all(where):
            import torch
            device = next(x for x in (*inputs, *outputs) if _on_cuda(x)).device
            with torch.cuda.device(device):
                stream = torch.cuda.current_stream().cuda_stream
                _ok(_core.i_b200_exec_into(program, given.array, given.count, wanted.array,
                                           wanted.count, ctypes.c_void_p(stream)))
        else:
            if any(where):
                import torch
                for x in (*inputs, *outputs):
                    if _on_cuda(x):
                        torch.cuda.current_stream(x.device).synchronize()
            _ok(_core.i_exec_into(program, given.array, given.count, wanted.array, wanted.count))
        return outputs[0] if len(outputs) == 1 else tuple(outputs)


I = Component(_ptr=_core.i_identity())


def i(src):
    return Component(src)
