"""The kernel language (`import newt_b200.language as nl`).

Mirrors newt/language.py of the reference: the dtype objects, the `constexpr`
annotation with host-side arithmetic (:23-75) and the device-only builtins
(:95-256).  The builtins carry no behaviour here: inside `@jit` functions the
front end recognises them by the `_newt_builtin` tag and evaluates them
symbolically; called from ordinary Python they raise.
"""

import operator as _op

from .types import (  # noqa: F401
    bfloat16, float16, float32, float64, int1, int8, int16, int32, int64, uint8, uint32,
)


class constexpr:
    """Annotation of compile-time kernel parameters; also a tiny value wrapper
    whose arithmetic works on the host (e.g. in grid lambdas)."""

    def __init__(self, value=None):
        self.value = value

    def __class_getitem__(cls, item):
        return cls

    @staticmethod
    def _raw(x):
        return x.value if isinstance(x, constexpr) else x

    def _bin(self, other, fn, swap=False):
        a, b = self.value, self._raw(other)
        return constexpr(fn(b, a) if swap else fn(a, b))

    def __add__(self, o): return self._bin(o, _op.add)
    def __radd__(self, o): return self._bin(o, _op.add, True)
    def __sub__(self, o): return self._bin(o, _op.sub)
    def __rsub__(self, o): return self._bin(o, _op.sub, True)
    def __mul__(self, o): return self._bin(o, _op.mul)
    def __rmul__(self, o): return self._bin(o, _op.mul, True)
    def __floordiv__(self, o): return self._bin(o, _op.floordiv)
    def __rfloordiv__(self, o): return self._bin(o, _op.floordiv, True)
    def __mod__(self, o): return self._bin(o, _op.mod)
    def __eq__(self, o): return self.value == self._raw(o)
    def __ne__(self, o): return self.value != self._raw(o)
    def __lt__(self, o): return self.value < self._raw(o)
    def __le__(self, o): return self.value <= self._raw(o)
    def __gt__(self, o): return self.value > self._raw(o)
    def __ge__(self, o): return self.value >= self._raw(o)
    def __hash__(self): return hash(self.value)
    def __index__(self): return int(self.value)
    def __int__(self): return int(self.value)
    def __float__(self): return float(self.value)
    def __bool__(self): return bool(self.value)
    def __repr__(self): return f"constexpr[{self.value!r}]"


# name -> (signature shown in help(), one-line description)
_BUILTINS = {
    "program_id": ("(axis)", "Index of this program instance along grid axis 0..2."),
    "num_programs": ("(axis)", "Number of program instances along a grid axis."),
    "arange": ("(start, end)", "1-D int32 block [start, end); the length must be a power of two."),
    "zeros": ("(shape, dtype=float32)", "Block of zeros; every dim a power of two."),
    "full": ("(shape, value, dtype=float32)", "Block filled with a scalar."),
    "load": ("(pointer, mask=None, other=None)", "Load a block; masked-off lanes read `other` (default 0)."),
    "store": ("(pointer, value, mask=None)", "Store a block, casting to the pointee type."),
    "expand_dims": ("(x, axis)", "Insert a size-1 dimension (x[:, None])."),
    "broadcast_to": ("(x, shape)", "Broadcast a block to a larger shape."),
    "reshape": ("(x, shape)", "Row-major reshape with the same element count."),
    "trans": ("(x)", "Transpose a 2-D block."),
    "cast": ("(x, dtype)", "Elementwise cast (x.to(dtype))."),
    "sum": ("(x, axis=None)", "Sum along an axis or over the whole block; 16-bit floats reduce in fp32."),
    "max": ("(x, axis=None)", "Maximum along an axis or over the whole block."),
    "min": ("(x, axis=None)", "Minimum along an axis or over the whole block."),
    "dot": ("(a, b, acc=None, out_dtype=float32)",
            "Block matmul a[M,K] @ b[K,N] -> [M,N] with fp32 accumulation on the tensor cores."),
    "exp": ("(x)", ""), "exp2": ("(x)", ""), "log": ("(x)", ""), "log2": ("(x)", ""),
    "sqrt": ("(x)", ""), "rsqrt": ("(x)", ""), "sin": ("(x)", ""), "cos": ("(x)", ""),
    "tanh": ("(x)", ""), "erf": ("(x)", ""), "sigmoid": ("(x)", ""), "abs": ("(x)", ""),
    "floor": ("(x)", ""), "ceil": ("(x)", ""),
    "maximum": ("(a, b)", ""), "minimum": ("(a, b)", ""),
    "where": ("(cond, a, b)", "Elementwise select."),
    "fma": ("(a, b, c)", "a * b + c, fused."),
    "atomic_add": ("(pointer, value, mask=None)", ""),
    "atomic_max": ("(pointer, value, mask=None)", ""),
    "cdiv": ("(a, b)", "Ceiling division."),
    "multiple_of": ("(x, value)", "Compiler hint; accepted and ignored."),
    "max_contiguous": ("(x, value)", "Compiler hint; accepted and ignored."),
    "static_assert": ("(cond, msg='')", "Compile-time assertion on constexpr values."),
    "static_print": ("(*args)", "Print constexpr values at compile time."),
}


def _make_builtin(name, sig, doc):
    def builtin(*args, **kwargs):
        raise RuntimeError(
            f"nl.{name} can only be called inside a @newt.jit kernel "
            f"(or via the interpreter with NEWT_INTERPRET=1)")

    builtin.__name__ = builtin.__qualname__ = name
    builtin.__doc__ = f"nl.{name}{sig}\n\n{doc}".rstrip()
    builtin._newt_builtin = name
    return builtin


for _name, (_sig, _doc) in _BUILTINS.items():
    globals()[_name] = _make_builtin(_name, _sig, _doc)
del _name, _sig, _doc
