"""Scalar element types, pointer types and the promotion / broadcasting rules of
the kernel language.

Same surface as the reference's type module (newt/compiler/types.py): dtype
objects named `float32`, `float16`, ...; `pointer_type(elem)` with the
`.element_ty` alias that `ptr.dtype.element_ty` reads (:60-77); `promote`
(:86-99) and `broadcast_shapes` (:102-117) with the same results.
"""

from dataclasses import dataclass


@dataclass(frozen=True)
class dtype:
    name: str        # language-level name, e.g. "float32"
    ctype: str       # CUDA C spelling
    itemsize: int
    kind: str        # 'f' float, 'i' signed, 'u' unsigned, 'b' bool
    rank: int        # position in the promotion lattice (wider / "floatier" = higher)

    @property
    def is_floating(self):
        return self.kind == "f"

    @property
    def is_int(self):
        return self.kind in "iub"

    def __repr__(self):
        return f"nl.{self.name}"


_SPECS = [
    # name        ctype            size kind
    ("int1",     "bool",            1, "b"),
    ("int8",     "signed char",     1, "i"),
    ("uint8",    "unsigned char",   1, "u"),
    ("int16",    "short",           2, "i"),
    ("int32",    "int",             4, "i"),
    ("uint32",   "unsigned int",    4, "u"),
    ("int64",    "long long",       8, "i"),
    ("float16",  "__half",          2, "f"),
    ("bfloat16", "__nv_bfloat16",   2, "f"),
    ("float32",  "float",           4, "f"),
    ("float64",  "double",          8, "f"),
]
ALL_DTYPES = [dtype(n, c, s, k, r) for r, (n, c, s, k) in enumerate(_SPECS)]
BY_NAME = {d.name: d for d in ALL_DTYPES}
globals().update(BY_NAME)

TORCH_TO_NEWT = {"torch.bool": BY_NAME["int1"]}
TORCH_TO_NEWT.update({f"torch.{d.name}": d for d in ALL_DTYPES if d.name != "int1"})


class pointer_type:
    """Type of a kernel argument that is a tensor: pointer to `element`."""

    def __init__(self, element):
        self.element = element
        self.element_ty = element
        self.name = f"pointer<{element.name}>"

    @property
    def ctype(self):
        return self.element.ctype + "*"

    def __eq__(self, other):
        return isinstance(other, pointer_type) and other.element == self.element

    def __hash__(self):
        return hash(("pointer", self.element.name))

    def __repr__(self):
        return self.name


def promote(a, b):
    """Result type of a binary op: floats win over ints, then the wider type;
    float16 with bfloat16 has no winner and goes to float32."""
    if a == b:
        return a
    if a.is_floating != b.is_floating:
        return a if a.is_floating else b
    if {a.name, b.name} == {"float16", "bfloat16"}:
        return BY_NAME["float32"]
    return a if a.rank >= b.rank else b


def broadcast_shapes(s1, s2):
    """NumPy broadcasting on compile-time shapes; () is a scalar."""
    if not s1:
        return tuple(s2)
    if not s2:
        return tuple(s1)
    n = max(len(s1), len(s2))
    a = (1,) * (n - len(s1)) + tuple(s1)
    b = (1,) * (n - len(s2)) + tuple(s2)
    out = []
    for x, y in zip(a, b):
        if x != y and 1 not in (x, y):
            raise TypeError(f"incompatible block shapes {tuple(s1)} and {tuple(s2)}")
        out.append(max(x, y))
    return tuple(out)
