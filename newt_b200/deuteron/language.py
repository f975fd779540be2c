"""The tile language (`import newt_b200.deuteron as dt`): what a kernel body may call.

Everything here also works on plain torch tensors, which is what makes a `@dt.kernel`
function runnable as ordinary PyTorch: called with tiles that span whole dimensions, the
body computes its result eagerly.  That run is the oracle tile-size candidates are checked
against and is exposed as `Kernel.ref` (the reference does the same,
deuteron/language.py:1-8, deuteron/runtime.py:226-231).

One deliberate difference: the reference allocates `dt.zeros` / `dt.full` on a hard-coded
"cuda" device (deuteron/language.py:83-90), so `.ref` cannot run on host tensors for any
kernel with an accumulator.  Here the eager allocators follow the device of the tensors the
kernel was called with.
"""

import contextlib
import threading
from dataclasses import dataclass

import torch

float32, float16, bfloat16 = torch.float32, torch.float16, torch.bfloat16
int32, int64 = torch.int32, torch.int64

_state = threading.local()


@contextlib.contextmanager
def eager_device(device):
    """While active, dt.zeros / dt.full allocate on `device` (None: no preference)."""
    before = getattr(_state, "device", None)
    _state.device = device
    try:
        yield
    finally:
        _state.device = before


def _where_to_allocate():
    chosen = getattr(_state, "device", None)
    if chosen is None:
        chosen = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    return chosen


@dataclass
class Tile:
    """One tile of an iteration dimension.  In an eager run it is the whole dimension; in the
    compiled kernel it is BLOCK_<NAME> elements, with offsets and a mask for the ragged end."""
    size: int
    name: str = None

    def __post_init__(self):
        self.size = int(self.size)

    def as_slice(self):
        return slice(0, self.size)

    def __repr__(self):
        return f"Tile({self.name or '?'}, {self.size})"


def _as_torch_index(index):
    parts = index if isinstance(index, tuple) else (index,)
    return tuple(part.as_slice() if isinstance(part, Tile) else part for part in parts)


def _extent(entry):
    return entry.size if isinstance(entry, Tile) else int(entry)


class EagerTensor:
    """A tensor argument during an eager run: indexing it with tiles reads or writes the
    spanned region of the real tensor."""

    def __init__(self, tensor):
        self._t = tensor

    def __getitem__(self, index):
        return self._t[_as_torch_index(index)]

    def __setitem__(self, index, value):
        self._t[_as_torch_index(index)] = value

    def __getattr__(self, attribute):          # shape, dtype, device, size(), ...
        return getattr(self._t, attribute)


def tile(extents):
    """`for t in dt.tile(n)` / `for tm, tn in dt.tile([m, n])`.  The outermost tile loop of a
    kernel becomes its launch grid and inner ones loops over tiles; an eager run gets a single
    tile per dimension, as long as the dimension."""
    if isinstance(extents, (list, tuple)):
        yield tuple(Tile(e) for e in extents)
    else:
        yield Tile(extents)


def zeros(shape, dtype=torch.float32):
    return torch.zeros([_extent(e) for e in shape], dtype=dtype, device=_where_to_allocate())


def full(shape, value, dtype=torch.float32):
    return torch.full([_extent(e) for e in shape], value, dtype=dtype, device=_where_to_allocate())


def relu(x):
    return torch.clamp_min(x, 0)


# the rest of the elementwise vocabulary is torch's own
for _fn in ("exp", "log", "sqrt", "rsqrt", "sigmoid", "tanh", "erf", "abs", "maximum", "minimum", "where"):
    globals()[_fn] = getattr(torch, _fn)
del _fn


# dt.<name>(args...) in a compiled kernel -> nl.<function>(args..., *trailing constants)
ELEMENTWISE = {
    "exp": ("exp", ()), "log": ("log", ()), "sqrt": ("sqrt", ()), "rsqrt": ("rsqrt", ()),
    "sigmoid": ("sigmoid", ()), "tanh": ("tanh", ()), "erf": ("erf", ()), "abs": ("abs", ()),
    "relu": ("maximum", (0.0,)),
    "maximum": ("maximum", ()), "minimum": ("minimum", ()), "where": ("where", ()),
}
# tensor method -> (nl reduction, the identity that padding lanes are given)
REDUCTIONS = {
    "sum": ("sum", 0.0),
    "max": ("max", float("-inf")), "amax": ("max", float("-inf")),
    "min": ("min", float("inf")), "amin": ("min", float("inf")),
}
DTYPE_NAMES = {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16",
               torch.int32: "int32", torch.int64: "int64"}
