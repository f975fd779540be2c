"""The tile language (`import newt_b200.deuteron as dt`), after deuteron/language.py.

Every function here has an eager implementation on torch tensors: calling a
`@dt.kernel` function with full-size tiles runs it as plain PyTorch.  That eager
run is the oracle candidate configurations are checked against
(deuteron/runtime.py:226-231 of the reference) and is exposed as `Kernel.ref`.

One deliberate difference: the reference allocates `dt.zeros` / `dt.full` on a
hard-coded "cuda" device (deuteron/language.py:83-90), which makes `.ref`
unusable on host tensors for any kernel with an accumulator.  Here the eager
allocators follow the device of the tensors the kernel was called with.
"""

import contextlib
import threading

import torch

float32 = torch.float32
float16 = torch.float16
bfloat16 = torch.bfloat16
int32 = torch.int32
int64 = torch.int64

_eager = threading.local()


@contextlib.contextmanager
def eager_device(device):
    """Device that dt.zeros / dt.full allocate on during an eager run."""
    prev = getattr(_eager, "device", None)
    _eager.device = device
    try:
        yield
    finally:
        _eager.device = prev


def _alloc_device():
    dev = getattr(_eager, "device", None)
    if dev is not None:
        return dev
    return torch.device("cuda") if torch.cuda.is_available() else torch.device("cpu")


class Tile:
    """One tile of an iteration dimension.  Eagerly it spans the whole
    dimension; compiled it is a BLOCK_<NAME> constexpr with offsets and a mask."""

    def __init__(self, size, name=None):
        self.size = int(size)
        self.name = name

    def as_slice(self):
        return slice(0, self.size)

    def __repr__(self):
        return f"Tile({self.name or '?'}, {self.size})"


def _index(idx):
    idx = idx if isinstance(idx, tuple) else (idx,)
    return tuple(i.as_slice() if isinstance(i, Tile) else i for i in idx)


class EagerTensor:
    """Tensor argument as the eager run sees it: Tile indices act as full slices,
    loads give plain tensors, stores write through."""

    def __init__(self, tensor):
        self._t = tensor

    def __getitem__(self, idx):
        return self._t[_index(idx)]

    def __setitem__(self, idx, value):
        self._t[_index(idx)] = value

    @property
    def shape(self):
        return self._t.shape

    @property
    def dtype(self):
        return self._t.dtype

    @property
    def device(self):
        return self._t.device

    def size(self, dim=None):
        return self._t.size() if dim is None else self._t.size(dim)


def tile(sizes):
    """`for t in dt.tile(n)` / `for tm, tn in dt.tile([m, n])`.  The outermost tile
    loop of a kernel becomes the launch grid, inner ones become loops over
    tiles; eagerly each yields one full-size tile."""
    if isinstance(sizes, (list, tuple)):
        yield tuple(Tile(s) for s in sizes)
    else:
        yield Tile(sizes)


def _sizes(shape):
    return [s.size if isinstance(s, Tile) else int(s) for s in shape]


def zeros(shape, dtype=torch.float32):
    return torch.zeros(_sizes(shape), dtype=dtype, device=_alloc_device())


def full(shape, value, dtype=torch.float32):
    return torch.full(_sizes(shape), value, dtype=dtype, device=_alloc_device())


exp, log, sqrt, rsqrt = torch.exp, torch.log, torch.sqrt, torch.rsqrt
sigmoid, tanh, erf, abs = torch.sigmoid, torch.tanh, torch.erf, torch.abs
maximum, minimum, where = torch.maximum, torch.minimum, torch.where


def relu(x):
    return torch.clamp_min(x, 0)


# dt.<name>(args...) -> newt expression over the already generated operand texts
ELEMENTWISE = {
    "exp": "nl.exp({0})", "log": "nl.log({0})", "sqrt": "nl.sqrt({0})",
    "rsqrt": "nl.rsqrt({0})", "sigmoid": "nl.sigmoid({0})", "tanh": "nl.tanh({0})",
    "erf": "nl.erf({0})", "abs": "nl.abs({0})", "relu": "nl.maximum({0}, 0.0)",
    "maximum": "nl.maximum({0}, {1})", "minimum": "nl.minimum({0}, {1})",
    "where": "nl.where({0}, {1}, {2})",
}
# tensor method -> (newt reduction, identity that padded lanes must hold)
REDUCTIONS = {
    "sum": ("nl.sum", "0.0"),
    "max": ("nl.max", "float('-inf')"), "amax": ("nl.max", "float('-inf')"),
    "min": ("nl.min", "float('inf')"), "amin": ("nl.min", "float('inf')"),
}
DTYPE_NAMES = {torch.float32: "nl.float32", torch.float16: "nl.float16",
               torch.bfloat16: "nl.bfloat16", torch.int32: "nl.int32", torch.int64: "nl.int64"}
