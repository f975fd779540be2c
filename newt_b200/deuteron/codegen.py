"""Tile DSL -> newt kernel, in two steps with a small intermediate form between them.

A `@dt.kernel` function is *read* (its Python syntax tree, never executed) into a `Program`:
axes -- iteration dimensions cut into tiles -- and a list of statements over values that know
their rank and, per dimension, which axis pads them.  The program is then *built* into the
syntax tree of one `@newt.jit` kernel in which every tile size is a constexpr, so one kernel
serves every configuration the autotuner tries.  The jit takes that tree as it is
(`JITFunction.from_ast`); `Kernel.to_newt_source` prints it.

What the reference's compiler does with text (deuteron/codegen.py:51-484: one visitor that
prints newt source, with the mask of padded lanes carried along as a string) is done here on
structure: a value's mask is derived from its axes when it is needed, which is where a
reduction wraps its operand in `nl.where(mask, x, identity)` (reference :382-410) and where
`mean()` counts its valid lanes.  The printed kernel keeps the reference's shape
(deuteron/codegen.py:453-484), since users read it:

    signature   <t>_ptr, <t>_d0.., <t>_s0.., scalars, BLOCK_<AXIS>: nl.constexpr
    grid axes   pid_i = nl.program_id(i); offs_<a> = pid_i * BLOCK + nl.arange(0, BLOCK)
    loop axes   for _i_<a> in range(0, nl.cdiv(extent, BLOCK)): offs_<a> = _i_<a> * BLOCK + arange
    loads       nl.load(ptr + offs_a[:, None] * s0 + offs_b[None, :] * s1, mask=..., other=0.0)
    acc += a @ b   ->   acc = nl.dot(a, b, acc)
"""

import ast
from dataclasses import dataclass, field

from . import language as dl


class TraceError(Exception):
    """A `@dt.kernel` function uses something the tile language does not have."""


# --------------------------------------------------------------------------- intermediate form

@dataclass(frozen=True)
class Axis:
    """An iteration dimension cut into tiles of BLOCK_<VAR> elements."""
    var: str         # the tile variable of the kernel function ("full<k>" for a ':' index)
    extent: str      # runtime symbol of the dimension's length, e.g. "x_d1"
    role: str        # "grid" | "loop" | "whole"

    @property
    def block(self):
        return f"BLOCK_{self.var.upper()}"

    @property
    def offs(self):
        return f"offs_{self.var}"

    @property
    def mask(self):
        return f"mask_{self.var}"

    # what the launcher reads (runtime.py)
    @property
    def size(self):
        return self.extent

    @property
    def kind(self):
        return "full" if self.role == "whole" else self.role


@dataclass
class Val:
    """A value of the kernel body: `tree` computes it, `pads[d]` is the axis whose padding
    lanes dimension d carries (None: the dimension has none)."""
    tree: ast.expr
    pads: tuple = ()

    @property
    def rank(self):
        return len(self.pads)


@dataclass
class Program:
    name: str
    tensors: dict                 # name -> rank, in parameter order
    scalars: list
    axes: list                    # tile variables first, whole-dimension axes after them
    grid: list
    body: list                    # ast statements of the generated kernel
    stored: set = field(default_factory=set)


@dataclass
class KernelSource:
    name: str
    fndef: ast.FunctionDef
    source: str
    params: list                      # ("tensor" | "scalar", python name), launch order
    tile_vars: list
    grid_tiles: list
    tunable: list                     # constexpr names the autotuner may vary
    store_params: set = field(default_factory=set)
    has_dot: bool = False


# --------------------------------------------------------------------------- syntax-tree helpers

def _name(ident):
    return ast.Name(id=ident, ctx=ast.Load())


def _const(value):
    return ast.Constant(value=value)


def _nl(fn, *args, **kwargs):
    return ast.Call(func=ast.Attribute(value=_name("nl"), attr=fn, ctx=ast.Load()), args=list(args),
                    keywords=[ast.keyword(arg=k, value=v) for k, v in kwargs.items()])


def _binary(op, left, right):
    return ast.BinOp(left=left, op=op(), right=right)


def _index(base, items):
    """base[items...] where an item is ':' (a full slice) or None (a new axis)."""
    elts = [ast.Slice() if it == ":" else _const(None) for it in items]
    return ast.Subscript(value=base, slice=elts[0] if len(elts) == 1 else ast.Tuple(elts=elts, ctx=ast.Load()),
                         ctx=ast.Load())


def _along(vector, dim, rank):
    """A rank-1 value laid along dimension `dim` of a rank-`rank` block."""
    if rank == 1:
        return vector
    return _index(vector, [":" if d == dim else None for d in range(rank)])


def _assign(target, value):
    return ast.Assign(targets=[ast.Name(id=target, ctx=ast.Store())], value=value)


def _and_all(terms):
    out = terms[0]
    for t in terms[1:]:
        out = _binary(ast.BitAnd, out, t)
    return out


def mask_of(val):
    """Tree of the boolean block that is true on the lanes of `val` that hold data, or None
    when no dimension of it is padded."""
    terms = [_along(_name(ax.mask), d, val.rank) for d, ax in enumerate(val.pads) if ax is not None]
    return _and_all(terms) if terms else None


def _broadcast_pads(*vals):
    """numpy broadcasting on the padding axes: dimensions align from the right and a padded
    dimension wins over an unpadded one."""
    rank = max((v.rank for v in vals), default=0)
    pads = [None] * rank
    for v in vals:
        for d, ax in enumerate(v.pads):
            at = rank - v.rank + d
            if pads[at] is None:
                pads[at] = ax
    return tuple(pads)


_ARITHMETIC = {ast.Add: ast.Add, ast.Sub: ast.Sub, ast.Mult: ast.Mult, ast.Div: ast.Div,
               ast.FloorDiv: ast.FloorDiv, ast.Mod: ast.Mod, ast.Pow: ast.Pow}
_IN_PLACE = {ast.Add, ast.Sub, ast.Mult, ast.Div}
_COMPARISONS = (ast.Eq, ast.NotEq, ast.Lt, ast.LtE, ast.Gt, ast.GtE)


# --------------------------------------------------------------------------- reading the function

class _Reader:
    """Walks the kernel function once, top to bottom, and leaves the generated statements in
    `self.body` (a stack of statement lists follows the nesting of tile loops)."""

    def __init__(self, fn, fndef, tensors, scalars, dtypes):
        self.fn, self.fndef = fn, fndef
        self.tensors, self.scalars, self.dtypes = tensors, scalars, dtypes
        self.by_var = {}          # tile variable -> Axis
        self.whole = {}           # extent symbol -> Axis of a ':' index
        self.grid = []
        self.locals = {}          # name -> pads of the value it holds
        self.stored = set()
        self.body = []
        self.has_dot = False
        self._into = [self.body]

    # ---- diagnostics -----------------------------------------------------------------

    def reject(self, node, why):
        where = getattr(node, "lineno", None)
        at = f" (line {where} of the kernel)" if where is not None else ""
        raise TraceError(f"@dt.kernel {self.fndef.name}{at}: {why}")

    def emit(self, stmt):
        self._into[-1].append(stmt)

    # ---- names of the tile language ---------------------------------------------------------

    def dt_member(self, func):
        """The attribute name if `func` is `<deuteron module>.<name>`, else None."""
        if isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name):
            owner = self.fn.__globals__.get(func.value.id)
            module = getattr(owner, "__name__", "")
            if module.endswith("deuteron") or module.endswith("deuteron.language"):
                return func.attr
        return None

    def shape_entry(self, node):
        """`t.shape[i]` of a tensor parameter -> "t_d<i>", else None."""
        if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Attribute) \
                and node.value.attr == "shape" and isinstance(node.value.value, ast.Name) \
                and node.value.value.id in self.tensors:
            if not (isinstance(node.slice, ast.Constant) and isinstance(node.slice.value, int)):
                self.reject(node, "a shape is indexed with an integer literal")
            return f"{node.value.value.id}_d{node.slice.value}"
        return None

    def extent_symbol(self, node):
        sym = self.shape_entry(node)
        if sym is not None:
            return sym
        if isinstance(node, ast.Constant) and isinstance(node.value, int):
            return str(node.value)
        if isinstance(node, ast.Name) and node.id in self.scalars:
            return node.id
        self.reject(node, "a tiled extent is `tensor.shape[i]`, an integer literal or a scalar "
                          "parameter of the kernel")

    # ---- tile loops ----------------------------------------------------------------------------

    def tile_loop(self, node):
        call = node.iter
        if node.orelse or not (isinstance(call, ast.Call) and self.dt_member(call.func) == "tile"):
            self.reject(node, "loops of a kernel run over `dt.tile(...)` and have no else branch")
        if len(call.args) != 1 or call.keywords:
            self.reject(node, "dt.tile takes exactly one argument: an extent or a list of extents")
        arg = call.args[0]
        extents = [self.extent_symbol(e)
                   for e in (arg.elts if isinstance(arg, (ast.List, ast.Tuple)) else [arg])]
        targets = node.target.elts if isinstance(node.target, ast.Tuple) else [node.target]
        if len(targets) != len(extents) or not all(isinstance(t, ast.Name) for t in targets):
            self.reject(node, f"dt.tile yields {len(extents)} tile(s): bind each to a plain name")
        if not self.grid:
            return self.grid_loop(node, [t.id for t in targets], extents)
        if len(targets) != 1:
            self.reject(node, "only the outermost tile loop may cut several dimensions at once "
                              "(it becomes the launch grid); nest the inner ones")
        axis = Axis(targets[0].id, extents[0], "loop")
        self.by_var[axis.var] = axis
        counter = f"_i_{axis.var}"
        loop = ast.For(target=ast.Name(id=counter, ctx=ast.Store()),
                       iter=ast.Call(func=_name("range"),
                                     args=[_const(0), _nl("cdiv", self.symbol(axis.extent), _name(axis.block))],
                                     keywords=[]),
                       body=[], orelse=[])
        self.emit(loop)
        self._into.append(loop.body)
        self.axis_setup(axis, _name(counter))
        for stmt in node.body:
            self.statement(stmt)
        self._into.pop()

    def grid_loop(self, node, names, extents):
        if len(names) > 3:
            self.reject(node, "a launch grid has at most three dimensions")
        for i, (var, extent) in enumerate(zip(names, extents)):
            axis = Axis(var, extent, "grid")
            self.by_var[var] = axis
            self.grid.append(axis)
            self.emit(_assign(f"pid_{i}", _nl("program_id", _const(i))))
            self.axis_setup(axis, _name(f"pid_{i}"))
        for stmt in node.body:
            self.statement(stmt)

    def axis_setup(self, axis, position):
        """offs_<a> = position * BLOCK + arange(0, BLOCK);  mask_<a> = offs_<a> < extent"""
        lanes = _nl("arange", _const(0), _name(axis.block))
        offs = lanes if position is None else \
            _binary(ast.Add, _binary(ast.Mult, position, _name(axis.block)), lanes)
        self.emit(_assign(axis.offs, offs))
        self.emit(_assign(axis.mask, ast.Compare(left=_name(axis.offs), ops=[ast.Lt()],
                                                 comparators=[self.symbol(axis.extent)])))

    @staticmethod
    def symbol(text):
        return _const(int(text)) if text.lstrip("-").isdigit() else _name(text)

    # ---- statements --------------------------------------------------------------------------------

    def statement(self, stmt):
        if isinstance(stmt, ast.For):
            return self.tile_loop(stmt)
        if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant):
            return None                                   # a docstring or a stray literal
        if isinstance(stmt, ast.Assign) and len(stmt.targets) == 1:
            target = stmt.targets[0]
            value = self.value(stmt.value)
            if isinstance(target, ast.Name):
                self.locals[target.id] = value.pads
                return self.emit(_assign(target.id, value.tree))
            if isinstance(target, ast.Subscript):
                return self.write(stmt, target, value)
        if isinstance(stmt, ast.AugAssign) and isinstance(stmt.target, ast.Name):
            return self.update(stmt)
        self.reject(stmt, f"`{type(stmt).__name__}` statements are not part of the tile language "
                          f"(there are tile loops, `name = value`, `name op= value` and "
                          f"`tensor[tiles] = value`)")

    def update(self, stmt):
        name = stmt.target.id
        if name not in self.locals:
            self.reject(stmt, f"`{name}` is updated in place before it has been given a value")
        rhs = stmt.value
        if isinstance(stmt.op, ast.Add) and isinstance(rhs, ast.BinOp) and isinstance(rhs.op, ast.MatMult):
            a, b = self.value(rhs.left), self.value(rhs.right)    # acc += a @ b: one fused dot
            self.has_dot = True
            self.locals[name] = (None, None)
            return self.emit(_assign(name, _nl("dot", a.tree, b.tree, _name(name))))
        if type(stmt.op) not in _IN_PLACE:
            self.reject(stmt, "in-place updates are `+=`, `-=`, `*=` and `/=`")
        value = self.value(rhs)
        self.locals[name] = _broadcast_pads(Val(_name(name), self.locals[name]), value)
        self.emit(_assign(name, _binary(type(stmt.op), _name(name), value.tree)))

    # ---- tensors -----------------------------------------------------------------------------------------

    def element_axes(self, node, sub):
        """The axes that index tensor `sub.value` in `t[a, b]`, one per dimension."""
        tensor = sub.value.id
        rank = self.tensors[tensor]
        picks = sub.slice.elts if isinstance(sub.slice, ast.Tuple) else [sub.slice]
        if len(picks) != rank:
            self.reject(node, f"`{tensor}` has {rank} dimension(s), {len(picks)} index(es) given")
        if rank not in (1, 2):
            self.reject(node, "tensors are read and written as 1-D or 2-D tiles")
        axes = []
        for d, pick in enumerate(picks):
            if isinstance(pick, ast.Name) and pick.id in self.by_var:
                axes.append(self.by_var[pick.id])
            elif isinstance(pick, ast.Slice) and pick.lower is None and pick.upper is None and pick.step is None:
                extent = f"{tensor}_d{d}"
                if extent not in self.whole:       # one whole-dimension axis per distinct extent
                    self.whole[extent] = Axis(f"full{len(self.whole)}", extent, "whole")
                axes.append(self.whole[extent])
            else:
                self.reject(node, "a tensor is indexed by tile variables and `:` only")
        return tensor, tuple(axes)

    @staticmethod
    def address(tensor, axes):
        tree = _name(f"{tensor}_ptr")
        for d, axis in enumerate(axes):
            tree = _binary(ast.Add, tree, _binary(ast.Mult, _along(_name(axis.offs), d, len(axes)),
                                                  _name(f"{tensor}_s{d}")))
        return tree

    def read(self, node):
        import torch

        tensor, axes = self.element_axes(node, node)
        val = Val(None, axes)
        zero = 0 if self.dtypes[tensor] in (torch.int32, torch.int64) else 0.0
        val.tree = _nl("load", self.address(tensor, axes), mask=mask_of(val), other=_const(zero))
        return val

    def write(self, node, target, value):
        if not (isinstance(target.value, ast.Name) and target.value.id in self.tensors):
            self.reject(node, "only tensor parameters of the kernel can be written")
        tensor, axes = self.element_axes(node, target)
        self.stored.add(tensor)
        self.emit(ast.Expr(value=_nl("store", self.address(tensor, axes), value.tree,
                                     mask=mask_of(Val(None, axes)))))

    # ---- values ------------------------------------------------------------------------------------------------

    def value(self, node):
        if isinstance(node, ast.Constant):
            return Val(_const(node.value))
        if isinstance(node, ast.Name):
            if node.id in self.locals:
                return Val(_name(node.id), self.locals[node.id])
            if node.id in self.scalars:
                return Val(_name(node.id))
            if node.id in self.by_var:
                self.reject(node, f"`{node.id}` is a tile: it can index a tensor or size a block, "
                                  f"it has no value of its own")
            self.reject(node, f"`{node.id}` has not been given a value")
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
            inner = self.value(node.operand)
            return Val(ast.UnaryOp(op=ast.USub(), operand=inner.tree), inner.pads)
        if isinstance(node, ast.BinOp):
            left, right = self.value(node.left), self.value(node.right)
            if isinstance(node.op, ast.MatMult):
                self.has_dot = True
                return Val(_nl("dot", left.tree, right.tree), (None, None))
            if type(node.op) not in _ARITHMETIC:
                self.reject(node, f"operator `{type(node.op).__name__}` is not part of the tile language")
            return Val(_binary(type(node.op), left.tree, right.tree), _broadcast_pads(left, right))
        if isinstance(node, ast.Compare):
            if len(node.ops) != 1 or not isinstance(node.ops[0], _COMPARISONS):
                self.reject(node, "comparisons take two operands and one of == != < <= > >=")
            left, right = self.value(node.left), self.value(node.comparators[0])
            return Val(ast.Compare(left=left.tree, ops=[type(node.ops[0])()], comparators=[right.tree]),
                       _broadcast_pads(left, right))
        if isinstance(node, ast.Subscript):
            return self.subscript(node)
        if isinstance(node, ast.Call):
            return self.call(node)
        self.reject(node, f"`{type(node).__name__}` expressions are not part of the tile language")

    def subscript(self, node):
        if isinstance(node.value, ast.Name) and node.value.id in self.tensors:
            return self.read(node)
        sym = self.shape_entry(node)
        if sym is not None:
            return Val(_name(sym))
        base = self.value(node.value)
        picks = node.slice.elts if isinstance(node.slice, ast.Tuple) else [node.slice]
        items, pads, taken = [], [], 0
        for pick in picks:
            if isinstance(pick, ast.Constant) and pick.value is None:
                items.append(None)
                pads.append(None)
            elif isinstance(pick, ast.Slice) and pick.lower is None and pick.upper is None and pick.step is None:
                if taken >= base.rank:
                    self.reject(node, "more `:` than the value has dimensions")
                items.append(":")
                pads.append(base.pads[taken])
                taken += 1
            else:
                self.reject(node, "a computed value is only ever reshaped with `:` and `None`")
        pads.extend(base.pads[taken:])
        return Val(_index(base.tree, items), tuple(pads))

    def call(self, node):
        func = node.func
        member = self.dt_member(func)
        if member in ("zeros", "full"):
            return self.block_of_constants(node, member)
        if member is not None:
            if member not in dl.ELEMENTWISE:
                self.reject(node, f"dt.{member} has no compiled form")
            fn, extra = dl.ELEMENTWISE[member]
            args = [self.value(a) for a in node.args]
            return Val(_nl(fn, *[a.tree for a in args], *[_const(c) for c in extra]),
                       _broadcast_pads(*args))
        if isinstance(func, ast.Name) and func.id in ("float", "int") and len(node.args) == 1 \
                and isinstance(node.args[0], ast.Constant):
            return Val(ast.Call(func=_name(func.id), args=[_const(node.args[0].value)], keywords=[]))
        if isinstance(func, ast.Attribute):
            base = self.value(func.value)
            if func.attr in dl.REDUCTIONS:
                return self.reduce(node, base, func.attr)
            if func.attr == "mean":
                return self.mean(node, base)
            if func.attr == "to":
                self.reject(node, "there is no `.to()`: a store converts to the tensor's type, and "
                                  "dt.zeros / dt.full take a dtype")
        self.reject(node, "this call is not part of the tile language")

    def block_of_constants(self, node, which):
        if not node.args:
            self.reject(node, f"dt.{which} needs a shape")
        shape = node.args[0]
        dims = []
        for entry in (shape.elts if isinstance(shape, (ast.List, ast.Tuple)) else [shape]):
            if isinstance(entry, ast.Name) and entry.id in self.by_var:
                dims.append(_name(self.by_var[entry.id].block))
            elif isinstance(entry, ast.Constant) and isinstance(entry.value, int):
                dims.append(_const(entry.value))
            else:
                self.reject(node, f"the shape of dt.{which} is made of tile variables and integer literals")
        dtype = "float32"
        for kw in node.keywords:
            if kw.arg == "dtype":
                try:
                    chosen = eval(compile(ast.Expression(kw.value), "<dtype>", "eval"),  # noqa: S307
                                  self.fn.__globals__)
                except Exception:  # noqa: BLE001
                    chosen = None
                if chosen not in dl.DTYPE_NAMES:
                    self.reject(node, "dtype must be one of dt.float32/float16/bfloat16/int32/int64")
                dtype = dl.DTYPE_NAMES[chosen]
        shape_tree = ast.Tuple(elts=dims, ctx=ast.Load())
        dtype_tree = ast.Attribute(value=_name("nl"), attr=dtype, ctx=ast.Load())
        pads = (None,) * len(dims)
        if which == "zeros":
            return Val(_nl("zeros", shape_tree, dtype=dtype_tree), pads)
        if len(node.args) < 2:
            self.reject(node, "dt.full needs a fill value")
        return Val(_nl("full", shape_tree, self.value(node.args[1]).tree, dtype=dtype_tree), pads)

    # ---- reductions --------------------------------------------------------------------------------------------------

    def reduction_axis(self, node, base):
        axis = None
        if node.args and isinstance(node.args[0], ast.Constant):
            axis = node.args[0].value
        for kw in node.keywords:
            if kw.arg in ("axis", "dim") and isinstance(kw.value, ast.Constant):
                axis = kw.value.value
        if axis is None:
            return None, ()
        if axis < 0:
            axis += base.rank
        if not 0 <= axis < max(base.rank, 1):
            self.reject(node, f"axis {axis} of a value with {base.rank} dimension(s)")
        return axis, tuple(p for d, p in enumerate(base.pads) if d != axis)

    def reduce(self, node, base, method):
        """Padding lanes must not take part: they are replaced by the reduction's identity."""
        fn, identity = dl.REDUCTIONS[method]
        axis, pads = self.reduction_axis(node, base)
        mask = mask_of(base)
        operand = base.tree if mask is None else _nl("where", mask, base.tree, _identity(identity))
        kwargs = {} if axis is None else {"axis": _const(axis)}
        return Val(_nl(fn, operand, **kwargs), pads)

    def mean(self, node, base):
        """Sum over the valid lanes divided by their number (the reference has no mean(),
        deuteron/codegen.py:412-413)."""
        axis, pads = self.reduction_axis(node, base)
        kwargs = {} if axis is None else {"axis": _const(axis)}
        mask = mask_of(base)
        shape_of = ast.Attribute(value=base.tree, attr="shape", ctx=ast.Load())
        if mask is not None:
            total = _nl("sum", _nl("where", mask, base.tree, _const(0.0)), **kwargs)
            ones = _nl("broadcast_to", _nl("where", mask, _const(1.0), _const(0.0)), shape_of)
            count = _nl("sum", ones, **kwargs)
        else:
            if base.rank == 0:
                self.reject(node, "mean() of a value that is not a block")
            total = _nl("sum", base.tree, **kwargs)
            dims = range(base.rank) if axis is None else [axis]
            count = None
            for d in dims:
                extent = ast.Subscript(value=shape_of, slice=_const(d), ctx=ast.Load())
                count = extent if count is None else _binary(ast.Mult, count, extent)
        return Val(_binary(ast.Div, total, count), pads)


def _identity(value):
    """0.0, or float('-inf') / float('inf') spelled as the call the jit front end folds."""
    if value in (float("inf"), float("-inf")):
        return ast.Call(func=_name("float"), args=[_const("-inf" if value < 0 else "inf")], keywords=[])
    return _const(value)


# --------------------------------------------------------------------------- entry point

def read_program(fn, fndef, args):
    import torch

    names = [a.arg for a in fndef.args.args]
    if len(names) != len(args):
        raise TraceError(f"@dt.kernel {fndef.name}: takes {len(names)} argument(s), {len(args)} given")
    tensors, scalars, dtypes = {}, [], {}
    for name, arg in zip(names, args):
        if torch.is_tensor(arg):
            tensors[name], dtypes[name] = arg.dim(), arg.dtype
        elif isinstance(arg, (int, float)) and not isinstance(arg, bool):
            scalars.append(name)
        else:
            raise TraceError(f"@dt.kernel {fndef.name}: argument `{name}` is a {type(arg).__name__}; "
                             f"kernels take tensors and int / float scalars")
    reader = _Reader(fn, fndef, tensors, scalars, dtypes)
    for stmt in fndef.body:
        if isinstance(stmt, ast.Expr) and isinstance(stmt.value, ast.Constant):
            continue
        if not isinstance(stmt, ast.For):
            reader.reject(stmt, "the top level of a kernel holds tile loops only "
                                "(`for ... in dt.tile(...)`)")
        reader.tile_loop(stmt)
    # whole-dimension axes are the same for every program: set up ahead of the body
    setup = _Reader(fn, fndef, tensors, scalars, dtypes)
    for axis in reader.whole.values():
        setup.axis_setup(axis, None)
    program = Program(f"{fndef.name}_newt", tensors, scalars,
                      list(reader.by_var.values()) + list(reader.whole.values()), reader.grid,
                      setup.body + reader.body, reader.stored)
    return program, reader


def build_kernel(program):
    """The `ast.FunctionDef` of the newt kernel; statements are numbered the way
    `ast.unparse` lays them out, so diagnostics of the jit front end point into the printed text."""
    params = []
    for tensor, rank in program.tensors.items():
        params.append(ast.arg(arg=f"{tensor}_ptr"))
        params += [ast.arg(arg=f"{tensor}_d{d}") for d in range(rank)]
        params += [ast.arg(arg=f"{tensor}_s{d}") for d in range(rank)]
    params += [ast.arg(arg=s) for s in program.scalars]
    constexpr = ast.Attribute(value=_name("nl"), attr="constexpr", ctx=ast.Load())
    params += [ast.arg(arg=axis.block, annotation=constexpr) for axis in program.axes]
    fndef = ast.FunctionDef(
        name=program.name,
        args=ast.arguments(posonlyargs=[], args=params, kwonlyargs=[], kw_defaults=[], defaults=[]),
        body=program.body or [ast.Pass()], decorator_list=[], type_params=[])
    ast.fix_missing_locations(fndef)
    line = [_HEADER_LINES + 1]       # the `def` line: after the header and the decorator

    def number(stmts):
        for stmt in stmts:
            line[0] += 1
            for node in ast.walk(stmt):
                if not isinstance(node, ast.stmt) or node is stmt:
                    node.lineno = node.end_lineno = line[0]
            if isinstance(stmt, ast.For):
                number(stmt.body)

    fndef.lineno = line[0]
    number(fndef.body)
    return fndef


_HEADER_LINES = 4     # two imports, a blank line, the decorator


def generate(fn, fndef, args, newt_module="newt_b200"):
    """Reads `fn` for these example arguments and returns its KernelSource."""
    program, reader = read_program(fn, fndef, args)
    kernel = build_kernel(program)
    text = (f"import {newt_module} as newt\nimport {newt_module}.language as nl\n\n"
            f"@newt.jit\n{ast.unparse(kernel)}\n")
    params = [("tensor", t) for t in program.tensors] + [("scalar", s) for s in program.scalars]
    return KernelSource(program.name, kernel, text, params, program.axes, program.grid,
                        [axis.block for axis in reader.by_var.values()], program.stored,
                        reader.has_dot)
