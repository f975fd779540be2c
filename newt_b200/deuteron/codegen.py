"""Tile DSL -> newt kernel text, after deuteron/codegen.py of the reference.

A `@dt.kernel` function is read at the AST level and rewritten into the source
of one `@newt.jit` kernel in which every tile size is a constexpr, so a single
text serves every configuration the autotuner tries.  The shape of that text is
kept as the reference produces it (deuteron/codegen.py:453-484), because users
inspect it through `Kernel.to_newt_source` and because the sm_100a lowering
recognises the matmul K loop in exactly this spelling:

    signature   <t>_ptr, <t>_d0.., <t>_s0.., scalars, BLOCK_<TILE>: nl.constexpr
    grid tiles  pid_i = nl.program_id(i); offs_<t> = pid_i * BLOCK + nl.arange(0, BLOCK)
    inner tiles for _i_<t> in range(0, nl.cdiv(size, BLOCK)): offs_<t> = _i_<t> * BLOCK + arange
    loads       nl.load(ptr + offs_a[:, None] * s0 + offs_b[None, :] * s1, mask=..., other=0.0)
    acc += a @ b   ->   acc = nl.dot(a, b, acc)
    reductions over a padded dimension are wrapped in nl.where(mask, x, identity)
"""

import ast
from dataclasses import dataclass, field

from . import language as dl


class TraceError(Exception):
    pass


@dataclass
class TileVar:
    name: str        # the Python-level tile variable
    size: str        # runtime symbol of the iterated extent, e.g. "x_d1"
    kind: str        # "grid" | "loop" | "full"
    block: str       # constexpr holding the tile size

    @property
    def offs(self):
        return f"offs_{self.name}"

    @property
    def mask(self):
        return f"mask_{self.name}"


@dataclass
class Value:
    """Generated text of an expression, the mask of its padded lanes (if any)
    and its rank."""
    code: str
    mask: str = None
    ndim: int = 0


@dataclass
class KernelSource:
    name: str
    source: str
    params: list                      # ("tensor" | "scalar", python name), launch order
    tile_vars: list
    grid_tiles: list
    tunable: list                     # constexpr names the autotuner may vary
    store_params: set = field(default_factory=set)


_ARITH = {ast.Add: "+", ast.Sub: "-", ast.Mult: "*", ast.Div: "/", ast.FloorDiv: "//",
          ast.Mod: "%", ast.Pow: "**"}
_COMPARE = {ast.Eq: "==", ast.NotEq: "!=", ast.Lt: "<", ast.LtE: "<=", ast.Gt: ">",
            ast.GtE: ">="}


class _Emitter:
    def __init__(self, fn, fndef, tensors, scalars, dtypes):
        self.fn, self.fndef = fn, fndef
        self.tensors, self.scalars, self.dtypes = tensors, scalars, dtypes
        self.out = []
        self.depth = 1
        self.tiles, self.full_tiles, self.grid_tiles = {}, {}, []
        self.values = {}
        self.stores = set()
        self.grid_seen = False

    def fail(self, node, msg):
        raise TraceError(f"{self.fndef.name}:{getattr(node, 'lineno', '?')}: {msg}")

    def line(self, text):
        self.out.append("    " * self.depth + text)

    # ---- tiles ---------------------------------------------------------------

    def is_dt(self, func, name=None):
        if not (isinstance(func, ast.Attribute) and isinstance(func.value, ast.Name)):
            return False
        mod = self.fn.__globals__.get(func.value.id)
        modname = getattr(mod, "__name__", "")
        if not (modname.endswith("deuteron") or modname.endswith("deuteron.language")):
            return False
        return name is None or func.attr == name

    def extent(self, node):
        """Text of a dimension size: x.shape[i], an int literal or a scalar parameter."""
        if isinstance(node, ast.Subscript) and isinstance(node.value, ast.Attribute) \
                and node.value.attr == "shape" and isinstance(node.value.value, ast.Name) \
                and node.value.value.id in self.tensors:
            if not (isinstance(node.slice, ast.Constant) and isinstance(node.slice.value, int)):
                self.fail(node, "shape index must be a literal")
            return f"{node.value.value.id}_d{node.slice.value}"
        if isinstance(node, ast.Constant) and isinstance(node.value, int):
            return str(node.value)
        if isinstance(node, ast.Name) and node.id in self.scalars:
            return node.id
        self.fail(node, "tile sizes must be x.shape[i], an int literal, or a scalar param")

    def for_loop(self, node):
        if node.orelse:
            self.fail(node, "for/else not supported")
        it = node.iter
        if not (isinstance(it, ast.Call) and self.is_dt(it.func, "tile")):
            self.fail(node, "expected dt.tile(...)")
        if len(it.args) != 1:
            self.fail(node, "dt.tile takes one argument")
        arg = it.args[0]
        extents = [self.extent(e) for e in
                   (arg.elts if isinstance(arg, (ast.List, ast.Tuple)) else [arg])]
        targets = node.target.elts if isinstance(node.target, ast.Tuple) else [node.target]
        if len(targets) != len(extents):
            self.fail(node, f"{len(targets)} tile vars but {len(extents)} sizes")
        if not all(isinstance(t, ast.Name) for t in targets):
            self.fail(node, "tile targets must be plain names")
        names = [t.id for t in targets]
        if not self.grid_seen:
            self.grid_seen = True
            if len(names) > 3:
                self.fail(node, "grid tile loops support at most 3 dimensions")
            for axis, (name, size) in enumerate(zip(names, extents)):
                tv = TileVar(name, size, "grid", f"BLOCK_{name.upper()}")
                self.tiles[name] = tv
                self.grid_tiles.append(tv)
                self.line(f"pid_{axis} = nl.program_id({axis})")
                self.line(f"{tv.offs} = pid_{axis} * {tv.block} + nl.arange(0, {tv.block})")
                self.line(f"{tv.mask} = {tv.offs} < {size}")
            for stmt in node.body:
                self.statement(stmt)
            return
        if len(names) != 1:
            self.fail(node, "inner tile loops iterate one dimension at a time")
        tv = TileVar(names[0], extents[0], "loop", f"BLOCK_{names[0].upper()}")
        self.tiles[tv.name] = tv
        self.line(f"for _i_{tv.name} in range(0, nl.cdiv({tv.size}, {tv.block})):")
        self.depth += 1
        self.line(f"{tv.offs} = _i_{tv.name} * {tv.block} + nl.arange(0, {tv.block})")
        self.line(f"{tv.mask} = {tv.offs} < {tv.size}")
        for stmt in node.body:
            self.statement(stmt)
        self.depth -= 1

    # ---- statements --------------------------------------------------------------

    def statement(self, stmt):
        if isinstance(stmt, ast.For):
            return self.for_loop(stmt)
        if isinstance(stmt, ast.Expr):
            if isinstance(stmt.value, ast.Constant):
                return
            self.fail(stmt, "expression statements have no effect in deuteron kernels")
        if isinstance(stmt, ast.Assign):
            if len(stmt.targets) != 1:
                self.fail(stmt, "single assignment targets only")
            target = stmt.targets[0]
            value = self.expr(stmt.value)
            if isinstance(target, ast.Subscript):
                return self.store(stmt, target, value)
            if isinstance(target, ast.Name):
                self.values[target.id] = Value(target.id, value.mask, value.ndim)
                return self.line(f"{target.id} = {value.code}")
            self.fail(stmt, "unsupported assignment target")
        if isinstance(stmt, ast.AugAssign):
            if not isinstance(stmt.target, ast.Name):
                self.fail(stmt, "augmented assignment needs a plain name target")
            name = stmt.target.id
            if name not in self.values:
                self.fail(stmt, f"'{name}' not defined before augmented assignment")
            if isinstance(stmt.op, ast.Add) and isinstance(stmt.value, ast.BinOp) \
                    and isinstance(stmt.value.op, ast.MatMult):
                a, b = self.expr(stmt.value.left), self.expr(stmt.value.right)
                self.values[name] = Value(name, None, 2)
                return self.line(f"{name} = nl.dot({a.code}, {b.code}, {name})")
            sym = {ast.Add: "+", ast.Sub: "-", ast.Mult: "*", ast.Div: "/"}.get(type(stmt.op))
            if sym is None:
                self.fail(stmt, "unsupported augmented op")
            cur, rhs = self.values[name], self.expr(stmt.value)
            self.values[name] = Value(name, cur.mask, max(cur.ndim, rhs.ndim))
            return self.line(f"{name} = {name} {sym} ({rhs.code})")
        self.fail(stmt, f"unsupported statement: {type(stmt).__name__}")

    # ---- tensor access ---------------------------------------------------------------

    def address(self, node, sub):
        """(tensor name, pointer text, mask text, rank) of t[tile, ...]."""
        name = sub.value.id
        rank = self.tensors[name]
        idx = sub.slice.elts if isinstance(sub.slice, ast.Tuple) else [sub.slice]
        if len(idx) != rank:
            self.fail(node, f"'{name}' has {rank} dims but {len(idx)} indices given")
        tiles = []
        for d, e in enumerate(idx):
            if isinstance(e, ast.Name) and e.id in self.tiles:
                tiles.append(self.tiles[e.id])
            elif isinstance(e, ast.Slice) and e.lower is None and e.upper is None:
                size = f"{name}_d{d}"
                if size not in self.full_tiles:
                    k = len(self.full_tiles)
                    self.full_tiles[size] = TileVar(f"full{k}", size, "full", f"BLOCK_FULL{k}")
                tiles.append(self.full_tiles[size])
            else:
                self.fail(node, "tensor indices must be tile variables or ':'")
        if rank == 1:
            t, = tiles
            return name, f"{name}_ptr + {t.offs} * {name}_s0", t.mask, 1
        if rank == 2:
            r, c = tiles
            return (name,
                    f"{name}_ptr + {r.offs}[:, None] * {name}_s0 + {c.offs}[None, :] * {name}_s1",
                    f"{r.mask}[:, None] & {c.mask}[None, :]", 2)
        self.fail(node, "only 1D/2D tensor access is supported")

    def store(self, node, target, value):
        if not (isinstance(target.value, ast.Name) and target.value.id in self.tensors):
            self.fail(node, "stores must target a tensor parameter")
        name, ptr, mask, _ = self.address(node, target)
        self.stores.add(name)
        self.line(f"nl.store({ptr}, {value.code}, mask={mask})")

    # ---- expressions -------------------------------------------------------------------

    def expr(self, node):
        if isinstance(node, ast.Constant):
            return Value(repr(node.value))
        if isinstance(node, ast.Name):
            if node.id in self.values:
                return self.values[node.id]
            if node.id in self.scalars:
                return Value(node.id)
            if node.id in self.tiles:
                self.fail(node, f"tile '{node.id}' can only be used as an index or size")
            self.fail(node, f"unknown name '{node.id}'")
        if isinstance(node, ast.UnaryOp) and isinstance(node.op, ast.USub):
            v = self.expr(node.operand)
            return Value(f"(-{v.code})", v.mask, v.ndim)
        if isinstance(node, ast.BinOp):
            a, b = self.expr(node.left), self.expr(node.right)
            if isinstance(node.op, ast.MatMult):
                return Value(f"nl.dot({a.code}, {b.code})", None, 2)
            sym = _ARITH.get(type(node.op))
            if sym is None:
                self.fail(node, f"unsupported operator {type(node.op).__name__}")
            return Value(f"({a.code} {sym} {b.code})", a.mask or b.mask, max(a.ndim, b.ndim))
        if isinstance(node, ast.Compare):
            if len(node.ops) != 1:
                self.fail(node, "chained comparisons not supported")
            sym = _COMPARE.get(type(node.ops[0]))
            a, b = self.expr(node.left), self.expr(node.comparators[0])
            return Value(f"({a.code} {sym} {b.code})", a.mask or b.mask, max(a.ndim, b.ndim))
        if isinstance(node, ast.Subscript):
            return self.subscript(node)
        if isinstance(node, ast.Call):
            return self.call(node)
        self.fail(node, f"unsupported expression: {type(node).__name__}")

    def subscript(self, node):
        if isinstance(node.value, ast.Name) and node.value.id in self.tensors:
            name, ptr, mask, rank = self.address(node, node)
            import torch

            zero = "0" if self.dtypes[name] in (torch.int32, torch.int64) else "0.0"
            return Value(f"nl.load({ptr}, mask={mask}, other={zero})", mask, rank)
        if isinstance(node.value, ast.Attribute) and node.value.attr == "shape" \
                and isinstance(node.value.value, ast.Name) and node.value.value.id in self.tensors:
            return Value(self.extent(node))
        base = self.expr(node.value)
        idx = node.slice.elts if isinstance(node.slice, ast.Tuple) else [node.slice]
        parts, added = [], 0
        for e in idx:
            if isinstance(e, ast.Constant) and e.value is None:
                parts.append("None")
                added += 1
            elif isinstance(e, ast.Slice) and e.lower is None and e.upper is None:
                parts.append(":")
            else:
                self.fail(node, "only ':' and None subscripts on computed values")
        sel = ", ".join(parts)
        mask = f"({base.mask})[{sel}]" if base.mask and added else base.mask
        return Value(f"({base.code})[{sel}]", mask, base.ndim + added)

    def call(self, node):
        f = node.func
        if isinstance(f, ast.Attribute) and self.is_dt(f):
            if f.attr in ("zeros", "full"):
                return self.alloc(node, f.attr)
            template = dl.ELEMENTWISE.get(f.attr)
            if template is None:
                self.fail(node, f"dt.{f.attr} is not supported in compiled kernels")
            args = [self.expr(a) for a in node.args]
            return Value(template.format(*[a.code for a in args]),
                         next((a.mask for a in args if a.mask), None),
                         max((a.ndim for a in args), default=0))
        if isinstance(f, ast.Name) and f.id in ("float", "int") and node.args \
                and isinstance(node.args[0], ast.Constant):
            return Value(f"{f.id}({node.args[0].value!r})")
        if isinstance(f, ast.Attribute):
            base = self.expr(f.value)
            if f.attr in dl.REDUCTIONS or f.attr == "mean":
                return self.reduction(node, base, f.attr)
            if f.attr == "to":
                self.fail(node, "use dt.zeros(..., dtype=...) / implicit store casts instead of .to()")
        self.fail(node, f"unsupported call {ast.dump(f)[:60]}")

    def alloc(self, node, which):
        shape = node.args[0]
        dims = []
        for e in (shape.elts if isinstance(shape, (ast.List, ast.Tuple)) else [shape]):
            if isinstance(e, ast.Name) and e.id in self.tiles:
                dims.append(self.tiles[e.id].block)
            elif isinstance(e, ast.Constant):
                dims.append(str(e.value))
            else:
                self.fail(node, "dt.zeros shape entries must be tile vars or int literals")
        dtype = "nl.float32"
        for kw in node.keywords:
            if kw.arg == "dtype":
                try:
                    val = eval(compile(ast.Expression(kw.value), "<dtype>", "eval"),  # noqa: S307
                               self.fn.__globals__)
                except Exception:  # noqa: BLE001
                    val = None
                dtype = dl.DTYPE_NAMES.get(val)
                if dtype is None:
                    self.fail(node, "unsupported dtype")
        shape_text = "(" + ", ".join(dims) + ",)"
        if which == "zeros":
            return Value(f"nl.zeros({shape_text}, dtype={dtype})", None, len(dims))
        fill = self.expr(node.args[1])
        return Value(f"nl.full({shape_text}, {fill.code}, dtype={dtype})", None, len(dims))

    def reduction(self, node, base, method):
        axis = None
        if node.args and isinstance(node.args[0], ast.Constant):
            axis = node.args[0].value
        for kw in node.keywords:
            if kw.arg in ("axis", "dim") and isinstance(kw.value, ast.Constant):
                axis = kw.value.value
        if axis is not None and axis < 0:
            if base.ndim <= 0:
                self.fail(node, "cannot resolve negative axis; use a non-negative one")
            axis += base.ndim
        if method == "mean":
            # sum over the valid lanes divided by their number (the reference leaves mean()
            # out, deuteron/codegen.py:412-413): padded lanes count for nothing
            arg = "" if axis is None else f", axis={axis}"
            if base.mask:
                total = f"nl.sum(nl.where({base.mask}, {base.code}, 0.0){arg})"
                count = (f"nl.sum(nl.broadcast_to(nl.where({base.mask}, 1.0, 0.0), "
                         f"({base.code}).shape){arg})")
            else:
                total = f"nl.sum({base.code}{arg})"
                if base.ndim <= 0:
                    self.fail(node, "mean() of a value whose rank is not known")
                dims = range(base.ndim) if axis is None else [axis]
                count = " * ".join(f"({base.code}).shape[{d}]" for d in dims)
            return Value(f"({total} / ({count}))", None, 0 if axis is None else max(0, base.ndim - 1))
        fn, identity = dl.REDUCTIONS[method]
        inner = f"nl.where({base.mask}, {base.code}, {identity})" if base.mask else base.code
        arg = "" if axis is None else f", axis={axis}"
        return Value(f"{fn}({inner}{arg})", None, 0 if axis is None else max(0, base.ndim - 1))


def generate(fn, fndef, args, newt_module="newt_b200"):
    """Traces `fn` for these example arguments and returns its KernelSource."""
    import torch

    names = [a.arg for a in fndef.args.args]
    if len(names) != len(args):
        raise TraceError(f"{fndef.name}: expected {len(names)} args, got {len(args)}")
    tensors, scalars, dtypes = {}, [], {}
    for name, val in zip(names, args):
        if torch.is_tensor(val):
            tensors[name] = val.dim()
            dtypes[name] = val.dtype
        elif isinstance(val, (int, float)):
            scalars.append(name)
        else:
            raise TraceError(f"unsupported argument type for '{name}': {type(val)}")

    em = _Emitter(fn, fndef, tensors, scalars, dtypes)
    body = fndef.body
    if body and isinstance(body[0], ast.Expr) and isinstance(body[0].value, ast.Constant):
        body = body[1:]
    for stmt in body:
        if not isinstance(stmt, ast.For):
            em.fail(stmt, "top level of a deuteron kernel must be `for ... in dt.tile(...)`")
        em.for_loop(stmt)

    prologue = []
    for tv in em.full_tiles.values():   # whole-dimension tiles are set up before the body
        prologue.append(f"    {tv.offs} = nl.arange(0, {tv.block})")
        prologue.append(f"    {tv.mask} = {tv.offs} < {tv.size}")

    signature, params = [], []
    for name, rank in tensors.items():
        signature.append(f"{name}_ptr")
        signature += [f"{name}_d{d}" for d in range(rank)]
        signature += [f"{name}_s{d}" for d in range(rank)]
        params.append(("tensor", name))
    for name in scalars:
        signature.append(name)
        params.append(("scalar", name))
    tile_vars = list(em.tiles.values()) + list(em.full_tiles.values())
    signature += [f"{tv.block}: nl.constexpr" for tv in tile_vars]

    kname = f"{fndef.name}_newt"
    text = [f"import {newt_module} as newt", f"import {newt_module}.language as nl", "",
            "@newt.jit", f"def {kname}({', '.join(signature)}):"] + prologue + em.out
    return KernelSource(kname, "\n".join(text) + "\n", params, tile_vars, em.grid_tiles,
                        [tv.block for tv in em.tiles.values()], em.stores)
