"""Lowering: traced kernel graph -> launch plan on a hand-written sm_100a kernel.

The reference lowers every kernel through one generic emitter
(newt/compiler/codegen.py).  This backend instead owns a small set of
hand-written kernels (libnewt_b200.so) and recognises the programs they
implement:

    elementwise add          examples/01_vector_add.py:14-21
    fused row softmax        examples/02_fused_softmax.py:15-24
    layernorm forward        examples/03_layernorm.py:13-27
    matmul K loop (nl.dot)   examples/04_matmul.py:14-45, benchmarks/bench.py:90-108,
                             and the text deuteron generates (deuteron/codegen.py:104-175)
    flash attention loop     examples/05_fused_attention.py:14-48 (+ batch*heads, causal)

Recognition is structural (on the expression graph, not on source text) and
every quantity a kernel needs -- extents, strides, which argument plays which
role -- is recovered from the graph as a polynomial in the runtime arguments
and evaluated at launch.  A program that matches none of them -- block arithmetic,
reductions, runtime loops, dots on shapes no tensor-core tile takes -- is turned into CUDA
text and compiled at run time (pointwise.py, PointwisePlan); what that lowering refuses too
raises CompileError naming what is missing.  Nothing falls back to another backend or to the CPU.
"""

import ctypes

from .. import types as tp
from . import pointwise
from .affine import Analyzer, NotAffine, Poly
from .trace import CompileError, Node


_RUNTIME = None


def _runtime():
    """(abi, kernels) of the runtime package, imported at the first launch: the runtime imports
    this module, and a launch asks for them every time."""
    global _RUNTIME
    if _RUNTIME is None:
        from ..runtime import abi, kernels
        _RUNTIME = (abi, kernels)
    return _RUNTIME


class Unmatched(Exception):
    """Internal: this recogniser does not apply (reason for diagnostics)."""


# --------------------------------------------------------------------------- patterns

class Cap:
    """Pattern wildcard: binds a name to whatever node stands there; a name used
    twice must bind the same node."""

    def __init__(self, name, pred=None):
        self.name = name
        self.pred = pred


class Pat:
    def __init__(self, op, args, **attrs):
        self.op = op
        self.args = args
        self.attrs = attrs


def p_bin(fn, a, b):
    return Pat("bin", [a, b], fn=fn)


def p_math(fn, x):
    return Pat("math", [x], fn=fn)


def p_reduce(fn, x):
    return Pat("reduce", [x], fn=fn)


def p_const(value):
    return Pat("const", [value])


def match(pat, node, caps):
    if isinstance(pat, Cap):
        if pat.name in caps:
            return caps[pat.name] is node
        if pat.pred is not None and not pat.pred(node):
            return False
        caps[pat.name] = node
        return True
    if isinstance(pat, Pat):
        if not isinstance(node, Node) or node.op != pat.op:
            return False
        attrs = dict(node.attrs)
        for k, v in pat.attrs.items():
            if attrs.get(k) != v:
                return False
        if len(pat.args) != len(node.args):
            return False
        return all(match(p, a, caps) for p, a in zip(pat.args, node.args))
    # literal
    if isinstance(node, Node):
        return False
    if isinstance(pat, float) and isinstance(node, (int, float)):
        return float(node) == pat or (pat != pat and node != node)
    return pat == node


def match_commutative(fn, pa, pb, node, caps):
    """bin(fn, pa, pb) with the operands in either order."""
    for x, y in ((pa, pb), (pb, pa)):
        trial = dict(caps)
        if match(p_bin(fn, x, y), node, trial):
            caps.clear()
            caps.update(trial)
            return True
    return False


# --------------------------------------------------------------------------- helpers

def _param_only(poly):
    return all(a[0] == "param" for a in poly.atoms())


def _compile_int(poly):
    """Host function args_dict -> int for a polynomial in runtime parameters."""
    if not _param_only(poly):
        raise Unmatched(f"quantity {poly!r} depends on more than runtime arguments")
    c = poly.const_value()
    if c is not None:
        return lambda a, _c=c: _c
    return eval("lambda a: " + poly.to_python("a"))  # noqa: S307 - generated from a Poly


def _param_name(node):
    if isinstance(node, Node) and node.op == "param":
        return dict(node.attrs)["name"]
    return None


def _top_level_stores(trace):
    return [e for e in trace.effects if e[0] == "store"]


def _loops(trace):
    return [e[1] for e in trace.effects if e[0] == "for"]


class RowAccess:
    """A 1-D pointer block `base + row_offset(pid) + (ax0 + c)`: one contiguous
    row per program."""

    def __init__(self, an, ptr, rank1_only=True):
        if len(ptr.shape) != 1:
            raise Unmatched("not a 1-D pointer block")
        self.base, poly = an.pointer(ptr)
        qr = poly.coeff_of(("ax", 0))
        if qr is None:
            raise Unmatched("non-linear column index")
        q, r = qr
        if q.const_value() != 1:
            raise Unmatched("columns are not unit-stride")
        if r.has_kind("ax", "iter", "carried"):
            raise Unmatched("row offset depends on more than the program id")
        self.pid_axes = sorted(a[1] for a in r.atoms() if a[0] == "pid")
        self.offset = r  # polynomial in pid + params


def _mask_bound_1d(an, mask, index_poly):
    """For mask == (index < bound) returns the polynomial `bound - (index - ax0)`,
    i.e. the number of valid columns counted from ax0 = 0; `index_poly` is the
    element index the pointers use (without base offset)."""
    if mask is None:
        return None
    if mask.op != "cmp":
        raise Unmatched("mask is not a single comparison")
    fn = dict(mask.attrs)["fn"]
    a, b = mask.args
    try:
        pa, pb = an._aligned(a, b, len(mask.shape))
    except NotAffine as e:
        raise Unmatched(f"mask is not affine ({e})")
    if fn == "lt":
        d = pa - pb          # d < 0
    elif fn == "gt":
        d = pb - pa
    else:
        raise Unmatched(f"mask comparison '{fn}'")
    qr = d.coeff_of(("ax", 0))
    if qr is None or qr[0].const_value() != 1:
        raise Unmatched("mask does not bound the column index")
    rest = qr[1]            # ax0 + rest < 0  ->  ax0 < -rest
    return -rest


# --------------------------------------------------------------------------- plans

class Plan:
    """What one specialization of a kernel does at launch."""

    kind = ""
    entry = ""       # C-ABI entry point the plan calls

    def launch(self, grid, args):
        raise NotImplementedError

    def describe(self):
        return f"{self.kind} -> {self.entry}"


def _split_row_offset(off, what):
    """off = pid0 * stride + const  (polynomials in runtime params)."""
    qr = off.coeff_of(("pid", 0))
    if qr is None:
        raise Unmatched(f"{what}: row offset is not linear in program_id(0)")
    stride, const = qr
    if not _param_only(stride) or not _param_only(const):
        raise Unmatched(f"{what}: row offset uses more than program_id(0) and arguments")
    return stride, const


def _row_hardware_key(plan):
    """Row kernels pick their own threads-per-row and vectors-per-thread from the row length:
    every block / warp configuration of the source runs the same device code."""
    return (plan.entry,)


def _rows_of(plan, grid, args):
    """Rows a row-kernel launch covers: one per program, or BLOCK rows per program clipped
    by the row mask for the 2-D (tile) spelling."""
    rows = grid[0] * plan.rows_per_program
    if plan.row_bound is not None:
        rows = min(rows, plan.row_bound(args))
    for name, fn in plan.unit_strides:
        if fn(args) != 1:
            raise CompileError(f"{plan.kind}: '{name}' is not unit-stride along the row "
                               f"(stride {fn(args)})")
    return rows


class SoftmaxPlan(Plan):
    kind, entry = "row softmax", "nb200_softmax_f32"
    rows_per_program, row_bound, unit_strides = 1, None, ()
    hardware_key = _row_hardware_key

    def __init__(self, x, out, n, block, sx, cx, so, co):
        self.x, self.out, self.block = x, out, block
        self.n, self.sx, self.cx, self.so, self.co = map(_compile_int, (n, sx, cx, so, co))

    def launch(self, grid, args):
        from ..runtime import kernels

        rows = _rows_of(self, grid, args)
        n = min(self.n(args), self.block)
        if rows <= 0 or n <= 0:
            return
        x, out = args[self.x], args[self.out]
        cx, co = self.cx(args), self.co(args)
        if cx:
            x = x.reshape(-1)[cx:] if x.is_contiguous() else _offset_view(x, cx)
        if co:
            out = out.reshape(-1)[co:] if out.is_contiguous() else _offset_view(out, co)
        kernels.softmax_f32(x, out, rows, n, self.sx(args), self.so(args))


class LayerNormPlan(Plan):
    kind, entry = "layernorm forward", "nb200_layernorm"
    rows_per_program, row_bound, unit_strides = 1, None, ()
    hardware_key = _row_hardware_key

    def __init__(self, x, w, b, out, eps, n, block, sx, so):
        self.x, self.w, self.b, self.out, self.eps, self.block = x, w, b, out, eps, block
        self.n, self.sx, self.so = map(_compile_int, (n, sx, so))

    def launch(self, grid, args):
        from ..runtime import kernels

        rows = _rows_of(self, grid, args)
        n = min(self.n(args), self.block)
        if rows <= 0 or n <= 0:
            return
        eps = args[self.eps] if isinstance(self.eps, str) else self.eps
        kernels.layernorm(args[self.x], args[self.w], args[self.b], args[self.out], rows, n,
                          self.sx(args), self.so(args), eps)


class AddPlan(Plan):
    kind, entry = "elementwise add", "nb200_add_f32"

    def __init__(self, x, y, out, n, block):
        self.x, self.y, self.out, self.block = x, y, out, block
        self.n = _compile_int(n) if n is not None else None

    def launch(self, grid, args):
        from ..runtime import kernels

        covered = grid[0] * self.block
        n = covered if self.n is None else min(self.n(args), covered)
        if n <= 0:
            return
        kernels.add_f32(args[self.x], args[self.y], args[self.out], n)


def _offset_view(t, elems):
    import torch

    return torch.as_strided(t, (t.numel() - elems,), (1,), t.storage_offset() + elems)


# --------------------------------------------------------------------------- row recognisers

def _single_store(trace, what):
    if _loops(trace):
        raise Unmatched(f"{what}: kernel has a runtime loop")
    stores = _top_level_stores(trace)
    if len(stores) != 1:
        raise Unmatched(f"{what}: expected exactly one store, found {len(stores)}")
    return stores[0]


def lower_add(trace, an):
    _, ptr, value, mask, _ = _single_store(trace, "add")
    x, y = Cap("x"), Cap("y")
    caps = {}
    if not match(p_bin("add", Pat("load", [x, Cap("mx"), Cap("ox")]),
                       Pat("load", [y, Cap("my"), Cap("oy")])), value, caps):
        raise Unmatched("add: stored value is not load(x) + load(y)")
    if caps["mx"] is not mask or caps["my"] is not mask:
        raise Unmatched("add: loads and store use different masks")
    accs = [RowAccess(an, p) for p in (caps["x"], caps["y"], ptr)]
    block = ptr.shape[0]
    for acc, nm in zip(accs, "xyo"):
        if acc.offset != accs[0].offset:
            raise Unmatched("add: operands are addressed differently")
    stride, const = _split_row_offset(accs[0].offset, "add")
    if stride.const_value() != block or not const.is_zero():
        raise Unmatched("add: programs do not tile the vector contiguously")
    for node in (caps["x"], caps["y"], ptr):
        if node.dtype.element != tp.float32:
            raise Unmatched("add: only float32 vectors have a kernel")
    n = None
    if mask is not None:
        bound = _mask_bound_1d(an, mask, None)   # ax0 < bound, bound = n - pid0*BLOCK
        n = bound + Poly.atom(("pid", 0)) * Poly.const(block)
        if not _param_only(n):
            raise Unmatched("add: mask is not `offsets < n`")
    return AddPlan(accs[0].base, accs[1].base, accs[2].base, n, block)


def _row_common(an, ptr_x, ptr_o, mask, what):
    ax, ao = RowAccess(an, ptr_x), RowAccess(an, ptr_o)
    block = ptr_x.shape[0]
    sx, cx = _split_row_offset(ax.offset, what)
    so, co = _split_row_offset(ao.offset, what)
    n = Poly.const(block)
    if mask is not None:
        n = _mask_bound_1d(an, mask, None)
        if not _param_only(n):
            raise Unmatched(f"{what}: column mask is not `cols < N`")
    return ax, ao, block, sx, cx, so, co, n


def lower_softmax(trace, an):
    _, ptr, value, mask, _ = _single_store(trace, "softmax")
    x = Cap("x", lambda n: isinstance(n, Node) and n.op == "load")
    shifted = p_bin("sub", x, p_reduce("max", x))
    num = p_math("exp", shifted)
    caps = {}
    if not match(p_bin("div", num, p_reduce("sum", num)), value, caps):
        raise Unmatched("softmax: stored value is not exp(x - max(x)) / sum(exp(x - max(x)))")
    load = caps["x"]
    ptr_x, lmask, other = load.args
    if lmask is not mask:
        raise Unmatched("softmax: load and store use different masks")
    if lmask is not None and other != float("-inf"):
        raise Unmatched("softmax: masked lanes must load -inf")
    if load.dtype != tp.float32 or ptr.dtype.element != tp.float32:
        raise Unmatched("softmax: only float32 rows have a kernel")
    ax, ao, block, sx, cx, so, co, n = _row_common(an, ptr_x, ptr, mask, "softmax")
    return SoftmaxPlan(ax.base, ao.base, n, block, sx, cx, so, co)


def lower_layernorm(trace, an):
    _, ptr, value, mask, _ = _single_store(trace, "layernorm")
    is_load = lambda n: isinstance(n, Node) and n.op == "load"  # noqa: E731
    x, w, b = Cap("x", is_load), Cap("w", is_load), Cap("b", is_load)
    count, eps = Cap("count"), Cap("eps")
    mean = p_bin("div", p_reduce("sum", x), count)
    centred = p_bin("sub", x, mean)
    diff_masked = Pat("where", [Cap("wmask"), centred, p_const(0.0)])
    caps = {}
    ok = False
    for diff in (diff_masked, centred):
        var = p_bin("div", p_reduce("sum", p_bin("mul", diff, diff)), count)
        rstd = p_math("rsqrt", p_bin("add", var, eps))
        trial = {}
        if match(p_bin("add", p_bin("mul", p_bin("mul", centred, rstd), w), b), value, trial):
            caps, ok = trial, True
            break
    if not ok:
        raise Unmatched("layernorm: stored value is not (x - mean) * rsqrt(var + eps) * w + b "
                        "with two-pass statistics")
    lx, lw, lb = caps["x"], caps["w"], caps["b"]
    if "wmask" in caps and caps["wmask"] is not mask:
        raise Unmatched("layernorm: variance mask differs from the load mask")
    if "wmask" not in caps and mask is not None:
        raise Unmatched("layernorm: padded lanes are not masked out of the variance")
    for ld in (lx, lw, lb):
        if ld.args[1] is not mask:
            raise Unmatched("layernorm: loads use different masks")
    if lx.args[2] not in (None, 0.0, 0):
        raise Unmatched("layernorm: masked lanes of x must load 0")
    dt = lx.dtype
    if dt not in (tp.float32, tp.float16, tp.bfloat16) or lw.dtype != dt or lb.dtype != dt \
            or ptr.dtype.element != dt:
        raise Unmatched("layernorm: x, w, b and out must share one of float32/float16/bfloat16")
    ax, ao, block, sx, cx, so, co, n = _row_common(an, lx.args[0], ptr, mask, "layernorm")
    if not cx.is_zero() or not co.is_zero():
        raise Unmatched("layernorm: constant pointer offsets are not supported")
    for ld, nm in ((lw, "w"), (lb, "b")):
        acc = RowAccess(an, ld.args[0])
        if not acc.offset.is_zero():
            raise Unmatched(f"layernorm: {nm} must be indexed by the column only")
    # the divisor of both statistics must be the row length
    cnt = caps["count"]
    try:
        cnt_poly = an.poly(cnt)
    except NotAffine:
        raise Unmatched("layernorm: divisor is not an integer count")
    if cnt_poly != n:
        raise Unmatched("layernorm: statistics are not divided by the row length")
    e = caps["eps"]
    if _param_name(e) is not None:
        eps = _param_name(e)
    elif isinstance(e, Node) and e.op == "const":
        eps = float(e.args[0])
    else:
        raise Unmatched("layernorm: eps must be an argument or a literal")
    lwb = RowAccess(an, lw.args[0]).base, RowAccess(an, lb.args[0]).base
    return LayerNormPlan(ax.base, lwb[0], lwb[1], ao.base, eps, n, block, sx, so)


# --------------------------------------------------------------------------- row programs as 2-D tiles
#
# deuteron writes softmax and layernorm over [BLOCK_M rows, whole row] tiles with axis-1
# reductions and masks propagated into them (deuteron/codegen.py:382-410 of the reference):
#     m = nl.max(nl.where(mask, row, -inf), axis=1);  e = nl.exp(row - m[:, None]);  ...
# The same row kernels serve them; a program then covers BLOCK_M rows.

def _row_tile(an, ptr, mask, what):
    """(TileAccess, row-extent fn, column-extent polynomial) of a [rows, whole-row] tile."""
    t = TileAccess(an, ptr, what)
    step = t.step_of(0, "pid")
    if step is None or step[0] != ("pid", 0) or step[1] != t.shape[0] or not t.origin[1].is_zero():
        raise Unmatched(f"{what}: programs must tile the rows by BLOCK and span whole rows")
    bounds = _tile_bounds(an, mask, t, what)
    if len(bounds.get(1, [])) != 1:
        raise Unmatched(f"{what}: the row length must be given by one column mask")
    return t, _extent_fn("row", bounds.get(0)), bounds[1][0]


def _finish_tile_plan(plan, tx, to, row_fns, extra_unit=()):
    plan.rows_per_program = tx.shape[0]
    plan.row_bound = _extent_fn("row", *[[]]) if not row_fns else (
        lambda a, fns=row_fns: min(f(a) for f in fns))
    plan.unit_strides = tuple((t.base, _compile_int(t.stride[1])) for t in (tx, to)) + \
        tuple(extra_unit)
    return plan


def lower_softmax_tile(trace, an):
    _, ptr, value, omask, _ = _single_store(trace, "tile softmax")
    row = Cap("row", lambda n: isinstance(n, Node) and n.op == "load")
    m1 = Cap("mask")
    neg_inf = float("-inf")
    rmax = Pat("reduce", [Pat("where", [m1, row, p_const(neg_inf)])], fn="max", axis=1)
    e = p_math("exp", p_bin("sub", row, Pat("expand", [rmax], axis=1)))
    den = Pat("reduce", [Pat("where", [m1, e, p_const(0.0)])], fn="sum", axis=1)
    caps = {}
    if not match(p_bin("div", e, Pat("expand", [den], axis=1)), value, caps):
        raise Unmatched("tile softmax: stored value is not exp(row - max) / sum(exp(row - max)) "
                        "with masked axis-1 reductions")
    load = caps["row"]
    if load.args[1] is not caps["mask"]:
        raise Unmatched("tile softmax: reductions are masked differently from the load")
    if load.dtype != tp.float32 or ptr.dtype.element != tp.float32:
        raise Unmatched("tile softmax: only float32 rows have a kernel")
    tx, rows_x, n_x = _row_tile(an, load.args[0], load.args[1], "tile softmax input")
    to, rows_o, n_o = _row_tile(an, ptr, omask, "tile softmax output")
    if tx.shape != to.shape:
        raise Unmatched("tile softmax: input and output tiles differ")
    zero = Poly()
    plan = SoftmaxPlan(tx.base, to.base, n_x, tx.shape[1], tx.stride[0], zero, to.stride[0], zero)
    n_out = _compile_int(n_o)
    n_in = plan.n
    plan.n = lambda a: min(n_in(a), n_out(a))
    return _finish_tile_plan(plan, tx, to, [f for f in (rows_x, rows_o) if f is not None])


def lower_layernorm_tile(trace, an):
    _, ptr, value, omask, _ = _single_store(trace, "tile layernorm")
    is_load = lambda n: isinstance(n, Node) and n.op == "load"  # noqa: E731
    row, w, b = Cap("row", is_load), Cap("w", is_load), Cap("b", is_load)
    m1, count, eps = Cap("mask"), Cap("count"), Cap("eps")
    mean = p_bin("div", Pat("reduce", [Pat("where", [m1, row, p_const(0.0)])], fn="sum", axis=1),
                 count)
    diff = p_bin("sub", row, Pat("expand", [mean], axis=1))
    var = p_bin("div", Pat("reduce", [Pat("where", [m1, p_bin("mul", diff, diff), p_const(0.0)])],
                           fn="sum", axis=1), count)
    rstd = p_math("rsqrt", p_bin("add", var, eps))
    caps = {}
    if not match(p_bin("add", p_bin("mul", p_bin("mul", diff, Pat("expand", [rstd], axis=1)), w),
                       b), value, caps):
        raise Unmatched("tile layernorm: stored value is not (row - mean) * rsqrt(var + eps) * w "
                        "+ b with masked two-pass statistics")
    lx, lw, lb = caps["row"], caps["w"], caps["b"]
    if lx.args[1] is not caps["mask"]:
        raise Unmatched("tile layernorm: reductions are masked differently from the load")
    dt = lx.dtype
    if dt not in (tp.float32, tp.float16, tp.bfloat16) or lw.dtype != dt or lb.dtype != dt \
            or ptr.dtype.element != dt:
        raise Unmatched("tile layernorm: x, w, b and out must share one of "
                        "float32/float16/bfloat16")
    tx, rows_x, n_x = _row_tile(an, lx.args[0], lx.args[1], "tile layernorm input")
    to, rows_o, n_o = _row_tile(an, ptr, omask, "tile layernorm output")
    try:
        if an.poly(caps["count"]) != n_x:
            raise Unmatched("tile layernorm: statistics are not divided by the row length")
    except NotAffine:
        raise Unmatched("tile layernorm: divisor is not an integer count")
    extra = []
    for ld, nm in ((lw, "w"), (lb, "b")):
        if len(ld.shape) != 1:
            raise Unmatched(f"tile layernorm: {nm} must be a 1-D load over the row")
        base, poly = an.pointer(ld.args[0])
        q, r = poly.coeff_of(("ax", 0))
        if not r.is_zero() or not _param_only(q):
            raise Unmatched(f"tile layernorm: {nm} must be indexed by the column only")
        extra.append((base, _compile_int(q)))
    e = caps["eps"]
    if _param_name(e) is not None:
        eps_v = _param_name(e)
    elif isinstance(e, Node) and e.op == "const":
        eps_v = float(e.args[0])
    else:
        raise Unmatched("tile layernorm: eps must be an argument or a literal")
    plan = LayerNormPlan(tx.base, extra[0][0], extra[1][0], to.base, eps_v, n_x, tx.shape[1],
                         tx.stride[0], to.stride[0])
    return _finish_tile_plan(plan, tx, to, [f for f in (rows_x, rows_o) if f is not None], extra)


# --------------------------------------------------------------------------- scalar expressions

_PY_OPS = {"add": "({0} + {1})", "sub": "({0} - {1})", "mul": "({0} * {1})",
           "floordiv": "({0} // {1})", "div": "({0} // {1})", "mod": "({0} % {1})",
           "cdiv": "(-(-{0} // {1}))", "min": "min({0}, {1})", "max": "max({0}, {1})"}


def _scalar_source(v):
    """Python source for an integer scalar of the graph, over the dict `a` of
    runtime arguments."""
    if isinstance(v, bool) or not isinstance(v, (int, Node)):
        raise Unmatched(f"cannot evaluate {v!r} on the host")
    if isinstance(v, int):
        return repr(v)
    if v.shape != () or not v.dtype.is_int:
        raise Unmatched("loop bounds must be integer scalars")
    if v.op == "const":
        return repr(v.args[0])
    if v.op == "param":
        return f"a[{dict(v.attrs)['name']!r}]"
    if v.op == "neg":
        return f"(-{_scalar_source(v.args[0])})"
    if v.op == "cast":
        return _scalar_source(v.args[0])
    if v.op == "bin":
        fn = dict(v.attrs)["fn"]
        if fn in _PY_OPS:
            return _PY_OPS[fn].format(_scalar_source(v.args[0]), _scalar_source(v.args[1]))
    raise Unmatched(f"loop bound uses '{v.op}', which the host cannot evaluate")


def _compile_scalar(v):
    return eval("lambda a: " + _scalar_source(v))  # noqa: S307 - generated from the graph


def _trip_count_fn(loop):
    lo, hi, step = (_compile_scalar(x) for x in (loop.lo, loop.hi, loop.step))
    return lambda a: max(0, -(-(hi(a) - lo(a)) // step(a))) if step(a) > 0 else 0


# --------------------------------------------------------------------------- 2-D tiles

class TileAccess:
    """A 2-D pointer block  base + idx0 * s0 + idx1 * s1  where each index is
    `ax_d + (program id | loop iteration) * BLOCK_d`."""

    def __init__(self, an, ptr, what, allow_batch=False):
        if len(ptr.shape) != 2:
            raise Unmatched(f"{what}: not a 2-D pointer block")
        self.shape = ptr.shape
        self.batch = None    # (("pid", axis), stride polynomial) of a leading batch/head index
        try:
            self.base, poly = an.pointer(ptr)
        except NotAffine as e:
            raise Unmatched(f"{what}: pointer block is not affine ({e})")
        qr0 = poly.coeff_of(("ax", 0))
        qr1 = qr0[1].coeff_of(("ax", 1)) if qr0 else None
        if qr0 is None or qr1 is None:
            raise Unmatched(f"{what}: pointer block is not linear in its indices")
        self.stride = [qr0[0], qr1[0]]
        rest = qr1[1]
        for s in self.stride:
            if not _param_only(s) or s.is_zero():
                raise Unmatched(f"{what}: strides must be runtime arguments or constants")
        # distribute the remaining terms (pid / iter multiples) over the two dims
        self.origin = [Poly(), Poly()]   # index offset of each dim, in elements of that dim
        const = Poly()
        for atom in sorted(rest.atoms(), key=repr):
            if atom[0] == "param":
                continue
            if atom[0] not in ("pid", "iter"):
                raise Unmatched(f"{what}: offset depends on {atom}")
        leftovers = rest
        for atom in sorted({a for a in rest.atoms() if a[0] in ("pid", "iter")}, key=repr):
            q, leftovers = leftovers.coeff_of(atom)
            placed = False
            # prefer the dim whose stride is not the constant 1 (dividing by 1 always works)
            order = sorted((0, 1), key=lambda d: self.stride[d].const_value() == 1)
            for d in order:
                blocks = q.divide_by(self.stride[d])
                if blocks is not None and blocks.const_value() is not None:
                    self.origin[d] = self.origin[d] + Poly.atom(atom) * blocks
                    placed = True
                    break
            if not placed and allow_batch and atom[0] == "pid" and self.batch is None \
                    and _param_only(q):
                self.batch = (atom, q)
                placed = True
            if not placed:
                raise Unmatched(f"{what}: {atom} does not step by whole blocks")
        if not leftovers.is_zero():
            raise Unmatched(f"{what}: constant pointer offsets are not supported")

    def step_of(self, d, kind):
        """(atom, blocks) if dim d advances with exactly one atom of `kind`."""
        terms = [(m, c) for m, c in self.origin[d].terms.items()]
        if len(terms) != 1 or len(terms[0][0]) != 1 or terms[0][0][0][0] != kind:
            return None
        return terms[0][0][0], terms[0][1]


def _split_and(mask):
    if mask is None:
        return []
    if mask.op == "bin" and dict(mask.attrs)["fn"] == "and":
        return _split_and(mask.args[0]) + _split_and(mask.args[1])
    return [mask]


def _comparison(an, term, what):
    """(fn, lhs - rhs) of a mask term, seen through x[:, None] / x[None, :]."""
    if term.op == "expand":
        fn, d = _comparison(an, term.args[0], what)
        axis = dict(term.attrs)["axis"]
        return fn, d.map_atoms(lambda a: Poly.atom(("ax", a[1] + 1))
                               if a[0] == "ax" and a[1] >= axis else None)
    if term.op == "broadcast":
        fn, d = _comparison(an, term.args[0], what)
        k = len(term.shape) - len(term.args[0].shape)
        return fn, d.map_atoms(lambda a: Poly.atom(("ax", a[1] + k)) if a[0] == "ax" else None)
    if term.op != "cmp":
        raise Unmatched(f"{what}: mask term is not a comparison")
    try:
        pa, pb = an._aligned(term.args[0], term.args[1], len(term.shape))
    except NotAffine as e:
        raise Unmatched(f"{what}: mask is not affine ({e})")
    return dict(term.attrs)["fn"], pa - pb


def _tile_bounds(an, mask, tile, what):
    """Per-dimension extent polynomials implied by a mask built from
    `index_d < bound_d` comparisons; checks that index_d is the tile's own."""
    bounds = {}
    for term in _split_and(mask):
        fn, d = _comparison(an, term, what)
        if len(term.shape) < 2:
            d = d.map_atoms(lambda a, k=2 - len(term.shape): Poly.atom(("ax", a[1] + k))
                            if a[0] == "ax" else None)
        if fn == "gt":
            d = -d
        elif fn != "lt":
            raise Unmatched(f"{what}: mask comparison '{fn}'")
        dims = [k for k in (0, 1) if ("ax", k) in d.atoms()]
        if len(dims) != 1:
            raise Unmatched(f"{what}: a mask term must bound exactly one index")
        k = dims[0]
        q, rest = d.coeff_of(("ax", k))
        if q.const_value() != 1:
            raise Unmatched(f"{what}: mask index is scaled")
        moving = Poly({m: c for m, c in rest.terms.items()
                       if any(a[0] != "param" for a in m)})
        bound = -(rest - moving)
        if moving != tile.origin[k]:
            raise Unmatched(f"{what}: mask bounds a different index than the pointers use")
        bounds.setdefault(k, []).append(bound)
    return bounds


def _extent_fn(what, *bound_lists):
    """Host function for an extent named by one or more masks.  All masks must
    agree at launch: a kernel that loads with one extent and stores with another
    is not the matmul this backend implements."""
    polys = []
    for bl in bound_lists:
        for p in bl or []:
            if p not in polys:
                polys.append(p)
    if not polys:
        return None
    fns = [_compile_int(p) for p in polys]
    if len(fns) == 1:
        return fns[0]

    def extent(a):
        vals = {f(a) for f in fns}
        if len(vals) != 1:
            raise CompileError(f"matmul: masks give different {what} extents {sorted(vals)}")
        return vals.pop()

    return extent


# --------------------------------------------------------------------------- GEMM

class GemmPlan(Plan):
    kind, entry = "matmul K loop", "nb200_gemm"

    def __init__(self):
        self.a = self.b = self.c = None
        self.block = (0, 0, 0)
        self.pid_m = self.pid_n = 0
        self.m_bound = self.n_bound = self.k_bound = None
        self.trips = None
        self.lda = self.ldb = self.ldc = None
        self.inner = ()
        self.num_stages = 3
        self._derived = {}
        self._ready = {}            # (scalars, pointers) -> the library call as it was made last time
        self.row_k = 64   # K elements per 128-byte row: 64 for fp16/bf16, 32 for fp32 (run as tf32)

    def _extents(self, grid, args):
        bm, bn, bk = self.block
        gm = grid[self.pid_m] if self.pid_m < len(grid) else 1
        gn = grid[self.pid_n] if self.pid_n < len(grid) else 1
        m, n, k = gm * bm, gn * bn, self.trips(args) * bk
        if self.m_bound is not None:
            m = min(m, self.m_bound(args))
        if self.n_bound is not None:
            n = min(n, self.n_bound(args))
        if self.k_bound is not None:
            k = min(k, self.k_bound(args))
        return max(m, 0), max(n, 0), max(k, 0)

    def hardware_key(self):
        """What distinguishes this plan on the device.  BLOCK_M = BLOCK_N = 256 asks for the
        CTA-pair kernel (one 256-row tcgen05 MMA over two SMs) whose ring slot holds BLOCK_K
        = one, two or three 128-byte rows of K (64, 128, 192 elements of fp16/bf16; 32, 64, 96
        of fp32); otherwise the tcgen05 tile is picked by BLOCK_N (when it is a tile the
        kernel has) and num_stages is the ring depth -- except that BLOCK_K = two 128-byte rows
        with 64 or 128 columns picks the ring whose slots hold two K slabs (half as many copies
        to issue: what small problems are bound by)."""
        bm, bn, bk = self.block
        rk = self.row_k
        if bm == 256 and bn == 512:        # two 256-column MMAs on one 512-column accumulator
            return ("gemm-pair-wide", 2 * rk if bk == 2 * rk else rk, 0)
        if bm == 256 and bn == 256:
            bk = bk if bk in (rk, 2 * rk, 3 * rk) else 2 * rk
            return ("gemm-pair", bk, self.num_stages if bk == rk else 0)
        if bk == 2 * rk and bn in (64, 128):
            return ("gemm-2slab", bn, 0)
        return ("gemm", bn if bn in (64, 128, 256) else 0, self.num_stages)

    def config(self):
        from ..runtime import kernels

        if self._config is None:
            kind, x, stages = self.hardware_key()
            if kind == "gemm-pair":
                self._config = kernels.gemm_config(block_m=256, block_n=256, block_k=x,
                                                   stages=stages, cta_pair=1)
            elif kind == "gemm-pair-wide":
                self._config = kernels.gemm_config(block_m=256, block_n=512, block_k=x, cta_pair=1)
            elif kind == "gemm-2slab":
                self._config = kernels.gemm_config(block_n=x, block_k=2 * self.row_k)
            else:
                self._config = kernels.gemm_config(block_n=x, stages=stages)
        return self._config

    _config = None

    generic = None      # set by lower(): builds the run-time compiled plan of the same program

    def launch(self, grid, args):
        """The tensor-core kernel, after copying operands that bulk tensor copies cannot fetch
        as they lie (see `_launch_tensor_core`); what that path still refuses -- a C that is not
        unit-stride along its rows -- runs the same program through the generic lowering, on
        the CUDA cores."""
        abi = _runtime()[0]

        # The choice is made per launch: strides are run-time values of one specialization, so
        # a launch the tensor core refuses says nothing about the next one.  The generic plan
        # is compiled at the first refusal and kept for later ones.
        try:
            return self._launch_tensor_core(grid, args)
        except (CompileError, abi.UnsupportedError) as e:
            if self.generic is None:
                raise
            if self._generic_plan is None:
                try:
                    self._generic_plan = self.generic()
                except CompileError as second:
                    raise CompileError(f"{e}; and the generic lowering does not take the program "
                                       f"either: {second}") from e
        self._generic_plan.launch(grid, args)

    _generic_plan = None

    def _launch_tensor_core(self, grid, args, acc32=None):
        """`acc32`: an fp32 buffer laid out like C that takes the accumulator instead of C."""
        abi, kernels = _runtime()

        # extents and strides are polynomials in the scalar arguments: evaluated once per
        # distinct (grid, scalars), the usual case being the same call repeated
        if self._scalars is None:
            self._scalars = [name for name, v in args.items()
                             if isinstance(v, (int, float)) and not isinstance(v, bool)]
        key = (grid, *[args[name] for name in self._scalars])
        derived = self._derived.get(key)
        if derived is None:
            if len(self._derived) >= 256:
                self._derived.clear()
            derived = self._derived[key] = (
                self._extents(grid, args), {name: fn(args) for name, fn in self.inner},
                self.lda(args), self.ldb(args), self.ldc(args))
        (m, n, k), inner, lda, ldb, ldc = derived
        if m == 0 or n == 0:
            return
        a, b, c = args[self.a], args[self.b], args[self.c]
        if acc32 is None:
            # the same tensors again: the call as it was made last time (everything else it
            # depends on -- extents, strides -- is in `key`)
            again = (key, a.data_ptr(), b.data_ptr(), c.data_ptr())
            ready = self._ready.get(again)
            if ready is not None:
                entry, call = ready
                rc = entry(*call, kernels.raw_stream())
                if rc:
                    abi.check(rc)
                return
        if inner[self.c] != 1:
            raise CompileError(
                f"matmul: '{self.c}' is not unit-stride along its fast dimension "
                f"(stride {inner[self.c]})")
        if acc32 is not None:
            c = acc32
        per16 = 16 // a.element_size()

        def fetchable(t, pitch, unit):      # what a bulk tensor copy needs of an operand
            return unit == 1 and pitch % per16 == 0 and t.data_ptr() % 16 == 0

        def remember(entry, *call):          # only calls that take the caller's tensors as they lie
            if acc32 is None and a is args[self.a] and b is args[self.b]:
                if len(self._ready) >= 64:
                    self._ready.clear()
                self._ready[again] = (entry, call)

        # An operand laid out otherwise (a pitch that is not a multiple of 16 bytes, a
        # misaligned base, a transposed A) is first copied into a row-major workspace.
        if not fetchable(a, lda, inner[self.a]):
            a, lda = kernels.repitched("a", a, m, k, lda, inner[self.a])
            self.repitched += 1
        if fetchable(b, inner[self.b], ldb) and inner[self.b] != 1:
            # B[k, n] at k * 1 + n * stride: the caller handed over B^T, which is what the
            # tensor core wants anyway
            if acc32 is not None and self.row_k != 32:
                kernels.gemm_acc32(a, b, c, m, n, k, lda, inner[self.b], ldc, True, self.config())
            elif self._split_bytes(kernels, m, n, k, a.dtype):
                kernels.gemm_split(a, b, c, m, n, k, lda, inner[self.b], ldc, self.config(), True,
                                   self._split_bytes(kernels, m, n, k, a.dtype))
            else:
                kernels.gemm_bt(a, b, c, m, n, k, lda, inner[self.b], ldc, self.config())
                remember(abi.load().nb200_gemm_bt, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k,
                         lda, inner[self.b], ldc, abi.dtype_code(a.dtype), ctypes.byref(self.config()))
            return
        if not fetchable(b, ldb, inner[self.b]):
            b, ldb = kernels.repitched("b", b, k, n, ldb, inner[self.b])
            self.repitched += 1
        if acc32 is not None and self.row_k != 32:
            kernels.gemm_acc32(a, b, c, m, n, k, lda, ldb, ldc, False, self.config())
        elif self._split_bytes(kernels, m, n, k, a.dtype):
            kernels.gemm_split(a, b, c, m, n, k, lda, ldb, ldc, self.config(), False,
                               self._split_bytes(kernels, m, n, k, a.dtype))
        else:
            kernels.gemm(a, b, c, m, n, k, lda, ldb, ldc, self.config())
            remember(abi.load().nb200_gemm, a.data_ptr(), b.data_ptr(), c.data_ptr(), m, n, k, lda,
                     ldb, ldc, abi.dtype_code(a.dtype), ctypes.byref(self.config()))

    def _split_bytes(self, kernels, m, n, k, dtype):
        """Workspace with which the library cuts the last round of tiles along K (a small C with
        a long K), 0 when this problem's tiles stay whole; asked once per shape."""
        if self._split is None:
            self._split = {}
        need = self._split.get((m, n, k))
        if need is None:
            if len(self._split) >= 256:
                self._split.clear()
            need = self._split[(m, n, k)] = kernels.gemm_split_bytes(m, n, k, dtype, self.config())
        return need

    _split = None
    repitched = 0       # how many operands launches of this plan had to copy first
    _scalars = None     # names of the scalar arguments, found at the first launch


def lower_gemm(trace, an, num_stages, epilogue=False):
    """The matmul k loop.  With `epilogue`, the stored value may be any expression of the
    accumulator (bias, activation, scaling, a reduction over the tile) and the store may be of
    any dtype; returns (plan, (loop uid, accumulator name), the store's pointer node, the store
    effect) then."""
    loops = _loops(trace)
    stores = _top_level_stores(trace)
    if len(loops) != 1 or len(stores) != 1:
        raise Unmatched("matmul: expected one K loop followed by one store")
    loop = loops[0]
    if loop.effects:
        raise Unmatched("matmul: the K loop has side effects")
    acc_name = None
    for name, (ph, init, nxt) in loop.carried.items():
        if nxt.op == "dot":
            if acc_name is not None:
                raise Unmatched("matmul: two accumulators")
            acc_name = name
        elif ("carried", loop.uid, name) not in an.closed_forms:
            raise Unmatched(f"matmul: loop-carried '{name}' is neither the accumulator nor an "
                            f"induction")
    if acc_name is None:
        raise Unmatched("matmul: no `acc = nl.dot(a, b, acc)` in the loop")
    ph, init, dot = loop.carried[acc_name]
    a, b, acc_in = dot.args
    if acc_in is not ph:
        raise Unmatched("matmul: nl.dot does not accumulate into the carried block")
    if not (init.op == "full" and init.args[0] == 0):
        raise Unmatched("matmul: accumulator does not start at zero")
    for name, v in (("a", a), ("b", b)):
        if v.op != "load":
            raise Unmatched(f"matmul: operand {name} of nl.dot is not loaded directly from memory")
        if v.args[1] is not None and v.args[2] not in (None, 0, 0.0):
            raise Unmatched(f"matmul: masked lanes of {name} must read 0")
    if a.dtype not in (tp.float16, tp.bfloat16, tp.float32):
        raise Unmatched(f"matmul: {a.dtype.name} operands have no tcgen05 kernel")

    _, c_ptr, c_val, c_mask, _ = stores[0]
    out = c_val.args[0] if c_val.op == "cast" else c_val
    at = dict(out.attrs)
    plain = out.op == "loopout" and at.get("loop") == loop.uid and at.get("name") == acc_name \
        and c_ptr.dtype.element == a.dtype
    if not plain and not epilogue:
        raise Unmatched("matmul: the stored value is not the accumulator cast to the operand "
                        "dtype (taken by the matmul-with-epilogue plan)")
    if plain and epilogue:
        raise Unmatched("matmul with epilogue: the store is the plain accumulator")

    ta = TileAccess(an, a.args[0], "matmul A")
    tb = TileAccess(an, b.args[0], "matmul B")
    tc = TileAccess(an, c_ptr, "matmul C")
    bm, bk = ta.shape
    bk2, bn = tb.shape
    it = ("iter", loop.uid)
    if ta.step_of(1, "iter") != (it, bk) or tb.step_of(0, "iter") != (it, bk):
        raise Unmatched("matmul: A and B do not advance by BLOCK_K per iteration")
    sm, sn = ta.step_of(0, "pid"), tb.step_of(1, "pid")
    if sm is None or sn is None or sm[1] != bm or sn[1] != bn or sm[0] == sn[0]:
        raise Unmatched("matmul: program ids do not tile M and N by BLOCK_M / BLOCK_N")
    if tc.step_of(0, "pid") != sm or tc.step_of(1, "pid") != sn:
        raise Unmatched("matmul: C is not addressed by the same (row, column) blocks")

    ba = _tile_bounds(an, a.args[1], ta, "matmul A")
    bb = _tile_bounds(an, b.args[1], tb, "matmul B")
    bc = _tile_bounds(an, c_mask, tc, "matmul C")

    plan = GemmPlan()
    plan.a, plan.b, plan.c = ta.base, tb.base, tc.base
    plan.block = (bm, bn, bk)
    plan.pid_m, plan.pid_n = sm[0][1], sn[0][1]
    plan.m_bound = _extent_fn("M", ba.get(0), bc.get(0))
    plan.n_bound = _extent_fn("N", bb.get(1), bc.get(1))
    plan.k_bound = _extent_fn("K", ba.get(1), bb.get(0))
    plan.trips = _trip_count_fn(loop)
    plan.lda, plan.ldb, plan.ldc = (_compile_int(t.stride[0]) for t in (ta, tb, tc))
    plan.inner = tuple((nm, _compile_int(t.stride[1])) for nm, t in
                       ((ta.base, ta), (tb.base, tb), (tc.base, tc)))
    plan.num_stages = num_stages
    plan.row_k = 32 if a.dtype == tp.float32 else 64
    if epilogue:
        return plan, (loop.uid, acc_name), c_ptr, stores[0]
    return plan


class GemmEpiloguePlan(Plan):
    """A matmul k loop whose accumulator goes through more arithmetic before the store (bias,
    activation, scaling, another output type, a row reduction).

    Where that arithmetic is elementwise in the accumulator it is spliced into the tensor-core
    kernel itself, as the reference keeps everything after a k loop in the same kernel
    (newt/compiler/codegen.py:1854-1871): the program's own graph is turned into an epilogue
    functor (frontend/pointwise.py `generate_epilogue`) and the library's device templates
    (csrc/gemm_device.cuh) are compiled with it by NVRTC, one kernel per tile configuration;
    the host half of the launch -- checks, tensor maps, parameter block -- stays in the library
    (`nb200_gemm_plan`).  Nothing but the program's own tensors is touched.

    What cannot run there (a reduction over the tile, operands bulk tensor copies cannot fetch
    as they lie) takes two kernels: the product on the tensor core into an fp32 buffer laid out
    like C (`nb200_gemm_acc32`; fp32 operands: the tf32 entry points), then the rest of the
    program as a generated kernel that reads the accumulator from that buffer -- one extra pass
    over C (4 bytes written and read per element)."""

    kind, entry = "matmul K loop + epilogue", "run-time compiled tcgen05 kernel with the epilogue inside"

    def __init__(self, trace, gemm, acc, c_ptr, num_warps, store):
        self.gemm = gemm
        self.fused_source = None
        self.fused_reason = None
        try:
            text, self.fused_params = pointwise.generate_epilogue(
                trace, acc, store, gemm.block[:2], (gemm.pid_m, gemm.pid_n))
            self.fused_source = text
            self.c_element = c_ptr.dtype.element
            if self.c_element not in (tp.float16, tp.bfloat16, tp.float32):
                raise pointwise.Unsupported(f"C of type {self.c_element.name}")
        except pointwise.Unsupported as why:
            self.fused_source, self.fused_reason = None, str(why)
        self._fused_kernels = {}     # template instance -> nvrtc.Kernel
        self._fused_launches = {}    # (pointers, extents, pitches) -> what nb200_gemm_plan answered
        self._args_type = None
        # The two-kernel route.  Its epilogue streams a BLOCK_M x BLOCK_N tile per program through
        # HBM once; the kernel's num_warps was chosen for the k loop.  Eight elements per thread
        # keep enough loads in flight: up to 32 warps for the tiles a tensor-core matmul uses.
        bm, bn, _ = gemm.block
        warps = num_warps
        while warps < 32 and warps * 32 * 8 < bm * bn:
            warps *= 2
        self._split_args = (trace, warps, {acc: ("nb_acc", c_ptr)})
        self._epilogue = None
        if self.fused_source is None:
            self.epilogue           # compile-time refusals surface when the plan is made
        self._whole = lambda: PointwisePlan(trace, num_warps)    # the program in one generated kernel
        self._whole_plan = None

    @property
    def epilogue(self):
        if self._epilogue is None:
            self._epilogue = PointwisePlan(*self._split_args)
        return self._epilogue

    def describe(self):
        if self.fused_source is not None:
            return "tcgen05 GEMM with the program's epilogue compiled in (NVRTC)"
        return f"nb200_gemm_acc32 + run-time compiled kernel ({self.fused_reason})"

    def hardware_key(self):
        tail = ("fused",) if self.fused_source is not None else (self.epilogue.kernel_name,)
        return ("gemm+epilogue",) + self.gemm.hardware_key() + tail

    # ---- one kernel --------------------------------------------------------------------------

    def _fused_kernel(self, launch, dtype_code, c_code):
        from ..runtime import nvrtc

        key = (launch.pair, launch.block_n, launch.stages, launch.ksub, dtype_code, c_code)
        kernel = self._fused_kernels.get(key)
        if kernel is None:
            codes = {0: "NB200_F32", 1: "NB200_F16", 2: "NB200_BF16"}
            if launch.pair:
                body = (f"nb200::gemm::gemm_pair_body<{launch.stages}, {launch.ksub}, {codes[dtype_code]}, "
                        f"{codes[c_code]}, NbEpilogue, {2 if launch.block_n == 512 else 1}>(ta, tb, p, ea);")
            else:
                body = (f"nb200::gemm::gemm_body<{launch.block_n}, {launch.stages}, {launch.ksub}, "
                        f"{codes[dtype_code]}, "
                        f"{codes[c_code]}, NbEpilogue>(ta, tb, p, ea);")
            name = "nb_gemm_epilogue"
            source = (
                f"// device templates {nvrtc.device_headers_digest()}\n"     # part of the cache key
                '#include "gemm_device.cuh"\n' + self.fused_source +
                f'\nextern "C" __global__ void __launch_bounds__(192, 1) {name}(\n'
                "    const __grid_constant__ CUtensorMap ta, const __grid_constant__ CUtensorMap tb,\n"
                "    const __grid_constant__ nb200::gemm::GemmParams p, const NbEpilogue::Args ea) {\n"
                f"  {body}\n}}\n")
            kernel = nvrtc.Kernel(nvrtc.compile_cubin_cached(source, name + ".cu",
                                                             extra_opts=(f"-I{nvrtc.device_headers()}",)), name)
            kernel.source = source
            self._fused_kernels[key] = kernel
        return kernel

    def _launch_fused(self, grid, args):
        """False when this launch's operands need a copy first (the two-kernel route does that)."""
        import ctypes

        from ..runtime import abi, kernels, nvrtc

        g = self.gemm
        m, n, k = g._extents(grid, args)
        if m == 0 or n == 0:
            return True
        inner = {name: fn(args) for name, fn in g.inner}
        lda, ldb, ldc = g.lda(args), g.ldb(args), g.ldc(args)
        a, b, c = args[g.a], args[g.b], args[g.c]
        if inner[g.c] != 1 or inner[g.a] != 1:
            return False
        b_transposed = inner[g.b] != 1
        if b_transposed and ldb != 1:
            return False
        pitch_b = inner[g.b] if b_transposed else ldb
        # the host half of the launch is a function of the pointers, extents and pitches: the
        # usual case is the same call repeated, which finds its tensor maps and parameters here
        key = (a.data_ptr(), b.data_ptr(), c.data_ptr(), a.dtype, c.dtype, m, n, k, lda, pitch_b, ldc,
               b_transposed)
        planned = self._fused_launches.get(key)
        if planned is None:
            lib = abi.load()
            tma, tmb = nvrtc.new_tensor_map(), nvrtc.new_tensor_map()
            params = (ctypes.c_char * int(lib.nb200_gemm_params_bytes()))()
            launch = abi.GemmLaunch()
            cfg = g.config()
            dtype_code, c_code = abi.dtype_code(a.dtype), abi.dtype_code(c.dtype)
            rc = lib.nb200_gemm_plan(
                kernels._dev_ptr(g.a, a), kernels._dev_ptr(g.b, b), kernels._dev_ptr(g.c, c), m, n, k,
                lda, pitch_b, ldc, dtype_code, c_code, 1 if b_transposed else 0, ctypes.byref(cfg),
                ctypes.byref(tma), ctypes.byref(tmb), ctypes.byref(params), ctypes.byref(launch))
            if rc == abi.E_UNSUPPORTED:
                return False          # a pitch or base bulk tensor copies cannot fetch
            abi.check(rc)
            kernel = None if (launch.nothing or launch.only_clear) else \
                self._fused_kernel(launch, dtype_code, c_code)
            if len(self._fused_launches) >= 64:
                self._fused_launches.clear()
            planned = self._fused_launches[key] = (tma, tmb, params, launch, kernel)
        tma, tmb, params, launch, kernel = planned
        if launch.nothing:
            return True
        if launch.only_clear:
            return False          # K == 0: the generated kernel applies the epilogue to zeros
        if self._args_type is None:
            self._args_type = pointwise.struct_type(self.fused_params)
        ea = pointwise.marshal_struct(self.fused_params, args, self._args_type)
        kernel.launch((launch.grid,), launch.block, [tma, tmb, params, ea], kernels.raw_stream(),
                      launch.smem_bytes, cluster=launch.cluster if launch.cluster > 1 else None)
        return True

    # ---- launch -----------------------------------------------------------------------------------

    def launch(self, grid, args):
        import torch

        from ..runtime import abi

        if self.fused_source is not None and self._launch_fused(grid, args):
            return
        c = args[self.gemm.c]
        m, n, _ = self.gemm._extents(grid, args)
        if m == 0 or n == 0:
            return
        ldc = self.gemm.ldc(args)
        # The fp32 buffer comes from torch's caching allocator per launch: it is allocated,
        # written and read on the current stream, so launches on different streams never share
        # one, and the allocator reuses the block on this stream without touching the driver.
        buf = torch.empty(max((m - 1) * ldc + n, 1), dtype=torch.float32, device=c.device)
        try:
            self.gemm._launch_tensor_core(grid, args, acc32=buf)
        except (CompileError, abi.UnsupportedError) as e:
            # a layout the tensor-core path does not take (C not unit-stride along its rows);
            # decided per launch, the one-kernel plan is compiled once and kept
            if self._whole_plan is None:
                try:
                    self._whole_plan = self._whole()
                except pointwise.Unsupported as second:
                    raise CompileError(f"{e}; and the generic lowering does not take the program "
                                       f"either: {second}") from e
            return self._whole_plan.launch(grid, args)
        self.epilogue.launch(grid, {**args, "nb_acc": buf})


# --------------------------------------------------------------------------- attention

class AttentionPlan(Plan):
    kind, entry = "flash attention loop", "nb200_attention_fwd"

    def __init__(self):
        self.q = self.k = self.v = self.o = None
        self.block_m = 0
        self.pid_m = 0
        self.pid_head = None
        self.seq_q = self.seq_kv = None
        self.d = 0
        self.scale = None          # parameter name or float
        self.causal = False
        self.strides = {}          # tensor -> (head stride fn | None, row stride fn, inner stride fn)

    def launch(self, grid, args):
        import torch

        from ..runtime import kernels

        gm = grid[self.pid_m] if self.pid_m < len(grid) else 1
        bh = 1
        if self.pid_head is not None:
            bh = grid[self.pid_head] if self.pid_head < len(grid) else 1
        seq_q = gm * self.block_m
        if self.seq_q is not None:
            seq_q = min(seq_q, self.seq_q(args))
        seq_kv = self.seq_kv(args)
        if seq_q <= 0 or bh <= 0:
            return
        scale = args[self.scale] if isinstance(self.scale, str) else self.scale
        views = {}
        for name, seq in ((self.q, seq_q), (self.k, seq_kv), (self.v, seq_kv), (self.o, seq_q)):
            hs, rs, inner = self.strides[name]
            if inner(args) != 1:
                raise CompileError(f"attention: '{name}' is not unit-stride along head_dim")
            # a single head needs no head stride; give TMA the natural one
            head_stride = hs(args) if hs is not None else rs(args) * seq
            views[name] = torch.as_strided(args[name], (bh, seq, self.d),
                                           (head_stride, rs(args), 1),
                                           args[name].storage_offset())
        kernels.attention_fwd(views[self.q], views[self.k], views[self.v], views[self.o], scale,
                              self.causal)


def _carried_by_placeholder(loop):
    return {ph.uid: (name, init, nxt) for name, (ph, init, nxt) in loop.carried.items()}


def lower_attention(trace, an, num_stages):
    loops, stores = _loops(trace), _top_level_stores(trace)
    if len(loops) != 1 or len(stores) != 1:
        raise Unmatched("attention: expected one KV loop followed by one store")
    loop = loops[0]
    if loop.effects:
        raise Unmatched("attention: the KV loop has side effects")
    by_ph = _carried_by_placeholder(loop)
    accs = [(n, v) for n, v in loop.carried.items() if v[2].op == "dot"]
    if len(accs) != 1 or len(loop.carried) != 3:
        raise Unmatched("attention: the loop must carry exactly (m_i, l_i, acc)")
    acc_name, (acc_ph, acc_init, pv) = accs[0]

    neg_inf = float("-inf")
    q, k, v = (Cap(n, lambda x: isinstance(x, Node) and x.op == "load") for n in "qkv")
    qkm = Pat("where", [Cap("keep"), p_bin("mul", Pat("dot", [q, Pat("trans", [k]), None]),
                                             Cap("scale")), p_const(neg_inf)])
    m_ph = Cap("m_ph", lambda x: isinstance(x, Node) and x.op == "carried")
    m_new = p_bin("max", m_ph, Pat("reduce", [qkm], fn="max", axis=1))
    alpha = p_math("exp", p_bin("sub", m_ph, m_new))
    prob = p_math("exp", p_bin("sub", qkm, Pat("expand", [m_new], axis=1)))
    pv_pat = Pat("dot", [Pat("cast", [prob]), v,
                         p_bin("mul", Cap("acc_ph"), Pat("expand", [alpha], axis=1))])
    caps = {}
    if not match(pv_pat, pv, caps):
        raise Unmatched("attention: the accumulator update is not "
                        "dot(exp(qk - m_new).to(dtype), v, acc * exp(m_i - m_new))")
    if caps["acc_ph"] is not acc_ph:
        raise Unmatched("attention: the rescaled block is not the carried accumulator")
    m_name, m_init, m_next = by_ph[caps["m_ph"].uid]
    l_entries = [(n, v) for n, v in loop.carried.items() if n not in (acc_name, m_name)]
    l_name, (l_ph, l_init, l_next) = l_entries[0]
    c2 = dict(caps)
    if not match(m_new, m_next, c2):
        raise Unmatched("attention: m_i is not updated to maximum(m_i, max(qk))")
    c3 = dict(caps)
    c3["l_ph"] = l_ph
    if not match(p_bin("add", p_bin("mul", Cap("l_ph"), alpha),
                       Pat("reduce", [prob], fn="sum", axis=1)), l_next, c3):
        raise Unmatched("attention: l_i is not updated to l_i * alpha + sum(p)")
    if not (m_init.op == "full" and m_init.args[0] == neg_inf and l_init.op == "full"
            and l_init.args[0] == 0 and acc_init.op == "full" and acc_init.args[0] == 0):
        raise Unmatched("attention: running state must start at (-inf, 0, 0)")

    _, o_ptr, o_val, o_mask, _ = stores[0]
    want = p_bin("div", Pat("loopout", [], loop=loop.uid, name=acc_name),
                 Pat("expand", [Pat("loopout", [], loop=loop.uid, name=l_name)], axis=1))
    if not match(want, o_val, {}):
        raise Unmatched("attention: the stored value is not acc / l_i")

    ql, kl, vl = caps["q"], caps["k"], caps["v"]
    dt = ql.dtype
    if dt not in (tp.float16, tp.bfloat16) or kl.dtype != dt or vl.dtype != dt \
            or o_ptr.dtype.element != dt or pv.args[0].dtype != dt:
        raise Unmatched("attention: q, k, v, p and out must share float16 or bfloat16")
    for ld, nm in ((ql, "q"), (kl, "k"), (vl, "v")):
        if ld.args[1] is not None and ld.args[2] not in (None, 0, 0.0):
            raise Unmatched(f"attention: masked lanes of {nm} must read 0")

    tq = TileAccess(an, ql.args[0], "attention Q", allow_batch=True)
    tk = TileAccess(an, kl.args[0], "attention K", allow_batch=True)
    tv = TileAccess(an, vl.args[0], "attention V", allow_batch=True)
    to = TileAccess(an, o_ptr, "attention O", allow_batch=True)
    bm, d = tq.shape
    bn = tk.shape[0]
    if tk.shape[1] != d or tv.shape != (bn, d) or to.shape != (bm, d):
        raise Unmatched("attention: tile shapes are inconsistent")
    if d not in (64, 128):
        raise Unmatched(f"attention: head_dim {d} has no kernel (64 and 128 only)")
    it = ("iter", loop.uid)
    sm = tq.step_of(0, "pid")
    if sm is None or sm[1] != bm or to.step_of(0, "pid") != sm:
        raise Unmatched("attention: program_id does not tile the query rows by BLOCK_M")
    for t, nm in ((tk, "K"), (tv, "V")):
        if t.step_of(0, "iter") != (it, bn):
            raise Unmatched(f"attention: {nm} does not advance by BLOCK_N rows per iteration")
    for t in (tq, tk, tv, to):
        if not t.origin[1].is_zero():
            raise Unmatched("attention: head_dim must be addressed from 0")
    heads = {t.batch[0] for t in (tq, tk, tv, to) if t.batch is not None}
    if len(heads) > 1 or (heads and any(t.batch is None for t in (tq, tk, tv, to))):
        raise Unmatched("attention: q, k, v and out must share one batch*head index")

    # masks: key bound and causal term
    kv_bounds, causal = [], False
    for term in _split_and(caps["keep"]):
        fn, dpoly = _comparison(an, term, "attention mask")
        if len(term.shape) < 2:
            raise Unmatched("attention: score mask is not 2-D")
        has0, has1 = ("ax", 0) in dpoly.atoms(), ("ax", 1) in dpoly.atoms()
        if has1 and not has0 and fn == "lt":
            qd, rest = dpoly.coeff_of(("ax", 1))
            moving = Poly({m: c for m, c in rest.terms.items() if any(a[0] != "param" for a in m)})
            if qd.const_value() != 1 or moving != tk.origin[0]:
                raise Unmatched("attention: key mask bounds a different index than K uses")
            kv_bounds.append(-(rest - moving))
        elif has0 and has1:
            # offs_n[None, :] <= offs_m[:, None]   (or the mirrored >=)
            expect = Poly.atom(("ax", 1)) + tk.origin[0] - Poly.atom(("ax", 0)) - tq.origin[0]
            if (fn == "le" and dpoly == expect) or (fn == "ge" and dpoly == -expect):
                causal = True
            else:
                raise Unmatched("attention: only the causal mask `key index <= query index` "
                                "is supported")
        else:
            raise Unmatched("attention: unsupported score mask term")
    if len(kv_bounds) != 1:
        raise Unmatched("attention: scores must be masked by `key index < N` exactly once")
    seq_kv = kv_bounds[0]
    kb = _tile_bounds(an, kl.args[1], tk, "attention K").get(0, [seq_kv])
    vb = _tile_bounds(an, vl.args[1], tv, "attention V").get(0, [seq_kv])
    if any(b != seq_kv for b in kb + vb):
        raise Unmatched("attention: K/V load masks and the score mask disagree on N")
    qb = _tile_bounds(an, ql.args[1], tq, "attention Q").get(0, [])
    ob = _tile_bounds(an, o_mask, to, "attention O").get(0, [])

    # loop range: 0 .. N step BLOCK_N, or 0 .. min(N, (pid + 1) * BLOCK_M) when causal
    try:
        if an.poly(loop.lo) != Poly.const(0) or an.poly(loop.step) != Poly.const(bn):
            raise Unmatched("attention: the KV loop must be range(0, hi, BLOCK_N)")
    except NotAffine:
        raise Unmatched("attention: the KV loop bounds are not affine")
    hi_ok = False
    hi = loop.hi
    try:
        hi_ok = an.poly(hi) == seq_kv
    except NotAffine:
        pass
    if not hi_ok and causal and isinstance(hi, Node) and hi.op == "bin" \
            and dict(hi.attrs)["fn"] == "min":
        diag = (Poly.atom(sm[0]) + Poly.const(1)) * Poly.const(bm)
        try:
            sides = [an.poly(x) for x in hi.args]
            hi_ok = seq_kv in sides and diag in sides
        except NotAffine:
            pass
    if not hi_ok:
        raise Unmatched("attention: the KV loop must cover keys [0, N) (or stop at the "
                        "diagonal block when causal)")

    sc = caps["scale"]
    plan = AttentionPlan()
    if _param_name(sc) is not None:
        plan.scale = _param_name(sc)
    elif isinstance(sc, Node) and sc.op == "const":
        plan.scale = float(sc.args[0])
    else:
        raise Unmatched("attention: scale must be an argument or a literal")
    plan.q, plan.k, plan.v, plan.o = tq.base, tk.base, tv.base, to.base
    plan.block_m, plan.d, plan.causal = bm, d, causal
    plan.pid_m = sm[0][1]
    plan.pid_head = next(iter(heads))[1] if heads else None
    plan.seq_q = _extent_fn("query", qb, ob)
    plan.seq_kv = _compile_int(seq_kv)
    for t in (tq, tk, tv, to):
        plan.strides[t.base] = (_compile_int(t.batch[1]) if t.batch else None,
                                _compile_int(t.stride[0]), _compile_int(t.stride[1]))
    return plan


# --------------------------------------------------------------------------- driver

_RECOGNISERS = []


class PointwisePlan(Plan):
    """A program that is none of the tuned ones: generated CUDA, compiled by NVRTC for sm_100a
    on first launch, one CUDA block per program instance (frontend/pointwise.py)."""

    kind, entry = "block arithmetic", "run-time compiled kernel (NVRTC, sm_100a)"

    def __init__(self, trace, num_warps, computed_elsewhere=None):
        self.num_warps = num_warps
        self.source, self.kernel_name, self.params, self.shared_bytes = \
            pointwise.generate(trace, num_warps, computed_elsewhere)
        self._kernel = None

    def hardware_key(self):
        return ("pointwise", self.kernel_name, self.num_warps)

    def launch(self, grid, args):
        from ..runtime import kernels, nvrtc

        if self._kernel is None:
            self._kernel = nvrtc.Kernel(
                nvrtc.compile_cubin_cached(self.source, self.kernel_name + ".cu"), self.kernel_name)
        self._kernel.launch(grid, self.num_warps * 32, pointwise.marshal(self.params, args),
                            kernels.raw_stream(), self.shared_bytes)


def _lower_gemm_epilogue(trace, an, num_stages, num_warps):
    gemm, acc, c_ptr, store = lower_gemm(trace, an, num_stages, epilogue=True)
    try:
        return GemmEpiloguePlan(trace, gemm, acc, c_ptr, num_warps, store)
    except pointwise.Unsupported as e:
        raise Unmatched(f"matmul with epilogue: {e}")


def lower(trace, num_warps=4, num_stages=3):
    """Picks the launch plan for a traced kernel or raises CompileError."""
    an = Analyzer(trace)
    an.resolve_inductions()
    reasons = []
    attempts = [("add", lambda: lower_add(trace, an)),
                ("softmax", lambda: lower_softmax(trace, an)),
                ("layernorm", lambda: lower_layernorm(trace, an)),
                ("tile softmax", lambda: lower_softmax_tile(trace, an)),
                ("tile layernorm", lambda: lower_layernorm_tile(trace, an)),
                ("matmul", lambda: lower_gemm(trace, an, num_stages)),
                ("matmul with epilogue", lambda: _lower_gemm_epilogue(trace, an, num_stages, num_warps)),
                ("attention", lambda: lower_attention(trace, an, num_stages))]
    attempts += [(n, (lambda f=f: f(trace, an, num_stages))) for n, f in _RECOGNISERS]
    if any(e[0] == "atomic" for e in trace.effects):
        attempts = []        # none of the tuned programs updates memory atomically
    def generic():
        try:
            return PointwisePlan(trace, num_warps)
        except pointwise.Unsupported as e:
            raise CompileError(f"{trace.name}: {e}") from e

    for name, attempt in attempts:
        try:
            plan = attempt()
            if isinstance(plan, GemmPlan):
                plan.generic = generic
            return plan
        except Unmatched as e:
            reasons.append(str(e))
        except NotAffine as e:
            reasons.append(f"{name}: address arithmetic is not affine ({e})")
    # not one of the tuned programs: compiled at run time by the generic lowering
    try:
        return PointwisePlan(trace, num_warps)
    except pointwise.Unsupported as e:
        reasons.append(f"generic lowering: {e}")
    raise CompileError(
        f"{trace.name}: no sm_100a kernel implements this program yet (the generic lowering "
        f"refused it as well).  Closest matches:\n  - "
        + "\n  - ".join(reasons))
