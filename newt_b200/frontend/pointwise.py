"""Generic lowering of block programs to CUDA text.

Everything the block language can say that is not one of the tuned programs -- arithmetic on
blocks of compile-time shape, loads through pointer blocks, broadcasting, `nl.where`, casts,
`nl.sum / max / min`, atomics, masked stores, runtime `for` / `while` loops, `nl.dot` on shapes
or layouts no tensor-core tile takes -- is compiled at run time, like the reference compiles
all programs: one CUDA block of `num_warps * 32` threads per program instance.

* For each `nl.store` (or atomic) the threads stride over the elements of the stored block and
  evaluate the expression for their element, on demand, from the leaves.
* A reduction is computed first, by the whole block, into shared memory, and read from there.
* A runtime loop that only computes (no store, no reduction that changes per iteration) is run
  privately by each thread for the element it is working on: carried values are registers.
* Any other runtime loop is a C loop that all threads run together: carried scalars are
  registers (every thread computes the same value), a carried block that moves by one scalar
  per iteration (`ptrs += BLOCK_K * stride`) is its first value plus a running offset, other
  carried blocks live in shared memory and are updated in place when element e only reads
  element e, through a staging copy otherwise.
* `nl.dot` is summed per output element on the CUDA cores (fp32 accumulation; fp32 operands
  rounded to tf32 first).  The matmul and attention programs never come here unless their
  operands are laid out so that bulk tensor copies cannot fetch them.

Numerics follow the reference's elementwise rules (newt/compiler/codegen.py:1196-1284,
2011-2030): fp16 / bf16 operations are computed in fp32 and rounded back after every
operation; Python constants were already given the dtype of the block they meet by the
tracer; integer `/` is C division; math functions are the precise single-precision ones
(`expf`, `rsqrtf`, ...), no fast-math.  Control flow follows newt/compiler/codegen.py:993-1105
(`visit_For`, `visit_While`, `visit_If`, `visit_Break`, `visit_Continue`).
"""

import ctypes
import hashlib
import math
import re

from .. import types as tp
from .trace import Node

THREADS_PER_WARP = 32


class Unsupported(Exception):
    """The trace contains something this lowering does not handle."""


_F32 = tp.float32


def _is_half(dt):
    return dt in (tp.float16, tp.bfloat16)


def _literal(value, dt):
    if dt == tp.int1:
        return "true" if value else "false"
    if dt.is_int:
        v = int(value)
        return f"{v}LL" if dt.itemsize == 8 else (f"{v}u" if dt.kind == "u" else f"{v}")
    v = float(value)
    if math.isnan(v):
        text = "__int_as_float(0x7fc00000)"
    elif math.isinf(v):
        text = "__int_as_float(0x7f800000)" if v > 0 else "__int_as_float(0xff800000)"
    else:
        text = repr(v)
        if "e" not in text and "." not in text:
            text += ".0"
        if dt != tp.float64:
            text += "f"
    if dt == tp.float64:
        return text if text[-1] != "f" else f"(double){text}"
    if dt == tp.float16:
        return f"__float2half_rn({text})"
    if dt == tp.bfloat16:
        return f"__float2bfloat16_rn({text})"
    return text


# One fp32 value rounded to a 16-bit float (round to nearest even, as `__float2half_rn` /
# `__float2bfloat16_rn`) with the two-lane conversion instruction, the other lane fed a zero: on
# sm_100a the scalar `cvt.rn.bf16.f32` issues at a fraction of the rate of `cvt.rn.bf16x2.f32`,
# and a chain of 16-bit operations rounds after every one of them.
_ROUNDING_HELPERS = """
static __device__ __forceinline__ __half nb_to_f16(float x) { return __low2half(__floats2half2_rn(x, 0.0f)); }
static __device__ __forceinline__ __nv_bfloat16 nb_to_bf16(float x) {
  return __low2bfloat16(__floats2bfloat162_rn(x, 0.0f));
}
"""


def _convert(expr, src, dst):
    """C expression converting `expr` of dtype `src` to `dst`."""
    if src == dst:
        return expr
    if _is_half(src):
        as_float = f"__half2float({expr})" if src == tp.float16 else f"__bfloat162float({expr})"
        return as_float if dst == _F32 else _convert(as_float, _F32, dst)
    if dst == tp.float16:
        return f"nb_to_f16({_convert(expr, src, _F32)})"
    if dst == tp.bfloat16:
        return f"nb_to_bf16({_convert(expr, src, _F32)})"
    if dst == tp.int1:
        return f"(({expr}) != 0)"
    return f"(({dst.ctype})({expr}))"


_MATH = {"exp": "expf", "exp2": "exp2f", "log": "logf", "log2": "log2f", "sqrt": "sqrtf",
         "rsqrt": "rsqrtf", "sin": "sinf", "cos": "cosf", "tanh": "tanhf", "erf": "erff",
         "floor": "floorf", "ceil": "ceilf", "abs": "fabsf"}
_INFIX = {"add": "+", "sub": "-", "mul": "*", "and": "&", "or": "|", "xor": "^", "shl": "<<",
          "shr": ">>"}
_CMP = {"lt": "<", "le": "<=", "gt": ">", "ge": ">=", "eq": "==", "ne": "!="}


class _Context:
    """What all statement lists of one kernel share."""

    def __init__(self, trace, threads):
        self.trace = trace
        self._analyzer = None
        self._unit = {}        # pointer node uid -> does it advance by one element along its last axis
        self.loops = {loop.uid: loop for loop in trace.loops}
        self.live = _live_names(trace)
        self.threads = threads
        self.reduced = {}      # reduce node uid -> (shared array, result shape)
        self.final = {}        # (loop uid, carried name) -> where a finished block-level loop left it
        self.depends = {}      # (node uid, loop uid) -> bool
        self.pure = {}         # loop uid -> bool
        self.helpers = set()
        self.staging = set()   # nodes whose shared-memory copy is being written right now
        self.arrays = []       # (name, dtype, count, byte offset) in shared memory
        self.shared_bytes = 0
        self.counter = 0
        self.program_ids = {}  # grid axis -> C expression, when the code does not run one CUDA
                               # block per program instance

    def fresh(self, prefix="v"):
        self.counter += 1
        return f"{prefix}{self.counter}"

    def either(self, wide, narrow):
        """The eight-lane form of a statement list when every 16-bit tensor of the launch starts
        on a 16-byte boundary (one test per kernel: `nb_wide`), else the one-element form -- from
        a base that is off, every 16-byte access would fall back lane by lane, which is slower
        than never having formed the lanes."""
        self.wide_used = True
        out = ["if (nb_wide) {"]
        for lines in (wide, narrow):
            lines = list(lines)
            if lines and lines[-1] == "__syncthreads();":
                lines.pop()
            out += ["  " + ln for ln in lines]
            out.append("} else {")
        out[-1] = "}"
        out.append("__syncthreads();")
        return out

    def wide_declaration(self):
        if not self.wide_used:
            return []
        names = [name for name, node in self.trace.params.items()
                 if isinstance(node.dtype, tp.pointer_type)
                 and (self.wide_all or node.dtype.element.itemsize == 2)]
        test = " | ".join(f"(unsigned long long){n}" for n in names)
        return [f"const bool nb_wide = (({test}) & 15ull) == 0;"]

    wide_used = False
    wide_all = False       # the test covers every tensor, not only the 16-bit ones

    def unit_stride(self, ptr):
        """True when the pointer block is affine in the block's indices and neighbours along its
        last axis are neighbours in memory (the proof vector accesses need)."""
        hit = self._unit.get(ptr.uid)
        if hit is None:
            from .affine import Analyzer, NotAffine, Poly
            if self._analyzer is None:
                self._analyzer = Analyzer(self.trace)
            hit = False
            try:
                split = self._analyzer.poly(ptr).coeff_of(("ax", len(ptr.shape) - 1))
                hit = bool(ptr.shape) and split is not None and split[0] == Poly.const(1)
            except NotAffine:
                pass
            self._unit[ptr.uid] = hit
        return hit

    def mask_deciders(self, mask):
        """The lanes of a group whose mask values decide the conjunction over the whole group:
        a subset of {"first", "last"}, or None when every lane has to be looked at.  `offs < n`
        with offs rising by one per lane holds for all lanes when it holds for the last."""
        from .affine import NotAffine, Poly
        if not isinstance(mask, Node):
            return None
        if not mask.shape or mask.shape[-1] == 1:
            return {"first"}                      # the same value in every lane
        if mask.op in ("broadcast", "splat"):
            inner = mask.args[0]
            if not isinstance(inner, Node) or not inner.shape or inner.shape[-1] == 1:
                return {"first"}
            return self.mask_deciders(inner) if inner.shape[-1] == mask.shape[-1] else None
        if mask.op == "expand":
            if dict(mask.attrs)["axis"] == len(mask.shape) - 1:
                return {"first"}                  # the new axis is the lanes' one
            return self.mask_deciders(mask.args[0])
        if mask.op == "bin" and dict(mask.attrs)["fn"] == "and":
            both = [self.mask_deciders(a) for a in mask.args]
            return None if None in both else both[0] | both[1]
        if mask.op != "cmp":
            return None
        fn = dict(mask.attrs)["fn"]
        if self._analyzer is None:
            from .affine import Analyzer
            self._analyzer = Analyzer(self.trace)
        try:
            pa, pb = self._analyzer._aligned(mask.args[0], mask.args[1], len(mask.shape))
            split = (pa - pb).coeff_of(("ax", len(mask.shape) - 1))
        except NotAffine:
            return None
        if split is None or not split[0].is_const():
            return None
        rise = split[0].const_value()             # change of a - b from one lane to the next
        if rise == 0:
            return {"first"}
        if fn in ("lt", "le"):
            return {"last"} if rise > 0 else {"first"}
        if fn in ("gt", "ge"):
            return {"first"} if rise > 0 else {"last"}
        return None

    def alloc(self, dt, count, prefix):
        """A shared-memory array of `count` elements; returns its name."""
        name = f"{prefix}{len(self.arrays)}"
        offset = (self.shared_bytes + 15) // 16 * 16
        size = 8 if isinstance(dt, tp.pointer_type) else dt.itemsize
        self.shared_bytes = offset + max(count, 1) * size
        if self.shared_bytes > _SHARED_LIMIT:
            raise Unsupported(f"the blocks kept across iterations and the reductions need "
                              f"{self.shared_bytes} bytes of shared memory; a CTA has {_SHARED_LIMIT}")
        self.arrays.append((name, dt, count, offset))
        return name

    def shared_declarations(self):
        """Declarations of the shared arrays, and the dynamic shared memory to launch with."""
        if not self.arrays and "reduce" not in self.helpers:
            return [], 0
        lines = ["__shared__ unsigned long long nb_scratch[32];"]
        dynamic = 0
        if self.arrays:
            if self.shared_bytes + 256 <= _STATIC_SHARED_LIMIT:
                lines.append(f"__shared__ __align__(16) unsigned char nb_shared[{self.shared_bytes}];")
            else:
                lines.append("extern __shared__ __align__(16) unsigned char nb_shared[];")
                dynamic = self.shared_bytes
        for name, dt, _, offset in self.arrays:
            lines.append(f"{dt.ctype}* const {name} = reinterpret_cast<{dt.ctype}*>(nb_shared + {offset});")
        return lines, dynamic


class _Body:
    """Statements that compute one element of one store (or one pass of a loop body)."""

    def __init__(self, ctx, loop_state=None):
        self.ctx = ctx
        self.lines = []
        self.memo = {}
        self.reduced = ctx.reduced
        # (loop uid, carried name) -> variable holding its current value; (loop uid, None) -> the
        # loop variable
        self.loop_state = dict(loop_state or {})
        self.loop_final = {}    # (loop uid, name) -> offset form left by a loop emitted in this body
        self.lanes = 0          # > 0: each trip computes this many neighbours along the last axis,
                                # whose index is written `(nb_v + k)` for lane k

    def var(self, dt, expr):
        name = self.ctx.fresh()
        if isinstance(dt, tp.pointer_type):
            self.lines.append(f"{dt.ctype} const {name} = {expr};")
        else:
            self.lines.append(f"const {dt.ctype} {name} = {expr};")
        return name


def _operand_dims(node_shape, dims, operand_shape):
    """Index expressions of an operand that broadcasts into a node with `dims`."""
    r = len(operand_shape)
    if r == 0:
        return ()
    tail = dims[len(dims) - r:]
    return tuple("0" if operand_shape[i] == 1 and node_shape[len(node_shape) - r + i] != 1
                 else tail[i] for i in range(r))


def _emit(body, node, dims):
    if not isinstance(node, Node):
        raise Unsupported(f"non-node operand {node!r}")
    if node.op != "reduce" and node.uid in body.reduced and node.uid not in body.ctx.staging:
        array, shape = body.reduced[node.uid]     # staged in shared memory by the scheduler
        return f"{array}[{_linear(dims, shape)}]"
    key = (node.uid, dims)
    hit = body.memo.get(key)
    if hit is not None:
        return hit
    out = _emit_new(body, node, dims)
    body.memo[key] = out
    return out


def _compute_type(dt):
    return _F32 if _is_half(dt) else dt


def _emit_new(body, node, dims):
    op, dt = node.op, node.dtype
    at = dict(node.attrs)

    def sub(x, shape=None):
        return _emit(body, x, _operand_dims(node.shape, dims, x.shape if shape is None else shape))

    if op == "param":
        return at["name"]
    if op == "const":
        return _literal(node.args[0], dt)
    if op == "full":
        return _literal(node.args[0], dt)
    if op == "pid":
        named = body.ctx.program_ids.get(at["axis"])      # an epilogue spliced into another kernel
        return named if named is not None else f"(int)blockIdx.{'xyz'[at['axis']]}"
    if op == "nprog":
        if body.ctx.program_ids:
            raise Unsupported("nl.num_programs in code spliced into the matmul kernel")
        return f"(int)gridDim.{'xyz'[at['axis']]}"
    if op == "arange":
        return f"({int(node.args[0])} + {dims[0]})"
    if op == "splat":
        return sub(node.args[0])
    if op == "broadcast":
        return sub(node.args[0])
    if op == "expand":
        child = node.args[0]
        axis = at["axis"]
        return _emit(body, child, dims[:axis] + dims[axis + 1:])
    if op == "trans":
        return _emit(body, node.args[0], (dims[1], dims[0]))
    if op == "reshape":
        # same elements in row-major order: linear index here -> indices of the operand
        child = node.args[0]
        lin = "0"
        for d, extent in enumerate(node.shape):
            lin = f"({lin} * {extent} + {dims[d]})"
        lin = body.var(tp.int32, lin)
        cdims, rem = [], lin
        for d in range(len(child.shape) - 1, 0, -1):
            cdims.append(body.var(tp.int32, f"{rem} % {child.shape[d]}"))
            rem = body.var(tp.int32, f"{rem} / {child.shape[d]}")
        if child.shape:
            cdims.append(rem)
        return _emit(body, child, tuple(reversed(cdims)))
    if op == "cast":
        x = node.args[0]
        return body.var(dt, _convert(sub(x), x.dtype, dt))
    if op in ("ptradd", "ptrsub"):
        ptr, off = node.args
        sign = "+" if op == "ptradd" else "-"
        return body.var(dt, f"{sub(ptr)} {sign} (long long)({sub(off)})")
    if op == "load":
        ptr, mask, other = node.args
        if body.lanes:
            packed = _emit_lanes_load(body, node, dims)
            if packed is not None:
                return packed
        p = sub(ptr)
        if mask is None:
            return body.var(dt, f"*{p}")
        fill = _literal(other if other is not None else 0, dt) if not isinstance(other, Node) \
            else _convert(sub(other), other.dtype, dt)
        return body.var(dt, f"{sub(mask)} ? *{p} : {fill}")
    if op == "neg":
        x = node.args[0]
        cd = _compute_type(dt)
        return body.var(dt, _convert(f"(-{_convert(sub(x), x.dtype, cd)})", cd, dt))
    if op == "not":
        return body.var(dt, f"!{sub(node.args[0])}")
    if op == "inv":
        return body.var(dt, f"~{sub(node.args[0])}")
    if op == "where":
        c, a, b = node.args
        return body.var(dt, f"{sub(c)} ? {_convert(sub(a), a.dtype, dt)} : {_convert(sub(b), b.dtype, dt)}")
    if op == "cmp":
        a, b = node.args
        cd = _compute_type(tp.promote(a.dtype, b.dtype))
        return body.var(dt, f"{_convert(sub(a), a.dtype, cd)} {_CMP[at['fn']]} {_convert(sub(b), b.dtype, cd)}")
    if op == "math":
        x = node.args[0]
        fn = at["fn"]
        cd = _compute_type(dt)
        arg = _convert(sub(x), x.dtype, cd)
        if cd.is_int:
            if fn != "abs":
                raise Unsupported(f"nl.{fn} on integers")
            expr = f"({arg} < 0 ? -{arg} : {arg})"
        elif fn == "sigmoid":
            one = "1.0" if cd == tp.float64 else "1.0f"
            e = "exp" if cd == tp.float64 else "expf"
            expr = f"{one} / ({one} + {e}(-{arg}))"
        else:
            name = _MATH[fn]
            if cd == tp.float64:
                name = name[:-1] if fn != "abs" else "fabs"
            expr = f"{name}({arg})"
        return body.var(dt, _convert(f"({expr})", cd, dt))
    if op == "bin":
        a, b = node.args
        fn = at["fn"]
        cd = _compute_type(dt)
        x, y = _convert(sub(a), a.dtype, cd), _convert(sub(b), b.dtype, cd)
        if fn in _INFIX:
            if fn in ("and", "or", "xor", "shl", "shr") and not cd.is_int:
                raise Unsupported(f"bitwise '{fn}' on floats")
            expr = f"{x} {_INFIX[fn]} {y}"
        elif fn == "div":
            expr = f"{x} / {y}"
        elif fn == "floordiv":
            expr = f"{x} / {y}" if cd.is_int else f"{'floor' if cd == tp.float64 else 'floorf'}({x} / {y})"
        elif fn == "mod":
            expr = f"{x} % {y}" if cd.is_int else f"{'fmod' if cd == tp.float64 else 'fmodf'}({x}, {y})"
        elif fn == "pow":
            if b.op == "const" and b.args[0] == 2:     # x ** 2 is x * x (codegen.py:1254-1256)
                expr = f"{x} * {x}"
            elif cd.is_int:
                raise Unsupported("integer ** needs the constant exponent 2")
            else:
                expr = f"{'pow' if cd == tp.float64 else 'powf'}({x}, {y})"
        elif fn in ("max", "min"):
            if cd.is_int:
                expr = f"({x} {'>' if fn == 'max' else '<'} {y} ? {x} : {y})"
            else:
                f = "f" + fn
                expr = f"{f if cd == tp.float64 else f + 'f'}({x}, {y})"
        elif fn == "cdiv":
            expr = f"({x} + {y} - 1) / {y}"
        else:
            raise Unsupported(f"operator '{fn}'")
        return body.var(dt, _convert(f"({expr})", cd, dt))
    if op == "loopvar":
        name = body.loop_state.get((at["loop"], None))
        if name is None:
            raise Unsupported("a loop variable is used outside its loop")
        return name
    if op == "carried":
        st = body.loop_state.get((at["loop"], at["name"]))
        if st is None:
            raise Unsupported(f"loop-carried '{at['name']}' is used outside its loop")
        return _state_value(body, st, node, dims)
    if op == "loopout":
        key = (at["loop"], at["name"])
        st = body.ctx.final.get(key) or body.loop_final.get(key)
        if st is not None:
            return _state_value(body, st, node, dims)
        hit = body.memo.get(("loopout",) + key + (dims,))
        return hit if hit is not None else _emit_loop(body, node, dims)
    if op == "dot":
        return _emit_dot(body, node, dims)
    if op == "reduce":
        slot = body.reduced.get(node.uid)
        if slot is None:
            raise Unsupported("a reduction inside a reduction's own operand chain was not materialised")
        name, shape = slot
        return f"{name}[{_linear(dims, shape)}]"
    raise Unsupported(f"'{op}' has no elementwise lowering")



# ---- sixteen bytes at a time ---------------------------------------------------------------
#
# 16-bit tensors: a thread that loads and stores one element per access moves two bytes per
# instruction and the memory pipeline, not HBM, sets the pace (4.6 TB/s for relu(2x + y) where
# fp32 reaches the copy rate).  When the stored block's last axis is a multiple of eight and its
# pointer advances by one element along it, an element loop trip computes eight neighbours
# ("lanes"): index `(nb_v + k)` for lane k.  A load whose pointer is proven unit-stride along
# the same axis fetches its eight lanes with one 16-byte access when, at run time, the address
# is 16-byte aligned and all eight masks hold, and lane by lane otherwise; the store does the
# same.  Everything else about an element (arithmetic, rounding after every operation,
# broadcasts, reductions read from shared memory) is evaluated per lane exactly as before.

_LANE_BASE = "nb_v"
LANES_ENABLED = True        # off: every generated loop handles one element per trip (for comparisons)


_LANE_TOKEN = re.compile(r"^\((nb_v\d*) \+ (\d+)\)$")


def _lane_dims(dims, k):
    """The indices of lane k of the group `dims` belongs to."""
    base = _LANE_TOKEN.match(dims[-1]).group(1)
    return dims[:-1] + (f"({base} + {k})",)


def _lane_of(dims, lanes):
    """Which lane the indices `dims` describe, when only the last one moves with the lane."""
    if not dims or any(_LANE_BASE in d for d in dims[:-1]):
        return None
    m = _LANE_TOKEN.match(dims[-1])
    return int(m.group(2)) if m and int(m.group(2)) < lanes else None


def _aligned16(p):
    return f"((unsigned long long)({p}) & 15ull) == 0"


_LANE_SIMPLE = None


def _simple_for_lanes(roots):
    """(True when nothing but elementwise arithmetic, broadcasts, loads and materialised
    reductions lies below `roots`, the 16-bit loads found)."""
    global _LANE_SIMPLE
    if _LANE_SIMPLE is None:
        _LANE_SIMPLE = _ELEMENTWISE + ("param", "const", "full", "pid", "nprog", "arange", "splat",
                                       "broadcast", "expand", "load", "reduce")
    seen, todo, narrow = set(), [r for r in roots if isinstance(r, Node)], []
    while todo:
        n = todo.pop()
        if n.uid in seen:
            continue
        seen.add(n.uid)
        if n.op not in _LANE_SIMPLE:
            return False, narrow
        if n.op == "load" and not isinstance(n.dtype, tp.pointer_type) and n.dtype.itemsize == 2:
            narrow.append(n)
        if n.op != "reduce":          # a reduction is read from shared memory, not recomputed
            todo += [a for a in n.args if isinstance(a, Node)]
    return True, narrow


def _side_body(body):
    """A statement list for a nested block of `body`: sees what `body` has computed, keeps what
    it computes to itself."""
    side = _Body(body.ctx, body.loop_state)
    side.lanes = body.lanes
    side.memo = dict(body.memo)
    side.loop_final = dict(body.loop_final)
    return side


def _whole_group(body, mask, mask_at, lanes):
    """Conditions under which every lane of a group passes `mask`: the deciding lanes' values
    where the mask is known to rise or fall along the lanes, else all of them."""
    if mask is None:
        return []
    deciders = body.ctx.mask_deciders(mask)
    if deciders is None:
        return list(dict.fromkeys(mask_at(k) for k in range(lanes)))
    return [mask_at(0 if d == "first" else lanes - 1) for d in sorted(deciders)]


def _emit_lanes_load(body, node, dims):
    """All lanes of a unit-stride load at once; None when this load is not of that kind."""
    lanes = body.lanes
    dt = node.dtype
    ptr, mask, other = node.args
    if isinstance(dt, tp.pointer_type) or (dt.itemsize * lanes) % 16 or ptr.shape != node.shape:
        return None
    lane = _lane_of(dims, lanes)
    if lane is None or not body.ctx.unit_stride(ptr):
        return None
    pieces = dt.itemsize * lanes // 16      # 16-byte accesses per group of lanes
    per = lanes // pieces

    def at(x, k):
        return _emit(body, x, _operand_dims(node.shape, _lane_dims(dims, k), x.shape))

    p0 = at(ptr, 0)
    conds = [_aligned16(p0)] + _whole_group(body, mask, lambda k: at(mask, k), lanes)
    whole = body.var(tp.int1, " && ".join(conds))
    arr = body.ctx.fresh("q")
    ct = dt.ctype
    body.lines.append(f"{ct} {arr}[{lanes}];")
    body.lines.append(f"if ({whole}) {{")
    for piece in range(pieces):
        body.lines.append(f"  const uint4 t{piece} = reinterpret_cast<const uint4*>({p0})[{piece}];")
        body.lines.append(f"  const {ct}* s{piece} = reinterpret_cast<const {ct}*>(&t{piece});")
        body.lines += [f"  {arr}[{piece * per + k}] = s{piece}[{k}];" for k in range(per)]
    body.lines.append("} else {")
    rare = _side_body(body)         # what only the lane-by-lane path needs stays inside its braces

    def rare_at(x, k):
        return _emit(rare, x, _operand_dims(node.shape, _lane_dims(dims, k), x.shape))

    for k in range(lanes):
        if mask is None:
            rare.lines.append(f"{arr}[{k}] = {p0}[{k}];")
        else:
            fill = _convert(rare_at(other, k), other.dtype, dt) if isinstance(other, Node) \
                else _literal(other if other is not None else 0, dt)
            rare.lines.append(f"{arr}[{k}] = {rare_at(mask, k)} ? {p0}[{k}] : {fill};")
    body.lines += ["  " + ln for ln in rare.lines]
    body.lines.append("}")
    for k in range(lanes):
        body.memo[(node.uid, _lane_dims(dims, k))] = f"{arr}[{k}]"
    return f"{arr}[{lane}]"


def _emit_lanes_store(body, ptr, value, mask, dims, lanes):
    """The store of one group of lanes (`dims`: its lane 0): 16-byte pieces when the address is
    aligned and every lane's mask holds, lane by lane otherwise."""
    elem, shape = ptr.dtype.element, ptr.shape
    each = [_lane_dims(dims, k) for k in range(lanes)]
    # An fp32 value on its way to a 16-bit tensor is rounded two lanes per instruction in the
    # 16-byte form (the same round-to-nearest; a scalar conversion per lane runs at a fraction
    # of that rate and made a bf16 chain 25 % slower than torch's).
    f32 = None
    if elem in (tp.float16, tp.bfloat16) and lanes % 2 == 0:
        if value.dtype == tp.float32:
            f32 = value
        elif (value.op == "cast" and value.dtype == elem and isinstance(value.args[0], Node)
              and value.args[0].dtype == tp.float32 and value.args[0].shape == value.shape):
            f32 = value.args[0]
    if f32 is not None:
        singles = [_emit(body, f32, _operand_dims(shape, d, f32.shape)) for d in each]
        vals = [_convert(v, tp.float32, elem) for v in singles]
    else:
        vals = [_convert(_emit(body, value, _operand_dims(shape, d, value.shape)), value.dtype, elem)
                for d in each]
    p0 = _emit(body, ptr, each[0])
    ct = elem.ctype

    def guard_at(where, k):
        return _emit(where, mask, _operand_dims(shape, each[k], mask.shape))

    def one_by_one(where, pointer_of):
        for k in range(lanes):
            stmt = f"{pointer_of(k)} = {vals[k]};"
            where.lines.append(f"if ({guard_at(where, k)}) {stmt}" if mask is not None else stmt)

    if not body.ctx.unit_stride(ptr):        # no neighbours in memory: every lane its own pointer
        one_by_one(body, lambda k: "*" + _emit(body, ptr, each[k]))
        return
    if (elem.itemsize * lanes) % 16:
        one_by_one(body, lambda k: f"{p0}[{k}]")
        return
    pieces = elem.itemsize * lanes // 16
    conds = [_aligned16(p0)] + _whole_group(body, mask, lambda k: guard_at(body, k), lanes)
    body.lines.append(f"if ({' && '.join(conds)}) {{")
    body.lines.append(f"  __align__(16) {ct} w[{lanes}];")
    if f32 is not None:
        two, pack = (("__half2", "__floats2half2_rn") if elem == tp.float16
                     else ("__nv_bfloat162", "__floats2bfloat162_rn"))
        body.lines += [f"  reinterpret_cast<{two}*>(w)[{k // 2}] = {pack}({singles[k]}, {singles[k + 1]});"
                       for k in range(0, lanes, 2)]
    else:
        body.lines += [f"  w[{k}] = {vals[k]};" for k in range(lanes)]
    body.lines += [f"  reinterpret_cast<uint4*>({p0})[{piece}] = reinterpret_cast<const uint4*>(w)[{piece}];"
                   for piece in range(pieces)]
    body.lines.append("} else {")
    rare = _side_body(body)
    one_by_one(rare, lambda k: f"{p0}[{k}]")
    body.lines += ["  " + ln for ln in rare.lines]
    body.lines.append("}")


# ---- the expression graph, seen through loops -------------------------------------------

_ELEMENTWISE = ("bin", "math", "where", "cast", "neg", "not", "inv", "cmp", "ptradd", "ptrsub")


def _effect_roots(eff):
    return [x for x in eff[1:4] if isinstance(x, Node)]


def _live_names(trace):
    """(loop uid, name) of the carried values something reads: a store, a loop bound or
    condition, or the next value of another live name.  The tracer lists every name a loop
    body assigns as carried; the ones that are only ever overwritten (`cols = start + offs`)
    are dropped here."""
    loops = {loop.uid: loop for loop in trace.loops}
    live, todo = set(), []

    def scan(roots):
        seen = set()
        stack = [r for r in roots if isinstance(r, Node)]
        while stack:
            n = stack.pop()
            if n.uid in seen:
                continue
            seen.add(n.uid)
            if n.op in ("carried", "loopout"):
                at = dict(n.attrs)
                key = (at["loop"], at["name"])
                if key not in live:
                    live.add(key)
                    todo.append(key)
            stack += [a for a in n.args if isinstance(a, Node)]

    def scan_effects(effects):
        for eff in effects:
            if eff[0] in ("for", "while"):
                scan([eff[1].lo, eff[1].hi, eff[1].step, eff[1].cond])
                scan_effects(eff[1].effects)
            else:
                scan(_effect_roots(eff))

    scan_effects(trace.effects)
    while todo:
        uid, name = todo.pop()
        _, init, nxt = loops[uid].values[name]
        scan([init, nxt])
    return live


def _carried(ctx, loop):
    """The live carried names of a loop, in a fixed order: name -> (placeholder, init, next)."""
    return {name: triple for name, triple in sorted(loop.values.items()) if (loop.uid, name) in ctx.live}


def _outside_roots(ctx, loop):
    """What a loop evaluates before its first iteration."""
    return [x for x in [init for (_, init, _) in _carried(ctx, loop).values()] +
            [loop.lo, loop.hi, loop.step] if isinstance(x, Node)]


def _inside_roots(ctx, loop):
    """What a loop evaluates every iteration, nested loops included."""
    roots = [nxt for (_, _, nxt) in _carried(ctx, loop).values()]
    if loop.cond is not None:
        roots.append(loop.cond)
    for eff in loop.effects:
        if eff[0] in ("for", "while"):
            roots += _outside_roots(ctx, eff[1]) + _inside_roots(ctx, eff[1])
        else:
            roots += _effect_roots(eff)
    return roots


def _walk(ctx, roots, visit):
    """Depth-first over the nodes below `roots`; a loop result leads into the loop's own
    expressions.  `visit(node)` returning False stops the descent below that node."""
    seen = set()
    todo = [r for r in roots if isinstance(r, Node)]
    while todo:
        n = todo.pop()
        if n.uid in seen:
            continue
        seen.add(n.uid)
        if visit(n) is False:
            continue
        todo += [a for a in n.args if isinstance(a, Node)]
        if n.op == "loopout":
            loop = ctx.loops[dict(n.attrs)["loop"]]
            todo += _outside_roots(ctx, loop) + _inside_roots(ctx, loop)


def _depends(ctx, node, loop_uid):
    """Does `node` change from one iteration of loop `loop_uid` to the next?"""
    key = (node.uid, loop_uid)
    hit = ctx.depends.get(key)
    if hit is None:
        found = []

        def visit(n):
            if n.op in ("carried", "loopvar") and dict(n.attrs)["loop"] == loop_uid:
                found.append(n)
            return not found

        _walk(ctx, [node], visit)
        hit = ctx.depends[key] = bool(found)
    return hit


def _carried_below(ctx, roots, loop_uid):
    """Names of loop `loop_uid`'s carried values that `roots` read."""
    out = set()

    def visit(n):
        if n.op == "carried" and dict(n.attrs)["loop"] == loop_uid:
            out.add(dict(n.attrs)["name"])

    _walk(ctx, roots, visit)
    return out


def _nested(loop):
    out = []
    for eff in loop.effects:
        if eff[0] in ("for", "while"):
            out += [eff[1]] + _nested(eff[1])
    return out


def _has_effects(loop):
    return any(eff[0] in ("store", "atomic") or (eff[0] in ("for", "while") and _has_effects(eff[1]))
               for eff in loop.effects)


def _is_pure(ctx, loop):
    """A pure loop neither touches memory nor needs the whole block to work together inside an
    iteration, so each thread can run it privately for the element it is computing."""
    hit = ctx.pure.get(loop.uid)
    if hit is None:
        hit = not _has_effects(loop) and all(_is_pure(ctx, n) for n in _nested(loop))
        if hit:
            reduces = []
            _walk(ctx, _inside_roots(ctx, loop), lambda n: reduces.append(n) if n.op == "reduce" else None)
            hit = not any(_depends(ctx, r, loop.uid) for r in reduces)
        ctx.pure[loop.uid] = hit
    return hit


def _induction(ph, nxt):
    """A carried block that moves by the same scalar for all of its elements each iteration
    (`ptrs += BLOCK_K * stride`, `offs += BLOCK`): returns (step node, '+' or '-'), else None.
    Such a block is kept as its initial value plus one running scalar."""
    if ph.shape == ():
        return None
    step, sign = None, "+"
    if nxt.op in ("ptradd", "ptrsub") and nxt.args[0] is ph:
        step, sign = nxt.args[1], "+" if nxt.op == "ptradd" else "-"
    elif nxt.op == "bin" and ph.dtype.is_int and nxt.dtype == ph.dtype:
        fn = dict(nxt.attrs)["fn"]
        if fn == "add" and nxt.args[0] is ph:
            step = nxt.args[1]
        elif fn == "add" and nxt.args[1] is ph:
            step = nxt.args[0]
        elif fn == "sub" and nxt.args[0] is ph:
            step, sign = nxt.args[1], "-"
    while step is not None and step.op in ("splat", "broadcast") and step.args[0].shape == ():
        step = step.args[0]
    if step is None or step.shape != () or not step.dtype.is_int:
        return None
    return step, sign


def _is_cheap(node):
    """Loaded (or constant) data, possibly cast or reshuffled: cheaper to fetch again than to
    stage."""
    while node.op in ("cast", "trans", "broadcast", "expand", "splat", "reshape"):
        node = node.args[0]
    return node.op in ("load", "const", "full", "param", "arange")


def _linear(dims, shape):
    index = "0"
    for d, extent in enumerate(shape):
        index = f"({index} * {extent} + {dims[d]})"
    return index


def _state_value(body, st, node, dims):
    """The current value of a loop-carried name for the element `dims`."""
    if isinstance(st, str):
        return st                                   # a register: per element, or a scalar
    if st[0] == "ind":
        _, init, off = st
        base = _emit(body, init, _operand_dims(node.shape, dims, init.shape))
        if node.is_pointer:
            return body.var(node.dtype, f"{base} + {off}")
        return body.var(node.dtype, f"({node.dtype.ctype})({base} + {off})")
    if st[0] == "gmem":
        # computed by another kernel into a buffer laid out like the tensor `like` walks:
        # element (dims) sits at the same offset from the buffer's start as like(dims) from
        # its own base argument
        _, name, like, base = st
        where = _emit(body, like, _operand_dims(node.shape, dims, like.shape))
        return body.var(node.dtype, f"{name}[{where} - {base}]")
    _, array, shape = st                            # a block kept in shared memory
    return f"{array}[{_linear(dims, shape)}]"


def _emit_dot(body, node, dims):
    """One element of `nl.dot(a, b, acc)` on the CUDA cores: the tuned tensor-core kernels take
    the matmul and attention programs; a dot anywhere else (small tiles, odd shapes, fused
    epilogues) is summed here in fp32, fp32 operands rounded to tf32 first as the tensor core
    would (newt/compiler/codegen.py:2174-2201)."""
    a, b, acc = node.args
    ctx = body.ctx
    i, j = dims
    d = ctx.fresh("d")
    first = _emit(body, acc, dims) if acc is not None else "0.0f"
    body.lines.append(f"float {d} = {first};")
    kk = ctx.fresh("kk")
    inner = _Body(ctx, body.loop_state)
    x = _convert(_emit(inner, a, (i, kk)), a.dtype, _F32)
    y = _convert(_emit(inner, b, (kk, j)), b.dtype, _F32)
    if a.dtype == _F32:
        ctx.helpers.add("tf32")
        x, y = f"nb_tf32({x})", f"nb_tf32({y})"
    inner.lines.append(f"{d} = fmaf({x}, {y}, {d});")
    body.lines.append(f"for (int {kk} = 0; {kk} < {a.shape[1]}; ++{kk}) {{")
    body.lines += ["  " + ln for ln in inner.lines]
    body.lines.append("}")
    return d


def _emit_loop(body, node, dims):
    """The value a pure runtime loop leaves in one of its carried names, for one element: the
    carried values this one depends on become local variables, updated in a C loop.  Each thread
    walks the loop for its own element, so carried blocks need no storage of their own."""
    ctx = body.ctx
    at = dict(node.attrs)
    loop = ctx.loops[at["loop"]]
    if not _is_pure(ctx, loop):
        raise Unsupported("the result of a loop that has not run yet")
    want = at["name"]
    names, todo = set(), [want]
    while todo:
        name = todo.pop()
        if name in names:
            continue
        names.add(name)
        todo += sorted(_carried_below(ctx, [loop.values[name][2], loop.cond], loop.uid) - names)
    names = sorted(names)
    state, dims_of, steps = {}, {}, {}
    for name in names:
        ph, init, nxt = loop.values[name]
        steps[name] = _induction(ph, nxt)
        if steps[name] is not None:
            off = ctx.fresh("off")
            body.lines.append(f"long long {off} = 0;")
            state[(loop.uid, name)] = ("ind", init, off)
            continue
        if len(ph.shape) > len(node.shape) or any(
                a not in (1, b) for a, b in zip(reversed(ph.shape), reversed(node.shape))):
            raise Unsupported(f"loop-carried '{name}' {ph.shape} does not broadcast to '{want}' {node.shape}")
        dims_of[name] = _operand_dims(node.shape, dims, ph.shape)
        first = _emit(body, init, _operand_dims(ph.shape, dims_of[name], init.shape))
        var = ctx.fresh("c")
        body.lines.append(f"{ph.dtype.ctype} {var} = {first if ph.is_pointer else _convert(first, init.dtype, ph.dtype)};")
        state[(loop.uid, name)] = var
    inner_state = dict(body.loop_state)
    inner_state.update(state)
    if loop.kind == "for":
        lo, hi, step = (_emit(body, b, ()) if isinstance(b, Node) else str(int(b))
                        for b in (loop.lo, loop.hi, loop.step))
        iv = ctx.fresh("k")
        inner_state[(loop.uid, None)] = iv
        body.lines.append(f"for (int {iv} = {lo}; ({step}) > 0 ? {iv} < {hi} : {iv} > {hi}; {iv} += {step}) {{")
    else:
        body.lines.append("for (;;) {")
    inner = _Body(ctx, inner_state)
    if loop.kind == "while":
        inner.lines.append(f"if (!({_emit(inner, loop.cond, ())})) break;")
    updates = []
    for name in names:
        ph, _, nxt = loop.values[name]
        if steps[name] is not None:
            step, sign = steps[name]
            tmp = inner.var(tp.int64, f"(long long)({_emit(inner, step, ())})")
            updates.append(f"{state[(loop.uid, name)][2]} {sign}= {tmp};")
            continue
        value = _emit(inner, nxt, _operand_dims(ph.shape, dims_of[name], nxt.shape))
        tmp = inner.var(ph.dtype, value if ph.is_pointer else _convert(value, nxt.dtype, ph.dtype))
        updates.append(f"{state[(loop.uid, name)]} = {tmp};")
    body.lines += ["  " + ln for ln in inner.lines + updates]
    body.lines.append("}")
    for name in names:     # the other carried values are now known for these indices as well
        if steps[name] is None:
            body.memo[("loopout", loop.uid, name, dims_of[name])] = state[(loop.uid, name)]
    body.loop_final.update({k: v for k, v in state.items() if not isinstance(v, str)})
    return _state_value(body, state[(loop.uid, want)], node, dims)


_REDUCE_HELPERS = """
// Block-wide fold of one value per thread; the result is valid in thread 0.  OP: 0 sum, 1 max, 2 min.
template <int OP, typename T> __device__ __forceinline__ T nb_fold(T a, T b) {
  if (OP == 0) return a + b;
  if (OP == 1) return a > b ? a : b;
  return a < b ? a : b;
}
template <> __device__ __forceinline__ float nb_fold<1, float>(float a, float b) { return fmaxf(a, b); }
template <> __device__ __forceinline__ float nb_fold<2, float>(float a, float b) { return fminf(a, b); }
template <> __device__ __forceinline__ double nb_fold<1, double>(double a, double b) { return fmax(a, b); }
template <> __device__ __forceinline__ double nb_fold<2, double>(double a, double b) { return fmin(a, b); }
template <int OP, typename T> __device__ __forceinline__ T nb_block_reduce(T v, T* scratch) {
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) v = nb_fold<OP, T>(v, __shfl_xor_sync(0xffffffffu, v, s));
  const int warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  __syncthreads();                       // scratch may still be read by the previous round
  if ((threadIdx.x & 31) == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    v = scratch[threadIdx.x < warps ? threadIdx.x : 0];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) {
      const T other = __shfl_xor_sync(0xffffffffu, v, s);
      if ((threadIdx.x ^ s) < warps && threadIdx.x < warps) v = nb_fold<OP, T>(v, other);
    }
  }
  return v;
}
"""

_REDUCE_OPS = {"sum": 0, "max": 1, "min": 2}

_ATOMIC_MAX_F32 = """
// atomicMax has no float overload: compare-and-swap until the stored value is not smaller
__device__ __forceinline__ void nb_atomic_max_f32(float* address, float value) {
  int* as_int = reinterpret_cast<int*>(address);
  int seen = *as_int;
  while (__int_as_float(seen) < value) {
    const int before = seen;
    seen = atomicCAS(as_int, before, __float_as_int(value));
    if (seen == before) break;
  }
}
"""


def _read_after_write(clash):
    return (f"values loaded from '{sorted(clash)[0]}' are consumed after the program stored to it "
            f"(a load is evaluated where its value is used, so it would see the new contents)")


def _reduce_init(fn, dt):
    if fn == "sum":
        return _literal(0, dt)
    if dt.is_floating:
        return _literal(float("-inf") if fn == "max" else float("inf"), dt)
    if dt == tp.int1:        # max of booleans is "any", min is "all"
        return "false" if fn == "max" else "true"
    bits = dt.itemsize * 8
    if dt.kind == "u":
        return _literal(0 if fn == "max" else 2 ** bits - 1, dt)
    lo, hi = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
    # INT_MIN has no literal of its own
    return f"(({dt.ctype})({lo + 1}{'LL' if bits == 64 else ''} - 1))" if fn == "max" else _literal(hi, dt)


def _materialise_reduce(node, name, threads, ctx, state=None, lanes_allowed=True):
    """Statements that leave the result of reduction `node` in the shared array `name`."""
    at = dict(node.attrs)
    fn, axis = at["fn"], at["axis"]
    if fn not in _REDUCE_OPS:
        raise Unsupported(f"reduction '{fn}'")
    x = node.args[0]
    dt = node.dtype
    shape = x.shape
    if axis is None:                   # everything into one value
        out_shape, length = (), 1
        for s in shape:
            length *= s
    else:
        out_shape, length = node.shape, shape[axis]
    outs = 1
    for s in out_shape:
        outs *= s
    body = _Body(ctx, state)
    # Folding along the last axis of a block read from 16-bit tensors: eight neighbours per trip
    # (see "sixteen bytes at a time"), when the whole block shares out the terms.
    lanes = 0
    if lanes_allowed and LANES_ENABLED and not state and outs < threads and length >= 2 * threads and length % 8 == 0 and \
            (axis == len(shape) - 1 or (axis is None and len(shape) == 1)):
        simple, narrow = _simple_for_lanes((x,))
        if simple and any(ld.shape and ld.shape[-1] == length and ctx.unit_stride(ld.args[0])
                          for ld in narrow):
            lanes = 8
    if lanes:
        body.lanes = lanes
        js = [f"j{d}" for d in range(len(out_shape))]
        first = tuple(js[:len(shape) - 1]) + (f"({_LANE_BASE} + 0)",)
        vals = [_convert(_emit(body, x, _lane_dims(first, k)), x.dtype, dt) for k in range(lanes)]
        op = _REDUCE_OPS[fn]
        init = _reduce_init(fn, dt)
        lines = []
        decompose = []
        rem = "o"
        for d in range(len(out_shape) - 1, 0, -1):
            decompose.append(f"const int j{d} = {rem} % {out_shape[d]};")
            decompose.append(f"const int p{d} = {rem} / {out_shape[d]};")
            rem = f"p{d}"
        if out_shape:
            decompose.append(f"const int j0 = {rem};")
        lines.append(f"for (int o = 0; o < {outs}; ++o) {{")
        lines += ["  " + ln for ln in decompose]
        lines.append(f"  {dt.ctype} acc = {init};")
        lines.append(f"  for (int k = threadIdx.x; k < {length // lanes}; k += {threads}) {{")
        lines.append(f"    const int {_LANE_BASE} = k * {lanes};")
        lines += ["    " + ln for ln in body.lines]
        lines += [f"    acc = nb_fold<{op}, {dt.ctype}>(acc, {v});" for v in vals]
        lines.append("  }")
        lines.append(f"  acc = nb_block_reduce<{op}, {dt.ctype}>(acc, reinterpret_cast<{dt.ctype}*>(nb_scratch));")
        lines.append(f"  if (threadIdx.x == 0) {name}[o] = acc;")
        lines.append("}")
        return ctx.either(lines, _materialise_reduce(node, name, threads, ctx, state, lanes_allowed=False))[:-1]
    # index of x for output element (j0, j1, ...) and position k along the reduced extent
    if axis is None:
        xdims, pre, rem = [], [], "k"
        for d in range(len(shape) - 1, 0, -1):
            pre.append(f"const int x{d} = {rem} % {shape[d]};")
            pre.append(f"const int y{d} = {rem} / {shape[d]};")
            rem = f"y{d}"
        pre.append(f"const int x0 = {rem};")
        xdims = tuple(f"x{d}" for d in range(len(shape)))
    else:
        pre = []
        js = [f"j{d}" for d in range(len(out_shape))]
        xdims = tuple(js[:axis] + ["k"] + js[axis:])
    val = _convert(_emit(body, x, xdims), x.dtype, dt)
    op = _REDUCE_OPS[fn]
    init = _reduce_init(fn, dt)
    inner = pre + body.lines + [f"acc = nb_fold<{op}, {dt.ctype}>(acc, {val});"]
    lines = []
    decompose = []
    rem = "o"
    for d in range(len(out_shape) - 1, 0, -1):
        decompose.append(f"const int j{d} = {rem} % {out_shape[d]};")
        decompose.append(f"const int p{d} = {rem} / {out_shape[d]};")
        rem = f"p{d}"
    if out_shape:
        decompose.append(f"const int j0 = {rem};")
    if outs >= threads or length < 2 * threads:
        # enough results for every thread to fold one of its own, or too few terms to share out
        lines.append(f"for (int o = threadIdx.x; o < {outs}; o += {threads}) {{")
        lines += ["  " + ln for ln in decompose]
        lines.append(f"  {dt.ctype} acc = {init};")
        lines.append(f"  for (int k = 0; k < {length}; ++k) {{")
        lines += ["    " + ln for ln in inner]
        lines.append("  }")
        lines.append(f"  {name}[o] = acc;")
        lines.append("}")
    else:
        # few results: the whole block folds each of them together
        lines.append(f"for (int o = 0; o < {outs}; ++o) {{")
        lines += ["  " + ln for ln in decompose]
        lines.append(f"  {dt.ctype} acc = {init};")
        lines.append(f"  for (int k = threadIdx.x; k < {length}; k += {threads}) {{")
        lines += ["    " + ln for ln in inner]
        lines.append("  }")
        lines.append(f"  acc = nb_block_reduce<{op}, {dt.ctype}>(acc, reinterpret_cast<{dt.ctype}*>(nb_scratch));")
        lines.append(f"  if (threadIdx.x == 0) {name}[o] = acc;")
        lines.append("}")
    return lines


def _base_param(ptr, loops=None):
    """The pointer argument a pointer value walks from (a pointer carried by a loop starts at
    its initial value)."""
    while True:
        if ptr.op in ("ptradd", "ptrsub", "broadcast", "expand", "splat", "trans", "reshape"):
            ptr = ptr.args[0]
        elif ptr.op in ("carried", "loopout") and loops is not None:
            at = dict(ptr.attrs)
            ptr = loops[at["loop"]].values[at["name"]][1]
        else:
            break
    if ptr.op != "param":
        raise Unsupported("a pointer that is not derived from a kernel argument")
    return dict(ptr.attrs)["name"]


_TF32_HELPER = """
// fp32 operands of nl.dot are rounded to tf32 (10 explicit mantissa bits, ties away from zero)
__device__ __forceinline__ float nb_tf32(float x) {
  unsigned r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}
"""

_STATIC_SHARED_LIMIT = 48 * 1024
_SHARED_LIMIT = 227 * 1024


class _Scheduler:
    """Writes the block-level statements of a kernel: one element loop per store, atomic or
    reduction, and a C loop run by all threads together for every runtime loop that stores or
    reduces inside its body.  In such a loop carried scalars are registers (every thread
    computes the same value), carried blocks that only move by a scalar are an offset, and the
    other carried blocks live in shared memory."""

    def __init__(self, ctx):
        self.ctx = ctx
        self.live = set()          # reductions whose shared array holds the current value

    # -- pieces ---------------------------------------------------------------------------

    def scalar(self, expr, state):
        """Statements + C expression of a scalar, evaluated by every thread."""
        if not isinstance(expr, Node):
            return [], str(int(expr))
        body = _Body(self.ctx, state)
        return body.lines, _emit(body, expr, ())

    def element_loop(self, shape, state, finish):
        """`finish(body, dims)` appends the statement(s) done for each element of `shape`."""
        threads = self.ctx.threads
        numel = 1
        for s in shape:
            numel *= s
        body = _Body(self.ctx, state)
        dims = tuple(f"i{d}" for d in range(len(shape)))
        finish(body, dims)
        lines = []
        if shape:
            if not any(ln.lstrip().startswith("for (") for ln in body.lines):
                lines.append("#pragma unroll 8")
            lines.append(f"for (int e = threadIdx.x; e < {numel}; e += {threads}) {{")
            lines.append("  int r = e;")
            for d in range(len(shape) - 1, 0, -1):
                lines.append(f"  const int i{d} = r % {shape[d]};")
                lines.append(f"  r /= {shape[d]};")
            lines.append("  const int i0 = r;")
        else:
            lines.append("if (threadIdx.x == 0) {")
        lines += ["  " + ln for ln in body.lines]
        lines.append("}")
        lines.append("__syncthreads();")
        return lines

    def lanes_for(self, eff, state):
        """How many neighbours a trip of this store's element loop computes: 8 for a plain store
        of a 16-bit block whose last axis is a multiple of 8 and unit-stride in memory, with
        nothing but elementwise arithmetic, broadcasts and materialised reductions between the
        loads and the store; else 0 (one element per trip)."""
        _, ptr, value, mask, _lineno = eff[:5]
        if eff[0] != "store" or state or not LANES_ENABLED:
            return 0
        elem, shape = ptr.dtype.element, ptr.shape
        if elem.itemsize != 2 or not shape or shape[-1] % 8 or not self.ctx.unit_stride(ptr):
            return 0
        return 8 if _simple_for_lanes((value, mask))[0] else 0

    def lane_loop(self, shape, state, lanes, finish):
        """`element_loop` with `lanes` neighbours along the last axis per trip: `finish(body,
        dims)` gets the indices of lane 0."""
        threads = self.ctx.threads
        numel = 1
        for s in shape:
            numel *= s
        body = _Body(self.ctx, state)
        body.lanes = lanes
        dims = tuple(f"i{d}" for d in range(len(shape) - 1)) + (f"({_LANE_BASE} + 0)",)
        finish(body, dims)
        per_row = shape[-1] // lanes
        lines = ["#pragma unroll 2",
                 f"for (int e = threadIdx.x; e < {numel // lanes}; e += {threads}) {{",
                 "  int r = e;",
                 f"  const int {_LANE_BASE} = (r % {per_row}) * {lanes};",
                 f"  r /= {per_row};"]
        for d in range(len(shape) - 2, 0, -1):
            lines.append(f"  const int i{d} = r % {shape[d]};")
            lines.append(f"  r /= {shape[d]};")
        if len(shape) >= 2:
            lines.append("  const int i0 = r;")
        lines += ["  " + ln for ln in body.lines]
        lines.append("}")
        lines.append("__syncthreads();")
        return lines

    def fill(self, array, shape, value, state, dt):
        """array[e] = value(e) for a block kept in shared memory."""
        def finish(body, dims):
            v = _emit(body, value, _operand_dims(shape, dims, value.shape))
            v = v if isinstance(dt, tp.pointer_type) else _convert(v, value.dtype, dt)
            body.lines.append(f"{array}[{_linear(dims, shape)}] = {v};")
        return self.element_loop(shape, state, finish)

    def need(self, roots, state, only=None):
        """Materialises what the expressions below `roots` read from shared memory and is not
        current: reductions, and operands of `nl.dot` that are computed rather than loaded
        (attention's P in P @ V) -- a dot reads each operand element once per output column
        or row, so computing it in place would repeat that work that many times."""
        ctx = self.ctx
        found = {}
        seen = set()
        todo = [(r, False) for r in roots if isinstance(r, Node)]
        while todo:
            n, in_pure = todo.pop()
            if (n.uid, in_pure) in seen:
                continue
            seen.add((n.uid, in_pure))
            if n.op == "reduce":
                found[n.uid] = n
            if n.op == "dot" and not in_pure:
                for operand in n.args[:2]:
                    if not _is_cheap(operand):
                        found[operand.uid] = operand
            todo += [(a, in_pure) for a in n.args if isinstance(a, Node)]
            if n.op == "loopout":
                at = dict(n.attrs)
                if (at["loop"], at["name"]) in ctx.final:
                    continue          # that loop has run; its result is read, not recomputed
                loop = ctx.loops[at["loop"]]
                # what a pure loop computes from its own state stays in the thread that runs it
                todo += [(r, in_pure) for r in _outside_roots(ctx, loop)]
                todo += [(r, True) for r in _inside_roots(ctx, loop)]
        lines = []
        for uid in sorted(found):      # node ids follow program order: operands come first
            node = found[uid]
            if uid in self.live or (only is not None and not only(node)):
                continue
            if node.op != "reduce":
                if uid not in ctx.reduced:
                    numel = 1
                    for s in node.shape:
                        numel *= s
                    ctx.reduced[uid] = (ctx.alloc(node.dtype, numel, "nb_s"), node.shape)
                ctx.staging.add(uid)
                lines += self.fill(ctx.reduced[uid][0], node.shape, node, state, node.dtype)
                ctx.staging.discard(uid)
                self.live.add(uid)
                continue
            if uid not in ctx.reduced:
                outs = 1
                for s in (node.shape if dict(node.attrs)["axis"] is not None else ()):
                    outs *= s
                name = ctx.alloc(node.dtype, outs, "nb_r")
                ctx.reduced[uid] = (name, () if dict(node.attrs)["axis"] is None else node.shape)
            ctx.helpers.add("reduce")
            lines += _materialise_reduce(node, ctx.reduced[uid][0], ctx.threads, ctx, state)
            lines.append("__syncthreads();")
            self.live.add(uid)
        return lines

    def store(self, eff, state):
        ctx = self.ctx
        _, ptr, value, mask, _lineno = eff[:5]
        atomic = eff[5] if eff[0] == "atomic" else None
        elem = ptr.dtype.element
        shape = ptr.shape

        def finish(body, dims):
            p = _emit(body, ptr, dims)
            val = _convert(_emit(body, value, _operand_dims(shape, dims, value.shape)), value.dtype, elem)
            guard = _emit(body, mask, _operand_dims(shape, dims, mask.shape)) if mask is not None else None
            if atomic is None:
                stmt = f"*{p} = {val};"
            elif atomic == "add":
                if elem == tp.int64:
                    stmt = f"atomicAdd(reinterpret_cast<unsigned long long*>({p}), (unsigned long long)({val}));"
                elif elem.name in ("float32", "float64", "float16", "bfloat16", "int32", "uint32"):
                    stmt = f"atomicAdd({p}, {val});"
                else:
                    raise Unsupported(f"nl.atomic_add on {elem.name}")
            elif elem == tp.float32:
                ctx.helpers.add("atomic_max_f32")
                stmt = f"nb_atomic_max_f32({p}, {val});"
            elif elem.name in ("int32", "uint32", "int64"):
                stmt = f"atomicMax({p}, {val});"
            else:
                raise Unsupported(f"nl.atomic_max on {elem.name}")
            body.lines.append(f"if ({guard}) {stmt}" if guard else stmt)

        lanes = self.lanes_for(eff, state)
        if lanes:
            def finish_lanes(body, dims):
                _emit_lanes_store(body, ptr, value, mask, dims, lanes)

            return self.need(_effect_roots(eff), state) + self.ctx.either(
                self.lane_loop(shape, state, lanes, finish_lanes),
                self.element_loop(shape, state, finish))
        return self.need(_effect_roots(eff), state) + self.element_loop(shape, state, finish)

    # -- statements -----------------------------------------------------------------------

    def run(self, effects, state):
        lines = []
        for eff in effects:
            if eff[0] in ("for", "while"):
                if not _is_pure(self.ctx, eff[1]):     # a pure loop is emitted where its results are used
                    lines += self.block_loop(eff[1], state)
            elif eff[0] in ("store", "atomic"):
                lines += self.store(eff, state)
            else:
                raise Unsupported(f"effect '{eff[0]}'")
        return lines

    def block_loop(self, loop, state):
        ctx = self.ctx
        out = self.need(_outside_roots(ctx, loop), state)
        inside = _inside_roots(ctx, loop)
        varying = [loop.uid] + [n.uid for n in _nested(loop)]
        # reductions the body uses but does not change are done once, before the loop
        out += self.need(inside, state, only=lambda r: not any(_depends(ctx, r, u) for u in varying))
        inner = dict(state)
        scalars, inductions, blocks = [], [], []
        carried = _carried(ctx, loop)
        for name, (ph, init, nxt) in carried.items():
            key = (loop.uid, name)
            step = _induction(ph, nxt)
            if ph.shape == ():
                lines, v = self.scalar(init, state)
                var = ctx.fresh("c")
                out += lines + [f"{ph.dtype.ctype} {var} = {v if ph.is_pointer else _convert(v, init.dtype, ph.dtype)};"]
                inner[key] = var
                scalars.append(name)
            elif step is not None:
                off = ctx.fresh("off")
                out.append(f"long long {off} = 0;")
                inner[key] = ("ind", init, off)
                inductions.append((name, step))
            else:
                numel = 1
                for s in ph.shape:
                    numel *= s
                array = ctx.alloc(ph.dtype, numel, "nb_c")
                inner[key] = ("smem", array, ph.shape)
                out += self.fill(array, ph.shape, init, state, ph.dtype)
                blocks.append(name)
        if loop.kind == "for":
            bounds = []
            for b in (loop.lo, loop.hi, loop.step):
                lines, v = self.scalar(b, state)
                out += lines
                bounds.append(v)
            lo, hi, step = bounds
            iv = ctx.fresh("k")
            inner[(loop.uid, None)] = iv
            out.append(f"for (int {iv} = {lo}; ({step}) > 0 ? {iv} < {hi} : {iv} > {hi}; {iv} += {step}) {{")
        else:
            out.append("for (;;) {")
        live_outside = set(self.live)
        body = []
        if loop.kind == "while":
            body += self.need([loop.cond], inner)
            lines, v = self.scalar(loop.cond, inner)
            body += lines + [f"if (!({v})) break;"]
        body += self.run(loop.effects, inner)
        # next values: everything is computed from this iteration's state before any of it changes
        body += self.need([nxt for (_, _, nxt) in carried.values()], inner)
        assigns = []
        for name in scalars:
            ph, _, nxt = loop.values[name]
            lines, v = self.scalar(nxt, inner)
            tmp = ctx.fresh("t")
            decl = f"{ph.dtype.ctype} const {tmp}" if ph.is_pointer else f"const {ph.dtype.ctype} {tmp}"
            body += lines + [f"{decl} = {v if ph.is_pointer else _convert(v, nxt.dtype, ph.dtype)};"]
            assigns.append(f"{inner[(loop.uid, name)]} = {tmp};")
        for name, (step, sign) in inductions:
            lines, v = self.scalar(step, inner)
            tmp = ctx.fresh("t")
            body += lines + [f"const long long {tmp} = (long long)({v});"]
            assigns.append(f"{inner[(loop.uid, name)][2]} {sign}= {tmp};")
        reads = {name: _carried_below(ctx, [loop.values[name][2]], loop.uid) & set(blocks)
                 for name in blocks}
        copies = []
        for name in blocks:
            ph, _, nxt = loop.values[name]
            _, array, shape = inner[(loop.uid, name)]
            in_place = _same_index_only(ctx, nxt, ph) and \
                not any(name in reads[other] for other in blocks if other != name)
            if in_place:       # element e is read and written by the same thread only
                body += self.fill(array, shape, nxt, inner, ph.dtype)
                continue
            numel = 1
            for s in shape:
                numel *= s
            staged = ctx.alloc(ph.dtype, numel, "nb_n")
            body += self.fill(staged, shape, nxt, inner, ph.dtype)
            copies += [f"for (int e = threadIdx.x; e < {numel}; e += {ctx.threads}) {array}[e] = {staged}[e];"]
        if copies:
            body += copies + ["__syncthreads();"]
        body += assigns
        out += ["  " + ln for ln in body]
        out.append("}")
        self.live = live_outside
        for name in carried:
            ctx.final[(loop.uid, name)] = inner[(loop.uid, name)]
        return out


def _same_index_only(ctx, root, ph):
    """True when element e of `root` reads the carried block `ph` at element e only."""
    memo = {}

    def go(n, same):
        if n is ph:
            return same
        if n.op == "reduce":
            return True      # materialised before the update starts, read from its own array
        key = (n.uid, same)
        if key in memo:
            return memo[key]
        memo[key] = True
        ok = True
        children = [(a, same and a.shape == n.shape and
                     (n.op in _ELEMENTWISE or (n.op == "dot" and i == 2)))
                    for i, a in enumerate(n.args) if isinstance(a, Node)]
        if n.op == "loopout":
            loop = ctx.loops[dict(n.attrs)["loop"]]
            children += [(r, False) for r in _outside_roots(ctx, loop) + _inside_roots(ctx, loop)]
        for a, child_same in children:
            if not go(a, child_same):
                ok = False
                break
        memo[key] = ok
        return ok

    return go(root, True)


def _check_order(ctx, effects, written):
    """Loads are evaluated inside the statement that uses them, i.e. possibly after stores that
    the source program placed later.  Refuses the programs where that could change a result:
    a tensor read by a statement after another statement stored to it."""

    def loads(roots):
        out = set()
        _walk(ctx, roots, lambda n: out.add(_base_param(n.args[0], ctx.loops)) if n.op == "load" else None)
        return out

    def in_place(eff):
        """A statement may read the tensor it stores to only through the very pointers it
        stores through (x[i] = f(x[i])): any other element may already be overwritten by
        another thread."""
        target = _base_param(eff[1], ctx.loops)

        def visit(n):
            if n.op == "load" and n.args[0] is not eff[1] and _base_param(n.args[0], ctx.loops) == target:
                raise Unsupported(f"'{target}' is stored to and read at other elements by one statement")

        _walk(ctx, _effect_roots(eff), visit)

    def groups(loop):
        """(roots, written parameter or None) for everything a loop evaluates per iteration."""
        out = [([nxt for (_, _, nxt) in _carried(ctx, loop).values()] + [loop.cond], None)]
        for eff in loop.effects:
            if eff[0] in ("for", "while"):
                out += [(_outside_roots(ctx, eff[1]), None)] + groups(eff[1])
            else:
                in_place(eff)
                out.append((_effect_roots(eff), _base_param(eff[1], ctx.loops)))
        return out

    for eff in effects:
        if eff[0] in ("for", "while"):
            loop = eff[1]
            if _is_pure(ctx, loop):
                continue
            parts = [(_outside_roots(ctx, loop), None)] + groups(loop)
            reads = [loads(roots) for roots, _ in parts]
            for i, (_, target) in enumerate(parts):
                clash = set().union(*reads) & written
                if clash:
                    raise Unsupported(_read_after_write(clash))
                if target is not None and any(target in r for j, r in enumerate(reads) if j != i):
                    raise Unsupported(f"'{target}' is stored to and read by different statements "
                                      f"of a runtime loop")
            written |= {t for _, t in parts if t is not None}
        else:
            in_place(eff)
            clash = loads(_effect_roots(eff)) & written
            if clash:
                raise Unsupported(_read_after_write(clash))
            written.add(_base_param(eff[1], ctx.loops))



# ---- a row per program, kept in registers ------------------------------------------------------
#
# Programs of the softmax / layernorm family -- one 1-D block per program instance, reductions
# over the whole block, elementwise arithmetic around them, stores of the block -- need not go
# through memory between their passes.  Every thread owns BLOCK / threads elements (groups of
# lanes `(g * threads + threadIdx.x) * lanes + k`, so a warp touches consecutive 16-byte pieces);
# the program is written out as straight-line code over one statement list, so a load or an
# `exp` that the row maximum, the row sum and the stored value all use is evaluated once per
# element and stays in a register; a reduction folds the thread's own values, then the block's
# (`nb_block_reduce`), and is read back from shared memory by what follows.  This is what makes
# a log-softmax, a softmax with a temperature, an RMSNorm or a layernorm without bias -- programs
# the tuned row kernels do not recognise -- run at one pass over HBM instead of one per
# reduction.

_RESIDENT_MAX_PER_THREAD = 32


def _resident_shape(ctx, trace):
    """(block extent, lanes) when the program is of that family, else None."""
    threads = ctx.threads
    if not LANES_ENABLED or not trace.effects or any(eff[0] != "store" for eff in trace.effects):
        return None
    extent, smallest, reduces = None, 8, 0
    seen, todo = set(), []
    for eff in trace.effects:
        ptr = eff[1]
        if len(ptr.shape) != 1:
            return None
        if extent not in (None, ptr.shape[0]):
            return None
        extent = ptr.shape[0]
        smallest = min(smallest, ptr.dtype.element.itemsize)
        todo += [r for r in _effect_roots(eff) if isinstance(r, Node)]
    _simple_for_lanes(())            # fills the table of operations lanes can evaluate
    simple = _LANE_SIMPLE
    while todo:
        n = todo.pop()
        if n.uid in seen:
            continue
        seen.add(n.uid)
        if n.op not in simple or n.shape not in ((), (1,), (extent,)):
            return None
        if n.op == "reduce":
            reduces += 1
            if n.shape != () or n.args[0].shape != (extent,) or dict(n.attrs)["fn"] not in _REDUCE_OPS:
                return None
        if n.op == "load" and n.shape == (extent,) and not isinstance(n.dtype, tp.pointer_type):
            smallest = min(smallest, n.dtype.itemsize)
        todo += [a for a in n.args if isinstance(a, Node)]
    if not reduces or extent % threads or extent // threads > _RESIDENT_MAX_PER_THREAD:
        return None
    lanes = 16 // smallest
    if extent % (threads * lanes):
        lanes = 1
    return extent, lanes


def _resident_lines(ctx, trace, extent, lanes):
    """The whole program as straight-line code, `lanes` neighbours per group."""
    threads = ctx.threads
    body = _Body(ctx, {})
    body.lanes = lanes
    groups = extent // (threads * lanes)
    first = []
    for g in range(groups):
        body.lines.append(f"const int nb_v{g} = ({g * threads} + (int)threadIdx.x) * {lanes};")
        first.append((f"(nb_v{g} + 0)",))
    done = set()

    def fold(node):
        at = dict(node.attrs)
        x, dt, op = node.args[0], node.dtype, _REDUCE_OPS[at["fn"]]
        name = ctx.alloc(dt, 1, "nb_r")
        ctx.helpers.add("reduce")
        acc = ctx.fresh("a")
        terms = [_convert(_emit(body, x, _lane_dims(d, k)), x.dtype, dt)
                 for d in first for k in range(lanes)]
        body.lines.append(f"{dt.ctype} {acc} = {_reduce_init(at['fn'], dt)};")
        body.lines += [f"{acc} = nb_fold<{op}, {dt.ctype}>({acc}, {t});" for t in terms]
        body.lines.append(f"{acc} = nb_block_reduce<{op}, {dt.ctype}>({acc}, "
                          f"reinterpret_cast<{dt.ctype}*>(nb_scratch));")
        body.lines.append(f"if (threadIdx.x == 0) {name}[0] = {acc};")
        body.lines.append("__syncthreads();")
        ctx.reduced[node.uid] = (name, ())

    def reductions_below(roots):
        found, seen, todo = {}, set(), [r for r in roots if isinstance(r, Node)]
        while todo:
            n = todo.pop()
            if n.uid in seen:
                continue
            seen.add(n.uid)
            if n.op == "reduce" and n.uid not in done:
                found[n.uid] = n
            todo += [a for a in n.args if isinstance(a, Node)]
        return [found[u] for u in sorted(found)]       # program order: operands come first

    for eff in trace.effects:
        _, ptr, value, mask, _lineno = eff[:5]
        for node in reductions_below(_effect_roots(eff)):
            fold(node)
            done.add(node.uid)
        for d in first:
            if lanes > 1:
                _emit_lanes_store(body, ptr, value, mask, d, lanes)
            else:
                p = _emit(body, ptr, d)
                val = _convert(_emit(body, value, _operand_dims(ptr.shape, d, value.shape)),
                               value.dtype, ptr.dtype.element)
                guard = _emit(body, mask, _operand_dims(ptr.shape, d, mask.shape)) \
                    if mask is not None else None
                body.lines.append(f"if ({guard}) *{p} = {val};" if guard else f"*{p} = {val};")
    for uid in done:          # the other form of the program folds for itself
        del ctx.reduced[uid]
    return ["{"] + ["  " + ln for ln in body.lines] + ["}"]


def _resident_program(ctx, trace):
    shape = _resident_shape(ctx, trace)
    if shape is None:
        return None
    extent, lanes = shape
    if lanes == 1:
        return _resident_lines(ctx, trace, extent, 1)
    ctx.wide_all = True
    return ctx.either(_resident_lines(ctx, trace, extent, lanes),
                      _resident_lines(ctx, trace, extent, 1))


def generate(trace, num_warps, computed_elsewhere=None):
    """Returns (cuda_source, kernel_name, [(param name, dtype or pointer_type)], bytes of
    dynamic shared memory).

    `computed_elsewhere`: {(loop uid, carried name): (buffer parameter name, pointer node)} --
    results of loops that another kernel has already left in device memory (the accumulator of
    a matmul k loop run on the tensor core).  The generated kernel takes each buffer as one
    more pointer argument, after the program's own, and reads the value for an element at the
    offset at which the pointer node addresses its tensor; the loop itself is not emitted."""
    ctx = _Context(trace, num_warps * THREADS_PER_WARP)
    extra_params = []
    for (uid, name), (buffer, like) in (computed_elsewhere or {}).items():
        ph = ctx.loops[uid].values[name][0]
        ctx.final[(uid, name)] = ("gmem", buffer, like, _base_param(like, ctx.loops))
        extra_params.append((buffer, tp.pointer_type(ph.dtype)))
    if not any(eff[0] in ("store", "atomic") or (eff[0] in ("for", "while") and _has_effects(eff[1]))
               for eff in trace.effects):
        raise Unsupported("the program stores nothing")
    _check_order(ctx, trace.effects, set())
    lines = None if computed_elsewhere else _resident_program(ctx, trace)
    if lines is None:
        lines = _Scheduler(ctx).run(trace.effects, {})
    while lines and lines[-1] == "__syncthreads();":
        lines.pop()

    params = [(name, node.dtype) for name, node in trace.params.items()] + extra_params
    # Elements are independent, so the loads of several iterations may be issued before the
    # stores of earlier ones; `__restrict__` says so (a tensor passed under two names is still
    # fine as long as element i is only read for element i, as in any in-place elementwise call).
    decl = ", ".join(f"{t.ctype} __restrict__ {name}" if isinstance(t, tp.pointer_type)
                     else f"{t.ctype} {name}" for name, t in params)
    helpers = ""
    if "atomic_max_f32" in ctx.helpers:
        helpers += _ATOMIC_MAX_F32
    if "tf32" in ctx.helpers:
        helpers += _TF32_HELPER
    if "reduce" in ctx.helpers:
        helpers += _REDUCE_HELPERS
    shared, dynamic = ctx.shared_declarations()
    body_text = "\n  ".join(shared + ctx.wide_declaration() + lines)
    digest = hashlib.sha1((decl + body_text).encode()).hexdigest()[:8]
    kernel_name = f"{trace.name}_{digest}"
    source = (
        "#include <cuda_fp16.h>\n#include <cuda_bf16.h>\n" + _ROUNDING_HELPERS + helpers + "\n"
        f"extern \"C\" __global__ void __launch_bounds__({ctx.threads}) {kernel_name}({decl}) {{\n  "
        f"{body_text}\n}}\n")
    return source, kernel_name, params, dynamic


def generate_epilogue(trace, accumulator, store, block, axes):
    """The code a matmul program has after its k loop, as a functor for the tensor-core kernel's
    epilogue (csrc/gemm_device.cuh `EPI`): `apply` gets 32 consecutive columns of one row of the
    fp32 accumulator and leaves in them the value the program stores, evaluated element by
    element exactly as the one-block-per-program kernel would (same graph, same emitter), with
    the program ids and block indices derived from the element's row and column.

    accumulator: (loop uid, carried name) of the k loop's result; store: the program's store
    effect; block: (BLOCK_M, BLOCK_N); axes: (grid axis of the row blocks, of the column blocks).
    Returns (CUDA text defining `struct NbEpilogue`, [(param name, type)] of its Args struct).
    Raises Unsupported for what cannot run there (reductions over the tile, further loops that
    store, anything needing shared memory): those programs take the two-kernel route."""
    ctx = _Context(trace, THREADS_PER_WARP)
    ctx.final[accumulator] = "nb_acc"
    ctx.program_ids = {axes[0]: "nb_pid_m", axes[1]: "nb_pid_n"}
    _, ptr, value, mask, _lineno = store[:5]
    if len(ptr.shape) != 2:
        raise Unsupported("the store after the k loop is not a 2-D tile")
    body = _Body(ctx)
    dims = ("nb_i", "nb_j")
    elem = ptr.dtype.element
    # The kernel's epilogue rounds the fp32 value it gets back to C's type (round to nearest, two
    # elements per instruction), so a program's own final rounding of an fp32 value to that type
    # is left to it: float -> 16-bit -> float -> 16-bit gives the same bits as float -> 16-bit.
    if (value.op == "cast" and value.dtype == elem and elem in (tp.float16, tp.bfloat16)
            and value.args[0].dtype == tp.float32 and value.args[0].shape == value.shape):
        value = value.args[0]
    out = _convert(_emit(body, value, _operand_dims(ptr.shape, dims, value.shape)), value.dtype,
                   tp.float32 if value.dtype == tp.float32 else elem)
    if ctx.arrays or ctx.helpers:
        raise Unsupported("the code after the k loop needs shared memory or helper routines")
    params = [(name, node.dtype) for name, node in trace.params.items()]
    fields = "\n".join(f"    {t.ctype} {name};" for name, t in params)
    unpack = "\n".join(f"    {t.ctype} const {name} = nb_a.{name}; (void){name};" if isinstance(t, tp.pointer_type)
                       else f"    const {t.ctype} {name} = nb_a.{name}; (void){name};" for name, t in params)
    early, late, staged = _split_epilogue(body.lines, out)
    bm, bn = block
    index = (f"    const int nb_pid_m = nb_row / {bm}, nb_i = nb_row % {bm}; (void)nb_pid_m; (void)nb_i;\n"
             "#pragma unroll\n"
             "    for (int nb_k = 0; nb_k < 32; ++nb_k) {\n"
             "      const int nb_col = nb_col0 + nb_k;\n"
             f"      const int nb_pid_n = nb_col / {bn}, nb_j = nb_col % {bn}; (void)nb_pid_n; (void)nb_j;\n")
    members = "\n".join(f"    {ctype} {name}[32];" for name, ctype in staged)
    keep = "\n".join(f"      nb_s.{name}[nb_k] = {name};" for name, _ in staged)
    take = "\n".join(f"      const {ctype} {name} = nb_s.{name}[nb_k];" for name, ctype in staged)
    indent = lambda lines: "\n".join("      " + ln for ln in lines)  # noqa: E731
    text = _ROUNDING_HELPERS + f"""
struct NbEpilogue {{
  struct Args {{
{fields}
  }};
  struct Staged {{
{members}
  }};
  // what the code reads besides the accumulator: issued while the accumulator is on its way
  static __device__ __forceinline__ void fetch(Staged& nb_s, int nb_row, int nb_col0, const Args& nb_a) {{
{unpack}
{index}{indent(early)}
{keep}
    }}
  }}
  static __device__ __forceinline__ void apply(float (&nb_v)[32], const Staged& nb_s, int nb_row, int nb_col0,
                                               const Args& nb_a) {{
{unpack}
{index}      const float nb_acc = nb_v[nb_k];
{take}
{indent(late)}
      nb_v[nb_k] = (float)({out});
    }}
  }}
}};
"""
    return text, params


_DECLARATION = re.compile(r"^(?P<type>(?:const\s+)?[A-Za-z_][\w:<>, ]*?(?:\s*\*)?)\s*(?:const\s+)?(?P<name>[A-Za-z_]\w*) = (?P<expr>.*);$")
_WORD = re.compile(r"[A-Za-z_]\w*")


def _split_epilogue(lines, out):
    """The straight-line body of an epilogue in two parts: the statements that do not depend on
    the accumulator (index arithmetic, the loads of a bias or a residual) and the rest.  Returns
    (early lines, late lines, [(name, C type)] of the early values the late part or the result
    uses).  A body with anything but plain declarations stays whole, as the late part."""
    parsed = []
    for ln in lines:
        m = _DECLARATION.match(ln.strip())
        if m is None:
            return [], list(lines), []
        parsed.append((ln.strip(), m.group("type").strip(), m.group("name"), set(_WORD.findall(m.group("expr")))))
    late_names = {"nb_acc"}
    early, late = [], []
    for ln, ctype, name, used in parsed:
        if used & late_names:
            late_names.add(name)
            late.append((ln, used))
        else:
            early.append((ln, ctype, name))
    wanted = set(_WORD.findall(out))
    for _, used in late:
        wanted |= used
    staged = []
    for ln, ctype, name in early:
        if name in wanted:
            if "*" in ctype:      # a pointer the late part dereferences: keep the body whole
                return [], list(lines), []
            staged.append((name, ctype[len("const "):].strip() if ctype.startswith("const ") else ctype))
    return [ln for ln, _, _ in early], [ln for ln, _ in late], staged


def struct_type(params):
    """The ctypes structure laid out like the `Args` struct `generate_epilogue` declares."""
    fields = []
    for name, t in params:
        if isinstance(t, tp.pointer_type):
            fields.append((name, ctypes.c_void_p))
        else:
            ctype = _CTYPES.get(t.name)
            if ctype is None:
                raise TypeError(f"argument '{name}': scalars of type {t.name} cannot be passed to a kernel")
            fields.append((name, ctype))
    return type("NbEpilogueArgs", (ctypes.Structure,), {"_fields_": fields})


def marshal_struct(params, args, struct=None):
    """An instance of `struct_type(params)` holding this launch's arguments."""
    packed = (struct or struct_type(params))()
    for name, t in params:
        v = args[name]
        setattr(packed, name, v.data_ptr() if isinstance(t, tp.pointer_type) else v)
    return packed


_CTYPES = {"int1": ctypes.c_bool, "int8": ctypes.c_int8, "uint8": ctypes.c_uint8,
           "int16": ctypes.c_int16, "int32": ctypes.c_int32, "uint32": ctypes.c_uint32,
           "int64": ctypes.c_int64, "float32": ctypes.c_float, "float64": ctypes.c_double}


def marshal(params, args):
    """ctypes values for a launch, in parameter order."""
    out = []
    for name, t in params:
        v = args[name]
        if isinstance(t, tp.pointer_type):
            out.append(ctypes.c_void_p(v.data_ptr()))
        else:
            ctype = _CTYPES.get(t.name)
            if ctype is None:
                raise TypeError(f"argument '{name}': scalars of type {t.name} cannot be passed to a kernel")
            out.append(ctype(v))
    return out
