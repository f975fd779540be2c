"""Generic lowering of loop-free block programs to CUDA text.

Everything the block language can say without a runtime `for` or `nl.dot` is arithmetic on
blocks of compile-time shape: loads through pointer blocks, broadcasting, elementwise math,
`nl.where`, casts, `nl.sum / max / min`, masked stores.  Such a program needs no tuned kernel
-- it is bound by HBM -- so it is compiled at run time, like the reference compiles all
programs: one CUDA block of `num_warps * 32` threads per program instance; for each `nl.store`,
the threads stride over the elements of the stored block and evaluate the expression for their
element.  A reduction is computed first, by the whole block, into shared memory, and read from
there by the expressions that use it.

Numerics follow the reference's elementwise rules (newt/compiler/codegen.py:1196-1284,
2011-2030): fp16 / bf16 operations are computed in fp32 and rounded back after every
operation; Python constants were already given the dtype of the block they meet by the
tracer; integer `/` is C division; math functions are the precise single-precision ones
(`expf`, `rsqrtf`, ...), no fast-math.
"""

import ctypes
import hashlib
import math

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


def _convert(expr, src, dst):
    """C expression converting `expr` of dtype `src` to `dst`."""
    if src == dst:
        return expr
    if _is_half(src):
        as_float = f"__half2float({expr})" if src == tp.float16 else f"__bfloat162float({expr})"
        return as_float if dst == _F32 else _convert(as_float, _F32, dst)
    if dst == tp.float16:
        return f"__float2half_rn({_convert(expr, src, _F32)})"
    if dst == tp.bfloat16:
        return f"__float2bfloat16_rn({_convert(expr, src, _F32)})"
    if dst == tp.int1:
        return f"(({expr}) != 0)"
    return f"(({dst.ctype})({expr}))"


_MATH = {"exp": "expf", "exp2": "exp2f", "log": "logf", "log2": "log2f", "sqrt": "sqrtf",
         "rsqrt": "rsqrtf", "sin": "sinf", "cos": "cosf", "tanh": "tanhf", "erf": "erff",
         "floor": "floorf", "ceil": "ceilf", "abs": "fabsf"}
_INFIX = {"add": "+", "sub": "-", "mul": "*", "and": "&", "or": "|", "xor": "^", "shl": "<<",
          "shr": ">>"}
_CMP = {"lt": "<", "le": "<=", "gt": ">", "ge": ">=", "eq": "==", "ne": "!="}


class _Body:
    """Statements that compute one element of one store."""

    def __init__(self, reduced=None):
        self.lines = []
        self.memo = {}
        self.reduced = reduced if reduced is not None else {}   # reduce node uid -> (array, shape)

    def var(self, dt, expr):
        name = f"v{len(self.lines)}"
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
        return f"(int)blockIdx.{'xyz'[at['axis']]}"
    if op == "nprog":
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
    if op == "reduce":
        slot = body.reduced.get(node.uid)
        if slot is None:
            raise Unsupported("a reduction inside a reduction's own operand chain was not materialised")
        name, shape = slot
        index = "0"
        for d, extent in enumerate(shape):
            index = f"({index} * {extent} + {dims[d]})"
        return f"{name}[{index}]"
    raise Unsupported(f"'{op}' has no elementwise lowering")


def _reads_from(node, seen, out, reduces=None):
    """Names of the pointer parameters that `node`'s value loads from (and, in `reduces`, the
    reductions it goes through)."""
    if not isinstance(node, Node) or node.uid in seen:
        return
    seen.add(node.uid)
    if node.op == "load":
        out.add(_base_param(node.args[0]))
    if node.op == "reduce" and reduces is not None:
        reduces[node.uid] = node
    for a in node.args:
        _reads_from(a, seen, out, reduces)


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


def _reduce_init(fn, dt):
    if fn == "sum":
        return _literal(0, dt)
    if dt.is_floating:
        return _literal(float("-inf") if fn == "max" else float("inf"), dt)
    bits = dt.itemsize * 8
    if dt.kind == "u":
        return _literal(0 if fn == "max" else 2 ** bits - 1, dt)
    lo, hi = -(2 ** (bits - 1)), 2 ** (bits - 1) - 1
    # INT_MIN has no literal of its own
    return f"(({dt.ctype})({lo + 1}{'LL' if bits == 64 else ''} - 1))" if fn == "max" else _literal(hi, dt)


def _materialise_reduce(node, name, threads, reduced):
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
    body = _Body(reduced)
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
    if outs >= threads:
        # enough results for every thread to fold one of its own, serially
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
    return "\n  ".join(lines), outs * dt.itemsize


def _base_param(ptr):
    while ptr.op in ("ptradd", "ptrsub", "broadcast", "expand", "splat", "trans"):
        ptr = ptr.args[0]
    if ptr.op != "param":
        raise Unsupported("a pointer that is not derived from a kernel argument")
    return dict(ptr.attrs)["name"]


def generate(trace, num_warps):
    """Returns (cuda_source, kernel_name, [(param name, dtype or pointer_type)])."""
    if trace.loops:
        raise Unsupported("the program has a runtime loop")
    stores = []
    for eff in trace.effects:
        if eff[0] not in ("store", "atomic"):
            raise Unsupported(f"effect '{eff[0]}'")
        stores.append(eff)
    if not stores:
        raise Unsupported("the program stores nothing")

    threads = num_warps * THREADS_PER_WARP
    written = set()
    chunks = []
    reduced = {}        # reduce node uid -> (shared array, result shape)
    shared_decls = []
    shared_bytes = 0
    uses_atomic_max_f32 = False
    for eff in stores:
        _, ptr, value, mask, _lineno = eff[:5]
        atomic = eff[5] if eff[0] == "atomic" else None
        reads = set()
        reduces = {}
        for n in (value, mask, ptr):
            _reads_from(n, set(), reads, reduces)
        # Reductions are materialised in shared memory, in the order they were written (node ids
        # are in program order, so an inner reduction comes before the one that uses it).
        for uid in sorted(reduces):
            if uid in reduced:
                continue
            node = reduces[uid]
            name = f"nb_r{len(reduced)}"
            text, nbytes = _materialise_reduce(node, name, threads, reduced)
            shared_bytes += nbytes
            if shared_bytes > 40 * 1024:
                raise Unsupported("the reductions' results do not fit in shared memory")
            outs = max(nbytes // node.dtype.itemsize, 1)
            shared_decls.append(f"__shared__ {node.dtype.ctype} {name}[{outs}];")
            reduced[uid] = (name, () if dict(node.attrs)["axis"] is None else node.shape)
            chunks.append(text)
        # Loads are evaluated inside the statement that uses them, i.e. after earlier stores of
        # the program; the source program read them before.  Refuse the programs where that
        # could differ.
        clash = reads & written
        if clash:
            raise Unsupported(f"'{sorted(clash)[0]}' is read after the program stored to it")
        written.add(_base_param(ptr))

        shape = ptr.shape
        numel = 1
        for s in shape:
            numel *= s
        body = _Body(reduced)
        dims = tuple(f"i{d}" for d in range(len(shape)))
        p = _emit(body, ptr, dims)
        val = _convert(_emit(body, value, _operand_dims(shape, dims, value.shape)), value.dtype,
                       ptr.dtype.element)
        guard = _emit(body, mask, _operand_dims(shape, dims, mask.shape)) if mask is not None else None
        lines = []
        if shape:
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
        elem = ptr.dtype.element
        if atomic is None:
            store = f"*{p} = {val};"
        elif atomic == "add":
            if elem == tp.int64:
                store = f"atomicAdd(reinterpret_cast<unsigned long long*>({p}), (unsigned long long)({val}));"
            elif elem.name in ("float32", "float64", "float16", "bfloat16", "int32", "uint32"):
                store = f"atomicAdd({p}, {val});"
            else:
                raise Unsupported(f"nl.atomic_add on {elem.name}")
        else:
            if elem == tp.float32:
                uses_atomic_max_f32 = True
                store = f"nb_atomic_max_f32({p}, {val});"
            elif elem.name in ("int32", "uint32", "int64"):
                store = f"atomicMax({p}, {val});"
            else:
                raise Unsupported(f"nl.atomic_max on {elem.name}")
        lines.append(f"  if ({guard}) {store}" if guard else f"  {store}")
        lines.append("}")
        chunks.append("\n  ".join(lines))

    params = [(name, node.dtype) for name, node in trace.params.items()]
    # Elements are independent, so the loads of several iterations may be issued before the
    # stores of earlier ones; `__restrict__` says so (a tensor passed under two names is still
    # fine as long as element i is only read for element i, as in any in-place elementwise call).
    decl = ", ".join(f"{t.ctype} __restrict__ {name}" if isinstance(t, tp.pointer_type)
                     else f"{t.ctype} {name}" for name, t in params)
    body_text = "\n  __syncthreads();\n  ".join(chunks)
    helpers = ""
    if uses_atomic_max_f32:
        helpers += _ATOMIC_MAX_F32
    if reduced:
        helpers += _REDUCE_HELPERS
        shared_decls.insert(0, "__shared__ unsigned long long nb_scratch[32];")
        body_text = "\n  ".join(shared_decls) + "\n  " + body_text
    digest = hashlib.sha1((decl + body_text).encode()).hexdigest()[:8]
    kernel_name = f"{trace.name}_{digest}"
    source = (
        "#include <cuda_fp16.h>\n#include <cuda_bf16.h>\n" + helpers + "\n"
        f"extern \"C\" __global__ void __launch_bounds__({threads}) {kernel_name}({decl}) {{\n  "
        f"{body_text}\n}}\n")
    return source, kernel_name, params


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
        elif t.name in _CTYPES:
            out.append(_CTYPES[t.name](v))
        else:
            raise TypeError(f"argument '{name}': scalars of type {t.name} cannot be passed to a kernel")
    return out
