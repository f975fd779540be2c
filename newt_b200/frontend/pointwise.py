"""Generic lowering of loop-free, reduction-free block programs to CUDA text.

Everything the block language can say without `for`, `nl.dot` or a reduction is arithmetic
on blocks of compile-time shape: loads through pointer blocks, broadcasting, elementwise math,
`nl.where`, casts, masked stores.  Such a program needs no tuned kernel -- it is bound by HBM
and every output element depends on a fixed expression of loaded elements -- so it is
compiled at run time, like the reference compiles all programs: one CUDA block of
`num_warps * 32` threads per program instance; for each `nl.store`, the threads stride over
the elements of the stored block and evaluate the expression for their element.

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

    def __init__(self):
        self.lines = []
        self.memo = {}

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
            if cd.is_int:
                raise Unsupported("integer ** with a runtime exponent")
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
    raise Unsupported(f"'{op}' has no elementwise lowering")


def _reads_from(node, seen, out):
    """Names of the pointer parameters that `node`'s value loads from."""
    if not isinstance(node, Node) or node.uid in seen:
        return
    seen.add(node.uid)
    if node.op == "load":
        out.add(_base_param(node.args[0]))
    for a in node.args:
        _reads_from(a, seen, out)


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
        if eff[0] != "store":
            raise Unsupported(f"effect '{eff[0]}'")
        stores.append(eff)
    if not stores:
        raise Unsupported("the program stores nothing")

    threads = num_warps * THREADS_PER_WARP
    written = set()
    chunks = []
    for _, ptr, value, mask, _lineno in stores:
        reads = set()
        for n in (value, mask, ptr):
            _reads_from(n, set(), reads)
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
        body = _Body()
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
        store = f"*{p} = {val};"
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
    digest = hashlib.sha1((decl + body_text).encode()).hexdigest()[:8]
    kernel_name = f"{trace.name}_{digest}"
    source = (
        "#include <cuda_fp16.h>\n#include <cuda_bf16.h>\n\n"
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
