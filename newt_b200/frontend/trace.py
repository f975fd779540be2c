"""Symbolic evaluation of a `@jit` kernel body.

The reference walks the kernel's AST and prints CUDA C++ as it goes
(newt/compiler/codegen.py:780-1110 statements, :1114-1465 expressions).  This
front end walks the same AST but builds a small expression graph instead:
every block or runtime scalar is a `Node` (op, operands, static shape, dtype);
compile-time values (constexprs, Python literals, shapes) stay plain Python and
fold as they go, which is also how branches on constexprs are pruned
(reference: codegen.py:1067-1074).  Stores and runtime loops become entries of
an effect list.  `lower.py` then matches that graph against the hand-written
sm_100a kernels.

Kept from the reference's semantics, because results depend on them:
  * power-of-two block dims for arange/zeros/full (codegen.py:1490, 1506-1508);
  * a Python scalar combined with a block adopts the block's dtype
    (codegen.py:1211-1221); block (x) block promotes (types.py:86-99);
  * reductions of 16-bit floats produce fp32 (codegen.py:1908);
  * loop-carried values must keep shape and dtype (codegen.py:826-865).
"""

import ast
import math

from .. import types as tp


class CompileError(Exception):
    """A kernel uses the language in a way the compiler rejects."""


def _is_pow2(n):
    return isinstance(n, int) and n > 0 and (n & (n - 1)) == 0


class Node:
    """One value of the expression graph.  Nodes are interned per trace, so two
    structurally identical expressions are the same object."""

    __slots__ = ("op", "args", "attrs", "shape", "dtype", "uid")

    def __init__(self, op, args, attrs, shape, dtype, uid):
        self.op = op
        self.args = args
        self.attrs = attrs
        self.shape = shape
        self.dtype = dtype
        self.uid = uid

    @property
    def is_pointer(self):
        return isinstance(self.dtype, tp.pointer_type)

    def __repr__(self):
        a = ", ".join(f"%{x.uid}" if isinstance(x, Node) else repr(x) for x in self.args)
        extra = f" {self.attrs}" if self.attrs else ""
        return f"%{self.uid} = {self.op}({a}){extra} : {self.dtype}{list(self.shape)}"

    # blocks are not Python values: catch accidental host-side use
    def __bool__(self):
        raise CompileError("a block or runtime scalar cannot be used as a Python condition")


class Loop:
    """A `for v in range(lo, hi, step)` whose bounds are not all compile-time."""

    def __init__(self, uid, lo, hi, step, lineno, kind="for"):
        self.uid = uid
        self.kind = kind         # "for" (range) or "while"
        self.lo, self.hi, self.step = lo, hi, step
        self.cond = None         # while: scalar bool Node over the carried placeholders
        self.lineno = lineno
        self.var = None          # Node 'loopvar'
        self.carried = {}        # name -> (placeholder Node, init, next)
        self.escaping = {}       # same triples for names first bound inside the body and visible
                                 # after the loop with their last value (zero when it never ran)
        self.effects = []        # effects issued inside the body

    @property
    def values(self):
        """Everything the loop hands on: carried names and names that escape the body."""
        return {**self.escaping, **self.carried}


class Trace:
    """Result of tracing one specialization."""

    def __init__(self, name):
        self.name = name
        self.effects = []        # ("store", ptr, value, mask, lineno) | ("for", Loop)
                                 # | ("atomic", ptr, value, mask, lineno, "add" | "max")
        self.loops = []
        self.params = {}         # runtime parameter name -> Node
        self.constexprs = {}
        self.nodes = []

    def dump(self):
        return "\n".join(repr(n) for n in self.nodes)


_BINOPS = {ast.Add: "add", ast.Sub: "sub", ast.Mult: "mul", ast.Div: "div",
           ast.FloorDiv: "floordiv", ast.Mod: "mod", ast.Pow: "pow",
           ast.BitAnd: "and", ast.BitOr: "or", ast.BitXor: "xor",
           ast.LShift: "shl", ast.RShift: "shr"}
_CMPOPS = {ast.Lt: "lt", ast.LtE: "le", ast.Gt: "gt", ast.GtE: "ge", ast.Eq: "eq",
           ast.NotEq: "ne"}
_PY_BIN = {"add": lambda a, b: a + b, "sub": lambda a, b: a - b, "mul": lambda a, b: a * b,
           "div": lambda a, b: a / b, "floordiv": lambda a, b: a // b,
           "mod": lambda a, b: a % b, "pow": lambda a, b: a ** b, "and": lambda a, b: a & b,
           "or": lambda a, b: a | b, "xor": lambda a, b: a ^ b, "shl": lambda a, b: a << b,
           "shr": lambda a, b: a >> b}
_PY_CMP = {"lt": lambda a, b: a < b, "le": lambda a, b: a <= b, "gt": lambda a, b: a > b,
           "ge": lambda a, b: a >= b, "eq": lambda a, b: a == b, "ne": lambda a, b: a != b}
_MATH1 = ("exp", "exp2", "log", "log2", "sqrt", "rsqrt", "sin", "cos", "tanh", "erf",
          "sigmoid", "abs", "floor", "ceil")
_HOST_CALLS = {"float": float, "int": int, "bool": bool, "min": min, "max": max, "abs": abs,
               "len": len, "tuple": tuple, "list": list, "range": range, "isinstance": isinstance}


class _PromoteScalar(Exception):
    """Internal: a Python number is changed inside a runtime loop; trace the loop again with
    it as a typed scalar."""

    def __init__(self, name):
        super().__init__(name)
        self.name = name


def _unwrap_constexpr(v):
    from .. import language as nl

    return v.value if isinstance(v, nl.constexpr) else v


class Tracer(ast.NodeVisitor):
    def __init__(self, fndef, fn_globals, runtime_types, constexprs, num_warps=4):
        self.fndef = fndef
        self.globals = fn_globals
        self.trace = Trace(fndef.name)
        self.trace.constexprs = dict(constexprs)
        self._intern = {}
        self.env = {}
        self.effects = self.trace.effects
        self.num_warps = num_warps
        self._loop_ids = 0
        self._pred = None        # scalar bool Node: condition of the enclosing runtime `if`s
        self._depth = 0          # enclosing loops; names the `break`/`continue` flags in env
        for name, val in constexprs.items():
            self.env[name] = _unwrap_constexpr(val)
        for name, t in runtime_types.items():
            node = self.node("param", (), (("name", name),), (), t)
            self.trace.params[name] = node
            self.env[name] = node

    # ---- infrastructure ------------------------------------------------------

    def err(self, where, msg):
        line = getattr(where, "lineno", "?")
        raise CompileError(f"{self.fndef.name}:{line}: {msg}")

    def node(self, op, args, attrs, shape, dtype):
        key = (op, tuple(("n", a.uid) if isinstance(a, Node) else ("c", repr(a)) for a in args),
               attrs, tuple(shape), dtype.name if dtype is not None else None)
        hit = self._intern.get(key)
        if hit is None:
            hit = Node(op, tuple(args), attrs, tuple(shape), dtype, len(self.trace.nodes))
            self.trace.nodes.append(hit)
            self._intern[key] = hit
        return hit

    def run(self):
        self._block(self.fndef.body)
        return self.trace

    # ---- break / continue ------------------------------------------------------
    #
    # Each enclosing loop has two flags in the environment, "\0brk<depth>" and "\0cont<depth>"
    # (names no source can spell): False, True, or a scalar bool node once a `break` or
    # `continue` ran under a runtime condition.  They are ordinary variables, so the merge at
    # the end of a runtime `if` turns `if c: break` into `brk = where(c, True, brk)`.  While a
    # flag is a node the rest of the iteration still runs, with memory accesses masked and
    # assignments keeping the old value where the flag is set.

    def _flag(self, kind, depth=None):
        return f"\0{kind}{self._depth if depth is None else depth}"

    def _skip(self, where=None):
        """True / False / node: are the statements that follow skipped?"""
        acc = False
        for depth in range(1, self._depth + 1):
            for kind in ("brk", "cont"):
                f = self.env.get(self._flag(kind, depth), False)
                if f is True:
                    return True
                if isinstance(f, Node):
                    acc = f if acc is False else self.binop("or", acc, f, where)
        return acc

    def _block(self, stmts):
        for stmt in stmts:
            if self._skip(stmt) is True:
                return
            self.visit(stmt)

    def _jump(self, node, kind):
        if self._depth == 0:
            self.err(node, f"`{'break' if kind == 'brk' else 'continue'}` outside a loop")
        skip = self._skip(node)
        name = self._flag(kind)
        if skip is False:
            self.env[name] = True
        else:       # taken only where the iteration is still live
            live = self.node("not", (skip,), (), (), tp.int1)
            self.env[name] = self.binop("or", self.env.get(name, False), live, node)

    def visit_Break(self, node):
        self._jump(node, "brk")

    def visit_Continue(self, node):
        self._jump(node, "cont")

    @staticmethod
    def _own_jumps(body, kind):
        """Does `body` hold a break/continue that belongs to this loop (not to a nested one)?"""
        todo = list(body)
        while todo:
            n = todo.pop()
            if isinstance(n, kind):
                return True
            if isinstance(n, (ast.For, ast.While)):
                continue
            todo += list(ast.iter_child_nodes(n))
        return False

    # ---- value helpers ---------------------------------------------------------

    def as_node(self, v, like=None, where=None):
        """Materialise a Python scalar as a constant node; `like` gives the dtype
        a scalar adopts when it meets a block."""
        if isinstance(v, Node):
            return v
        if isinstance(v, bool):
            dt = tp.int1
        elif isinstance(v, int):
            dt = like if like is not None and not isinstance(like, tp.pointer_type) else tp.int32
            if like is None and not -(2 ** 31) <= v < 2 ** 31:
                dt = tp.int64
        elif isinstance(v, float):
            dt = like if (like is not None and getattr(like, "is_floating", False)) else tp.float32
        else:
            self.err(where, f"cannot use {type(v).__name__} value {v!r} as a kernel value")
        return self.node("const", (v,), (), (), dt)

    def binop(self, op, a, b, where):
        a, b = _unwrap_constexpr(a), _unwrap_constexpr(b)
        if not isinstance(a, Node) and not isinstance(b, Node):
            try:
                return _PY_BIN[op](a, b)
            except Exception as e:  # noqa: BLE001
                self.err(where, f"constant expression failed: {e}")
        an = a if isinstance(a, Node) else None
        bn = b if isinstance(b, Node) else None
        # pointer arithmetic: pointer +/- integer
        if (an is not None and an.is_pointer) or (bn is not None and bn.is_pointer):
            if op not in ("add", "sub") or (bn is not None and bn.is_pointer and op == "sub"):
                self.err(where, "pointers support only `ptr + int` and `ptr - int`")
            ptr, off = (an, b) if an is not None and an.is_pointer else (bn, a)
            if isinstance(off, Node):
                if off.is_pointer:
                    self.err(where, "cannot add two pointers")
                if not off.dtype.is_int:
                    self.err(where, "pointer offsets must be integers")
            elif not isinstance(off, int) or isinstance(off, bool):
                self.err(where, "pointer offsets must be integers")
            off = self.as_node(off, tp.int32, where)
            shape = tp.broadcast_shapes(ptr.shape, off.shape)
            return self.node("ptradd" if op == "add" else "ptrsub", (ptr, off), (), shape, ptr.dtype)
        # scalar adopts the block's dtype; two nodes promote
        if an is None:
            a = self.as_node(a, self._adopt(a, bn.dtype), where)
        if bn is None:
            b = self.as_node(b, self._adopt(b, an.dtype), where)
        dt = tp.promote(a.dtype, b.dtype)
        if op == "div" and dt.is_int:
            pass  # int / int stays integer division, as in the reference's C lowering
        if op in ("and", "or", "xor", "shl", "shr", "mod", "floordiv") and not dt.is_int \
                and op not in ("mod", "floordiv"):
            self.err(where, f"operator '{op}' needs integer or bool operands")
        try:
            shape = tp.broadcast_shapes(a.shape, b.shape)
        except TypeError as e:
            self.err(where, str(e))
        return self.node("bin", (a, b), (("fn", op),), shape, dt)

    @staticmethod
    def _adopt(scalar, block_dt):
        if isinstance(scalar, bool):
            return tp.int1
        if isinstance(scalar, float) and not block_dt.is_floating:
            return tp.float32
        return block_dt

    def compare(self, op, a, b, where):
        a, b = _unwrap_constexpr(a), _unwrap_constexpr(b)
        if not isinstance(a, Node) and not isinstance(b, Node):
            return _PY_CMP[op](a, b)
        if not isinstance(a, Node):
            a = self.as_node(a, self._adopt(a, b.dtype), where)
        if not isinstance(b, Node):
            b = self.as_node(b, self._adopt(b, a.dtype), where)
        try:
            shape = tp.broadcast_shapes(a.shape, b.shape)
        except TypeError as e:
            self.err(where, str(e))
        return self.node("cmp", (a, b), (("fn", op),), shape, tp.int1)

    # ---- statements --------------------------------------------------------------

    def generic_visit(self, node):
        self.err(node, f"unsupported syntax: {type(node).__name__}")

    def visit_Expr(self, node):
        if isinstance(node.value, ast.Constant):
            return  # docstring
        self.eval(node.value)

    def visit_Pass(self, node):
        pass

    def visit_Assert(self, node):
        pass  # host-level asserts are ignored on the device (newt/compiler/codegen.py:1104-1105)

    def visit_Return(self, node):
        if node.value is not None:
            self.err(node, "kernels cannot return a value")
        self.err(node, "early `return` is not supported by the sm_100a front end yet")

    def _bind(self, name, value, where):
        """`name = value`, keeping the old value where a conditional break/continue has already
        ended the iteration."""
        skip = self._skip(where)
        old = self.env.get(name)
        if isinstance(skip, Node) and old is not None and old is not value:
            scalar = (Node, int, float, bool)
            if not isinstance(old, scalar) or not isinstance(_unwrap_constexpr(value), scalar):
                self.err(where, f"'{name}' is a compile-time object assigned after a conditional "
                                f"break/continue")
            if isinstance(old, Node) and old.is_pointer or isinstance(value, Node) and value.is_pointer:
                self.err(where, f"pointer '{name}' is assigned after a conditional break/continue")
            value = self.b_where(where, skip, old, value)
        self.env[name] = value

    def _assign(self, target, value, where):
        if isinstance(target, ast.Name):
            self._bind(target.id, value, where)
        elif isinstance(target, (ast.Tuple, ast.List)):
            if not isinstance(value, (tuple, list)) or len(value) != len(target.elts):
                self.err(where, "cannot unpack: shapes of target and value differ")
            for t, v in zip(target.elts, value):
                self._assign(t, v, where)
        else:
            self.err(where, "assignment targets must be names (blocks are immutable values)")

    def visit_Assign(self, node):
        value = self.eval(node.value)
        for t in node.targets:
            self._assign(t, value, node)

    def visit_AnnAssign(self, node):
        if node.value is not None:
            self._assign(node.target, self.eval(node.value), node)

    def visit_AugAssign(self, node):
        if not isinstance(node.target, ast.Name):
            self.err(node, "augmented assignment needs a plain name")
        if node.target.id not in self.env:
            self.err(node, f"'{node.target.id}' is not defined")
        cur = self.env[node.target.id]
        op = _BINOPS.get(type(node.op))
        if op is None:
            self.err(node, f"unsupported operator {type(node.op).__name__}")
        self._bind(node.target.id, self.binop(op, cur, self.eval(node.value), node), node)

    def visit_If(self, node):
        cond = _unwrap_constexpr(self.eval(node.test))
        if isinstance(cond, Node):
            if cond.shape != ():
                self.err(node, "`if` takes a scalar condition, this one is a block: use nl.where for "
                               "elementwise selection")
            return self._runtime_if(node, cond)
        self._block(node.body if cond else node.orelse)

    def _runtime_if(self, node, cond):
        """`if` on a runtime scalar, by if-conversion: both arms are traced, loads, stores and
        atomics inside them are masked by the (negated) condition, and every name the arms
        leave different is merged with a select.  All programs of a grid run the same
        instructions either way; only the taken arm touches memory."""
        if cond.dtype != tp.int1:
            cond = self.compare("ne", cond, 0, node)
        before = dict(self.env)
        outer = self._pred

        def arm(stmts, c):
            self.env = dict(before)
            self._pred = c if outer is None else self.binop("and", outer, c, node)
            self._block(stmts)
            return self.env

        then_env = arm(node.body, cond)
        else_env = arm(node.orelse, self.node("not", (cond,), (), (), tp.int1))
        self._pred = outer
        merged = dict(before)
        for name in sorted(set(then_env) | set(else_env)):
            a, b = then_env.get(name, before.get(name)), else_env.get(name, before.get(name))
            if a is b:
                merged[name] = a
                continue
            if a is None or b is None:
                merged.pop(name, None)       # defined in one arm only: unusable afterwards
                continue
            if not isinstance(a, (Node, int, float, bool)) or not isinstance(b, (Node, int, float, bool)):
                if a == b:
                    merged[name] = a
                    continue
                self.err(node, f"'{name}' is bound to different compile-time objects in the two "
                               f"arms of a runtime `if`")
            if isinstance(a, Node) and a.is_pointer or isinstance(b, Node) and b.is_pointer:
                self.err(node, f"'{name}': a runtime `if` cannot choose between pointers")
            merged[name] = self.b_where(node, cond, a, b)
        self.env = merged

    def visit_While(self, node):
        if node.orelse:
            self.err(node, "while/else is not supported")
        self._retry_promoting(node, lambda promote: self._symbolic_loop(node, None, None, None, promote))

    def visit_For(self, node):
        if node.orelse:
            self.err(node, "for/else is not supported")
        it = node.iter
        if not (isinstance(it, ast.Call) and isinstance(it.func, ast.Name) and it.func.id == "range"):
            self.err(node, "loops must iterate over range(...)")
        if not isinstance(node.target, ast.Name):
            self.err(node, "the loop variable must be a plain name")
        args = [_unwrap_constexpr(self.eval(a)) for a in it.args]
        if not 1 <= len(args) <= 3:
            self.err(node, "range() takes 1 to 3 arguments")
        lo, hi, step = (0, args[0], 1) if len(args) == 1 else \
            (args[0], args[1], args[2] if len(args) == 3 else 1)
        for b in (lo, hi, step):
            if isinstance(b, Node) and (b.shape != () or not b.dtype.is_int):
                self.err(node, "range() bounds must be integer scalars")
        if not any(isinstance(b, Node) for b in (lo, hi, step)):
            self._depth += 1                  # compile-time loop: unrolled
            brk, cont = self._flag("brk"), self._flag("cont")
            self.env[brk] = False
            for i in range(lo, hi, step):
                if self.env[brk] is True:
                    break
                self.env[node.target.id] = i
                self.env[cont] = False
                self._block(node.body)
            # a flag that became a node has done its work: every later assignment and access
            # of the loop was guarded by it
            self.env.pop(cont, None)
            self.env.pop(brk, None)
            self._depth -= 1
            return
        self._retry_promoting(node, lambda promote: self._symbolic_loop(node, lo, hi, step, promote))

    def _retry_promoting(self, node, trace_loop):
        """Traces a runtime loop; a Python number that the body changes is made a typed scalar
        of the program and the loop is traced again (`s = 0; for i in range(n): s += i`)."""
        promote = set()
        while True:
            env, n_eff, n_loops = dict(self.env), len(self.effects), len(self.trace.loops)
            effects, depth, pred = self.effects, self._depth, self._pred
            try:
                return trace_loop(promote)
            except _PromoteScalar as e:
                if e.name in promote:
                    raise
                promote.add(e.name)
                self.env, self.effects, self._depth, self._pred = env, effects, depth, pred
                del self.effects[n_eff:]
                del self.trace.loops[n_loops:]

    def _symbolic_loop(self, node, lo, hi, step, promote=()):
        self._loop_ids += 1
        is_while = isinstance(node, ast.While)
        loop = Loop(self._loop_ids, lo, hi, step, node.lineno, "while" if is_while else "for")
        self.trace.loops.append(loop)
        assigned = set()
        for sub in node.body:
            for n in ast.walk(sub):
                if isinstance(n, ast.Name) and isinstance(n.ctx, ast.Store):
                    assigned.add(n.id)
        if not is_while:
            assigned.discard(node.target.id)
        self._depth += 1
        brk, cont = self._flag("brk"), self._flag("cont")
        self.env[brk] = False
        if self._own_jumps(node.body, ast.Break):
            self.env[brk] = self.as_node(False)     # carried: a break also ends later iterations
            assigned.add(brk)
        placeholders = {}
        for name in sorted(assigned):
            init = self.env.get(name)
            if name in promote and isinstance(init, (int, float)) and not isinstance(init, bool):
                init = self.as_node(init, None, node)
            if isinstance(init, Node):
                ph = self.node("carried", (), (("loop", loop.uid), ("name", name)), init.shape,
                               init.dtype)
                placeholders[name] = (ph, init)
                self.env[name] = ph
            elif name in self.env:
                placeholders[name] = (None, init)
        if is_while:
            cond = _unwrap_constexpr(self.eval(node.test))
            if not isinstance(cond, Node):
                self.err(node, "`while` on a compile-time condition: " +
                         ("it would never end" if cond else "the body never runs; remove it"))
            if cond.shape != ():
                self.err(node, "`while` on a block: the condition must be a scalar")
            loop.cond = cond if cond.dtype == tp.int1 else self.compare("ne", cond, 0, node)
            if isinstance(self.env[brk], Node):
                loop.cond = self.binop("and", loop.cond,
                                       self.node("not", (self.env[brk],), (), (), tp.int1), node)
        else:
            loop.var = self.node("loopvar", (), (("loop", loop.uid),), (), tp.int32)
            self.env[node.target.id] = loop.var
        outer_effects, self.effects = self.effects, loop.effects
        self.env[cont] = False
        self._block(node.body)
        self.effects = outer_effects
        self.env.pop(cont, None)
        self._depth -= 1
        for name, (ph, init) in placeholders.items():
            nxt = self.env[name]
            if ph is None:
                if nxt is not init and nxt != init:
                    if isinstance(init, (int, float)) and not isinstance(init, bool):
                        raise _PromoteScalar(name)
                    self.err(node, f"'{name}' is a compile-time value changed inside a runtime loop")
                continue
            if nxt is ph:
                self.env[name] = init  # never reassigned: not loop-carried
                continue
            if not isinstance(nxt, Node):
                nxt = self.as_node(nxt, init.dtype, node)
            if nxt.shape != init.shape and nxt.shape != ():
                self.err(node, f"loop-carried '{name}' changes shape {init.shape} -> {nxt.shape}")
            if nxt.is_pointer != init.is_pointer:
                self.err(node, f"loop-carried '{name}' changes between pointer and value")
            if not init.is_pointer and nxt.dtype != init.dtype:
                if init.dtype.is_int and nxt.dtype.is_floating:
                    self.err(node, f"loop-carried '{name}' is stored as {init.dtype.name} but "
                                   f"updated with {nxt.dtype.name}")
                nxt = self.cast(nxt, init.dtype)
            loop.carried[name] = (ph, init, nxt)
            self.env[name] = self.node("loopout", (), (("loop", loop.uid), ("name", name)),
                                       init.shape, init.dtype)
        self.env.pop(brk, None)
        for name in sorted(assigned):
            value = self.env.get(name)
            if name in placeholders or name.startswith("\0") or not isinstance(value, Node) \
                    or value.is_pointer:
                continue
            # first bound inside the body: afterwards it holds the last iteration's value
            # (the reference declares such names before the loop, newt/compiler/codegen.py:93-157)
            ph = self.node("carried", (), (("loop", loop.uid), ("name", name)), value.shape, value.dtype)
            zero = self.node("full", (False if value.dtype == tp.int1 else 0,), (), value.shape, value.dtype)
            loop.escaping[name] = (ph, zero, value)
            self.env[name] = self.node("loopout", (), (("loop", loop.uid), ("name", name)),
                                       value.shape, value.dtype)
        self.effects.append(("while" if is_while else "for", loop))

    # ---- expressions -----------------------------------------------------------------

    def eval(self, node):
        method = getattr(self, "e_" + type(node).__name__, None)
        if method is None:
            self.err(node, f"unsupported expression: {type(node).__name__}")
        return method(node)

    def e_Constant(self, node):
        return node.value

    def e_Name(self, node):
        if node.id in self.env:
            return self.env[node.id]
        if node.id in self.globals:
            return self.globals[node.id]
        if node.id in _HOST_CALLS:
            return _HOST_CALLS[node.id]
        self.err(node, f"name '{node.id}' is not defined")

    def e_Tuple(self, node):
        return tuple(self.eval(e) for e in node.elts)

    e_List = e_Tuple

    def e_Attribute(self, node):
        base = self.eval(node.value)
        if isinstance(base, Node):
            if node.attr == "dtype":
                return base.dtype
            if node.attr == "shape":
                return base.shape
            if node.attr == "T":
                return self.b_trans(node, base)
            if node.attr == "to":
                return lambda dt, _n=node, _b=base: self.b_cast(_n, _b, dt)
            self.err(node, f"blocks have no attribute '{node.attr}'")
        try:
            return getattr(base, node.attr)
        except AttributeError:
            self.err(node, f"{base!r} has no attribute '{node.attr}'")

    def e_BinOp(self, node):
        op = _BINOPS.get(type(node.op))
        if op is None:
            self.err(node, f"unsupported operator {type(node.op).__name__}")
        return self.binop(op, self.eval(node.left), self.eval(node.right), node)

    def e_UnaryOp(self, node):
        v = _unwrap_constexpr(self.eval(node.operand))
        if isinstance(node.op, ast.USub):
            return self.node("neg", (v,), (), v.shape, v.dtype) if isinstance(v, Node) else -v
        if isinstance(node.op, ast.UAdd):
            return v
        if isinstance(node.op, ast.Not):
            if isinstance(v, Node):
                return self.node("not", (v,), (), v.shape, tp.int1)
            return not v
        if isinstance(node.op, ast.Invert):
            if isinstance(v, Node):
                return self.node("not" if v.dtype == tp.int1 else "inv", (v,), (), v.shape, v.dtype)
            return ~v
        self.err(node, "unsupported unary operator")

    def e_Compare(self, node):
        if len(node.ops) != 1:
            self.err(node, "chained comparisons are not supported")
        op = _CMPOPS.get(type(node.ops[0]))
        if op is None:
            self.err(node, "unsupported comparison")
        return self.compare(op, self.eval(node.left), self.eval(node.comparators[0]), node)

    def e_BoolOp(self, node):
        vals = [_unwrap_constexpr(self.eval(v)) for v in node.values]
        if any(isinstance(v, Node) for v in vals):
            fn = "and" if isinstance(node.op, ast.And) else "or"
            acc = vals[0]
            for v in vals[1:]:
                acc = self.binop(fn, acc, v, node)
            return acc
        if isinstance(node.op, ast.And):
            return all(vals)
        return any(vals)

    def e_IfExp(self, node):
        cond = _unwrap_constexpr(self.eval(node.test))
        if isinstance(cond, Node):
            self.err(node, "conditional expressions need a compile-time condition; use nl.where")
        return self.eval(node.body if cond else node.orelse)

    def e_Subscript(self, node):
        base = self.eval(node.value)
        idx = node.slice
        if not isinstance(base, Node):
            key = self.eval(idx)
            try:
                return base[key]
            except Exception as e:  # noqa: BLE001
                self.err(node, f"cannot index {base!r}: {e}")
        elts = idx.elts if isinstance(idx, ast.Tuple) else [idx]
        out = base
        axis = 0
        for e in elts:
            if isinstance(e, ast.Constant) and e.value is None:
                out = self.b_expand_dims(node, out, axis)
                axis += 1
            elif isinstance(e, ast.Slice) and e.lower is None and e.upper is None and e.step is None:
                axis += 1
            else:
                self.err(node, "blocks support only ':' and None subscripts")
        if axis - sum(1 for e in elts if isinstance(e, ast.Constant)) > len(base.shape):
            self.err(node, "too many indices for block")
        return out

    def e_Call(self, node):
        fn = self.eval(node.func)
        args = [self.eval(a) for a in node.args]
        kwargs = {k.arg: self.eval(k.value) for k in node.keywords}
        name = getattr(fn, "_newt_builtin", None)
        if name is not None:
            impl = getattr(self, "b_" + name, None)
            if impl is None:
                self.err(node, f"nl.{name} is not supported by the sm_100a front end yet")
            try:
                return impl(node, *args, **kwargs)
            except TypeError as e:
                if "b_" + name in str(e) or "argument" in str(e):
                    self.err(node, f"bad call to nl.{name}: {e}")
                raise
        if any(isinstance(a, Node) for a in list(args) + list(kwargs.values())) and \
                not getattr(fn, "__name__", "") == "<lambda>":
            self.err(node, f"cannot call {getattr(fn, '__name__', fn)!r} on kernel values")
        try:
            return fn(*[_unwrap_constexpr(a) for a in args],
                      **{k: _unwrap_constexpr(v) for k, v in kwargs.items()})
        except CompileError:
            raise
        except Exception as e:  # noqa: BLE001
            self.err(node, f"call to {getattr(fn, '__name__', fn)!r} failed: {e}")

    # ---- builtins ---------------------------------------------------------------------

    def _shape_arg(self, where, shape):
        shape = _unwrap_constexpr(shape)
        if isinstance(shape, int):
            shape = (shape,)
        shape = tuple(int(_unwrap_constexpr(s)) for s in shape)
        for s in shape:
            if not _is_pow2(s):
                self.err(where, f"block dimensions must be powers of two, got {shape}")
        return shape

    def _dtype_arg(self, where, dt):
        if not isinstance(dt, tp.dtype):
            self.err(where, f"expected a dtype such as nl.float32, got {dt!r}")
        return dt

    def b_program_id(self, where, axis):
        axis = _unwrap_constexpr(axis)
        if axis not in (0, 1, 2):
            self.err(where, "program_id axis must be 0, 1 or 2")
        return self.node("pid", (), (("axis", axis),), (), tp.int32)

    def b_num_programs(self, where, axis):
        axis = _unwrap_constexpr(axis)
        if axis not in (0, 1, 2):
            self.err(where, "num_programs axis must be 0, 1 or 2")
        return self.node("nprog", (), (("axis", axis),), (), tp.int32)

    def b_arange(self, where, start, end):
        start, end = _unwrap_constexpr(start), _unwrap_constexpr(end)
        if not isinstance(start, int) or not isinstance(end, int):
            self.err(where, "arange bounds must be compile-time integers")
        if not _is_pow2(end - start):
            self.err(where, f"arange length must be a power of two, got {end - start}")
        return self.node("arange", (start, end), (), (end - start,), tp.int32)

    def b_zeros(self, where, shape, dtype=tp.float32):
        return self.b_full(where, shape, 0, dtype)

    def b_full(self, where, shape, value, dtype=tp.float32):
        shape = self._shape_arg(where, shape)
        dtype = self._dtype_arg(where, _unwrap_constexpr(dtype))
        value = _unwrap_constexpr(value)
        if isinstance(value, Node):
            if value.shape != ():
                self.err(where, "nl.full needs a scalar fill value")
            return self.node("splat", (self.cast(value, dtype),), (), shape, dtype)
        return self.node("full", (float(value) if dtype.is_floating else int(value),), (), shape,
                         dtype)

    def b_load(self, where, pointer, mask=None, other=None):
        if not isinstance(pointer, Node) or not pointer.is_pointer:
            self.err(where, "nl.load needs a pointer or a block of pointers")
        mask = self._predicated(where, self._mask_arg(where, mask, pointer.shape))
        elem = pointer.dtype.element
        other = _unwrap_constexpr(other)
        if other is not None and not isinstance(other, Node):
            other = float(other) if elem.is_floating else int(other)
        if other is not None and mask is None:
            other = None
        return self.node("load", (pointer, mask, other), (), pointer.shape, elem)

    def _mask_arg(self, where, mask, shape):
        mask = _unwrap_constexpr(mask)
        if mask is None:
            return None
        if not isinstance(mask, Node):
            if mask is True:
                return None
            self.err(where, "mask must be a bool block")
        if shape == () and mask.shape != ():
            self.err(where, "a scalar pointer cannot take a block mask")
        try:
            if tp.broadcast_shapes(mask.shape, shape) != tuple(shape):
                raise TypeError
        except TypeError:
            self.err(where, f"mask shape {mask.shape} does not broadcast to {tuple(shape)}")
        return mask

    def _predicated(self, where, mask):
        """Inside the arm of a runtime `if`, memory is only touched where the arm is taken."""
        if self._pred is None:
            return mask
        return self._pred if mask is None else self.binop("and", mask, self._pred, where)

    def b_store(self, where, pointer, value, mask=None):
        if not isinstance(pointer, Node) or not pointer.is_pointer:
            self.err(where, "nl.store needs a pointer or a block of pointers")
        value = _unwrap_constexpr(value)
        if not isinstance(value, Node):
            value = self.as_node(value, pointer.dtype.element, where)
        try:
            if tp.broadcast_shapes(value.shape, pointer.shape) != pointer.shape:
                raise TypeError
        except TypeError:
            self.err(where, f"cannot store a {value.shape} block through {pointer.shape} pointers")
        mask = self._predicated(where, self._mask_arg(where, mask, pointer.shape))
        self.effects.append(("store", pointer, value, mask, getattr(where, "lineno", 0)))

    def _atomic(self, where, fn, pointer, value, mask):
        """nl.atomic_add / nl.atomic_max: a side effect, no value (newt/compiler/codegen.py:
        1750-1800).  Through a scalar pointer it is one update per program and takes a scalar."""
        if not isinstance(pointer, Node) or not pointer.is_pointer:
            self.err(where, f"nl.atomic_{fn} needs a pointer or a block of pointers")
        value = _unwrap_constexpr(value)
        if not isinstance(value, Node):
            value = self.as_node(value, pointer.dtype.element, where)
        mask = self._predicated(where, self._mask_arg(where, mask, pointer.shape))
        if pointer.shape == () and value.shape != ():
            self.err(where, "scalar-pointer atomic with a block value; reduce it first")
        try:
            if tp.broadcast_shapes(value.shape, pointer.shape) != pointer.shape:
                raise TypeError
        except TypeError:
            self.err(where, f"cannot apply a {value.shape} block through {pointer.shape} pointers")
        self.effects.append(("atomic", pointer, value, mask, getattr(where, "lineno", 0), fn))

    def b_atomic_add(self, where, pointer, value, mask=None):
        self._atomic(where, "add", pointer, value, mask)

    def b_atomic_max(self, where, pointer, value, mask=None):
        self._atomic(where, "max", pointer, value, mask)

    def b_expand_dims(self, where, x, axis):
        axis = _unwrap_constexpr(axis)
        if not isinstance(x, Node):
            self.err(where, "expand_dims needs a block")
        if axis < 0:
            axis += len(x.shape) + 1
        shape = x.shape[:axis] + (1,) + x.shape[axis:]
        return self.node("expand", (x,), (("axis", axis),), shape, x.dtype)

    def b_broadcast_to(self, where, x, shape):
        shape = self._shape_arg(where, shape)
        x = self.as_node(_unwrap_constexpr(x), None, where)
        try:
            if tp.broadcast_shapes(x.shape, shape) != shape:
                raise TypeError
        except TypeError:
            self.err(where, f"cannot broadcast {x.shape} to {shape}")
        return self.node("broadcast", (x,), (), shape, x.dtype)

    def b_reshape(self, where, x, shape):
        shape = self._shape_arg(where, shape)
        if math.prod(shape) != math.prod(x.shape):
            self.err(where, f"reshape {x.shape} -> {shape} changes the element count")
        return self.node("reshape", (x,), (), shape, x.dtype)

    def b_trans(self, where, x):
        if not isinstance(x, Node) or len(x.shape) != 2:
            self.err(where, "nl.trans needs a 2-D block")
        return self.node("trans", (x,), (), (x.shape[1], x.shape[0]), x.dtype)

    def cast(self, x, dtype):
        if x.dtype == dtype:
            return x
        return self.node("cast", (x,), (), x.shape, dtype)

    def b_cast(self, where, x, dtype):
        dtype = self._dtype_arg(where, _unwrap_constexpr(dtype))
        x = _unwrap_constexpr(x)
        if not isinstance(x, Node):
            x = self.as_node(x, dtype, where)
        if x.is_pointer:
            self.err(where, "pointers cannot be cast")
        return self.cast(x, dtype)

    def _reduce(self, where, fn, x, axis):
        if not isinstance(x, Node) or x.shape == ():
            self.err(where, f"nl.{fn} needs a block")
        axis = _unwrap_constexpr(axis)
        dt = x.dtype
        if dt in (tp.float16, tp.bfloat16):
            dt = tp.float32
        if dt == tp.int1 and fn == "sum":
            dt = tp.int32
        if axis is None:
            shape = ()
        else:
            if axis < 0:
                axis += len(x.shape)
            if not 0 <= axis < len(x.shape):
                self.err(where, f"axis {axis} out of range for a {len(x.shape)}-D block")
            shape = x.shape[:axis] + x.shape[axis + 1:]
            if len(x.shape) == 1:
                axis = None
        return self.node("reduce", (x,), (("fn", fn), ("axis", axis)), shape, dt)

    def b_sum(self, where, x, axis=None):
        return self._reduce(where, "sum", x, axis)

    def b_max(self, where, x, axis=None):
        return self._reduce(where, "max", x, axis)

    def b_min(self, where, x, axis=None):
        return self._reduce(where, "min", x, axis)

    def b_dot(self, where, a, b, acc=None, out_dtype=tp.float32):
        for name, v in (("a", a), ("b", b)):
            if not isinstance(v, Node) or len(v.shape) != 2:
                self.err(where, f"nl.dot operand '{name}' must be a 2-D block")
        if a.dtype != b.dtype:
            self.err(where, f"nl.dot operands must share a dtype, got {a.dtype.name} and "
                            f"{b.dtype.name}")
        if a.dtype not in (tp.float16, tp.bfloat16, tp.float32):
            self.err(where, f"nl.dot does not support {a.dtype.name} operands")
        m, k = a.shape
        k2, n = b.shape
        if k != k2:
            self.err(where, f"nl.dot inner dimensions differ: {a.shape} @ {b.shape}")
        if m % 16 or n % 16 or k % (8 if a.dtype == tp.float32 else 16):
            self.err(where, f"nl.dot needs M, N multiples of 16 and K a multiple of "
                            f"{8 if a.dtype == tp.float32 else 16}; got {m}x{k} @ {k2}x{n}")
        acc = _unwrap_constexpr(acc)
        if acc is not None:
            if not isinstance(acc, Node) or acc.shape != (m, n):
                self.err(where, f"nl.dot accumulator must be a {(m, n)} block")
            if acc.dtype != tp.float32:
                self.err(where, "nl.dot accumulates in float32")
        return self.node("dot", (a, b, acc), (), (m, n), tp.float32)

    def _math1(self, fn):
        def impl(where, x):
            x = _unwrap_constexpr(x)
            if not isinstance(x, Node):
                x = self.as_node(float(x) if fn != "abs" else x, None, where)
            dt = x.dtype
            if fn not in ("abs",) and not dt.is_floating:
                dt = tp.float32
                x = self.cast(x, dt)
            return self.node("math", (x,), (("fn", fn),), x.shape, dt)
        return impl

    def __getattr__(self, name):
        if name.startswith("b_") and name[2:] in _MATH1:
            return self._math1(name[2:])
        raise AttributeError(name)

    def _binary_fn(self, where, fn, a, b):
        a, b = _unwrap_constexpr(a), _unwrap_constexpr(b)
        if not isinstance(a, Node) and not isinstance(b, Node):
            return max(a, b) if fn == "max" else min(a, b)
        if not isinstance(a, Node):
            a = self.as_node(a, self._adopt(a, b.dtype), where)
        if not isinstance(b, Node):
            b = self.as_node(b, self._adopt(b, a.dtype), where)
        dt = tp.promote(a.dtype, b.dtype)
        shape = tp.broadcast_shapes(a.shape, b.shape)
        return self.node("bin", (a, b), (("fn", fn),), shape, dt)

    def b_maximum(self, where, a, b):
        return self._binary_fn(where, "max", a, b)

    def b_minimum(self, where, a, b):
        return self._binary_fn(where, "min", a, b)

    def b_where(self, where, cond, a, b):
        cond = _unwrap_constexpr(cond)
        if not isinstance(cond, Node):
            return a if cond else b
        a, b = _unwrap_constexpr(a), _unwrap_constexpr(b)
        if not isinstance(a, Node) and not isinstance(b, Node):
            a = self.as_node(a, None, where)
        if not isinstance(a, Node):
            a = self.as_node(a, self._adopt(a, b.dtype), where)
        if not isinstance(b, Node):
            b = self.as_node(b, self._adopt(b, a.dtype), where)
        dt = tp.promote(a.dtype, b.dtype)
        shape = tp.broadcast_shapes(cond.shape, tp.broadcast_shapes(a.shape, b.shape))
        return self.node("where", (cond, a, b), (), shape, dt)

    def b_fma(self, where, a, b, c):
        return self.binop("add", self.binop("mul", a, b, where), c, where)

    def b_cdiv(self, where, a, b):
        a, b = _unwrap_constexpr(a), _unwrap_constexpr(b)
        if not isinstance(a, Node) and not isinstance(b, Node):
            return -(-a // b)
        a = self.as_node(a, tp.int32, where)
        b = self.as_node(b, tp.int32, where)
        return self.node("bin", (a, b), (("fn", "cdiv"),), tp.broadcast_shapes(a.shape, b.shape),
                         tp.promote(a.dtype, b.dtype))

    def b_multiple_of(self, where, x, value):
        return x

    def b_max_contiguous(self, where, x, value):
        return x

    def b_static_assert(self, where, cond, msg=""):
        cond = _unwrap_constexpr(cond)
        if isinstance(cond, Node):
            self.err(where, "static_assert needs a compile-time condition")
        if not cond:
            self.err(where, f"static_assert failed: {msg}")

    def b_static_print(self, where, *args):
        print(*[_unwrap_constexpr(a) for a in args])


def trace_kernel(fndef, fn_globals, runtime_types, constexprs, num_warps=4):
    """Traces one specialization of a kernel; returns a Trace."""
    return Tracer(fndef, fn_globals, runtime_types, constexprs, num_warps).run()
