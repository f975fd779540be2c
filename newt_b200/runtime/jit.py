"""`@jit`: compile-on-first-launch wrapper with the launch protocol of the reference.

Everything a caller can observe is kept as newt/runtime/jit.py has it:
`kernel[grid](*args, **kwargs)`; `grid` a tuple, an int or a callable of
`meta = runtime args | constexprs | {"num_warps"}` (:210-219); reserved
keywords `num_warps` (power of two <= 32) and `num_stages` (1..8) (:169-174);
TypeError for binding problems (:104-120, 129-144), ValueError for a tensor on
another device (:195-199); an empty grid is a no-op (:220-221); a bare call
raises (:93-97); one specialization per (constexprs, argument types,
num_warps, num_stages) (:177-183).

What differs is what a specialization *is*: the kernel body is traced into an
expression graph (frontend/trace.py) and lowered to a launch plan on one of the
hand-written sm_100a kernels of libnewt_b200.so (frontend/lower.py).  There is
no other backend; a body no plan covers raises CompileError.
"""

import ast
import functools
import inspect
import os
import textwrap

from .. import types as tp
from ..frontend import lower as _lower
from ..frontend.trace import CompileError, trace_kernel


def _is_constexpr_annotation(ann):
    from .. import language as nl

    if ann is nl.constexpr or isinstance(ann, nl.constexpr):
        return True
    return isinstance(ann, str) and "constexpr" in ann


class CompiledKernel:
    """One specialization: its trace (for inspection) and its launch plan."""

    def __init__(self, name, trace, plan, num_warps, num_stages, param_names):
        self.name = name
        self.trace = trace
        self.plan = plan
        self.num_warps = num_warps
        self.num_stages = num_stages
        self.param_names = param_names


class _KernelHandle:
    """Stands where a Python function would for a kernel that only exists as a syntax tree
    (deuteron builds its kernels that way): a name and the globals its body refers to."""

    def __init__(self, name, fn_globals, doc=None):
        self.__name__ = self.__qualname__ = name
        self.__globals__ = fn_globals
        self.__doc__ = doc
        self.__module__ = fn_globals.get("__name__", "newt_b200.generated")


class JITFunction:
    def __init__(self, fn):
        source = textwrap.dedent(inspect.getsource(fn))
        tree = ast.parse(source)
        fndef = next(n for n in tree.body if isinstance(n, ast.FunctionDef))
        params = inspect.signature(fn).parameters
        self._setup(fn, fndef, list(params),
                    [n for n, p in params.items() if _is_constexpr_annotation(p.annotation)],
                    {n: p.default for n, p in params.items()
                     if p.default is not inspect.Parameter.empty})

    @classmethod
    def from_ast(cls, fndef, fn_globals):
        """A kernel given as an `ast.FunctionDef` (positional parameters, constexprs marked by a
        `...constexpr` annotation, no defaults) and the globals its names resolve in: what a
        front end that builds kernels programmatically hands over, with no source text, `exec`
        or `inspect` in between."""
        if fndef.args.defaults or fndef.args.kwonlyargs or fndef.args.vararg or fndef.args.kwarg:
            raise TypeError("from_ast: plain positional parameters only")
        names = [a.arg for a in fndef.args.args]
        constexprs = [a.arg for a in fndef.args.args
                      if a.annotation is not None and "constexpr" in ast.unparse(a.annotation)]
        self = cls.__new__(cls)
        self._setup(_KernelHandle(fndef.name, fn_globals, ast.get_docstring(fndef)), fndef, names,
                    constexprs, {})
        return self

    def _setup(self, fn, fndef, param_names, constexpr_names, defaults):
        functools.update_wrapper(self, fn)
        self.fn = fn
        self.fndef = fndef
        self.param_names = param_names
        self.constexpr_names = constexpr_names
        self._constexpr_set = frozenset(self.constexpr_names)
        self.defaults = defaults
        self.cache = {}
        self._fast = {}      # cheap per-launch key -> (CompiledKernel, names of the tensor arguments)
        self._name_set = set(self.param_names)
        self._is_constexpr = [n in self._constexpr_set for n in self.param_names]

    def __getitem__(self, grid):
        return functools.partial(self._run, grid)

    def __call__(self, *args, **kwargs):
        raise RuntimeError(
            f"@newt.jit kernel '{self.fn.__name__}' must be launched with a grid: "
            f"kernel[grid](...)")

    # ---- argument handling -------------------------------------------------------

    def _bind(self, args, kwargs):
        names = self.param_names
        if not self.defaults and len(args) + len(kwargs) == len(names):
            # the usual call: every parameter given once, tensors and sizes by position,
            # constexprs by keyword
            bound = dict(zip(names, args))
            bound.update(kwargs)
            if len(bound) == len(names) and bound.keys() == self._name_set:
                return bound
        if len(args) > len(names):
            raise TypeError(f"{self.fn.__name__}() takes {len(names)} arguments "
                            f"but {len(args)} were given")
        bound = dict(zip(names, args))
        unknown = []
        for k, v in kwargs.items():
            if k not in self.defaults and k not in names:
                unknown.append(k)
            elif k in bound:
                raise TypeError(f"duplicate argument {k}")
            else:
                bound[k] = v
        if unknown:
            raise TypeError(f"unknown kernel arguments: {unknown}")
        for k, v in self.defaults.items():
            bound.setdefault(k, v)
        missing = [n for n in names if n not in bound]
        if missing:
            raise TypeError(f"missing kernel arguments: {missing}")
        return bound

    @staticmethod
    def _type_of(name, val):
        import torch

        if isinstance(val, torch.Tensor):
            if not val.is_cuda:
                raise TypeError(f"argument '{name}' must be a CUDA tensor")
            elem = tp.TORCH_TO_NEWT.get(str(val.dtype))
            if elem is None:
                raise TypeError(f"unsupported tensor dtype {val.dtype} for '{name}'")
            return tp.pointer_type(elem)
        if isinstance(val, bool):
            return tp.int1
        if isinstance(val, int):
            if not -(2 ** 63) <= val < 2 ** 63:
                raise TypeError(f"integer argument '{name}'={val} does not fit int64")
            return tp.int32 if -(2 ** 31) <= val < 2 ** 31 else tp.int64
        if isinstance(val, float):
            return tp.float32
        raise TypeError(f"unsupported kernel argument type {type(val)} for '{name}'")

    # ---- compile -------------------------------------------------------------------

    def _compile(self, constexprs, runtime_types, num_warps, num_stages):
        trace = trace_kernel(self.fndef, self.fn.__globals__, runtime_types, constexprs, num_warps)
        plan = _lower.lower(trace, num_warps=num_warps, num_stages=num_stages)
        if os.environ.get("NEWT_DEBUG"):
            print(f"=== newt_b200: {self.fn.__name__} -> {plan.describe()} "
                  f"(warps={num_warps}, stages={num_stages}) ===")
            print(trace.dump())
        return CompiledKernel(self.fn.__name__, trace, plan, num_warps, num_stages,
                              [n for n in self.param_names if n not in self._constexpr_set])

    def specialize(self, *args, **kwargs):
        """Compiles (or fetches) the specialization these arguments select, without
        launching; returns the CompiledKernel.  Tensors may be replaced by
        `pointer_type` objects, so plans can be inspected without a GPU."""
        num_warps = kwargs.pop("num_warps", 4)
        num_stages = kwargs.pop("num_stages", 3)
        bound = self._bind(args, kwargs)
        return self._specialization(bound, num_warps, num_stages)[0]

    def _specialization(self, bound, num_warps, num_stages):
        if num_warps not in (1, 2, 4, 8, 16, 32):
            raise ValueError(f"num_warps must be a power of two <= 32, got {num_warps}")
        if not isinstance(num_stages, int) or not 1 <= num_stages <= 8:
            raise ValueError(f"num_stages must be in 1..8, got {num_stages}")
        cset = self._constexpr_set
        constexprs = {n: bound[n] for n in self.constexpr_names}
        runtime_types = {}
        for n in self.param_names:
            if n not in cset:
                v = bound[n]
                runtime_types[n] = v if isinstance(v, (tp.pointer_type, tp.dtype)) \
                    else self._type_of(n, v)
        key = (tuple(sorted((k, repr(v)) for k, v in constexprs.items())),
               tuple((n, t.name) for n, t in runtime_types.items()), num_warps, num_stages)
        compiled = self.cache.get(key)
        if compiled is None:
            compiled = self._compile(constexprs, runtime_types, num_warps, num_stages)
            self.cache[key] = compiled
        return compiled, constexprs, runtime_types

    # ---- launch --------------------------------------------------------------------

    def _fast_key(self, bound, num_warps, num_stages):
        """Key under which a launch finds its specialization without type inference: the
        constexpr values and, per runtime argument, what its type is inferred from (the torch
        dtype, int32 vs int64 by value, float) -- newt/runtime/jit.py:99-144 keys the same
        way.  A constexpr is keyed with its type: 2, 2.0 and True compare (and hash) equal in
        Python but select different specializations (the reference keys on repr, :177-183).
        None for an unhashable constexpr value."""
        parts = [(type(v), v) if c else
                 ((32 if -2147483648 <= v < 2147483648 else 64) if type(v) is int else
                  (type(v) if type(v) in (float, bool) else getattr(v, "dtype", type(v))))
                 for v, c in zip(map(bound.__getitem__, self.param_names), self._is_constexpr)]
        key = (tuple(parts), num_warps, num_stages)
        try:
            hash(key)
        except TypeError:
            return None
        return key

    def _run(self, grid, *args, **kwargs):
        import torch

        from . import kernels

        num_warps = kwargs.pop("num_warps", 4)
        num_stages = kwargs.pop("num_stages", 3)
        bound = self._bind(args, kwargs)
        key = self._fast_key(bound, num_warps, num_stages)
        hit = self._fast.get(key) if key is not None else None
        if hit is None:
            compiled, _, runtime_types = self._specialization(bound, num_warps, num_stages)
            tensors = [n for n, t in runtime_types.items() if isinstance(t, tp.pointer_type)]
            if key is not None and all(isinstance(bound[n], torch.Tensor) for n in tensors):
                self._fast[key] = (compiled, tensors)
        else:
            compiled, tensors = hit

        if tensors:
            current = kernels.current_device()
            for name in tensors:
                v = bound[name]
                if v.get_device() != current:      # -1 for a CPU tensor
                    if not v.is_cuda:
                        raise TypeError(f"argument '{name}' must be a CUDA tensor")
                    raise ValueError(
                        f"tensor '{name}' is on {v.device} but the current device is "
                        f"cuda:{current}; newt launches on the current device")

        if callable(grid):
            meta = {n: bound[n] for n in self.param_names}
            meta["num_warps"] = num_warps
            g = grid(meta)
        else:
            g = grid
        if type(g) is not tuple or not all(type(x) is int for x in g):
            g = (int(g),) if isinstance(g, int) else tuple(int(x) for x in g)
        if len(g) > 3:
            raise ValueError(f"grids have at most 3 dimensions, got {g}")
        if min(g, default=1) <= 0:
            return
        if tensors:
            trust = kernels._trust
            trust.checked = True      # `_dev_ptr` takes this launch's tensors as verified
            try:
                compiled.plan.launch(g, bound)
            finally:
                trust.checked = False
        else:
            compiled.plan.launch(g, bound)


def jit(fn=None):
    if fn is None:
        return jit
    return JITFunction(fn)
