"""`compile_fn`: a kernel's AST -> what will run for one specialization, without a GPU.

The reference's generator returns `(cuda_source, shared_memory_bytes)` for every kernel
(newt/compiler/codegen.py:2758-2765); its GPU-free tests drive it directly
(tests/test_codegen_cpu.py:22-31).  Here a specialization lowers to a launch plan: for the
tuned programs (vector add, row softmax, layernorm, the matmul K loop, the attention loop) the
kernel is prebuilt in libnewt_b200, so the "source" is a one-line comment naming the C-ABI
entry point; every other program gets generated CUDA.  The plan comes back as a third result.
"""

from .. import types as tp
from ..frontend import lower as _lower
from ..frontend.trace import CompileError, trace_kernel  # noqa: F401

UNIFORM = "uniform"     # a scalar or pointer argument: one value for the whole program instance
BLOCK = "block"


class Value:
    """A kernel parameter as the reference's generator is handed it: (kind, dtype, shape, name)."""

    def __init__(self, kind, dtype, shape=(), name=None):
        self.kind, self.dtype, self.shape, self.name = kind, dtype, tuple(shape), name


def compile_fn(fndef, fn_globals, params, constexprs, num_warps=4, kernel_name=None, num_stages=3):
    """`params`: [(name, Value | dtype | pointer_type)] in declaration order; `constexprs`:
    {name: value}.  Returns (source, dynamic shared memory bytes, plan)."""
    runtime_types = {}
    for name, value in params:
        t = value.dtype if isinstance(value, Value) else value
        if not isinstance(t, (tp.dtype, tp.pointer_type)):
            raise TypeError(f"parameter '{name}': expected a dtype or pointer_type, got {t!r}")
        runtime_types[name] = t
    trace = trace_kernel(fndef, fn_globals, runtime_types, dict(constexprs), num_warps)
    if kernel_name:
        trace.name = kernel_name
    plan = _lower.lower(trace, num_warps=num_warps, num_stages=num_stages)
    if isinstance(plan, _lower.PointwisePlan):
        return plan.source, plan.shared_bytes, plan
    return f"// {trace.name}: {plan.describe()} (prebuilt sm_100a kernel in libnewt_b200)\n", 0, plan
