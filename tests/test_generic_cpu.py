"""Control flow and dots outside the tuned kernels, without a GPU: every program of
tests/generic_programs.py lowers to generated CUDA and NVRTC compiles it for sm_100a."""

import pytest
import torch

import generic_programs as gp
import newt_b200 as newt
import newt_b200.language as nl
from newt_b200 import types as tp
from newt_b200.frontend.lower import GemmEpiloguePlan, GemmPlan, PointwisePlan
from newt_b200.runtime import nvrtc


def _specialize(name):
    kernel, _grid, args, meta, _checks = gp.build(name, "cpu")
    types = [tp.pointer_type(tp.TORCH_TO_NEWT[str(a.dtype)]) if isinstance(a, torch.Tensor) else a
             for a in args]
    return kernel.specialize(*types, **meta)


@pytest.mark.parametrize("name", sorted(gp.CASES))
def test_program_lowers_and_compiles(name):
    plan = _specialize(name).plan
    if isinstance(plan, GemmPlan):      # what runs if the tensor-core path refuses the operands
        plan = plan.generic()
    if isinstance(plan, GemmEpiloguePlan):      # tensor-core product + generated epilogue
        assert "nb_acc[" in plan.epilogue.source and "fmaf(" not in plan.epilogue.source
        plan = plan.epilogue
    assert isinstance(plan, PointwisePlan)
    cubin = nvrtc.compile_cubin(plan.source, name + ".cu")
    assert len(cubin) > 1000


def test_pure_loops_stay_in_registers():
    """A loop that only computes is run by each thread for its own element: no shared memory,
    no barrier; a walking pointer block is its first value plus one running offset."""
    plan = _specialize("weighted_tiles").plan
    assert "__syncthreads" not in plan.source and "nb_shared" not in plan.source
    assert "long long off" in plan.source
    plan = _specialize("ragged_matmul").plan.generic()
    assert "nb_shared" not in plan.source and "fmaf(" in plan.source


def test_loops_that_reduce_run_block_wide():
    plan = _specialize("running_softmax_stats").plan
    assert "nb_block_reduce" in plan.source or "nb_fold" in plan.source
    assert plan.source.count("for (int k") >= 1 and "__syncthreads" in plan.source
    plan = _specialize("small_head_attention").plan
    assert "nb_c0" in plan.source          # the accumulator block lives in shared memory


def test_names_only_overwritten_in_a_loop_are_not_carried():
    plan = _specialize("tiled_layernorm").plan
    assert isinstance(plan, PointwisePlan)


def test_break_under_a_runtime_condition_ends_a_while_loop():
    src = _specialize("capped_growth").plan.source
    assert "for (;;)" in src and "break;" in src


def test_control_flow_errors():
    F32 = tp.pointer_type(tp.float32)

    with pytest.raises(newt.CompileError, match="BLOCK too small"):
        gp.chosen_at_compile_time.specialize(F32, F32, 4, MODE="triple", BLOCK=8)
    with pytest.raises(newt.CompileError):       # the other arm is traced when it is the one taken
        gp.chosen_at_compile_time.specialize(F32, F32, 4, MODE="other", BLOCK=16)

    @newt.jit
    def block_condition(x_ptr, BLOCK: nl.constexpr):
        x = nl.load(x_ptr + nl.arange(0, BLOCK))
        if x > 0:
            nl.store(x_ptr + nl.arange(0, BLOCK), x)

    with pytest.raises(newt.CompileError, match="nl.where"):
        block_condition.specialize(F32, BLOCK=64)

    @newt.jit
    def pointer_choice(x_ptr, y_ptr, flag, BLOCK: nl.constexpr):
        p = x_ptr
        if flag == 1:
            p = y_ptr
        nl.store(p + nl.arange(0, BLOCK), 1.0)

    with pytest.raises(newt.CompileError, match="pointers"):
        pointer_choice.specialize(F32, F32, 1, BLOCK=64)

    @newt.jit
    def endless(x_ptr, BLOCK: nl.constexpr):
        while True:
            nl.store(x_ptr + nl.arange(0, BLOCK), 1.0)

    with pytest.raises(newt.CompileError, match="never end"):
        endless.specialize(F32, BLOCK=64)

    @newt.jit
    def stored_then_read(x_ptr, n, BLOCK: nl.constexpr):
        offs = nl.arange(0, BLOCK)
        for t in range(n):                     # each pass reads what the pass before stored
            x = nl.load(x_ptr + offs + t)
            nl.store(x_ptr + offs + t + 1, x)

    with pytest.raises(newt.CompileError, match="stored to"):
        stored_then_read.specialize(F32, 4, BLOCK=64)


def test_sixteen_bit_elementwise_gets_the_sixteen_byte_path():
    """fp16 / bf16 blocks whose last axis is unit-stride and a multiple of eight are walked
    eight neighbours per trip with 16-byte accesses; fp32 keeps one element per trip; a block
    indexed through a stride argument (unit stride not provable) keeps one element per trip."""
    import newt_b200 as newt
    from newt_b200 import language as nl, types as tp
    from newt_b200.runtime import nvrtc

    @newt.jit
    def scale(x_ptr, o_ptr, n, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        nl.store(o_ptr + offs, nl.load(x_ptr + offs, mask=offs < n, other=0.0) * 3.0, mask=offs < n)

    @newt.jit
    def strided(x_ptr, o_ptr, n, stride, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        nl.store(o_ptr + offs * stride, nl.load(x_ptr + offs * stride, mask=offs < n, other=0.0),
                 mask=offs < n)

    for elem, wide in ((tp.float16, True), (tp.bfloat16, True), (tp.float32, False)):
        p = tp.pointer_type(elem)
        plan = scale.specialize(p, p, 1 << 20, BLOCK=1024).plan
        assert ("uint4" in plan.source) == wide
        nvrtc.compile_cubin(plan.source, "scale.cu")
    p = tp.pointer_type(tp.float16)
    assert "uint4" not in strided.specialize(p, p, 1 << 20, 2, BLOCK=1024).plan.source
    assert "uint4" not in scale.specialize(p, p, 1 << 20, BLOCK=4).plan.source     # 4 is not a multiple of 8


def test_a_row_program_outside_the_tuned_shapes_is_written_as_one_pass():
    """log-softmax: the row is loaded once per element and `exp` evaluated once per element
    (the sum and nothing else uses it), although two reductions and the store all read the row;
    blocks that do not split evenly over the threads keep the loop form."""
    import newt_b200 as newt
    from newt_b200 import language as nl, types as tp
    from newt_b200.runtime import nvrtc

    @newt.jit
    def log_softmax(x_ptr, out_ptr, N, stride, BLOCK_N: nl.constexpr):
        row = nl.program_id(0)
        cols = nl.arange(0, BLOCK_N)
        mask = cols < N
        x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf"))
        z = x - nl.max(x, axis=0)
        nl.store(out_ptr + row * stride + cols, z - nl.log(nl.sum(nl.exp(z), axis=0)), mask=mask)

    p = tp.pointer_type(tp.float32)
    plan = log_softmax.specialize(p, p, 1000, 1024, BLOCK_N=1024).plan
    wide, narrow = plan.source.split("\n  } else {\n")       # aligned tensors / a base that is off
    assert wide.count("expf(") == 8 and narrow.count("expf(") == 8       # 1024 / 128 threads
    assert wide.count("const uint4 t0 = ") == 2                           # two groups of four lanes
    assert "for (int k" not in plan.source                                 # no pass over memory per reduction
    assert nvrtc.compile_cubin(plan.source, "log_softmax.cu")[:4] == b"\x7fELF"
    looped = log_softmax.specialize(p, p, 60, 64, BLOCK_N=64).plan         # 64 elements, 128 threads
    assert "nb_v0" not in looped.source
