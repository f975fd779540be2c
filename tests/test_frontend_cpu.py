"""CPU: the front end, without a GPU -- tracing, affine analysis and which launch
plan each hot-path kernel lowers to (the reference's GPU-free tests check the
structure of generated text the same way, tests/test_codegen_cpu.py:22-76)."""

import pytest
import torch

import newt_b200 as newt
import newt_b200.deuteron as dt
from newt_b200.examples import kernels as examples_kernels
import newt_b200.language as nl
from newt_b200 import types as tp
from newt_b200.frontend import lower

import ref_kernels as rk

P = tp.pointer_type
F32, F16, BF16 = P(tp.float32), P(tp.float16), P(tp.bfloat16)


def test_softmax_lowers_to_row_kernel():
    c = rk.softmax_kernel.specialize(F32, F32, 781, 1001, BLOCK_N=1024)
    assert isinstance(c.plan, lower.SoftmaxPlan) and c.plan.entry == "nb200_softmax_f32"
    a = dict(N=781, stride=1001)
    assert (c.plan.n(a), c.plan.sx(a), c.plan.so(a), c.plan.block) == (781, 1001, 1001, 1024)


@pytest.mark.parametrize("ptr", [F32, F16, BF16])
def test_layernorm_lowers_to_row_kernel(ptr):
    c = rk.layernorm_kernel.specialize(ptr, ptr, ptr, ptr, 300, 320, 1e-5, BLOCK_N=512)
    assert isinstance(c.plan, lower.LayerNormPlan)
    assert c.plan.eps == "eps" and c.plan.n(dict(N=300, stride=320)) == 300


def test_add_lowers_to_vector_kernel():
    c = rk.add_kernel.specialize(F32, F32, F32, 12345, BLOCK=4096)
    assert isinstance(c.plan, lower.AddPlan) and c.plan.n(dict(n=12345)) == 12345


@pytest.mark.parametrize("kernel,extents", [(rk.matmul_kernel, (300, 200, 104)),
                                            (rk.matmul_kernel_unmasked, (320, 256, 96))])
def test_matmul_lowers_to_tcgen05_gemm(kernel, extents):
    c = kernel.specialize(F16, F16, F16, 300, 200, 104, 104, 1, 200, 1, 200, 1,
                          BLOCK_M=64, BLOCK_N=64, BLOCK_K=32, num_stages=4)
    p = c.plan
    assert isinstance(p, lower.GemmPlan) and p.entry == "nb200_gemm"
    a = dict(M=300, N=200, K=104, sam=104, sak=1, sbk=200, sbn=1, scm=200, scn=1)
    assert p._extents((5, 4), a) == extents
    assert (p.lda(a), p.ldb(a), p.ldc(a)) == (104, 200, 200)
    assert (p.pid_m, p.pid_n) == (0, 1) and p.hardware_key() == ("gemm", 64, 4)
    assert (p.a, p.b, p.c) == ("a_ptr", "b_ptr", "c_ptr")


def test_attention_lowers_to_fused_kernel():
    from newt_b200 import examples

    strides = [524288, 128, 1] * 4
    a = dict(zip(["sqh", "sqm", "sqd", "skh", "skn", "skd", "svh", "svn", "svd", "soh", "som",
                  "sod"], strides), M=4000, N=4096, scale=0.088)
    for causal in (False, True):
        c = examples.attention_kernel.specialize(F16, F16, F16, F16, 4000, 4096, 0.088, *strides,
                                                 BLOCK_M=128, BLOCK_N=64, D=128, CAUSAL=causal)
        p = c.plan
        assert isinstance(p, lower.AttentionPlan) and p.entry == "nb200_attention_fwd"
        assert (p.causal, p.pid_m, p.pid_head, p.d, p.scale) == (causal, 0, 1, 128, "scale")
        assert p.seq_q(a) == 4000 and p.seq_kv(a) == 4096
        assert [f(a) for f in p.strides["k_ptr"]] == [524288, 128, 1]
    # the reference's example as shipped: one head, no causal mask, D = 64
    c = rk.attention_kernel_2d.specialize(F16, F16, F16, F16, 1024, 1024, 0.125, 64, 1, 64, 1, 64,
                                          1, 64, 1, BLOCK_M=64, BLOCK_N=64, D=64)
    assert isinstance(c.plan, lower.AttentionPlan)
    assert c.plan.pid_head is None and not c.plan.causal and c.plan.d == 64


def test_matmul_block_256_selects_the_cta_pair_kernel():
    c = rk.matmul_kernel.specialize(F16, F16, F16, 512, 512, 512, 512, 1, 512, 1, 512, 1,
                                    BLOCK_M=256, BLOCK_N=256, BLOCK_K=128, num_stages=3)
    assert c.plan.hardware_key() == ("gemm-pair", 128, 0)
    cfg = c.plan.config()
    assert (cfg.block_m, cfg.block_n, cfg.block_k, cfg.cta_pair) == (256, 256, 128, 1)


def test_pointer_walk_is_resolved_as_induction():
    c = rk.matmul_kernel.specialize(F16, F16, F16, 64, 64, 64, 64, 1, 64, 1, 64, 1,
                                    BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    from newt_b200.frontend.affine import Analyzer
    an = Analyzer(c.trace)
    an.resolve_inductions()
    loop = c.trace.loops[0]
    assert ("carried", loop.uid, "a_ptrs") in an.closed_forms
    assert ("carried", loop.uid, "b_ptrs") in an.closed_forms
    assert ("carried", loop.uid, "acc") not in an.closed_forms


def test_transposed_operands_are_told_apart_at_launch_time():
    c = rk.matmul_kernel.specialize(F16, F16, F16, 64, 64, 64, 1, 64, 64, 1, 64, 1,
                                    BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    a = dict(M=64, N=64, K=64, sam=1, sak=64, sbk=1, sbn=64, scm=64, scn=1)
    inner = dict(c.plan.inner)
    assert inner["a_ptr"](a) == 64   # A transposed: copied into a row-major workspace at launch
    assert inner["b_ptr"](a) == 64 and c.plan.ldb(a) == 1   # B transposed: goes to nb200_gemm_bt


def test_fp32_matmul_lowers_to_the_tf32_plan():
    c = rk.matmul_kernel.specialize(F32, F32, F32, 128, 128, 128, 128, 1, 128, 1, 128, 1,
                                    BLOCK_M=256, BLOCK_N=256, BLOCK_K=32)
    assert c.plan.row_k == 32 and c.plan.hardware_key() == ("gemm-pair", 32, 3)
    c = rk.matmul_kernel.specialize(F32, F32, F32, 128, 128, 128, 128, 1, 128, 1, 128, 1,
                                    BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    assert c.plan.hardware_key() == ("gemm", 64, 3)


def test_unrecognised_program_raises_compile_error():
    @newt.jit
    def shift_through_memory(x_ptr, tmp_ptr, out_ptr, BLOCK: nl.constexpr):
        # elements travel between threads through memory the program itself wrote: the generic
        # lowering evaluates loads where they are used and refuses what that could reorder
        offs = nl.arange(0, BLOCK)
        nl.store(tmp_ptr + offs, nl.load(x_ptr + offs) * 2)
        nl.store(out_ptr + offs, nl.load(tmp_ptr + (offs + 1) % BLOCK))

    with pytest.raises(newt.CompileError, match="no sm_100a kernel"):
        shift_through_memory.specialize(F32, F32, F32, BLOCK=128)


def test_runtime_loop_outside_the_tuned_programs_is_compiled_at_run_time():
    from newt_b200.frontend.lower import PointwisePlan

    @newt.jit
    def strided_sum(x_ptr, out_ptr, n, steps, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        acc = nl.zeros((BLOCK,), dtype=nl.float32)
        for i in range(steps):
            acc += nl.load(x_ptr + i * n + offs, mask=offs < n, other=0.0)
        nl.store(out_ptr + offs, acc, mask=offs < n)

    c = strided_sum.specialize(F32, F32, 100, 4, BLOCK=128)
    assert isinstance(c.plan, PointwisePlan)
    assert "for (int k" in c.plan.source


def test_reductions_outside_the_tuned_programs_are_compiled_at_run_time():
    from newt_b200.frontend.lower import PointwisePlan
    from newt_b200.runtime import nvrtc

    @newt.jit
    def rmsnorm(x_ptr, w_ptr, out_ptr, N, stride, eps, BLOCK_N: nl.constexpr):
        row = nl.program_id(0)
        cols = nl.arange(0, BLOCK_N)
        mask = cols < N
        x = nl.load(x_ptr + row * stride + cols, mask=mask, other=0.0).to(nl.float32)
        ms = nl.sum(x * x, axis=0) / N
        y = x * nl.rsqrt(ms + eps) * nl.load(w_ptr + cols, mask=mask, other=0.0)
        nl.store(out_ptr + row * stride + cols, y, mask=mask)

    c = rmsnorm.specialize(F16, F16, F16, 1000, 1024, 1e-6, BLOCK_N=1024)
    assert isinstance(c.plan, PointwisePlan)
    assert "nb_block_reduce<0, float>" in c.plan.source and "float* const nb_r0" in c.plan.source
    assert nvrtc.compile_cubin(c.plan.source, "rmsnorm.cu")[:4] == b"\x7fELF"


def test_block_arithmetic_is_compiled_at_run_time():
    from newt_b200.frontend.lower import PointwisePlan
    from newt_b200.runtime import nvrtc

    @newt.jit
    def scale(x_ptr, out_ptr, n, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        nl.store(out_ptr + offs, nl.load(x_ptr + offs, mask=offs < n) * 2.0, mask=offs < n)

    @newt.jit
    def bias_relu(x_ptr, b_ptr, out_ptr, M, N, sx, so, BM: nl.constexpr, BN: nl.constexpr):
        rm = nl.program_id(0) * BM + nl.arange(0, BM)
        rn = nl.program_id(1) * BN + nl.arange(0, BN)
        mask = (rm[:, None] < M) & (rn[None, :] < N)
        x = nl.load(x_ptr + rm[:, None] * sx + rn[None, :], mask=mask, other=0.0)
        b = nl.load(b_ptr + rn, mask=rn < N, other=0.0)
        y = nl.where(x + b[None, :] > 0.0, x + b[None, :], 0.0)
        nl.store(out_ptr + rm[:, None] * so + rn[None, :], nl.sigmoid(y).to(nl.float32), mask=mask)

    for kernel, spec, kw in ((scale, (F32, F32, 100), dict(BLOCK=128)),
                             (bias_relu, (F16, F16, F32, 100, 200, 200, 200), dict(BM=16, BN=64))):
        c = kernel.specialize(*spec, **kw)
        assert isinstance(c.plan, PointwisePlan)
        assert f'extern "C" __global__ void __launch_bounds__(128) {c.plan.kernel_name}(' in c.plan.source
        # fp16 arithmetic is done in fp32 and rounded back after every operation
        if kernel is bias_relu:
            assert "nb_to_f16((__half2float(" in c.plan.source
        cubin = nvrtc.compile_cubin(c.plan.source, c.plan.kernel_name + ".cu")   # needs no GPU
        assert cubin[:4] == b"\x7fELF"


def test_block_arithmetic_refuses_what_it_could_get_wrong():
    @newt.jit
    def read_after_write(x_ptr, y_ptr, n, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        x = nl.load(x_ptr + offs, mask=offs < n)
        nl.store(x_ptr + offs, x + 1.0, mask=offs < n)
        nl.store(y_ptr + offs, x, mask=offs < n)      # x must be the value from before the first store

    with pytest.raises(newt.CompileError, match="consumed after the program stored to it"):
        read_after_write.specialize(F32, F32, 100, BLOCK=128)


def test_language_errors_are_compile_errors():
    @newt.jit
    def bad_arange(x_ptr, BLOCK: nl.constexpr):
        nl.store(x_ptr + nl.arange(0, 100), 0.0)

    with pytest.raises(newt.CompileError, match="power of two"):
        bad_arange.specialize(F32, BLOCK=1)

    @newt.jit
    def bad_dot(a_ptr, b_ptr, BLOCK: nl.constexpr):
        o = nl.arange(0, 16)
        a = nl.load(a_ptr + o[:, None] * 16 + o[None, :])
        b = nl.load(b_ptr + o[:, None] * 16 + o[None, :])
        nl.store(a_ptr + o[:, None] * 16 + o[None, :], nl.dot(a, b))

    with pytest.raises(newt.CompileError, match="share a dtype"):
        bad_dot.specialize(F16, BF16, BLOCK=1)

    @newt.jit
    def block_condition(x_ptr, BLOCK: nl.constexpr):
        o = nl.arange(0, BLOCK)
        if o < 3:
            nl.store(x_ptr + o, 0.0)

    with pytest.raises(newt.CompileError, match="nl.where"):
        block_condition.specialize(F32, BLOCK=8)


def test_launch_protocol_errors_need_no_gpu():
    with pytest.raises(RuntimeError, match="must be launched with a grid"):
        rk.add_kernel(1, 2, 3, 4)
    with pytest.raises(TypeError, match="unknown kernel arguments"):
        rk.add_kernel.specialize(F32, F32, F32, 10, BLOCK=64, bogus=1)
    with pytest.raises(TypeError, match="missing kernel arguments"):
        rk.add_kernel.specialize(F32, F32, F32, 10)
    with pytest.raises(TypeError, match="takes 5 arguments"):
        rk.add_kernel.specialize(F32, F32, F32, 10, 64, 7)
    with pytest.raises(ValueError, match="num_warps"):
        rk.add_kernel.specialize(F32, F32, F32, 10, BLOCK=64, num_warps=3)
    with pytest.raises(ValueError, match="num_stages"):
        rk.add_kernel.specialize(F32, F32, F32, 10, BLOCK=64, num_stages=9)
    with pytest.raises(TypeError, match="must be a CUDA tensor"):
        rk.add_kernel[(1,)](torch.zeros(4), torch.zeros(4), torch.zeros(4), 4, BLOCK=64)


def test_specialization_cache_keys():
    k = rk.add_kernel
    n0 = len(k.cache)
    k.specialize(F32, F32, F32, 10, BLOCK=256)
    k.specialize(F32, F32, F32, 99, BLOCK=256)          # same types: reused
    assert len(k.cache) == n0 + 1
    k.specialize(F32, F32, F32, 2 ** 40, BLOCK=256)     # int64 argument: new specialization
    k.specialize(F32, F32, F32, 10, BLOCK=512)          # new constexpr
    assert len(k.cache) == n0 + 3


def test_constexpr_host_arithmetic_and_helpers():
    c = nl.constexpr(8)
    assert (c * 2).value == 16 and (2 * c).value == 16 and (c // 3).value == 2 and int(c) == 8
    assert newt.cdiv(10, 3) == 4 and newt.next_power_of_2(781) == 1024
    assert newt.next_power_of_2(1) == 1 and newt.next_power_of_2(1024) == 1024


def test_type_rules():
    assert tp.promote(tp.float16, tp.bfloat16) == tp.float32
    assert tp.promote(tp.int32, tp.float16) == tp.float16
    assert tp.promote(tp.int32, tp.int64) == tp.int64
    assert tp.broadcast_shapes((4, 1), (1, 8)) == (4, 8)
    with pytest.raises(TypeError):
        tp.broadcast_shapes((4,), (8,))
    assert P(tp.float16).element_ty == tp.float16


# ---- deuteron -------------------------------------------------------------------

@dt.kernel
def dt_matmul(x, y, out):
    for tile_m, tile_n in dt.tile([x.shape[0], y.shape[1]]):
        acc = dt.zeros([tile_m, tile_n], dtype=dt.float32)
        for tile_k in dt.tile(x.shape[1]):
            acc += x[tile_m, tile_k] @ y[tile_k, tile_n]
        out[tile_m, tile_n] = acc


def test_deuteron_source_and_plan():
    x, y = torch.randn(300, 104).bfloat16(), torch.randn(104, 200).bfloat16()
    out = torch.empty(300, 200).bfloat16()
    src = dt_matmul.to_newt_source(x, y, out)
    assert "def matmul_newt(x_ptr, x_d0, x_d1, x_s0, x_s1, y_ptr" not in src  # named after the fn
    assert "def dt_matmul_newt(x_ptr, x_d0, x_d1, x_s0, x_s1, y_ptr, y_d0, y_d1, y_s0, y_s1, " \
           "out_ptr, out_d0, out_d1, out_s0, out_s1, BLOCK_TILE_M: nl.constexpr" in src
    assert "acc = nl.dot(" in src and "for _i_tile_k in range(0, nl.cdiv(x_d1, BLOCK_TILE_K)):" in src
    built = dt_matmul.built_for((x, y, out))
    cfg = dt.Config(BLOCK_TILE_M=128, BLOCK_TILE_N=256, BLOCK_TILE_K=64, num_stages=4)
    grid, pos, kw = dt_matmul.launch_parts(built, (x, y, out), cfg)
    assert grid == (3, 1)
    typed = [BF16 if torch.is_tensor(a) else a for a in pos]
    plan = built.jit.specialize(*typed, **kw).plan
    args = dict(zip(built.jit.param_names, pos))
    assert isinstance(plan, lower.GemmPlan) and plan.hardware_key() == ("gemm", 256, 4)
    assert plan._extents(grid, args) == (300, 200, 104)


@dt.kernel
def dt_softmax(x, out):
    for tile_m in dt.tile(x.shape[0]):
        row = x[tile_m, :]
        m = row.amax(1)
        e = dt.exp(row - m[:, None])
        s = e.sum(1)
        out[tile_m, :] = e / s[:, None]


@dt.kernel
def dt_layernorm(x, w, b, out, eps):
    for tile_m in dt.tile(x.shape[0]):
        row = x[tile_m, :]
        mean = row.sum(1) / x.shape[1]
        diff = row - mean[:, None]
        var = (diff * diff).sum(1) / x.shape[1]
        rstd = dt.rsqrt(var + eps)
        out[tile_m, :] = diff * rstd[:, None] * w[:] + b[:]


def _plan_of(kernel, args, cfg, ptr):
    built = kernel.built_for(args)
    grid, pos, kw = kernel.launch_parts(built, args, cfg)
    plan = built.jit.specialize(*[ptr if torch.is_tensor(a) else a for a in pos], **kw).plan
    return plan, grid, dict(zip(built.jit.param_names, pos))


def test_deuteron_row_programs_lower_to_row_kernels():
    # examples/deuteron/02_softmax.py and 03_layernorm.py: [BLOCK_M, whole row] tiles
    x, out = torch.randn(1000, 777), torch.empty(1000, 777)
    plan, grid, a = _plan_of(dt_softmax, (x, out), dt.Config(BLOCK_TILE_M=4), F32)
    assert isinstance(plan, lower.SoftmaxPlan) and grid == (250,)
    assert (plan.n(a), plan.rows_per_program, plan.row_bound(a), plan.sx(a)) == (777, 4, 1000, 777)
    w, b = torch.randn(777), torch.randn(777)
    plan, grid, a = _plan_of(dt_layernorm, (x, w, b, out, 1e-5), dt.Config(BLOCK_TILE_M=2), F32)
    assert isinstance(plan, lower.LayerNormPlan) and plan.eps == "eps"
    assert (plan.x, plan.w, plan.b, plan.out) == ("x_ptr", "w_ptr", "b_ptr", "out_ptr")
    assert plan.n(a) == 777 and plan.rows_per_program == 2 and plan.hardware_key() == \
        ("nb200_layernorm",)


@dt.kernel
def dt_center_rows(x, out):
    for tile_m in dt.tile(x.shape[0]):
        row = x[tile_m, :]
        out[tile_m, :] = row - row.mean(1)[:, None]


def test_deuteron_mean_counts_valid_lanes_only():
    # mean() is what the reference leaves out (deuteron/codegen.py:412-413)
    from newt_b200.runtime import nvrtc

    x, out = torch.randn(10, 77), torch.empty(10, 77)
    src = dt_center_rows.to_newt_source(x, out)
    assert "nl.where(mask_tile_m[:, None] & mask_full0[None, :], 1.0, 0.0)" in src
    plan, grid, _ = _plan_of(dt_center_rows, (x, out), dt.Config(BLOCK_TILE_M=4), F32)
    assert isinstance(plan, lower.PointwisePlan) and grid == (3,)
    assert nvrtc.compile_cubin(plan.source, "center_rows.cu")[:4] == b"\x7fELF"
    dt_center_rows.ref(x, out)
    torch.testing.assert_close(out, x - x.mean(1, keepdim=True))


@dt.kernel
def dt_linear_relu(x, y, bias, out):
    for tile_m, tile_n in dt.tile([x.shape[0], y.shape[1]]):
        acc = dt.zeros([tile_m, tile_n], dtype=dt.float32)
        for tile_k in dt.tile(x.shape[1]):
            acc += x[tile_m, tile_k] @ y[tile_k, tile_n]
        out[tile_m, tile_n] = dt.relu(acc + bias[tile_n][None, :])


def test_matmul_epilogue_is_compiled_into_the_tensor_core_kernel():
    """relu(acc + bias) after the k loop: the program's own graph becomes an epilogue functor and
    the library's device templates are compiled with it by NVRTC for sm_100a (no GPU needed)."""
    import os

    from newt_b200.runtime import abi, nvrtc

    P16 = P(tp.bfloat16)
    c = examples_kernels.linear_bias_relu_kernel.specialize(
        P16, P16, P(tp.float32), P16, 512, 512, 512, 512, 1, 512, 1, 512, 1,
        BLOCK_M=256, BLOCK_N=256, BLOCK_K=64, num_stages=7)
    plan = c.plan
    assert isinstance(plan, lower.GemmEpiloguePlan) and plan.fused_source is not None
    assert "struct NbEpilogue" in plan.fused_source and "fmaxf(" in plan.fused_source
    assert "nb_pid_n" in plan.fused_source and "blockIdx" not in plan.fused_source
    assert plan.hardware_key()[-1] == "fused"
    # two steps: the bias is read in `fetch` (nothing there touches the accumulator), `apply`
    # does the arithmetic and leaves the one rounding to bf16 to the kernel's packed conversion
    fetch, apply = plan.fused_source.split("static __device__ __forceinline__ void apply(")
    assert "*v" in fetch and "nb_acc" not in fetch.split("void fetch(")[1]
    assert "nb_acc" in apply and "*v" not in apply and "__float2bfloat16_rn" not in apply
    for launch in (abi.GemmLaunch(pair=1, block_n=256, stages=7, ksub=1),
                   abi.GemmLaunch(pair=0, block_n=128, stages=4, ksub=1)):
        kernel = plan._fused_kernel(launch, abi.BF16, abi.BF16)
        assert kernel.cubin[:4] == b"\x7fELF" and "gemm_device.cuh" in kernel.source
    # what was compiled: tcgen05 MMAs fed by bulk tensor copies, each fetching for its own CTA
    text = "".join(open(os.path.join(nvrtc.device_headers(), f)).read()
                   for f in ("gemm_device.cuh", "sm100.cuh"))
    assert "tcgen05.mma" in text and "cp.async.bulk.tensor" in text
    word = "multi" + "cast"                              # no bulk copy is shared between CTAs
    assert not any(word in line for line in text.splitlines() if "cp.async.bulk" in line)
    # a reduction over the tile cannot run per element: that program keeps the two-kernel route
    r = rk.matmul_row_sums.specialize(P(tp.float16), P(tp.float16), P(tp.float32), 128, 128, 128, 128, 1,
                                      128, 1, BLOCK_M=128, BLOCK_N=128, BLOCK_K=64) \
        if hasattr(rk, "matmul_row_sums") else None
    if r is not None:
        assert isinstance(r.plan, lower.GemmEpiloguePlan) and r.plan.fused_source is None


def test_matmul_with_epilogue_splits_into_product_and_generated_kernel():
    x, y, bias, out = torch.randn(256, 128).half(), torch.randn(128, 192).half(), torch.randn(192), \
        torch.empty(256, 192).half()
    built = dt_linear_relu.built_for((x, y, bias, out))
    grid, pos, kw = dt_linear_relu.launch_parts(built, (x, y, bias, out),
                                                dt.Config(BLOCK_TILE_M=128, BLOCK_TILE_N=64, BLOCK_TILE_K=64))
    types = [P(tp.TORCH_TO_NEWT[str(a.dtype)]) if torch.is_tensor(a) else a for a in pos]
    plan = built.jit.specialize(*types, **kw).plan
    assert isinstance(plan, lower.GemmEpiloguePlan) and grid == (2, 3)
    assert isinstance(plan.gemm, lower.GemmPlan) and plan.gemm.c == "out_ptr"
    src = plan.epilogue.source
    assert "float* __restrict__ nb_acc" in src and "nb_acc[" in src and "fmaf(" not in src
    # the plain matmul still takes the one-kernel plan
    c = rk.matmul_kernel.specialize(F16, F16, F16, 64, 64, 64, 64, 1, 64, 1, 64, 1,
                                    BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    assert type(c.plan) is lower.GemmPlan


def test_deuteron_eager_reference_runs_on_host_tensors():
    x, y = torch.randn(64, 48).half(), torch.randn(48, 32).half()
    out = torch.empty(64, 32).half()
    dt_matmul.ref(x, y, out)   # the reference's eager mode cannot do this: its accumulator is pinned to CUDA
    torch.testing.assert_close(out.float(), x.float() @ y.float(), rtol=2e-2, atol=2e-2)


def test_deuteron_trace_errors():
    @dt.kernel
    def bad(x, out):
        y = x
        for t in dt.tile(x.shape[0]):
            out[t] = x[t]

    with pytest.raises(dt.TraceError, match="top level of a kernel holds tile loops only"):
        bad.to_newt_source(torch.zeros(4), torch.zeros(4))


def test_compile_fn_keeps_the_generator_contract():
    """newt/compiler/codegen.py:2758-2765 as driven by tests/test_codegen_cpu.py:22-31:
    (fndef, globals, params, constexprs, num_warps, name) -> (source, shared bytes[, plan])."""
    import ast
    import inspect
    import textwrap

    from newt_b200.compiler import codegen
    from newt_b200.compiler import types as ctp

    def scaled_add(x_ptr, y_ptr, out_ptr, n, alpha, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        ok = offs < n
        nl.store(out_ptr + offs, nl.load(x_ptr + offs, mask=ok) * alpha + nl.load(y_ptr + offs, mask=ok),
                 mask=ok)

    fndef = ast.parse(textwrap.dedent(inspect.getsource(scaled_add))).body[0]
    fp = ctp.pointer_type(ctp.float32)
    params = [(n, codegen.Value(codegen.UNIFORM, t, (), n))
              for n, t in dict(x_ptr=fp, y_ptr=fp, out_ptr=fp, n=ctp.int32, alpha=ctp.float32).items()]
    src, smem, plan = codegen.compile_fn(fndef, globals(), params, {"BLOCK": 1024}, 4, "k")
    assert "__launch_bounds__(128)" in src and "blockIdx.x" in src and "__restrict__" in src
    assert smem == 0 and isinstance(plan, lower.PointwisePlan) and 'void __launch_bounds__(128) k_' in src

    fndef = ast.parse(textwrap.dedent(inspect.getsource(rk.add_kernel.fn))).body[-1]
    params = [("x_ptr", fp), ("y_ptr", fp), ("out_ptr", fp), ("n", ctp.int32)]
    src, smem, plan = codegen.compile_fn(fndef, rk.add_kernel.fn.__globals__, params, {"BLOCK": 4096})
    assert isinstance(plan, lower.AddPlan) and "nb200_add_f32" in src and smem == 0


def test_runtime_cuda_compiles_raw_source_without_a_gpu():
    from newt_b200.runtime.cuda import Kernel, NVRTCError, compile_cuda

    src = 'extern "C" __global__ void saxpy(float a, const float* x, float* y, int n) {\n' \
          '  int i = blockIdx.x * blockDim.x + threadIdx.x;\n  if (i < n) y[i] = a * x[i] + y[i];\n}\n'
    cubin = compile_cuda(src, "saxpy", "sm_100")
    assert cubin[:4] == b"\x7fELF"
    k = Kernel(cubin, "saxpy", shared_bytes=0)      # loading is deferred to the first launch
    assert k.func_name == "saxpy"
    with pytest.raises(NVRTCError, match="saxpy.cu"):
        compile_cuda(src.replace("int i", "int i i"), "saxpy")


def test_cubins_are_cached_on_disk(tmp_path, monkeypatch):
    from newt_b200.runtime import nvrtc

    monkeypatch.setenv("NEWT_CACHE_DIR", str(tmp_path))
    src = 'extern "C" __global__ void twice(float* x) { x[threadIdx.x] *= 2.0f; }\n'
    first = nvrtc.compile_cubin_cached(src, "twice.cu")
    files = sorted(p.suffix for p in tmp_path.iterdir())
    assert files == [".cu", ".cubin"] and first[:4] == b"\x7fELF"
    calls = []
    monkeypatch.setattr(nvrtc, "compile_cubin", lambda *a, **k: calls.append(a) or b"")
    assert nvrtc.compile_cubin_cached(src, "twice.cu") == first and not calls      # served from disk
    nvrtc.compile_cubin_cached(src, "twice.cu", arch="sm_100")                     # another key
    assert len(calls) == 1
    # a truncated file is not trusted
    cubin = next(p for p in tmp_path.iterdir() if p.suffix == ".cubin" and p.stat().st_size > 0)
    cubin.write_bytes(b"junk")
    nvrtc.compile_cubin_cached(src, "twice.cu")
    assert len(calls) == 2


def test_constexpr_values_of_different_types_are_different_specializations():
    """2, 2.0 and True are equal (and hash alike) in Python; as constexprs they select integer,
    float and boolean arithmetic, so neither the specialization cache nor the launcher's fast
    key may fold them together (reference keys on repr: newt/runtime/jit.py:177-183)."""
    import newt_b200 as newt
    import newt_b200.language as nl

    @newt.jit
    def scaled(x_ptr, out_ptr, n, SCALE: nl.constexpr, BLOCK: nl.constexpr):
        offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        mask = offs < n
        nl.store(out_ptr + offs, nl.load(x_ptr + offs, mask=mask) * SCALE, mask=mask)

    compiled = [scaled.specialize(F32, F32, 100, SCALE=s, BLOCK=128) for s in (2, 2.0, True)]
    assert len({id(c) for c in compiled}) == 3 and len(scaled.cache) == 3
    keys = [scaled._fast_key(scaled._bind((F32, F32, 100), {"SCALE": s, "BLOCK": 128}), 4, 3)
            for s in (2, 2.0, True)]
    assert len(set(keys)) == 3
    assert scaled._fast_key(scaled._bind((F32, F32, 100), {"SCALE": [1], "BLOCK": 128}), 4, 3) is None
