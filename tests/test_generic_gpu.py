"""Control flow and dots outside the tuned kernels, on the device: the programs of
tests/generic_programs.py run through the generic lowering and are compared with torch on the
CPU.  Integer results and pure data movement are bit-exact; the tolerances of the
floating-point cases are stated with each case (fold order differs from torch's; fp32 dot
operands are rounded to tf32, as on the tensor core)."""

import pytest
import torch

import generic_programs as gp
import newt_b200 as newt
from newt_b200 import language as nl

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", sorted(gp.CASES))
def test_program_matches_torch(name):
    kernel, grid, args, meta, checks = gp.build(name, "cuda")
    kernel[grid](*args, **meta)
    torch.cuda.synchronize()
    for got, want, rtol, atol in checks:
        got = got.cpu()
        if rtol == 0 and atol == 0:
            assert torch.equal(got, want), f"{name}: {(got != want).sum().item()} elements differ"
        else:
            torch.testing.assert_close(got.float(), want.float(), rtol=rtol, atol=atol)


def test_ragged_matmul_is_copied_to_a_fetchable_layout_and_runs_on_the_tensor_core():
    """The same program text: operands whose pitches bulk tensor copies cannot fetch are first
    copied into an aligned workspace (two operands here), aligned ones are used as they lie."""
    from newt_b200.frontend.lower import GemmPlan

    kernel, grid, args, meta, checks = gp.build("ragged_matmul", "cuda")
    compiled = kernel.specialize(*args, **meta)
    assert isinstance(compiled.plan, GemmPlan)
    before = compiled.plan.repitched
    kernel[grid](*args, **meta)
    assert compiled.plan.repitched == before + 2 and compiled.plan._generic_plan is None

    m, n, k = 128, 128, 64
    g = torch.Generator().manual_seed(3)
    a = torch.randn(m, k, generator=g).half().cuda()
    b = torch.randn(k, n, generator=g).half().cuda()
    c = torch.zeros(m, n, device="cuda", dtype=torch.float16)
    kernel[(1, 1)](a, b, c, m, n, k, k, 1, n, 1, n, 1, BM=128, BN=128, BK=64)
    assert compiled.plan.repitched == before + 2
    torch.testing.assert_close(c.float().cpu(), (a.float() @ b.float()).cpu(), rtol=2e-3, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_transposed_a_and_odd_sizes_on_the_tensor_core(dtype):
    """A given transposed, odd M, N, K (rows of 333, 257 and 1001 elements) and a base pointer
    that is not 16-byte aligned: all three operands' layouts are ones TMA refuses."""
    import newt_b200 as newt
    from newt_b200.frontend.lower import GemmPlan

    m, n, k = 333, 257, 1001
    g = torch.Generator().manual_seed(11)
    a = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
    b = (torch.randn(k, n, generator=g) * 0.5).to(dtype)
    at = a.t().contiguous().cuda()                     # [k, m]: A[i, j] at j * m + i
    b_store = torch.empty(k * n + 1, device="cuda", dtype=dtype)
    b_dev = b_store[1:].view(k, n)                     # base off by one element
    b_dev.copy_(b)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    kernel = gp.ragged_matmul
    kernel[(newt.cdiv(m, 64), newt.cdiv(n, 64))](at, b_dev, c, m, n, k, 1, m, n, 1, n, 1,
                                                  BM=64, BN=64, BK=32)
    torch.cuda.synchronize()
    plan = kernel.specialize(at, b_dev, c, m, n, k, 1, m, n, 1, n, 1, BM=64, BN=64, BK=32).plan
    assert isinstance(plan, GemmPlan) and plan._generic_plan is None and plan.repitched >= 2
    ref = a.double() @ b.double()
    err = ((c.cpu().double() - ref).norm() / ref.norm()).item()
    assert err <= (2e-3 if dtype == torch.float32 else 1e-3), err


def test_repitch_entry_point_is_bit_exact():
    """nb200_repitch moves bits: any two strides in, row-major with a 16-byte pitch out."""
    from newt_b200.runtime import kernels

    for dtype, rows, cols in ((torch.float16, 130, 75), (torch.float32, 65, 200), (torch.bfloat16, 1, 1)):
        g = torch.Generator().manual_seed(rows)
        x = torch.randn(rows, cols, generator=g).to(dtype)
        for src, rs, cs in ((x.cuda(), cols, 1), (x.t().contiguous().cuda(), 1, rows)):
            ws, pitch = kernels.repitched("a", src, rows, cols, rs, cs)
            assert pitch % (16 // x.element_size()) == 0 and pitch >= cols
            got = ws[:rows * pitch].view(rows, pitch)[:, :cols].cpu()
            assert torch.equal(got, x)


def test_matmul_with_epilogue_runs_the_product_on_the_tensor_core():
    """Bias and activation after the k loop: the product goes through nb200_gemm_acc32 into an
    fp32 buffer, the epilogue is a generated kernel reading it; one rounding, at the store."""
    from newt_b200.frontend.lower import GemmEpiloguePlan

    m, n, k = 512, 768, 256
    g = torch.Generator().manual_seed(5)
    a = (torch.randn(m, k, generator=g) * 0.5).bfloat16()
    b = (torch.randn(k, n, generator=g) * 0.5).bfloat16()
    bias = torch.randn(n, generator=g)
    ad, bd, biasd = a.cuda(), b.cuda(), bias.cuda()
    c = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    meta = dict(BM=128, BN=128, BK=64)
    plan = gp.matmul_bias_relu.specialize(ad, bd, biasd, c, m, n, k, **meta).plan
    assert isinstance(plan, GemmEpiloguePlan)
    gp.matmul_bias_relu[(m // 128, n // 128)](ad, bd, biasd, c, m, n, k, **meta)
    torch.cuda.synchronize()
    want = torch.relu(a.double() @ b.double() + bias.double())
    # fp32 accumulation and one bf16 rounding: half an ulp of bf16 (2^-9) plus the sum's error
    torch.testing.assert_close(c.cpu().double(), want, rtol=2 ** -8, atol=2e-3)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("transposed", [False, True])
def test_gemm_acc32_keeps_the_accumulator(dtype, transposed):
    from newt_b200.runtime import kernels

    m, n, k = 200, 136, 264
    g = torch.Generator().manual_seed(6)
    a = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
    b = (torch.randn(k, n, generator=g) * 0.5).to(dtype)
    bd = b.t().contiguous().cuda() if transposed else b.cuda()
    c = torch.full((m, n + 3), float("nan"), device="cuda")            # a pitch of its own
    kernels.gemm_acc32(a.cuda(), bd, c, m, n, k, k, k if transposed else n, n + 3, transposed)
    torch.cuda.synchronize()
    want = a.double() @ b.double()
    got = c[:, :n].cpu().double()
    assert ((got - want).norm() / want.norm()).item() < 1e-6          # fp32 sums of exact products
    assert torch.isnan(c[:, n:]).all()


def test_epilogue_matmul_with_a_transposed_result_takes_the_one_kernel_path():
    """C written with unit stride down its columns: the tensor-core kernels do not store that
    way, so the whole program (k loop and epilogue) runs as one generated kernel."""
    from newt_b200.examples import kernels as K
    from newt_b200.frontend.lower import GemmEpiloguePlan

    m, n, k = 64, 96, 64
    g = torch.Generator().manual_seed(8)
    a = (torch.randn(m, k, generator=g) * 0.5).half()
    b = (torch.randn(k, n, generator=g) * 0.5).half()
    bias = torch.randn(n, generator=g)
    ad, bd, biasd = a.cuda(), b.cuda(), bias.cuda()
    ct = torch.full((n, m), float("nan"), device="cuda", dtype=torch.float16)
    meta = dict(BLOCK_M=32, BLOCK_N=32, BLOCK_K=32)
    args = (ad, bd, biasd, ct, m, n, k, k, 1, n, 1, 1, m)
    K.linear_bias_relu_kernel[(2, 3)](*args, **meta)
    torch.cuda.synchronize()
    plan = K.linear_bias_relu_kernel.specialize(*args, **meta).plan
    assert isinstance(plan, GemmEpiloguePlan) and plan._whole_plan is not None
    want = torch.relu(a.float() @ b.float() + bias)
    torch.testing.assert_close(ct.t().cpu().float(), want, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("m,n,k,dtype", [(64, 96, 64, torch.float16), (300, 200, 136, torch.bfloat16),
                                         (1024, 768, 512, torch.bfloat16),
                                         (2048, 2048, 1024, torch.float16),
                                         (300, 200, 136, torch.float32), (1024, 768, 512, torch.float32)])
def test_epilogue_is_compiled_into_the_tensor_core_kernel(m, n, k, dtype):
    """bias + relu after the k loop: one launch of the tcgen05 kernel with the program's own
    epilogue compiled in (ragged edges, the one-CTA and the CTA-pair tiles), no fp32 buffer."""
    from newt_b200.examples import kernels as K
    from newt_b200.frontend.lower import GemmEpiloguePlan
    from newt_b200.runtime import abi

    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) * 0.5).to(dtype)
    b = (torch.randn(k, n, generator=g) * 0.5).to(dtype)
    bias = torch.randn(n, generator=g)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    K.linear_bias_relu(a.cuda(), b.cuda(), bias.cuda(), c)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    plans = [r.plan for r in K.linear_bias_relu_kernel.cache.values()
             if isinstance(r.plan, GemmEpiloguePlan) and r.plan._fused_kernels]
    assert plans, "the epilogue ran as a second kernel"
    assert all(p._whole_plan is None for p in plans)
    want = torch.relu(a.double() @ b.double() + bias.double())
    got = c.cpu().double()
    assert not torch.isnan(got).any()
    tol = {torch.bfloat16: 2 ** -8, torch.float16: 2 ** -10, torch.float32: 2e-3}[dtype]   # fp32 runs as tf32
    assert ((got - want).norm() / want.norm()).item() < tol


@newt.jit
def _relu_axpy(x_ptr, y_ptr, o_ptr, n, BLOCK: nl.constexpr):
    offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    m = offs < n
    x = nl.load(x_ptr + offs, mask=m, other=0.0)
    y = nl.load(y_ptr + offs, mask=m, other=0.0)
    nl.store(o_ptr + offs, nl.maximum(x * 2.0 + y, 0.0), mask=m)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("n,offset", [(1 << 16, 0), ((1 << 16) - 3, 0), (5000, 1), (8, 0), (7, 0)])
def test_sixteen_bit_blocks_move_sixteen_bytes_at_a_time(dtype, n, offset):
    """A 16-bit elementwise program: eight neighbours per trip through one 16-byte access where
    the address is aligned and all eight masks hold, lane by lane at the ragged tail and from a
    base off by one element; bit-exact against the same operations in torch either way, and
    nothing written outside [0, n)."""
    g = torch.Generator().manual_seed(n + offset)
    x = torch.randn(n + 16, generator=g).to(dtype).cuda()
    y = torch.randn(n + 16, generator=g).to(dtype).cuda()
    o = torch.full((n + 16,), 7.0, device="cuda", dtype=dtype)
    xs, ys, os_ = x[offset:offset + n], y[offset:offset + n], o[offset:offset + n]
    block = 1024
    _relu_axpy[(newt.cdiv(n, block),)](xs, ys, os_, n, BLOCK=block)
    torch.cuda.synchronize()
    plan = _relu_axpy.specialize(xs, ys, os_, n, BLOCK=block).plan
    assert "uint4" in plan.source          # the program was given the 16-byte path
    want = torch.relu((xs * 2.0).to(dtype) + ys)
    assert torch.equal(os_, want)
    assert (o[:offset] == 7.0).all() and (o[offset + n:] == 7.0).all()


# ---- rows kept in registers: programs of the softmax / layernorm family the tuned kernels do
# ---- not recognise (a temperature, a logarithm, no mean, no bias)

@newt.jit
def _log_softmax(x_ptr, out_ptr, N, stride, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf"))
    z = x - nl.max(x, axis=0)
    nl.store(out_ptr + row * stride + cols, z - nl.log(nl.sum(nl.exp(z), axis=0)), mask=mask)


@newt.jit
def _softmax_with_temperature(x_ptr, out_ptr, N, stride, inv_t, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf")) * inv_t
    e = nl.exp(x - nl.max(x, axis=0))
    nl.store(out_ptr + row * stride + cols, e / nl.sum(e, axis=0), mask=mask)


@newt.jit
def _rmsnorm(x_ptr, w_ptr, out_ptr, N, stride, eps, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=0.0).to(nl.float32)
    ms = nl.sum(x * x, axis=0) / N
    y = x * nl.rsqrt(ms + eps) * nl.load(w_ptr + cols, mask=mask, other=0.0)
    nl.store(out_ptr + row * stride + cols, y, mask=mask)


@newt.jit
def _layernorm_without_bias(x_ptr, w_ptr, out_ptr, N, stride, eps, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=0.0).to(nl.float32)
    mean = nl.sum(x, axis=0) / N
    d = nl.where(mask, x - mean, 0.0)
    var = nl.sum(d * d, axis=0) / N
    y = d * nl.rsqrt(var + eps) * nl.load(w_ptr + cols, mask=mask, other=0.0)
    nl.store(out_ptr + row * stride + cols, y, mask=mask)


@pytest.mark.parametrize("n,block,offset", [(1024, 1024, 0), (1000, 1024, 0), (4096, 4096, 0),
                                            (2040, 2048, 0), (1000, 1024, 1)])
def test_rows_of_the_softmax_family_stay_in_registers(n, block, offset):
    """fp32 rows: whole vectors, a ragged tail (masked lanes), and a base that is off by one
    element (the one-element form of the same program)."""
    from newt_b200.frontend.lower import PointwisePlan

    rows = 37
    g = torch.Generator().manual_seed(n + offset)
    pitch = block + 8
    x = (torch.randn(rows * pitch + 8, generator=g) * 3).cuda()
    xs = x[offset:offset + rows * pitch].view(rows, pitch)
    for kernel, extra, want in (
            (_log_softmax, (), torch.log_softmax(xs[:, :n].double(), -1)),
            (_softmax_with_temperature, (0.37,), torch.softmax(xs[:, :n].double() * 0.37, -1))):
        o = torch.full((rows * pitch + 8,), 7.0, device="cuda")
        os_ = o[offset:offset + rows * pitch].view(rows, pitch)
        kernel[(rows,)](xs, os_, n, pitch, *extra, BLOCK_N=block)
        torch.cuda.synchronize()
        plan = kernel.specialize(xs, os_, n, pitch, *extra, BLOCK_N=block).plan
        assert isinstance(plan, PointwisePlan) and "nb_v0" in plan.source
        torch.testing.assert_close(os_[:, :n].double().cpu(), want.cpu(), rtol=2e-5, atol=2e-6)
        assert (os_[:, n:] == 7.0).all() and (o[:offset] == 7.0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,block", [(1024, 1024), (1000, 1024), (4096, 4096)])
def test_rows_of_the_layernorm_family_stay_in_registers(dtype, n, block):
    rows = 29
    g = torch.Generator().manual_seed(n)
    x = torch.randn(rows, block, generator=g).to(dtype).cuda()
    w = (1 + 0.1 * torch.randn(block, generator=g)).to(dtype).cuda()
    xd, wd = x[:, :n].double(), w[:n].double()
    tol = {torch.float16: 2e-3, torch.bfloat16: 1.6e-2, torch.float32: 1e-5}[dtype]
    rms = xd * torch.rsqrt((xd * xd).mean(-1, keepdim=True) + 1e-6) * wd
    d = xd - xd.mean(-1, keepdim=True)
    ln = d * torch.rsqrt((d * d).mean(-1, keepdim=True) + 1e-5) * wd
    for kernel, eps, want in ((_rmsnorm, 1e-6, rms), (_layernorm_without_bias, 1e-5, ln)):
        o = torch.full((rows, block), 7.0, device="cuda", dtype=dtype)
        kernel[(rows,)](x, w, o, n, block, eps, BLOCK_N=block)
        torch.cuda.synchronize()
        assert "nb_v0" in kernel.specialize(x, w, o, n, block, eps, BLOCK_N=block).plan.source
        torch.testing.assert_close(o[:, :n].double().cpu(), want.cpu(), rtol=tol, atol=tol)
        assert (o[:, n:] == 7.0).all()
