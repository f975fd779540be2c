"""GPU: the operator API end to end -- `@jit` kernels launched with the reference's
protocol, `@autotune`, `@heuristics`, `@dt.kernel` -- with results checked against the
CPU oracle.  Shapes follow the reference's own tests (tests/test_vector_add.py,
test_softmax_layernorm.py, test_matmul.py, test_deuteron.py, test_review_fixes.py)."""

import pytest
import torch

import newt_b200 as newt
import newt_b200.deuteron as dt
import newt_b200.language as nl
from newt_b200.runtime import abi, kernels
from oracle import cport, torch_ref

import ref_kernels as rk

pytestmark = pytest.mark.gpu


def _rand(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("n", [1024, 1 << 20, 12345])
def test_vector_add_bit_exact(n):
    x, y = _rand(n, 1), _rand(n, 2)
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty_like(xd)
    grid = lambda meta: (newt.cdiv(n, meta["BLOCK"]),)  # noqa: E731
    rk.add_kernel[grid](xd, yd, out, n, BLOCK=4096)
    assert torch.equal(out.cpu(), cport.add_f32(x, y))


@pytest.mark.parametrize("m,n", [(8, 128), (128, 1024), (32, 781), (4096, 2500)])
def test_softmax_kernel(m, n):
    x = _rand((m, n), 3)
    xd = x.cuda()
    out = torch.empty_like(xd)
    block = newt.next_power_of_2(n)
    rk.softmax_kernel[(m,)](xd, out, n, xd.stride(0), BLOCK_N=block,
                            num_warps=4 if block < 4096 else 8)
    torch.testing.assert_close(out.cpu(), torch_ref.softmax(x), rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("m,n", [(8, 128), (64, 2048), (16, 300)])
def test_layernorm_kernel(dtype, m, n):
    x, w, b = _rand((m, n), 4, dtype), _rand(n, 5, dtype), _rand(n, 6, dtype)
    xd = x.cuda()
    out = torch.empty_like(xd)
    rk.layernorm_kernel[(m,)](xd, w.cuda(), b.cuda(), out, n, xd.stride(0), 1e-5,
                              BLOCK_N=newt.next_power_of_2(n), num_warps=8)
    ref = torch_ref.layernorm(x, w, b)
    if dtype == torch.float32:
        torch.testing.assert_close(out.cpu(), ref, rtol=1e-3, atol=1e-4)
    else:
        assert torch_ref.rel_frobenius(out.cpu().float(), ref) <= 1e-2


def _run_matmul(kernel, m, n, k, dtype, bm=64, bn=64, bk=32, ld_pad=0, **kw):
    a = _rand((m, k), 7, dtype, 0.5)
    b = _rand((k, n), 8, dtype, 0.5)
    # ld_pad: keep the data ragged but make the row pitch a multiple of 8 elements (TMA)
    ka = -(-k // 8) * 8 if ld_pad else k
    na = -(-n // 8) * 8 if ld_pad else n
    a_dev = torch.empty(m, ka, device="cuda", dtype=dtype)[:, :k]
    a_dev.copy_(a)
    b_dev = torch.empty(k, na, device="cuda", dtype=dtype)[:, :n]
    b_dev.copy_(b)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    grid = (newt.cdiv(m, bm), newt.cdiv(n, bn))
    kernel[grid](a_dev, b_dev, c, m, n, k, a_dev.stride(0), a_dev.stride(1), b_dev.stride(0),
                 b_dev.stride(1), c.stride(0), c.stride(1), BLOCK_M=bm, BLOCK_N=bn, BLOCK_K=bk, **kw)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    return a, b, c.cpu()


@pytest.mark.parametrize("m,n,k,pad", [(64, 64, 32, 0), (256, 256, 128, 0), (300, 200, 100, 4),
                                       (129, 264, 72, 0)])
def test_matmul_fp16(m, n, k, pad):
    # (300, 200, 100): the reference's ragged case; row pitch padded to a multiple of 8
    # elements, which is what TMA needs
    a, b, c = _run_matmul(rk.matmul_kernel, m, n, k, torch.float16, ld_pad=pad)
    ref = torch_ref.matmul(a, b)
    assert torch_ref.rel_frobenius(c.float(), ref) <= 1e-2
    torch.testing.assert_close(c.float(), ref.half().float(), rtol=1e-2, atol=1e-2)
    if m * n * k <= 256 * 256 * 128:
        torch.testing.assert_close(c.float(), cport.matmul(a, b).float(), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("m,n,k,bm,bn,bk,pad", [(128, 128, 128, 64, 64, 32, 0),   # tests/test_matmul.py:67-70
                                               (300, 200, 100, 64, 64, 32, 4),
                                               (512, 768, 160, 128, 256, 32, 0),
                                               (512, 512, 256, 256, 256, 64, 0)])   # CTA pair
def test_matmul_fp32_runs_as_tf32(m, n, k, bm, bn, bk, pad):
    # nl.dot on fp32 blocks is a tf32 product with fp32 accumulation (newt/language.py:165-167)
    a, b, c = _run_matmul(rk.matmul_kernel, m, n, k, torch.float32, bm=bm, bn=bn, bk=bk, ld_pad=pad)
    ref = a.double() @ b.double()
    torch.testing.assert_close(c.double(), ref, rtol=1e-2, atol=1e-2)      # the reference's bar
    assert torch_ref.rel_frobenius(c, ref) <= 2e-3                         # tf32 inputs: ~2^-11 each
    if m * n * k <= 512 * 768 * 160:
        # the oracle rounds the operands to tf32 as the reference does; the tensor core drops
        # the low mantissa bits instead, so the two differ by rounding of the operands only
        assert torch_ref.rel_frobenius(c, cport.matmul(a, b)) <= 2e-3


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_matmul_with_b_transposed(dtype):
    # the same kernel text, called with B^T in memory: stride_bk = 1, stride_bn = row pitch
    m, n, k = 192, 320, 136
    a = _rand((m, k), 21, dtype, 0.5)
    b = _rand((k, n), 22, dtype, 0.5)
    bt = b.t().contiguous().cuda()            # [n, k], pitch 136: a multiple of 8
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    rk.matmul_kernel[(newt.cdiv(m, 64), newt.cdiv(n, 64))](
        a.cuda(), bt, c, m, n, k, k, 1, 1, k, n, 1, BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    assert torch_ref.rel_frobenius(c.cpu().float(), a.double() @ b.double()) <= (
        2e-3 if dtype == torch.float32 else 1e-2)


def test_matmul_bf16_and_tiles():
    for bn, stages in ((64, 2), (128, 3), (256, 4)):
        a, b, c = _run_matmul(rk.matmul_kernel, 256, 512, 192, torch.bfloat16, bm=128, bn=bn,
                              bk=64, num_stages=stages)
        assert torch_ref.rel_frobenius(c.float(), torch_ref.matmul(a, b)) <= 1e-2


def test_matmul_small_c_long_k_splits_the_tiles():
    # 16 tiles of 256 x 256 for 74 CTA pairs, 256 k steps each: the launcher asks the library,
    # which cuts the tiles along K and sums the parts through a workspace of the launch's own
    m = n = 1024
    k = 16384
    calls = []
    real = kernels.gemm_split

    def spy(*args, **kw):
        calls.append(args[3:6])
        return real(*args, **kw)

    kernels.gemm_split = spy
    try:
        a, b, c = _run_matmul(rk.matmul_kernel, m, n, k, torch.float16, bm=256, bn=256, bk=64)
    finally:
        kernels.gemm_split = real
    assert calls == [(m, n, k)]
    assert torch_ref.rel_frobenius(c.float(), torch_ref.matmul(a, b)) <= 1e-2


def test_matmul_unmasked_kernel():
    a, b, c = _run_matmul(rk.matmul_kernel_unmasked, 256, 256, 128, torch.float16, bm=128,
                          bn=128, bk=64)
    assert torch_ref.rel_frobenius(c.float(), torch_ref.matmul(a, b)) <= 1e-2


def test_matmul_unaligned_pitch_is_copied_first():
    """A 200-byte pitch is not TMA-legal: the C-ABI call refuses it with a message (no launch
    is attempted); the `@jit` launch copies such operands into an aligned workspace first
    (nb200_repitch) and runs the same tensor-core kernel."""
    from newt_b200.runtime import kernels

    a = _rand((64, 100), 21, torch.float16, 0.5)
    b = _rand((100, 64), 22, torch.float16, 0.5)
    ad, bd = a.cuda(), b.cuda()
    c = torch.zeros(64, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(abi.UnsupportedError, match="multiple of 8"):
        kernels.gemm(ad, bd, c, 64, 64, 100, 100, 64, 64)
    rk.matmul_kernel[(1, 1)](ad, bd, c, 64, 64, 100, 100, 1, 64, 1, 64, 1,
                             BLOCK_M=64, BLOCK_N=64, BLOCK_K=32)
    assert torch_ref.rel_frobenius(c.cpu().float(), torch_ref.matmul(a, b)) <= 2e-3


def test_autotune_picks_a_config_and_caches_it():
    tuned = newt.autotune(
        configs=[newt.Config({"BLOCK_M": 128, "BLOCK_N": 256, "BLOCK_K": 64}, num_stages=4),
                 newt.Config({"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64}, num_stages=4),
                 newt.Config({"BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64}, num_stages=3)],
        key=["M", "N", "K"])(rk.matmul_kernel)
    m = n = k = 512
    a, b = _rand((m, k), 9, torch.float16, 0.5), _rand((k, n), 10, torch.float16, 0.5)
    ad, bd = a.cuda(), b.cuda()
    c = torch.empty(m, n, device="cuda", dtype=torch.float16)
    grid = lambda meta: (newt.cdiv(m, meta["BLOCK_M"]), newt.cdiv(n, meta["BLOCK_N"]))  # noqa: E731
    for _ in range(2):
        tuned[grid](ad, bd, c, m, n, k, k, 1, n, 1, n, 1)
    assert tuned.best_config in tuned.configs and len(tuned.cache) == 1
    assert torch_ref.rel_frobenius(c.cpu().float(), torch_ref.matmul(a, b)) <= 1e-2


def test_heuristics_and_grid_meta():
    seen = {}
    h = newt.heuristics({"BLOCK": lambda args: 256 if args["n"] < 1000 else 1024})(rk.add_kernel)
    n = 700
    x, y = _rand(n, 11).cuda(), _rand(n, 12).cuda()
    out = torch.empty_like(x)

    def grid(meta):
        seen.update(meta)
        return (newt.cdiv(meta["n"], meta["BLOCK"]),)

    h[grid](x, y, out, n)
    assert seen["BLOCK"] == 256 and seen["n"] == n and seen["num_warps"] == 4
    assert torch.equal(out, x + y)


def test_zero_grid_is_noop_and_wrong_device_type():
    x = torch.ones(16, device="cuda")
    out = torch.zeros(16, device="cuda")
    rk.add_kernel[(0,)](x, x, out, 16, BLOCK=16)
    assert out.sum().item() == 0


def test_autotune_reset_to_zero_first_call():
    calls = []

    class FakeJit:
        param_names = ["x", "n"]
        defaults = {}
        __name__ = "fake"

        def __getitem__(self, grid):
            def run(x, n, **kw):
                calls.append(float(x.sum().item()))
                x += 1
            return run

    tuner = newt.Autotuner(FakeJit(), [newt.Config({}), newt.Config({})], key=["n"],
                           reset_to_zero=["x"], warmup=0, rep=1)
    x = torch.zeros(4, device="cuda")
    tuner[(1,)](x, 4)
    assert x.sum().item() == 4.0      # buffer was cleared after tuning, then one real run
    assert all(c == 0.0 for c in calls)  # every timed call started from zero


def test_attention_example_as_shipped():
    # examples/05_fused_attention.py:66-80: M = N = 1024, D = 64, fp16, single head, vs SDPA
    m = n = 1024
    d = 64
    q, k, v = (_rand((m, d), s, torch.float16) for s in (21, 22, 23))
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o = torch.empty_like(qd)
    rk.attention_kernel_2d[(newt.cdiv(m, 64),)](
        qd, kd, vd, o, m, n, 1.0 / d ** 0.5, qd.stride(0), qd.stride(1), kd.stride(0),
        kd.stride(1), vd.stride(0), vd.stride(1), o.stride(0), o.stride(1),
        BLOCK_M=64, BLOCK_N=64, D=d, num_warps=4)
    ref = torch_ref.attention(q[None], k[None], v[None], 1.0 / d ** 0.5)[0]
    assert (o.cpu().float() - ref).abs().max().item() < 2e-2      # the example's own bar
    assert torch_ref.rel_frobenius(o.cpu().float(), ref) <= 1e-2


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attention_batched(causal, dtype):
    from newt_b200 import examples

    b, h, s, d = 2, 3, 640, 128
    q, k, v = (_rand((b, h, s, d), sd, dtype) for sd in (24, 25, 26))
    o = examples.attention(q.cuda(), k.cuda(), v.cuda(), causal=causal)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    ref = torch_ref.attention(q.reshape(b * h, s, d), k.reshape(b * h, s, d),
                              v.reshape(b * h, s, d), 1.0 / d ** 0.5, causal)
    assert torch_ref.rel_frobenius(o.cpu().reshape(b * h, s, d).float(), ref) <= 1e-2


# ---- deuteron ---------------------------------------------------------------------

@dt.kernel(config={"BLOCK_TILE_M": 128, "BLOCK_TILE_N": 128, "BLOCK_TILE_K": 64, "num_stages": 4})
def dt_matmul_fixed(x, y, out):
    for tile_m, tile_n in dt.tile([x.shape[0], y.shape[1]]):
        acc = dt.zeros([tile_m, tile_n], dtype=dt.float32)
        for tile_k in dt.tile(x.shape[1]):
            acc += x[tile_m, tile_k] @ y[tile_k, tile_n]
        out[tile_m, tile_n] = acc


@dt.kernel
def dt_matmul_tuned(x, y, out):
    for tile_m, tile_n in dt.tile([x.shape[0], y.shape[1]]):
        acc = dt.zeros([tile_m, tile_n], dtype=dt.float32)
        for tile_k in dt.tile(x.shape[1]):
            acc += x[tile_m, tile_k] @ y[tile_k, tile_n]
        out[tile_m, tile_n] = acc


def test_deuteron_matmul_fixed_config():
    x, y = _rand((512, 384), 13, torch.float16, 0.5), _rand((384, 256), 14, torch.float16, 0.5)
    out = torch.empty(512, 256, device="cuda", dtype=torch.float16)
    dt_matmul_fixed(x.cuda(), y.cuda(), out)
    assert torch_ref.rel_frobenius(out.cpu().float(), torch_ref.matmul(x, y)) <= 1e-2


def test_deuteron_matmul_autotuned_bf16(tmp_path, monkeypatch):
    monkeypatch.setenv("DEUTERON_CACHE_DIR", str(tmp_path))
    x, y = _rand((1024, 768), 15, torch.bfloat16, 0.5), _rand((768, 512), 16, torch.bfloat16, 0.5)
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty(1024, 512, device="cuda", dtype=torch.bfloat16)
    dt_matmul_tuned(xd, yd, out)
    assert torch_ref.rel_frobenius(out.cpu().float(), torch_ref.matmul(x, y)) <= 1e-2
    best = dt_matmul_tuned.best_config
    assert best["BLOCK_TILE_N"] in (64, 128, 256) and (tmp_path / "configs.json").exists()
    ref = torch.empty_like(out)
    dt_matmul_tuned.ref(xd, yd, ref)          # eager oracle on the device
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


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


def test_deuteron_softmax_non_pow2_columns(tmp_path, monkeypatch):
    # tests/test_deuteron.py:64-71 of the reference: 1000 x 777
    monkeypatch.setenv("DEUTERON_CACHE_DIR", str(tmp_path))
    x = _rand((1000, 777), 31)
    out = torch.empty(1000, 777, device="cuda")
    dt_softmax(x.cuda(), out)
    torch.testing.assert_close(out.cpu(), torch_ref.softmax(x), rtol=1e-5, atol=1e-9)


def test_deuteron_layernorm(tmp_path, monkeypatch):
    # examples/deuteron/03_layernorm.py: 4096 x 1500 fp32, err < 1e-3
    monkeypatch.setenv("DEUTERON_CACHE_DIR", str(tmp_path))
    x, w, b = _rand((512, 1500), 32), _rand(1500, 33), _rand(1500, 34)
    out = torch.empty(512, 1500, device="cuda")
    dt_layernorm(x.cuda(), w.cuda(), b.cuda(), out, 1e-5)
    assert (out.cpu() - torch_ref.layernorm(x, w, b)).abs().max().item() < 1e-3


# ---- block arithmetic outside the tuned programs: generated CUDA, compiled at run time ----

@newt.jit
def pw_gelu_residual(x_ptr, y_ptr, out_ptr, n, BLOCK: nl.constexpr):
    offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    m = offs < n
    v = nl.load(x_ptr + offs, mask=m, other=0.0)
    inner = 0.7978845608028654 * (v + 0.044715 * v * v * v)
    g = 0.5 * v * (1.0 + nl.tanh(inner))
    nl.store(out_ptr + offs, g + nl.load(y_ptr + offs, mask=m), mask=m)


@newt.jit
def pw_bias_relu_2d(x_ptr, b_ptr, out_ptr, M, N, sx, so, BM: nl.constexpr, BN: nl.constexpr):
    rm = nl.program_id(0) * BM + nl.arange(0, BM)
    rn = nl.program_id(1) * BN + nl.arange(0, BN)
    mask = (rm[:, None] < M) & (rn[None, :] < N)
    x = nl.load(x_ptr + rm[:, None] * sx + rn[None, :], mask=mask, other=0.0)
    b = nl.load(b_ptr + rn, mask=rn < N, other=0.0)
    nl.store(out_ptr + rm[:, None] * so + rn[None, :], nl.maximum(x + b[None, :], 0.0), mask=mask)


@newt.jit
def pw_mixed(x_ptr, i_ptr, f_out, i_out, n, alpha, BLOCK: nl.constexpr):
    offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    m = offs < n
    x = nl.load(x_ptr + offs, mask=m, other=1.0)
    k = nl.load(i_ptr + offs, mask=m, other=0)
    y = nl.where(k % 3 == 0, nl.exp(-nl.abs(x)) * alpha, nl.sqrt(nl.abs(x)) / (1.0 + nl.sigmoid(x)))
    nl.store(f_out + offs, y.to(nl.float16), mask=m)
    nl.store(i_out + offs, (k * 7 + offs) // 5 - (k >> 1), mask=m)


def test_generated_elementwise_fp32():
    n = 100_003
    x, y = _rand((n,), 31), _rand((n,), 32)
    out = torch.full((n,), float("nan"), device="cuda")
    pw_gelu_residual[(newt.cdiv(n, 1024),)](x.cuda(), y.cuda(), out, n, BLOCK=1024)
    torch.cuda.synchronize()
    ref = torch.nn.functional.gelu(x.double(), approximate="tanh") + y.double()
    torch.testing.assert_close(out.cpu().double(), ref, rtol=2e-6, atol=2e-6)


def test_generated_elementwise_fp16_2d_broadcast_is_bit_exact():
    m, n = 300, 517
    x, b = _rand((m, n), 33, torch.float16), _rand((n,), 34, torch.float16)
    xd = torch.zeros(m, n + 3, device="cuda", dtype=torch.float16)[:, :n]   # a row pitch that is not n
    xd.copy_(x)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)
    pw_bias_relu_2d[(newt.cdiv(m, 32), newt.cdiv(n, 64))](xd, b.cuda(), out, m, n, xd.stride(0),
                                                           out.stride(0), BM=32, BN=64, num_warps=8)
    torch.cuda.synchronize()
    # every fp16 operation is one fp32 operation rounded to fp16, which is what torch does on CPU
    assert torch.equal(out.cpu(), torch.relu(x + b[None, :]))


def test_generated_elementwise_mixed_types_two_stores():
    n = 5000
    x = _rand((n,), 35)
    k = torch.randint(-1000, 1000, (n,), generator=torch.Generator().manual_seed(36), dtype=torch.int32)
    f_out = torch.full((n,), float("nan"), device="cuda", dtype=torch.float16)
    i_out = torch.full((n,), -1, device="cuda", dtype=torch.int32)
    pw_mixed[(newt.cdiv(n, 256),)](x.cuda(), k.cuda(), f_out, i_out, n, 0.25, BLOCK=256)
    torch.cuda.synchronize()
    xd = x.double()
    # `%`, `//` and `>>` are C's on int32 (truncating division), as in the reference's lowering
    c_mod = torch.fmod(k, 3)
    want_f = torch.where(c_mod == 0, torch.exp(-xd.abs()) * 0.25,
                         xd.abs().sqrt() / (1.0 + torch.sigmoid(xd)))
    torch.testing.assert_close(f_out.cpu().double(), want_f, rtol=2e-3, atol=1e-6)
    t = k * 7 + torch.arange(n, dtype=torch.int32)
    want_i = torch.div(t, 5, rounding_mode="trunc") - (k >> 1)
    assert torch.equal(i_out.cpu(), want_i.to(torch.int32))


@dt.kernel
def dt_fused_gelu_residual(x, y, out):
    # examples/deuteron/04_fused_ops.py of the reference
    for t in dt.tile(x.shape[0]):
        v = x[t]
        inner = 0.7978845608028654 * (v + 0.044715 * v * v * v)
        g = 0.5 * v * (1.0 + dt.tanh(inner))
        out[t] = g + y[t]


def test_deuteron_fused_elementwise_chain(tmp_path, monkeypatch):
    monkeypatch.setenv("DEUTERON_CACHE_DIR", str(tmp_path))
    n = 1 << 18
    x, y = _rand((n,), 37), _rand((n,), 38)
    out = torch.full((n,), float("nan"), device="cuda")
    dt_fused_gelu_residual(x.cuda(), y.cuda(), out)
    torch.cuda.synchronize()
    ref = torch.nn.functional.gelu(x.double(), approximate="tanh") + y.double()
    assert (out.cpu().double() - ref).abs().max().item() < 1e-5     # the example's own bar


@dt.kernel
def dt_center_rows(x, out):
    for tile_m in dt.tile(x.shape[0]):
        row = x[tile_m, :]
        out[tile_m, :] = row - row.mean(1)[:, None]


@dt.kernel(config={"BLOCK_TILE_M": 32, "BLOCK_TILE_N": 64})
def dt_scale_by_mean(x, out):
    for tile_m, tile_n in dt.tile([x.shape[0], x.shape[1]]):
        block = x[tile_m, tile_n]
        out[tile_m, tile_n] = block / block.mean()


def test_deuteron_mean(tmp_path, monkeypatch):
    """mean() over the valid lanes of a tile: along an axis of ragged rows, and over a whole
    tile (every tile here is full, so each is scaled by its own mean)."""
    monkeypatch.setenv("DEUTERON_CACHE_DIR", str(tmp_path))
    x = _rand((37, 777), 41)
    out = torch.full((37, 777), float("nan"), device="cuda")
    dt_center_rows(x.cuda(), out)
    torch.testing.assert_close(out.cpu(), x - x.mean(1, keepdim=True), rtol=1e-5, atol=1e-5)
    x = _rand((64, 128), 42).abs() + 1.0
    out = torch.full((64, 128), float("nan"), device="cuda")
    dt_scale_by_mean(x.cuda(), out)
    want = x.clone()
    for i in range(0, 64, 32):
        for j in range(0, 128, 64):
            want[i:i + 32, j:j + 64] /= x[i:i + 32, j:j + 64].mean()
    torch.testing.assert_close(out.cpu(), want, rtol=1e-5, atol=1e-6)


@newt.jit
def pw_rmsnorm(x_ptr, w_ptr, out_ptr, N, stride, eps, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=0.0).to(nl.float32)
    ms = nl.sum(x * x, axis=0) / N
    y = x * nl.rsqrt(ms + eps) * nl.load(w_ptr + cols, mask=mask, other=0.0)
    nl.store(out_ptr + row * stride + cols, y, mask=mask)


@newt.jit
def pw_log_softmax(x_ptr, out_ptr, N, stride, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf"))
    z = x - nl.max(x, axis=0)
    nl.store(out_ptr + row * stride + cols, z - nl.log(nl.sum(nl.exp(z), axis=0)), mask=mask)


@newt.jit
def pw_tile_stats(x_ptr, colmax_ptr, rowsum_ptr, total_ptr, M, N, sx, BM: nl.constexpr, BN: nl.constexpr):
    # one program per BN columns, walking BM rows: column maxima, and per program row sums + a total
    pid = nl.program_id(0)
    rn = pid * BN + nl.arange(0, BN)
    rm = nl.arange(0, BM)
    mask = (rm[:, None] < M) & (rn[None, :] < N)
    x = nl.load(x_ptr + rm[:, None] * sx + rn[None, :], mask=mask, other=float("-inf"))
    nl.store(colmax_ptr + rn, nl.max(x, axis=0), mask=rn < N)
    z = nl.where(mask, x, 0.0)
    nl.store(rowsum_ptr + pid * BM + rm, nl.sum(z, axis=1))
    nl.store(total_ptr + pid, nl.sum(z))


def test_generated_row_reductions():
    m, n = 37, 1000
    x, w = _rand((m, n), 41, torch.float16), _rand((n,), 42, torch.float16)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float16)
    pw_rmsnorm[(m,)](x.cuda(), w.cuda(), out, n, n, 1e-6, BLOCK_N=1024, num_warps=8)
    xf = x.float()
    ref = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert torch_ref.rel_frobenius(out.cpu().float(), ref) <= 1e-3
    xs = _rand((m, n), 43)
    outs = torch.full((m, n), float("nan"), device="cuda")
    pw_log_softmax[(m,)](xs.cuda(), outs, n, n, BLOCK_N=1024)
    torch.cuda.synchronize()
    torch.testing.assert_close(outs.cpu(), torch.log_softmax(xs, -1), rtol=1e-5, atol=1e-5)


def test_generated_reductions_over_2d_blocks():
    m, n, bm, bn = 50, 300, 64, 128
    x = _rand((m, n), 44)
    progs = newt.cdiv(n, bn)
    colmax = torch.full((n,), float("nan"), device="cuda")
    rowsum = torch.full((progs, bm), float("nan"), device="cuda")
    total = torch.full((progs,), float("nan"), device="cuda")
    pw_tile_stats[(progs,)](x.cuda(), colmax, rowsum, total, m, n, n, BM=bm, BN=bn)
    torch.cuda.synchronize()
    assert torch.equal(colmax.cpu(), x.max(0).values)                       # max is exact
    xp = torch.zeros(bm, progs * bn)
    xp[:m, :n] = x
    want_rows = xp.view(bm, progs, bn).sum(-1).t()
    torch.testing.assert_close(rowsum.cpu(), want_rows, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(total.cpu(), want_rows.sum(-1), rtol=1e-5, atol=1e-4)


def test_runtime_cuda_kernel_launches_raw_source():
    """newt/runtime/cuda.py `compile_cuda` + `Kernel.launch` by name (tests/test_runtime_smoke.py):
    NVRTC -> cubin -> driver launch on torch tensors, no compiler in between."""
    import ctypes

    from newt_b200.runtime.cuda import Kernel, compile_cuda

    src = 'extern "C" __global__ void scale_shift(float a, const float* x, const float* y, float* out, int n) {\n' \
          '  int i = blockIdx.x * blockDim.x + threadIdx.x;\n  if (i < n) out[i] = a * x[i] + y[i];\n}\n'
    cap = torch.cuda.get_device_capability()
    k = Kernel(compile_cuda(src, "scale_shift", f"sm_{cap[0]}{cap[1]}"), "scale_shift")
    n = (1 << 18) + 7
    x, y = _rand(n, 51), _rand(n, 52)
    xd, yd = x.cuda(), y.cuda()
    out = torch.empty_like(xd)
    k.launch(grid=((n + 255) // 256,), block=(256,),
             args=[ctypes.c_float(2.5), ctypes.c_void_p(xd.data_ptr()), ctypes.c_void_p(yd.data_ptr()),
                   ctypes.c_void_p(out.data_ptr()), ctypes.c_int32(n)],
             stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.cpu(), 2.5 * x + y, rtol=1e-6, atol=1e-6)


@dt.kernel(config={"BLOCK_TILE_M": 128, "BLOCK_TILE_N": 128, "BLOCK_TILE_K": 64, "num_stages": 4})
def dt_linear_relu(x, y, bias, out):
    for tile_m, tile_n in dt.tile([x.shape[0], y.shape[1]]):
        acc = dt.zeros([tile_m, tile_n], dtype=dt.float32)
        for tile_k in dt.tile(x.shape[1]):
            acc += x[tile_m, tile_k] @ y[tile_k, tile_n]
        out[tile_m, tile_n] = dt.relu(acc + bias[tile_n][None, :])


def test_deuteron_matmul_with_epilogue():
    """A tile loop whose accumulator goes through bias + relu before the store: the product
    runs on the tensor core, the epilogue as a generated kernel; checked against the kernel's
    own eager run and against fp64."""
    x, y = _rand((300, 200), 61, torch.float16, 0.5), _rand((200, 264), 62, torch.float16, 0.5)
    bias = _rand((264,), 63)
    out = torch.full((300, 264), float("nan"), device="cuda", dtype=torch.float16)
    dt_linear_relu(x.cuda(), y.cuda(), bias.cuda(), out)
    torch.cuda.synchronize()
    eager = torch.empty(300, 264, dtype=torch.float16)
    dt_linear_relu.ref(x, y, bias, eager)
    want = torch.relu(x.double() @ y.double() + bias.double())
    torch.testing.assert_close(out.cpu().double(), want, rtol=2 ** -10, atol=2e-3)
    torch.testing.assert_close(out.cpu().float(), eager.float(), rtol=2e-3, atol=2e-3)
