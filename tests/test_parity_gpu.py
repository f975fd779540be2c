"""GPU: the hand-written sm_100a kernels, called through the C ABI, against
(a) vectors the reference produced and (b) the CPU oracle on seeded inputs.

Bars: bit-exact for fp32 add; rtol 1e-5 for fp32 softmax; relative Frobenius
error <= 1e-2 against an fp32 oracle for 16-bit layernorm / matmul / attention.
"""

import ctypes

import pytest
import torch

from newt_b200.runtime import abi, kernels
from oracle import cport, torch_ref

pytestmark = pytest.mark.gpu


def _dev(t):
    return t.cuda()


# ---- K0 ---------------------------------------------------------------------

def test_add_golden_bit_exact(golden):
    for n in golden.cases("add"):
        x, y = _dev(golden.get(f"add/{n}/x")), _dev(golden.get(f"add/{n}/y"))
        out = torch.empty_like(x)
        kernels.add_f32(x, y, out, x.numel())
        assert torch.equal(out.cpu(), golden.get(f"add/{n}/expected"))


@pytest.mark.parametrize("n", [0, 1, 3, 4, 1023, 1 << 20, (1 << 24) + 5])
def test_add_sizes_and_misalignment(n):
    g = torch.Generator().manual_seed(n)
    x, y = torch.randn(n + 1, generator=g), torch.randn(n + 1, generator=g)
    xd, yd = _dev(x), _dev(y)
    out = torch.full((n + 1,), 7.0, device="cuda")
    kernels.add_f32(xd[:n], yd[:n], out[:n], n)           # aligned
    assert torch.equal(out[:n].cpu(), x[:n] + y[:n]) and out[n].item() == 7.0
    out.fill_(7.0)
    kernels.add_f32(xd[1:], yd[1:], out[1:], n)           # 4-byte aligned only
    assert torch.equal(out[1:].cpu(), x[1:] + y[1:]) and out[0].item() == 7.0


# ---- K1 ---------------------------------------------------------------------

def _softmax(x):
    out = torch.empty_like(x)
    kernels.softmax_f32(x, out, x.shape[0], x.shape[1], x.stride(0), out.stride(0))
    return out


def test_softmax_golden(golden):
    for case in golden.cases("softmax"):
        x = golden.get(f"softmax/{case}/x")
        got = _softmax(_dev(x)).cpu()
        torch.testing.assert_close(got, golden.get(f"softmax/{case}/expected_eager"),
                                   rtol=1e-5, atol=1e-9)
        torch.testing.assert_close(got, golden.get(f"softmax/{case}/expected_torch"),
                                   rtol=1e-5, atol=1e-9)


@pytest.mark.parametrize("m,n", [(1, 1), (3, 7), (8, 128), (128, 1024), (32, 781), (5, 2500),
                                 (64, 4096), (7, 8191), (3, 16384), (2, 32768), (4096, 4096)])
def test_softmax_vs_oracle(m, n):
    g = torch.Generator().manual_seed(1000 + n)
    x = torch.randn(m, n, generator=g)
    got = _softmax(_dev(x)).cpu()
    rows = slice(0, min(m, 64))  # the C oracle is single-threaded; torch covers all rows
    torch.testing.assert_close(got[rows], cport.softmax_f32(x[rows].contiguous()),
                               rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(got, torch_ref.softmax(x), rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(got.sum(-1), torch.ones(m), rtol=1e-5, atol=0)


def test_softmax_strided_rows_and_unaligned_base():
    g = torch.Generator().manual_seed(7)
    big = torch.randn(9, 1001, generator=g)
    xd = _dev(big)
    x = xd[:, 1:782]                      # row stride 1001, base off by 4 bytes
    out_big = torch.zeros_like(xd)
    out = out_big[:, 1:782]
    kernels.softmax_f32(x, out, 9, 781, x.stride(0), out.stride(0))
    torch.testing.assert_close(out.cpu(), torch_ref.softmax(big[:, 1:782]), rtol=1e-5, atol=1e-9)
    assert out_big[:, 0].abs().sum().item() == 0 and out_big[:, 782:].abs().sum().item() == 0


def test_softmax_empty_and_too_wide():
    x = torch.empty(0, 16, device="cuda")
    kernels.softmax_f32(x, x, 0, 16, 16, 16)
    x = torch.empty(1, 40000, device="cuda")
    with pytest.raises(abi.UnsupportedError):
        kernels.softmax_f32(x, x, 1, 40000, 40000, 40000)


# ---- K2 ---------------------------------------------------------------------

def _layernorm(x, w, b, eps=1e-5):
    out = torch.empty_like(x)
    kernels.layernorm(x, w, b, out, x.shape[0], x.shape[1], x.stride(0), out.stride(0), eps)
    return out


def test_layernorm_golden(golden):
    for case in golden.cases("layernorm_f32"):
        p = f"layernorm_f32/{case}"
        got = _layernorm(*(_dev(golden.get(f"{p}/{k}")) for k in "xwb")).cpu()
        torch.testing.assert_close(got, golden.get(p + "/expected_eager"), rtol=1e-3, atol=1e-4)
        torch.testing.assert_close(got, golden.get(p + "/expected_torch"), rtol=1e-3, atol=1e-4)
    for name in ("f16", "bf16"):
        for case in golden.cases(f"layernorm_{name}"):
            p = f"layernorm_{name}/{case}"
            got = _layernorm(*(_dev(golden.get(f"{p}/{k}")) for k in "xwb")).cpu()
            assert torch_ref.rel_frobenius(got.float(), golden.get(p + "/expected_f32")) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n", [(1, 1), (8, 128), (64, 2048), (16, 300), (33, 4096), (5, 8200),
                                 (2, 16384)])
def test_layernorm_vs_oracle(dtype, m, n):
    g = torch.Generator().manual_seed(2000 + n)
    x = torch.randn(m, n, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(n, generator=g)).to(dtype)
    b = (0.1 * torch.randn(n, generator=g)).to(dtype)
    got = _layernorm(_dev(x), _dev(w), _dev(b)).cpu()
    want_c = cport.layernorm(x, w, b, 1e-5)
    if dtype == torch.float32:
        torch.testing.assert_close(got, want_c, rtol=1e-4, atol=1e-5)
    else:
        # same fp32 arithmetic, one rounding: at most one 16-bit ulp apart
        assert torch_ref.rel_frobenius(got.float(), want_c.float()) <= 4e-3
    if n > 1:
        assert torch_ref.rel_frobenius(got.float(), torch_ref.layernorm(x, w, b)) <= 1e-2


def test_layernorm_config2_shape_fp16():
    g = torch.Generator().manual_seed(2)
    m, n = 8192, 4096
    x = torch.randn(m, n, generator=g).half()
    w = (1 + 0.1 * torch.randn(n, generator=g)).half()
    b = (0.1 * torch.randn(n, generator=g)).half()
    got = _layernorm(_dev(x), _dev(w), _dev(b)).cpu()
    assert torch_ref.rel_frobenius(got.float(), torch_ref.layernorm(x, w, b)) <= 1e-2


# ---- K3 / K4 ------------------------------------------------------------------

def _gemm(a, b, block_n=0, stages=0):
    m, k = a.shape
    n = b.shape[1]
    c = torch.full((m, n), float("nan"), device="cuda", dtype=a.dtype)
    run = kernels.gemm_tf32 if a.dtype == torch.float32 else kernels.gemm
    run(a, b, c, m, n, k, a.stride(0), b.stride(0), c.stride(0),
        kernels.gemm_config(block_n=block_n, stages=stages))
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    return c


def test_gemm_golden(golden):
    for name in ("f16", "bf16"):
        for case in golden.cases(f"matmul_{name}"):
            p = f"matmul_{name}/{case}"
            a, b = golden.get(p + "/a"), golden.get(p + "/b")
            m, k = a.shape
            n = b.shape[1]
            # TMA wants row pitches that are multiples of 8 elements: pad the pitch, not the data
            kp, np_ = -(-k // 8) * 8, -(-n // 8) * 8
            ad = torch.zeros(m, kp, device="cuda", dtype=a.dtype)[:, :k]
            bd = torch.zeros(k, np_, device="cuda", dtype=a.dtype)[:, :n]
            ad.copy_(a)
            bd.copy_(b)
            got = _gemm(ad, bd).cpu()
            assert torch_ref.rel_frobenius(got.float(), golden.get(p + "/expected_f32")) <= 1e-2
            tol = 1e-2 if name == "f16" else 2e-2
            torch.testing.assert_close(got.float(), golden.get(p + "/expected_eager").float(),
                                       rtol=tol, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block_n", [64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(1, 8, 8), (128, 64, 64), (130, 72, 200), (257, 520, 136),
                                   (1024, 1024, 1024)])
def test_gemm_vs_oracle(dtype, block_n, m, n, k):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype)
    b = torch.randn(k, n, generator=g).to(dtype)
    got = _gemm(a.cuda(), b.cuda(), block_n).cpu()
    assert torch_ref.rel_frobenius(got.float(), torch_ref.matmul(a, b)) <= 1e-2
    if m * n * k <= 130 * 72 * 200:
        want = cport.matmul(a, b)
        assert torch_ref.rel_frobenius(got.float(), want.float()) <= 4e-3


def test_gemm_f32_golden_runs_as_tf32(golden):
    p = "matmul_f32/128x128x128"
    a, b = golden.get(p + "/a"), golden.get(p + "/b")
    got = _gemm(a.cuda(), b.cuda()).cpu()
    # the reference's bar for nl.dot on fp32 blocks (tests/test_matmul.py:67-70)
    torch.testing.assert_close(got, golden.get(p + "/expected_f32"), rtol=1e-2, atol=1e-2)
    assert torch_ref.rel_frobenius(got, cport.matmul(a, b)) <= 2e-3


@pytest.mark.parametrize("config", [dict(block_n=64), dict(block_n=128), dict(block_n=256, stages=2),
                                    dict(block_m=256, block_n=256),
                                    dict(block_m=256, block_n=256, block_k=32, stages=5),
                                    dict(block_m=256, block_n=256, block_k=96)])
@pytest.mark.parametrize("m,n,k", [(1, 4, 4), (128, 64, 32), (130, 72, 200), (257, 520, 132),
                                   (1024, 1024, 1024)])
def test_gemm_tf32_vs_oracle(config, m, n, k):
    g = torch.Generator().manual_seed(m * 5 + n * 3 + k)
    a = torch.randn(m, k, generator=g) / k ** 0.5
    b = torch.randn(k, n, generator=g)
    c = torch.full((m, n), float("nan"), device="cuda")
    kernels.gemm_tf32(a.cuda(), b.cuda(), c, m, n, k, k, n, n, kernels.gemm_config(**config))
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    got = c.cpu()
    ref = a.double() @ b.double()
    assert torch_ref.rel_frobenius(got, ref) <= 2e-3
    if m * n * k <= 130 * 72 * 200:
        assert torch_ref.rel_frobenius(got, cport.matmul(a, b)) <= 2e-3
    # exact where tf32 is exact: small integers
    ai = torch.randint(-8, 9, (m, k), generator=g).float()
    bi = torch.randint(-8, 9, (k, n), generator=g).float()
    kernels.gemm_tf32(ai.cuda(), bi.cuda(), c, m, n, k, k, n, n, kernels.gemm_config(**config))
    torch.cuda.synchronize()
    assert torch.equal(c.cpu(), ai @ bi)


def test_gemm_tf32_rules():
    a = torch.zeros(64, 102, device="cuda")   # pitch 408 B: not a multiple of 16
    b = torch.zeros(102, 66, device="cuda")   # B goes through the transposing pass: any pitch
    c = torch.zeros(64, 64, device="cuda")
    assert "multiple of 4" in kernels.gemm_check(a, b, c, 64, 64, 102, 102, 66, 64)
    assert kernels.gemm_check(a, b, c, 64, 64, 100, 104, 66, 64) is None
    with pytest.raises(abi.UnsupportedError, match="multiple of 4"):
        kernels.gemm(a, b, c, 64, 64, 100, 104, 66, 64)      # B's pitch of 264 bytes: not in place


@pytest.mark.parametrize("config", [dict(block_n=64), dict(block_n=128, block_k=64), dict(block_n=256),
                                    dict(block_m=256, block_n=256),
                                    dict(block_m=256, block_n=256, block_k=32, stages=5)])
@pytest.mark.parametrize("m,n,k", [(128, 64, 32), (130, 72, 200), (257, 520, 132), (1024, 1024, 1024)])
def test_gemm_tf32_reads_b_in_place(config, m, n, k):
    """fp32 B as [K, N] with a 16-byte pitch is an MN-major tf32 operand (the swizzle on 32-byte
    atoms): same result, bit for bit, as through the transposing pass, whose K-major product
    sums the same terms in the same order."""
    g = torch.Generator().manual_seed(m * 3 + n * 5 + k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).cuda()
    b = torch.randn(k, n, generator=g).cuda()
    c = torch.full((m, n), float("nan"), device="cuda")
    kernels.gemm(a, b, c, m, n, k, k, n, n, kernels.gemm_config(**config))      # in place
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    assert torch_ref.rel_frobenius(c.cpu(), a.cpu().double() @ b.cpu().double()) <= 2e-3
    via = torch.full((m, n), float("nan"), device="cuda")
    abi.set_tuning("tf32_in_place", 0)
    try:
        ws = torch.empty(int(abi.load().nb200_gemm_tf32_workspace_bytes(n, k)), dtype=torch.uint8,
                         device="cuda")
        abi.check(abi.load().nb200_gemm_tf32(
            ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
            ctypes.c_void_p(via.data_ptr()), m, n, k, k, n, n,
            ctypes.byref(kernels.gemm_config(**config)), ctypes.c_void_p(ws.data_ptr()), ws.numel(),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
    finally:
        abi.set_tuning("tf32_in_place", 1)
    assert torch.equal(c, via)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("config", [dict(block_n=64), dict(block_n=256), dict(block_m=256, block_n=256)])
@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (130, 72, 200), (700, 1000, 328)])
def test_gemm_bt_vs_oracle(dtype, config, m, n, k):
    # B handed over transposed ([N, K]); the pitch of B^T is padded to what TMA needs
    g = torch.Generator().manual_seed(m + n * 3 + k * 7)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype)
    b = torch.randn(k, n, generator=g).to(dtype)
    bt = torch.zeros(n, k + 8, dtype=dtype)[:, :k]
    bt.copy_(b.t())
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    btd = bt.cuda() if bt.is_contiguous() else torch.zeros(n, k + 8, dtype=dtype, device="cuda")[:, :k].copy_(bt)
    kernels.gemm_bt(a.cuda(), btd, c, m, n, k, k, btd.stride(0), n, kernels.gemm_config(**config))
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    assert torch_ref.rel_frobenius(c.cpu().float(), a.double() @ b.double()) <= tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("block_k,stages", [(64, 4), (64, 7), (128, 3), (192, 2)])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (130, 72, 200), (700, 1000, 328),
                                   (2048, 2048, 2048)])
def test_gemm_cta_pair_vs_oracle(dtype, block_k, stages, m, n, k):
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k + 1)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype).cuda()
    b = torch.randn(k, n, generator=g).to(dtype).cuda()
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    kernels.gemm(a, b, c, m, n, k, k, n, n,
                 kernels.gemm_config(block_m=256, block_n=256, block_k=block_k, stages=stages,
                                     cta_pair=1))
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    assert torch_ref.rel_frobenius(c.cpu().float(), torch_ref.matmul(a.cpu(), b.cpu())) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block_n", [64, 128])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("m,n,k", [(128, 64, 64), (128, 128, 128), (130, 72, 200), (300, 192, 320),
                                   (700, 1000, 328), (1024, 1024, 1024)])
def test_gemm_two_slab_slots_vs_oracle(dtype, block_n, transposed, m, n, k):
    """Ring slots of two K slabs (one copy per operand and slot where the shapes allow the wide
    tensor maps, slab by slab at ragged K or N), B as [K, N] and as [N, K]."""
    g = torch.Generator().manual_seed(m * 11 + n * 3 + k + block_n)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype)
    b = torch.randn(k, n, generator=g).to(dtype)
    kp = (k + 7) // 8 * 8
    ad = torch.zeros(m, kp, dtype=dtype, device="cuda")[:, :k].copy_(a)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    row_k = 32 if dtype == torch.float32 else 64
    cfg = kernels.gemm_config(block_n=block_n, block_k=2 * row_k)
    if transposed:
        bd = torch.zeros(n, kp, dtype=dtype, device="cuda")[:, :k].copy_(b.t())
        kernels.gemm_bt(ad, bd, c, m, n, k, kp, kp, n, cfg)
    else:
        np_ = (n + 7) // 8 * 8
        bd = torch.zeros(k, np_, dtype=dtype, device="cuda")[:, :n].copy_(b)
        kernels.gemm(ad, bd, c, m, n, k, kp, np_, n, cfg)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    got = c.cpu().double()
    assert not torch.isnan(got).any()
    assert torch_ref.rel_frobenius(got, a.double() @ b.double()) <= tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block_k", [1, 2])            # in 128-byte rows of K
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 512, 64), (130, 72, 200), (700, 1000, 328), (512, 1024, 512),
                                   (2048, 2048, 1024)])
def test_gemm_wide_pair_vs_oracle(dtype, block_k, transposed, m, n, k):
    """256 x 512 tiles per CTA pair: two 256-column MMAs per K step on one accumulator that
    takes all of tensor memory; ragged edges in all three extents, B either way round."""
    g = torch.Generator().manual_seed(m * 13 + n * 3 + k + block_k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype)
    b = torch.randn(k, n, generator=g).to(dtype)
    kp, np_ = (k + 7) // 8 * 8, (n + 7) // 8 * 8
    ad = torch.zeros(m, kp, dtype=dtype, device="cuda")[:, :k].copy_(a)
    c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
    row_k = 32 if dtype == torch.float32 else 64
    cfg = kernels.gemm_config(block_m=256, block_n=512, block_k=block_k * row_k, cta_pair=1)
    if transposed:
        bd = torch.zeros(n, kp, dtype=dtype, device="cuda")[:, :k].copy_(b.t())
        kernels.gemm_bt(ad, bd, c, m, n, k, kp, kp, n, cfg)
    else:
        bd = torch.zeros(k, np_, dtype=dtype, device="cuda")[:, :n].copy_(b)
        kernels.gemm(ad, bd, c, m, n, k, kp, np_, n, cfg)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    got = c.cpu().double()
    assert not torch.isnan(got).any()
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    assert torch_ref.rel_frobenius(got, a.double() @ b.double()) <= tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block_n,block_k", [(256, 1), (256, 2), (512, 1), (512, 2)])   # block_k in 128-byte rows
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 512, 40960), (700, 1000, 4104), (1024, 1024, 2048), (2560, 2304, 2048)])
def test_gemm_split_tail_vs_oracle(dtype, block_n, block_k, transposed, m, n, k):
    """The last round of tiles cut along K and summed through the workspace: one tile over all
    pairs, ragged extents, a round of whole tiles before the split ones, both tile widths, B
    either way round; the same call twice gives the same bits."""
    g = torch.Generator().manual_seed(m * 7 + n * 5 + k + block_n + block_k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype)
    b = torch.randn(k, n, generator=g).to(dtype)
    np_ = (n + 7) // 8 * 8
    row_k = 32 if dtype == torch.float32 else 64
    cfg = kernels.gemm_config(block_m=256, block_n=block_n, block_k=block_k * row_k, cta_pair=1)
    ad = a.cuda()
    bd = b.t().contiguous().cuda() if transposed else torch.zeros(k, np_, dtype=dtype, device="cuda")[:, :n].copy_(b)
    ldb = k if transposed else np_
    abi.set_tuning("gemm_split_tail", 1)
    try:
        need = kernels.gemm_split_bytes(m, n, k, dtype, cfg)
        if need == 0:
            pytest.skip("every pair would get fewer than four k steps")
        outs = []
        for _ in range(2):
            c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
            kernels.gemm_split(ad, bd, c, m, n, k, k, ldb, n, cfg, transposed, need)
            torch.cuda.synchronize()
            assert abi.read_status() == (0, 0)
            outs.append(c)
    finally:
        abi.set_tuning("gemm_split_tail", 0)
    assert torch.equal(outs[0], outs[1])
    got = outs[0].cpu().double()
    assert not torch.isnan(got).any()
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    assert torch_ref.rel_frobenius(got, a.double() @ b.double()) <= tol


def test_gemm_split_tail_rule_and_small_workspace():
    """Square problems keep their tiles whole, a small C with a long K is split; a workspace that
    is too small means the unsplit product, not an error."""
    wide = kernels.gemm_config(block_m=256, block_n=512, block_k=64, cta_pair=1)
    assert kernels.gemm_split_bytes(4096, 4096, 4096, torch.bfloat16, wide) == 0   # 128 tiles: a round of 54
    assert kernels.gemm_split_bytes(4096, 4096, 4096, torch.bfloat16) > 0   # left to the library: 256 x 256, 34 tiles in halves
    assert kernels.gemm_split_bytes(8192, 8192, 8192, torch.bfloat16) == 0
    assert kernels.gemm_split_bytes(1024, 1024, 1024, torch.float16) == 0
    cfg = kernels.gemm_config(block_m=256, block_n=256, block_k=64, cta_pair=1)
    m, n, k = 1024, 1024, 16384
    need = kernels.gemm_split_bytes(m, n, k, torch.bfloat16, cfg)
    assert need > 0
    g = torch.Generator(device="cuda").manual_seed(11)
    a = (torch.randn(m, k, device="cuda", generator=g) / k ** 0.5).bfloat16()
    b = torch.randn(k, n, device="cuda", generator=g).bfloat16()
    whole, split, starved = (torch.empty(m, n, device="cuda", dtype=torch.bfloat16) for _ in range(3))
    kernels.gemm(a, b, whole, m, n, k, k, n, n, cfg)
    kernels.gemm_split(a, b, split, m, n, k, k, n, n, cfg)
    assert kernels.gemm_split_bytes(m, n, k, torch.bfloat16) == need   # no config: the same tile
    by_default = torch.empty_like(split)
    kernels.gemm_split(a, b, by_default, m, n, k, k, n, n)
    ws = torch.empty(4096, dtype=torch.uint8, device="cuda")
    abi.check(abi.load().nb200_gemm_split(a.data_ptr(), b.data_ptr(), starved.data_ptr(), m, n, k, k, n, n,
                                          abi.dtype_code(a.dtype), 0, ctypes.byref(cfg), ws.data_ptr(),
                                          ws.numel(), kernels.raw_stream()))
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    assert torch.equal(starved, whole)
    assert torch.equal(by_default, split)
    ref = a.float() @ b.float()
    assert torch_ref.rel_frobenius(split.float().cpu(), ref.cpu()) <= 1e-2
    assert (split.float() - whole.float()).abs().max().item() <= 0.05


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("block_k", [1, 2])            # in 128-byte rows of K
@pytest.mark.parametrize("m,n,k", [(512, 1024, 64), (512, 1024, 192), (700, 1000, 328), (1024, 2048, 4096)])
def test_gemm_wide_pair_half_by_half_rings(dtype, block_k, m, n, k):
    """256 x 512 tiles issue the last ring of k steps -- and, with a long K, the first -- one
    256-column half at a time: the same MMAs per accumulator column in the same order, so the
    bits do not depend on the knob; K shorter than a ring, a ring and a half, ragged, long."""
    g = torch.Generator().manual_seed(m + n + k + block_k)
    a = (torch.randn(m, k, generator=g) / k ** 0.5).to(dtype).cuda()
    np_ = (n + 7) // 8 * 8
    b = torch.zeros(k, np_, dtype=dtype, device="cuda")[:, :n].copy_(torch.randn(k, n, generator=g).to(dtype))
    row_k = 32 if dtype == torch.float32 else 64
    cfg = kernels.gemm_config(block_m=256, block_n=512, block_k=block_k * row_k, cta_pair=1)
    outs = []
    try:
        for knob in (-1, 1, 2, 0):
            abi.set_tuning("gemm_half_tail", knob)
            c = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
            kernels.gemm(a, b, c, m, n, k, k, np_, n, cfg)
            torch.cuda.synchronize()
            assert abi.read_status() == (0, 0)
            outs.append(c)
    finally:
        abi.set_tuning("gemm_half_tail", 0)
    for c in outs[1:]:
        assert torch.equal(c, outs[0])
    tol = 2e-3 if dtype == torch.float32 else 1e-2
    assert torch_ref.rel_frobenius(outs[0].cpu().double(), a.cpu().double() @ b[:, :n].cpu().double()) <= tol


def test_gemm_linearity_at_full_size():
    # size-independent property at the benchmark size: (A1 + A2) @ B == A1 @ B + A2 @ B
    # up to rounding, and a spot-checked block against the fp32 oracle
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    a1 = (torch.randn(n, n, device="cuda", generator=g) / n ** 0.5).half()
    a2 = (torch.randn(n, n, device="cuda", generator=g) / n ** 0.5).half()
    b = torch.randn(n, n, device="cuda", generator=g).half()
    c1, c2, c12 = _gemm(a1, b), _gemm(a2, b), _gemm((a1.float() + a2.float()).half(), b)
    err = ((c1.float() + c2.float() - c12.float()).norm() / c12.float().norm()).item()
    assert err <= 2e-3
    rows = slice(4096 - 64, 4096 + 64)
    ref = a1[rows].float().cpu() @ b.float().cpu()
    assert torch_ref.rel_frobenius(c1[rows].cpu().float(), ref) <= 1e-2


def test_gemm_empty_and_k_zero():
    a = torch.zeros(0, 64, device="cuda", dtype=torch.float16)
    b = torch.zeros(64, 64, device="cuda", dtype=torch.float16)
    _gemm(a, b)
    a = torch.zeros(16, 0, device="cuda", dtype=torch.float16)
    b = torch.zeros(0, 16, device="cuda", dtype=torch.float16)
    c = torch.ones(16, 16, device="cuda", dtype=torch.float16)
    kernels.gemm(a, b, c, 16, 16, 0, 8, 16, 16)
    assert c.abs().sum().item() == 0


def test_gemm_check_rejects_without_launching():
    a = torch.zeros(64, 100, device="cuda", dtype=torch.float16)
    b = torch.zeros(100, 64, device="cuda", dtype=torch.float16)
    c = torch.zeros(64, 64, device="cuda", dtype=torch.float16)
    assert "multiple of 8" in kernels.gemm_check(a, b, c, 64, 64, 100, 100, 64, 64)
    assert kernels.gemm_check(a, b, c, 64, 64, 96, 104, 64, 64) is None
    af = torch.zeros(64, 66, device="cuda")          # an fp32 pitch of 264 bytes
    with pytest.raises(abi.UnsupportedError, match="multiple of 4"):
        kernels.gemm(af, af, af, 64, 64, 64, 66, 66, 66)


# ---- K5 -------------------------------------------------------------------------

def _attention(q, k, v, causal, scale=None):
    o = torch.full(q.shape, float("nan"), device="cuda", dtype=q.dtype)
    kernels.attention_fwd(q, k, v, o, scale or 1.0 / q.shape[-1] ** 0.5, causal)
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    return o


def test_attention_golden(golden):
    for case in golden.cases("attention"):
        p = f"attention/{case}"
        q, k, v = (golden.get(f"{p}/{n}") for n in "qkv")
        got = _attention(q.cuda(), k.cuda(), v.cuda(), case.startswith("causal")).cpu()
        assert torch_ref.rel_frobenius(got.float(), golden.get(p + "/expected_f32")) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,sq,skv,d", [(1, 1, 1, 64), (2, 128, 128, 128), (3, 200, 333, 128),
                                         (2, 333, 333, 64), (1, 100, 700, 128), (2, 513, 129, 64)])
def test_attention_vs_oracle(dtype, causal, bh, sq, skv, d):
    g = torch.Generator().manual_seed(bh + sq * 3 + skv * 5 + d)
    q, k, v = (torch.randn(bh, s, d, generator=g).to(dtype) for s in (sq, skv, skv))
    got = _attention(q.cuda(), k.cuda(), v.cuda(), causal).cpu()
    scale = 1.0 / d ** 0.5
    # the C oracle follows the reference's loop literally (P rounded to the input type)
    want = cport.attention(q, k, v, scale, causal=causal, block_n=128)
    assert torch_ref.rel_frobenius(got.float(), want.float()) <= (4e-3 if dtype == torch.float16
                                                                    else 1.6e-2)
    if not (causal and sq > skv):   # SDPA leaves rows with no visible key undefined
        assert torch_ref.rel_frobenius(got.float(), torch_ref.attention(q, k, v, scale, causal)) <= 1e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("step", [3.0, 12.0, 40.0])
def test_attention_rising_and_falling_scores(dtype, step):
    # The row maximum climbs by `step` (natural-log units) per 128-key block and then falls
    # again: small steps stay below every threshold, medium ones move the reference between
    # blocks, large ones force a block to be exponentiated again with a new reference.
    bh, s, d = 2, 1024, 128
    g = torch.Generator().manual_seed(int(step))
    q = torch.randn(bh, s, d, generator=g)
    k = torch.randn(bh, s, d, generator=g) * 0.05
    v = torch.randn(bh, s, d, generator=g)
    q[..., 0] = 1.0
    block = torch.arange(s) // 128
    level = torch.minimum(block, 7 - block).float() * step     # 0, 1, 2, 3, 3, 2, 1, 0 steps
    k[..., 0] = level * d ** 0.5                               # score offset = level after scaling
    q, k, v = (t.to(dtype) for t in (q, k, v))
    for causal in (False, True):
        got = _attention(q.cuda(), k.cuda(), v.cuda(), causal).cpu()
        want = torch_ref.attention(q, k, v, 1.0 / d ** 0.5, causal)
        assert torch.isfinite(got.float()).all()
        assert torch_ref.rel_frobenius(got.float(), want) <= 1e-2


def test_attention_strided_heads_and_rows():
    # q, k, v as slices of one packed [bh, s, 3 * d] projection output
    bh, s, d = 4, 384, 128
    g = torch.Generator().manual_seed(11)
    qkv = torch.randn(bh, s, 3 * d, generator=g).half()
    dev = qkv.cuda()
    q, k, v = dev[..., :d], dev[..., d:2 * d], dev[..., 2 * d:]
    got = _attention(q, k, v, True).cpu()
    ref = torch_ref.attention(qkv[..., :d], qkv[..., d:2 * d], qkv[..., 2 * d:], 1 / d ** 0.5, True)
    assert torch_ref.rel_frobenius(got.float(), ref) <= 1e-2


def test_attention_rows_sum_property_at_config_size():
    # with V = ones every output element is exactly sum(p)/l = 1 up to rounding, at any size
    bh, s, d = 8, 4096, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(bh, s, d, device="cuda", generator=g).half()
    k = torch.randn(bh, s, d, device="cuda", generator=g).half()
    v = torch.ones(bh, s, d, device="cuda", dtype=torch.float16)
    o = _attention(q, k, v, True)
    assert (o.float() - 1.0).abs().max().item() <= 2e-3
    # and one head against the fp32 oracle
    v = torch.randn(bh, s, d, device="cuda", generator=g).half()
    o = _attention(q, k, v, True)
    ref = torch_ref.attention(q[:1].cpu(), k[:1].cpu(), v[:1].cpu(), 1 / d ** 0.5, True)
    assert torch_ref.rel_frobenius(o[:1].cpu().float(), ref) <= 1e-2
    # and the last head: its tiles are the second and third ones a persistent CTA works on
    ref = torch_ref.attention(q[-1:].cpu(), k[-1:].cpu(), v[-1:].cpu(), 1 / d ** 0.5, True)
    assert torch_ref.rel_frobenius(o[-1:].cpu().float(), ref) <= 1e-2


@pytest.mark.parametrize("causal", [False, True])
def test_attention_many_short_tiles(causal):
    # 600 Q tiles of one to three KV blocks: every CTA walks several tiles, with tiles of one
    # block (only one softmax group has work) and tile boundaries at every ring position
    bh, sq, skv, d = 200, 384, 300, 64
    g = torch.Generator().manual_seed(23)
    q, k, v = (torch.randn(bh, s, d, generator=g).half() for s in (sq, skv, skv))
    got = _attention(q.cuda(), k.cuda(), v.cuda(), causal).cpu()
    want = torch_ref.attention(q, k, v, 1.0 / d ** 0.5, causal)
    if causal:   # rows past the last key see every key
        want[:, skv:] = torch_ref.attention(q[:, skv:], k, v, 1.0 / d ** 0.5, False)
    assert torch_ref.rel_frobenius(got.float(), want) <= 1e-2


def test_attention_argument_errors():
    q = torch.zeros(1, 16, 96, device="cuda", dtype=torch.float16)
    with pytest.raises(abi.UnsupportedError, match="head_dim"):
        kernels.attention_fwd(q, q, q, q, 0.1, False)
    q = torch.zeros(1, 16, 64, device="cuda", dtype=torch.float32)
    with pytest.raises(abi.UnsupportedError, match="fp16 and bf16"):
        kernels.attention_fwd(q, q, q, q, 0.1, False)
    q = torch.zeros(1, 16, 64, device="cuda", dtype=torch.float16)
    e = torch.zeros(1, 0, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(abi.KernelLibraryError, match="empty key"):
        kernels.attention_fwd(q, e, e, q, 0.1, False)
    kernels.attention_fwd(e, q, q, e, 0.1, False)   # no queries: nothing to do


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("bh,sq,skv,d", [(160, 640, 640, 128), (3, 255, 1000, 128), (5, 129, 257, 64)])
def test_attention_odd_tile_counts(causal, bh, sq, skv, d):
    # An odd number of 128-row Q tiles per head (the last pair of a head has one tile only),
    # fewer than 256 query rows, and several pairs per persistent CTA (160 heads x 3 pairs).
    g = torch.Generator().manual_seed(bh + sq + skv)
    q, k, v = (torch.randn(bh, s, d, generator=g).half() for s in (sq, skv, skv))
    got = _attention(q.cuda(), k.cuda(), v.cuda(), causal).cpu()
    want = torch_ref.attention(q, k, v, 1.0 / d ** 0.5, causal)
    assert torch_ref.rel_frobenius(got.float(), want) <= 1e-2


# ---- bounded waits ----------------------------------------------------------------

def test_a_wait_that_runs_out_is_reported_and_the_device_stays_usable():
    """A kernel waits on a barrier nothing signals, with the limit turned down to 200 us: it
    returns by itself, the status word says so once, and the next launch is fine."""
    import ctypes

    lib = abi.load()
    abi.read_status()                       # start clean
    abi.set_tuning("wait_limit_us", 200)
    try:
        abi.check(lib.nb200_selftest_wait_timeout(0xabc, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
        with pytest.raises(abi.KernelLibraryError) as e:
            abi.read_status()
        assert e.value.code == abi.E_DEVICE and "code 6" in str(e.value) and "0xabc" in str(e.value)
    finally:
        abi.set_tuning("wait_limit_us", 0)  # back to the default
    assert abi.read_status() == (0, 0)      # reported once, then clear
    x = torch.randn(64, 1000, device="cuda")
    out = torch.empty_like(x)
    kernels.softmax_f32(x, out, 64, 1000, x.stride(0), out.stride(0))
    torch.testing.assert_close(out, torch.softmax(x, dim=-1), rtol=1e-5, atol=1e-8)
    assert abi.read_status() == (0, 0)
