"""GPU: the hand-written sm_100a kernels, called through the C ABI, against
(a) vectors the reference produced and (b) the CPU oracle on seeded inputs.

Bars: bit-exact for fp32 add; rtol 1e-5 for fp32 softmax; relative Frobenius
error <= 1e-2 against an fp32 oracle for 16-bit layernorm / matmul / attention.
"""

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
