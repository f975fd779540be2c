"""CPU: the C oracle (oracle/newt_oracle.c) against vectors produced by the reference itself."""

import pytest
import torch

from oracle import cport, torch_ref


def test_add_bit_exact(golden):
    for n in golden.cases("add"):
        x, y = golden.get(f"add/{n}/x"), golden.get(f"add/{n}/y")
        assert torch.equal(cport.add_f32(x, y), golden.get(f"add/{n}/expected"))


def test_softmax_matches_reference_eager_and_torch(golden):
    for case in golden.cases("softmax"):
        x = golden.get(f"softmax/{case}/x")
        got = cport.softmax_f32(x)
        # rtol 1e-5 is the parity bar for fp32 softmax
        torch.testing.assert_close(got, golden.get(f"softmax/{case}/expected_eager"),
                                   rtol=1e-5, atol=1e-9)
        torch.testing.assert_close(got, golden.get(f"softmax/{case}/expected_torch"),
                                   rtol=1e-5, atol=1e-9)


def test_layernorm_f32_matches_reference(golden):
    for case in golden.cases("layernorm_f32"):
        p = f"layernorm_f32/{case}"
        got = cport.layernorm(golden.get(p + "/x"), golden.get(p + "/w"), golden.get(p + "/b"), 1e-5)
        # tolerances of the reference's own test (tests/test_softmax_layernorm.py:62)
        torch.testing.assert_close(got, golden.get(p + "/expected_eager"), rtol=1e-3, atol=1e-4)
        torch.testing.assert_close(got, golden.get(p + "/expected_torch"), rtol=1e-3, atol=1e-4)
        assert torch_ref.rel_frobenius(got, golden.get(p + "/expected_torch")) < 1e-5


@pytest.mark.parametrize("name", ["f16", "bf16"])
def test_layernorm_16bit_matches_fp32_oracle(golden, name):
    for case in golden.cases(f"layernorm_{name}"):
        p = f"layernorm_{name}/{case}"
        got = cport.layernorm(golden.get(p + "/x"), golden.get(p + "/w"), golden.get(p + "/b"), 1e-5)
        assert torch_ref.rel_frobenius(got.float(), golden.get(p + "/expected_f32")) <= 1e-2


@pytest.mark.parametrize("name", ["f16", "bf16"])
def test_matmul_matches_reference(golden, name):
    for case in golden.cases(f"matmul_{name}"):
        p = f"matmul_{name}/{case}"
        got = cport.matmul(golden.get(p + "/a"), golden.get(p + "/b"))
        assert torch_ref.rel_frobenius(got.float(), golden.get(p + "/expected_f32")) <= 1e-2
        tol = 1e-2 if name == "f16" else 2e-2  # tests/test_matmul.py:56,63
        torch.testing.assert_close(got.float(), golden.get(p + "/expected_eager").float(),
                                   rtol=tol, atol=tol)


def test_matmul_f32_follows_the_tf32_path(golden):
    p = "matmul_f32/128x128x128"
    a, b = golden.get(p + "/a"), golden.get(p + "/b")
    got = cport.matmul(a, b)
    # the reference's own bar for nl.dot on fp32 (tests/test_matmul.py:67-70)
    torch.testing.assert_close(got, golden.get(p + "/expected_f32"), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(got, golden.get(p + "/expected_eager"), rtol=1e-2, atol=1e-2)
    # operands rounded to 10 mantissa bits, products and sums in fp32
    def tf32(x):
        u = x.view(torch.int32)
        return ((u + 0x1000) & ~0x1fff).view(torch.float32)
    want = torch.zeros(128, 128)
    ar, br = tf32(a), tf32(b)
    for kk in range(128):
        want += ar[:, kk:kk + 1] * br[kk:kk + 1, :]
    assert torch.equal(got, want)
    assert 1e-5 < torch_ref.rel_frobenius(got, golden.get(p + "/expected_f32")) < 2e-3


def test_attention_matches_sdpa(golden):
    for case in golden.cases("attention"):
        p = f"attention/{case}"
        q, k, v = (golden.get(f"{p}/{n}") for n in "qkv")
        causal = case.startswith("causal")
        scale = 1.0 / (q.shape[-1] ** 0.5)
        for block_n in (64, 128):
            got = cport.attention(q, k, v, scale, causal=causal, block_n=block_n)
            assert torch_ref.rel_frobenius(got.float(), golden.get(p + "/expected_f32")) <= 1e-2


def test_edge_cases():
    assert cport.add_f32(torch.empty(0), torch.empty(0)).numel() == 0
    assert cport.softmax_f32(torch.empty(0, 16)).shape == (0, 16)
    one = cport.softmax_f32(torch.tensor([[3.0]]))
    assert one.item() == 1.0
    x = torch.full((2, 5), -1e30)
    torch.testing.assert_close(cport.softmax_f32(x), torch.full((2, 5), 0.2))
