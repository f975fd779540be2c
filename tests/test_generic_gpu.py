"""Control flow and dots outside the tuned kernels, on the device: the programs of
tests/generic_programs.py run through the generic lowering and are compared with torch on the
CPU.  Integer results and pure data movement are bit-exact; the tolerances of the
floating-point cases are stated with each case (fold order differs from torch's; fp32 dot
operands are rounded to tf32, as on the tensor core)."""

import pytest
import torch

import generic_programs as gp

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


def test_ragged_matmul_took_the_generic_path_and_aligned_one_the_tensor_core():
    """The same program text: operands whose pitches bulk tensor copies cannot fetch run on the
    CUDA cores, aligned ones on the tcgen05 kernel."""
    from newt_b200.frontend.lower import GemmPlan

    kernel, grid, args, meta, checks = gp.build("ragged_matmul", "cuda")
    compiled = kernel.specialize(*args, **meta)
    assert isinstance(compiled.plan, GemmPlan)
    kernel[grid](*args, **meta)
    assert compiled.plan._generic_plan is not None

    m, n, k = 128, 128, 64
    g = torch.Generator().manual_seed(3)
    a = torch.randn(m, k, generator=g).half().cuda()
    b = torch.randn(k, n, generator=g).half().cuda()
    c = torch.zeros(m, n, device="cuda", dtype=torch.float16)
    kernel[(1, 1)](a, b, c, m, n, k, k, 1, n, 1, n, 1, BM=128, BN=128, BK=64)
    torch.testing.assert_close(c.float().cpu(), (a.float() @ b.float()).cpu(), rtol=2e-3, atol=2e-2)
