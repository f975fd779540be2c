"""nb200_gemm_tf32_static: the tf32 product for callers that have no workspace to pass.

Who they are: code that sits behind the reference's launcher, which gives a kernel only the
user's tensors and scalars and owns no device allocator, and plug-ins of a host process whose
memory pool already holds the whole GPU.  The entry point keeps the transposed copy of B in a
4 MiB array that is part of the library, so it may not allocate and it has a size limit.

Collected last on purpose (the file name sorts after every other test file): if it fails, a
run that stops at the first failure has already run everything else.  It needs nothing from
the other tests and leaves nothing behind for them."""

import ctypes

import pytest
import torch

from newt_b200.runtime import abi
from oracle import torch_ref

pytestmark = pytest.mark.gpu

LIMIT_FLOATS = 1 << 20   # n * round_up(k, 4) that the built-in scratch holds


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _static(a, b, c):
    m, k = a.shape
    n = b.shape[1]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return abi.load().nb200_gemm_tf32_static(_ptr(a), _ptr(b), _ptr(c), m, n, k, a.stride(0),
                                             b.stride(0), c.stride(0), None, stream)


def _with_workspace(a, b, c):
    m, k = a.shape
    n = b.shape[1]
    lib = abi.load()
    ws = torch.empty(lib.nb200_gemm_tf32_workspace_bytes(n, k), dtype=torch.uint8, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    abi.check(lib.nb200_gemm_tf32(_ptr(a), _ptr(b), _ptr(c), m, n, k, a.stride(0), b.stride(0),
                                  c.stride(0), None, _ptr(ws), ws.numel(), stream))


def test_static_scratch_matches_the_workspace_entry_point_twice_in_a_row():
    g = torch.Generator().manual_seed(77)
    # two calls in a row on one stream, the second with a smaller and ragged B so that it finds
    # the first call's leftovers in the scratch array
    for m, n, k in ((512, 1024, 1020), (300, 200, 100)):
        a = (torch.randn(m, k, generator=g) / k ** 0.5).cuda()
        b = torch.randn(k, n, generator=g).cuda()
        if k % 4:   # A's row pitch must be a multiple of 16 bytes for TMA
            a = torch.nn.functional.pad(a, (0, 4 - k % 4))[:, :k]
        got = torch.full((m, n), float("nan"), device="cuda")
        want = torch.full((m, n), float("nan"), device="cuda")
        abi.check(_static(a, b, got))
        _with_workspace(a, b, want)
        torch.cuda.synchronize()
        assert abi.read_status() == (0, 0)
        # the bar the other tf32 tests use, against the workspace entry point and against fp64
        assert torch_ref.rel_frobenius(got.cpu(), want.cpu()) <= 2e-3
        assert torch_ref.rel_frobenius(got.cpu(), a.double().cpu() @ b.double().cpu()) <= 2e-3


def _free_bytes():
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]     # cudaMemGetInfo: what the driver has left


def test_static_scratch_allocates_nothing():
    """The property in the entry point's name: device memory the driver has free, and what
    torch's allocator holds, are the same before and after calls (the first call on a device
    only looks up the address of the built-in array)."""
    g = torch.Generator().manual_seed(78)
    m, n, k = 256, 512, 768
    a = (torch.randn(m, k, generator=g) / k ** 0.5).cuda()
    b = torch.randn(k, n, generator=g).cuda()
    got = torch.empty(m, n, device="cuda")
    abi.check(_static(a, b, got))           # first call in a fresh process: address look-up
    free0, held0, reserved0 = _free_bytes(), torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(3):
        abi.check(_static(a, b, got))
    assert _free_bytes() == free0
    assert torch.cuda.memory_allocated() == held0 and torch.cuda.memory_reserved() == reserved0
    assert abi.read_status() == (0, 0)
    assert torch_ref.rel_frobenius(got.cpu(), a.double().cpu() @ b.double().cpu()) <= 2e-3


def test_static_scratch_with_a_misaligned_b():
    """B one element off a 16-byte boundary: the transposing pass reads it element by element."""
    g = torch.Generator().manual_seed(79)
    m, n, k = 128, 200, 96
    a = (torch.randn(m, k, generator=g) / k ** 0.5).cuda()
    flat = torch.randn(k * n + 1, generator=g).cuda()
    b = flat[1:].view(k, n)
    assert b.data_ptr() % 16 == 4
    got = torch.full((m, n), float("nan"), device="cuda")
    abi.check(_static(a, b, got))
    torch.cuda.synchronize()
    assert abi.read_status() == (0, 0)
    assert torch_ref.rel_frobenius(got.cpu(), a.double().cpu() @ b.double().cpu()) <= 2e-3


def test_static_scratch_limit_when_k_is_a_multiple_of_8192():
    """Such a k is stored with a pitch 32 floats longer, so n = 128 no longer fits, n = 127 does."""
    k = 8192
    a = torch.zeros(128, k, device="cuda")
    for n, fits in ((128, False), (127, True)):
        b = torch.zeros(k, n, device="cuda")
        c = torch.full((128, n), 7.0, device="cuda")
        rc = _static(a, b, c)
        torch.cuda.synchronize()
        if fits:
            abi.check(rc)
            assert torch.all(c == 0.0)
        else:
            assert rc == abi.E_UNSUPPORTED and torch.all(c == 7.0)


def test_static_scratch_refuses_what_does_not_fit():
    k, n = 1024, 1028                       # 1028 * 1024 floats: just over the limit
    assert n * k > LIMIT_FLOATS
    a = torch.zeros(128, k, device="cuda")
    b = torch.zeros(k, n, device="cuda")
    c = torch.full((128, n), 7.0, device="cuda")
    rc = _static(a, b, c)
    assert rc == abi.E_UNSUPPORTED and "1048576" in abi.last_error()
    torch.cuda.synchronize()
    assert torch.all(c == 7.0)              # refused before anything was launched
    # at the limit itself it runs
    b = torch.zeros(k, 1024, device="cuda")
    c = torch.full((128, 1024), 7.0, device="cuda")
    abi.check(_static(a, b, c))
    torch.cuda.synchronize()
    assert torch.all(c == 0.0)
