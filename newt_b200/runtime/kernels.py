"""Tensor-level launchers over the C ABI: torch CUDA tensors in, kernel launch on
torch's current stream.  These are what the lowering plans of the JIT front end
call; they add nothing to the arithmetic.  Like the reference launcher
(newt/runtime/jit.py:190-223) they refuse tensors that are not on the current
CUDA device.  Some need scratch memory beside the caller's tensors (the transposed copy of an
fp32 B, a re-pitched copy of an operand bulk tensor copies cannot fetch, the partial sums of
tiles that were cut along K): they take it
from torch's caching allocator per launch, on the current stream, so launches on different
streams never share a buffer; the others never allocate.
"""

import ctypes
import threading

import torch

from . import abi


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_trust = threading.local()     # .checked: the JIT launcher has verified the tensors of this launch


_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def current_device():
    """Index of the current CUDA device (the raw getter once CUDA is up: a launch asks this for
    every call)."""
    if _raw_device is not None and torch.cuda.is_initialized():
        return _raw_device()
    return torch.cuda.current_device()


def raw_stream():
    """The current stream of the current device as an integer handle."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _stream():
    if _raw_stream is not None:      # the handle without building a torch.cuda.Stream object
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class checked_tensors:
    """Inside this block `_dev_ptr` takes tensors as already verified (CUDA, current device):
    the JIT launcher checks every tensor argument once per launch (runtime/jit.py `_run`)."""

    def __enter__(self):
        _trust.checked = True

    def __exit__(self, *exc):
        _trust.checked = False


def _dev_ptr(name, t):
    if getattr(_trust, "checked", False):
        return ctypes.c_void_p(t.data_ptr())
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"argument '{name}' must be a CUDA tensor")
    if t.device.index not in (None, torch.cuda.current_device()):
        raise ValueError(
            f"tensor '{name}' is on {t.device} but the current device is "
            f"cuda:{torch.cuda.current_device()}; newt launches on the current device")
    return ctypes.c_void_p(t.data_ptr())


def add_f32(x, y, out, n):
    abi.check(abi.load().nb200_add_f32(_dev_ptr("x", x), _dev_ptr("y", y), _dev_ptr("out", out),
                                       int(n), _stream()))


def softmax_f32(x, out, rows, n, stride_x, stride_out):
    abi.check(abi.load().nb200_softmax_f32(_dev_ptr("x", x), _dev_ptr("out", out), int(rows),
                                           int(n), int(stride_x), int(stride_out), _stream()))


def layernorm(x, w, b, out, rows, n, stride_x, stride_out, eps):
    abi.check(abi.load().nb200_layernorm(
        _dev_ptr("x", x), _dev_ptr("w", w), _dev_ptr("b", b), _dev_ptr("out", out), int(rows),
        int(n), int(stride_x), int(stride_out), float(eps), abi.dtype_code(x.dtype), _stream()))


def gemm_config(block_m=0, block_n=0, block_k=0, stages=0, cta_pair=0):
    return abi.GemmConfig(block_m, block_n, block_k, stages, cta_pair)


def gemm(a, b, c, m, n, k, lda, ldb, ldc, config=None):
    cfg = ctypes.byref(config) if config is not None else None
    abi.check(abi.load().nb200_gemm(_dev_ptr("a", a), _dev_ptr("b", b), _dev_ptr("c", c), int(m),
                                    int(n), int(k), int(lda), int(ldb), int(ldc),
                                    abi.dtype_code(a.dtype), cfg, _stream()))


def gemm_bt(a, bt, c, m, n, k, lda, ldbt, ldc, config=None):
    """C = A @ B with B given transposed: bt is [N, K] with row stride ldbt."""
    cfg = ctypes.byref(config) if config is not None else None
    abi.check(abi.load().nb200_gemm_bt(_dev_ptr("a", a), _dev_ptr("b", bt), _dev_ptr("c", c), int(m),
                                       int(n), int(k), int(lda), int(ldbt), int(ldc),
                                       abi.dtype_code(a.dtype), cfg, _stream()))


def gemm_split_bytes(m, n, k, dtype, config=None):
    """Bytes of workspace with which `gemm_split` cuts the last round of tiles along K; 0 when the
    tiles of this problem stay whole."""
    cfg = ctypes.byref(config) if config is not None else None
    return int(abi.load().nb200_gemm_split_workspace_bytes(int(m), int(n), int(k),
                                                           abi.dtype_code(dtype), cfg))


def gemm_split(a, b, c, m, n, k, lda, ldb, ldc, config=None, b_transposed=False, need=None):
    """`gemm` / `gemm_bt` with a split tail (nb200_gemm_split): when the last round of whole tiles
    would leave part of the chip idle, its tiles are cut along K and summed through a workspace,
    a fresh tensor of torch's caching allocator (allocated and used on the current stream).
    `need`: the workspace size if the caller has asked for it before."""
    if need is None:
        need = gemm_split_bytes(m, n, k, a.dtype, config)
    if need == 0:
        return (gemm_bt if b_transposed else gemm)(a, b, c, m, n, k, lda, ldb, ldc, config)
    ws = torch.empty(need, dtype=torch.uint8, device=a.device)
    cfg = ctypes.byref(config) if config is not None else None
    abi.check(abi.load().nb200_gemm_split(_dev_ptr("a", a), _dev_ptr("b", b), _dev_ptr("c", c), int(m),
                                          int(n), int(k), int(lda), int(ldb), int(ldc),
                                          abi.dtype_code(a.dtype), 1 if b_transposed else 0, cfg,
                                          ctypes.c_void_p(ws.data_ptr()), need, _stream()))


def gemm_tf32(a, b, c, m, n, k, lda, ldb, ldc, config=None):
    """fp32 C = A @ B (tf32 product, fp32 accumulation) with B as [K, N].  A B whose base and
    pitch are 16-byte aligned is read in place; any other is transposed into a workspace first,
    a fresh tensor of torch's caching allocator: allocated and used on the current stream, so
    the allocator's stream-ordered reuse keeps concurrent launches apart."""
    if b.data_ptr() % 16 == 0 and int(ldb) % 4 == 0:
        return gemm(a, b, c, m, n, k, lda, ldb, ldc, config)
    need = int(abi.load().nb200_gemm_tf32_workspace_bytes(int(n), int(k)))
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=a.device)
    cfg = ctypes.byref(config) if config is not None else None
    abi.check(abi.load().nb200_gemm_tf32(_dev_ptr("a", a), _dev_ptr("b", b), _dev_ptr("c", c), int(m),
                                         int(n), int(k), int(lda), int(ldb), int(ldc), cfg,
                                         ctypes.c_void_p(ws.data_ptr()), ws.numel(), _stream()))


def gemm_acc32(a, b, c, m, n, k, lda, ldb, ldc, b_transposed=False, config=None):
    """fp32 C = A @ B for fp16 / bf16 operands: the accumulator as it is, not rounded."""
    cfg = ctypes.byref(config) if config is not None else None
    abi.check(abi.load().nb200_gemm_acc32(_dev_ptr("a", a), _dev_ptr("b", b), _dev_ptr("c", c),
                                          int(m), int(n), int(k), int(lda), int(ldb), int(ldc),
                                          abi.dtype_code(a.dtype), 1 if b_transposed else 0, cfg,
                                          _stream()))


def repitched(slot, t, rows, cols, row_stride, col_stride):
    """A row-major copy of the [rows, cols] matrix that starts at `t` with the given strides
    (in elements), as a fresh tensor of torch's caching allocator (allocated and used on the
    current stream); returns (tensor of t's dtype, pitch in elements).  The pitch is a multiple
    of 16 bytes, which is what the tensor-core GEMM needs of its operands.  `slot` ("a" or "b")
    only names the operand in error messages."""
    eb = t.element_size()
    pitch = -(-int(cols) // (16 // eb)) * (16 // eb)
    ws = torch.empty(max(int(rows) * pitch, 16), dtype=t.dtype, device=t.device)
    abi.check(abi.load().nb200_repitch(_dev_ptr(slot, t), ctypes.c_void_p(ws.data_ptr()), int(rows),
                                       int(cols), int(row_stride), int(col_stride), pitch, eb,
                                       _stream()))
    return ws, pitch


def gemm_check(a, b, c, m, n, k, lda, ldb, ldc, config=None):
    """Returns None if the tcgen05 path can run this problem, else the reason (str)."""
    cfg = ctypes.byref(config) if config is not None else None
    rc = abi.load().nb200_gemm_check(_dev_ptr("a", a), _dev_ptr("b", b), _dev_ptr("c", c), int(m),
                                     int(n), int(k), int(lda), int(ldb), int(ldc),
                                     abi.dtype_code(a.dtype), cfg)
    return None if rc == 0 else abi.last_error()


def attention_fwd(q, k, v, o, scale, causal):
    """q,o: [bh, seq_q, d]; k,v: [bh, seq_kv, d]; innermost stride 1."""
    bh, sq, d = q.shape
    skv = k.shape[1]
    for name, t in (("q", q), ("k", k), ("v", v), ("o", o)):
        if t.stride(2) != 1:
            raise ValueError(f"attention: '{name}' must have unit stride along head_dim")
    abi.check(abi.load().nb200_attention_fwd(
        _dev_ptr("q", q), _dev_ptr("k", k), _dev_ptr("v", v), _dev_ptr("o", o), bh, sq, skv, d,
        q.stride(0), q.stride(1), k.stride(0), k.stride(1), v.stride(0), v.stride(1),
        o.stride(0), o.stride(1), float(scale), int(bool(causal)), abi.dtype_code(q.dtype),
        _stream()))
