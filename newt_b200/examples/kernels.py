"""`@jit` kernels of examples/01-04 of the reference and their launch wrappers."""

import torch

import newt_b200 as newt
import newt_b200.language as nl


@newt.jit
def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: nl.constexpr):
    pid = nl.program_id(0)
    offs = pid * BLOCK + nl.arange(0, BLOCK)
    mask = offs < n
    x = nl.load(x_ptr + offs, mask=mask)
    y = nl.load(y_ptr + offs, mask=mask)
    nl.store(out_ptr + offs, x + y, mask=mask)


def add(x, y, out=None):
    """examples/01_vector_add.py:24-29"""
    out = torch.empty_like(x) if out is None else out
    n = x.numel()
    add_kernel[lambda meta: (newt.cdiv(n, meta["BLOCK"]),)](x, y, out, n, BLOCK=4096)
    return out


@newt.jit
def gelu_residual_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: nl.constexpr):
    """out = gelu(x) + y, tanh approximation: the chain of examples/deuteron/04_fused_ops.py
    written against the block language.  Not one of the tuned programs: it goes through the
    generic elementwise lowering."""
    offs = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    mask = offs < n
    v = nl.load(x_ptr + offs, mask=mask, other=0.0)
    inner = 0.7978845608028654 * (v + 0.044715 * v * v * v)
    g = 0.5 * v * (1.0 + nl.tanh(inner))
    nl.store(out_ptr + offs, g + nl.load(y_ptr + offs, mask=mask, other=0.0), mask=mask)


def gelu_residual(x, y, out=None, BLOCK=2048, num_warps=8):
    out = torch.empty_like(x) if out is None else out
    n = x.numel()
    gelu_residual_kernel[(newt.cdiv(n, BLOCK),)](x, y, out, n, BLOCK=BLOCK, num_warps=num_warps)
    return out


@newt.jit
def softmax_kernel(x_ptr, out_ptr, N, stride, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf"))
    x = x - nl.max(x, axis=0)
    num = nl.exp(x)
    den = nl.sum(num, axis=0)
    nl.store(out_ptr + row * stride + cols, num / den, mask=mask)


def softmax(x, out=None):
    """examples/02_fused_softmax.py:27-33"""
    m, n = x.shape
    out = torch.empty_like(x) if out is None else out
    block = newt.next_power_of_2(n)
    softmax_kernel[(m,)](x, out, n, x.stride(0), BLOCK_N=block,
                         num_warps=4 if block < 4096 else 8)
    return out


# Rows of the same family that are not the tuned programs -- a temperature, a logarithm, no
# mean -- go through the generic lowering, which keeps such a row in registers.
@newt.jit
def softmax_temperature_kernel(x_ptr, out_ptr, N, stride, inv_t, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf")) * inv_t
    e = nl.exp(x - nl.max(x, axis=0))
    nl.store(out_ptr + row * stride + cols, e / nl.sum(e, axis=0), mask=mask)


@newt.jit
def log_softmax_kernel(x_ptr, out_ptr, N, stride, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=float("-inf"))
    z = x - nl.max(x, axis=0)
    nl.store(out_ptr + row * stride + cols, z - nl.log(nl.sum(nl.exp(z), axis=0)), mask=mask)


@newt.jit
def rmsnorm_kernel(x_ptr, w_ptr, out_ptr, N, stride, eps, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=0.0).to(nl.float32)
    ms = nl.sum(x * x, axis=0) / N
    y = x * nl.rsqrt(ms + eps) * nl.load(w_ptr + cols, mask=mask, other=0.0)
    nl.store(out_ptr + row * stride + cols, y, mask=mask)


def _row_launch(kernel, x, out, *extra):
    m, n = x.shape
    block = newt.next_power_of_2(n)
    kernel[(m,)](*extra[:-1], n, x.stride(0), *extra[-1], BLOCK_N=block,
                 num_warps=4 if block < 4096 else 8)
    return out


def softmax_temperature(x, temperature, out=None):
    out = torch.empty_like(x) if out is None else out
    return _row_launch(softmax_temperature_kernel, x, out, x, out, (1.0 / temperature,))


def log_softmax(x, out=None):
    out = torch.empty_like(x) if out is None else out
    return _row_launch(log_softmax_kernel, x, out, x, out, ())


def rmsnorm(x, w, eps=1e-6, out=None):
    out = torch.empty_like(x) if out is None else out
    return _row_launch(rmsnorm_kernel, x, out, x, w, out, (eps,))


@newt.jit
def layernorm_kernel(x_ptr, w_ptr, b_ptr, out_ptr, N, stride, eps, BLOCK_N: nl.constexpr):
    row = nl.program_id(0)
    cols = nl.arange(0, BLOCK_N)
    mask = cols < N
    x = nl.load(x_ptr + row * stride + cols, mask=mask, other=0.0)
    mean = nl.sum(x, axis=0) / N
    diff = nl.where(mask, x - mean, 0.0)
    var = nl.sum(diff * diff, axis=0) / N
    rstd = nl.rsqrt(var + eps)
    w = nl.load(w_ptr + cols, mask=mask)
    b = nl.load(b_ptr + cols, mask=mask)
    y = (x - mean) * rstd * w + b
    nl.store(out_ptr + row * stride + cols, y, mask=mask)


def layernorm(x, w, b, eps=1e-5, out=None):
    """examples/03_layernorm.py:30-36"""
    m, n = x.shape
    out = torch.empty_like(x) if out is None else out
    layernorm_kernel[(m,)](x, w, b, out, n, x.stride(0), eps,
                           BLOCK_N=newt.next_power_of_2(n), num_warps=8)
    return out


# Tile / pipeline choices for sm_100a: 128-row tcgen05 MMAs (256 rows = a CTA pair), 64..256
# columns, 64-element K slabs per TMA stage, ring depth as num_stages.
@newt.autotune(
    configs=[
        newt.Config({"BLOCK_M": 256, "BLOCK_N": 512, "BLOCK_K": 64}, num_warps=4, num_stages=4),
        newt.Config({"BLOCK_M": 256, "BLOCK_N": 512, "BLOCK_K": 32}, num_warps=4, num_stages=4),   # fp32: one row of K
        newt.Config({"BLOCK_M": 256, "BLOCK_N": 256, "BLOCK_K": 128}, num_warps=4, num_stages=3),
        newt.Config({"BLOCK_M": 256, "BLOCK_N": 256, "BLOCK_K": 64}, num_warps=4, num_stages=6),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 256, "BLOCK_K": 64}, num_warps=4, num_stages=4),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 256, "BLOCK_K": 64}, num_warps=4, num_stages=3),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64}, num_warps=4, num_stages=6),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 64}, num_warps=4, num_stages=4),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 64}, num_warps=4, num_stages=8),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 128, "BLOCK_K": 128}, num_warps=4, num_stages=3),
        newt.Config({"BLOCK_M": 128, "BLOCK_N": 64, "BLOCK_K": 128}, num_warps=4, num_stages=4),
    ],
    key=["M", "N", "K"],
)
@newt.jit
def matmul_kernel(a_ptr, b_ptr, c_ptr, M, N, K,
                  sam, sak, sbk, sbn, scm, scn,
                  BLOCK_M: nl.constexpr, BLOCK_N: nl.constexpr, BLOCK_K: nl.constexpr):
    pid_m = nl.program_id(0)
    pid_n = nl.program_id(1)
    offs_m = pid_m * BLOCK_M + nl.arange(0, BLOCK_M)
    offs_n = pid_n * BLOCK_N + nl.arange(0, BLOCK_N)
    offs_k = nl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + offs_m[:, None] * sam + offs_k[None, :] * sak
    b_ptrs = b_ptr + offs_k[:, None] * sbk + offs_n[None, :] * sbn
    acc = nl.zeros((BLOCK_M, BLOCK_N), dtype=nl.float32)
    for k in range(nl.cdiv(K, BLOCK_K)):
        a_mask = (offs_m[:, None] < M) & (offs_k[None, :] < K - k * BLOCK_K)
        b_mask = (offs_k[:, None] < K - k * BLOCK_K) & (offs_n[None, :] < N)
        a = nl.load(a_ptrs, mask=a_mask, other=0.0)
        b = nl.load(b_ptrs, mask=b_mask, other=0.0)
        acc = nl.dot(a, b, acc)
        a_ptrs += BLOCK_K * sak
        b_ptrs += BLOCK_K * sbk
    c_ptrs = c_ptr + offs_m[:, None] * scm + offs_n[None, :] * scn
    c_mask = (offs_m[:, None] < M) & (offs_n[None, :] < N)
    nl.store(c_ptrs, acc.to(c_ptr.dtype.element_ty), mask=c_mask)


def matmul(a, b, c=None):
    """examples/04_matmul.py:48-56"""
    m, k = a.shape
    _, n = b.shape
    c = torch.empty(m, n, device=a.device, dtype=a.dtype) if c is None else c
    grid = lambda meta: (newt.cdiv(m, meta["BLOCK_M"]), newt.cdiv(n, meta["BLOCK_N"]))  # noqa: E731
    matmul_kernel[grid](a, b, c, m, n, k, a.stride(0), a.stride(1), b.stride(0), b.stride(1),
                        c.stride(0), c.stride(1))
    return c


@newt.jit
def linear_bias_relu_kernel(a_ptr, b_ptr, bias_ptr, c_ptr, M, N, K, sam, sak, sbk, sbn, scm, scn,
                            BLOCK_M: nl.constexpr, BLOCK_N: nl.constexpr, BLOCK_K: nl.constexpr):
    """relu(A @ B + bias): the matmul of examples/04_matmul.py:22-45 with an epilogue fused after
    the k loop (as tests/test_ops.py:458-473 does with arithmetic and a reduction)."""
    offs_m = nl.program_id(0) * BLOCK_M + nl.arange(0, BLOCK_M)
    offs_n = nl.program_id(1) * BLOCK_N + nl.arange(0, BLOCK_N)
    offs_k = nl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + offs_m[:, None] * sam + offs_k[None, :] * sak
    b_ptrs = b_ptr + offs_k[:, None] * sbk + offs_n[None, :] * sbn
    acc = nl.zeros((BLOCK_M, BLOCK_N), dtype=nl.float32)
    for k in range(nl.cdiv(K, BLOCK_K)):
        a = nl.load(a_ptrs, mask=(offs_m[:, None] < M) & (offs_k[None, :] < K - k * BLOCK_K), other=0.0)
        b = nl.load(b_ptrs, mask=(offs_k[:, None] < K - k * BLOCK_K) & (offs_n[None, :] < N), other=0.0)
        acc = nl.dot(a, b, acc)
        a_ptrs += BLOCK_K * sak
        b_ptrs += BLOCK_K * sbk
    bias = nl.load(bias_ptr + offs_n, mask=offs_n < N, other=0.0)
    out = nl.maximum(acc + bias[None, :], 0.0)
    nl.store(c_ptr + offs_m[:, None] * scm + offs_n[None, :] * scn, out.to(c_ptr.dtype.element_ty),
             mask=(offs_m[:, None] < M) & (offs_n[None, :] < N))


def linear_bias_relu(a, b, bias, c=None, BLOCK_M=256, BLOCK_N=None, BLOCK_K=64, num_stages=None):
    m, k = a.shape
    _, n = b.shape
    if BLOCK_N is None:
        # 256 x 512 tiles once they fill the 74 CTA pairs of a B200 several times over (1553 against
        # 1515 TFLOP/s at 8192^3), 256 x 256 below (4096^3: 1425 against 1314 -- the wide tile's
        # epilogue is not hidden behind a second accumulator, and two rounds show it twice)
        BLOCK_N = 512 if BLOCK_M == 256 and newt.cdiv(m, 256) * newt.cdiv(n, 512) >= 4 * 74 else 256
    if num_stages is None:
        num_stages = 4 if BLOCK_N == 512 else 6
    c = torch.empty(m, n, device=a.device, dtype=a.dtype) if c is None else c
    linear_bias_relu_kernel[(newt.cdiv(m, BLOCK_M), newt.cdiv(n, BLOCK_N))](
        a, b, bias, c, m, n, k, a.stride(0), a.stride(1), b.stride(0), b.stride(1), c.stride(0),
        c.stride(1), BLOCK_M=BLOCK_M, BLOCK_N=BLOCK_N, BLOCK_K=BLOCK_K, num_stages=num_stages)
    return c


# examples/05_fused_attention.py:14-48 of the reference, with a batch*head grid axis and an
# optional causal mask (both written with operations that example already uses).
@newt.jit
def attention_kernel(q_ptr, k_ptr, v_ptr, o_ptr, M, N, scale,
                     sqh, sqm, sqd, skh, skn, skd, svh, svn, svd, soh, som, sod,
                     BLOCK_M: nl.constexpr, BLOCK_N: nl.constexpr, D: nl.constexpr,
                     CAUSAL: nl.constexpr):
    pid = nl.program_id(0)
    head = nl.program_id(1)
    offs_m = pid * BLOCK_M + nl.arange(0, BLOCK_M)
    offs_d = nl.arange(0, D)
    qmask = offs_m[:, None] < M
    q = nl.load(q_ptr + head * sqh + offs_m[:, None] * sqm + offs_d[None, :] * sqd,
                mask=qmask, other=0.0)                                  # [BM, D]

    m_i = nl.full((BLOCK_M,), float("-inf"), dtype=nl.float32)         # row maxes
    l_i = nl.zeros((BLOCK_M,), dtype=nl.float32)                       # row sums
    acc = nl.zeros((BLOCK_M, D), dtype=nl.float32)                     # output acc

    hi = N
    if CAUSAL:
        hi = nl.minimum(N, (pid + 1) * BLOCK_M)                        # skip blocks above the diagonal
    for start_n in range(0, hi, BLOCK_N):
        offs_n = start_n + nl.arange(0, BLOCK_N)
        nmask = offs_n[:, None] < N
        k = nl.load(k_ptr + head * skh + offs_n[:, None] * skn + offs_d[None, :] * skd,
                    mask=nmask, other=0.0)                              # [BN, D]
        qk = nl.dot(q, nl.trans(k)) * scale                            # [BM, BN]
        keep = offs_n[None, :] < N
        if CAUSAL:
            keep = keep & (offs_n[None, :] <= offs_m[:, None])
        qk = nl.where(keep, qk, float("-inf"))
        m_new = nl.maximum(m_i, nl.max(qk, axis=1))
        alpha = nl.exp(m_i - m_new)
        p = nl.exp(qk - m_new[:, None])
        l_i = l_i * alpha + nl.sum(p, axis=1)
        acc = acc * alpha[:, None]
        v = nl.load(v_ptr + head * svh + offs_n[:, None] * svn + offs_d[None, :] * svd,
                    mask=nmask, other=0.0)                              # [BN, D]
        acc = nl.dot(p.to(q_ptr.dtype.element_ty), v, acc)
        m_i = m_new

    acc = acc / l_i[:, None]
    nl.store(o_ptr + head * soh + offs_m[:, None] * som + offs_d[None, :] * sod, acc, mask=qmask)


def attention(q, k, v, causal=False, out=None, BLOCK_M=128, BLOCK_N=128, num_warps=4):
    """q, k, v: [batch*heads, seq, head_dim] (or [batch, heads, seq, head_dim] contiguous)."""
    if q.dim() == 4:
        b, h, s, d = q.shape
        o = attention(q.reshape(b * h, s, d), k.reshape(b * h, -1, d), v.reshape(b * h, -1, d),
                      causal, None if out is None else out.reshape(b * h, s, d), BLOCK_M, BLOCK_N,
                      num_warps)
        return o.reshape(b, h, s, d)
    bh, m, d = q.shape
    n = k.shape[1]
    o = torch.empty_like(q) if out is None else out
    grid = (newt.cdiv(m, BLOCK_M), bh)
    attention_kernel[grid](q, k, v, o, m, n, 1.0 / d ** 0.5,
                           q.stride(0), q.stride(1), q.stride(2), k.stride(0), k.stride(1),
                           k.stride(2), v.stride(0), v.stride(1), v.stride(2), o.stride(0),
                           o.stride(1), o.stride(2), BLOCK_M=BLOCK_M, BLOCK_N=BLOCK_N, D=d,
                           CAUSAL=bool(causal), num_warps=num_warps)
    return o
