"""The user-level kernels of the hot path, written against newt_b200 exactly as
the reference's examples and tests write them against newt (same text modulo the
import): examples/01..04, benchmarks/bench.py:90-108.  Shared by CPU structure
tests and GPU parity tests."""

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


@newt.jit
def layernorm_kernel(x_ptr, w_ptr, b_ptr, out_ptr, N, stride, eps,
                     BLOCK_N: nl.constexpr):
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


@newt.jit
def matmul_kernel_unmasked(a_ptr, b_ptr, c_ptr, M, N, K, sam, sak, sbk, sbn, scm, scn,
                           BLOCK_M: nl.constexpr, BLOCK_N: nl.constexpr, BLOCK_K: nl.constexpr):
    pid_m = nl.program_id(0)
    pid_n = nl.program_id(1)
    offs_m = pid_m * BLOCK_M + nl.arange(0, BLOCK_M)
    offs_n = pid_n * BLOCK_N + nl.arange(0, BLOCK_N)
    offs_k = nl.arange(0, BLOCK_K)
    a_ptrs = a_ptr + offs_m[:, None] * sam + offs_k[None, :] * sak
    b_ptrs = b_ptr + offs_k[:, None] * sbk + offs_n[None, :] * sbn
    acc = nl.zeros((BLOCK_M, BLOCK_N), dtype=nl.float32)
    for k in range(K // BLOCK_K):
        a = nl.load(a_ptrs)
        b = nl.load(b_ptrs)
        acc = nl.dot(a, b, acc)
        a_ptrs += BLOCK_K * sak
        b_ptrs += BLOCK_K * sbk
    c_ptrs = c_ptr + offs_m[:, None] * scm + offs_n[None, :] * scn
    nl.store(c_ptrs, acc.to(nl.float16))


@newt.jit
def attention_kernel_2d(q_ptr, k_ptr, v_ptr, o_ptr, M, N, scale,
                        sqm, sqd, skn, skd, svn, svd, som, sod,
                        BLOCK_M: nl.constexpr, BLOCK_N: nl.constexpr, D: nl.constexpr):
    # examples/05_fused_attention.py:14-48 as shipped: single head, non-causal
    pid = nl.program_id(0)
    offs_m = pid * BLOCK_M + nl.arange(0, BLOCK_M)
    offs_d = nl.arange(0, D)
    qmask = offs_m[:, None] < M
    q = nl.load(q_ptr + offs_m[:, None] * sqm + offs_d[None, :] * sqd, mask=qmask, other=0.0)
    m_i = nl.full((BLOCK_M,), float("-inf"), dtype=nl.float32)
    l_i = nl.zeros((BLOCK_M,), dtype=nl.float32)
    acc = nl.zeros((BLOCK_M, D), dtype=nl.float32)
    for start_n in range(0, N, BLOCK_N):
        offs_n = start_n + nl.arange(0, BLOCK_N)
        nmask = offs_n[:, None] < N
        k = nl.load(k_ptr + offs_n[:, None] * skn + offs_d[None, :] * skd, mask=nmask, other=0.0)
        qk = nl.dot(q, nl.trans(k)) * scale
        qk = nl.where(offs_n[None, :] < N, qk, float("-inf"))
        m_new = nl.maximum(m_i, nl.max(qk, axis=1))
        alpha = nl.exp(m_i - m_new)
        p = nl.exp(qk - m_new[:, None])
        l_i = l_i * alpha + nl.sum(p, axis=1)
        acc = acc * alpha[:, None]
        v = nl.load(v_ptr + offs_n[:, None] * svn + offs_d[None, :] * svd, mask=nmask, other=0.0)
        acc = nl.dot(p.to(nl.float16), v, acc)
        m_i = m_new
    acc = acc / l_i[:, None]
    nl.store(o_ptr + offs_m[:, None] * som + offs_d[None, :] * sod, acc, mask=qmask)
