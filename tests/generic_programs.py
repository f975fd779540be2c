"""Programs with control flow and with dots outside the tuned kernels, shared by the CPU test
(every program lowers and its generated CUDA compiles for sm_100a) and the GPU test (the
results match torch).  The shapes of the control flow follow the reference's own control-flow
and operator tests (tests/test_control_flow.py, tests/test_ops.py, tests/test_matmul.py:52-57,
tests/test_review_fixes.py): runtime loops with accumulators, scalars and walking pointers,
`while`, runtime `if`, `break` / `continue`, nested loops, stores and reductions inside loops,
small and odd-shaped dots.

Each case: name -> (kernel, grid, build) where `build(device)` returns
(args, meta, checks) and `checks` is a list of (output tensor, expected CPU tensor, rtol, atol).
"""

import torch

import newt_b200 as newt
import newt_b200.language as nl


def _draw(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


# ---- loops that only compute ------------------------------------------------------------------

@newt.jit
def weighted_tiles(x_ptr, o_ptr, n_tiles, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    acc = nl.zeros((BLOCK,), dtype=nl.float32)
    p = x_ptr + offs
    for t in range(n_tiles):
        acc = acc + nl.load(p) * (t + 1)
        p += BLOCK
    nl.store(o_ptr + offs, acc)


def _weighted_tiles(dev):
    tiles, block = 7, 256
    x = _draw(tiles * block, 1)
    o = torch.empty(block, device=dev)
    w = torch.arange(1, tiles + 1, dtype=torch.float32)[:, None]
    return (x.to(dev), o, tiles), dict(BLOCK=block), [(o, (x.view(tiles, block) * w).sum(0), 1e-5, 1e-5)]


@newt.jit
def sum_of_cubes(o_ptr, n, BLOCK: nl.constexpr):
    s = 0
    for i in range(n):
        s = s + i * i * i
    nl.store(o_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.int32) + s)


def _sum_of_cubes(dev):
    o = torch.empty(64, device=dev, dtype=torch.int32)
    return (o, 13), dict(BLOCK=64), [(o, torch.full((64,), sum(i ** 3 for i in range(13)), dtype=torch.int32), 0, 0)]


@newt.jit
def strided_range(o_ptr, lo, hi, BLOCK: nl.constexpr):
    s = 0
    for i in range(lo, hi, 3):
        s += i
    for i in range(hi, lo, -2):
        s += i * 100
    nl.store(o_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.int32) + s)


def _strided_range(dev):
    o = torch.empty(32, device=dev, dtype=torch.int32)
    want = sum(range(2, 20, 3)) + 100 * sum(range(20, 2, -2))
    return (o, 2, 20), dict(BLOCK=32), [(o, torch.full((32,), want, dtype=torch.int32), 0, 0)]


@newt.jit
def nested_products(o_ptr, n, m, BLOCK: nl.constexpr):
    s = 0
    for i in range(n):
        for j in range(m):
            s = s + i * j + 1
    nl.store(o_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.int32) + s)


def _nested_products(dev):
    o = torch.empty(32, device=dev, dtype=torch.int32)
    want = sum(i * j + 1 for i in range(6) for j in range(5))
    return (o, 6, 5), dict(BLOCK=32), [(o, torch.full((32,), want, dtype=torch.int32), 0, 0)]


@newt.jit
def next_power(o_ptr, n, BLOCK: nl.constexpr):
    v = 1
    steps = 0
    while v < n:
        v = v * 2
        steps += 1
    nl.store(o_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.int32) + v * 1000 + steps)


def _next_power(dev):
    o = torch.empty(32, device=dev, dtype=torch.int32)
    return (o, 300), dict(BLOCK=32), [(o, torch.full((32,), 512 * 1000 + 9, dtype=torch.int32), 0, 0)]


@newt.jit
def capped_growth(o_ptr, n, cap, BLOCK: nl.constexpr):
    v = 1
    c = 0
    while v < n:
        v = v * 3
        c += 1
        if c == cap:
            break
    nl.store(o_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.int32) + v * 100 + c)


def _capped_growth(dev):
    o = torch.empty(32, device=dev, dtype=torch.int32)
    return (o, 100000, 4), dict(BLOCK=32), [(o, torch.full((32,), 81 * 100 + 4, dtype=torch.int32), 0, 0)]


@newt.jit
def skipping(o_ptr, n, stop, BLOCK: nl.constexpr):
    s = 0
    for i in range(n):
        if i == stop:
            break
        if i % 3 == 1:
            continue
        for j in range(4):
            s = s + i * j
    t = 0
    for i in range(12):          # the same with compile-time bounds: unrolled
        if i == 9:
            break
        if i % 3 == 1:
            continue
        t = t + i
    nl.store(o_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.int32) + s * 1000 + t)


def _skipping(dev):
    o = torch.empty(32, device=dev, dtype=torch.int32)
    s = sum(i * j for i in range(9) if i % 3 != 1 for j in range(4))
    t = sum(i for i in range(9) if i % 3 != 1)
    return (o, 20, 9), dict(BLOCK=32), [(o, torch.full((32,), s * 1000 + t, dtype=torch.int32), 0, 0)]


@newt.jit
def two_way(x_ptr, o_ptr, side_ptr, flag, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    x = nl.load(x_ptr + offs)
    y = nl.zeros((BLOCK,), dtype=nl.float32)
    if flag == 1:
        y = x * 2
    else:
        y = x * 3
        nl.store(side_ptr + offs, x + 1)       # only the taken arm touches memory
    if flag > 5:
        y = y + 100
    nl.store(o_ptr + offs, y)


def _two_way(flag):
    def build(dev):
        x = _draw(128, 3)
        o = torch.empty(128, device=dev)
        side = torch.full((128,), -7.0, device=dev)
        y = x * 2 if flag == 1 else x * 3
        if flag > 5:
            y = y + 100
        want_side = torch.full((128,), -7.0) if flag == 1 else x + 1
        return (x.to(dev), o, side, flag), dict(BLOCK=128), [(o, y, 0, 0), (side, want_side, 0, 0)]
    return build


# ---- loops that store, loops that reduce --------------------------------------------------------

@newt.jit
def scale_tiles(x_ptr, o_ptr, n, n_tiles, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    for t in range(n_tiles):
        i = t * BLOCK + offs
        ok = i < n
        x = nl.load(x_ptr + i, mask=ok, other=0.0)
        nl.store(o_ptr + i, x * 2 + t, mask=ok)


def _scale_tiles(dev):
    n, block = 1000, 128
    tiles = -(-n // block)
    x = _draw(n, 4)
    o = torch.zeros(n, device=dev)
    t = (torch.arange(n) // block).float()
    return (x.to(dev), o, n, tiles), dict(BLOCK=block), [(o, x * 2 + t, 0, 0)]


@newt.jit
def running_softmax_stats(x_ptr, m_ptr, l_ptr, n, stride, BLOCK: nl.constexpr):
    """Row maximum and softmax denominator, one pass over column tiles (the online update)."""
    row = nl.program_id(0)
    offs = nl.arange(0, BLOCK)
    m = -float("inf")
    l = 0.0
    for start in range(0, n, BLOCK):
        cols = start + offs
        x = nl.load(x_ptr + row * stride + cols, mask=cols < n, other=-float("inf"))
        m_new = nl.maximum(m, nl.max(x, axis=0))
        l = l * nl.exp(m - m_new) + nl.sum(nl.exp(x - m_new), axis=0)
        m = m_new
    nl.store(m_ptr + row, m)
    nl.store(l_ptr + row, l)


def _running_softmax_stats(dev):
    rows, n = 5, 700
    x = _draw((rows, n), 5, scale=3.0)
    m = torch.empty(rows, device=dev)
    l = torch.empty(rows, device=dev)
    want_m = x.max(dim=1).values
    want_l = torch.exp(x - want_m[:, None]).sum(dim=1)
    return (x.to(dev), m, l, n, n), dict(BLOCK=256), [(m, want_m, 0, 0), (l, want_l, 2e-5, 1e-6)], (rows,)


@newt.jit
def tiled_layernorm(x_ptr, w_ptr, y_ptr, n, stride, eps, BLOCK: nl.constexpr):
    """Layernorm of rows longer than a block: two loops for the statistics, one that stores."""
    row = nl.program_id(0)
    offs = nl.arange(0, BLOCK)
    part = nl.zeros((BLOCK,), dtype=nl.float32)
    for start in range(0, n, BLOCK):
        cols = start + offs
        part += nl.load(x_ptr + row * stride + cols, mask=cols < n, other=0.0).to(nl.float32)
    mean = nl.sum(part, axis=0) / n
    part2 = nl.zeros((BLOCK,), dtype=nl.float32)
    for start in range(0, n, BLOCK):
        cols = start + offs
        x = nl.load(x_ptr + row * stride + cols, mask=cols < n, other=0.0).to(nl.float32)
        d = nl.where(cols < n, x - mean, 0.0)
        part2 += d * d
    rstd = nl.rsqrt(nl.sum(part2, axis=0) / n + eps)
    for start in range(0, n, BLOCK):
        cols = start + offs
        ok = cols < n
        x = nl.load(x_ptr + row * stride + cols, mask=ok, other=0.0).to(nl.float32)
        w = nl.load(w_ptr + cols, mask=ok, other=0.0)
        nl.store(y_ptr + row * stride + cols, (x - mean) * rstd * w, mask=ok)


def _tiled_layernorm(dev):
    rows, n = 6, 1000
    x = _draw((rows, n), 6, torch.float16)
    w = _draw(n, 7, torch.float16)
    y = torch.zeros(rows, n, device=dev, dtype=torch.float16)
    xf = x.float()
    want = (xf - xf.mean(1, keepdim=True)) * torch.rsqrt(xf.var(1, unbiased=False, keepdim=True) + 1e-5) * w.float()
    return (x.to(dev), w.to(dev), y, n, n, 1e-5), dict(BLOCK=256), [(y, want.half(), 2e-3, 2e-3)], (rows,)


@newt.jit
def power_iteration(a_ptr, v_ptr, o_ptr, steps, N: nl.constexpr):
    """v <- normalise(A v), a few times: the carried block is read at other elements than the
    one being written (through the reduction), so it is staged."""
    r = nl.arange(0, N)
    a = nl.load(a_ptr + r[:, None] * N + r[None, :])
    v = nl.load(v_ptr + r)
    for _ in range(steps):
        w = nl.sum(a * v[None, :], axis=1)
        v = w / nl.sqrt(nl.sum(w * w, axis=0))
    nl.store(o_ptr + r, v)


def _power_iteration(dev):
    n = 32
    a = _draw((n, n), 8)
    a = a @ a.T / n + torch.eye(n)
    v = _draw(n, 9)
    o = torch.empty(n, device=dev)
    want = v.clone()
    for _ in range(5):
        w = a @ want
        want = w / w.norm()
    return (a.to(dev), v.to(dev), o, 5), dict(N=n), [(o, want, 1e-4, 1e-5)]


# ---- dots outside the tuned kernels --------------------------------------------------------------

@newt.jit
def one_tile_dot(a_ptr, b_ptr, c_ptr, M: nl.constexpr, N: nl.constexpr, K: nl.constexpr):
    rm = nl.arange(0, M)
    rn = nl.arange(0, N)
    rk = nl.arange(0, K)
    a = nl.load(a_ptr + rm[:, None] * K + rk[None, :])
    b = nl.load(b_ptr + rk[:, None] * N + rn[None, :])
    nl.store(c_ptr + rm[:, None] * N + rn[None, :], nl.dot(a, b))


def _one_tile_dot(dtype, m, n, k):
    def build(dev):
        a = _draw((m, k), 10, dtype)
        b = _draw((k, n), 11, dtype)
        c = torch.empty(m, n, device=dev)
        if dtype == torch.float32:       # tf32: 10 mantissa bits survive
            want, rtol, atol = a @ b, 5e-3, 5e-2
        else:
            want, rtol, atol = a.float() @ b.float(), 1e-4, 1e-4
        return (a.to(dev), b.to(dev), c), dict(M=m, N=n, K=k), [(c, want, rtol, atol)]
    return build


@newt.jit
def ragged_matmul(a_ptr, b_ptr, c_ptr, M, N, K, sam, sak, sbk, sbn, scm, scn,
                  BM: nl.constexpr, BN: nl.constexpr, BK: nl.constexpr):
    """A matmul whose row pitches no bulk tensor copy accepts (odd K and N): every load masked."""
    rm = nl.program_id(0) * BM + nl.arange(0, BM)
    rn = nl.program_id(1) * BN + nl.arange(0, BN)
    rk = nl.arange(0, BK)
    a_ptrs = a_ptr + rm[:, None] * sam + rk[None, :] * sak
    b_ptrs = b_ptr + rk[:, None] * sbk + rn[None, :] * sbn
    acc = nl.zeros((BM, BN), dtype=nl.float32)
    for k in range(0, nl.cdiv(K, BK)):
        left = K - k * BK
        a = nl.load(a_ptrs, mask=(rm[:, None] < M) & (rk[None, :] < left), other=0.0)
        b = nl.load(b_ptrs, mask=(rk[:, None] < left) & (rn[None, :] < N), other=0.0)
        acc = nl.dot(a, b, acc)
        a_ptrs += BK * sak
        b_ptrs += BK * sbk
    nl.store(c_ptr + rm[:, None] * scm + rn[None, :] * scn, acc.to(c_ptr.dtype.element_ty),
             mask=(rm[:, None] < M) & (rn[None, :] < N))


def _ragged_matmul(dev):
    m, n, k = 75, 51, 37
    a = _draw((m, k), 12, torch.float16)
    b = _draw((k, n), 13, torch.float16)
    c = torch.zeros(m, n, device=dev, dtype=torch.float16)
    want = (a.float() @ b.float()).half()
    args = (a.to(dev), b.to(dev), c, m, n, k, k, 1, n, 1, n, 1)
    return args, dict(BM=32, BN=32, BK=16), [(c, want, 2e-3, 2e-3)], (3, 2)


@newt.jit
def matmul_bias_relu(a_ptr, b_ptr, bias_ptr, c_ptr, M, N, K, BM: nl.constexpr, BN: nl.constexpr,
                     BK: nl.constexpr):
    """The epilogue (bias, activation) fused after the k loop."""
    rm = nl.program_id(0) * BM + nl.arange(0, BM)
    rn = nl.program_id(1) * BN + nl.arange(0, BN)
    rk = nl.arange(0, BK)
    acc = nl.zeros((BM, BN), dtype=nl.float32)
    for k in range(0, K, BK):
        a = nl.load(a_ptr + rm[:, None] * K + (k + rk)[None, :])
        b = nl.load(b_ptr + (k + rk)[:, None] * N + rn[None, :])
        acc = nl.dot(a, b, acc)
    bias = nl.load(bias_ptr + rn)
    out = nl.maximum(acc + bias[None, :], 0.0)
    nl.store(c_ptr + rm[:, None] * N + rn[None, :], out.to(nl.bfloat16))


def _matmul_bias_relu(dev):
    m, n, k = 64, 96, 64
    a = _draw((m, k), 14, torch.bfloat16)
    b = _draw((k, n), 15, torch.bfloat16)
    bias = _draw(n, 16)
    c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    want = torch.relu(a.float() @ b.float() + bias).bfloat16()
    return (a.to(dev), b.to(dev), bias.to(dev), c, m, n, k), dict(BM=32, BN=32, BK=32), \
        [(c, want, 1e-2, 1e-2)], (2, 3)


@newt.jit
def gram_matrix(a_ptr, c_ptr, M: nl.constexpr, K: nl.constexpr):
    """A^T A: the left operand is a transposed block."""
    rm = nl.arange(0, M)
    rk = nl.arange(0, K)
    a = nl.load(a_ptr + rk[:, None] * M + rm[None, :])       # [K, M]
    nl.store(c_ptr + rm[:, None] * M + rm[None, :], nl.dot(nl.trans(a), a))


def _gram_matrix(dev):
    m, k = 32, 64
    a = _draw((k, m), 17, torch.float16)
    c = torch.empty(m, m, device=dev)
    return (a.to(dev), c), dict(M=m, K=k), [(c, a.float().T @ a.float(), 1e-4, 1e-4)]


@newt.jit
def small_head_attention(q_ptr, k_ptr, v_ptr, o_ptr, S, scale, BM: nl.constexpr, BN: nl.constexpr,
                         D: nl.constexpr):
    """The flash-attention loop at a head size no tensor-core tile takes (D = 16): reductions,
    dots and carried blocks in one loop."""
    rm = nl.program_id(0) * BM + nl.arange(0, BM)
    rd = nl.arange(0, D)
    q = nl.load(q_ptr + rm[:, None] * D + rd[None, :])
    m_i = nl.full((BM,), -float("inf"), dtype=nl.float32)
    l_i = nl.zeros((BM,), dtype=nl.float32)
    acc = nl.zeros((BM, D), dtype=nl.float32)
    for start in range(0, S, BN):
        rn = start + nl.arange(0, BN)
        k = nl.load(k_ptr + rn[:, None] * D + rd[None, :])
        v = nl.load(v_ptr + rn[:, None] * D + rd[None, :])
        s = nl.dot(q, nl.trans(k)) * scale
        m_new = nl.maximum(m_i, nl.max(s, axis=1))
        alpha = nl.exp(m_i - m_new)
        p = nl.exp(s - m_new[:, None])
        l_i = l_i * alpha + nl.sum(p, axis=1)
        acc = nl.dot(p.to(nl.float16), v, acc * alpha[:, None])
        m_i = m_new
    nl.store(o_ptr + rm[:, None] * D + rd[None, :], (acc / l_i[:, None]).to(nl.float16))


def _small_head_attention(dev):
    s, d = 64, 16
    q = _draw((s, d), 18, torch.float16)
    k = _draw((s, d), 19, torch.float16)
    v = _draw((s, d), 20, torch.float16)
    o = torch.empty(s, d, device=dev, dtype=torch.float16)
    p = torch.softmax(q.float() @ k.float().T * 0.25, dim=-1)
    want = (p @ v.float()).half()
    return (q.to(dev), k.to(dev), v.to(dev), o, s, 0.25), dict(BM=16, BN=16, D=d), \
        [(o, want, 5e-3, 5e-3)], (4,)


# ---- names, pointers and masks across control flow ---------------------------------------------

@newt.jit
def last_value(x_ptr, y_ptr, n, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    for i in range(n):
        t = nl.load(x_ptr + offs) + i      # first bound inside the loop, read after it
    nl.store(y_ptr + offs, t)


def _last_value(dev):
    x = _draw(64, 30)
    y = torch.empty(64, device=dev)
    return (x.to(dev), y, 3), dict(BLOCK=64), [(y, x + 2, 0, 0)]


@newt.jit
def switch_source(a_ptr, b_ptr, out_ptr, n, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    p = a_ptr + offs
    for i in range(n):
        nl.store(out_ptr + i * BLOCK + offs, nl.load(p))
        p = b_ptr + offs                   # a carried pointer block that changes its tensor


def _switch_source(dev):
    a = _draw(64, 31)
    b = _draw(64, 32)
    out = torch.empty(192, device=dev)
    return (a.to(dev), b.to(dev), out, 3), dict(BLOCK=64), [(out, torch.cat([a, b, b]), 0, 0)]


@newt.jit
def count_large(x_ptr, y_ptr, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    big = nl.load(x_ptr + offs) > 100.0
    nl.store(y_ptr, nl.max(big).to(nl.int32))
    nl.store(y_ptr + 1, nl.sum(big).to(nl.int32))


def _count_large(dev):
    x = torch.zeros(256)
    x[[3, 77, 130, 255]] = 500.0
    y = torch.empty(2, device=dev, dtype=torch.int32)
    return (x.to(dev), y), dict(BLOCK=256), [(y, torch.tensor([1, 4], dtype=torch.int32), 0, 0)]


@newt.jit
def any_and_all(x_ptr, y_ptr, BLOCK: nl.constexpr):
    """max of booleans is "any", min is "all": the folds must start from false and true."""
    offs = nl.arange(0, BLOCK)
    v = nl.load(x_ptr + offs)
    nl.store(y_ptr, nl.max(v > 100.0).to(nl.int32))       # nothing is: 0
    nl.store(y_ptr + 1, nl.sum(v > 100.0).to(nl.int32))   # ... counted: 0
    nl.store(y_ptr + 2, nl.min(v < 100.0).to(nl.int32))   # everything is: 1
    nl.store(y_ptr + 3, nl.min(v > -1.0).to(nl.int32))    # one is not: 0


def _any_and_all(dev):
    x = torch.zeros(256)
    x[200] = -5.0
    y = torch.full((4,), 7, device=dev, dtype=torch.int32)
    return (x.to(dev), y), dict(BLOCK=256), [(y, torch.tensor([0, 0, 1, 0], dtype=torch.int32), 0, 0)]


@newt.jit
def bound_in_both_arms(x_ptr, y_ptr, flag, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    if flag == 1:
        t = nl.load(x_ptr + offs) * 2
    else:
        t = nl.load(x_ptr + offs) * 3
    nl.store(y_ptr + offs, t)


def _bound_in_both_arms(flag):
    def build(dev):
        x = _draw(64, 33)
        y = torch.empty(64, device=dev)
        return (x.to(dev), y, flag), dict(BLOCK=64), [(y, x * (2 if flag == 1 else 3), 0, 0)]
    return build


@newt.jit
def fill_from_other_tensor(p_ptr, q_ptr, y_ptr, n, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    spare = nl.load(q_ptr + offs)
    nl.store(y_ptr + offs, nl.load(p_ptr + offs, mask=offs < n, other=spare))


def _fill_from_other_tensor(dev):
    p = _draw(64, 34)
    q = _draw(64, 35)
    y = torch.empty(64, device=dev)
    want = torch.where(torch.arange(64) < 9, p, q)
    return (p.to(dev), q.to(dev), y, 9), dict(BLOCK=64), [(y, want, 0, 0)]


@newt.jit
def small_types(a_ptr, h_ptr, oa_ptr, oh_ptr, BLOCK: nl.constexpr):
    offs = nl.arange(0, BLOCK)
    nl.store(oa_ptr + offs, nl.load(a_ptr + offs) + 200)     # the constant becomes uint8: wraps
    nl.store(oh_ptr + offs, nl.load(h_ptr + offs) * 0.1)     # the constant becomes fp16


def _small_types(dev):
    a = torch.arange(64, dtype=torch.uint8) * 3
    h = _draw(64, 36, torch.float16)
    oa = torch.empty(64, device=dev, dtype=torch.uint8)
    oh = torch.empty(64, device=dev, dtype=torch.float32)
    want_h = (h * torch.tensor(0.1, dtype=torch.float16)).float()
    return (a.to(dev), h.to(dev), oa, oh), dict(BLOCK=64), [(oa, a + 200, 0, 0), (oh, want_h, 0, 0)]


@newt.jit
def two_phase_accumulate(a_ptr, b_ptr, o_ptr, K, full, tail, BM: nl.constexpr, BN: nl.constexpr,
                         BK: nl.constexpr):
    """Whole k-blocks in one loop, the masked remainder in a second one on the same accumulator
    and the same walked pointers; the second loop may run zero times."""
    rm = nl.arange(0, BM)
    rn = nl.arange(0, BN)
    rk = nl.arange(0, BK)
    a_ptrs = a_ptr + rm[:, None] * K + rk[None, :]
    b_ptrs = b_ptr + rk[:, None] * BN + rn[None, :]
    acc = nl.zeros((BM, BN), dtype=nl.float32)
    for _ in range(full):
        acc = nl.dot(nl.load(a_ptrs), nl.load(b_ptrs), acc)
        a_ptrs += BK
        b_ptrs += BK * BN
    for t in range(tail):
        live = (t * BK + rk) < (K - full * BK)
        acc = nl.dot(nl.load(a_ptrs, mask=live[None, :], other=0.0),
                     nl.load(b_ptrs, mask=live[:, None], other=0.0), acc)
    nl.store(o_ptr + rm[:, None] * BN + rn[None, :], acc)


def _two_phase_accumulate(k):
    def build(dev):
        bm, bn, bk = 32, 32, 16
        a = _draw((bm, k), 40, torch.float16, 0.3)
        b = _draw((k, bn), 41, torch.float16, 0.3)
        o = torch.empty(bm, bn, device=dev)
        full, tail = k // bk, 1 if k % bk else 0
        return (a.to(dev), b.to(dev), o, k, full, tail), dict(BM=bm, BN=bn, BK=bk), \
            [(o, a.float() @ b.float(), 1e-4, 1e-4)]
    return build


@newt.jit
def logging_k_loop(a_ptr, b_ptr, o_ptr, log_ptr, K, BM: nl.constexpr, BN: nl.constexpr,
                   BK: nl.constexpr):
    """A store inside the k loop next to the dot: the loop runs block-wide, the accumulator
    lives in shared memory."""
    rm = nl.arange(0, BM)
    rn = nl.arange(0, BN)
    rk = nl.arange(0, BK)
    a_ptrs = a_ptr + rm[:, None] * K + rk[None, :]
    b_ptrs = b_ptr + rk[:, None] * BN + rn[None, :]
    acc = nl.zeros((BM, BN), dtype=nl.float32)
    for i in range(K // BK):
        acc = nl.dot(nl.load(a_ptrs), nl.load(b_ptrs), acc)
        nl.store(log_ptr + i * BM + rm, rm.to(nl.float32) + i)
        a_ptrs += BK
        b_ptrs += BK * BN
    nl.store(o_ptr + rm[:, None] * BN + rn[None, :], acc)


def _logging_k_loop(dev):
    bm, bn, bk, k = 32, 32, 16, 64
    a = _draw((bm, k), 42, torch.float16, 0.3)
    b = _draw((k, bn), 43, torch.float16, 0.3)
    o = torch.empty(bm, bn, device=dev)
    log = torch.zeros(k // bk * bm, device=dev)
    want_log = (torch.arange(bm).float()[None, :] + torch.arange(k // bk).float()[:, None]).reshape(-1)
    return (a.to(dev), b.to(dev), o, log, k), dict(BM=bm, BN=bn, BK=bk), \
        [(o, a.float() @ b.float(), 1e-4, 1e-4), (log, want_log, 0, 0)]


@newt.jit
def dot_row_sums(a_ptr, b_ptr, o_ptr, M: nl.constexpr, N: nl.constexpr, K: nl.constexpr):
    """A dot whose result goes through elementwise arithmetic and a reduction before the store."""
    rm = nl.arange(0, M)
    rn = nl.arange(0, N)
    rk = nl.arange(0, K)
    a = nl.load(a_ptr + rm[:, None] * K + rk[None, :])
    b = nl.load(b_ptr + rk[:, None] * N + rn[None, :])
    c = nl.dot(a, b) * 2.0 + 1.0
    nl.store(o_ptr + rm, nl.sum(c, axis=1))


def _dot_row_sums(dev):
    m, n, k = 32, 64, 32
    a = _draw((m, k), 44, torch.float16, 0.3)
    b = _draw((k, n), 45, torch.float16, 0.3)
    o = torch.empty(m, device=dev)
    return (a.to(dev), b.to(dev), o), dict(M=m, N=n, K=k), \
        [(o, (a.float() @ b.float() * 2 + 1).sum(1), 1e-4, 1e-4)]


# ---- launch geometry and compile-time constructs ------------------------------------------------

@newt.jit
def grid_coordinates(o_ptr, BLOCK: nl.constexpr):
    """Three grid axes and their extents: program (x, y, z) writes its linear index."""
    x, y, z = nl.program_id(0), nl.program_id(1), nl.program_id(2)
    nx, ny = nl.num_programs(0), nl.num_programs(1)
    lin = (z * ny + y) * nx + x
    offs = nl.arange(0, BLOCK)
    nl.store(o_ptr + lin * BLOCK + offs, nl.zeros((BLOCK,), dtype=nl.int32) + lin * 10 + nl.num_programs(2))


def _grid_coordinates(dev):
    gx, gy, gz, block = 3, 4, 2, 32
    o = torch.full((gx * gy * gz * block,), -1, device=dev, dtype=torch.int32)
    want = (torch.arange(gx * gy * gz, dtype=torch.int32) * 10 + gz).repeat_interleave(block)
    return (o,), dict(BLOCK=block), [(o, want, 0, 0)], (gx, gy, gz)


@newt.jit
def chosen_at_compile_time(x_ptr, o_ptr, n, MODE: nl.constexpr, BLOCK: nl.constexpr):
    """A constexpr branch is pruned: the arm not taken is never traced (it would not lower),
    a tuple assignment unpacks, a block smaller than the thread count leaves threads idle."""
    nl.static_assert(BLOCK >= 16, "BLOCK too small")
    offs, ok = nl.arange(0, BLOCK), nl.arange(0, BLOCK) < n
    x = nl.load(x_ptr + offs, mask=ok)
    if MODE == "triple":
        y = x * 3
    else:
        y = nl.no_such_function(x)
    nl.store(o_ptr + offs, y, mask=ok)


def _chosen_at_compile_time(n, block, warps):
    def build(dev):
        x = _draw(block, 50)
        o = torch.full((block,), 5.0, device=dev)
        want = torch.full((block,), 5.0)
        want[:n] = x[:n] * 3
        return (x.to(dev), o, n), dict(MODE="triple", BLOCK=block, num_warps=warps), [(o, want, 0, 0)]
    return build


CASES = {
    "weighted_tiles": (weighted_tiles, _weighted_tiles),
    "sum_of_cubes": (sum_of_cubes, _sum_of_cubes),
    "strided_range": (strided_range, _strided_range),
    "nested_products": (nested_products, _nested_products),
    "next_power": (next_power, _next_power),
    "capped_growth": (capped_growth, _capped_growth),
    "skipping": (skipping, _skipping),
    "two_way_then": (two_way, _two_way(1)),
    "two_way_else": (two_way, _two_way(0)),
    "two_way_both": (two_way, _two_way(9)),
    "last_value": (last_value, _last_value),
    "switch_source": (switch_source, _switch_source),
    "count_large": (count_large, _count_large),
    "any_and_all": (any_and_all, _any_and_all),
    "bound_in_both_arms_then": (bound_in_both_arms, _bound_in_both_arms(1)),
    "bound_in_both_arms_else": (bound_in_both_arms, _bound_in_both_arms(0)),
    "fill_from_other_tensor": (fill_from_other_tensor, _fill_from_other_tensor),
    "small_types": (small_types, _small_types),
    "grid_coordinates": (grid_coordinates, _grid_coordinates),
    "pruned_branch_tiny_block": (chosen_at_compile_time, _chosen_at_compile_time(16, 16, 4)),
    "pruned_branch_one_element": (chosen_at_compile_time, _chosen_at_compile_time(1, 64, 1)),
    "scale_tiles": (scale_tiles, _scale_tiles),
    "running_softmax_stats": (running_softmax_stats, _running_softmax_stats),
    "tiled_layernorm": (tiled_layernorm, _tiled_layernorm),
    "power_iteration": (power_iteration, _power_iteration),
    "dot_16x16x16_f16": (one_tile_dot, _one_tile_dot(torch.float16, 16, 16, 16)),
    "dot_32x16x64_bf16": (one_tile_dot, _one_tile_dot(torch.bfloat16, 32, 16, 64)),
    "dot_16x32x8_tf32": (one_tile_dot, _one_tile_dot(torch.float32, 16, 32, 8)),
    "ragged_matmul": (ragged_matmul, _ragged_matmul),
    "matmul_bias_relu": (matmul_bias_relu, _matmul_bias_relu),
    "gram_matrix": (gram_matrix, _gram_matrix),
    "dot_row_sums": (dot_row_sums, _dot_row_sums),
    "two_phase_accumulate_no_tail": (two_phase_accumulate, _two_phase_accumulate(48)),
    "two_phase_accumulate_tail": (two_phase_accumulate, _two_phase_accumulate(40)),
    "logging_k_loop": (logging_k_loop, _logging_k_loop),
    "small_head_attention": (small_head_attention, _small_head_attention),
}


def build(name, device):
    """(kernel, grid, args, meta, checks) of a case."""
    kernel, make = CASES[name]
    made = make(device)
    args, meta, checks = made[:3]
    grid = made[3] if len(made) > 3 else (1,)
    return kernel, grid, args, meta, checks
