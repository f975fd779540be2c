"""The block language outside the five tuned programs, on the device: every operator family
the reference's operator tests exercise (tests/test_ops.py: binary, integer, unary, casts,
reductions along an axis and over a whole block, broadcasting, reshape, transpose, strided and
gathered loads, loads through a scalar pointer), here through the generic lowering
(frontend/pointwise.py) and checked against torch on the CPU.

Bars: bit-exact where the result is one correctly rounded operation or pure data movement;
rtol 2e-6 for the single-precision math functions; rtol 1e-5 for sums (the fold order differs
from torch's)."""

import pytest
import torch

import newt_b200 as newt
import newt_b200.language as nl
from newt_b200.runtime import abi

pytestmark = pytest.mark.gpu


def _draw(shape, seed, dtype=torch.float32, positive=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    return (x.abs() + 0.1 if positive else x).to(dtype)


@newt.jit
def two_operand(a_ptr, b_ptr, out_ptr, n, WHAT: nl.constexpr, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    ok = i < n
    a = nl.load(a_ptr + i, mask=ok)
    b = nl.load(b_ptr + i, mask=ok, other=1.0)
    if WHAT == "a+b":
        r = a + b
    elif WHAT == "a-b":
        r = a - b
    elif WHAT == "a*b":
        r = a * b
    elif WHAT == "a/b":
        r = a / b
    elif WHAT == "a**2":
        r = a ** 2
    elif WHAT == "max":
        r = nl.maximum(a, b)
    elif WHAT == "min":
        r = nl.minimum(a, b)
    elif WHAT == "fma":
        r = nl.fma(a, b, a)
    elif WHAT == "where":
        r = nl.where(a > 0, a, b)
    elif WHAT == "scaled":
        r = a * 0.1 + 3      # Python constants take the block's dtype
    nl.store(out_ptr + i, r, mask=ok)


TWO_OPERAND = {
    "a+b": lambda a, b: a + b, "a-b": lambda a, b: a - b, "a*b": lambda a, b: a * b,
    "a/b": lambda a, b: a / b, "a**2": lambda a, b: a * a, "max": torch.maximum,
    "min": torch.minimum, "where": lambda a, b: torch.where(a > 0, a, b),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("what", list(TWO_OPERAND))
def test_two_operand_ops_are_correctly_rounded(what, dtype):
    n = 3000
    a, b = _draw((n,), 1, dtype), _draw((n,), 2, dtype, positive=True)
    out = torch.full((n,), float("nan"), device="cuda", dtype=dtype)
    two_operand[(newt.cdiv(n, 512),)](a.cuda(), b.cuda(), out, n, WHAT=what, BLOCK=512)
    torch.cuda.synchronize()
    # one fp32 operation rounded once to the block's dtype: what torch computes on the CPU
    assert torch.equal(out.cpu(), TWO_OPERAND[what](a, b))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_fma_and_constants(dtype):
    n = 1000
    a, b = _draw((n,), 3, dtype), _draw((n,), 4, dtype)
    out = torch.empty(n, device="cuda", dtype=dtype)
    two_operand[(2,)](a.cuda(), b.cuda(), out, n, WHAT="fma", BLOCK=512)
    tenth = torch.tensor(0.1, dtype=dtype)          # 0.1 rounded to the block's dtype first
    if dtype == torch.float16:
        # 16-bit blocks: a multiply and an add, each rounded to the block's dtype
        assert torch.equal(out.cpu(), ((a * b) + a))
        two_operand[(2,)](a.cuda(), b.cuda(), out, n, WHAT="scaled", BLOCK=512)
        assert torch.equal(out.cpu(), (a * tenth) + torch.tensor(3, dtype=dtype))
    else:
        # fp32: the compiler may contract the pair into one fused multiply-add, as it may in
        # the reference's generated code (same NVRTC defaults): fused or not, within an ulp
        torch.testing.assert_close(out.cpu().double(), a.double() * b.double() + a.double(),
                                   rtol=3e-7, atol=1e-7)
        two_operand[(2,)](a.cuda(), b.cuda(), out, n, WHAT="scaled", BLOCK=512)
        torch.testing.assert_close(out.cpu().double(), a.double() * tenth.double() + 3.0,
                                   rtol=3e-7, atol=1e-7)


@newt.jit
def integer_ops(a_ptr, b_ptr, out_ptr, n, WHAT: nl.constexpr, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    ok = i < n
    a = nl.load(a_ptr + i, mask=ok)
    b = nl.load(b_ptr + i, mask=ok, other=1)
    if WHAT == "and":
        r = a & b
    elif WHAT == "or":
        r = a | b
    elif WHAT == "xor":
        r = a ^ b
    elif WHAT == "shifts":
        r = (a << 2) + (b >> 1)
    elif WHAT == "mod":
        r = a % b
    elif WHAT == "floordiv":
        r = a // b
    elif WHAT == "neg_abs":
        r = nl.abs(-a) - b
    nl.store(out_ptr + i, r, mask=ok)


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
@pytest.mark.parametrize("what,ref", [
    ("and", lambda a, b: a & b), ("or", lambda a, b: a | b), ("xor", lambda a, b: a ^ b),
    ("shifts", lambda a, b: (a << 2) + (b >> 1)),
    ("mod", lambda a, b: torch.fmod(a, b)),                                   # C semantics
    ("floordiv", lambda a, b: torch.div(a, b, rounding_mode="trunc")),        # C semantics
    ("neg_abs", lambda a, b: a.abs() - b)])
def test_integer_ops(what, ref, dtype):
    n = 2000
    g = torch.Generator().manual_seed(5)
    a = torch.randint(-5000, 5000, (n,), generator=g, dtype=dtype)
    b = torch.randint(1, 97, (n,), generator=g, dtype=dtype)
    out = torch.zeros(n, device="cuda", dtype=dtype)
    integer_ops[(newt.cdiv(n, 256),)](a.cuda(), b.cuda(), out, n, WHAT=what, BLOCK=256)
    assert torch.equal(out.cpu(), ref(a, b))


@newt.jit
def one_operand(x_ptr, out_ptr, n, FN: nl.constexpr, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    ok = i < n
    x = nl.load(x_ptr + i, mask=ok, other=1.0)
    if FN == "exp":
        r = nl.exp(x)
    elif FN == "exp2":
        r = nl.exp2(x)
    elif FN == "log":
        r = nl.log(x)
    elif FN == "log2":
        r = nl.log2(x)
    elif FN == "sqrt":
        r = nl.sqrt(x)
    elif FN == "rsqrt":
        r = nl.rsqrt(x)
    elif FN == "sin":
        r = nl.sin(x)
    elif FN == "cos":
        r = nl.cos(x)
    elif FN == "tanh":
        r = nl.tanh(x)
    elif FN == "erf":
        r = nl.erf(x)
    elif FN == "sigmoid":
        r = nl.sigmoid(x)
    elif FN == "abs":
        r = nl.abs(x)
    elif FN == "floor":
        r = nl.floor(x)
    elif FN == "ceil":
        r = nl.ceil(x)
    elif FN == "neg":
        r = -x
    nl.store(out_ptr + i, r, mask=ok)


ONE_OPERAND = {"exp": torch.exp, "exp2": torch.exp2, "log": torch.log, "log2": torch.log2,
               "sqrt": torch.sqrt, "rsqrt": torch.rsqrt, "sin": torch.sin, "cos": torch.cos,
               "tanh": torch.tanh, "erf": torch.erf, "sigmoid": torch.sigmoid, "abs": torch.abs,
               "floor": torch.floor, "ceil": torch.ceil, "neg": torch.neg}


@pytest.mark.parametrize("fn", list(ONE_OPERAND))
def test_one_operand_functions(fn):
    n = 4097
    x = _draw((n,), 6, positive=fn in ("log", "log2", "sqrt", "rsqrt")) * 3
    out = torch.full((n,), float("nan"), device="cuda")
    one_operand[(newt.cdiv(n, 1024),)](x.cuda(), out, n, FN=fn, BLOCK=1024, num_warps=8)
    want = ONE_OPERAND[fn](x.double())
    if fn in ("abs", "floor", "ceil", "neg", "sqrt"):
        assert torch.equal(out.cpu().double(), want.float().double())
    else:
        torch.testing.assert_close(out.cpu().double(), want, rtol=2e-6, atol=1e-7)
    # 16-bit blocks: the function in fp32, rounded once
    xh = x.half()
    outh = torch.empty(n, device="cuda", dtype=torch.float16)
    one_operand[(newt.cdiv(n, 1024),)](xh.cuda(), outh, n, FN=fn, BLOCK=1024)
    wanth = ONE_OPERAND[fn](xh.float()).half()     # overflows to inf where the device's does
    torch.testing.assert_close(outh.cpu().float(), wanth.float(), rtol=2e-3, atol=1e-6)


@newt.jit
def convert(x_ptr, out_ptr, n, TO: nl.constexpr, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    nl.store(out_ptr + i, nl.load(x_ptr + i, mask=i < n).to(TO), mask=i < n)


@pytest.mark.parametrize("src,dst,to", [
    (torch.float32, torch.float16, nl.float16), (torch.float16, torch.float32, nl.float32),
    (torch.float32, torch.bfloat16, nl.bfloat16), (torch.bfloat16, torch.float16, nl.float16),
    (torch.float32, torch.int32, nl.int32), (torch.int32, torch.float32, nl.float32),
    (torch.int64, torch.int32, nl.int32), (torch.int32, torch.float16, nl.float16)])
def test_casts(src, dst, to):
    n = 1500
    x = (_draw((n,), 7) * 50).to(src)
    out = torch.zeros(n, device="cuda", dtype=dst)
    convert[(newt.cdiv(n, 512),)](x.cuda(), out, n, TO=to, BLOCK=512)
    assert torch.equal(out.cpu(), x.to(dst))


@newt.jit
def reduce_tile(x_ptr, out_ptr, M, N, sx, HOW: nl.constexpr, AXIS: nl.constexpr,
                BM: nl.constexpr, BN: nl.constexpr):
    r = nl.arange(0, BM)
    c = nl.arange(0, BN)
    inside = (r[:, None] < M) & (c[None, :] < N)
    if HOW == "sum":
        v = nl.sum(nl.load(x_ptr + r[:, None] * sx + c[None, :], mask=inside, other=0.0), axis=AXIS)
    elif HOW == "max":
        v = nl.max(nl.load(x_ptr + r[:, None] * sx + c[None, :], mask=inside, other=float("-inf")),
                   axis=AXIS)
    else:
        v = nl.min(nl.load(x_ptr + r[:, None] * sx + c[None, :], mask=inside, other=float("inf")),
                   axis=AXIS)
    if AXIS == 0:
        nl.store(out_ptr + c, v, mask=c < N)
    else:
        nl.store(out_ptr + r, v, mask=r < M)


@pytest.mark.parametrize("how", ["sum", "max", "min"])
@pytest.mark.parametrize("axis", [0, 1])
@pytest.mark.parametrize("m,n,bm,bn", [(32, 64, 32, 64), (17, 100, 32, 128), (128, 128, 128, 128),
                                       (3, 600, 4, 1024)])
def test_reduce_along_an_axis(how, axis, m, n, bm, bn):
    x = _draw((m, n), 8)
    out = torch.full((n if axis == 0 else m,), float("nan"), device="cuda")
    reduce_tile[(1,)](x.cuda(), out, m, n, n, HOW=how, AXIS=axis, BM=bm, BN=bn)
    if how == "sum":
        torch.testing.assert_close(out.cpu(), x.sum(axis), rtol=1e-5, atol=1e-5)
    else:
        want = x.max(axis).values if how == "max" else x.min(axis).values
        assert torch.equal(out.cpu(), want)


@newt.jit
def reduce_block(x_ptr, out_ptr, n, HOW: nl.constexpr, BLOCK: nl.constexpr):
    i = nl.arange(0, BLOCK)
    if HOW == "sum":
        nl.store(out_ptr, nl.sum(nl.load(x_ptr + i, mask=i < n, other=0.0)))
    else:
        nl.store(out_ptr, nl.max(nl.load(x_ptr + i, mask=i < n, other=float("-inf"))))


@pytest.mark.parametrize("how", ["sum", "max"])
@pytest.mark.parametrize("n,block", [(32, 32), (100, 128), (1024, 1024), (5000, 8192)])
@pytest.mark.parametrize("warps", [1, 4, 8])
def test_reduce_a_whole_block(how, n, block, warps):
    x = _draw((n,), 9)
    out = torch.full((1,), float("nan"), device="cuda")
    reduce_block[(1,)](x.cuda(), out, n, HOW=how, BLOCK=block, num_warps=warps)
    if how == "sum":
        torch.testing.assert_close(out.cpu()[0], x.sum(), rtol=1e-5, atol=1e-4)
    else:
        assert out.cpu()[0] == x.max()


def test_sum_of_fp16_accumulates_in_fp32():
    # 4096 halves of 0.25 sum to 1024 in fp32; in fp16 the running sum would stall at 512
    x = torch.full((4096,), 0.25, dtype=torch.float16)
    out = torch.zeros(1, device="cuda")
    reduce_block[(1,)](x.cuda(), out, 4096, HOW="sum", BLOCK=4096)
    assert out.item() == 1024.0


@newt.jit
def outer_scaled(a_ptr, b_ptr, out_ptr, BM: nl.constexpr, BN: nl.constexpr):
    a = nl.load(a_ptr + nl.arange(0, BM))
    b = nl.load(b_ptr + nl.arange(0, BN))
    where = nl.arange(0, BM)[:, None] * BN + nl.arange(0, BN)[None, :]
    nl.store(out_ptr + where, a[:, None] * 100 + b[None, :])


@newt.jit
def repeat_rows(a_ptr, out_ptr, BM: nl.constexpr, BN: nl.constexpr):
    a = nl.load(a_ptr + nl.arange(0, BM))
    wide = nl.broadcast_to(a[:, None], (BM, BN))
    nl.store(out_ptr + nl.arange(0, BM * BN), nl.reshape(wide, (BM * BN,)))


@newt.jit
def transpose_tile(x_ptr, out_ptr, BM: nl.constexpr, BN: nl.constexpr):
    src = nl.arange(0, BM)[:, None] * BN + nl.arange(0, BN)[None, :]
    dst = nl.arange(0, BN)[:, None] * BM + nl.arange(0, BM)[None, :]
    nl.store(out_ptr + dst, nl.trans(nl.load(x_ptr + src)))


def test_broadcast_reshape_transpose():
    a, b = _draw((32,), 10), _draw((64,), 11)
    out = torch.empty(32, 64, device="cuda")
    outer_scaled[(1,)](a.cuda(), b.cuda(), out, BM=32, BN=64)
    # (a * 100 + b may be one fused multiply-add)
    torch.testing.assert_close(out.cpu().double(), a.double()[:, None] * 100 + b.double()[None, :],
                               rtol=3e-7, atol=1e-7)
    flat = torch.empty(16 * 32, device="cuda")
    repeat_rows[(1,)](a[:16].cuda(), flat, BM=16, BN=32)
    assert torch.equal(flat.cpu().view(16, 32), a[:16, None].expand(16, 32))
    x = _draw((32, 64), 12)
    xt = torch.empty(64, 32, device="cuda")
    transpose_tile[(1,)](x.cuda(), xt, BM=32, BN=64)
    assert torch.equal(xt.cpu(), x.t())


@newt.jit
def strided_double(x_ptr, out_ptr, n, step, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    nl.store(out_ptr + i, nl.load(x_ptr + i * step, mask=i < n) * 2, mask=i < n)


@newt.jit
def gather(x_ptr, idx_ptr, out_ptr, n, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    which = nl.load(idx_ptr + i, mask=i < n)
    nl.store(out_ptr + i, nl.load(x_ptr + which, mask=i < n), mask=i < n)


@newt.jit
def add_scalar_from_memory(s_ptr, out_ptr, BLOCK: nl.constexpr):
    s = nl.load(s_ptr)       # one value for the whole program
    nl.store(out_ptr + nl.arange(0, BLOCK), nl.zeros((BLOCK,), dtype=nl.float32) + s)


def test_strided_gathered_and_scalar_loads():
    base = _draw((2000,), 13)
    n = 1000
    out = torch.empty(n, device="cuda")
    strided_double[(newt.cdiv(n, 256),)](base.cuda(), out, n, 2, BLOCK=256)
    assert torch.equal(out.cpu(), base[::2] * 2)
    x = _draw((4096,), 14)
    idx = torch.randperm(4096, generator=torch.Generator().manual_seed(15)).to(torch.int32)
    got = torch.empty(4096, device="cuda")
    gather[(4,)](x.cuda(), idx.cuda(), got, 4096, BLOCK=1024)
    assert torch.equal(got.cpu(), x[idx.long()])
    o = torch.empty(128, device="cuda")
    add_scalar_from_memory[(1,)](torch.tensor([42.0], device="cuda"), o, BLOCK=128)
    torch.cuda.synchronize()
    assert torch.all(o == 42.0) and abi.read_status() == (0, 0)


@newt.jit
def histogram(idx_ptr, hist_ptr, n, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    which = nl.load(idx_ptr + i, mask=i < n)
    nl.atomic_add(hist_ptr + which, 1.0, mask=i < n)


@newt.jit
def running_max(x_ptr, out_ptr, n, BLOCK: nl.constexpr):
    i = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
    nl.atomic_max(out_ptr, nl.max(nl.load(x_ptr + i, mask=i < n, other=0)))   # one update per program


def test_atomics():
    n, bins = 100_000, 64
    g = torch.Generator().manual_seed(16)
    idx = torch.randint(0, bins, (n,), generator=g, dtype=torch.int32)
    hist = torch.zeros(bins, device="cuda")
    histogram[(newt.cdiv(n, 1024),)](idx.cuda(), hist, n, BLOCK=1024)
    assert torch.equal(hist.cpu(), torch.bincount(idx.long(), minlength=bins).float())
    x = torch.randint(0, 1_000_000, (10_000,), generator=g, dtype=torch.int32)
    top = torch.zeros(1, device="cuda", dtype=torch.int32)
    running_max[(newt.cdiv(10_000, 1024),)](x.cuda(), top, 10_000, BLOCK=1024)
    assert top.item() == x.max().item()
    xf = _draw((10_000,), 17)
    topf = torch.full((1,), float("-inf"), device="cuda")
    running_max[(newt.cdiv(10_000, 1024),)](xf.cuda(), topf, 10_000, BLOCK=1024)
    assert topf.item() == max(xf.max().item(), 0.0)       # masked lanes read 0
