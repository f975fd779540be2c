"""Benchmark suite over the sizes the reference publishes (benchmarks/bench.py:170-300 and
benchmarks/results.md of the reference): vector add, fused softmax, layernorm, fp16 matmul,
fp32/tf32 matmul, plus causal attention, each next to the torch call on the same tensors.

    python -m newt_b200.examples.suite [--quick] [--kernel add|fused|softmax|layernorm|rows|matmul|matmul_long_k|matmul_tf32|matmul_epilogue|attention]

Clock and metric definitions are the reference's: `do_bench` (median, L2 flushed between
reps); GB/s = bytes read + written / t; TFLOP/s = 2*M*N*K / t.  Prints markdown tables.
"""

import argparse
import time

import torch

from .. import testing
from . import kernels as K


def _bench(fn, **kw):
    """`do_bench` from an idle chip: after seconds under the 1 kW power cap the clocks stay
    low for a while, and a small problem measured right behind a large one reads 30 % low."""
    torch.cuda.synchronize()
    time.sleep(0.5)
    return testing.do_bench(fn, **kw)


def _row(name, size, ours_ms, torch_ms, unit_per_ms):
    ours, ref = unit_per_ms / ours_ms, unit_per_ms / torch_ms
    return f"| {name} | {size} | {ours:.1f} | {ref:.1f} | {ours / ref:.2f} |"


def bench_add(quick):
    out = ["| kernel | n | newt_b200 GB/s | torch GB/s | ratio |", "|---|---|---|---|---|"]
    for n in ([1 << 20, 1 << 24] if quick else [1 << 20, 1 << 24, 1 << 26, 1 << 27]):
        x, y = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        o = torch.empty_like(x)
        a = _bench(lambda: K.add(x, y, o))
        b = _bench(lambda: torch.add(x, y, out=o))
        out.append(_row("add fp32", n, a, b, 3 * n * 4 / 1e6))
    return out


def bench_fused(quick):
    """gelu(x) + y in one generated kernel against the two torch launches
    (examples/deuteron/04_fused_ops.py); bytes = 3 * n * 4."""
    out = ["| kernel | n | newt_b200 GB/s | torch GB/s | ratio |", "|---|---|---|---|---|"]
    for n in ([1 << 22, 1 << 26] if quick else [1 << 20, 1 << 22, 1 << 24, 1 << 26]):
        x, y = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
        o = torch.empty_like(x)
        a = _bench(lambda: K.gelu_residual(x, y, o))
        b = _bench(lambda: torch.add(torch.nn.functional.gelu(x, approximate="tanh"), y, out=o))
        out.append(_row("gelu+residual fp32", n, a, b, 3 * n * 4 / 1e6))
    n = 1 << 26                # 16-bit blocks move sixteen bytes per access
    for dt in (torch.float16, torch.bfloat16):
        x, y = torch.randn(n, device="cuda").to(dt), torch.randn(n, device="cuda").to(dt)
        o = torch.empty_like(x)
        a = _bench(lambda: K.gelu_residual(x, y, o))
        b = _bench(lambda: torch.add(torch.nn.functional.gelu(x, approximate="tanh"), y, out=o))
        out.append(_row(f"gelu+residual {str(dt)[6:]}", n, a, b, 3 * n * 2 / 1e6))
    return out


def bench_softmax(quick):
    out = ["| kernel | M x N | newt_b200 GB/s | torch GB/s | ratio |", "|---|---|---|---|---|"]
    for n in ([1024, 4096] if quick else [1024, 4096, 8192, 16384]):
        x = torch.randn(4096, n, device="cuda")
        o = torch.empty_like(x)
        a = _bench(lambda: K.softmax(x, o))
        b = _bench(lambda: torch.softmax(x, -1, out=o))
        out.append(_row("softmax fp32", f"4096x{n}", a, b, 2 * 4096 * n * 4 / 1e6))
    return out


def bench_layernorm(quick):
    out = ["| kernel | M x N | newt_b200 GB/s | torch GB/s | ratio |", "|---|---|---|---|---|"]
    cases = [(torch.float32, 4096, n) for n in ([1024, 4096] if quick else [1024, 2048, 4096, 8192])]
    cases.append((torch.float16, 8192, 4096))
    for dt, m, n in cases:
        x = torch.randn(m, n, device="cuda").to(dt)
        w, b_ = torch.randn(n, device="cuda").to(dt), torch.randn(n, device="cuda").to(dt)
        o = torch.empty_like(x)
        a = _bench(lambda: K.layernorm(x, w, b_, 1e-5, o))
        b = _bench(lambda: torch.nn.functional.layer_norm(x, (n,), w, b_, 1e-5))
        out.append(_row(f"layernorm {str(dt)[6:]}", f"{m}x{n}", a, b, 2 * m * n * x.element_size() / 1e6))
    return out


def bench_rows(quick):
    """Rows of the softmax / layernorm family that the tuned kernels do not recognise, through
    the generic lowering (a row kept in registers), against torch's fused calls."""
    out = ["| kernel | M x N | newt_b200 GB/s | torch GB/s | ratio |", "|---|---|---|---|---|"]
    for n in ([4096] if quick else [1024, 4096, 8192]):
        x = torch.randn(4096, n, device="cuda")
        o = torch.empty_like(x)
        gb = 2 * 4096 * n * 4 / 1e6
        a = _bench(lambda: K.softmax_temperature(x, 2.0, o))
        b = _bench(lambda: torch.softmax(x * 0.5, -1, out=o))
        out.append(_row("softmax(x / T) fp32", f"4096x{n}", a, b, gb))
        a = _bench(lambda: K.log_softmax(x, o))
        b = _bench(lambda: torch.log_softmax(x, -1, out=o))
        out.append(_row("log_softmax fp32", f"4096x{n}", a, b, gb))
    for dt in (torch.float16, torch.bfloat16):
        x = torch.randn(8192, 4096, device="cuda").to(dt)
        w = torch.randn(4096, device="cuda").to(dt)
        o = torch.empty_like(x)
        a = _bench(lambda: K.rmsnorm(x, w, 1e-6, o))
        b = _bench(lambda: torch.nn.functional.rms_norm(x, (4096,), w, 1e-6))
        out.append(_row(f"rmsnorm {str(dt)[6:]}", "8192x4096", a, b, 2 * x.numel() * 2 / 1e6))
    return out


def bench_matmul(quick):
    out = ["| kernel | M=N=K | newt_b200 TFLOP/s | torch TFLOP/s | ratio |", "|---|---|---|---|---|"]
    for dt in (torch.float16, torch.bfloat16):
        for n in ([1024, 4096] if quick else [1024, 2048, 4096, 8192]):
            a_ = (torch.randn(n, n, device="cuda") / n ** 0.5).to(dt)
            b_ = (torch.randn(n, n, device="cuda") / n ** 0.5).to(dt)
            c = torch.empty(n, n, device="cuda", dtype=dt)
            K.matmul(a_, b_, c)     # autotunes: seconds of load, which the rest in _bench lets the chip recover from
            a = _bench(lambda: K.matmul(a_, b_, c))
            b = _bench(lambda: torch.matmul(a_, b_, out=c))
            row = _row(f"matmul {str(dt)[6:]}", n, a, b, 2 * n ** 3 / 1e9)
            out.append(row + f" <!-- {K.matmul_kernel.best_config} -->")
    return out


def bench_matmul_long_k(quick):
    """A small C with a long K: few tiles, many k steps each.  The configurations with 256-row
    CTA-pair tiles have the library cut the tiles along K over all pairs (nb200_gemm_split);
    the autotuner times them next to the single-CTA tiles."""
    out = ["| kernel | M x N x K | newt_b200 TFLOP/s | torch TFLOP/s | ratio |", "|---|---|---|---|---|"]
    shapes = [(1024, 1024, 16384), (512, 512, 65536)]
    if not quick:
        shapes += [(256, 256, 65536), (2048, 1024, 16384), (1024, 1024, 65536)]
    for m, n, k in shapes:
        a_ = (torch.randn(m, k, device="cuda") / k ** 0.5).bfloat16()
        b_ = torch.randn(k, n, device="cuda").bfloat16()
        c = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        K.matmul(a_, b_, c)     # autotunes: seconds of load, which the rest in _bench lets the chip recover from
        a = _bench(lambda: K.matmul(a_, b_, c))
        b = _bench(lambda: torch.matmul(a_, b_, out=c))
        row = _row("matmul bf16", f"{m}x{n}x{k}", a, b, 2 * m * n * k / 1e9)
        out.append(row + f" <!-- {K.matmul_kernel.best_config} -->")
    return out


def bench_matmul_tf32(quick):
    """fp32 operands, tf32 product (benchmarks/bench.py:291-294: torch runs with allow_tf32).
    Our time includes the pass that transposes B for the tensor core."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    out = ["| kernel | M=N=K | newt_b200 TFLOP/s | torch TFLOP/s | ratio |", "|---|---|---|---|---|"]
    try:
        for n in ([1024, 4096] if quick else [1024, 2048, 4096, 8192]):
            a_ = torch.randn(n, n, device="cuda") / n ** 0.5
            b_ = torch.randn(n, n, device="cuda") / n ** 0.5
            c = torch.empty(n, n, device="cuda")
            K.matmul(a_, b_, c)     # autotunes: seconds of load, which the rest in _bench lets the chip recover from
            a = _bench(lambda: K.matmul(a_, b_, c))
            b = _bench(lambda: torch.matmul(a_, b_, out=c))
            row = _row("matmul fp32/tf32", n, a, b, 2 * n ** 3 / 1e9)
            out.append(row + f" <!-- {K.matmul_kernel.best_config} -->")
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return out


def bench_matmul_epilogue(quick):
    """relu(A @ B + bias) in bf16: tensor-core product into an fp32 buffer plus a generated
    epilogue kernel, against torch's matmul + add + relu (three launches)."""
    out = ["| kernel | M=N=K | newt_b200 TFLOP/s | torch TFLOP/s | ratio |", "|---|---|---|---|---|"]
    for n in ([2048] if quick else [2048, 4096, 8192]):
        a_ = (torch.randn(n, n, device="cuda") / n ** 0.5).bfloat16()
        b_ = (torch.randn(n, n, device="cuda") / n ** 0.5).bfloat16()
        bias = torch.randn(n, device="cuda")
        c = torch.empty(n, n, device="cuda", dtype=torch.bfloat16)
        a = _bench(lambda: K.linear_bias_relu(a_, b_, bias, c))
        b = _bench(lambda: torch.relu_(torch.matmul(a_, b_, out=c).add_(bias)))
        out.append(_row("relu(A@B+bias) bf16", n, a, b, 2 * n ** 3 / 1e9))
    return out


def bench_attention(quick):
    out = ["| kernel | B x H x S x D | newt_b200 TFLOP/s | torch SDPA TFLOP/s | ratio |",
           "|---|---|---|---|---|"]
    for causal in (True, False):
        for b, h, s, d in ([(4, 32, 4096, 128)] if quick else [(16, 32, 4096, 128), (4, 32, 8192, 128),
                                                                (16, 32, 2048, 64)]):
            q, k, v = (torch.randn(b, h, s, d, device="cuda").half() for _ in range(3))
            o = torch.empty_like(q)
            flop = 4 * b * h * s * s * d * (0.5 if causal else 1.0)
            a = _bench(lambda: K.attention(q, k, v, causal, o), warmup=3, rep=10)
            t = _bench(lambda: torch.nn.functional.scaled_dot_product_attention(
                q, k, v, is_causal=causal), warmup=3, rep=10)
            out.append(_row(f"attention fp16 {'causal' if causal else 'full'}", f"{b}x{h}x{s}x{d}",
                            a, t, flop / 1e9))
    return out


SUITES = {"add": bench_add, "fused": bench_fused, "softmax": bench_softmax, "layernorm": bench_layernorm,
          "rows": bench_rows, "matmul": bench_matmul, "matmul_long_k": bench_matmul_long_k,
          "matmul_tf32": bench_matmul_tf32,
          "matmul_epilogue": bench_matmul_epilogue, "attention": bench_attention}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--kernel", choices=sorted(SUITES))
    args = ap.parse_args()
    print(f"device: {torch.cuda.get_device_name()}  torch {torch.__version__}\n")
    for name in ([args.kernel] if args.kernel else list(SUITES)):
        print(f"### {name}\n")
        print("\n".join(SUITES[name](args.quick)))
        print()


if __name__ == "__main__":
    main()
