#!/usr/bin/env python
"""Benchmark of the newt_b200 hot path.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

The headline of the line is the bf16 matmul; with the default `--workload all` the same line
carries, under "workloads", one record per other configuration (softmax, layernorm, attention,
the fp16 `@jit` + `@autotune` matmul sweep), each with its own roofline, CPU baseline,
end-to-end figure, clocks and a parity check of the very tensors that were timed.

A "step" is one pass of one workload over one batch of seeded synthetic input:

    matmul     C = A @ B, bf16, one 8192-row block of A per GPU against a replicated
               8192x8192 B, launched as the deuteron `@dt.kernel` tile loop (the headline:
               matmul TFLOP/s at 8192^3; at N GPUs the blocks are rows 8192*r.. of one
               [8192*N, 8192] A, i.e. the M-sharded configuration at N = 8)
    softmax    fused row softmax, fp32 [4096, 4096]
    layernorm  layernorm forward, fp16 [8192, 4096]
    attention  causal attention forward, fp16 [16, 32, 4096, 128] split by batch*head
    matmul_f16 C = A @ B, fp16, M = N = K in {1024, 2048, 4096, 8192}, launched as the
               `@autotune`d `@jit` matmul_kernel (first call tunes, outside the timed steps)

Multi-GPU runs shard independent units (row blocks, heads) across ranks; there is no
collective on the data path.  Timing: CUDA events around every step on the launching
stream, L2 flushed (256 MB write) before each timed step, max over ranks.
`--impl reference` times the reference's CPU path (the torch calls its tests use as
expected values, restated under oracle/) on the host cores instead.
"""

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


# --------------------------------------------------------------------------- peaks

def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "tflops_burst": float(p["bf16_tflops"]),
                "tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops_burst": 1590.0, "tflops_sustained": 1400.0,
            "source": "fallback"}


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "100"],
                stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(names, parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- workloads

def _seeded(shape, seed, dtype, scale=1.0, shift=0.0):
    """Draw on the CPU in fp32 from a seed, scale, round to dtype (identical on every box)."""
    g = torch.Generator().manual_seed(seed)
    return _pin((torch.randn(shape, generator=g) * scale + shift).to(dtype))


def _pin(t):
    return t.pin_memory() if torch.cuda.is_available() else t


def _spread(count, total, seed):
    """`count` distinct indices of range(total): the first, the last and a seeded draw between."""
    count = min(count, total)
    g = torch.Generator().manual_seed(seed)
    picks = {0, total - 1}
    for i in torch.randperm(total, generator=g).tolist():
        if len(picks) >= count:
            break
        picks.add(i)
    return sorted(picks)[:count]


class Workload:
    def __init__(self, small=False, autotune=True):
        pass

    name = ""
    metric = ""
    unit = ""
    dtype = ""
    bound = "hbm"
    scaling = "weak"
    kernels_per_step = 1

    def host_inputs(self, rank, world):  # -> list of pinned CPU tensors
        raise NotImplementedError

    def to_device(self, host):  # -> device state used by step()
        raise NotImplementedError

    def step(self, dev):
        raise NotImplementedError

    def result(self, dev):  # tensor read back in the e2e loop
        raise NotImplementedError

    def units_per_step(self):  # per rank, in the metric's base unit (bytes or flop)
        raise NotImplementedError

    def e2e_step(self, host, out_host):
        """One end-to-end step: pinned host inputs -> device, the kernel through the public
        API, result -> pinned host memory; everything on the current stream."""
        d = self.to_device(host)
        self.step(d)
        out_host.copy_(self.result(d), non_blocking=True)

    def cpu_sample(self, host):  # -> (callable, units processed by it, description)
        raise NotImplementedError

    def parity(self, host, out):
        """Compares `out` (the timed run's own result, on the host) with the CPU oracle.
        -> {"against", "metric", "err", "bar", "pass", "checked"}"""
        raise NotImplementedError

    def traffic_bytes(self):  # DRAM bytes per launch from the ncu capture, or None
        return None

    def config(self, world):
        raise NotImplementedError


def _frobenius_parity(got, want, against, checked):
    from oracle import torch_ref

    err = torch_ref.rel_frobenius(got.float(), want)
    return {"against": against, "metric": "relative Frobenius error vs fp32", "err": err,
            "bar": 1e-2, "pass": bool(err <= 1e-2), "checked": checked}


class SoftmaxWorkload(Workload):
    name, metric, unit, dtype, bound = "softmax", "softmax_hbm_gbs", "GB/s", "f32", "hbm"
    M, N = 4096, 4096

    def host_inputs(self, rank, world):
        return [_seeded((self.M, self.N), 1 + 1000 * rank, torch.float32)]

    def to_device(self, host):
        x = host[0].cuda(non_blocking=True)
        return {"x": x, "out": torch.empty_like(x)}

    def step(self, dev):
        from newt_b200 import examples
        examples.softmax(dev["x"], dev["out"])     # @newt.jit softmax_kernel[(M,)](...)

    def result(self, dev):
        return dev["out"]

    def units_per_step(self):
        return 2 * self.M * self.N * 4  # bytes read + written (benchmarks/bench.py:208 of the reference)

    def cpu_sample(self, host):
        from oracle import torch_ref
        x = host[0]
        return (lambda: torch_ref.softmax(x)), self.units_per_step(), "full [4096,4096] fp32"

    def parity(self, host, out):
        from oracle import torch_ref
        want = torch_ref.softmax(host[0])
        rtol, atol = 1e-5, 1e-9
        err = ((out - want).abs() / (want.abs() + atol / rtol)).max().item()
        return {"against": "oracle.torch_ref.softmax (torch.softmax, CPU fp32)",
                "metric": "max |got - want| / (|want| + atol/rtol): allclose(rtol=1e-5, atol=1e-9)",
                "err": err, "bar": rtol, "pass": bool(err <= rtol),
                "checked": f"all {self.M} x {self.N} elements of the timed output"}

    def traffic_bytes(self):
        return 82.3e6 if (self.M, self.N) == (4096, 4096) else None

    def config(self, world):
        return {"workload": "fused row softmax fp32 [4096,4096] per GPU", "rows": self.M,
                "cols": self.N, "parallelism": f"replicas x{world}", "l2": "flushed between steps"}


class LayerNormWorkload(Workload):
    name, metric, unit, dtype, bound = "layernorm", "layernorm_hbm_gbs", "GB/s", "f16", "hbm"
    M, N = 8192, 4096

    def host_inputs(self, rank, world):
        return [_seeded((self.M, self.N), 2 + 1000 * rank, torch.float16),
                _seeded((self.N,), 21, torch.float16, 0.1, 1.0),
                _seeded((self.N,), 22, torch.float16, 0.1, 0.0)]

    def to_device(self, host):
        x, w, b = (h.cuda(non_blocking=True) for h in host)
        return {"x": x, "w": w, "b": b, "out": torch.empty_like(x)}

    def step(self, dev):
        from newt_b200 import examples
        examples.layernorm(dev["x"], dev["w"], dev["b"], 1e-5, dev["out"])   # @newt.jit kernel

    def result(self, dev):
        return dev["out"]

    def units_per_step(self):
        return 2 * self.M * self.N * 2

    def cpu_sample(self, host):
        from oracle import torch_ref
        x, w, b = host
        return (lambda: torch_ref.layernorm(x, w, b)), self.units_per_step(), \
            "full [8192,4096] fp16 (fp32 math)"

    def parity(self, host, out):
        from oracle import torch_ref
        x, w, b = host
        return _frobenius_parity(out, torch_ref.layernorm(x, w, b),
                                 "oracle.torch_ref.layernorm (F.layer_norm, CPU fp32)",
                                 f"all {self.M} x {self.N} elements of the timed output")

    def traffic_bytes(self):
        return 83.1e6 if (self.M, self.N) == (8192, 4096) else None

    def config(self, world):
        return {"workload": "layernorm forward fp16 [8192,4096] per GPU", "rows": self.M,
                "cols": self.N, "eps": 1e-5, "parallelism": f"replicas x{world}",
                "l2": "flushed between steps"}


class MatmulWorkload(Workload):
    """bf16 C = A @ B through the deuteron tile loop; one 8192-row block of A per GPU."""

    name, metric, unit, dtype, bound = "matmul", "matmul_tflops", "TFLOP/s", "bf16", "tensor"
    M = N = K = 8192
    CPU_ROWS = 1024
    PARITY_ROWS = 256

    def __init__(self, small=False, autotune=True):
        from newt_b200 import examples

        self.kernel = examples.tile_matmul   # the @dt.kernel tile loop; first call autotunes
        if not autotune:                     # profiling runs: skip the search, use a fixed tile
            self.use_tile(256, 256, 128, 3)
        if small:                            # profiler-sized case: 160 MB of operands, > L2
            self.N = self.K = 4096

    def use_tile(self, bm, bn, bk, stages):
        import newt_b200.deuteron as dt
        from newt_b200 import examples

        self.kernel = dt.Kernel(examples.tile_matmul.fn, config={
            "BLOCK_TILE_M": bm, "BLOCK_TILE_N": bn, "BLOCK_TILE_K": bk, "num_stages": stages})

    def host_inputs(self, rank, world):
        scale = 1.0 / self.K ** 0.5
        return [_seeded((self.M, self.K), 40 + rank, torch.bfloat16, scale),   # block `rank` of A
                _seeded((self.K, self.N), 4, torch.bfloat16, scale)]           # B, same on every rank

    def to_device(self, host):
        a, b = (h.cuda(non_blocking=True) for h in host)
        return {"a": a, "b": b, "out": torch.empty(self.M, self.N, device="cuda",
                                                   dtype=host[0].dtype)}

    def step(self, dev):
        self.kernel(dev["a"], dev["b"], dev["out"])

    def launch_block(self, a, b, out):
        self.kernel(a, b, out)

    def result(self, dev):
        return dev["out"]

    def units_per_step(self):
        return 2 * self.M * self.N * self.K

    E2E_CHUNKS = 8

    def e2e_step(self, host, out_host, fanout=None):
        """Same bytes as the plain step, moved as a pipeline: B first, then row blocks of A
        alternate between two streams, so block i's copy in, its matmul (one launch per block)
        and its copy out overlap the neighbouring blocks' transfers.
        `fanout` (a process group): only rank 0 uploads the replicated B; the others receive it
        by an NCCL broadcast into their own HBM before their launches."""
        a_h, b_h = host
        main = torch.cuda.current_stream()
        if not hasattr(self, "_side"):
            self._side = [torch.cuda.Stream(), torch.cuda.Stream()]
            self._e2e_out = torch.empty(self.M, self.N, device="cuda", dtype=a_h.dtype)
        if fanout is not None:
            import torch.distributed as dist

            b = b_h.cuda(non_blocking=True) if dist.get_rank() == 0 else \
                torch.empty(b_h.shape, dtype=b_h.dtype, device="cuda")
            dist.broadcast(b, src=0, group=fanout)
        else:
            b = b_h.cuda(non_blocking=True)
        ready = torch.cuda.Event()
        ready.record(main)
        chunks = max(1, min(self.E2E_CHUNKS, self.M // 128))
        rows = self.M // chunks
        for i in range(chunks):
            st = self._side[i % 2]
            st.wait_event(ready)
            with torch.cuda.stream(st):
                a_i = a_h[i * rows:(i + 1) * rows].cuda(non_blocking=True)
                out_i = self._e2e_out[i * rows:(i + 1) * rows]
                self.launch_block(a_i, b, out_i)
                out_host[i * rows:(i + 1) * rows].copy_(out_i, non_blocking=True)
                a_i.record_stream(st)
        b.record_stream(self._side[0])
        b.record_stream(self._side[1])
        for st in self._side:
            main.wait_stream(st)

    def cpu_sample(self, host):
        from oracle import torch_ref
        a, b = host
        rows = a[:self.CPU_ROWS]
        out = torch.empty(self.CPU_ROWS, self.N, dtype=a.dtype)
        return (lambda: torch_ref.deuteron_matmul(rows, b, out)), \
            2 * self.CPU_ROWS * self.N * self.K, \
            f"{self.CPU_ROWS} of the block's {self.M} rows (eager tile loop, fp32 accumulate)"

    def parity(self, host, out):
        from oracle import torch_ref
        a, b = host
        rows = _spread(self.PARITY_ROWS, self.M, 7)
        idx = torch.tensor(rows)
        return _frobenius_parity(out[idx], torch_ref.matmul(a[idx], b),
                                 "oracle.torch_ref.matmul (a.float() @ b.float(), CPU)",
                                 f"{len(rows)} rows of the timed output spread over all "
                                 f"{self.M} (first, last, seeded draw), every column")

    def traffic_bytes(self):
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this very case
        return 971.5e6 if (self.M, self.N, self.K) == (8192, 8192, 8192) else None

    def config(self, world):
        return {"workload": "bf16 matmul, one [8192,8192] block of A per GPU x B [8192,8192] "
                            "(deuteron @dt.kernel tile loop, fp32 accumulate)",
                "m_per_gpu": self.M, "n": self.N, "k": self.K, "global_m": self.M * world,
                "parallelism": f"A row-blocks over {world} GPU(s), B replicated, no collective",
                "l2": "flushed between steps",
                "tile": dict(self.kernel.best_config or {})}


class MatmulF16Workload(MatmulWorkload):
    """fp16 C = A @ B, M = N = K = n, through `@newt.autotune` over `@newt.jit matmul_kernel`
    exactly as examples/04_matmul.py:48-56 of the reference launches it."""

    name, metric, unit, dtype, bound = "matmul_f16", "matmul_f16_tflops", "TFLOP/s", "f16", "tensor"

    def __init__(self, n=8192, small=False, autotune=True):
        self.M = self.N = self.K = int(n)
        self.CPU_ROWS = min(1024, self.M)

    def host_inputs(self, rank, world):
        scale = 1.0 / self.K ** 0.5
        seed = 3 + int(math.log2(self.K)) + 1000 * rank
        return [_seeded((self.M, self.K), seed, torch.float16, scale),
                _seeded((self.K, self.N), seed + 500, torch.float16, scale)]

    def step(self, dev):
        from newt_b200 import examples
        examples.matmul(dev["a"], dev["b"], dev["out"])

    def launch_block(self, a, b, out):
        from newt_b200 import examples
        examples.matmul(a, b, out)

    def cpu_sample(self, host):
        from oracle import torch_ref
        a, b = host
        rows = a[:self.CPU_ROWS]
        return (lambda: torch_ref.matmul(rows, b)), 2 * self.CPU_ROWS * self.N * self.K, \
            f"{self.CPU_ROWS} of {self.M} rows, a.float() @ b.float()"

    def traffic_bytes(self):
        return None

    def config(self, world):
        from newt_b200 import examples
        best = getattr(examples.matmul_kernel, "best_config", None)
        tile = None
        if best is not None:
            tile = dict(best.kwargs, num_stages=best.num_stages)
        return {"workload": f"fp16 matmul {self.M}^3 via @newt.jit + @newt.autotune",
                "m": self.M, "n": self.N, "k": self.K, "parallelism": f"replicas x{world}",
                "l2": "flushed between steps", "tile": tile}


class AttentionWorkload(Workload):
    """Causal attention forward, fp16 [16, 32, 4096, 128]; the 512 (batch, head) pairs are
    split evenly over the ranks, so this workload scales strongly (fixed total work)."""

    name, metric, unit, dtype, bound = "attention", "attention_tflops", "TFLOP/s", "f16", "tensor"
    scaling = "strong"
    B, H, S, D = 16, 32, 4096, 128
    CPU_HEADS = 8
    PARITY_HEADS = 8

    def __init__(self, small=False, autotune=True):
        if small:                            # profiler-sized case: 2 x 32 heads, 256 MB of q/k/v/o
            self.B = 2

    def host_inputs(self, rank, world):
        self.heads = max(1, self.B * self.H // world)
        first = rank * self.heads
        # one seed per (tensor, rank shard): shards are independent, no exchange needed
        return [_seeded((self.heads, self.S, self.D), 500 + 10 * first + t, torch.float16)
                for t in range(3)]

    def to_device(self, host):
        q, k, v = (h.cuda(non_blocking=True) for h in host)
        return {"q": q, "k": k, "v": v, "out": torch.empty_like(q)}

    def step(self, dev):
        from newt_b200 import examples
        examples.attention(dev["q"], dev["k"], dev["v"], causal=True, out=dev["out"])

    def result(self, dev):
        return dev["out"]

    def units_per_step(self):
        return 4 * self.heads * self.S * self.S * self.D // 2   # causal convention: half the square

    E2E_CHUNKS = 8

    def e2e_step(self, host, out_host):
        """Heads are independent: chunks of (batch, head) pairs alternate between two streams,
        each doing copy in -> attention -> copy out, so transfers in both directions overlap."""
        from newt_b200 import examples

        main = torch.cuda.current_stream()
        if not hasattr(self, "_side"):
            self._side = [torch.cuda.Stream(), torch.cuda.Stream()]
        chunks = min(self.E2E_CHUNKS, self.heads)
        per = -(-self.heads // chunks)
        for i in range(chunks):
            lo, hi = i * per, min(self.heads, (i + 1) * per)
            if lo >= hi:
                break
            st = self._side[i % 2]
            st.wait_stream(main)
            with torch.cuda.stream(st):
                q, k, v = (h[lo:hi].cuda(non_blocking=True) for h in host)
                o = examples.attention(q, k, v, causal=True)
                out_host[lo:hi].copy_(o, non_blocking=True)
                for t in (q, k, v, o):
                    t.record_stream(st)
        for st in self._side:
            main.wait_stream(st)

    def cpu_sample(self, host):
        from oracle import torch_ref
        q, k, v = (h[:self.CPU_HEADS] for h in host)
        scale = 1.0 / self.D ** 0.5
        return (lambda: torch_ref.attention(q, k, v, scale, True)), \
            4 * q.shape[0] * self.S * self.S * self.D // 2, \
            f"{q.shape[0]} of the {self.B * self.H} (batch, head) pairs, " \
            f"F.scaled_dot_product_attention fp32"

    def parity(self, host, out):
        from oracle import torch_ref
        heads = _spread(self.PARITY_HEADS, self.heads, 11)
        idx = torch.tensor(heads)
        q, k, v = (h[idx] for h in host)
        want = torch_ref.attention(q, k, v, 1.0 / self.D ** 0.5, True)
        return _frobenius_parity(
            out[idx], want, "oracle.torch_ref.attention (F.scaled_dot_product_attention, CPU fp32)",
            f"{len(heads)} (batch, head) pairs of each rank's shard of the timed output "
            f"(first, last, seeded draw), every row")

    def traffic_bytes(self):
        # captured on the --small case (64 heads); DRAM traffic grows with the head count
        return 246.0e6 / 64 * self.heads if (self.S, self.D) == (4096, 128) else None

    def config(self, world):
        return {"workload": "causal attention forward fp16 [16,32,4096,128], scale 1/sqrt(128)",
                "batch": self.B, "heads": self.H, "seq_len": self.S, "head_dim": self.D,
                "parallelism": f"batch*head over {world} GPU(s), no collective",
                "l2": "flushed between steps"}


WORKLOADS = {w.name: w for w in (MatmulWorkload, SoftmaxWorkload, LayerNormWorkload,
                                 AttentionWorkload, MatmulF16Workload)}
DEFAULT_WORKLOAD = "matmul"            # the headline of the line
F16_SWEEP = (1024, 2048, 4096, 8192)   # M = N = K of the fp16 @autotune sweep


# --------------------------------------------------------------------------- runners

def max_over_ranks(values, world, device):
    """Element-wise maximum of a list of floats over all ranks (the job is as slow as its
    slowest rank); identity for a single process."""
    if world <= 1:
        return list(values)
    import torch.distributed as dist

    t = torch.tensor(values, device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def job_throughput(units_per_rank_step, world, steps, total_ms, unit):
    """Whole-job value: the units all ranks processed divided by the slowest rank's time."""
    scale = 1e9 if unit == "GB/s" else 1e12
    return units_per_rank_step * world * steps / (total_ms * 1e-3) / scale


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def time_cpu(fn, repeats=3):
    fn()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def reference_record(args, wl):
    """The reference's CPU path for one workload, timed on the host cores."""
    torch.set_num_threads(os.cpu_count() or 1)
    host = wl.host_inputs(0, 1)
    fn, units, sample = wl.cpu_sample(host)
    for _ in range(max(1, min(args.warmup, 2))):
        fn()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    scale = 1e9 if wl.unit == "GB/s" else 1e12
    value = units / sec / scale
    return {
        "impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic (seeded N(0,1))",
        "config": wl.config(args.gpus),
        "cpu_baseline": {"value": value, "unit": wl.unit, "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }


def run_reference(args, wl):
    """Reference arm: rank 0 alone runs and prints; the other ranks leave without work."""
    rank, _, _ = _dist_env()
    if rank != 0:
        return
    print(json.dumps(reference_record(args, wl)), flush=True)


def run_reference_all(args):
    """Reference arm of the default run: the headline's CPU path, the others beside it."""
    rank, _, _ = _dist_env()
    if rank != 0:
        return
    line = reference_record(args, WORKLOADS[DEFAULT_WORKLOAD]())
    few = argparse.Namespace(**dict(vars(args), steps=min(args.steps, 3), warmup=1))
    extra = {name: _brief(reference_record(few, WORKLOADS[name]()))
             for name in ("softmax", "layernorm", "attention")}
    extra["matmul_f16_autotune"] = {
        "sizes": {str(n): _brief(reference_record(few, MatmulF16Workload(n))) for n in F16_SWEEP}}
    line["workloads"] = extra
    print(json.dumps(line), flush=True)


class GpuContext:
    """What the workloads of one bench process share: ranks, the L2 flush buffer, the barrier."""

    def __init__(self):
        import torch.distributed as dist

        self.rank, self.world, self.local = _dist_env()
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (the kernels have no CPU fallback)")
        torch.cuda.set_device(self.local)
        self.dist = dist
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
        self.flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int32, device="cuda")
        self.peaks = measured_peaks()
        torch.cuda.synchronize()

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def _event():
    return torch.cuda.Event(enable_timing=True)


def protocol_floor_ms(ctx, nbytes, reps=20):
    """A plain device copy of the same size (nbytes read + written in all) under the very
    protocol the HBM-bound steps are timed with: what that protocol can show at best."""
    src = torch.empty(nbytes // 2, dtype=torch.uint8, device="cuda").random_(0, 255)
    dst = torch.empty_like(src)
    for _ in range(3):
        ctx.flush.zero_()
        dst.copy_(src)
    pairs = [(_event(), _event()) for _ in range(reps)]
    for s, e in pairs:
        ctx.flush.zero_()
        s.record()
        dst.copy_(src)
        e.record()
    torch.cuda.synchronize()
    return statistics.median(s.elapsed_time(e) for s, e in pairs)


def empty_launch_ms(ctx, reps=20):
    """What the same protocol reads for a launch that moves nothing (a 32-byte copy): the part
    of every step time that is the launch itself, not the kernel's traffic."""
    return protocol_floor_ms(ctx, 64, reps)


def measure(ctx, args, wl):
    """Times one workload on this rank's GPU; rank 0 gets the record (the others None)."""
    rank, world = ctx.rank, ctx.world
    steps = args.steps
    host = wl.host_inputs(rank, world)
    dev = wl.to_device(host)
    flush = ctx.flush
    torch.cuda.synchronize()

    w0, w1 = _event(), _event()
    for _ in range(max(args.warmup, 3)):       # the first call also tunes where there is a search
        flush.zero_()
        w0.record()
        wl.step(dev)
        w1.record()
    ctx.barrier()
    warm_step_ms = max(w0.elapsed_time(w1), 1e-3)

    sampler = ClockSampler(ctx.local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)      # nvidia-smi needs a few hundred ms to come up

    # ---- device-resident timed region: K steps, one event pair per step ------
    starts = [_event() for _ in range(steps)]
    ends = [_event() for _ in range(steps)]
    ctx.barrier()
    # Untimed steps on every rank, queued straight ahead of the timed ones: the pause and the
    # barrier above left the GPU idle, and the first launches after that pay for the ramp (a
    # 28 us row kernel read 59 us there).  About 0.7 ms of them: one matmul step, a couple of
    # dozen row-kernel steps.
    for _ in range(min(32, max(1, math.ceil(0.7 / warm_step_ms)))):
        flush.zero_()
        wl.step(dev)
    for i in range(steps):
        flush.zero_()
        starts[i].record()
        wl.step(dev)
        ends[i].record()
    ctx.barrier()
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    total_ms = sum(step_ms)
    timed_config = wl.config(world)      # as of the timed steps (later launches may tune other shapes)

    # ---- parity of the very tensors that were just timed ----------------------
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    timed_out = wl.result(dev).cpu()
    par = wl.parity(host, timed_out)
    del timed_out
    errs = max_over_ranks([par["err"], 0.0 if par["pass"] else 1.0], world, "cuda")
    par["err"], par["pass"] = errs[0], errs[1] == 0.0
    if world > 1:
        par["checked"] += f"; worst of {world} ranks"

    # ---- HBM-bound: the same steps back to back over rotating buffer sets ------
    rotating_ms = floor_ms = launch_only_ms = None
    if wl.bound == "hbm":
        sets = [dev] + [wl.to_device(host) for _ in range(7)]    # 8 x 128 MB > L2, no flush
        reps = max(steps, 40)
        for s in sets:
            wl.step(s)
        r0, r1 = _event(), _event()
        ctx.barrier()
        r0.record()
        for i in range(reps):
            wl.step(sets[i % 8])
        r1.record()
        ctx.barrier()
        rotating_ms = r0.elapsed_time(r1) / reps
        del sets
        floor_ms = protocol_floor_ms(ctx, wl.units_per_step())
        launch_only_ms = empty_launch_ms(ctx)
    clocks = sampler.stop() if rank == 0 else None     # sampled over the device-timed regions

    # ---- end-to-end region: pinned host -> device, step, result -> host -------
    out_host = _pin(torch.empty(wl.result(dev).shape, dtype=wl.result(dev).dtype))
    h2d = sum(h.numel() * h.element_size() for h in host)
    d2h = out_host.numel() * out_host.element_size()
    e2e_steps = max(3, min(steps, 10))

    def timed_e2e(fn):
        fn()
        ctx.barrier()
        e0, e1 = _event(), _event()
        e0.record()
        for _ in range(e2e_steps):
            fn()
        e1.record()
        ctx.barrier()
        return e0.elapsed_time(e1) / e2e_steps

    e2e_ms = timed_e2e(lambda: wl.e2e_step(host, out_host))
    fanout_ms = None
    if world > 1 and wl.name == "matmul":
        group = ctx.dist.group.WORLD
        fanout_ms = timed_e2e(lambda: wl.e2e_step(host, out_host, fanout=group))

    # the three legs of a step one after the other (no overlap), each between its own events
    legs = []
    for _ in range(3):
        ev = [_event() for _ in range(4)]
        ctx.barrier()
        ev[0].record()
        d = wl.to_device(host)
        ev[1].record()
        wl.step(d)
        ev[2].record()
        out_host.copy_(wl.result(d), non_blocking=True)
        ev[3].record()
        torch.cuda.synchronize()
        legs.append([ev[i].elapsed_time(ev[i + 1]) for i in range(3)])
        del d
    h2d_ms, kernel_ms, d2h_ms = (statistics.median(leg[i] for leg in legs) for i in range(3))

    vals = [total_ms, e2e_ms, h2d_ms, kernel_ms, d2h_ms, rotating_ms or 0.0, fanout_ms or 0.0]
    total_ms, e2e_ms, h2d_ms, kernel_ms, d2h_ms, rotating_ms, fanout_ms = \
        max_over_ranks(vals, world, "cuda")
    if rank != 0:
        return None

    peaks = ctx.peaks
    scale = 1e9 if wl.unit == "GB/s" else 1e12
    units = wl.units_per_step()
    value = job_throughput(units, world, steps, total_ms, wl.unit)
    launch_ms = total_ms / (steps * wl.kernels_per_step)
    achieved = units / wl.kernels_per_step / (launch_ms * 1e-3) / scale
    peak = peaks["hbm_gbs"] if wl.bound == "hbm" else peaks["tflops_burst"]
    roofline = {"bound": wl.bound, "achieved": achieved, "peak": peak, "unit": wl.unit,
                "frac": achieved / peak,
                "traffic": None if args.small else wl.traffic_bytes(),
                "peak_source": peaks["source"] + (" copy bandwidth" if wl.bound == "hbm"
                                                  else " cuBLAS bf16 burst")}
    if wl.bound == "hbm":
        back_to_back = units / (rotating_ms * 1e-3) / scale
        roofline.update({
            "protocol_floor_ms": floor_ms,
            "protocol_floor_note": "torch copy_ of the same bytes (half read, half written) "
                                   "timed by the identical flush + event protocol",
            "vs_protocol_floor": floor_ms / launch_ms,
            "empty_launch_ms": launch_only_ms,
            "net_of_launch": {"achieved": units / max(launch_ms - launch_only_ms, 1e-6) / 1e-3 / scale,
                              "how": "the same bytes over the step time less what an empty "
                                     "launch reads between the same events"},
            "back_to_back": {"achieved": back_to_back, "frac": back_to_back / peak,
                             "ms_per_step": rotating_ms,
                             "how": "no flush: steps back to back over 8 rotating input/output "
                                    "sets (1 GB > L2), one event pair around all of them"}})
    rec = {
        "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world,
        "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / steps, "higher_is_better": True, "scaling": wl.scaling,
        "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic (seeded N(0,1) drawn on the host, copied to HBM before timing)",
        "config": dict(timed_config, **({"small": True} if args.small else {})),
        "roofline": roofline,
        "e2e": {"value": job_throughput(units, world, 1, e2e_ms, wl.unit), "unit": wl.unit,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                "how": "pinned host -> device -> public API launch -> pinned host, every step",
                "legs_serial": {"h2d_ms": h2d_ms, "kernel_ms": kernel_ms, "d2h_ms": d2h_ms,
                                "h2d_gbs_per_gpu": h2d / (h2d_ms * 1e-3) / 1e9,
                                "d2h_gbs_per_gpu": d2h / (d2h_ms * 1e-3) / 1e9,
                                "how": "one step with its three legs run one after the other, "
                                       "each between its own event pair; max over ranks"}},
        "gpu_launches": steps * wl.kernels_per_step,
        "clocks": clocks,
        "step_ms": {"min": min(step_ms), "median": statistics.median(step_ms),
                    "max": max(step_ms), "slowest": step_ms.index(max(step_ms))},
        "parity": par,
    }
    if fanout_ms:
        b_bytes = host[1].numel() * host[1].element_size()
        rec["e2e_nvlink_fanout"] = {
            "value": job_throughput(units, world, 1, fanout_ms, wl.unit), "unit": wl.unit,
            "ms_per_step": fanout_ms,
            "h2d_bytes_per_step": {"rank0": h2d, "others": h2d - b_bytes},
            "how": "as e2e, but only rank 0 uploads the replicated B; the other ranks receive "
                   "it by NCCL broadcast over NVLink into their own HBM before their launches"}
    if world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        fn, cpu_units, sample = wl.cpu_sample(host)
        best = time_cpu(fn)
        rec["cpu_baseline"] = {"value": cpu_units / best / scale, "unit": wl.unit,
                               "cores": torch.get_num_threads(), "kind": "port", "sample": sample}
    return rec


def _brief(rec):
    """A sub-record of the line: what the headline carries, minus the run-wide keys."""
    if rec is None:
        return None
    drop = ("n_gpus", "warmup", "higher_is_better", "vs_baseline", "data", "impl")
    return {k: v for k, v in rec.items() if k not in drop}


def run_gpu(args):
    ctx = GpuContext()
    opts = dict(small=args.small, autotune=not args.no_autotune)

    def make(name):
        wl = WORKLOADS[name](**opts)
        if args.no_autotune and name == "matmul":
            wl.use_tile(*(int(v) for v in args.tile.split(",")))
        return wl

    headline = DEFAULT_WORKLOAD if args.workload == "all" else args.workload
    line = measure(ctx, args, make(headline))
    if args.workload == "all":
        extra = {}
        for name in ("softmax", "layernorm", "attention"):
            extra[name] = _brief(measure(ctx, args, make(name)))
            torch.cuda.empty_cache()
        sweep = {}
        for n in F16_SWEEP:
            sweep[str(n)] = _brief(measure(ctx, args, MatmulF16Workload(n)))
            torch.cuda.empty_cache()
        if ctx.rank == 0:
            launches = line["gpu_launches"] + sum(r["gpu_launches"] for r in extra.values()) + \
                sum(r["gpu_launches"] for r in sweep.values())
            extra["matmul_f16_autotune"] = {
                "metric": "matmul_f16_tflops", "unit": "TFLOP/s",
                "how": "M = N = K per key; @newt.autotune over @newt.jit matmul_kernel, tuned by "
                       "the first (untimed) call", "sizes": sweep}
            line["workloads"] = extra
            line["gpu_launches_all_workloads"] = launches
    if ctx.rank == 0:
        print(json.dumps(line), flush=True)
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="all", choices=sorted(WORKLOADS) + ["all"],
                    help="all = the matmul headline plus every other configuration as sub-records")
    ap.add_argument("--impl", default="newt_b200", choices=["newt_b200", "reference"])
    ap.add_argument("--small", action="store_true",
                    help="profiler-sized variant of the workload (never a reported number)")
    ap.add_argument("--no-autotune", action="store_true",
                    help="fixed tile configuration instead of the first-call search")
    ap.add_argument("--tile", default="256,512,64,4",
                    help="BLOCK_M,BLOCK_N,BLOCK_K,num_stages used with --no-autotune (matmul)")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=INT",
                    help="library tuning knob (nb200_set_tuning), e.g. row_tpr=256")
    args = ap.parse_args()
    for item in args.tune:
        from newt_b200.runtime import abi
        key, _, val = item.partition("=")
        abi.set_tuning(key, int(val))
    if args.impl == "reference":
        if args.workload == "all":
            run_reference_all(args)
        else:
            run_reference(args, WORKLOADS[args.workload]())
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
