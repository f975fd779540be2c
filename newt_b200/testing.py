"""Timing and comparison helpers with the semantics of newt/testing.py.

`do_bench` is the reference's clock (:6-24): one untimed call, `warmup` calls, then `rep`
calls each preceded by a 256 MB write that evicts L2, each timed with a CUDA event pair on
the current stream; the result is the requested quantile (median by default) in milliseconds.
"""

import torch

_L2_FLUSH_BYTES = 256 << 20
_flush_buffers = {}      # device index -> int32 buffer that is rewritten before every timed call


def _evict_l2():
    device = torch.cuda.current_device()
    if device not in _flush_buffers:
        _flush_buffers[device] = torch.empty(_L2_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda")
    _flush_buffers[device].zero_()


def do_bench(fn, warmup=10, rep=50, quantile=0.5):
    fn()                             # whatever the first call compiles or tunes stays outside
    torch.cuda.synchronize()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(rep)]
    for begin, finish in events:
        _evict_l2()
        begin.record()
        fn()
        finish.record()
    torch.cuda.synchronize()
    elapsed = sorted(begin.elapsed_time(finish) for begin, finish in events)
    return elapsed[min(int(rep * quantile), rep - 1)]


def assert_close(actual, expected, rtol=1e-3, atol=1e-3, msg=""):
    if torch.allclose(actual, expected, rtol=rtol, atol=atol):
        return
    gap = (actual - expected).abs()
    worst_abs = gap.max().item()
    worst_rel = (gap / expected.abs().clamp_min(1e-6)).max().item()
    raise AssertionError(f"{msg} mismatch: max abs err {worst_abs:.3e}, max rel err {worst_rel:.3e}")
