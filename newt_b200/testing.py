"""Timing and comparison helpers with the semantics of newt/testing.py.

`do_bench` is the reference's clock (:6-24): one untimed call, `warmup` calls,
then `rep` calls each preceded by a 256 MB write that evicts L2, timed with a
CUDA event pair on the current stream; the result is the requested quantile
(median by default) in milliseconds.
"""

import torch

_flush = {}


def _flush_buffer():
    dev = torch.cuda.current_device()
    buf = _flush.get(dev)
    if buf is None:
        buf = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.int32, device="cuda")
        _flush[dev] = buf
    return buf


def do_bench(fn, warmup=10, rep=50, quantile=0.5):
    fn()
    torch.cuda.synchronize()
    flush = _flush_buffer()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
             for _ in range(rep)]
    for start, end in pairs:
        flush.zero_()
        start.record()
        fn()
        end.record()
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in pairs)
    return times[min(len(times) - 1, int(len(times) * quantile))]


def assert_close(actual, expected, rtol=1e-3, atol=1e-3, msg=""):
    if torch.allclose(actual, expected, rtol=rtol, atol=atol):
        return
    diff = (actual - expected).abs()
    rel = diff / expected.abs().clamp_min(1e-6)
    raise AssertionError(f"{msg} mismatch: max abs err {diff.max().item():.3e}, "
                         f"max rel err {rel.max().item():.3e}")
