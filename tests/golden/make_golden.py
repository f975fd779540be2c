"""Generates tests/golden/*.npz by running the REFERENCE project on CPU.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py <path of the reference checkout>

What is recorded, per case, is the seeded input and the reference's own result:
  * `deuteron` eager mode (`Kernel.ref`, deuteron/runtime.py:71-73) of the
    reference's example kernels (examples/deuteron/01..03) -- the reference's
    algorithm executed by the reference's code;
  * the torch expressions the reference's tests use as expected values
    (tests/test_softmax_layernorm.py:47,61, tests/test_matmul.py:55,
    tests/test_vector_add.py:30, examples/05_fused_attention.py:75-77).
The matmul eager mode allocates its accumulator with a hard-coded CUDA device
(deuteron/language.py:83-85); this script points that allocator at the CPU and
changes nothing else.

bfloat16 arrays are stored as their uint16 bit patterns (numpy has no bf16).
The fixtures are read by tests/test_oracle.py (oracle vs reference) and
tests/test_parity_gpu.py (CUDA kernels vs reference); neither needs the
reference checkout at run time.
"""

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t):
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def _load_example(ref_root, rel):
    spec = importlib.util.spec_from_file_location("ref_example_" + os.path.basename(rel)[:-3],
                                                  os.path.join(ref_root, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root):
    sys.path.insert(0, ref_root)
    import deuteron  # the reference package
    import deuteron.language as dl

    def cpu_zeros(shape, dtype=torch.float32):
        sizes = [s.size if isinstance(s, dl.Tile) else int(s) for s in shape]
        return torch.zeros(*sizes, dtype=dtype)

    deuteron.zeros = cpu_zeros
    dl.zeros = cpu_zeros

    ex_mm = _load_example(ref_root, "examples/deuteron/01_matmul.py")
    ex_sm = _load_example(ref_root, "examples/deuteron/02_softmax.py")
    ex_ln = _load_example(ref_root, "examples/deuteron/03_layernorm.py")

    g = torch.Generator().manual_seed(20260101)

    def randn(*shape, dtype=torch.float32, scale=1.0):
        return (torch.randn(*shape, generator=g) * scale).to(dtype)

    out = {}

    # K0 vector add (tests/test_vector_add.py:22-31 sizes incl. the ragged 12345)
    for n in (1024, 12345):
        x, y = randn(n), randn(n)
        out[f"add/{n}/x"], out[f"add/{n}/y"] = _np(x), _np(y)
        out[f"add/{n}/expected"] = _np(x + y)

    # K1 softmax (tests/test_softmax_layernorm.py:41 shapes, plus a 4096-wide row)
    for m, n in ((8, 128), (32, 781), (4, 1024), (2, 4096)):
        x = randn(m, n)
        eager = torch.empty_like(x)
        ex_sm.softmax.ref(x, eager)
        out[f"softmax/{m}x{n}/x"] = _np(x)
        out[f"softmax/{m}x{n}/expected_eager"] = _np(eager)
        out[f"softmax/{m}x{n}/expected_torch"] = _np(torch.softmax(x, dim=-1))

    # K2 layernorm fp32 (tests/test_softmax_layernorm.py:53 shapes) via eager mode and torch
    for m, n in ((8, 128), (4, 2048), (16, 300)):
        x, w, b = randn(m, n), randn(n), randn(n)
        eager = torch.empty_like(x)
        ex_ln.layernorm.ref(x, w, b, eager, 1e-5)
        for k, v in (("x", x), ("w", w), ("b", b), ("expected_eager", eager),
                     ("expected_torch", torch.nn.functional.layer_norm(x, (n,), w, b, 1e-5))):
            out[f"layernorm_f32/{m}x{n}/{k}"] = _np(v)
    # K2 layernorm 16-bit: fp32 oracle computed from the rounded inputs
    for name, dt in (("f16", torch.float16), ("bf16", torch.bfloat16)):
        for m, n in ((4, 4096), (16, 300)):
            x = randn(m, n, dtype=dt)
            w = (1.0 + 0.1 * torch.randn(n, generator=g)).to(dt)
            b = (0.1 * torch.randn(n, generator=g)).to(dt)
            exp = torch.nn.functional.layer_norm(x.float(), (n,), w.float(), b.float(), 1e-5)
            for k, v in (("x", x), ("w", w), ("b", b), ("expected_f32", exp)):
                out[f"layernorm_{name}/{m}x{n}/{k}"] = _np(v)

    # K3/K4 matmul (tests/test_matmul.py:52-65 shapes), eager deuteron + torch fp32
    for name, dt, shapes in (("f16", torch.float16, ((64, 64, 32), (256, 256, 128), (300, 200, 100))),
                             ("bf16", torch.bfloat16, ((256, 128, 64),))):
        for m, n, k in shapes:
            a, b = randn(m, k, dtype=dt, scale=0.5), randn(k, n, dtype=dt, scale=0.5)
            eager = torch.empty(m, n, dtype=dt)
            ex_mm.matmul.ref(a, b, eager)
            key = f"matmul_{name}/{m}x{n}x{k}"
            out[key + "/a"], out[key + "/b"] = _np(a), _np(b)
            out[key + "/expected_eager"] = _np(eager)
            out[key + "/expected_f32"] = _np(a.float() @ b.float())

    # K5 attention: the shipped single-head non-causal form and the batched causal form
    for key, bh, s, d, causal in (("attention/noncausal_1x256x64", 1, 256, 64, False),
                                  ("attention/causal_2x192x128", 2, 192, 128, True)):
        q, k, v = (randn(bh, s, d, dtype=torch.float16) for _ in range(3))
        exp = torch.nn.functional.scaled_dot_product_attention(
            q.float()[None], k.float()[None], v.float()[None], is_causal=causal)[0]
        out[key + "/q"], out[key + "/k"], out[key + "/v"] = _np(q), _np(k), _np(v)
        out[key + "/expected_f32"] = _np(exp)

    # fp32 matmul, the case of tests/test_matmul.py:67-70 (nl.dot on fp32 runs as tf32 on the
    # device; the test's expected value is the fp32 product, within rtol = atol = 1e-2).
    # Appended last so that the draws above keep their values.
    a, b = randn(128, 128, dtype=torch.float32, scale=0.5), randn(128, 128, dtype=torch.float32, scale=0.5)
    eager = torch.empty(128, 128, dtype=torch.float32)
    ex_mm.matmul.ref(a, b, eager)
    key = "matmul_f32/128x128x128"
    out[key + "/a"], out[key + "/b"] = _np(a), _np(b)
    out[key + "/expected_eager"] = _np(eager)
    out[key + "/expected_f32"] = _np(a @ b)

    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path) / 1e6:.2f} MB")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
