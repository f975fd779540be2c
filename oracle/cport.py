"""TEST INFRASTRUCTURE: ctypes wrapper of oracle/newt_oracle.c (CPU only).

Each function takes CPU torch tensors (or numpy arrays) and returns a new CPU
tensor, computed by the plain-C restatement of the reference kernel named in
its docstring.
"""

import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libnewt_oracle.so")
_lib = None

_DT = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}


def build(force=False):
    """Compiles newt_oracle.c with gcc (make -C oracle)."""
    src = os.path.join(_HERE, "newt_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or \
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _t(x):
    t = torch.as_tensor(x)
    assert t.device.type == "cpu", "the oracle runs on host memory only"
    return t


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


_i64 = ctypes.c_int64


def add_f32(x, y):
    """K0, examples/01_vector_add.py:14-21."""
    x, y = _t(x).contiguous(), _t(y).contiguous()
    out = torch.empty_like(x)
    _load().oracle_add_f32(_p(x), _p(y), _p(out), _i64(x.numel()))
    return out


def softmax_f32(x):
    """K1, examples/02_fused_softmax.py:15-24 (rows of a 2-D fp32 tensor)."""
    x = _t(x)
    assert x.dtype == torch.float32 and x.dim() == 2 and (x.shape[1] <= 1 or x.stride(1) == 1)
    out = torch.empty(x.shape, dtype=x.dtype)
    _load().oracle_softmax_f32(_p(x), _p(out), _i64(x.shape[0]), _i64(x.shape[1]),
                               _i64(x.stride(0)), _i64(out.stride(0)))
    return out


def layernorm(x, w, b, eps=1e-5):
    """K2, examples/03_layernorm.py:13-27."""
    x, w, b = _t(x), _t(w).contiguous(), _t(b).contiguous()
    assert x.dim() == 2 and (x.shape[1] <= 1 or x.stride(1) == 1)
    assert x.dtype == w.dtype == b.dtype
    out = torch.empty(x.shape, dtype=x.dtype)
    _load().oracle_layernorm(_p(x), _p(w), _p(b), _p(out), _i64(x.shape[0]), _i64(x.shape[1]),
                             _i64(x.stride(0)), _i64(out.stride(0)), ctypes.c_float(eps),
                             ctypes.c_int(_DT[x.dtype]))
    return out


def matmul(a, b):
    """K3/K4, examples/04_matmul.py:14-45 and examples/deuteron/01_matmul.py:12-18."""
    a, b = _t(a), _t(b)
    assert a.dtype == b.dtype and a.stride(1) == 1 and b.stride(1) == 1
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    c = torch.empty((m, n), dtype=a.dtype)
    _load().oracle_matmul(_p(a), _p(b), _p(c), _i64(m), _i64(n), _i64(k), _i64(a.stride(0)),
                          _i64(b.stride(0)), _i64(c.stride(0)), ctypes.c_int(_DT[a.dtype]))
    return c


def attention(q, k, v, scale, causal=False, block_n=64):
    """K5, examples/05_fused_attention.py:14-48 over [batch*heads, seq, d] tensors."""
    q, k, v = _t(q), _t(k), _t(v)
    assert q.dim() == 3 and q.stride(2) == 1 and k.stride(2) == 1 and v.stride(2) == 1
    bh, sq, d = q.shape
    skv = k.shape[1]
    o = torch.empty((bh, sq, d), dtype=q.dtype)
    _load().oracle_attention(
        _p(q), _p(k), _p(v), _p(o), _i64(bh), _i64(sq), _i64(skv), _i64(d),
        _i64(q.stride(0)), _i64(q.stride(1)), _i64(k.stride(0)), _i64(k.stride(1)),
        _i64(v.stride(0)), _i64(v.stride(1)), _i64(o.stride(0)), _i64(o.stride(1)),
        ctypes.c_float(scale), ctypes.c_int(int(causal)), ctypes.c_int(block_n),
        ctypes.c_int(_DT[q.dtype]))
    return o
