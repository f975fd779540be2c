"""TEST INFRASTRUCTURE: the torch calls the reference's tests and examples use
as their expected values, restated on CPU tensors (fp32 math from the already
rounded 16-bit inputs).  Used for full-size parity and as the timed CPU
baseline; never imported by the product.
"""

import torch
import torch.nn.functional as F


def add(x, y):
    """tests/test_vector_add.py:30 -- `x + y`, compared with torch.equal."""
    return x + y


def softmax(x):
    """examples/02_fused_softmax.py:39, tests/test_softmax_layernorm.py:47."""
    return torch.softmax(x, dim=-1)


def layernorm(x, w, b, eps=1e-5):
    """examples/03_layernorm.py:45, tests/test_softmax_layernorm.py:61; fp32 oracle of 16-bit inputs."""
    n = x.shape[-1]
    return F.layer_norm(x.float(), (n,), w.float(), b.float(), eps)


def matmul(a, b):
    """tests/test_matmul.py:55 -- `a.float() @ b.float()`."""
    return a.float() @ b.float()


def deuteron_matmul(x, y, out):
    """examples/deuteron/01_matmul.py:13-18 run as its eager mode does
    (deuteron/runtime.py:71-73, full-size tiles), with the fp32 accumulator on
    the host instead of the hard-coded CUDA device of deuteron/language.py:83-85."""
    acc = torch.zeros(x.shape[0], y.shape[1], dtype=torch.float32)
    acc += x.float() @ y.float()
    out[:, :] = acc
    return out


def attention(q, k, v, scale, causal=False):
    """examples/05_fused_attention.py:75-77 -- F.scaled_dot_product_attention,
    on [batch*heads, seq, d] tensors, fp32 math."""
    return F.scaled_dot_product_attention(q.float()[None], k.float()[None], v.float()[None],
                                          is_causal=causal, scale=scale)[0]


def rel_frobenius(actual, expected):
    """||actual - expected||_F / ||expected||_F in fp64."""
    a, e = actual.double(), expected.double()
    return ((a - e).norm() / e.norm().clamp_min(1e-30)).item()
