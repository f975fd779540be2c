"""The user-level kernels of the hot path, written against the operator API the way
the reference's examples/ directory writes them (examples/01..05 and
examples/deuteron/01_matmul.py), each with the small host wrapper the example
has.  bench.py and __graft_entry__.smoke() launch these."""

from .kernels import (add, add_kernel, attention, attention_kernel, layernorm,  # noqa: F401
                      layernorm_kernel, matmul, matmul_kernel,
                      softmax, softmax_kernel)
from .tiles import tile_matmul  # noqa: F401
