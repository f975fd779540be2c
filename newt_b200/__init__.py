"""newt_b200 -- a B200-native (sm_100a) backend behind the operator API of newt.

    import newt_b200 as newt
    import newt_b200.language as nl

    @newt.jit
    def add_kernel(x_ptr, y_ptr, out_ptr, n, BLOCK: nl.constexpr):
        pid = nl.program_id(0)
        offs = pid * BLOCK + nl.arange(0, BLOCK)
        mask = offs < n
        nl.store(out_ptr + offs, nl.load(x_ptr + offs, mask=mask) + nl.load(y_ptr + offs, mask=mask),
                 mask=mask)

    add_kernel[(newt.cdiv(n, 1024),)](x, y, out, n, BLOCK=1024)

The names exported here are the ones newt/__init__.py of the reference exports
(:18-51).  `install_aliases()` additionally registers this package under the
module names `newt` and `deuteron`, so kernels written against the reference
import unchanged.
"""

import sys as _sys

from . import language, testing, types
from .frontend.trace import CompileError
from .runtime.autotuner import Autotuner, Config, Heuristics, autotune, heuristics
from .runtime.jit import JITFunction, jit

__version__ = "0.1.0"


def cdiv(a, b):
    return -(-a // b)


def next_power_of_2(n):
    n = int(n)
    return 1 if n <= 1 else 1 << (n - 1).bit_length()


def install_aliases():
    """Makes `import newt`, `import newt.language as nl` and `import deuteron`
    resolve to this package."""
    from . import deuteron

    _sys.modules.setdefault("newt", _sys.modules[__name__])
    _sys.modules.setdefault("newt.language", language)
    _sys.modules.setdefault("newt.testing", testing)
    _sys.modules.setdefault("deuteron", deuteron)


__all__ = ["Autotuner", "CompileError", "Config", "Heuristics", "JITFunction", "__version__",
           "autotune", "cdiv", "heuristics", "jit", "language", "next_power_of_2", "testing",
           "install_aliases"]
