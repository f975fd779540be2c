"""newt_b200 -- a B200-native (sm_100a) backend behind the operator API of newt.

    import newt_b200 as newt
    import newt_b200.language as nl

    @newt.jit
    def scale_kernel(x_ptr, out_ptr, factor, n, BLOCK: nl.constexpr):
        lanes = nl.program_id(0) * BLOCK + nl.arange(0, BLOCK)
        inside = lanes < n
        nl.store(out_ptr + lanes, nl.load(x_ptr + lanes, mask=inside) * factor, mask=inside)

    scale_kernel[(newt.cdiv(n, 2048),)](x, out, 0.5, n, BLOCK=2048)

Exports the names of newt/__init__.py of the reference (:18-51).  `install_aliases()` also
registers this package under the module names `newt` and `deuteron`, so kernels written
against the reference import unchanged.
"""

import sys as _sys

from . import language, testing, types
from .frontend import trace as _trace
from .runtime import autotuner as _autotuner, jit as _jit

__version__ = "0.1.0"

# decorators and the classes behind them
jit, JITFunction = _jit.jit, _jit.JITFunction
autotune, heuristics = _autotuner.autotune, _autotuner.heuristics
Autotuner, Heuristics, Config = _autotuner.Autotuner, _autotuner.Heuristics, _autotuner.Config
CompileError = _trace.CompileError


def cdiv(a, b):
    """Ceiling of a / b for non-negative integers: how many blocks of b cover a."""
    return (a + b - 1) // b


def next_power_of_2(n):
    """The smallest power of two that is not below n (1 for n <= 1)."""
    return 1 << max(int(n) - 1, 0).bit_length()


def install_aliases():
    """Registers this package as `newt` and its tile language as `deuteron` -- with the
    submodules programs written against the reference import by name (`newt.language`,
    `newt.testing`, `newt.runtime[.jit|.autotuner|.cuda]`, `newt.compiler[.codegen|.types]`) --
    unless modules of those names are loaded already."""
    import importlib

    here = _sys.modules[__name__]
    _sys.modules.setdefault("newt", here)
    for sub in ("language", "testing", "types", "runtime", "runtime.jit", "runtime.autotuner",
                "runtime.cuda", "compiler", "compiler.codegen", "deuteron"):
        module = importlib.import_module(f"{__name__}.{sub}")
        _sys.modules.setdefault(f"newt.{sub}", module)
    _sys.modules.setdefault("newt.compiler.types", types)     # where the reference keeps them
    _sys.modules.setdefault("deuteron", _sys.modules[f"{__name__}.deuteron"])
    for sub in ("language", "codegen", "runtime"):
        _sys.modules.setdefault(f"deuteron.{sub}", _sys.modules[f"{__name__}.deuteron.{sub}"])


__all__ = ("jit", "autotune", "heuristics", "Config", "cdiv", "next_power_of_2", "language",
           "testing", "JITFunction", "Autotuner", "Heuristics", "CompileError", "install_aliases",
           "__version__")
