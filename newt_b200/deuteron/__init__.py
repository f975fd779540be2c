"""The tile language on top of newt_b200: kernels written over whole tensors and tiles of them,
compiled to sm_100a launches with tile sizes chosen by a search.

    import newt_b200.deuteron as dt

    @dt.kernel
    def row_softmax(x, out):
        for rows in dt.tile(x.shape[0]):
            block = x[rows, :]
            shifted = dt.exp(block - block.amax(1)[:, None])
            out[rows, :] = shifted / shifted.sum(1)[:, None]

    row_softmax(x, out)                        # build, pick tile sizes (remembered), launch
    row_softmax.ref(x, out)                    # the same body as plain PyTorch: the oracle
    print(row_softmax.to_newt_source(x, out))  # the newt kernel it was turned into

The public names are those of the reference's `deuteron` package (deuteron/__init__.py:19-44).
"""

from . import codegen as _codegen, language as _language, runtime as _runtime

TraceError = _codegen.TraceError
Config, Kernel, kernel = _runtime.Config, _runtime.Kernel, _runtime.kernel

_LANGUAGE_NAMES = ("EagerTensor", "Tile", "tile", "zeros", "full", "where", "maximum", "minimum",
                   "relu", "exp", "log", "sqrt", "rsqrt", "sigmoid", "tanh", "erf", "abs",
                   "float32", "float16", "bfloat16", "int32", "int64")
globals().update({_n: getattr(_language, _n) for _n in _LANGUAGE_NAMES})

__all__ = ["TraceError", "Config", "Kernel", "kernel", *_LANGUAGE_NAMES]
__version__ = "0.1.0"
