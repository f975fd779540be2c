"""ctypes binding of libnewt_b200.so, the C-ABI kernel library (include/newt_b200.h).

This is the only module that touches the shared object.  There is no fallback:
if the library has not been built, importing a kernel entry point raises.
The reference binds libcuda/libnvrtc the same bare-ctypes way
(newt/runtime/cuda.py:20-71); here the object behind ctypes is our own.
"""

import ctypes
import os

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_PATH = os.path.join(_PKG, "libnewt_b200.so")

OK, E_INVALID, E_UNSUPPORTED, E_CUDA, E_DEVICE = range(5)
F32, F16, BF16 = 0, 1, 2


class KernelLibraryError(RuntimeError):
    """A call into libnewt_b200.so returned a non-zero status."""

    def __init__(self, code, message):
        super().__init__(message)
        self.code = code


class UnsupportedError(KernelLibraryError):
    """The request is legal but no sm_100a kernel in the library covers it."""


class GemmConfig(ctypes.Structure):
    _fields_ = [
        ("block_m", ctypes.c_int32),
        ("block_n", ctypes.c_int32),
        ("block_k", ctypes.c_int32),
        ("stages", ctypes.c_int32),
        ("cta_pair", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 3),
    ]


class GemmLaunch(ctypes.Structure):
    """nb200_gemm_launch: which template instance a run-time compiled GEMM is, and its launch."""
    _fields_ = [(name, ctypes.c_int32) for name in
                ("pair", "block_n", "stages", "ksub", "grid", "block", "cluster", "smem_bytes",
                 "nothing", "only_clear")] + [("reserved", ctypes.c_int32 * 6)]


_i64 = ctypes.c_int64
_vp = ctypes.c_void_p

# name -> (restype, argtypes); must list every function include/newt_b200.h declares
SIGNATURES = {
    "nb200_abi_version": (ctypes.c_int, []),
    "nb200_last_error": (ctypes.c_char_p, []),
    "nb200_read_status": (ctypes.c_int, [ctypes.POINTER(ctypes.c_uint32),
                                         ctypes.POINTER(ctypes.c_uint32)]),
    "nb200_set_tuning": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_int]),
    "nb200_selftest_wait_timeout": (ctypes.c_int, [ctypes.c_uint32, _vp]),
    "nb200_add_f32": (ctypes.c_int, [_vp, _vp, _vp, _i64, _vp]),
    "nb200_softmax_f32": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i64, _i64, _vp]),
    "nb200_layernorm": (ctypes.c_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64,
                                       ctypes.c_float, ctypes.c_int, _vp]),
    "nb200_gemm": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                  ctypes.c_int, ctypes.POINTER(GemmConfig), _vp]),
    "nb200_gemm_bt": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                     ctypes.c_int, ctypes.POINTER(GemmConfig), _vp]),
    "nb200_gemm_tf32_workspace_bytes": (ctypes.c_int64, [_i64, _i64]),
    "nb200_gemm_tf32": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                       ctypes.POINTER(GemmConfig), _vp, _i64, _vp]),
    "nb200_gemm_tf32_static": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                              ctypes.POINTER(GemmConfig), _vp]),
    "nb200_gemm_acc32": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                        ctypes.c_int, ctypes.c_int, ctypes.POINTER(GemmConfig), _vp]),
    "nb200_gemm_split_workspace_bytes": (ctypes.c_int64, [_i64, _i64, _i64, ctypes.c_int,
                                                          ctypes.POINTER(GemmConfig)]),
    "nb200_gemm_split": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                        ctypes.c_int, ctypes.c_int, ctypes.POINTER(GemmConfig), _vp,
                                        _i64, _vp]),
    "nb200_gemm_params_bytes": (ctypes.c_int64, []),
    "nb200_gemm_plan": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, ctypes.POINTER(GemmConfig), _vp, _vp,
                                       _vp, ctypes.POINTER(GemmLaunch)]),
    "nb200_repitch": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i64, _i64, _i64, ctypes.c_int, _vp]),
    "nb200_gemm_check": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64,
                                        ctypes.c_int, ctypes.POINTER(GemmConfig)]),
    "nb200_attention_fwd": (ctypes.c_int, [_vp, _vp, _vp, _vp] + [_i64] * 12 +
                            [ctypes.c_float, ctypes.c_int, ctypes.c_int, _vp]),
}

_lib = None


def load():
    """Returns the loaded library; raises if it was never built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m newt_b200.csrc.build` "
            f"(nvcc, sm_100a). newt_b200 has no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error():
    return load().nb200_last_error().decode("utf-8", "replace")


def check(code):
    """Turns a status code of the C ABI into a Python exception."""
    if code == OK:
        return
    msg = last_error()
    if code == E_UNSUPPORTED:
        raise UnsupportedError(code, msg)
    raise KernelLibraryError(code, msg)


def set_tuning(key, value):
    check(load().nb200_set_tuning(key.encode(), int(value)))


def read_status():
    """Synchronises and raises if a kernel gave up on a bounded wait."""
    st, det = ctypes.c_uint32(0), ctypes.c_uint32(0)
    check(load().nb200_read_status(ctypes.byref(st), ctypes.byref(det)))
    return st.value, det.value


_dtype_codes = {}


def dtype_code(torch_dtype):
    if not _dtype_codes:
        import torch

        _dtype_codes.update({torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16})
    code = _dtype_codes.get(torch_dtype)
    if code is None:
        raise TypeError(f"dtype {torch_dtype} has no kernel in libnewt_b200")
    return code
