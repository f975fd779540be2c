"""The reference's low-level runtime interface, kept by name: NVRTC compile + driver launch on
raw ctypes arguments, no compiler in between (newt/runtime/cuda.py:124-154 `compile_cuda`,
:177-234 `Kernel`; exercised by tests/test_runtime_smoke.py).  Both are thin fronts of
runtime/nvrtc.py, which the generic lowering uses for its own kernels; the default
architecture is sm_100a.
"""

from . import nvrtc
from .nvrtc import CUDAError, NVRTCError  # noqa: F401  (re-exported)


def compile_cuda(source, name, arch="sm_100a", extra_opts=()):
    """CUDA C++ text -> cubin bytes for `arch` (`name` labels the translation unit)."""
    return nvrtc.compile_cubin(source, f"{name}.cu", arch, extra_opts)


class Kernel(nvrtc.Kernel):
    """A function of a cubin, launchable with a list of ctypes objects.  `shared_bytes` is the
    dynamic shared memory every launch asks for (opted in above 48 KB)."""

    def __init__(self, cubin, func_name, shared_bytes=0):
        super().__init__(cubin, func_name)
        self.shared_bytes = int(shared_bytes)

    def launch(self, grid, block, args, stream=0):
        super().launch(grid, block, args, stream, self.shared_bytes)
