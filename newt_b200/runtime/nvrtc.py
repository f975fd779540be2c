"""Run-time compilation of generated CUDA for sm_100a: NVRTC -> cubin -> module -> launch.

The five hot programs run through the prebuilt library; programs outside them that are pure
block arithmetic (newt_b200/frontend/pointwise.py) are compiled here, the way the reference
compiles everything (newt/runtime/cuda.py:124-154 `compile_cuda`, :177-234 `Kernel`): NVRTC
with `--gpu-architecture=sm_100a`, the cubin loaded with the driver API and launched on
torch's current stream.  libnvrtc and libcuda are bound with ctypes; nothing here touches the
device until a kernel is launched.
"""

import ctypes
import os
import threading

_lock = threading.Lock()
_nvrtc = None
_cuda = None


class NVRTCError(RuntimeError):
    """Compilation failed; the message carries the log and the numbered source
    (newt/runtime/jit.py:58-61 does the same)."""


class CUDAError(RuntimeError):
    pass


def _load_nvrtc():
    global _nvrtc
    if _nvrtc is None:
        last = None
        for name in ("libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so",
                     "libnvrtc.so.13"):
            try:
                _nvrtc = ctypes.CDLL(name)
                break
            except OSError as e:
                last = e
        if _nvrtc is None:
            raise NVRTCError(f"libnvrtc is not loadable: {last}")
    return _nvrtc


def _load_cuda():
    global _cuda
    if _cuda is None:
        try:
            _cuda = ctypes.CDLL("libcuda.so.1")
        except OSError as e:
            raise CUDAError(f"libcuda.so.1 is not loadable (no NVIDIA driver?): {e}") from e
    return _cuda


def _numbered(source):
    return "\n".join(f"{i + 1:4d} | {line}" for i, line in enumerate(source.splitlines()))


def compile_cubin(source, name="kernel.cu", arch="sm_100a", extra_opts=()):
    """CUDA C++ text -> cubin bytes for `arch`.  Works without a GPU."""
    lib = _load_nvrtc()
    prog = ctypes.c_void_p()
    rc = lib.nvrtcCreateProgram(ctypes.byref(prog), source.encode(), name.encode(), 0, None, None)
    if rc != 0:
        raise NVRTCError(f"nvrtcCreateProgram failed with code {rc}")
    try:
        include = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"
        opts = [f"--gpu-architecture={arch}", "--std=c++17", "-lineinfo", f"-I{include}",
                *extra_opts]
        arr = (ctypes.c_char_p * len(opts))(*[o.encode() for o in opts])
        rc = lib.nvrtcCompileProgram(prog, len(opts), arr)
        if rc != 0:
            size = ctypes.c_size_t()
            lib.nvrtcGetProgramLogSize(prog, ctypes.byref(size))
            log = ctypes.create_string_buffer(size.value or 1)
            lib.nvrtcGetProgramLog(prog, log)
            raise NVRTCError(f"NVRTC could not compile {name}:\n{log.value.decode(errors='replace')}\n"
                             f"{_numbered(source)}")
        size = ctypes.c_size_t()
        if lib.nvrtcGetCUBINSize(prog, ctypes.byref(size)) != 0 or size.value == 0:
            raise NVRTCError(f"NVRTC produced no cubin for {arch}")
        cubin = ctypes.create_string_buffer(size.value)
        if lib.nvrtcGetCUBIN(prog, cubin) != 0:
            raise NVRTCError("nvrtcGetCUBIN failed")
        return cubin.raw
    finally:
        lib.nvrtcDestroyProgram(ctypes.byref(prog))


def device_headers():
    """The folder of the kernel library's device templates (sm100.cuh, gemm_device.cuh): kernels
    compiled at run time from them get it as an include path."""
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")


_headers_digest = None


def device_headers_digest():
    """Hash of the device templates' text: a kernel compiled from them is stale when they change,
    although its own source (which only includes them) does not."""
    global _headers_digest
    if _headers_digest is None:
        import hashlib

        h = hashlib.sha256()
        folder = device_headers()
        for name in sorted(os.listdir(folder)):
            if name.endswith(".cuh"):
                with open(os.path.join(folder, name), "rb") as f:
                    h.update(f.read())
        _headers_digest = h.hexdigest()[:16]
    return _headers_digest


def cache_dir():
    """Where compiled cubins are kept between processes: $NEWT_CACHE_DIR, else ~/.newt/cache
    (the reference's convention, newt/runtime/jit.py:21-24); None if it cannot be created."""
    d = os.environ.get("NEWT_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".newt", "cache")
    try:
        os.makedirs(d, exist_ok=True)
    except OSError:
        return None
    return d


def _nvrtc_version():
    major, minor = ctypes.c_int(), ctypes.c_int()
    if _load_nvrtc().nvrtcVersion(ctypes.byref(major), ctypes.byref(minor)) != 0:
        return "?"
    return f"{major.value}.{minor.value}"


def compile_cubin_cached(source, name="kernel.cu", arch="sm_100a", extra_opts=()):
    """`compile_cubin` behind a disk cache keyed by the source text, the architecture, the
    options and the NVRTC version (newt/runtime/jit.py:50-66 keeps cubins the same way).  The
    source is stored next to the cubin for inspection.  Files are written to a temporary name
    and renamed, so concurrent processes (one per GPU) never read a partial cubin; a cache
    that cannot be read or written is skipped, not an error."""
    import hashlib
    import tempfile

    d = cache_dir()
    if d is None:
        return compile_cubin(source, name, arch, extra_opts)
    key = hashlib.sha256("\0".join([source, arch, *extra_opts, _nvrtc_version(), "b200-1"]).encode()
                         ).hexdigest()[:32]
    path = os.path.join(d, f"{key}.cubin")
    try:
        with open(path, "rb") as f:
            cubin = f.read()
        if cubin[:4] == b"\x7fELF":
            return cubin
    except OSError:
        pass
    cubin = compile_cubin(source, name, arch, extra_opts)
    for suffix, payload in ((".cubin", cubin), (".cu", source.encode())):
        try:
            fd, tmp = tempfile.mkstemp(dir=d, suffix=".tmp")
            with os.fdopen(fd, "wb") as f:
                f.write(payload)
            os.replace(tmp, os.path.join(d, key + suffix))
        except OSError:
            break
    return cubin


def _check(rc, what):
    if rc != 0:
        msg = ctypes.c_char_p()
        _load_cuda().cuGetErrorString(rc, ctypes.byref(msg))
        raise CUDAError(f"{what} failed: {msg.value.decode() if msg.value else rc}")


class Kernel:
    """One function of a cubin, loaded per device on first launch."""

    def __init__(self, cubin, func_name):
        self.cubin = cubin
        self.func_name = func_name
        self._functions = {}   # device index -> CUfunction
        self._shared = {}      # device index -> dynamic shared memory the function is opted in for

    def _function(self):
        import torch

        dev = torch.cuda.current_device()
        fn = self._functions.get(dev)
        if fn is None:
            with _lock:
                fn = self._functions.get(dev)
                if fn is None:
                    torch.cuda.init()
                    torch.zeros(1, device=f"cuda:{dev}")   # makes the primary context current
                    cu = _load_cuda()
                    module = ctypes.c_void_p()
                    _check(cu.cuModuleLoadData(ctypes.byref(module), self.cubin), "cuModuleLoadData")
                    fn = ctypes.c_void_p()
                    _check(cu.cuModuleGetFunction(ctypes.byref(fn), module, self.func_name.encode()),
                           "cuModuleGetFunction")
                    self._functions[dev] = fn
        return fn

    def launch(self, grid, block, args, stream, shared_bytes=0, cluster=None):
        """`args`: ctypes values in parameter order (structures and raw buffers are passed by
        value: a `__grid_constant__ CUtensorMap` parameter is what `new_tensor_map` returns); `stream`: a
        CUstream handle (int); `shared_bytes`: dynamic shared memory (above 48 KB the function
        is opted in first); `cluster`: thread blocks per cluster along x, for kernels whose
        CTAs work in clusters (launched through cuLaunchKernelEx with the cluster-dimension
        attribute)."""
        import torch

        cu = _cuda or _load_cuda()
        dev = torch.cuda.current_device()
        fn = self._functions.get(dev) or self._function()
        if shared_bytes > 48 * 1024 and self._shared.get(dev, 0) < shared_bytes:
            # CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES = 8
            _check(cu.cuFuncSetAttribute(fn, 8, ctypes.c_int(shared_bytes)), "cuFuncSetAttribute")
            self._shared[dev] = shared_bytes
        g = tuple(grid) + (1,) * (3 - len(grid))
        b = (block, 1, 1) if isinstance(block, int) else tuple(block) + (1,) * (3 - len(block))
        ptrs = (ctypes.c_void_p * len(args))(*map(ctypes.addressof, args))
        if cluster is None:
            _check(cu.cuLaunchKernel(fn, g[0], g[1], g[2], b[0], b[1], b[2], shared_bytes,
                                     ctypes.c_void_p(stream), ptrs, None), f"launch of {self.func_name}")
            return
        attr = _LaunchAttribute()
        attr.id = 4                                  # CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION
        attr.value.cluster_dim[:] = [int(cluster), 1, 1]
        config = _LaunchConfig(g[0], g[1], g[2], b[0], b[1], b[2], shared_bytes,
                               ctypes.c_void_p(stream), ctypes.pointer(attr), 1)
        _check(cu.cuLaunchKernelEx(ctypes.byref(config), fn, ptrs, None),
               f"cluster launch of {self.func_name}")


class _LaunchAttributeValue(ctypes.Union):       # CUlaunchAttributeValue: 64 bytes
    _fields_ = [("pad", ctypes.c_char * 64), ("cluster_dim", ctypes.c_uint * 3)]


class _LaunchAttribute(ctypes.Structure):        # CUlaunchAttribute
    _fields_ = [("id", ctypes.c_int), ("pad", ctypes.c_char * 4), ("value", _LaunchAttributeValue)]


class _LaunchConfig(ctypes.Structure):           # CUlaunchConfig
    _fields_ = [("grid_x", ctypes.c_uint), ("grid_y", ctypes.c_uint), ("grid_z", ctypes.c_uint),
                ("block_x", ctypes.c_uint), ("block_y", ctypes.c_uint), ("block_z", ctypes.c_uint),
                ("shared_bytes", ctypes.c_uint), ("stream", ctypes.c_void_p),
                ("attrs", ctypes.POINTER(_LaunchAttribute)), ("num_attrs", ctypes.c_uint)]


def new_tensor_map():
    """Storage for a CUtensorMap passed by value: sixteen 64-bit words on a 64-byte boundary
    (ctypes cannot ask for the alignment, so the words are a view into a larger buffer)."""
    raw = (ctypes.c_char * 192)()
    view = (ctypes.c_uint64 * 16).from_buffer(raw, (-ctypes.addressof(raw)) % 64)
    return view


_DATA_TYPES = {1: 0, 2: 1, 4: 2}     # bytes per element -> CU_TENSOR_MAP_DATA_TYPE_UINT8/16/32


def encode_tiled(address, elem_bytes, dims, strides_bytes, box, swizzle_128b=True):
    """cuTensorMapEncodeTiled for a row-major tensor: `dims` innermost first, `strides_bytes` of
    every dimension but the innermost, `box` the tile a copy moves.  No interleave, zero fill
    out of range, 256-byte L2 promotion, 128-byte swizzle unless told otherwise."""
    cu = _load_cuda()
    rank = len(dims)
    tmap = new_tensor_map()
    rc = cu.cuTensorMapEncodeTiled(
        ctypes.byref(tmap), _DATA_TYPES[elem_bytes], rank, ctypes.c_void_p(address),
        (ctypes.c_uint64 * rank)(*dims), (ctypes.c_uint64 * max(rank - 1, 1))(*strides_bytes),
        (ctypes.c_uint32 * rank)(*box), (ctypes.c_uint32 * rank)(*([1] * rank)),
        0, 3 if swizzle_128b else 0, 2, 0)
    _check(rc, "cuTensorMapEncodeTiled")
    return tmap
