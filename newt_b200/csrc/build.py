"""Builds libnewt_b200.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

Usage:  python -m newt_b200.csrc.build [--force] [--verbose]
"""

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libnewt_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def headers():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cuh")) + [
        os.path.join("..", "..", "include", "newt_b200.h")]


def _nvcc():
    cuda_home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def _digest(paths):
    """Hash of the files' contents and the compiler flags: what an object was built from."""
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target, deps):
    """An object is current when the digest stored beside it matches its sources.  Contents,
    not modification times: a copy of the tree to another machine keeps objects valid."""
    stamp = target + ".sha256"
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != _digest(deps)


def build(force=False, verbose=False):
    """Compiles every .cu under csrc/ and links the shared library. Returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = [os.path.join(HERE, h) for h in headers()] + [os.path.abspath(__file__)]
    objs, procs, digests = [], [], {}
    for src in sources():
        obj = os.path.join(OBJ_DIR, src[:-3] + ".o")
        objs.append(obj)
        deps = [os.path.join(HERE, src)] + hdrs
        if force or _stale(obj, deps):
            digests[src] = (obj, _digest(deps))
            cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + [
                "-c", os.path.join(HERE, src), "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE,
                                                stderr=subprocess.STDOUT, text=True)))
    failed = []
    for src, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(f"--- nvcc {src} ---\n{out}\n")
        if p.returncode != 0:
            failed.append(src)
        else:
            obj, digest = digests[src]
            with open(obj + ".sha256", "w") as f:
                f.write(digest)
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    if force or procs or not os.path.exists(LIB) or \
            any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [_nvcc(), "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
