"""Builds the CUDA kernel library (``libnvk.so``) in-tree with nvcc for sm_100a.

The library is the product: a C-ABI shared object (``include/nvk.h``) with no dependency on
torch or Python.  Object files go to ``nano-vllm-cpp_b200/build/``; the shared object sits next
to this file so that it travels with the source tree.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libnvk.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    """Every header an object may depend on: csrc/*.cuh, csrc/*.h and the C ABI header."""
    files = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    files.append(os.path.join(os.path.dirname(HERE), "include", "nvk.h"))
    return files


def _deps_mtime() -> float:
    return max(os.path.getmtime(f) for f in sources() + _headers())


def _compile(src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    hdr_time = max(os.path.getmtime(f) for f in _headers())
    if os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(src), hdr_time):
        return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".ptxas.log")
    with open(log, "w") as fh:
        fh.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    if force:
        for f in os.listdir(OBJ_DIR):
            if f.endswith(".o"):
                os.remove(os.path.join(OBJ_DIR, f))
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose), sources()))
    cmd = [nvcc(), "-shared", "-o", LIB, *objs, "-lcudart"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


HOST_DIR = os.path.join(HERE, "host")
HOST_LIB = os.path.join(HERE, "libnvk_host.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _gxx() -> str:
    for cand in ("/usr/bin/g++", shutil.which("g++")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("g++ not found")


def build_host(force: bool = False) -> str:
    """Builds the C++ operator layer (``libnvk_host.so``: Tensor, Context, operators, Attention layer,
    step metadata) on top of ``libnvk.so`` and its two test programs under ``build/``."""
    build()
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sorted(os.path.join(HOST_DIR, "src", f) for f in os.listdir(os.path.join(HOST_DIR, "src")) if f.endswith(".cpp"))
    hdrs = [os.path.join(dp, f) for dp, _, fs in os.walk(os.path.join(HOST_DIR, "include")) for f in fs]
    hdrs.append(os.path.join(os.path.dirname(HERE), "include", "nvk.h"))
    newest = max(os.path.getmtime(f) for f in srcs + hdrs + [LIB])
    inc = ["-I", os.path.join(HOST_DIR, "include"), "-I", os.path.join(os.path.dirname(HERE), "include"),
           "-I", os.path.join(CUDA_HOME, "include")]
    common = [_gxx(), "-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", *inc]
    link = ["-L", HERE, "-L", os.path.join(CUDA_HOME, "lib64"), "-lnvk", "-lcudart", "-Wl,-rpath,$ORIGIN"]
    if force or not os.path.exists(HOST_LIB) or os.path.getmtime(HOST_LIB) < newest:
        res = subprocess.run([*common, "-shared", "-o", HOST_LIB, *srcs, *link], capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"host layer build failed:\n{res.stdout}\n{res.stderr}")
    tests_dir = os.path.join(HOST_DIR, "tests")
    for name in sorted(f[:-4] for f in os.listdir(tests_dir) if f.endswith(".cpp")):
        exe = os.path.join(OBJ_DIR, name)
        src = os.path.join(tests_dir, name + ".cpp")
        dep = max(os.path.getmtime(src), os.path.getmtime(os.path.join(tests_dir, "check.h")), os.path.getmtime(HOST_LIB))
        if force or not os.path.exists(exe) or os.path.getmtime(exe) < dep:
            res = subprocess.run([*common, "-o", exe, src, "-L", HERE, "-L", os.path.join(CUDA_HOME, "lib64"),
                                  "-lnvk_host", "-lnvk", "-lcudart", "-Wl,-rpath,$ORIGIN/.."], capture_output=True, text=True)
            if res.returncode != 0:
                raise RuntimeError(f"host test build failed ({name}):\n{res.stdout}\n{res.stderr}")
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_host(force="--force" in sys.argv))
