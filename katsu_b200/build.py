"""In-tree build of the native libraries (no JIT cache, no pip install).

  katsu_b200/lib/libkatsu_cuda.so   csrc/*.cu, sm_100a only, the C ABI of include/katsu_cuda.h
  katsu_b200/lib/libkatsu_host.so   csrc/host/*.cpp, the C++ mirror of katsu-core's Tensor/Conv2D
                                    graph, calling the kernels only through that C ABI

Run as `python -m katsu_b200.build` (add --force to rebuild everything).
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
OBJ = os.path.join(PKG, "build")
INCLUDE = os.path.join(ROOT, "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
    "-I", INCLUDE, "-I", CSRC,
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wextra", "-I", INCLUDE, "-I", os.path.join(CSRC, "host")]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")


def _gxx() -> str:
    # The image exports CXX=/opt/gcc/bin/g++ for nvcc's benefit; the plain PATH compiler is the complete one.
    return shutil.which("g++") or "g++"


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str], log: str | None = None) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log:
        with open(log, "w") as fh:
            fh.write(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))


def build_cuda(force: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(INCLUDE, "katsu_cuda.h"))
    sources = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    objects, jobs = [], []
    for src in sources:
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objects.append(obj)
        if force or _newer(obj, [src] + headers):
            jobs.append(([nvcc, *NVCC_FLAGS, "-c", src, "-o", obj], obj[:-2] + ".ptxas.log"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        for fut in [pool.submit(_run, cmd, log) for cmd, log in jobs]:
            fut.result()
    out = os.path.join(LIB, "libkatsu_cuda.so")
    if force or jobs or _newer(out, objects):
        _run([nvcc, "-shared", "-cudart", "static", "-o", out, *objects, "-ldl"])
    return out


def build_host(force: bool = False) -> str:
    os.makedirs(LIB, exist_ok=True)
    host_dir = os.path.join(CSRC, "host")
    sources = sorted(os.path.join(host_dir, f) for f in os.listdir(host_dir) if f.endswith(".cpp"))
    headers = [os.path.join(host_dir, f) for f in os.listdir(host_dir) if f.endswith((".hpp", ".h"))]
    headers.append(os.path.join(INCLUDE, "katsu_cuda.h"))
    out = os.path.join(LIB, "libkatsu_host.so")
    if force or _newer(out, sources + headers + [os.path.join(LIB, "libkatsu_cuda.so")]):
        _run([_gxx(), *CXX_FLAGS, "-shared", "-o", out, *sources, "-L", LIB, "-lkatsu_cuda",
              "-Wl,-rpath,$ORIGIN"])
    return out


def build_all(force: bool = False) -> None:
    build_cuda(force)
    build_host(force)


if __name__ == "__main__":
    build_all("--force" in sys.argv)
    print("built", os.listdir(LIB))
