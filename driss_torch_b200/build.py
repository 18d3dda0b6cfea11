"""In-tree build of the two shared libraries (no cmake, no JIT cache).

* ``lib/libdtq_b200.so``   -- the torch-free CUDA kernels and their C ABI
  (``include/dtq_b200.h``), built with nvcc for sm_100a only.
* ``lib/libdriss_torch.so`` -- ``register_ops.cpp``: the ``TORCH_LIBRARY(DrissTorch)``
  registration that binds the C ABI into the PyTorch dispatcher, built with g++.

``python driss_torch_b200/build.py`` builds both; objects are rebuilt only when a
source or header is newer.  The reference builds one ``libdriss_torch.so`` through
scikit-build/CMake with the same architecture flags (CMakeLists.txt:25-27).
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = PKG / "build"
INCLUDE = ROOT / "include"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

KERNEL_SOURCES = [
    "common.cu",
    "saturated_cast.cu",
    "saturated_cast_t.cu",
    "amax.cu",
    "dynamic_scaled_quant.cu",
    "rowwise_quant.cu",
    "mx_cast.cu",
    "mx_cast_tma.cu",
    "mx_cast_dual.cu",
    "mx_cast_formats.cu",
    "mx_cast_amax.cu",
    "mx_gemm.cu",
]

NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "-Xptxas",
    "-v",
    "--cudart",
    "shared",
]


def _newest(paths) -> float:
    return max(p.stat().st_mtime for p in paths)


def _headers():
    return list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))


def _run(cmd, log: Path | None = None) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd)))


def build_kernels(force: bool = False, extra_flags=()) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    dep_time = _newest(_headers() + [Path(__file__)])
    jobs = []
    objs = []
    for name in KERNEL_SOURCES:
        src = CSRC / name
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, dep_time):
            cmd = [NVCC, *NVCC_FLAGS, *extra_flags, "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
            jobs.append((cmd, OBJ / (src.stem + ".ptxas.log")))
    with ThreadPoolExecutor(max_workers=max(1, min(len(jobs), os.cpu_count() or 1))) as pool:
        list(pool.map(lambda j: _run(*j), jobs))
    so = LIB / "libdtq_b200.so"
    if force or jobs or not so.exists():
        _run([NVCC, "-shared", "--cudart", "shared", "-o", str(so), *map(str, objs),
              "-Xlinker", "-rpath", "-Xlinker", str(CUDA_HOME / "lib64")])
    return so


def build_torch_binding(force: bool = False) -> Path:
    import torch
    from torch.utils.cpp_extension import include_paths

    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    src = CSRC / "register_ops.cpp"
    so = LIB / "libdriss_torch.so"
    kernels = LIB / "libdtq_b200.so"
    dep_time = max(src.stat().st_mtime, _newest(list(INCLUDE.glob("*.h"))))
    if not (force or not so.exists() or so.stat().st_mtime < dep_time):
        return so
    torch_lib = Path(torch.__file__).parent / "lib"
    incs = [f"-I{p}" for p in include_paths("cuda")] + [f"-I{INCLUDE}", f"-I{sysconfig.get_paths()['include']}"]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        "g++", "-std=c++17", "-O2", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", *incs, str(src),
        "-o", str(so),
        f"-L{LIB}", "-ldtq_b200", f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
        f"-L{CUDA_HOME / 'lib64'}", "-lcudart",
        "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}", f"-Wl,-rpath,{CUDA_HOME / 'lib64'}",
    ]
    assert kernels.exists(), "build the kernel library first"
    _run(cmd)
    return so


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_torch_binding(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", *(p.name for p in sorted(LIB.glob("*.so"))))
