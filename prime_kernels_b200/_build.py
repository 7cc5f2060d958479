"""In-tree build of the sm_100a shared libraries (no JIT cache, no pip install).

    python -m prime_kernels_b200._build          # build what is stale
    python -m prime_kernels_b200._build --force

Outputs (git-ignored, next to the sources so they travel with the tree):
    prime_kernels_b200/lib/libprime_kernels_b200.so        kernels + C ABI (nvcc, no torch)
    prime_kernels_b200/lib/libprime_kernels_b200_torch.so  TORCH_LIBRARY ops over the C ABI (g++)
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = LIB / "obj"
CUDA_SOURCES = ["rmsnorm_mxfp8.cu", "decode_megakernel.cu", "elementwise_ops.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA extension cannot be built")
    return exe


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def build_kernels(force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh"))
    flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
    jobs = []
    for name in CUDA_SOURCES:
        src, obj = CSRC / name, OBJ / (name + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append([_nvcc(), *flags, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=max(1, len(jobs))) as pool:
        list(pool.map(_run, jobs))
    out = LIB / "libprime_kernels_b200.so"
    objs = [OBJ / (n + ".o") for n in CUDA_SOURCES]
    if force or jobs or _stale(out, objs):
        _run([_nvcc(), "-shared", "-o", str(out), *map(str, objs), "-lcudart"])
    return out


def build_binding(force: bool = False) -> Path:
    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch_binding.cpp"
    header = PKG.parent / "include" / "prime_kernels_b200.h"
    out = LIB / "libprime_kernels_b200_torch.so"
    if not (force or _stale(out, [src, header, LIB / "libprime_kernels_b200.so"])):
        return out
    inc = [f"-I{p}" for p in cpp_extension.include_paths()] + ["-I/usr/local/cuda/include"]
    libdirs = cpp_extension.library_paths()
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
           "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, str(src), "-o", str(out),
           f"-L{LIB}", "-lprime_kernels_b200", *[f"-L{d}" for d in libdirs],
           "-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda",
           "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN"]
    _run(cmd)
    return out


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_binding(force)


if __name__ == "__main__":
    build_all("--force" in sys.argv)
    print("built", *(p.name for p in sorted(LIB.glob("*.so"))))
