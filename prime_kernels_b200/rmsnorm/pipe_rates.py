"""Builds (nvcc, sm_100a) and runs the instruction-throughput probe ``pipe_rates.cu`` on the current GPU.

    python -m prime_kernels_b200.rmsnorm.pipe_rates

The figures it prints (thread-ops per clock per SM) are the ones the arithmetic of the fused RMSNorm + MXFP8
kernels was chosen by: mixed ``fma.rn.f32.bf16`` and ``abs.bf16x2`` issue at half rate, the FP8 / E8M0 conversions
at about a sixth, ``max.bf16x2`` and plain fp32 FMA at full rate.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
import tempfile
from pathlib import Path


def main() -> int:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src = Path(__file__).with_name("pipe_rates.cu")
    with tempfile.TemporaryDirectory() as tmp:
        exe = Path(tmp) / "pipe_rates"
        subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-o", str(exe), str(src)],
                       check=True)
        return subprocess.run([str(exe)]).returncode


if __name__ == "__main__":
    sys.exit(main())
