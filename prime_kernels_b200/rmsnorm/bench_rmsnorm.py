"""Bandwidth table for the fused RMSNorm + residual + MXFP8 kernel.

    python -m prime_kernels_b200.rmsnorm.bench_rmsnorm [--pool-gib 2] [--reps 3] [--json]

Method follows the reference's benchmark (prime_kernels/rmsnorm/bench.cu:80-84,119-134): inputs rotate
through a pool much larger than L2 so no iteration re-reads cached lines, enough launches per
measurement to cover >= 20 ms, fastest of `reps`; GB/s uses the reference's traffic model
N*C*(2+2+1) + 4*N.  Launches go through the C ABI with preallocated outputs (no allocator in the loop).
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from .._cabi import library

CONFIG3 = [(m, c) for c in (960, 2048, 4096) for m in (1, 16, 128, 1024, 8192)]
REFERENCE_SWEEP = [(n, c) for n in (1024, 8192, 65536) for c in (1024, 2048, 4096, 8192, 16384)]


def measure(n, c, pool_elems, reps, dev):
    lib = library()
    shape = n * c
    slices = max(1, pool_elems // shape)
    branch = torch.randn(slices * shape, device=dev, dtype=torch.bfloat16)
    resid = torch.randn(slices * shape, device=dev, dtype=torch.bfloat16)
    weight = (1 + 0.1 * torch.randn(c, device=dev)).to(torch.bfloat16)
    vals = torch.empty(slices * shape, device=dev, dtype=torch.uint8)
    sb = lib.pk_rmsnorm_scale_bytes(n, c)
    scales = torch.empty(slices * sb, device=dev, dtype=torch.uint8)
    rrms = torch.empty(slices * n, device=dev, dtype=torch.float32)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def launch(i):
        nonlocal stream
        k = i % slices
        rc = lib.pk_fused_rmsnorm_residual_forward(vals.data_ptr() + k * shape, scales.data_ptr() + k * sb,
                                                   rrms.data_ptr() + 4 * k * n, branch.data_ptr() + 2 * k * shape,
                                                   resid.data_ptr() + 2 * k * shape, weight.data_ptr(), 1e-6, n, c, stream)
        assert rc == 0, rc

    for i in range(5):
        launch(i)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    launch(0)
    e1.record()
    torch.cuda.synchronize(dev)
    one = max(e0.elapsed_time(e1), 1e-3)
    per_graph = int(min(max(slices, 8), 256))
    # a CUDA graph of `per_graph` launches over rotating pool slices removes the per-launch host cost
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream(dev)
    with torch.cuda.stream(side):
        stream = side.cuda_stream
        with torch.cuda.graph(graph, stream=side):
            for i in range(per_graph):
                launch(i)
    torch.cuda.synchronize(dev)
    replays = int(min(max(20.0 / (one * per_graph), 3), 2000))
    best = float("inf")
    for _ in range(reps):
        e0.record()
        for _ in range(replays):
            graph.replay()
        e1.record()
        torch.cuda.synchronize(dev)
        best = min(best, e0.elapsed_time(e1) / (replays * per_graph))
    traffic = n * c * 5 + 4 * n
    return best * 1e3, traffic / (best * 1e-3) / 1e9


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--pool-gib", type=float, default=2.0)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--sweep", default="both", choices=["config3", "reference", "both"])
    args = ap.parse_args()
    dev = torch.device("cuda:0")
    peaks = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks.read_text())["hbm_gbs"] if peaks.exists() else 6650.0
    pool_elems = int(args.pool_gib * (1 << 30) / 2)
    shapes = (CONFIG3 if args.sweep in ("config3", "both") else []) + (REFERENCE_SWEEP if args.sweep in ("reference", "both") else [])
    rows = []
    for n, c in shapes:
        us, gbs = measure(n, c, pool_elems, args.reps, dev)
        rows.append({"N": n, "C": c, "us": round(us, 2), "GB/s": round(gbs, 1), "frac_of_measured_peak": round(gbs / peak, 3)})
        if not args.json:
            print(f"N={n:6d} C={c:6d}  {us:9.2f} us  {gbs:8.1f} GB/s  {gbs / peak:6.3f} of measured {peak:.0f} GB/s", flush=True)
    if args.json:
        print(json.dumps({"peak_gbs": peak, "rows": rows}))


if __name__ == "__main__":
    main()
