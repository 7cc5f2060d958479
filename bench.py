#!/usr/bin/env python
"""Benchmark of the decode hot path: SmolLM2-360M, batch 1, bf16, 512-token prompt then greedy decode
steps through the single-launch megakernel (one "step" = one decode step = one kernel launch).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints ONE JSON line.  `value` is tokens/s with every input resident in HBM (device-driven greedy
loop, CUDA events on the launching stream, max over ranks); `e2e` is the same metric through the
public `decode_step` API with host buffers (per step: pinned-host -> device copy of the step inputs,
launch, device -> host read of the greedy id); `roofline` relates the algorithmic bytes of a step
(weights + KV read) to the measured HBM copy bandwidth; `cpu_baseline` times the reference's own
oracle (HuggingFace eager bf16 on the host cores) on a bounded sample of the same workload.
N > 1 runs one independent replica per GPU (batch-1 decode does not shard; no collective on the
data path).  Inputs: random-init weights (seed 0), seeded uniform prompt ids; synthetic.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (geometry name, batch, context tokens before timing, default steps)
    "smollm2-360m-b1": ("smollm2-360m", 1, 512, 256),            # the headline: 512-token prompt, 256 greedy steps
    "smollm2-135m-b1": ("smollm2-135m", 1, 32, 64),              # 32-token prompt, 64 greedy steps
    "smollm2-1.7b-b1": ("smollm2-1.7b", 1, 1024, 256),           # 1024-token prompt, 256 steps
    "smollm2-1.7b-b8": ("smollm2-1.7b", 8, 1024, 64),
    "smollm2-1.7b-b64": ("smollm2-1.7b", 64, 1024, 16),
    "smollm2-360m-b4": ("smollm2-360m", 4, 512, 256),
    "smollm2-360m-b8": ("smollm2-360m", 8, 512, 256),
    # MXFP8 weights (E4M3 + E8M0 per 32 along K), context pre-filled to 4096 with normal(0,1) K/V, 128 steps
    "smollm2-360m-mxfp8-b1": ("smollm2-360m", 1, 4096, 128),
    "smollm2-360m-mxfp8-b4": ("smollm2-360m", 4, 4096, 128),
    "smollm2-360m-mxfp8-b16": ("smollm2-360m", 16, 4096, 32),
    "smollm2-1.7b-mxfp8-b1": ("smollm2-1.7b", 1, 1024, 128),
}
METRIC = "SmolLM2-360M bs1 decode tok/s & % HBM roofline; aggregate tok/s @1/2/4/8 GPUs"
# DRAM bytes per launch measured with ncu (dram__bytes_read + write) divided by the algorithmic bytes of the
# captured launch: decode_fast_kernel, SmolLM2-360M batch 1 at context 503-505: 747.7 MB / 744.3 MB;
# decode_fast_kernel, SmolLM2-1.7B batch 1 at context 203: 3467 MB / 3463 MB;
# decode_batched_kernel, SmolLM2-360M MXFP8 batch 16 at context 1027: 1051.7 MB / 1046.6 MB.  Traffic grows with
# the same units as the algorithmic bytes (weights + KV positions), so other contexts are scaled by them.
NCU_TRAFFIC_RATIO = {("smollm2-360m", 1, False): (1.005, "ncu capture of decode_fast_kernel at context 503-505"),
                     ("smollm2-1.7b", 1, False): (1.001, "ncu capture of decode_fast_kernel at context 203"),
                     ("smollm2-360m", 16, True): (1.005, "ncu capture of decode_batched_kernel at context 1027")}


def algorithmic_bytes(geom, batch, seq, mxfp8=False):
    """Bytes one decode step must move: every weight once (bf16, or E4M3 + one E8M0 per 32 for the matrices
    when `mxfp8`) + K/V of `seq` positions per request."""
    matrices = geom.layers * (geom.qkv_rows * geom.hidden + geom.hidden * geom.q_heads * 64
                              + 3 * geom.intermediate * geom.hidden) + geom.vocab * geom.hidden
    norms = geom.layers * 2 * geom.hidden + geom.hidden
    kv = 2 * geom.layers * geom.kv_heads * 64 * 2 * seq * batch
    if mxfp8:
        return matrices + matrices // 32 + 2 * norms + kv
    return 2 * (matrices + norms) + kv


class ClockSampler:
    """SM clock / throttle-reason samples taken while the timed region runs.  Read-only NVML queries from a
    thread of this process every 2 ms (an `nvidia-smi -lms` child needs longer to start than the timed
    region lasts); falls back to an `nvidia-smi` child when the NVML binding is missing."""

    REASONS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.thread = index, [], None, None
        self.stop = threading.Event()
        self.nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
        except Exception:
            self.nvml = None

    def _poll_nvml(self):
        n = self.nvml
        while not self.stop.is_set():
            try:
                mhz = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                try:
                    mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except AttributeError:
                    mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.rows.append((mhz, self.max_mhz, mask))
            except Exception:
                pass
            self.stop.wait(0.002)

    def _read_smi(self):
        for line in self.proc.stdout:
            c = [x.strip() for x in line.split(",")]
            if len(c) >= 6 and c[0].isdigit() and c[1].isdigit():
                mask = 0
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[2:6]):
                    if v.lower() == "active":
                        mask |= self.REASONS[name]
                self.rows.append((int(c[0]), int(c[1]), mask))

    def __enter__(self):
        self.stop.clear()
        if self.nvml is not None:
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return self
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.stop.set()
        if self.nvml is not None and self.thread is not None:
            self.thread.join(timeout=2)
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [r[0] for r in self.rows]
        mx = [r[1] for r in self.rows]
        mask = 0
        for r in self.rows:
            mask |= r[2]
        reasons = sorted(n for n, bit in self.REASONS.items() if mask & bit)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "source": "nvml" if self.nvml is not None else "nvidia-smi"}


def max_over_ranks(values, world, device="cpu"):
    """Element-wise maximum of `values` (list of floats) over all ranks of the default process group;
    with one rank it is the identity.  The timings of a replica run are reduced with this, so the
    reported throughput is bounded by the slowest replica."""
    import torch

    t = torch.tensor(values, dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def aggregate_throughput(world, batch, steps, ms_max):
    """Whole-job tokens/s of `world` independent replicas that each decoded `steps` tokens for `batch`
    requests within `ms_max` milliseconds (the slowest replica's time)."""
    return world * batch * steps / (ms_max * 1e-3)


def cpu_reference(geom, batch, prompt_len, sample_steps, seed=1234, warmup_steps=3):
    """HuggingFace eager bf16 decode on the host cores: prefill the prompt, `warmup_steps` untimed decode steps,
    then time `sample_steps` decode steps.  Returns (tok/s, threads, description)."""
    import torch

    from oracle import decode_hf
    from prime_kernels_b200 import harness

    # all host cores (torchrun pins OMP_NUM_THREADS=1 in its children; undo that for the CPU arm)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)))
    weights = harness.make_weights(geom, 0)
    prompt = torch.randint(0, geom.vocab, (batch, prompt_len), generator=torch.Generator().manual_seed(seed))
    res = decode_hf.run(geom, weights, prompt, sample_steps, warmup_steps=warmup_steps)
    toks = batch / res["seconds_per_step"]
    desc = (f"HF LlamaForCausalLM eager bf16 on CPU (the reference's own oracle), {geom.name} B={batch}, "
            f"{prompt_len}-token prompt prefilled and {warmup_steps} decode steps untimed, {sample_steps} timed decode steps")
    return toks, torch.get_num_threads(), desc


def config_block(wl, gname, batch, prompt_len, world):
    """The `config` object of a bench line: both arms print exactly this for the same workload (what differs
    between the arms goes into the line's `detail`)."""
    return {"workload": wl, "geometry": gname, "batch": batch, "prompt_tokens": prompt_len, "kv_block": 16,
            "replicas": world, "l2": "weights (>= 269 MB per step) exceed the 126 MB L2; no flush needed"}


def reference_cuda_kernel_same_box(geom, prompt_len, steps=20):
    """Supplementary to the CPU arm: the reference project's own decode kernel for this model (its 24-CTA sm_89
    design, compiled for sm_100a from the reference checkout by oracle/build_ref.sh with the device check shimmed),
    timed on this box's GPU at the workload's context with CUDA events.  Hidden-state step, no lm_head (the reference
    kernels have none).  Returns None when the oracle build or a GPU is missing."""
    import torch

    try:
        from oracle import ref_megakernel as REF
        from prime_kernels_b200 import harness
    except Exception:
        return None
    if not torch.cuda.is_available():
        return None
    if geom.name == "smollm2-360m" and REF.available_360m_fast():
        step, label = REF.decode_step_360m_fast, "decode_megakernel_360m_lossless (fast line, plain bf16 weights)"
    elif geom.name == "smollm2-135m" and REF.available():
        step, label = REF.decode_step, "decode_megakernel"
    else:
        return None
    dev = torch.device("cuda:0")
    weights = harness.weights_to(harness.make_weights(geom, 0), dev)
    cap = (prompt_len + 64 + 15) // 16 * 16
    kv = harness.PagedKV(geom, 1, cap, dev)
    for cache in kv.kv_caches:
        cache.normal_()
    pos = torch.tensor([prompt_len], dtype=torch.int64, device=dev)
    kw = dict(input_ids=torch.tensor([17], device=dev), positions=pos, seq_lens=(pos + 1).to(torch.int32),
              block_table=kv.block_table, slot_mapping=kv.slots(pos), embed=weights["embed"], layers=weights["layers"],
              final_norm=weights["final_norm"], kv_caches=kv.kv_caches,
              cos_sin_cache=harness.make_cos_sin_cache(geom, cap, dev), eps=1e-5)
    for _ in range(3):
        step(**kw)
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step(**kw)
    e1.record()
    torch.cuda.synchronize(dev)
    us = e0.elapsed_time(e1) / steps * 1e3
    return {"kernel": label, "us_per_step": round(us, 1), "tok_s": round(1e6 / us, 1), "context": prompt_len,
            "note": "the reference's CUDA kernel on this GPU (hidden-state step, no lm_head), CUDA events"}


def run_reference(args, wl):
    """The CPU arm: the reference's own oracle (HuggingFace eager bf16) on the host cores, a bounded sample of the
    same workload.  Imports nothing that loads the CUDA libraries of this repository; as a supplementary detail it
    also times the reference project's own CUDA kernel on this box when oracle/_ref holds its sm_100a build."""
    from prime_kernels_b200.geometry import GEOMETRIES

    gname, batch, prompt_len, _ = WORKLOADS[wl]
    if args.prompt_tokens:
        prompt_len = args.prompt_tokens
    geom = GEOMETRIES[gname]
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 16))          # bounded sample: at most 16 timed decode steps
    warm = max(3, min(args.warmup, 8))            # bounded like the sample
    toks, cores, desc = cpu_reference(geom, batch, prompt_len, steps, warmup_steps=warm)
    detail = {"note": "CPU arm: prompt prefilled and `warmup` decode steps untimed, then `steps` timed decode steps"}
    if batch == 1:
        try:
            same_box = reference_cuda_kernel_same_box(geom, prompt_len)
        except Exception as e:          # supplementary: never let it break the arm
            same_box = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
        if same_box:
            detail["reference_cuda_kernel_same_box"] = same_box
    line = {"metric": METRIC, "value": toks, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps,
            "steps_requested": args.steps, "warmup": warm, "ms_per_step": 1e3 * batch / toks, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": config_block(wl, gname, batch, prompt_len, int(os.environ.get("WORLD_SIZE", "1"))),
            "detail": detail,
            "cpu_baseline": {"value": toks, "unit": "tok/s", "cores": cores, "kind": "reference", "sample": desc},
            "e2e": {"value": toks, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def extra_measurements(dev, peak):
    """Secondary measurements of the same run (rank 0, one GPU): the fused RMSNorm + residual + MXFP8 kernel at
    three shapes with both traffic models, the reference project's own kernels on the same box when its
    benchmark executable was built (oracle/_ref), the CPU quantiser timed on the host, and short device-timed
    lines for the other two model sizes."""
    import subprocess as sp

    import numpy as np
    import torch

    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import harness
    from prime_kernels_b200.rmsnorm import bench_rmsnorm

    out = {"rmsnorm": [], "decode": []}
    pool = int(1.0 * (1 << 30) / 2)
    ref_bench = ROOT / "oracle" / "_ref" / "ref_rmsnorm_bench"
    for n, c in ((8192, 4096), (65536, 4096), (8192, 960)):
        us, gbs = bench_rmsnorm.measure(n, c, pool, 2, dev)
        full = n * c * 5 + n * ((c + 31) // 32) + 2 * c + 4 * n
        row = {"N": n, "C": c, "us": round(us, 2), "GBs_reference_model": round(gbs, 1),
               "GBs_full_model": round(full / (us * 1e-6) / 1e9, 1), "frac_of_measured_peak": round(gbs / peak, 3)}
        if ref_bench.exists() and c % 128 == 0:
            try:
                txt = sp.run([str(ref_bench), "--sweep", "--rows", str(n), "--cols", str(c), "--reps", "2", "--gib", "1.0"],
                             capture_output=True, text=True, timeout=120).stdout
                best = 0.0
                for ln in txt.splitlines():
                    f = ln.split()
                    if len(f) >= 4 and f[0] not in ("variant", "copy") and not ln.startswith(("#", "N=")):
                        try:
                            best = max(best, float(f[3]))
                        except ValueError:
                            pass
                row["reference_best_kernel_GBs_same_box"] = best or None
            except (OSError, sp.TimeoutExpired):
                row["reference_best_kernel_GBs_same_box"] = None
        out["rmsnorm"].append(row)
    # CPU quantiser (oracle): 1024 x 4096 rows, single thread
    try:
        from oracle import mxfp8

        g = np.random.default_rng(0)
        nb, cb = 1024, 4096
        x = torch.from_numpy(g.standard_normal((nb, cb), dtype=np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        w = torch.ones(cb, dtype=torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
        t0 = time.perf_counter()
        mxfp8.quantise_port(x, x, w, None, 1e-6)
        dt = time.perf_counter() - t0
        out["rmsnorm_cpu_baseline"] = {"value": (nb * cb * 5 + 4 * nb) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": "port",
                                       "sample": f"{nb} x {cb} rows through the plain-C quantiser oracle, one thread"}
    except Exception as e:      # the oracle library is test infrastructure; its absence must not break the bench
        out["rmsnorm_cpu_baseline"] = {"unavailable": str(e)[:120]}
    # (geometry, batch, context, timed steps, MXFP8 weights): the other two model sizes at batch 1 and the two batched
    # configurations (tensor-core kernel), short device-timed lines
    host_weights = {}
    for gname, batch, ctx, steps, mx in (("smollm2-135m", 1, 32, 64, False), ("smollm2-360m", 16, 4096, 16, True),
                                         ("smollm2-1.7b", 1, 1024, 32, False), ("smollm2-1.7b", 64, 1024, 8, False)):
        geom = D.GEOMETRIES[gname]
        if gname not in host_weights:
            host_weights.clear()                     # one model's host copy at a time
            host_weights[gname] = harness.make_weights(geom, 0)
        weights = harness.weights_to(host_weights[gname], dev)
        if mx:
            geom = geom.with_format(1)
            weights = D.pack_weights_mxfp8(weights)
        cap = ctx + steps + 80
        cap = (cap + 15) // 16 * 16
        kv = harness.PagedKV(geom, batch, cap, dev)
        for cache in kv.kv_caches:
            cache.normal_()
        sess = D.DecodeSession(geom, embed=weights["embed"], layers=weights["layers"], final_norm=weights["final_norm"],
                               kv_caches=kv.kv_caches, cos_sin_cache=harness.make_cos_sin_cache(geom, cap, dev),
                               block_table=kv.block_table, embed_lookup=weights.get("embed_lookup"))
        sess.start(torch.full((batch,), 17), torch.full((batch,), ctx))
        for _ in range(4):
            sess.step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            sess.step()
        e1.record()
        torch.cuda.synchronize(dev)
        D.check_status(geom, dev)
        ms = e0.elapsed_time(e1) / steps
        nbytes = algorithmic_bytes(geom, batch, ctx + 4 + steps // 2, mxfp8=mx)
        out["decode"].append({"workload": f"{gname}{'-mxfp8' if mx else ''}-b{batch}", "context": ctx, "steps": steps,
                              "ms_per_step": round(ms, 4), "tok_s": round(batch * 1e3 / ms, 1),
                              "roofline_frac_of_measured": round(nbytes / (ms * 1e-3) / 1e9 / peak, 3),
                              "note": "KV pre-filled with normal(0,1), device-driven greedy loop, CUDA events"})
        del sess, kv, weights
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--workload", default="smollm2-360m-b1", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary measurements (rmsnorm, other model sizes)")
    ap.add_argument("--prompt-tokens", type=int, default=None, help="override the workload's prompt length")
    args = ap.parse_args()
    wl = args.workload
    gname, batch, prompt_len, default_steps = WORKLOADS[wl]
    if args.prompt_tokens:
        prompt_len = args.prompt_tokens
    if args.steps is None:
        args.steps = default_steps
    if args.impl == "reference":
        run_reference(args, wl)
        return

    import torch

    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import harness

    geom = D.GEOMETRIES[gname]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the decode path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- synthetic model + prompt (replica r decodes its own stream: seed 1234 + r)
    mxfp8 = "mxfp8" in wl
    weights = harness.weights_to(harness.make_weights(geom, 0), dev)
    if mxfp8:
        geom = geom.with_format(1)
        weights = D.pack_weights_mxfp8(weights)
    K, W = args.steps, max(args.warmup, 3)
    capacity = prompt_len + 2 * (K + W) + 64
    capacity = min(D.MAX_SEQ, (capacity + 15) // 16 * 16)
    cos_sin = harness.make_cos_sin_cache(geom, capacity, dev)
    prompt = torch.randint(0, geom.vocab, (batch, prompt_len), generator=torch.Generator().manual_seed(1234 + rank))

    def new_session():
        kv = harness.PagedKV(geom, batch, capacity, dev)
        sess = D.DecodeSession(geom, embed=weights["embed"], layers=weights["layers"], final_norm=weights["final_norm"],
                               kv_caches=kv.kv_caches, cos_sin_cache=cos_sin, block_table=kv.block_table,
                               embed_lookup=weights.get("embed_lookup"))
        return kv, sess

    def prefill(sess):
        if mxfp8:
            # config 4: the context is pre-filled with normal(0,1) bf16 K/V (seed 3), not computed from a prompt
            g3 = torch.Generator(device=dev).manual_seed(3)
            for cache in sess.kv_caches:
                cache.copy_(torch.randn(cache.shape, generator=g3, device=dev, dtype=torch.float32).to(torch.bfloat16))
            sess.start(prompt[:, -1], torch.full((batch,), prompt_len - 1, dtype=torch.int64))
            return
        # the prompt goes through the same kernel, token by token (teacher forced), which fills the cache
        sess.start(prompt[:, 0], torch.zeros(batch, dtype=torch.int64))
        for t in range(prompt_len - 1):
            sess.step()
            sess.input_ids.copy_(prompt[:, t + 1].to(dev))
        D.check_status(geom, dev)

    # ---- device-resident greedy loop
    kv, sess = new_session()
    prefill(sess)
    for _ in range(W):
        sess.step()
    barrier()
    stream = torch.cuda.current_stream(dev)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    seq_first = int(sess.seq_lens[0])
    clocks = ClockSampler(local_rank)      # samples during the device-timed loop and during the end-to-end loop
    with clocks:
        barrier()
        ev0.record(stream)
        for _ in range(K):
            sess.step()
        ev1.record(stream)
        barrier()
    D.check_status(geom, dev)
    ms = ev0.elapsed_time(ev1)
    seq_last = seq_first + K - 1

    # ---- end to end through the public API with host buffers
    def run_e2e():
        kv2, sess2 = new_session()
        prefill(sess2)
        # D.HostStep: one pinned staging buffer + one device buffer for the four per-step inputs (28 bytes per
        # request, one host-to-device copy), the fused step, and the device-to-host copy of the greedy ids,
        # captured once into a CUDA graph and replayed every step; the inputs of every step come from the host
        step = D.HostStep(geom, batch, embed=weights["embed"], layers=weights["layers"], final_norm=weights["final_norm"],
                          kv_caches=kv2.kv_caches, cos_sin_cache=cos_sin, block_table=kv2.block_table,
                          embed_lookup=weights.get("embed_lookup"))
        # host side of a serving loop: block table and current ids as numpy arrays, slots computed on the CPU
        bt_host = kv2.block_table.cpu().numpy().astype("int64")
        cur = prompt[:, -1].clone().numpy()
        pos0 = prompt_len - 1

        def e2e_step(t):
            pos = pos0 + t
            nxt = step.step_numpy(cur, pos, pos + 1, bt_host[:batch, pos // 16] * 16 + pos % 16)
            cur[:] = nxt

        for t in range(W):
            e2e_step(t)
        barrier()
        with clocks:
            t0 = time.perf_counter()
            for t in range(W, W + K):
                e2e_step(t)
            torch.cuda.synchronize(dev)
            dt = time.perf_counter() - t0
        barrier()
        D.check_status(geom, dev)
        return dt

    e2e_s = float("nan") if args.no_e2e else run_e2e()

    ms_max, e2e_ms_max = max_over_ranks([ms, e2e_s * 1e3], world, dev)

    if rank == 0:
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peak, peak_src = float(json.loads(peaks_file.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = 6650.0, "fallback (earlier pool measurement)"
        mean_bytes = statistics.mean(algorithmic_bytes(geom, batch, s, mxfp8) for s in (seq_first, seq_last))
        step_ms = ms_max / K
        achieved = mean_bytes / (step_ms * 1e-3) / 1e9
        ratio = NCU_TRAFFIC_RATIO.get((gname, batch, bool(mxfp8)))
        line = {
            "metric": METRIC, "value": aggregate_throughput(world, batch, K, ms_max), "unit": "tok/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 activations, MXFP8 weights" if mxfp8 else "bf16", "data": "synthetic",
            "config": config_block(wl, gname, batch, prompt_len, world),
            "detail": {"context_during_timing": [seq_first, seq_last],
                       "timing": "CUDA events on the launching stream around K back-to-back launches"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": mean_bytes * ratio[0] if ratio else None,
                         "traffic_source": ratio[1] + ", scaled by algorithmic bytes" if ratio else None,
                         "peak_source": peak_src, "frac_of_8TBs_nominal": achieved / 8000.0,
                         "algorithmic_bytes_per_step": mean_bytes},
            "e2e": {"value": None if args.no_e2e else aggregate_throughput(world, batch, K, e2e_ms_max), "unit": "tok/s",
                    "h2d_bytes_per_step": batch * (8 + 8 + 4 + 8), "d2h_bytes_per_step": batch * 8},
            "gpu_launches": K,
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_cpu_baseline:
            toks, cores, desc = cpu_reference(geom, batch, prompt_len, 8)
            line["cpu_baseline"] = {"value": toks, "unit": "tok/s", "cores": cores, "kind": "reference", "sample": desc}
        if world == 1 and not args.no_extra and wl == "smollm2-360m-b1":
            del sess, kv
            torch.cuda.empty_cache()
            line["extra"] = extra_measurements(dev, peak)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
