"""Generates the committed golden fixtures (run in a container that has the reference checkout and
``transformers``):

    python tests/golden/make_golden.py [--only mxfp8|decode|decode360]

* ``mxfp8_reference.json`` -- digests and samples of the outputs of the reference project's own CPU
  ``reference()`` (prime_kernels/rmsnorm/test.cu:82-150, compiled into oracle/_ref by
  oracle/build_ref.sh) on the reference test's input recipe (LCG seed 12345, zero row, 240 outlier;
  test.cu:242-258) for the shapes test.cu:409-410 lists (those that finish in seconds on a CPU).
* ``decode_135m_b1.npz`` -- HuggingFace eager bf16 CPU run of the SmolLM2-135M geometry with
  seeded random weights (prime_kernels_b200.harness.make_weights seed 0), 32-token seeded prompt,
  64 greedy steps: the prompt, the KV cache after the prompt, and per step the greedy id, top-8
  logits, the logits at 512 fixed vocabulary positions and the final-normed hidden state.
* ``decode_360m_b1.npz`` -- the same oracle on the headline configuration (SmolLM2-360M geometry, 512-token
  prompt seeded like ``bench.py``, 256 greedy steps): the prompt and per step the greedy id, top-8 logits and
  the logits at 128 fixed vocabulary positions (the prompt's KV cache is too large to commit; the GPU test
  rebuilds it by running the prompt through the kernel).
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
HERE = Path(__file__).resolve().parent

MXFP8_SHAPES = [(128, 128), (128, 512), (256, 2048), (128, 3072), (256, 4096)]


def make_mxfp8():
    from oracle import mxfp8

    out = {"eps": 1e-5, "math": "fp32", "cases": []}
    for n, c in MXFP8_SHAPES:
        b, r, w = mxfp8.lcg_inputs(n, c)
        _, _, rr, _ = mxfp8.quantise_port(b, r, w, None, 1e-5)
        s = rr.astype(np.float32)                 # the driving rrms: float of the double-precision value
        vals, scales, rrms = mxfp8.quantise_ref(b, r, w, s, 1e-5, 1)
        out["cases"].append({
            "n": n, "c": c,
            "vals_sha256": hashlib.sha256(vals.tobytes()).hexdigest(),
            "scales_sha256": hashlib.sha256(scales.tobytes()).hexdigest(),
            "vals_row1_head": vals[1, :64].tolist(),
            "scales_head": scales[:64].tolist(),
            "row0_scale_bytes_all_zero": bool((scales.reshape(-1, 512)[:, 0:1] == 0).all()),
            "row1_group0_scale": int(scales[mxfp8.port().pk_sf_offset(1, 0, c // 128)]),
        })
    (HERE / "mxfp8_reference.json").write_text(json.dumps(out, indent=1))
    print("wrote mxfp8_reference.json")


def make_decode():
    from oracle import decode_hf
    from prime_kernels_b200 import harness
    from prime_kernels_b200.decode import SMOLLM2_135M as geom

    torch.set_num_threads(min(8, torch.get_num_threads()))
    weights = harness.make_weights(geom, seed=0)
    prompt = torch.randint(0, geom.vocab, (1, 32), generator=torch.Generator().manual_seed(1234))
    res = decode_hf.run(geom, weights, prompt, 64)
    logits = res["logits"][:, 0, :]                                  # [64, V] fp32
    sample_idx = torch.randperm(geom.vocab, generator=torch.Generator().manual_seed(99))[:512].sort().values
    top = logits.topk(8, dim=-1)
    np.savez_compressed(
        HERE / "decode_135m_b1.npz",
        prompt=prompt.numpy(),
        prefill_k=torch.stack([k[0] for k in res["prefill_k"]]).view(torch.int16).numpy(),   # [L, KVH, 31, 64]
        prefill_v=torch.stack([v[0] for v in res["prefill_v"]]).view(torch.int16).numpy(),
        ids=res["ids"][:, 0].numpy(),
        top_values=top.values.numpy(), top_indices=top.indices.numpy(),
        sample_idx=sample_idx.numpy(), sample_logits=logits[:, sample_idx].numpy(),
        hidden=res["hidden"][:, 0, :].view(torch.int16).numpy(),
        final_k_last=torch.stack([k[0, :, -1, :] for k in res["final_k"]]).view(torch.int16).numpy(),
    )
    print("wrote decode_135m_b1.npz; ids", res["ids"][:, 0].tolist()[:16], "s/step", res["seconds_per_step"])


def make_decode_360m():
    from oracle import decode_hf
    from prime_kernels_b200 import harness
    from prime_kernels_b200.decode import SMOLLM2_360M as geom

    weights = harness.make_weights(geom, seed=0)
    prompt = torch.randint(0, geom.vocab, (1, 512), generator=torch.Generator().manual_seed(1234))
    res = decode_hf.run(geom, weights, prompt, 256)
    logits = res["logits"][:, 0, :]                                  # [256, V] fp32
    sample_idx = torch.randperm(geom.vocab, generator=torch.Generator().manual_seed(99))[:128].sort().values
    top = logits.topk(8, dim=-1)
    np.savez_compressed(
        HERE / "decode_360m_b1.npz",
        prompt=prompt.numpy(), ids=res["ids"][:, 0].numpy(),
        top_values=top.values.numpy(), top_indices=top.indices.numpy(),
        sample_idx=sample_idx.numpy(), sample_logits=logits[:, sample_idx].numpy(),
    )
    margin = (top.values[:, 0] - top.values[:, 1]).min().item()
    print("wrote decode_360m_b1.npz; ids", res["ids"][:, 0].tolist()[:8], "min top-2 margin", margin,
          "s/step", res["seconds_per_step"])


if __name__ == "__main__":
    only = sys.argv[sys.argv.index("--only") + 1] if "--only" in sys.argv else None
    if only in (None, "mxfp8"):
        make_mxfp8()
    if only in (None, "decode"):
        make_decode()
    if only in (None, "decode360"):
        make_decode_360m()
