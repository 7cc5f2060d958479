"""CPU: the decode restatement (oracle/decode_restatement.py) against HuggingFace eager on a small
Llama geometry, and against the committed SmolLM2-135M golden run."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import decode_hf, decode_restatement as R
from prime_kernels_b200 import harness
from prime_kernels_b200.decode import SMOLLM2_135M, Geometry

GOLDEN = Path(__file__).parent / "golden" / "decode_135m_b1.npz"


def test_restatement_tracks_hf_eager_on_a_small_geometry():
    geom = Geometry("tiny", 192, 512, 3, 3, 1, vocab=1024)
    w = harness.make_weights(geom, 0, norm_weights="random")
    prompt = torch.randint(0, 1024, (2, 9), generator=torch.Generator().manual_seed(1234))
    ref = decode_hf.run(geom, w, prompt, 4)
    cs = harness.make_cos_sin_cache(geom, 64)
    keys = [[ref["prefill_k"][l][b].clone() for b in range(2)] for l in range(geom.layers)]
    vals = [[ref["prefill_v"][l][b].clone() for b in range(2)] for l in range(geom.layers)]
    cur = prompt[:, -1]
    for s in range(4):
        pos = torch.tensor([8 + s, 8 + s])
        hid, logits, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        assert (logits - ref["logits"][s]).abs().max() <= 2e-2          # the north star's bf16 tolerance
        assert (logits.argmax(-1) == ref["ids"][s]).all()
        cur = ref["ids"][s]
    # the cache the restatement built matches HF's to one bf16 ulp
    for l in range(geom.layers):
        k = torch.stack([keys[l][b] for b in range(2)]).float()
        assert (k - ref["final_k"][l].float()).abs().max() <= 2 ** -5


@pytest.mark.skipif(not GOLDEN.exists(), reason="golden fixture not generated")
def test_restatement_against_committed_135m_golden_first_steps():
    z = np.load(GOLDEN)
    geom = SMOLLM2_135M
    w = harness.make_weights(geom, 0)
    cs = harness.make_cos_sin_cache(geom, 128)
    pk = torch.from_numpy(z["prefill_k"]).view(torch.bfloat16)     # [L, KVH, 31, 64]
    pv = torch.from_numpy(z["prefill_v"]).view(torch.bfloat16)
    keys = [[pk[l].clone()] for l in range(geom.layers)]
    vals = [[pv[l].clone()] for l in range(geom.layers)]
    cur = torch.from_numpy(z["prompt"])[:, -1]
    sample_idx = torch.from_numpy(z["sample_idx"])
    for s in range(2):
        pos = torch.tensor([31 + s])
        hid, logits, _ = R.decode_step(geom, w, cur, pos, keys, vals, cs)
        want = torch.from_numpy(z["sample_logits"][s])
        assert (logits[0, sample_idx] - want).abs().max() <= 2e-2
        top_i = torch.from_numpy(z["top_indices"][s])
        top_v = torch.from_numpy(z["top_values"][s])
        assert (logits[0, top_i] - top_v).abs().max() <= 2e-2
        if top_v[0] - top_v[1] > 4e-2:
            assert int(logits.argmax(-1)) == int(z["ids"][s])
        cur = torch.tensor([int(z["ids"][s])])


def test_summation_order_noise_floor_on_the_headline_configuration():
    """Two CPU implementations with identical rounding points and identical KV caches (HuggingFace eager and
    the restatement, which differ only in fp32 summation order) on SmolLM2-360M with a 512-token context:
    their bf16 logits differ by 3-5e-2 over the vocabulary while the greedy ids agree.  This is the floor any
    independent implementation (the CUDA kernel included) sits on at this configuration; the per-step 2e-2
    target is only reachable on the shallower 135M / short-context configuration."""
    from prime_kernels_b200.decode import SMOLLM2_360M as geom

    w = harness.make_weights(geom, 0)
    prompt = torch.randint(0, geom.vocab, (1, 512), generator=torch.Generator().manual_seed(1234))
    ref = decode_hf.run(geom, w, prompt, 2)
    cs = harness.make_cos_sin_cache(geom, 640)
    keys = [[ref["prefill_k"][l][0].clone()] for l in range(geom.layers)]
    vals = [[ref["prefill_v"][l][0].clone()] for l in range(geom.layers)]
    cur = prompt[:, -1]
    worst = 0.0
    for s in range(2):
        _, logits, _ = R.decode_step(geom, w, cur, torch.tensor([511 + s]), keys, vals, cs)
        worst = max(worst, (logits - ref["logits"][s]).abs().max().item())
        assert (logits.argmax(-1) == ref["ids"][s]).all()
        cur = ref["ids"][s]
    assert 2e-2 < worst <= 1.25e-1
