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


def test_noise_floor_on_the_headline_configuration_in_both_probability_modes():
    """HuggingFace eager against the CPU restatement on SmolLM2-360M with HuggingFace's own 511-token prefill
    cache, two decode steps, in both softmax-probability modes.

    ``probs="bf16"`` has the same rounding points as HuggingFace (layer 0 comes out bit-identical, 0 of 960
    elements differ) and still ends 0.035-0.041 away at the logits: the first bf16 flips caused by fp32 summation
    order appear in layer 1 (65 of 960 elements) and this random-init 32-layer stack amplifies them.
    ``probs="fp32"`` (what the split-KV kernel computes) adds a real rounding-point difference -- 668 of 960
    layer-0 outputs differ by one bf16 ulp -- and ends 0.039-0.046 away.  Either way the per-step 2e-2 target is
    out of reach for an independent implementation at this depth; rounding the probabilities to bf16 does not
    close the gap.  Greedy ids agree in both modes."""
    from prime_kernels_b200.decode import SMOLLM2_360M as geom

    w = harness.make_weights(geom, 0)
    prompt = torch.randint(0, geom.vocab, (1, 512), generator=torch.Generator().manual_seed(1234))
    ref = decode_hf.run(geom, w, prompt, 2)
    cs = harness.make_cos_sin_cache(geom, 640)
    worst = {}
    for mode in ("fp32", "bf16"):
        keys = [[ref["prefill_k"][l][0].clone()] for l in range(geom.layers)]
        vals = [[ref["prefill_v"][l][0].clone()] for l in range(geom.layers)]
        cur = prompt[:, -1]
        worst[mode] = 0.0
        for s in range(2):
            _, logits, _ = R.decode_step(geom, w, cur, torch.tensor([511 + s]), keys, vals, cs, probs=mode)
            worst[mode] = max(worst[mode], (logits - ref["logits"][s]).abs().max().item())
            assert (logits.argmax(-1) == ref["ids"][s]).all()
            cur = ref["ids"][s]
    assert 2e-2 < worst["fp32"] <= 7e-2
    assert 2e-2 < worst["bf16"] <= 7e-2


def test_bf16_probabilities_reproduce_hf_layer_zero_exactly():
    """With the probabilities rounded to bf16 where HuggingFace rounds them, the first layer of the restatement
    equals HuggingFace eager bit for bit (small geometry, several requests): the rounding points of the whole
    layer are the ones HuggingFace uses."""
    geom = Geometry("tiny1", 192, 512, 1, 3, 1, vocab=512)
    w = harness.make_weights(geom, 3, norm_weights="random")
    prompt = torch.randint(0, 512, (3, 40), generator=torch.Generator().manual_seed(5))
    model = decode_hf.build_model(geom, w)
    with torch.no_grad():
        pre = model(input_ids=prompt[:, :-1], use_cache=True)
        pk, pv = decode_hf._cache_layers(pre.past_key_values)
        pk, pv = [k.clone() for k in pk], [v.clone() for v in pv]
        res = model(input_ids=prompt[:, -1:], past_key_values=pre.past_key_values, use_cache=True,
                    output_hidden_states=True)
    cs = harness.make_cos_sin_cache(geom, 64)
    keys = [[pk[0][b].clone() for b in range(3)]]
    vals = [[pv[0][b].clone() for b in range(3)]]
    hid, _, _ = R.decode_step(geom, w, prompt[:, -1], torch.tensor([39, 39, 39]), keys, vals, cs, probs="bf16")
    assert torch.equal(hid.float(), res.hidden_states[-1][:, -1].float())
