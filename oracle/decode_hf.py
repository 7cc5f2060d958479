"""TEST INFRASTRUCTURE: the decode oracle -- HuggingFace ``LlamaForCausalLM`` with eager attention in
bf16 on the CPU, the same oracle the reference project validated its decode kernels against
(research/smollm2_360m_decode/experiments/r26-a-before-wait/direct_bench.py:134-149: SDPA/eager prefill,
then eager decode steps, compared on final hidden, logits and greedy ids).

The arithmetic lives in the third-party ``transformers`` package (models/llama/modeling_llama.py;
version installed in this image: 5.5.x; the reference does not pin one).  Weights come from
``prime_kernels_b200.harness.make_weights`` so both sides see identical bf16 tensors.
"""
from __future__ import annotations

import time

import torch

HEAD_DIM = 64


def build_model(geometry, weights):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=geometry.vocab, hidden_size=geometry.hidden,
                      intermediate_size=geometry.intermediate, num_hidden_layers=geometry.layers,
                      num_attention_heads=geometry.q_heads, num_key_value_heads=geometry.kv_heads,
                      head_dim=HEAD_DIM, max_position_embeddings=8192, rms_norm_eps=geometry.eps,
                      rope_theta=geometry.rope_theta, tie_word_embeddings=True, attention_bias=False,
                      mlp_bias=False, hidden_act="silu")
    cfg._attn_implementation = "eager"
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    qd, kd = geometry.q_heads * HEAD_DIM, geometry.kv_heads * HEAD_DIM
    sd = {"model.embed_tokens.weight": weights["embed"].cpu(), "lm_head.weight": weights["embed"].cpu(),
          "model.norm.weight": weights["final_norm"].cpu()}
    for i, (n1, qkv, o, n2, gate_up, down) in enumerate(weights["layers"]):
        p = f"model.layers.{i}."
        qkv, gate_up = qkv.cpu(), gate_up.cpu()
        sd[p + "input_layernorm.weight"] = n1.cpu()
        sd[p + "self_attn.q_proj.weight"] = qkv[:qd].contiguous()
        sd[p + "self_attn.k_proj.weight"] = qkv[qd:qd + kd].contiguous()
        sd[p + "self_attn.v_proj.weight"] = qkv[qd + kd:].contiguous()
        sd[p + "self_attn.o_proj.weight"] = o.cpu()
        sd[p + "post_attention_layernorm.weight"] = n2.cpu()
        sd[p + "mlp.gate_proj.weight"] = gate_up[:geometry.intermediate].contiguous()
        sd[p + "mlp.up_proj.weight"] = gate_up[geometry.intermediate:].contiguous()
        sd[p + "mlp.down_proj.weight"] = down.cpu()
    model.load_state_dict(sd, strict=False, assign=True)
    # rotary inv_freq is a non-persistent buffer: rebuild it off the meta device
    from transformers.models.llama.modeling_llama import LlamaRotaryEmbedding
    model.model.rotary_emb = LlamaRotaryEmbedding(config=cfg, device="cpu")
    model.eval()
    return model


def _cache_layers(cache):
    """(keys, values) lists ``[L][B, kv_heads, T, 64]`` from whatever cache class this transformers has."""
    keys, values = [], []
    if hasattr(cache, "layers"):
        for layer in cache.layers:
            keys.append(layer.keys)
            values.append(layer.values)
    else:
        for k, v in zip(cache.key_cache, cache.value_cache):
            keys.append(k)
            values.append(v)
    return keys, values


@torch.no_grad()
def run(geometry, weights, prompt_ids: torch.Tensor, steps: int, forced_ids: torch.Tensor | None = None,
        model=None, warmup_steps: int = 0):
    """Prefill ``prompt_ids [B, T]`` then ``steps`` decode steps (greedy, or teacher-forced with
    ``forced_ids [steps, B]``).

    Returns a dict: ``prefill_k/prefill_v`` (lists ``[L][B, KVH, T, 64]`` bf16, the cache after the prompt
    *without* its last token -- the last prompt token is the first decode input), ``logits`` fp32
    ``[steps, B, V]``, ``hidden`` bf16 ``[steps, B, H]`` (final-normed), ``ids`` int64 ``[steps, B]``,
    ``seconds_per_step``.  ``warmup_steps`` greedy decode steps run first, untimed and unrecorded (timing use only:
    the recorded steps then continue from the context they leave).
    """
    model = model or build_model(geometry, weights)
    B, T = prompt_ids.shape
    out_logits, out_hidden, out_ids = [], [], []
    cache = None
    if T > 1:
        pre = model(input_ids=prompt_ids[:, :-1], use_cache=True)
        cache = pre.past_key_values
        pk, pv = _cache_layers(cache)
        prefill_k = [k.clone() for k in pk]
        prefill_v = [v.clone() for v in pv]
    else:
        prefill_k = [torch.zeros(B, geometry.kv_heads, 0, HEAD_DIM, dtype=torch.bfloat16)] * geometry.layers
        prefill_v = prefill_k
    cur = prompt_ids[:, -1:]
    for _ in range(warmup_steps):
        res = model(input_ids=cur, past_key_values=cache, use_cache=True, output_hidden_states=True)
        cache = res.past_key_values
        cur = res.logits[:, -1, :].float().argmax(dim=-1).view(B, 1)
    t0 = time.perf_counter()
    for s in range(steps):
        res = model(input_ids=cur, past_key_values=cache, use_cache=True, output_hidden_states=True)
        cache = res.past_key_values
        logits = res.logits[:, -1, :]
        out_logits.append(logits.float())
        out_hidden.append(res.hidden_states[-1][:, -1, :])
        nxt = logits.float().argmax(dim=-1)
        out_ids.append(nxt)
        cur = (forced_ids[s] if forced_ids is not None else nxt).view(B, 1)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    fk, fv = _cache_layers(cache)
    return {"prefill_k": prefill_k, "prefill_v": prefill_v, "logits": torch.stack(out_logits),
            "hidden": torch.stack(out_hidden), "ids": torch.stack(out_ids), "seconds_per_step": dt,
            "final_k": fk, "final_v": fv}
