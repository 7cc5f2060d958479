"""Caller-side router: sends pure-decode steps of a vLLM-style Llama model through the fused decode step.

Mirrors what the reference's opt-in vLLM backend does
(research/smollm2_360m_decode/experiments/b2-reproducibility-r1/decode_backend.after.py:61-338 in the
reference project): a model is eligible when it is an un-sharded bf16 Llama stack whose geometry the kernel
supports; a step is eligible when the FLASH_ATTN metadata says every request contributes exactly one token,
the batch fits, and the paged KV cache has the layout the kernel reads; everything else falls through to
the stock forward.  With batch-invariant mode, decode rows of a mixed prefill/decode step are recomputed by
the decode step so that a joining prefill does not change their arithmetic path ("repair").

Differences from the reference: the kernel is geometry-generic, so any head-dim-64 Llama configuration is
routed (not only two hard-coded ones) and the batch limit is ``decode.MAX_REQUESTS`` (one launch of the tensor-core
kernel from 4 requests on); nothing here imports vLLM
at module import -- the model, metadata and forward context are duck-typed, and :func:`install` takes the
class to patch and the forward-context getter as arguments (``install_into_vllm`` fetches them from vLLM).
Decode steps replayed from CUDA graphs do not re-enter Python, so the path a captured graph takes is fixed
at capture time, exactly as with the reference backend.
"""
from __future__ import annotations

from collections import Counter
from copy import copy
from typing import Callable, Optional

import torch

HEAD_DIM = 64
BLOCK_SIZE = 16
METADATA_CLASS = "FlashAttentionMetadata"

stats: Counter = Counter()


def geometry_for_config(config):
    """The kernel geometry for a HuggingFace / vLLM Llama config, or None when the kernel cannot run it."""
    from .decode import GEOMETRIES, Geometry

    heads = config.num_attention_heads
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // heads
    kv_heads = config.num_key_value_heads
    if head_dim != HEAD_DIM or heads % kv_heads or heads // kv_heads not in (1, 3):
        return None
    if config.hidden_size % 32 or config.intermediate_size % 32:
        return None
    for g in GEOMETRIES.values():
        if (g.hidden, g.intermediate, g.layers, g.q_heads, g.kv_heads) == (
                config.hidden_size, config.intermediate_size, config.num_hidden_layers, heads, kv_heads):
            return Geometry(g.name, g.hidden, g.intermediate, g.layers, g.q_heads, g.kv_heads,
                            getattr(config, "vocab_size", g.vocab), getattr(config, "rope_theta", g.rope_theta),
                            config.rms_norm_eps)
    return Geometry("llama-h%d-l%d" % (config.hidden_size, config.num_hidden_layers), config.hidden_size,
                    config.intermediate_size, config.num_hidden_layers, heads, kv_heads,
                    getattr(config, "vocab_size", 49152), getattr(config, "rope_theta", 10000.0), config.rms_norm_eps)


def model_geometry(model, tp_world: int = 1, pp_world: int = 1):
    """Model-only eligibility (the reference's ``_model_kernel_name``): un-sharded, bf16, fused QKV."""
    if getattr(model, "aux_hidden_state_layers", None):
        return None
    if tp_world != 1 or pp_world != 1:
        return None
    if model.embed_tokens.weight.dtype != torch.bfloat16:
        return None
    if not hasattr(model.layers[0].self_attn, "qkv_proj") or not hasattr(model.layers[0].mlp, "gate_up_proj"):
        return None
    return geometry_for_config(model.config)


def _kv_caches(model):
    return [layer.self_attn.attn.kv_cache for layer in model.layers]


def metadata_eligible(meta, model, geometry, batch: int) -> bool:
    """Step eligibility (the reference's ``_metadata_eligible``), for every geometry the kernel takes."""
    from .decode import MAX_REQUESTS, MAX_SEQ

    if meta is None or type(meta).__name__ != METADATA_CLASS:
        return False
    if meta.max_query_len != 1 or meta.num_actual_tokens != batch or not 0 < batch <= MAX_REQUESTS:
        return False
    caches = _kv_caches(model)
    first = caches[0]
    bt = meta.block_table
    # the reference's cache layout [blocks, kv_heads, 16, 128], or vLLM's FlashAttention layout
    # [2, blocks, 16, kv_heads, 64] (the kernels read either through strides)
    if first.ndim == 4:
        layout_ok = (first.shape[1] == geometry.kv_heads and first.shape[2] == BLOCK_SIZE
                     and first.shape[3] == 2 * HEAD_DIM and first.stride(3) == 1)
    elif first.ndim == 5:
        layout_ok = (first.shape[0] == 2 and first.shape[2] == BLOCK_SIZE and first.shape[3] == geometry.kv_heads
                     and first.shape[4] == HEAD_DIM and first.stride(4) == 1
                     and all(st % 8 == 0 for st in first.stride()[:4]))
    else:
        layout_ok = False
    if (first.dtype != torch.bfloat16 or not layout_ok
            or bt.dtype != torch.int32 or bt.shape[0] < batch or bt.stride(1) != 1 or bt.shape[1] < 1
            or bt.shape[1] * BLOCK_SIZE > MAX_SEQ):
        return False
    return all(kv.dtype == first.dtype and kv.shape == first.shape and kv.stride() == first.stride() for kv in caches)


def layer_weights(model):
    """The six per-layer tensors in the kernel's order: norm1, qkv, o, norm2, gate_up, down."""
    return [(layer.input_layernorm.weight, layer.self_attn.qkv_proj.weight, layer.self_attn.o_proj.weight,
             layer.post_attention_layernorm.weight, layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight)
            for layer in model.layers]


def decode_hidden_states(model, decode_step: Callable, geometry, input_ids, positions, meta):
    """One fused decode step for a pure-decode batch; returns the final-normed hidden states ``[B, H]``."""
    batch = input_ids.shape[0]
    out = decode_step(geometry, input_ids=input_ids, positions=positions, seq_lens=meta.seq_lens[:batch],
                      block_table=meta.block_table[:batch], slot_mapping=meta.slot_mapping[:batch],
                      embed=model.embed_tokens.weight, layers=layer_weights(model), final_norm=model.norm.weight,
                      kv_caches=_kv_caches(model), cos_sin_cache=model.layers[0].self_attn.rotary_emb.cos_sin_cache,
                      eps=model.norm.variance_epsilon)
    return out[0] if isinstance(out, tuple) else out


def decode_rows_of_mixed_batch(meta):
    """(request indices, token rows) of the requests that contribute exactly one token to a mixed step."""
    starts = meta.query_start_loc.cpu().tolist()
    requests = [i for i, (s, e) in enumerate(zip(starts, starts[1:])) if e - s == 1]
    return requests, [starts[i] for i in requests]


def repair_mixed_decode(model, decode_step: Callable, geometry, input_ids, positions, hidden_states, meta):
    """Recompute the decode rows of a mixed prefill/decode step with the fused decode step (batch-invariant
    mode of the reference backend): the same arithmetic path whether or not a prefill joined the step."""
    if meta is None or type(meta).__name__ != METADATA_CLASS or meta.max_query_len <= 1:
        return hidden_states
    if hidden_states.is_cuda and torch.cuda.is_current_stream_capturing():
        return hidden_states
    requests, rows = decode_rows_of_mixed_batch(meta)
    if not requests:
        return hidden_states
    dev = input_ids.device
    request_rows = torch.tensor(requests, dtype=torch.long, device=dev)
    token_rows = torch.tensor(rows, dtype=torch.long, device=dev)
    sub = copy(meta)
    sub.max_query_len = 1
    sub.num_actual_tokens = len(requests)
    sub.seq_lens = meta.seq_lens.index_select(0, request_rows)
    sub.block_table = meta.block_table.index_select(0, request_rows)
    sub.slot_mapping = meta.slot_mapping.index_select(0, token_rows)
    if not metadata_eligible(sub, model, geometry, len(requests)):
        return hidden_states
    decoded = decode_hidden_states(model, decode_step, geometry, input_ids.index_select(0, token_rows),
                                   positions.index_select(0, token_rows), sub)
    result = hidden_states.clone()
    result.index_copy_(0, token_rows, decoded.to(result.dtype))
    stats["backend_mixed_decode"] += len(requests)
    return result


def route(model, input_ids, positions, meta, *, decode_step: Optional[Callable] = None, tp_world: int = 1,
          pp_world: int = 1, inputs_embeds=None):
    """Hidden states from the fused decode step when the model and the step are eligible, else None (the caller
    runs its stock forward).  Counts every decision in :data:`stats` under the reference backend's keys."""
    geometry = model_geometry(model, tp_world, pp_world) if inputs_embeds is None else None
    if geometry is None:
        stats["stock_ineligible"] += 1
        return None
    if decode_step is None:
        from .decode import decode_step as fused

        decode_step = fused
    if meta is None or type(meta).__name__ != METADATA_CLASS or meta.max_query_len != 1:
        stats["stock_not_pure_decode"] += 1
        return None
    from .decode import MAX_REQUESTS

    batch = input_ids.shape[0]
    if batch > MAX_REQUESTS or meta.num_actual_tokens != batch:
        stats["stock_decode_over_max_batch"] += 1
        return None
    if not metadata_eligible(meta, model, geometry, batch):
        stats["stock_unsupported_metadata"] += 1
        return None
    stats["backend_decode"] += 1
    return decode_hidden_states(model, decode_step, geometry, input_ids, positions, meta)


def install(model_class, get_forward_context: Callable, *, decode_step: Optional[Callable] = None,
            world_sizes: Callable = lambda: (1, 1), batch_invariant: Callable = lambda: False):
    """Patch ``model_class.forward(self, input_ids, positions, intermediate_tensors, inputs_embeds=None, **kw)``.

    ``get_forward_context().attn_metadata`` must be a dict keyed by attention layer name (vLLM's forward
    context).  Returns the original forward; installing twice is a no-op."""
    if getattr(model_class.forward, "_prime_kernels_b200_decode_backend", False):
        return None
    original_forward = model_class.forward

    def layer_meta(self):
        attn_metadata = get_forward_context().attn_metadata
        if not isinstance(attn_metadata, dict):
            return None
        return attn_metadata.get(self.layers[0].self_attn.attn.layer_name)

    def forward(self, input_ids, positions, intermediate_tensors=None, inputs_embeds=None, **kwargs):
        tp, pp = world_sizes()
        meta = layer_meta(self)
        hidden = route(self, input_ids, positions, meta, decode_step=decode_step, tp_world=tp, pp_world=pp,
                       inputs_embeds=inputs_embeds)
        if hidden is not None:
            return hidden
        hidden = original_forward(self, input_ids, positions, intermediate_tensors, inputs_embeds, **kwargs)
        if batch_invariant() and inputs_embeds is None:
            geometry = model_geometry(self, tp, pp)
            if geometry is not None:
                step = decode_step
                if step is None:
                    from .decode import decode_step as step
                hidden = repair_mixed_decode(self, step, geometry, input_ids, positions, hidden, meta)
        return hidden

    forward._prime_kernels_b200_decode_backend = True
    model_class.forward = forward
    return original_forward


def install_into_vllm():
    """Install the router into vLLM's ``LlamaModel`` (needs vLLM importable; raises otherwise)."""
    import os

    from vllm.distributed import get_pp_group, get_tensor_model_parallel_world_size
    from vllm.forward_context import get_forward_context
    from vllm.model_executor.models.llama import LlamaModel

    return install(LlamaModel, get_forward_context,
                   world_sizes=lambda: (get_tensor_model_parallel_world_size(), get_pp_group().world_size),
                   batch_invariant=lambda: os.environ.get("VLLM_BATCH_INVARIANT") == "1")
