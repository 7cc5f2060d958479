"""Host-side routing logic of the vLLM-style decode backend, exercised on CPU with duck-typed stand-ins for
vLLM's LlamaModel, FlashAttentionMetadata and forward context and a stub decode step (no GPU work)."""
from types import SimpleNamespace

import pytest
import torch

from prime_kernels_b200 import decode_backend as db


class FlashAttentionMetadata:          # the router matches the class by name, like the reference backend
    def __init__(self, **kw):
        self.__dict__.update(kw)


class OtherMetadata(FlashAttentionMetadata):
    pass


def make_model(hidden=960, inter=2560, layers=2, heads=15, kv_heads=5, dtype=torch.bfloat16, blocks=8):
    def lin(o, i):
        return SimpleNamespace(weight=torch.zeros(o, i, dtype=dtype))

    def layer(idx):
        attn = SimpleNamespace(kv_cache=torch.zeros(blocks, kv_heads, 16, 128, dtype=torch.bfloat16),
                               layer_name=f"model.layers.{idx}.self_attn.attn")
        return SimpleNamespace(
            input_layernorm=SimpleNamespace(weight=torch.ones(hidden, dtype=dtype)),
            post_attention_layernorm=SimpleNamespace(weight=torch.ones(hidden, dtype=dtype)),
            self_attn=SimpleNamespace(qkv_proj=lin((heads + 2 * kv_heads) * 64, hidden), o_proj=lin(hidden, heads * 64),
                                      attn=attn, rotary_emb=SimpleNamespace(cos_sin_cache=torch.zeros(128, 64))),
            mlp=SimpleNamespace(gate_up_proj=lin(2 * inter, hidden), down_proj=lin(hidden, inter)))

    config = SimpleNamespace(hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers,
                             num_attention_heads=heads, num_key_value_heads=kv_heads, rms_norm_eps=1e-5,
                             vocab_size=49152, rope_theta=100000.0)
    return SimpleNamespace(config=config, layers=[layer(i) for i in range(layers)], aux_hidden_state_layers=(),
                           embed_tokens=SimpleNamespace(weight=torch.zeros(64, hidden, dtype=dtype)),
                           norm=SimpleNamespace(weight=torch.ones(hidden, dtype=dtype), variance_epsilon=1e-5))


def decode_meta(batch, cls=FlashAttentionMetadata, width=4):
    return cls(max_query_len=1, num_actual_tokens=batch, seq_lens=torch.arange(1, batch + 1, dtype=torch.int32),
               block_table=torch.zeros(batch, width, dtype=torch.int32),
               slot_mapping=torch.arange(batch, dtype=torch.int64),
               query_start_loc=torch.arange(batch + 1, dtype=torch.int32))


def stub_decode_step(geometry, **kw):
    """Returns a recognisable hidden state: row b is filled with 100 + input id of request b."""
    calls.append((geometry, kw))
    return (100 + kw["input_ids"].float())[:, None].expand(-1, geometry.hidden).to(torch.bfloat16)


calls = []


@pytest.fixture(autouse=True)
def _reset():
    calls.clear()
    db.stats.clear()


def test_geometry_detection():
    g = db.model_geometry(make_model())
    assert (g.name, g.hidden, g.layers, g.q_heads, g.kv_heads) == ("smollm2-360m", 960, 2, 15, 5) or g.hidden == 960
    assert db.model_geometry(make_model(), tp_world=2) is None                       # sharded: stock path
    assert db.model_geometry(make_model(dtype=torch.float16)) is None                # not bf16
    assert db.model_geometry(make_model(heads=16, kv_heads=8, hidden=1024)) is None  # GQA group 2: no kernel
    g17 = db.model_geometry(make_model(hidden=2048, inter=8192, layers=24, heads=32, kv_heads=32))
    assert g17.name == "smollm2-1.7b" and g17.rope_theta == 100000.0                 # config values win


def test_pure_decode_is_routed_and_counted():
    model = make_model()
    ids = torch.tensor([5, 6, 7])
    out = db.route(model, ids, torch.tensor([9, 9, 9]), decode_meta(3), decode_step=stub_decode_step)
    assert out.shape == (3, 960) and out[:, 0].tolist() == [105.0, 106.0, 107.0]
    geometry, kw = calls[0]
    assert len(kw["layers"]) == 2 and len(kw["layers"][0]) == 6 and len(kw["kv_caches"]) == 2
    assert kw["block_table"].shape[0] == 3 and kw["eps"] == 1e-5
    assert db.stats["backend_decode"] == 1


@pytest.mark.parametrize("why,mutate,key", [
    ("prefill in the batch", lambda m: setattr(m, "max_query_len", 7), "stock_not_pure_decode"),
    ("token count differs", lambda m: setattr(m, "num_actual_tokens", 2), "stock_decode_over_max_batch"),
    ("block table dtype", lambda m: setattr(m, "block_table", m.block_table.long()), "stock_unsupported_metadata"),
    ("context capacity too large", lambda m: setattr(m, "block_table", torch.zeros(3, 600, dtype=torch.int32)),
     "stock_unsupported_metadata"),
])
def test_ineligible_steps_fall_through(why, mutate, key):
    meta = decode_meta(3)
    mutate(meta)
    assert db.route(make_model(), torch.tensor([1, 2, 3]), torch.zeros(3, dtype=torch.long), meta,
                    decode_step=stub_decode_step) is None, why
    assert db.stats[key] == 1 and not calls


def test_other_metadata_class_batch_limit_and_cache_layout():
    model = make_model()
    z = torch.zeros(3, dtype=torch.long)
    assert db.route(model, z, z, decode_meta(3, OtherMetadata), decode_step=stub_decode_step) is None
    big = torch.zeros(65, dtype=torch.long)          # one launch takes up to 64 requests
    assert db.route(model, big, big, decode_meta(65), decode_step=stub_decode_step) is None
    assert db.stats["stock_decode_over_max_batch"] == 1
    model.layers[1].self_attn.attn.kv_cache = torch.zeros(8, 5, 32, 128, dtype=torch.bfloat16)   # block size 32
    assert db.route(model, z, z, decode_meta(3), decode_step=stub_decode_step) is None
    assert db.stats["stock_unsupported_metadata"] == 1


def test_vllm_native_cache_layout_is_routed():
    """vLLM's FlashAttention backend keeps K and V as planes of one tensor, [2, blocks, 16, kv_heads, 64]: the router
    takes it (the kernels read the cache through strides); other block sizes and head dims fall through."""
    model = make_model()
    kvh = model.config.num_key_value_heads
    for layer in model.layers:
        layer.self_attn.attn.kv_cache = torch.zeros(2, 8, 16, kvh, 64, dtype=torch.bfloat16)
    z = torch.zeros(3, dtype=torch.long)
    assert db.route(model, z, z, decode_meta(3), decode_step=stub_decode_step) is not None
    assert db.stats["backend_decode"] == 1 and calls[-1][1]["kv_caches"][0].ndim == 5
    for layer in model.layers:
        layer.self_attn.attn.kv_cache = torch.zeros(2, 8, 32, kvh, 64, dtype=torch.bfloat16)      # block size 32
    assert db.route(model, z, z, decode_meta(3), decode_step=stub_decode_step) is None
    for layer in model.layers:
        layer.self_attn.attn.kv_cache = torch.zeros(2, 8, 16, kvh, 128, dtype=torch.bfloat16)     # head dim 128
    assert db.route(model, z, z, decode_meta(3), decode_step=stub_decode_step) is None


def test_repair_recomputes_only_single_token_requests():
    model = make_model()
    # requests: 0 prefill (3 tokens), 1 decode, 2 prefill (2 tokens), 3 decode  -> token rows 3 and 6
    meta = FlashAttentionMetadata(max_query_len=3, num_actual_tokens=7, seq_lens=torch.tensor([3, 11, 2, 21], dtype=torch.int32),
                                  block_table=torch.arange(16, dtype=torch.int32).view(4, 4),
                                  slot_mapping=torch.arange(7, dtype=torch.int64) + 50,
                                  query_start_loc=torch.tensor([0, 3, 4, 6, 7], dtype=torch.int32))
    assert db.decode_rows_of_mixed_batch(meta) == ([1, 3], [3, 6])
    ids = torch.arange(7) + 10
    hidden = torch.zeros(7, 960, dtype=torch.bfloat16)
    geometry = db.model_geometry(model)
    out = db.repair_mixed_decode(model, stub_decode_step, geometry, ids, torch.arange(7), hidden, meta)
    assert out[:, 0].tolist() == [0, 0, 0, 113.0, 0, 0, 116.0] and hidden.abs().sum() == 0      # input untouched
    _, kw = calls[0]
    assert kw["seq_lens"].tolist() == [11, 21] and kw["slot_mapping"].tolist() == [53, 56]
    assert kw["block_table"].tolist() == [[4, 5, 6, 7], [12, 13, 14, 15]]
    assert db.stats["backend_mixed_decode"] == 2


def test_install_patches_forward_once_and_falls_back():
    class LlamaModel:
        def __init__(self):
            self.__dict__.update(make_model().__dict__)

        def forward(self, input_ids, positions, intermediate_tensors=None, inputs_embeds=None):
            return torch.full((input_ids.shape[0], 960), -1.0, dtype=torch.bfloat16)

    ctx = SimpleNamespace(attn_metadata={})
    original = db.install(LlamaModel, lambda: ctx, decode_step=stub_decode_step, batch_invariant=lambda: True)
    assert original is not None and db.install(LlamaModel, lambda: ctx) is None
    model = LlamaModel()
    name = model.layers[0].self_attn.attn.layer_name
    ids = torch.tensor([3, 4])
    ctx.attn_metadata = {name: decode_meta(2)}
    assert model.forward(ids, torch.zeros(2, dtype=torch.long))[:, 0].tolist() == [103.0, 104.0]      # fused path
    ctx.attn_metadata = None                                                                          # profiling run
    assert model.forward(ids, torch.zeros(2, dtype=torch.long))[:, 0].tolist() == [-1.0, -1.0]        # stock path
    mixed = FlashAttentionMetadata(max_query_len=2, num_actual_tokens=3, seq_lens=torch.tensor([2, 9], dtype=torch.int32),
                                   block_table=torch.zeros(2, 4, dtype=torch.int32), slot_mapping=torch.arange(3),
                                   query_start_loc=torch.tensor([0, 2, 3], dtype=torch.int32))
    ctx.attn_metadata = {name: mixed}
    out = model.forward(torch.tensor([7, 8, 9]), torch.zeros(3, dtype=torch.long))
    assert out[:, 0].tolist() == [-1.0, -1.0, 109.0]                     # stock forward, decode row repaired
