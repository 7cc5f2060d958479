"""GPU: the allocation-free decode entry point (pk_decode_step_static) against the regular one.

Some users of this library cannot hand it a scratch buffer: a serving engine that has already given
all free device memory to its KV-cache pool, or an embedder calling the C ABI from code that must not
touch the CUDA allocator.  For them the library keeps a fixed 2 MiB scratch array on the device.  This
test drives both entry points through the raw C ABI on identical inputs, twice in a row (the second
call reuses what the first left in the shared scratch), and requires the same hidden state, logits
and greedy ids; it also checks that an oversized request is refused instead of overrunning the array.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

from prime_kernels_b200 import harness

pytestmark = pytest.mark.gpu
LOGIT_TOL = 2e-2     # same bound the decode parity tests use


def _args(cabi, geom, dev, wd, kv, csd, ids, pos, hidden, logits, nxt, tables, workspace):
    a = cabi.PkDecodeArgs()
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    a.batch = ids.shape[0]
    a.input_ids, a.ids_i64 = ids.data_ptr(), 1
    a.positions = pos.data_ptr()
    seq = (pos + 1).to(torch.int32)
    slots = kv.slots(pos)
    a.seq_lens, a.slot_mapping = seq.data_ptr(), slots.data_ptr()
    a.block_table, a.bt_stride = kv.block_table.data_ptr(), kv.block_table.stride(0)
    a.layers, a.kv_layers = tables[0].data_ptr(), tables[1].data_ptr()
    a.embed, a.embed_lookup, a.final_norm = wd["embed"].data_ptr(), None, wd["final_norm"].data_ptr()
    kv0 = kv.kv_caches[0]
    a.k_off, a.v_off = 0, 64
    a.block_stride, a.token_stride, a.head_stride = kv0.stride(0), kv0.stride(2), kv0.stride(1)
    a.block_size = kv0.shape[2]
    a.cos_sin, a.cs_fp32 = csd.data_ptr(), 0
    a.out_hidden, a.logits, a.next_ids, a.layer_outputs = hidden.data_ptr(), logits.data_ptr(), nxt.data_ptr(), None
    a.workspace = workspace.data_ptr() if workspace is not None else None
    a.workspace_bytes = workspace.numel() if workspace is not None else 0
    a.max_seq_len = kv.block_table.shape[1] * kv0.shape[2]
    a.lm_head, a.advance = 1, 0
    return a, (seq, slots)          # keep the temporaries alive until the launch has been issued


def test_static_scratch_entry_matches_regular_entry(cuda_device):
    from prime_kernels_b200 import _cabi
    from prime_kernels_b200 import decode as D

    lib = _cabi.library()
    dev = cuda_device
    geom = D.Geometry("noalloc", 192, 512, 3, 3, 1, 1024)
    model = _cabi.PkDecodeModel(geom.hidden, geom.intermediate, geom.layers, geom.q_heads, geom.kv_heads,
                                geom.vocab, 0, geom.eps)
    B, ctx = 2, 45
    wd = harness.weights_to(harness.make_weights(geom, 4, norm_weights="random"), dev)
    csd = harness.make_cos_sin_cache(geom, 128, dev)
    gen = torch.Generator().manual_seed(5)
    keys = [torch.randn(B, geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(geom.layers)]
    vals = [torch.randn(B, geom.kv_heads, ctx, 64, generator=gen).to(torch.bfloat16) for _ in range(geom.layers)]

    def fresh():
        kv = harness.PagedKV(geom, B, 128, dev)
        kv.load_prefix(keys, vals)
        layer_t = torch.tensor([[t.data_ptr() for t in layer] for layer in wd["layers"]], dtype=torch.int64, device=dev)
        kv_t = torch.tensor([c.data_ptr() for c in kv.kv_caches], dtype=torch.int64, device=dev)
        out = (torch.zeros(B, geom.hidden, dtype=torch.bfloat16, device=dev),
               torch.zeros(B, geom.vocab, dtype=torch.bfloat16, device=dev),
               torch.zeros(B, dtype=torch.int64, device=dev))
        return kv, (layer_t, kv_t), out

    kv_a, tab_a, out_a = fresh()
    kv_b, tab_b, out_b = fresh()
    workspace = torch.zeros(D.workspace_bytes(geom, B), dtype=torch.uint8, device=dev)
    assert D.workspace_bytes(geom, B) <= lib.pk_decode_static_scratch_bytes()

    ids = torch.tensor([3, 900], device=dev)
    for step in range(2):                       # two calls in a row through each entry point
        pos = torch.full((B,), ctx + step, dtype=torch.int64, device=dev)
        a, keep_a = _args(_cabi, geom, dev, wd, kv_a, csd, ids, pos, *out_a, tab_a, workspace)
        assert lib.pk_decode_step(ctypes.byref(model), ctypes.byref(a)) == 0
        b, keep_b = _args(_cabi, geom, dev, wd, kv_b, csd, ids, pos, *out_b, tab_b, None)
        assert lib.pk_decode_step_static(ctypes.byref(model), ctypes.byref(b)) == 0
        stream = torch.cuda.current_stream(dev).cuda_stream
        assert lib.pk_decode_status(workspace.data_ptr(), stream) == 0
        assert lib.pk_decode_static_status(stream) == 0
        torch.cuda.synchronize(dev)
        assert (out_a[1].float() - out_b[1].float()).abs().max().item() <= LOGIT_TOL
        assert (out_a[0].float() - out_b[0].float()).abs().max().item() <= 2 ** -4
        assert torch.equal(out_a[2], out_b[2])
        assert out_a[1].float().abs().max().item() > 0          # the kernel really wrote logits
        for ca, cb in zip(kv_a.kv_caches, kv_b.kv_caches):      # both appended the same K/V
            assert torch.equal(ca, cb)
        ids = out_a[2].clone()
        del keep_a, keep_b


def test_static_scratch_entry_on_the_batch1_kernel_with_alternating_lm_head(cuda_device):
    """SmolLM2-360M widths at batch 1 (the specialised batch-1 kernel) through both entry points, with steps that
    ask for the greedy id alternating with hidden-only steps: the built-in scratch keeps the previous call's
    contents, so an argmax cell left over from an earlier call must never leak into a later id."""
    from prime_kernels_b200 import _cabi
    from prime_kernels_b200 import decode as D

    lib = _cabi.library()
    dev = cuda_device
    geom = D.Geometry("noalloc-360w", 960, 2560, 2, 15, 5, 2048)
    model = _cabi.PkDecodeModel(geom.hidden, geom.intermediate, geom.layers, geom.q_heads, geom.kv_heads,
                                geom.vocab, 0, geom.eps)
    wd = harness.weights_to(harness.make_weights(geom, 7, norm_weights="random"), dev)
    csd = harness.make_cos_sin_cache(geom, 128, dev)

    def fresh():
        kv = harness.PagedKV(geom, 1, 128, dev)
        layer_t = torch.tensor([[t.data_ptr() for t in layer] for layer in wd["layers"]], dtype=torch.int64, device=dev)
        kv_t = torch.tensor([c.data_ptr() for c in kv.kv_caches], dtype=torch.int64, device=dev)
        out = (torch.zeros(1, geom.hidden, dtype=torch.bfloat16, device=dev),
               torch.zeros(1, geom.vocab, dtype=torch.bfloat16, device=dev),
               torch.zeros(1, dtype=torch.int64, device=dev))
        return kv, (layer_t, kv_t), out

    kv_a, tab_a, out_a = fresh()
    kv_b, tab_b, out_b = fresh()
    workspace = torch.zeros(D.workspace_bytes(geom, 1), dtype=torch.uint8, device=dev)
    assert workspace.numel() <= lib.pk_decode_static_scratch_bytes()
    gen = torch.Generator().manual_seed(2)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for step, lm in enumerate([1, 0, 1, 0, 0, 1, 1]):
        ids = torch.randint(0, geom.vocab, (1,), generator=gen).to(dev)
        pos = torch.full((1,), step, dtype=torch.int64, device=dev)
        a, keep_a = _args(_cabi, geom, dev, wd, kv_a, csd, ids, pos, *out_a, tab_a, workspace)
        b, keep_b = _args(_cabi, geom, dev, wd, kv_b, csd, ids, pos, *out_b, tab_b, None)
        a.lm_head = b.lm_head = lm
        assert lib.pk_decode_step(ctypes.byref(model), ctypes.byref(a)) == 0
        assert lib.pk_decode_step_static(ctypes.byref(model), ctypes.byref(b)) == 0
        assert lib.pk_decode_status(workspace.data_ptr(), stream) == 0
        assert lib.pk_decode_static_status(stream) == 0
        torch.cuda.synchronize(dev)
        assert torch.equal(out_a[0], out_b[0])                 # same kernel, same inputs: same hidden state
        if lm:
            assert torch.equal(out_a[1], out_b[1]) and torch.equal(out_a[2], out_b[2])
            assert int(out_b[2][0]) == int(out_b[1][0].float().argmax())    # this step's own argmax
        del keep_a, keep_b


def test_static_scratch_refuses_oversized_requests(cuda_device):
    from prime_kernels_b200 import _cabi

    lib = _cabi.library()
    big = _cabi.PkDecodeModel(2048, 8192, 24, 32, 32, 49152, 0, 1e-5)       # SmolLM2-1.7B: > 2 MiB of scratch
    a = _cabi.PkDecodeArgs()
    a.batch = 1
    assert lib.pk_decode_workspace_bytes(ctypes.byref(big), 1) > lib.pk_decode_static_scratch_bytes()
    rc = lib.pk_decode_step_static(ctypes.byref(big), ctypes.byref(a))
    assert rc == 9112
    assert b"2_MiB" in lib.pk_status_string(rc)
