"""Geometry-generic single-launch decode step (sm_100a) with optional fused tied lm_head + argmax.

The keyword contract of ``decode_step`` is the reference's (prime_kernels/decode_megakernel/__init__.py:134-205
and prime_kernels/decode_megakernel_360m/__init__.py:122-214 in the reference project): vLLM
FLASH_ATTN-style decode metadata, fused ``qkv`` / ``gate_up`` weights, a paged bf16 KV cache
``[blocks, kv_heads, block_size, 128]`` (K in 0..63, V in 64..127) and a ``cos_sin_cache [max_pos, 64]``.
The returned hidden state is a view of a per-device buffer that the next call overwrites.

Extensions over the reference: any Llama geometry with head_dim 64 (SmolLM2 135M / 360M / 1.7B are
predefined), batch up to 8 per launch (64 per call), MXFP8-packed weights, and ``lm_head=True`` which also returns bf16
logits and greedy next ids computed inside the same launch.
"""
from __future__ import annotations

import torch

from .._cabi import library, load_ops
from ..geometry import GEOMETRIES, HEAD_DIM, SMOLLM2_135M, SMOLLM2_1P7B, SMOLLM2_360M, Geometry

load_ops()

__all__ = ["Geometry", "SMOLLM2_135M", "SMOLLM2_360M", "SMOLLM2_1P7B", "GEOMETRIES", "MAX_BATCH", "MAX_REQUESTS", "MAX_SEQ",
           "HEAD_DIM", "decode_step", "check_status", "DecodeSession", "HostStep", "workspace_bytes", "pack_matrix_mxfp8", "pack_weights_mxfp8",
           "unpack_matrix_mxfp8", "packed_row_bytes"]

MAX_BATCH = 8          # requests one launch of the CUDA-core kernels takes
MAX_REQUESTS = 64      # requests one decode_step call takes: larger batches run as one launch of the tensor-core kernel
MAX_SEQ = 8192


@torch.library.register_fake("prime_decode::decode_step")
def _decode_step_fake(input_ids, positions, seq_lens, block_table, slot_mapping, embed, embed_lookup, layers_table,
                      final_norm, kv_table, k_off, v_off, block_stride, token_stride, head_stride, block_size,
                      cos_sin_cache, out_hidden, logits, next_ids, layer_outputs, workspace, hidden, intermediate,
                      layers, q_heads, kv_heads, vocab, weight_format, eps, max_seq_len, lm_head, advance,
                      path=0):
    return 0


_tc_min_batch = 0      # batches from here on run on the tensor-core kernel; 0: the measured cross-over (tc_min_batch)


def tc_min_batch(geometry: Geometry) -> int:
    """Smallest batch that runs on the tensor-core kernel: 4 requests, 2 where a layer's weights are large enough to
    hide the kernel's grid barriers (hidden >= 2048: SmolLM2-1.7B), unless ``set_tensor_core_min_batch`` overrides."""
    if _tc_min_batch > 0:
        return _tc_min_batch
    return 2 if geometry.hidden >= 2048 else 4


def set_tensor_core_min_batch(n: int) -> None:
    """Smallest batch ``decode_step`` (and the C entries pk_decode_step / mk_decode) hand to the tensor-core kernel;
    ``MAX_BATCH + 1`` keeps batches up to 8 on the CUDA-core kernels, 0 restores the default (``tc_min_batch``)."""
    global _tc_min_batch
    _tc_min_batch = max(0, min(int(n), MAX_BATCH + 1))
    library().pk_decode_set_tc_min_batch(_tc_min_batch)


def workspace_bytes(geometry: Geometry, max_batch: int = MAX_BATCH) -> int:
    from .._cabi import PkDecodeModel
    import ctypes

    m = PkDecodeModel(geometry.hidden, geometry.intermediate, geometry.layers, geometry.q_heads, geometry.kv_heads,
                      geometry.vocab, geometry.weight_format, geometry.eps)
    return int(library().pk_decode_workspace_bytes(ctypes.byref(m), max_batch))


class _Runtime:
    """Per-(device, geometry) workspace, output buffers and cached pointer tables."""

    def __init__(self, geometry: Geometry, device: torch.device):
        self.geometry = geometry
        self.device = device
        # one workspace for all kernels: the tensor-core kernel's region lies behind the CUDA-core kernels' region
        self.scratch = torch.zeros(workspace_bytes(geometry, MAX_REQUESTS), dtype=torch.uint8, device=device)
        self.out = torch.empty((MAX_REQUESTS, geometry.hidden), dtype=torch.bfloat16, device=device)
        self.group = MAX_BATCH          # requests per launch; lowered when the geometry does not fit at that batch
        self.logits = None
        self.next_ids = None
        self.table_key = None
        self.layers_t = None
        self.kv_t = None

    def lm_buffers(self):
        if self.logits is None:
            self.logits = torch.empty((MAX_REQUESTS, self.geometry.vocab), dtype=torch.bfloat16, device=self.device)
            self.next_ids = torch.zeros((MAX_REQUESTS,), dtype=torch.int64, device=self.device)
        return self.logits, self.next_ids

    def tables(self, layers, kv_caches, embed, final_norm, embed_lookup):
        # Steady state of a serving loop: the key covers the data pointer of every weight and cache tensor, so a
        # caller that swaps any tensor is noticed; building it costs ~15 us for a 32-layer model, validation and
        # the device tables are only redone when it changes.
        key = (tuple(t.data_ptr() for layer in layers for t in layer), tuple(kv.data_ptr() for kv in kv_caches),
               embed.data_ptr(), final_norm.data_ptr(), 0 if embed_lookup is None else embed_lookup.data_ptr())
        if key == self.table_key:
            return self.layers_t, self.kv_t
        _check_kv(self.geometry, kv_caches)
        _check_weights(self.geometry, self.device, embed, final_norm, layers, embed_lookup)
        layer_table = torch.tensor([[t.data_ptr() for t in layer] for layer in layers], dtype=torch.int64)
        kv_table = torch.tensor([kv.data_ptr() for kv in kv_caches], dtype=torch.int64)
        if self.layers_t is None:
            self.layers_t = layer_table.to(self.device)
            self.kv_t = kv_table.to(self.device)
        else:
            # in place, so CUDA graphs captured with these tables see the new pointers
            self.layers_t.copy_(layer_table)
            self.kv_t.copy_(kv_table)
        self.table_key = key
        return self.layers_t, self.kv_t


_runtimes: dict = {}


def _runtime(geometry: Geometry, device: torch.device) -> _Runtime:
    key = (geometry, device)
    if key not in _runtimes:
        _runtimes[key] = _Runtime(geometry, device)
    return _runtimes[key]


def packed_row_bytes(k: int) -> int:
    return int(library().pk_mxfp8_packed_row_bytes(int(k)))


SCALE_MODES = {"roundup": 0, "floor": 1}


def pack_matrix_mxfp8(w: torch.Tensor, scale_mode: str = "roundup") -> torch.Tensor:
    """Quantise a bf16 CUDA matrix ``[rows, K]`` to the packed MXFP8 row format the decode GEMV streams:
    ``[K e4m3][K/32 e8m0][zero pad to 16 B]`` per row (uint8 ``[rows, packed_row_bytes(K)]``).  ``scale_mode``:
    ``"roundup"`` (scale 2^ceil(log2(amax / 448)): the fused norm-quant op's rule, never saturates) or ``"floor"``
    (scale 2^(floor(log2 amax) - 8): the block-scale rule of the reference's flash_moe kernels, may saturate)."""
    if scale_mode not in SCALE_MODES:
        raise ValueError(f"scale_mode must be one of {sorted(SCALE_MODES)}")
    if w.dtype != torch.bfloat16 or w.dim() != 2 or not w.is_cuda or not w.is_contiguous():
        raise ValueError("expected a contiguous 2-D BF16 CUDA tensor")
    rows, k = w.shape
    rb = packed_row_bytes(k)
    if rb < 0:
        raise ValueError("K must be a multiple of 32")
    out = torch.empty((rows, rb), dtype=torch.uint8, device=w.device)
    with torch.cuda.device(w.device):
        rc = library().pk_pack_weights_mxfp8_ex(w.data_ptr(), out.data_ptr(), rows, k, SCALE_MODES[scale_mode],
                                                torch.cuda.current_stream(w.device).cuda_stream)
    if rc != 0:
        raise RuntimeError(f"pack_weights_mxfp8 failed: {status_string(rc)}")
    return out


def pack_weights_mxfp8(weights: dict, scale_mode: str = "roundup") -> dict:
    """MXFP8 variant of a weight dict (``embed``, ``layers``, ``final_norm``): every projection matrix and
    the tied lm_head are packed; norm weights stay bf16; ``embed_lookup`` keeps the bf16 embedding rows."""
    pk = lambda m: pack_matrix_mxfp8(m, scale_mode)      # noqa: E731
    layers = [(n1, pk(qkv), pk(o), n2, pk(gu), pk(down)) for (n1, qkv, o, n2, gu, down) in weights["layers"]]
    return {"embed": pk(weights["embed"]), "embed_lookup": weights["embed"], "layers": layers,
            "final_norm": weights["final_norm"]}


def unpack_matrix_mxfp8(packed: torch.Tensor, k: int) -> torch.Tensor:
    """Exact bf16 de-quantisation of a packed matrix (plain PyTorch; for checks and oracles)."""
    vals = packed[:, :k].contiguous().view(torch.float8_e4m3fn).float().view(-1, k // 32, 32)
    scale = torch.exp2(packed[:, k:k + k // 32].float() - 127.0)
    return (vals * scale[..., None]).view(-1, k).to(torch.bfloat16)


def status_string(rc: int) -> str:
    return library().pk_status_string(int(rc)).decode()


def _check_kv(geometry: Geometry, kv_caches):
    first = kv_caches[0]
    if first.dtype != torch.bfloat16 or first.dim() not in (4, 5):
        raise ValueError("kv_caches must be 4-D or 5-D BF16 tensors")
    if first.dim() == 4:
        if first.shape[1] != geometry.kv_heads or first.shape[3] != 2 * HEAD_DIM or first.stride(3) != 1:
            raise ValueError(
                f"kv_caches must be [blocks, {geometry.kv_heads}, block_size, {2 * HEAD_DIM}] with unit last stride")
    elif (first.shape[0] != 2 or first.shape[3] != geometry.kv_heads or first.shape[4] != HEAD_DIM or first.stride(4) != 1
          or any(st % 8 for st in first.stride()[:4])):
        raise ValueError(f"5-D kv_caches must be [2, blocks, block_size, {geometry.kv_heads}, {HEAD_DIM}] with unit last "
                         "stride and the other strides multiples of 8 elements")
    for kv in kv_caches:
        if kv.shape != first.shape or kv.stride() != first.stride() or kv.dtype != first.dtype:
            raise ValueError("all layers must share one KV cache shape, dtype and strides")
        if not kv.is_cuda:
            raise ValueError("kv_caches must be CUDA tensors")


def _check_weights(geometry: Geometry, device, embed, final_norm, layers, embed_lookup):
    """Shapes, dtypes, contiguity and device of every tensor the kernel will stream with bulk copies: a matrix of
    the wrong size would otherwise become an out-of-bounds read on the device."""
    g = geometry
    h, i, ad = g.hidden, g.intermediate, g.q_heads * HEAD_DIM

    def check(t, name, shape, dtype):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.device != device:
            raise ValueError(f"{name} must be a CUDA tensor on {device}")
        if t.dtype != dtype or tuple(t.shape) != shape or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous {dtype} tensor of shape {shape}, got {t.dtype} {tuple(t.shape)}")
        if t.data_ptr() % 16:
            raise ValueError(f"{name} must be 16-byte aligned")

    if g.weight_format:
        mat = lambda rows, k: ((rows, packed_row_bytes(k)), torch.uint8)
    else:
        mat = lambda rows, k: ((rows, k), torch.bfloat16)
    check(embed, "embed", *mat(g.vocab, h))
    check(final_norm, "final_norm", (h,), torch.bfloat16)
    if embed_lookup is not None:
        check(embed_lookup, "embed_lookup", (g.vocab, h), torch.bfloat16)
    elif g.weight_format:
        raise ValueError("MXFP8 weights need embed_lookup (the bf16 embedding rows for the input lookup)")
    specs = (("norm1", (h,), torch.bfloat16), ("qkv",) + mat(g.qkv_rows, h), ("o",) + mat(h, ad),
             ("norm2", (h,), torch.bfloat16), ("gate_up",) + mat(2 * i, h), ("down",) + mat(h, i))
    for li, layer in enumerate(layers):
        if len(layer) != 6:
            raise ValueError(f"layer {li} must contain six weight tensors")
        for t, (name, shape, dtype) in zip(layer, specs):
            check(t, f"layer {li} {name}", shape, dtype)


def decode_step(geometry: Geometry, *, input_ids, positions, seq_lens, block_table, slot_mapping, embed, layers,
                final_norm, kv_caches, cos_sin_cache, eps, layer_outputs=None, lm_head=False, advance=False,
                embed_lookup=None, name="decode", tensor_cores=True):
    """One decode step for ``geometry``.  Returns the final-normed hidden ``[B, hidden]`` (a view of a
    shared buffer), or ``(hidden, logits, next_ids)`` when ``lm_head`` is true.  Up to ``MAX_BATCH`` requests run in
    one launch of the CUDA-core kernels; batches of 4 (``set_tensor_core_min_batch``) to ``MAX_REQUESTS`` requests run
    in one launch of the tensor-core kernel (``tensor_cores=False`` runs them on the CUDA-core kernels instead, above 8
    requests as consecutive launches each of which streams the weights again; ``"force"`` takes the tensor-core kernel
    at any batch)."""
    batch = input_ids.shape[0]
    if not 1 <= batch <= MAX_REQUESTS:
        raise ValueError(f"batch must be 1..{MAX_REQUESTS}, got {batch}")
    if eps != geometry.eps:
        raise ValueError(f"the kernel is built for rms eps {geometry.eps}, got {eps}")
    if len(layers) != geometry.layers or len(kv_caches) != geometry.layers:
        raise ValueError(f"expected {geometry.layers} layers and KV caches")
    if input_ids.dtype not in (torch.int32, torch.int64) or positions.dtype != torch.int64:
        raise ValueError("input_ids must be int32 or int64 and positions int64")
    if seq_lens.dtype != torch.int32 or block_table.dtype != torch.int32 or slot_mapping.dtype != torch.int64:
        raise ValueError("seq_lens and block_table must be int32, slot_mapping int64")
    if block_table.stride(1) != 1 or block_table.shape[0] < batch:
        raise ValueError("block_table rows must be contiguous and cover the batch")
    if cos_sin_cache.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("cos_sin_cache must be BF16 or FP32")
    device = input_ids.device
    kv0 = kv_caches[0]
    # cache layouts: [blocks, kv_heads, block_size, 128] (K in 0..63, V in 64..127: the reference's layout) or
    # [2, blocks, block_size, kv_heads, 64] (K and V planes: vLLM's FlashAttention layout)
    if kv0.ndim == 5:
        if kv0.shape[0] != 2 or kv0.shape[4] != 64 or kv0.stride(4) != 1:
            raise ValueError("5-D kv caches must be [2, blocks, block_size, kv_heads, 64] with a contiguous head dim")
        block_size = kv0.shape[2]
        kv_layout = (0, kv0.stride(0), kv0.stride(1), kv0.stride(2), kv0.stride(3))
    else:
        block_size = kv0.shape[2]
        kv_layout = (0, kv0.shape[3] // 2, kv0.stride(0), kv0.stride(2), kv0.stride(1))
    max_seq = block_table.shape[1] * block_size
    if max_seq > MAX_SEQ:
        raise ValueError(f"context limit {max_seq} exceeds the kernel's {MAX_SEQ}")

    rt = _runtime(geometry, device)
    layers_t, kv_t = rt.tables(layers, kv_caches, embed, final_norm, embed_lookup)    # validates when anything changed
    logits = next_ids = None
    if lm_head:
        logits, next_ids = rt.lm_buffers()

    def launch(g0, g1, lo, path=2):
        whole = g0 == 0 and g1 == batch                 # the common case: no slicing on the hot path
        cut = (lambda t: t) if whole else (lambda t: t[g0:g1])
        return torch.ops.prime_decode.decode_step(
            cut(input_ids), cut(positions), cut(seq_lens), cut(block_table), cut(slot_mapping), embed, embed_lookup,
            layers_t, final_norm, kv_t, *kv_layout, block_size,
            cos_sin_cache, rt.out if whole else rt.out[g0:g1], (logits if whole else logits[g0:g1]) if lm_head else None,
            (next_ids if whole else next_ids[g0:g1]) if lm_head else None, lo, rt.scratch, geometry.hidden,
            geometry.intermediate, geometry.layers, geometry.q_heads, geometry.kv_heads, geometry.vocab,
            geometry.weight_format, float(eps), max_seq, bool(lm_head), bool(advance), path)

    # one launch of the tensor-core kernel (projections as tcgen05 GEMMs, weights streamed once): batches of
    # _tc_min_batch requests or more, and smaller ones that the CUDA-core kernel cannot take in one launch for this
    # geometry (rt.group)
    def tensor_core_launch():
        rc = launch(0, batch, layer_outputs, 1)
        if rc != 0:
            raise RuntimeError(f"{name} failed: {status_string(rc)}")
        if lm_head:
            return rt.out[:batch], logits[:batch], next_ids[:batch]
        return rt.out[:batch]

    if tensor_cores == "force" or (tensor_cores and (batch >= tc_min_batch(geometry) or batch > MAX_BATCH or batch > rt.group)):
        return tensor_core_launch()
    # A launch of the CUDA-core kernels takes up to rt.group requests (MAX_BATCH, fewer when the geometry's activation
    # staging does not fit shared memory at that batch: status 9111 / 9105 lowers the group once and for all).
    # With tensor_cores=False larger batches run as consecutive launches over slices of the request arrays, each of
    # which streams the weights again.
    g0 = 0
    while g0 < batch:
        g1 = min(batch, g0 + rt.group)
        whole = g0 == 0 and g1 == batch
        lo = layer_outputs if whole or layer_outputs is None else \
            torch.empty((geometry.layers, g1 - g0, geometry.hidden), dtype=torch.bfloat16, device=device)
        rc = launch(g0, g1, lo)
        if rc in (9111, 9105) and g1 - g0 > 1 and rt.group > 1:
            rt.group = max(1, (g1 - g0) // 2)
            if tensor_cores and g0 == 0 and batch > rt.group:
                return tensor_core_launch()
            continue
        if rc != 0:
            raise RuntimeError(f"{name} failed: {status_string(rc)}")
        if lo is not None and lo is not layer_outputs:
            layer_outputs[:, g0:g1].copy_(lo)
        g0 = g1
    if lm_head:
        return rt.out[:batch], logits[:batch], next_ids[:batch]
    return rt.out[:batch]


def check_status(geometry: Geometry, device) -> None:
    """Synchronise and raise if a bounded device-side wait of an earlier step gave up."""
    device = torch.device(device)
    rt = _runtimes.get((geometry, device))
    if rt is None:
        return
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        rc = library().pk_decode_status(rt.scratch.data_ptr(), stream)
    if rc != 0:
        raise RuntimeError(f"decode failed on the device: {status_string(rc)}")


class DecodeSession:
    """Greedy generation driver: all step inputs live on the device and the kernel advances them in
    place (``advance=True``), so ``steps`` launches run back to back with no host round trip."""

    def __init__(self, geometry: Geometry, *, embed, layers, final_norm, kv_caches, cos_sin_cache, block_table,
                 embed_lookup=None):
        self.geometry = geometry
        self.embed, self.layers, self.final_norm = embed, layers, final_norm
        self.kv_caches, self.cos_sin_cache, self.block_table = kv_caches, cos_sin_cache, block_table
        self.embed_lookup = embed_lookup
        self.device = embed.device
        self.block_size = kv_caches[0].shape[2]

    def start(self, last_ids: torch.Tensor, context_lens: torch.Tensor):
        """``last_ids [B]``: the token to feed first; ``context_lens [B]``: tokens already in the cache."""
        dev = self.device
        self.input_ids = last_ids.to(dev, torch.int64).clone()
        self.positions = context_lens.to(dev, torch.int64).clone()
        self.seq_lens = (context_lens.to(dev, torch.int32) + 1).clone()
        bt = self.block_table
        rows = torch.arange(bt.shape[0], device=dev)[: self.input_ids.shape[0]]
        blk = bt[rows, (self.positions // self.block_size).long()].to(torch.int64)
        self.slot_mapping = blk * self.block_size + self.positions % self.block_size

    def step(self):
        return decode_step(self.geometry, input_ids=self.input_ids, positions=self.positions,
                           seq_lens=self.seq_lens, block_table=self.block_table, slot_mapping=self.slot_mapping,
                           embed=self.embed, layers=self.layers, final_norm=self.final_norm,
                           kv_caches=self.kv_caches, cos_sin_cache=self.cos_sin_cache, eps=self.geometry.eps,
                           lm_head=True, advance=True, embed_lookup=self.embed_lookup)

    def generate(self, steps: int, collect_logits: bool = False):
        """Run ``steps`` greedy steps; returns ids ``[steps, B]`` (and logits ``[steps, B, V]``)."""
        b = self.input_ids.shape[0]
        ids = torch.empty((steps, b), dtype=torch.int64, device=self.device)
        logs = torch.empty((steps, b, self.geometry.vocab), dtype=torch.bfloat16, device=self.device) if collect_logits else None
        for t in range(steps):
            _, logits, next_ids = self.step()
            ids[t].copy_(next_ids)
            if collect_logits:
                logs[t].copy_(logits)
        check_status(self.geometry, self.device)
        return (ids, logs) if collect_logits else ids


class HostStep:
    """One decode step driven from host buffers, for serving loops that produce the step inputs on the CPU.

    The four per-step inputs (ids, positions, slot mapping as int64, sequence lengths as int32) live in one pinned
    staging buffer and one device buffer, so a step is one host-to-device copy of 28 bytes per request, one kernel
    launch (tied lm_head + argmax fused) and one device-to-host copy of the greedy ids; with ``graph=True`` the
    three are captured once into a CUDA graph and replayed.  ``__call__`` returns the greedy next ids as a pinned
    host tensor ``[B]`` after synchronising the stream."""

    def __init__(self, geometry: Geometry, batch: int, *, embed, layers, final_norm, kv_caches, cos_sin_cache,
                 block_table, embed_lookup=None, graph: bool = True):
        self.geometry, self.batch = geometry, batch
        dev = embed.device
        self.device = dev
        self.h_buf = torch.empty(batch * 28, dtype=torch.uint8).pin_memory()
        self.d_buf = torch.empty(batch * 28, dtype=torch.uint8, device=dev)
        self.h_ids, self.h_pos, self.h_slot, self.h_seq = self._views(self.h_buf)
        d_ids, d_pos, d_slot, d_seq = self._views(self.d_buf)
        self.h_next = torch.empty(batch, dtype=torch.int64).pin_memory()
        self._kw = dict(input_ids=d_ids, positions=d_pos, seq_lens=d_seq, block_table=block_table, slot_mapping=d_slot,
                        embed=embed, layers=layers, final_norm=final_norm, kv_caches=kv_caches,
                        cos_sin_cache=cos_sin_cache, eps=geometry.eps, lm_head=True, embed_lookup=embed_lookup)
        self.graph = None
        if graph:
            self.h_ids.zero_()
            self.h_pos.zero_()
            self.h_slot.fill_(-1)          # a padded row: the capture run writes nothing into the cache
            self.h_seq.fill_(1)
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                self._enqueue()            # first call outside capture (workspace set-up, pointer tables)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=side):
                    self._enqueue()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            self.graph = g
        self._stream = torch.cuda.current_stream(dev)
        # numpy views of the pinned buffers (ids, positions, slots, sequence lengths, next ids)
        self._np = (self.h_ids.numpy(), self.h_pos.numpy(), self.h_slot.numpy(), self.h_seq.numpy(), self.h_next.numpy())

    def _views(self, buf):
        b = self.batch
        i64 = buf[: b * 24].view(torch.int64)
        return i64[:b], i64[b: 2 * b], i64[2 * b: 3 * b], buf[b * 24:].view(torch.int32)

    def _enqueue(self):
        self.d_buf.copy_(self.h_buf, non_blocking=True)
        _, _, nxt = decode_step(self.geometry, **self._kw)
        self.h_next.copy_(nxt, non_blocking=True)

    def __call__(self, ids, positions, seq_lens, slot_mapping):
        """Step inputs as host tensors ``[B]``; returns the greedy next ids (pinned host tensor, int64)."""
        self.h_ids.copy_(ids)
        self.h_pos.copy_(positions)
        self.h_seq.copy_(seq_lens)
        self.h_slot.copy_(slot_mapping)
        return self._run()

    def step_numpy(self, ids, positions, seq_lens, slot_mapping):
        """Same step with the inputs as numpy arrays, sequences or scalars (broadcast over the batch), written straight
        into the pinned staging buffer: no tensor dispatch on the host side of a serving loop.  Returns the greedy
        next ids as a numpy view ``[B]`` (int64) of the pinned result buffer."""
        n = self._np
        n[0][:] = ids
        n[1][:] = positions
        n[2][:] = slot_mapping
        n[3][:] = seq_lens
        self._run()
        return n[4]

    def _run(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._enqueue()
        self._stream.synchronize()
        return self.h_next

