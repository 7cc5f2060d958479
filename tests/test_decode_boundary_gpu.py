"""GPU tests of the drop-in C entries and of the failure path of the decode kernels.

* ``mk_decode`` / ``decode360`` are bound with ctypes exactly as a caller of the reference binds them
  (prime_kernels/decode_megakernel/__init__.py:72-91 and
  prime_kernels/decode_megakernel_360m/__init__.py:66-93 in the reference project: the same argtypes) and
  must give what the Python surface of this library gives on the same inputs.
* The failure path is exercised without ever hanging or faulting the GPU: a one-CTA probe whose bounded wait
  runs out (status 9110), and a launch on a workspace whose status word is already set, which must fall
  through every wait, report the code and leave the workspace usable.
"""
import ctypes

import pytest
import torch

from oracle import decode_restatement as R
from prime_kernels_b200 import harness

pytestmark = pytest.mark.gpu
vp, ci, ll, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_size_t


def _reference_style_library():
    """ctypes handle with the argtypes a reference caller declares (nothing of this package's own table)."""
    from prime_kernels_b200._cabi import LIBRARY

    lib = ctypes.CDLL(str(LIBRARY))
    lib.mk_workspace_bytes.argtypes, lib.mk_workspace_bytes.restype = [ci, ci], sz
    lib.mk_decode.argtypes = [vp, ci, vp, ci, vp, vp, vp, ci, vp, vp, vp, vp, vp, ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, sz, ci]
    lib.mk_decode.restype = ci
    lib.mk_status_string.argtypes, lib.mk_status_string.restype = [ci], ctypes.c_char_p
    lib.decode360_workspace_bytes.argtypes, lib.decode360_workspace_bytes.restype = [], sz
    lib.decode360_debug_bytes.argtypes, lib.decode360_debug_bytes.restype = [], sz
    lib.decode360.argtypes = [vp, ci, vp, vp, vp, vp, vp, vp, ci, vp, vp, vp, ll, ll, ll, ll, ll, ci, vp, ci, vp, vp, vp, sz,
                              vp, sz, ci, ci]
    lib.decode360.restype = ci
    lib.decode360_status_string.argtypes, lib.decode360_status_string.restype = [ci], ctypes.c_char_p
    return lib


def _tables(wd, kv, dev):
    layer_t = torch.tensor([[t.data_ptr() for t in layer] for layer in wd["layers"]], dtype=torch.int64, device=dev)
    kv_t = torch.tensor([c.data_ptr() for c in kv.kv_caches], dtype=torch.int64, device=dev)
    return layer_t, kv_t


def _filled_cache(geom, batch, cap, dev, seed):
    kv = harness.PagedKV(geom, batch, cap, dev, shuffle=True, seed=2)
    g = torch.Generator().manual_seed(seed)
    for cache in kv.kv_caches:
        cache.copy_((torch.randn(cache.shape, generator=g) * 0.5).to(torch.bfloat16))
    return kv


@pytest.mark.parametrize("batch", [1, 3])
def test_mk_decode_through_the_reference_binding(cuda_device, batch):
    """SmolLM2-135M through ``mk_decode`` with int32 ids and a caller-owned ``torch.empty`` scratch of
    ``mk_workspace_bytes`` bytes, against ``decode_megakernel.decode_step`` of this package."""
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel as MK

    dev = cuda_device
    lib = _reference_style_library()
    geom = D.SMOLLM2_135M
    wd = harness.weights_to(harness.make_weights(geom, 0, norm_weights="random"), dev)
    csd = harness.make_cos_sin_cache(geom, 256, dev)
    ctxs = [40, 7, 130][:batch]
    pos = torch.tensor(ctxs, dtype=torch.int64, device=dev)
    seq = (pos + 1).to(torch.int32)
    ids32 = torch.tensor([11, 2222, 40000][:batch], dtype=torch.int32, device=dev)
    kv_a, kv_b = _filled_cache(geom, batch, 256, dev, 9), _filled_cache(geom, batch, 256, dev, 9)
    layer_t, kv_t = _tables(wd, kv_a, dev)
    scratch = torch.empty(lib.mk_workspace_bytes(batch, 256), dtype=torch.uint8, device=dev)
    out = torch.zeros(batch, geom.hidden, dtype=torch.bfloat16, device=dev)
    kv0 = kv_a.kv_caches[0]
    slots = kv_a.slots(pos)
    rc = lib.mk_decode(torch.cuda.current_stream(dev).cuda_stream, batch, ids32.data_ptr(), 0, pos.data_ptr(), seq.data_ptr(),
                       kv_a.block_table.data_ptr(), kv_a.block_table.stride(0), slots.data_ptr(), layer_t.data_ptr(),
                       wd["embed"].data_ptr(), wd["final_norm"].data_ptr(), kv_t.data_ptr(), 0, 64, kv0.stride(0),
                       kv0.stride(2), kv0.stride(1), kv0.shape[2], csd.data_ptr(), 0, out.data_ptr(), scratch.data_ptr(),
                       scratch.numel(), kv_a.block_table.shape[1] * kv0.shape[2])
    assert rc == 0, lib.mk_status_string(rc)
    torch.cuda.synchronize(dev)
    want = MK.decode_step(input_ids=ids32, positions=pos, seq_lens=seq, block_table=kv_b.block_table,
                          slot_mapping=kv_b.slots(pos), embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"],
                          kv_caches=kv_b.kv_caches, cos_sin_cache=csd, eps=MK.EPS)
    D.check_status(geom, dev)
    assert torch.equal(out, want)
    for ca, cb in zip(kv_a.kv_caches, kv_b.kv_caches):
        assert torch.equal(ca, cb)
    _cabi_forget(scratch)


def _cabi_forget(t):
    from prime_kernels_b200._cabi import library

    library().pk_decode_workspace_forget(t.data_ptr())


def test_decode360_through_the_reference_binding(cuda_device):
    """SmolLM2-360M through ``decode360`` (28 arguments, ``layer_outputs`` requested, a ``debug`` buffer of
    ``decode360_debug_bytes`` passed and left untouched) against ``decode_megakernel_360m.decode_step``."""
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200 import decode_megakernel_360m as MK360

    dev = cuda_device
    lib = _reference_style_library()
    geom = D.SMOLLM2_360M
    wd = harness.weights_to(harness.make_weights(geom, 0), dev)
    csd = harness.make_cos_sin_cache(geom, 640, dev)
    for batch, ctxs in ((1, [520]), (2, [33, 300])):
        pos = torch.tensor(ctxs, dtype=torch.int64, device=dev)
        seq = (pos + 1).to(torch.int32)
        ids = torch.tensor([5, 48000][:batch], dtype=torch.int32, device=dev)
        kv_a, kv_b = _filled_cache(geom, batch, 640, dev, 4), _filled_cache(geom, batch, 640, dev, 4)
        layer_t, kv_t = _tables(wd, kv_a, dev)
        scratch = torch.empty(lib.decode360_workspace_bytes(), dtype=torch.uint8, device=dev)
        debug = torch.full((max(16, lib.decode360_debug_bytes()),), 0x5a, dtype=torch.uint8, device=dev)
        out = torch.zeros(batch, geom.hidden, dtype=torch.bfloat16, device=dev)
        lo = torch.zeros(geom.layers, batch, geom.hidden, dtype=torch.bfloat16, device=dev)
        kv0 = kv_a.kv_caches[0]
        slots = kv_a.slots(pos)
        rc = lib.decode360(torch.cuda.current_stream(dev).cuda_stream, batch, ids.data_ptr(), wd["embed"].data_ptr(),
                           wd["final_norm"].data_ptr(), pos.data_ptr(), seq.data_ptr(), kv_a.block_table.data_ptr(),
                           kv_a.block_table.stride(0), slots.data_ptr(), layer_t.data_ptr(), kv_t.data_ptr(), 0, 64,
                           kv0.stride(0), kv0.stride(2), kv0.stride(1), 16, csd.data_ptr(), 0, out.data_ptr(), lo.data_ptr(),
                           scratch.data_ptr(), scratch.numel(), debug.data_ptr(), debug.numel(),
                           kv_a.block_table.shape[1] * 16, -1)
        assert rc == 0, lib.decode360_status_string(rc)
        torch.cuda.synchronize(dev)
        lo_b = torch.zeros_like(lo)
        want = MK360.decode_step(input_ids=ids, positions=pos, seq_lens=seq, block_table=kv_b.block_table,
                                 slot_mapping=kv_b.slots(pos), embed=wd["embed"], layers=wd["layers"],
                                 final_norm=wd["final_norm"], kv_caches=kv_b.kv_caches, cos_sin_cache=csd, eps=MK360.EPS,
                                 layer_outputs=lo_b)
        D.check_status(geom, dev)
        assert torch.equal(out, want)
        assert torch.equal(lo, lo_b)
        assert (debug == 0x5a).all()
        for ca, cb in zip(kv_a.kv_caches, kv_b.kv_caches):
            assert torch.equal(ca, cb)
        _cabi_forget(scratch)


def test_bounded_wait_runs_out_and_reports_9110(cuda_device):
    """A one-CTA probe polls a flagged word that nothing writes with the decode kernels' bounded wait and a limit
    of a few thousand rounds: the launch returns by itself, ``pk_decode_status`` reports 9110 and clears it, and
    the next decode step on the same workspace (re-zeroed by the library) is correct."""
    from prime_kernels_b200 import decode as D
    from prime_kernels_b200._cabi import library

    dev = cuda_device
    lib = library()
    geom = D.Geometry("probe", 192, 512, 2, 3, 1, 1024)
    w = harness.make_weights(geom, 6, norm_weights="random")
    wd = harness.weights_to(w, dev)
    cs = harness.make_cos_sin_cache(geom, 64)
    kv = harness.PagedKV(geom, 1, 64, dev)
    keys = [[torch.zeros(geom.kv_heads, 0, 64, dtype=torch.bfloat16)] for _ in range(geom.layers)]
    vals = [[torch.zeros(geom.kv_heads, 0, 64, dtype=torch.bfloat16)] for _ in range(geom.layers)]

    def step(tok, p):
        pos = torch.tensor([p])
        return D.decode_step(geom, input_ids=torch.tensor([tok], device=dev), positions=pos.to(dev),
                             seq_lens=(pos + 1).to(torch.int32).to(dev), block_table=kv.block_table, slot_mapping=kv.slots(pos),
                             embed=wd["embed"], layers=wd["layers"], final_norm=wd["final_norm"], kv_caches=kv.kv_caches,
                             cos_sin_cache=cs.to(dev), eps=geom.eps, lm_head=True)

    step(3, 0)                                                   # creates the per-geometry workspace
    D.check_status(geom, dev)
    R.decode_step(geom, w, torch.tensor([3]), torch.tensor([0]), keys, vals, cs)
    ws = D._runtime(geom, dev).scratch
    stream = torch.cuda.current_stream(dev).cuda_stream
    assert lib.pk_decode_wait_probe(ws.data_ptr(), ws.numel(), 4096, stream) == 0
    assert lib.pk_decode_status(ws.data_ptr(), stream) == 9110
    assert lib.pk_status_string(9110) == b"device_wait_timed_out"
    assert lib.pk_decode_status(ws.data_ptr(), stream) == 0      # cleared
    _, logits, nxt = step(9, 1)
    D.check_status(geom, dev)
    _, rl, _ = R.decode_step(geom, w, torch.tensor([9]), torch.tensor([1]), keys, vals, cs)
    assert (logits.cpu().float() - rl).abs().max() <= 2e-2
    assert lib.pk_decode_wait_probe(None, 0, 16, stream) == 9103
    assert lib.pk_decode_wait_probe(ws.data_ptr(), ws.numel(), 0, stream) == 9111


@pytest.mark.parametrize("which", ["generic", "fast"])
def test_launch_on_a_failed_workspace_falls_through(cuda_device, which):
    """The status word of a workspace is set before a launch (as if an earlier step's wait had run out): every
    wait of the kernel must give up at once, the launch must end by itself, ``check_status`` must raise with the
    code, and the next step must be correct again.  Both kernels, several warps each taking the early exit."""
    from prime_kernels_b200 import decode as D

    dev = cuda_device
    if which == "fast":
        geom = D.Geometry("fall-360w", 960, 2560, 2, 15, 5, 2048)
    else:
        geom = D.Geometry("fall-generic", 192, 512, 2, 3, 1, 1024)
    batch = 1 if which == "fast" else 2
    w = harness.make_weights(geom, 8, norm_weights="random")
    wd = harness.weights_to(w, dev)
    cs = harness.make_cos_sin_cache(geom, 64)
    kv = harness.PagedKV(geom, batch, 64, dev)
    keys = [[torch.zeros(geom.kv_heads, 0, 64, dtype=torch.bfloat16) for _ in range(batch)] for _ in range(geom.layers)]
    vals = [[torch.zeros(geom.kv_heads, 0, 64, dtype=torch.bfloat16) for _ in range(batch)] for _ in range(geom.layers)]

    def step(toks, p, slot_ok=True):
        pos = torch.full((batch,), p, dtype=torch.int64)
        slots = kv.slots(pos) if slot_ok else torch.full((batch,), -1, dtype=torch.int64, device=dev)
        return D.decode_step(geom, input_ids=toks.to(dev), positions=pos.to(dev), seq_lens=(pos + 1).to(torch.int32).to(dev),
                             block_table=kv.block_table, slot_mapping=slots, embed=wd["embed"], layers=wd["layers"],
                             final_norm=wd["final_norm"], kv_caches=kv.kv_caches, cos_sin_cache=cs.to(dev), eps=geom.eps,
                             lm_head=True)

    toks = torch.arange(1, batch + 1)
    step(toks, 0)
    D.check_status(geom, dev)
    R.decode_step(geom, w, toks, torch.zeros(batch, dtype=torch.int64), keys, vals, cs)
    ws = D._runtime(geom, dev).scratch
    ws.view(torch.int32)[1] = 9110                               # the status word (control word 1)
    before = [c.clone() for c in kv.kv_caches]
    step(toks, 1, slot_ok=False)                                 # must return by itself
    torch.cuda.synchronize(dev)
    with pytest.raises(RuntimeError, match="device_wait_timed_out"):
        D.check_status(geom, dev)
    for c, b in zip(kv.kv_caches, before):
        assert torch.equal(c, b)
    _, logits, _ = step(toks, 1)
    D.check_status(geom, dev)
    _, rl, _ = R.decode_step(geom, w, toks, torch.ones(batch, dtype=torch.int64), keys, vals, cs)
    assert (logits.cpu().float() - rl).abs().max() <= 2e-2
