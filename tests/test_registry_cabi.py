"""CPU: registry behaviour (mirrors the reference registry's contract) and the C-ABI surface."""
import ctypes
import re
from pathlib import Path

import pytest

import prime_kernels_b200 as pk
from prime_kernels_b200 import _cabi
from prime_kernels_b200._spec import Arch

ROOT = Path(__file__).resolve().parents[1]


def test_manifest_tables_and_arch():
    assert set(pk.KERNELS) >= {"rmsnorm", "decode_megakernel", "decode_megakernel_360m"}
    for name in pk.KERNELS:
        spec = pk.spec(name)
        assert spec.sm_list == "sm_100a"
        assert spec.supports((10, 0)) and not spec.supports((8, 9)) and not spec.supports((10, 3))
        assert spec.module == f"prime_kernels_b200.{name}"
    assert pk.spec("rmsnorm").ops == "prime_rmsnorm"
    assert Arch.parse("10.0a").gencode() == "-gencode=arch=compute_100a,code=sm_100a"
    with pytest.raises(ValueError):
        Arch.parse("sm_100")


def test_unknown_kernel_raises_keyerror():
    with pytest.raises(KeyError):
        pk.spec("nope")


def test_status_without_a_device_reports_reason_and_load_raises():
    import torch

    if torch.cuda.is_available():
        pytest.skip("CPU-only check")
    st = pk.status()
    assert set(st) == set(pk.KERNELS)
    for name, reason in st.items():
        assert "requires a CUDA device (sm_100a)" in reason
        assert not pk.is_available(name)
        with pytest.raises(RuntimeError):
            pk.load(name)


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "prime_kernels_b200.h").read_text()
    declared = set(re.findall(r"\b((?:pk_|mk_|decode360)\w*)\s*\(", header))
    assert declared == set(_cabi.SYMBOLS), declared ^ set(_cabi.SYMBOLS)
    lib = _cabi.library()
    for name in declared:
        assert getattr(lib, name) is not None


def test_status_strings_and_sizes_without_a_device():
    lib = _cabi.library()
    assert lib.pk_status_string(9101).decode() == "batch_must_be_1_to_64"
    assert lib.mk_status_string(9110).decode() == "device_wait_timed_out"
    assert lib.decode360_status_string(9106).decode() == "kernel_requires_sm100"
    assert lib.pk_rmsnorm_scale_bytes(1, 960) == 8 * 512
    assert lib.pk_rmsnorm_scale_bytes(8192, 4096) == 64 * 32 * 512
    assert lib.mk_workspace_bytes(1, 2048) == lib.mk_workspace_bytes(8, 8192) > 0
    assert lib.decode360_workspace_bytes() > 0
    m = _cabi.PkDecodeModel(960, 2560, 32, 15, 5, 49152, 0, 1e-5)
    # from 4 requests on the workspace also holds the tensor-core kernel's region, behind the CUDA-core kernels' one
    assert lib.pk_decode_workspace_bytes(ctypes.byref(m), 8) > lib.decode360_workspace_bytes()
    assert lib.pk_decode_workspace_bytes(ctypes.byref(m), 3) < lib.decode360_workspace_bytes()


def test_argument_validation_needs_no_device():
    lib = _cabi.library()
    # contract violations are rejected before any CUDA call
    assert lib.pk_fused_rmsnorm_residual_forward(None, None, None, None, None, None, 1e-6, 4, 100, None) == 9111
    assert lib.pk_fused_rmsnorm_residual_forward(None, None, None, None, None, None, 1e-6, 4, 128, None) == 9103
    # the drop-in entries validate like the reference: batch first, then the context capacity, then pointers
    def mk(batch, max_seq):       # stream, B, ids, ids_i64, positions, seq_lens, block_table, bt_stride, slot_mapping,
        return lib.mk_decode(None, batch, None, 0, None, None, None, 128, None,     # layers, embed, final_norm, kv,
                             None, None, None, None, 0, 64, 0, 0, 0, 16,            # 5 strides, block_size,
                             None, 0, None, None, 0, max_seq)                       # cos_sin, fp32, out, scratch, bytes

    assert mk(9, 2048) == 9101
    assert mk(1, 9000) == 9102
    assert mk(1, 2048) == 9103

    def d360(batch, max_seq, debug_layer):
        return lib.decode360(None, batch, None, None, None, None, None, None, 128, None, None, None, 0, 64, 0, 0, 0, 16,
                             None, 0, None, None, None, 0, None, 0, max_seq, debug_layer)

    assert d360(9, 2048, -1) == 9101
    assert d360(1, 2048, 40) == 9109          # debug_layer_index out of range
    assert d360(1, 2048, -1) == 9103
    m = _cabi.PkDecodeModel(960, 2560, 32, 15, 5, 49152, 0, 1e-5)
    a = _cabi.PkDecodeArgs()
    a.batch = 65
    assert lib.pk_decode_step(ctypes.byref(m), ctypes.byref(a)) == 9101
    a.batch = 1
    a.max_seq_len = 9000
    assert lib.pk_decode_step(ctypes.byref(m), ctypes.byref(a)) == 9102
    a.max_seq_len = 128
    assert lib.pk_decode_step(ctypes.byref(m), ctypes.byref(a)) == 9103


def test_ops_are_registered_with_fake_kernels():
    import torch

    from prime_kernels_b200 import decode, rmsnorm  # noqa: F401  (registers fakes)

    x = torch.empty(130, 960, dtype=torch.bfloat16, device="meta")
    w = torch.empty(960, dtype=torch.bfloat16, device="meta")
    vals, scales, rrms = torch.ops.prime_rmsnorm.fused_rmsnorm_residual(x, x, w, 1e-6)
    assert vals.shape == (130, 960) and vals.dtype == torch.float8_e4m3fn
    assert scales.shape == (2 * 8 * 512,) and scales.dtype == torch.float8_e8m0fnu
    assert rrms.shape == (130,) and rrms.dtype == torch.float32
    out = torch.ops.prime_rmsnorm.fused_rmsnorm_residual_ex(x, x, w, 1e-6, True, True)
    assert out[3].shape == (130, 960)


def test_reference_constants_are_exported():
    from prime_kernels_b200 import decode_megakernel as a, decode_megakernel_360m as b

    assert (a.HIDDEN, a.KV_HEADS, a.HEAD_DIM, a.LAYERS, a.EPS, a.MAX_SEQ) == (576, 3, 64, 30, 1e-5, 8192)
    assert (b.HIDDEN, b.INTERMEDIATE, b.LAYERS, b.KV_HEADS, b.HEAD_DIM, b.BLOCK_SIZE, b.EPS) == (960, 2560, 32, 5, 64, 16, 1e-5)
    assert a.MAX_BATCH >= 4 and b.MAX_BATCH >= 2
    assert a.SOURCE.exists() and b.SOURCE.exists()


def test_decode_contract_errors_are_valueerrors():
    import torch

    from prime_kernels_b200 import decode_megakernel as a

    ids = torch.zeros(65, dtype=torch.int64)
    with pytest.raises(ValueError, match="batch must be 1..64"):
        a.decode_step(input_ids=ids, positions=ids, seq_lens=ids, block_table=ids, slot_mapping=ids, embed=None,
                      layers=[], final_norm=None, kv_caches=[], cos_sin_cache=None, eps=1e-5)
    ids = torch.zeros(1, dtype=torch.int64)
    with pytest.raises(ValueError, match="rms eps"):
        a.decode_step(input_ids=ids, positions=ids, seq_lens=ids, block_table=ids, slot_mapping=ids, embed=None,
                      layers=[], final_norm=None, kv_caches=[], cos_sin_cache=None, eps=1e-6)
    with pytest.raises(ValueError, match="expected 30 layers"):
        a.decode_step(input_ids=ids, positions=ids, seq_lens=ids, block_table=ids, slot_mapping=ids, embed=None,
                      layers=[], final_norm=None, kv_caches=[], cos_sin_cache=None, eps=1e-5)


def test_rmsnorm_dispatch_keeps_misaligned_pointers_off_the_bulk_copy_kernel():
    """The pipelined kernel moves data with bulk copies, which need 16-byte aligned global addresses; the C entry
    accepts `vals` at 8-byte alignment, so such a pointer must be routed to another kernel (host-side check)."""
    lib = _cabi.library()
    base = 1 << 20
    assert lib.pk_rmsnorm_dispatch(base, base, base, base, 8192, 8192) == 2
    assert lib.pk_rmsnorm_dispatch(base, base, base, base, 2048, 16384) == 2
    assert lib.pk_rmsnorm_dispatch(base + 8, base, base, base, 8192, 8192) == 0      # vals only 8-byte aligned
    assert lib.pk_rmsnorm_dispatch(base + 16, base, base, base, 8192, 8192) == 2     # 16 is enough for the pipe
    assert lib.pk_rmsnorm_dispatch(base, base + 16, base, base, 8192, 4096) == 0     # group kernel wants 32
    assert lib.pk_rmsnorm_dispatch(base, base, base, base, 8192, 4096) == 1
    assert lib.pk_rmsnorm_dispatch(base + 4, base, base, base, 8192, 8192) == -9107
    assert lib.pk_rmsnorm_dispatch(base, base, base, base, 128, 100) == -9111


def test_workspace_bytes_covers_every_batch_up_to_the_declared_maximum():
    """A caller that sizes the workspace for max_batch must be able to run every batch up to it: the size never
    shrinks as max_batch grows; from 4 requests on it contains the CUDA-core kernels' batch-8 region (batches 5..7
    run on the batch-8 kernel) followed by the tensor-core kernel's region; more than 64 requests per launch is
    refused (0)."""
    lib = _cabi.library()
    m = _cabi.PkDecodeModel(960, 2560, 32, 15, 5, 49152, 0, 1e-5)
    sizes = [lib.pk_decode_workspace_bytes(ctypes.byref(m), b) for b in range(1, 66)]
    assert all(sizes[i] <= sizes[i + 1] for i in range(63))
    assert sizes[3] > lib.decode360_workspace_bytes() > sizes[2]
    assert sizes[63] > 0 and sizes[64] == 0
    assert lib.pk_decode_workspace_bytes(ctypes.byref(m), 0) == 0
