"""TEST INFRASTRUCTURE: Python face of the MXFP8 quantiser oracles.

``port``  = oracle/mxfp8_oracle.c (plain-C restatement of prime_kernels/rmsnorm/test.cu:82-150
            and :57-65), built by oracle/Makefile into oracle/libpk_oracle.so.
``ref``   = the reference project's own ``reference()`` compiled from the reference checkout
            by oracle/build_ref.sh into oracle/_ref/libref_rmsnorm.so (may be absent).
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
_PORT = None
_REF = None

u8p = ctypes.POINTER(ctypes.c_uint8)
u16p = ctypes.POINTER(ctypes.c_uint16)
f32p = ctypes.POINTER(ctypes.c_float)
f64p = ctypes.POINTER(ctypes.c_double)


def _ptr(a, t):
    return a.ctypes.data_as(t) if a is not None else None


def build(force: bool = False) -> None:
    so = HERE / "libpk_oracle.so"
    src = HERE / "mxfp8_oracle.c"
    if force or not so.exists() or so.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(HERE), "libpk_oracle.so"], check=True, capture_output=True)


def port() -> ctypes.CDLL:
    global _PORT
    if _PORT is None:
        build()
        lib = ctypes.CDLL(str(HERE / "libpk_oracle.so"))
        lib.pk_bf16_to_float.argtypes = [ctypes.c_uint16]
        lib.pk_bf16_to_float.restype = ctypes.c_float
        lib.pk_float_to_bf16.argtypes = [ctypes.c_float]
        lib.pk_float_to_bf16.restype = ctypes.c_uint16
        lib.pk_float_to_e8m0_rp.argtypes = [ctypes.c_float]
        lib.pk_float_to_e8m0_rp.restype = ctypes.c_uint8
        lib.pk_e8m0_to_bf16.argtypes = [ctypes.c_uint8]
        lib.pk_e8m0_to_bf16.restype = ctypes.c_uint16
        lib.pk_bf16_to_e4m3.argtypes = [ctypes.c_uint16]
        lib.pk_bf16_to_e4m3.restype = ctypes.c_uint8
        lib.pk_sf_offset.argtypes = [ctypes.c_int] * 3
        lib.pk_sf_offset.restype = ctypes.c_int64
        lib.pk_scale_bytes.argtypes = [ctypes.c_int] * 2
        lib.pk_scale_bytes.restype = ctypes.c_int64
        lib.pk_oracle_rmsnorm_mxfp8.argtypes = [u16p, u16p, u16p, f32p, ctypes.c_float, ctypes.c_int,
                                                ctypes.c_int, ctypes.c_int, u8p, u8p, f64p, u16p]
        lib.pk_oracle_rmsnorm_mxfp8.restype = ctypes.c_int
        lib.pk_oracle_quantise_weight.argtypes = [u16p, ctypes.c_int64, ctypes.c_int, u8p, u8p]
        lib.pk_oracle_quantise_weight.restype = ctypes.c_int
        lib.pk_oracle_quantise_weight_floor.argtypes = [u16p, ctypes.c_int64, ctypes.c_int, u8p, u8p]
        lib.pk_oracle_quantise_weight_floor.restype = ctypes.c_int
        lib.pk_float_to_e4m3.argtypes = [ctypes.c_float]
        lib.pk_float_to_e4m3.restype = ctypes.c_uint8
        _PORT = lib
    return _PORT


def ref_available() -> bool:
    return (HERE / "_ref" / "libref_rmsnorm.so").exists()


def ref() -> ctypes.CDLL:
    global _REF
    if _REF is None:
        lib = ctypes.CDLL(str(HERE / "_ref" / "libref_rmsnorm.so"))
        lib.ref_rmsnorm_mxfp8.argtypes = [u16p, u16p, u16p, f32p, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, u8p, u8p, f64p]
        lib.ref_rmsnorm_mxfp8.restype = ctypes.c_int
        lib.ref_bf16_to_e4m3.argtypes = [ctypes.c_uint16]
        lib.ref_bf16_to_e4m3.restype = ctypes.c_uint8
        lib.ref_float_to_e8m0_rp.argtypes = [ctypes.c_float]
        lib.ref_float_to_e8m0_rp.restype = ctypes.c_uint8
        lib.ref_e8m0_to_bf16.argtypes = [ctypes.c_uint8]
        lib.ref_e8m0_to_bf16.restype = ctypes.c_uint16
        lib.ref_float_to_bf16.argtypes = [ctypes.c_float]
        lib.ref_float_to_bf16.restype = ctypes.c_uint16
        lib.ref_sf_offset_c.argtypes = [ctypes.c_int] * 3
        lib.ref_sf_offset_c.restype = ctypes.c_longlong
        _REF = lib
    return _REF


_REF_GPU = None


def ref_gpu_available() -> bool:
    return (HERE / "_ref" / "libref_rmsnorm_gpu.so").exists()


def ref_gpu() -> ctypes.CDLL:
    """The reference's own GPU kernels (oracle/ref_rmsnorm_gpu_wrapper.cu); device pointers as integers."""
    global _REF_GPU
    if _REF_GPU is None:
        lib = ctypes.CDLL(str(HERE / "_ref" / "libref_rmsnorm_gpu.so"))
        vp = ctypes.c_void_p
        lib.ref_rmsnorm_gpu.argtypes = [ctypes.c_char_p, vp, vp, vp, vp, vp, vp, ctypes.c_float, ctypes.c_int,
                                        ctypes.c_int, vp]
        lib.ref_rmsnorm_gpu.restype = ctypes.c_int
        _REF_GPU = lib
    return _REF_GPU


def scale_bytes(n: int, c: int) -> int:
    return ((n + 127) // 128) * ((c + 127) // 128) * 512


def quantise_port(branch, residual, weight, s, eps, mode=0, want_res=False):
    """Run the plain-C oracle.  Arrays are uint16 views of bf16; s is float32 [N] or None."""
    n, c = branch.shape
    vals = np.zeros((n, c), np.uint8)
    scales = np.zeros(scale_bytes(n, c), np.uint8)
    rrms = np.zeros(n, np.float64)
    res = np.zeros((n, c), np.uint16) if want_res else None
    b = np.ascontiguousarray(branch, np.uint16)
    r = np.ascontiguousarray(residual, np.uint16)
    w = np.ascontiguousarray(weight, np.uint16)
    sv = np.ascontiguousarray(s, np.float32) if s is not None else None
    rc = port().pk_oracle_rmsnorm_mxfp8(_ptr(b, u16p), _ptr(r, u16p), _ptr(w, u16p), _ptr(sv, f32p),
                                        float(eps), n, c, mode, _ptr(vals, u8p), _ptr(scales, u8p),
                                        _ptr(rrms, f64p), _ptr(res, u16p))
    if rc:
        raise ValueError("oracle rejected the shape (C must be a multiple of 32)")
    return vals, scales, rrms, res


def quantise_ref(branch, residual, weight, s, eps, math=1):
    """Run the reference project's own CPU reference (needs N, C multiples of 128)."""
    n, c = branch.shape
    vals = np.zeros((n, c), np.uint8)
    scales = np.zeros(scale_bytes(n, c), np.uint8)
    rrms = np.zeros(n, np.float64)
    b = np.ascontiguousarray(branch, np.uint16)
    r = np.ascontiguousarray(residual, np.uint16)
    w = np.ascontiguousarray(weight, np.uint16)
    sv = np.ascontiguousarray(s, np.float32)
    ref().ref_rmsnorm_mxfp8(_ptr(b, u16p), _ptr(r, u16p), _ptr(w, u16p), _ptr(sv, f32p), float(eps), n, c,
                            math, 32, _ptr(vals, u8p), _ptr(scales, u8p), _ptr(rrms, f64p))
    return vals, scales, rrms


def quantise_weight(w_bits, scale_mode="roundup"):
    """Per-32-along-K MXFP8 quantisation of a [rows, K] bf16 (uint16 view) matrix.  ``scale_mode``: "roundup" (the
    rmsnorm quantiser's rule, never saturates) or "floor" (the flash_moe block-scale rule, may saturate at 448)."""
    rows, k = w_bits.shape
    vals = np.zeros((rows, k), np.uint8)
    scales = np.zeros((rows, k // 32), np.uint8)
    w = np.ascontiguousarray(w_bits, np.uint16)
    fn = port().pk_oracle_quantise_weight if scale_mode == "roundup" else port().pk_oracle_quantise_weight_floor
    rc = fn(_ptr(w, u16p), rows, k, _ptr(vals, u8p), _ptr(scales, u8p))
    if rc:
        raise ValueError("K must be a multiple of 32")
    return vals, scales


def lcg_inputs(n: int, c: int):
    """The reference test's input recipe (prime_kernels/rmsnorm/test.cu:242-258): LCG seed 12345,
    uniform [-1, 1) rounded to bf16; row 0 all zero; residual[1, 5] = 240."""
    total = 2 * n * c + c
    state = np.empty(total, np.uint32)
    s = 12345
    # vectorised LCG: x_{k} = a^k x0 + c (a^k - 1)/(a - 1) mod 2^32, done by plain iteration in chunks
    a, cc = 1664525, 1013904223
    out = np.empty(total, np.uint32)
    x = s
    for i in range(total):
        x = (x * a + cc) & 0xFFFFFFFF
        out[i] = x
    f = (out >> 8).astype(np.float32) / np.float32(8388608.0) - np.float32(1.0)
    import torch
    bits = torch.from_numpy(f).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    branch = bits[: n * c].reshape(n, c).copy()
    residual = bits[n * c: 2 * n * c].reshape(n, c).copy()
    weight = bits[2 * n * c:].copy()
    branch[0, :] = 0
    residual[0, :] = 0
    if n > 1:
        residual[1, 5] = 0x4370  # bf16(240.0)
    return branch, residual, weight
