"""CPU: pins the plain-C MXFP8 oracle (oracle/mxfp8_oracle.c) against the reference project's own CPU
reference (oracle/_ref, when built) and against the committed golden digests produced by it."""
import hashlib
import json
import struct
from pathlib import Path

import numpy as np
import pytest

from oracle import mxfp8

GOLDEN = json.loads((Path(__file__).parent / "golden" / "mxfp8_reference.json").read_text())
needs_ref = pytest.mark.skipif(not mxfp8.ref_available(), reason="oracle/_ref not built (no reference checkout)")


def _f(u):
    return struct.unpack("f", struct.pack("I", u))[0]


@needs_ref
def test_e4m3_conversion_exhaustive_against_reference_intrinsic():
    p, r = mxfp8.port(), mxfp8.ref()
    assert all(p.pk_bf16_to_e4m3(b) == r.ref_bf16_to_e4m3(b) for b in range(65536))


@needs_ref
def test_e8m0_and_bf16_helpers_against_reference_intrinsics():
    p, r = mxfp8.port(), mxfp8.ref()
    assert all(p.pk_e8m0_to_bf16(e) == r.ref_e8m0_to_bf16(e) for e in range(256))
    for hi in range(0, 0x8000, 3):
        for lo in (0, 1, 0x7FFF, 0x8000, 0x8001, 0xFFFF):
            x = _f((hi << 16) | lo)
            if x != x:
                continue
            assert p.pk_float_to_e8m0_rp(x) == r.ref_float_to_e8m0_rp(x)
            assert p.pk_float_to_bf16(x) == r.ref_float_to_bf16(x)


@needs_ref
def test_scale_offsets_against_reference_layout():
    p, r = mxfp8.port(), mxfp8.ref()
    for nkt in (1, 4, 32):
        for m in list(range(0, 260, 7)) + [127, 128, 255]:
            for k in range(0, nkt * 4):
                assert p.pk_sf_offset(m, k, nkt) == r.ref_sf_offset_c(m, k, nkt)


def test_known_answers():
    p = mxfp8.port()
    assert p.pk_float_to_e8m0_rp(0.0) == 0                   # all-zero group -> scale byte 0
    assert p.pk_float_to_e8m0_rp(3.7 / 448.0) == 121         # ceil(log2(3.7/448)) = -6 -> 121
    assert p.pk_bf16_to_float(p.pk_e8m0_to_bf16(254 - 121)) == 64.0
    assert p.pk_bf16_to_e4m3(0x43E0) == 0x7E                 # 448 -> max finite
    assert p.pk_bf16_to_e4m3(0x4400) == 0x7E                 # 512 saturates
    assert p.pk_bf16_to_e4m3(0x0000) == 0x00 and p.pk_bf16_to_e4m3(0x8000) == 0x80
    assert p.pk_scale_bytes(1, 960) == 8 * 512 and p.pk_scale_bytes(130, 128) == 2 * 512


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=lambda c: f"{c['n']}x{c['c']}")
def test_quantiser_matches_committed_reference_digests(case):
    n, c = case["n"], case["c"]
    if n * c > 256 * 2048:
        pytest.skip("kept for the reference-library comparison below; LCG generation is slow in Python")
    b, r, w = mxfp8.lcg_inputs(n, c)
    _, _, rr, _ = mxfp8.quantise_port(b, r, w, None, GOLDEN["eps"])
    vals, scales, _, _ = mxfp8.quantise_port(b, r, w, rr.astype(np.float32), GOLDEN["eps"])
    assert hashlib.sha256(vals.tobytes()).hexdigest() == case["vals_sha256"]
    assert hashlib.sha256(scales.tobytes()).hexdigest() == case["scales_sha256"]
    assert vals[1, :64].tolist() == case["vals_row1_head"]
    assert (vals[0] == 0).all()                               # zero row: zero bytes, zero scales
    assert int(scales[mxfp8.port().pk_sf_offset(1, 0, c // 128)]) == case["row1_group0_scale"]


@needs_ref
@pytest.mark.parametrize("n,c", [(128, 128), (128, 512), (256, 1024)])
def test_quantiser_against_reference_library(n, c):
    rng = np.random.default_rng(n + c)
    import torch

    def bits(a):
        return torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)

    b, r = bits(rng.standard_normal((n, c))), bits(rng.standard_normal((n, c)))
    w = bits(1 + 0.1 * rng.standard_normal(c))
    b[0] = 0
    r[0] = 0
    r[1, 5] = 0x4370
    _, _, rr, _ = mxfp8.quantise_port(b, r, w, None, 1e-6)
    s = rr.astype(np.float32)
    v1, s1, r1, _ = mxfp8.quantise_port(b, r, w, s, 1e-6)
    v2, s2, r2 = mxfp8.quantise_ref(b, r, w, s, 1e-6, 1)
    assert (v1 == v2).all() and (s1 == s2).all() and np.allclose(r1, r2, rtol=1e-12)


def test_ragged_shapes_define_padding_as_zero():
    rng = np.random.default_rng(0)
    import torch

    n, c = 5, 960
    x = torch.from_numpy(rng.standard_normal((n, c)).astype(np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    w = torch.ones(c, dtype=torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    vals, scales, _, res = mxfp8.quantise_port(x, x, w, None, 1e-6, want_res=True)
    assert scales.size == 8 * 512
    tiles = scales.reshape(8, 32, 4, 4)            # [k_tile, m%32, (m/32)%4, k%4]
    assert (tiles[:, 5:, :, :] == 0).all() and (tiles[:, :, 1:, :] == 0).all()   # rows >= 5
    assert (tiles[7, :, :, 2:] == 0).all()          # 960/32 = 30 groups: k = 30, 31 are padding
    assert (tiles[:7, :5, 0, :] != 0).all()
    # mode 1 returns the bf16 sum as the updated residual
    _, _, _, res1 = mxfp8.quantise_port(x, x, w, None, 1e-6, mode=1, want_res=True)
    a = torch.from_numpy(x.view(np.int16)).view(torch.bfloat16).float()
    assert (torch.from_numpy(res1.view(np.int16)).view(torch.bfloat16).float() == (a + a).to(torch.bfloat16).float()).all()


def test_floor_scale_rule_known_answers_and_fp32_conversion():
    """The floor rule (flash_moe's block scale): e = clamp(biased_exponent(amax) - 8, 0, 254), values from fp32 with
    finite saturation.  Known answers, and the fp32 -> e4m3 conversion against PyTorch's own for in-range values."""
    import torch

    lib = mxfp8.port()
    # fp32 -> e4m3 against torch (round to nearest even; torch does not saturate, so stay within +-448)
    g = np.random.default_rng(7)
    xs = np.concatenate([g.uniform(-448, 448, 4000), g.uniform(-1, 1, 4000), g.uniform(-2 ** -6, 2 ** -6, 2000),
                         np.array([0.0, 2 ** -9, 2 ** -10, 3 * 2 ** -11, 448.0, -448.0, 256.0, 17.0, 18.0, 19.0, 1.0625])]).astype(np.float32)
    want = torch.from_numpy(xs).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([lib.pk_float_to_e4m3(float(x)) for x in xs], dtype=np.uint8)
    assert np.array_equal(got & 0x7f, want & 0x7f) and np.array_equal((got >> 7)[xs != 0], (want >> 7)[xs != 0])
    assert lib.pk_float_to_e4m3(486.0) == 0x7e and lib.pk_float_to_e4m3(-1e9) == 0xfe       # saturation
    # one group with amax 1.0: biased exponent 127 -> e = 119 (scale 2^-8); 1.0 -> 256 = 0x78; 1.9 -> 486.4 -> saturates
    w = np.zeros((1, 32), np.float32)
    w[0, 0], w[0, 1], w[0, 2] = 1.0, -0.5, 2.0 ** -9
    bits = torch.from_numpy(w).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    vals, scales = mxfp8.quantise_weight(bits, scale_mode="floor")
    assert scales[0, 0] == 119 and vals[0, 0] == 0x78 and vals[0, 1] == (0x80 | 0x70) and vals[0, 2] == 0x30   # 0.5 -> 128, 2^-9 -> 0.5
    w[0, 0] = 1.9
    bits = torch.from_numpy(w).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    vals, scales = mxfp8.quantise_weight(bits, scale_mode="floor")
    assert scales[0, 0] == 119 and vals[0, 0] == 0x7e          # 1.9 * 256 = 486 > 464: saturated at 448
    # the round-up rule on the same group never saturates: scale 2^-7 (sf 120), 1.9 * 128 = 243 -> 240
    vals2, scales2 = mxfp8.quantise_weight(bits, scale_mode="roundup")
    assert scales2[0, 0] == 120 and vals2[0, 0] == 0x77
    # all-zero group: e = clamp(0 - 8) = 0, values 0
    z = np.zeros((1, 32), np.uint16)
    vals, scales = mxfp8.quantise_weight(z, scale_mode="floor")
    assert scales[0, 0] == 0 and not vals.any()
