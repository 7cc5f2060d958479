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
