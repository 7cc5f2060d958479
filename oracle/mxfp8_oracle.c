/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's fused
 * RMSNorm + post-norm residual + MXFP8 quantiser, in plain C with integer bit arithmetic
 * (no CUDA headers).  Only tests, the smoke check and the benchmark's CPU-baseline leg may
 * load this; the product library never does.
 *
 * Follows, by reference file:line (paths inside the reference project):
 *   prime_kernels/rmsnorm/test.cu:82-150        reference(): per-row maths and rounding points
 *   prime_kernels/rmsnorm/test.cu:57-65         ref_sf_offset(): blocked 128x4 scale layout
 *   prime_kernels/rmsnorm/src/kernels/rmsnorm_03_fixed_32pt.cu:67-98   the same maths on device
 * The conversion helpers restate the documented behaviour of CUDA's
 * __float2bfloat16 (round-nearest-even), __nv_cvt_float_to_e8m0(SATFINITE, RoundPosInf),
 * __nv_cvt_e8m0_to_bf16raw and __nv_cvt_bfloat16raw_to_fp8(SATFINITE, E4M3).
 *
 * Pinning: tests/test_oracle_mxfp8.py checks every helper exhaustively (all 65536 bf16
 * patterns; float sweeps) and the whole quantiser on the reference test's shapes and its
 * known-answer rows against oracle/_ref (the reference's own reference() compiled from the
 * reference checkout), and against committed golden fixtures produced by that library.
 *
 * Extensions beyond the reference (which requires N % 128 == 0 and C % 128 == 0):
 *   - ragged N and C % 32 == 0: the scale buffer covers ceil(N/128) x ceil(C/128) tiles and
 *     every byte no (row, 32-group) maps to is 0;
 *   - mode 1 ("prenorm add"): sum = bf16(branch + residual), norm over sum, out = bf16(s*(sum*w));
 *   - optional bf16 copy of the pre-quantisation value (the "updated residual").
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

float pk_bf16_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }

/* fp32 -> bf16, round to nearest even; NaN -> 0x7FFF (CUDA's canonical bf16 NaN). */
uint16_t pk_float_to_bf16(float f) {
    uint32_t u = f2u(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
    uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;
    return (uint16_t)(u >> 16);
}

/* fp32 -> E8M0 (biased power-of-two exponent), magnitude rounded toward +inf, finite saturation. */
uint8_t pk_float_to_e8m0_rp(float x) {
    uint32_t u = f2u(x) & 0x7fffffffu;
    if (u > 0x7f800000u) return 0xff;            /* NaN */
    /* the CUDA host path first rounds |x| up to bf16 (8 exponent + 7 mantissa bits) */
    uint32_t b = u >> 16;
    if (u & 0xffffu) b += 1;                     /* round up toward +inf (may carry into exponent) */
    if (b >= 0x7f80u) return 0xfe;               /* inf / overflow -> largest finite */
    uint32_t e = b >> 7, m = b & 0x7fu;
    if (e == 0) {                                /* bf16 subnormal: value = m * 2^-133 */
        return (m > 0x40u) ? 1 : 0;              /* > 2^-127 rounds up to 2^-126, else 2^-127 */
    }
    if (m) e += 1;
    return (uint8_t)(e > 0xfe ? 0xfe : e);
}

/* E8M0 -> bf16 bit pattern of 2^(e-127). */
uint16_t pk_e8m0_to_bf16(uint8_t e) {
    if (e == 0xff) return 0x7fff;
    if (e == 0) return 0x0040;                   /* 2^-127 is a bf16 subnormal */
    return (uint16_t)((uint16_t)e << 7);
}

/* |value| (finite, fp32) -> FP8 E4M3 magnitude bits, round-nearest-even, finite saturation. */
static uint8_t pk_mag_to_e4m3(float a, uint8_t sign);

/* fp32 -> FP8 E4M3 (fn), round-nearest-even, finite saturation: what cvt.rn.satfinite.e4m3x2.f32 /
 * __nv_cvt_float2_to_fp8x2(.., __NV_SATFINITE, __NV_E4M3) do to one value. */
uint8_t pk_float_to_e4m3(float f) {
    uint32_t u = f2u(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    uint32_t mag = u & 0x7fffffffu;
    if (mag > 0x7f800000u) return 0x7f;                       /* NaN: canonical, sign dropped */
    if (mag == 0x7f800000u) return (uint8_t)(sign | 0x7e);    /* inf -> largest finite */
    return pk_mag_to_e4m3(u2f(mag), sign);
}

/* bf16 -> FP8 E4M3 (fn: no inf, max 448), round-nearest-even, finite saturation. */
uint8_t pk_bf16_to_e4m3(uint16_t b) {
    uint8_t sign = (uint8_t)((b >> 8) & 0x80);
    uint32_t mag = b & 0x7fffu;
    if (mag > 0x7f80u) return 0x7f;                           /* NaN: canonical, sign dropped */
    if (mag >= 0x7f80u) return (uint8_t)(sign | 0x7e);
    return pk_mag_to_e4m3(pk_bf16_to_float((uint16_t)mag), sign);
}

static uint8_t pk_mag_to_e4m3(float a, uint8_t sign) {
    if (a >= 464.0f) return (uint8_t)(sign | 0x7e);           /* >= halfway past 448 -> sat 448 */
    if (a < 0.0009765625f) return sign;                       /* < 2^-10: below half the min subnormal */
    /* scale so that one e4m3 ulp at this magnitude becomes 1.0, then round to nearest even */
    int e;
    (void)frexpf(a, &e);                                      /* a = f * 2^e, f in [0.5,1) */
    int exp = e - 1;                                          /* floor(log2 a) */
    if (exp < -6) exp = -6;                                   /* subnormal range: ulp 2^-9 */
    float ulp = ldexpf(1.0f, exp - 3);
    float q = a / ulp;                                        /* exact: power-of-two scaling */
    float r = nearbyintf(q);                                  /* default rounding mode: nearest even */
    float v = r * ulp;
    if (v > 448.0f) return (uint8_t)(sign | 0x7e);
    if (v == 0.0f) return sign;
    (void)frexpf(v, &e);
    exp = e - 1;
    uint8_t bits;
    if (exp < -6) {
        bits = (uint8_t)(v / ldexpf(1.0f, -9));               /* subnormal: mantissa only */
    } else {
        uint32_t mant = (uint32_t)(v / ldexpf(1.0f, exp - 3)) - 8u;
        bits = (uint8_t)(((uint32_t)(exp + 7) << 3) | mant);
    }
    return (uint8_t)(sign | bits);
}

/* Blocked scale layout [numMTiles, numKTiles, 32, 4, 4]; num_k_tiles = ceil(C/128). */
int64_t pk_sf_offset(int m, int k, int num_k_tiles) {
    int m_tile = m / 128, outer_m = m % 32, inner_m = (m / 32) % 4;
    int k_tile = k / 4, inner_k = k % 4;
    return ((int64_t)m_tile * num_k_tiles + k_tile) * 512 + outer_m * 16 + inner_m * 4 + inner_k;
}

int64_t pk_scale_bytes(int N, int C) {
    return (int64_t)((N + 127) / 128) * ((C + 127) / 128) * 512;
}

/*
 * s: per-row reciprocal RMS driving the quantiser (the kernel's own rrms output, as in the
 *    reference test), or NULL to use float(1/sqrt(mean_double + eps)).
 * mode 0: res = bf16( s*(branch*w) + residual )       (reference semantics)
 * mode 1: sum = bf16(branch + residual); res = bf16( s*(sum*w) ); norm statistics over sum
 * res_out: optional [N*C] bf16 -- mode 0: res; mode 1: sum.
 * rrms_ref: optional [N] double-precision 1/sqrt(mean(x^2) + eps).
 */
int pk_oracle_rmsnorm_mxfp8(const uint16_t* branch, const uint16_t* residual,
                            const uint16_t* weight, const float* s, float eps, int N, int C,
                            int mode, uint8_t* vals, uint8_t* scales, double* rrms_ref,
                            uint16_t* res_out) {
    if (C % 32 != 0 || N < 0 || C <= 0) return 1;
    const int nkt = (C + 127) / 128;
    memset(scales, 0, (size_t)pk_scale_bytes(N, C));
    uint16_t res[32];
    for (int row = 0; row < N; ++row) {
        const uint16_t* br = branch + (size_t)row * C;
        const uint16_t* rr = residual + (size_t)row * C;
        double ss = 0.0;
        for (int c = 0; c < C; ++c) {
            double v = mode ? (double)pk_bf16_to_float(pk_float_to_bf16(
                                  pk_bf16_to_float(br[c]) + pk_bf16_to_float(rr[c])))
                            : (double)pk_bf16_to_float(br[c]);
            ss += v * v;
        }
        const double rr_d = 1.0 / sqrt(ss / C + (double)eps);
        if (rrms_ref) rrms_ref[row] = rr_d;
        const float sv = s ? s[row] : (float)rr_d;
        for (int g = 0; g < C; g += 32) {
            float amax = 0.f;
            for (int k = 0; k < 32; ++k) {
                const int c = g + k;
                const float wv = pk_bf16_to_float(weight[c]);
                uint16_t out;
                if (mode) {
                    const uint16_t sum = pk_float_to_bf16(pk_bf16_to_float(br[c]) + pk_bf16_to_float(rr[c]));
                    const float prod = pk_bf16_to_float(sum) * wv;   /* exact in fp32 */
                    out = pk_float_to_bf16(sv * prod);
                    if (res_out) res_out[(size_t)row * C + c] = sum;
                } else {
                    const float prod = pk_bf16_to_float(br[c]) * wv; /* exact in fp32 */
                    const float nw = sv * prod;                      /* one fp32 rounding, no FMA */
                    out = pk_float_to_bf16(nw + pk_bf16_to_float(rr[c]));
                    if (res_out) res_out[(size_t)row * C + c] = out;
                }
                res[k] = out;
                const float a = fabsf(pk_bf16_to_float(out));
                amax = fmaxf(amax, a);
            }
            const float scale_factor = amax * (1.f / 448.f);
            const uint8_t sf = pk_float_to_e8m0_rp(scale_factor);
            const float inv = pk_bf16_to_float(pk_e8m0_to_bf16((uint8_t)(254 - sf)));
            for (int k = 0; k < 32; ++k) {
                const uint16_t scaled = pk_float_to_bf16(pk_bf16_to_float(res[k]) * inv);
                vals[(size_t)row * C + g + k] = pk_bf16_to_e4m3(scaled);
            }
            scales[pk_sf_offset(row, g / 32, nkt)] = sf;
        }
    }
    return 0;
}

/*
 * Weight quantiser used for the MXFP8 decode configuration: the same per-32 recipe applied
 * along K of a row-major [rows, K] bf16 matrix (scale = 2^ceil(log2(amax/448)), values
 * bf16(w * 2^-scale) -> e4m3).  Scales are written row-major [rows, K/32] (not blocked).
 */
int pk_oracle_quantise_weight(const uint16_t* w, int64_t rows, int K, uint8_t* vals, uint8_t* scales) {
    if (K % 32) return 1;
    for (int64_t r = 0; r < rows; ++r) {
        for (int g = 0; g < K; g += 32) {
            float amax = 0.f;
            for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(pk_bf16_to_float(w[r * K + g + k])));
            const uint8_t sf = pk_float_to_e8m0_rp(amax * (1.f / 448.f));
            const float inv = pk_bf16_to_float(pk_e8m0_to_bf16((uint8_t)(254 - sf)));
            for (int k = 0; k < 32; ++k)
                vals[r * K + g + k] = pk_bf16_to_e4m3(pk_float_to_bf16(pk_bf16_to_float(w[r * K + g + k]) * inv));
            scales[r * (K / 32) + g / 32] = sf;
        }
    }
    return 0;
}

/*
 * Second weight recipe ("floor"): the block-scale rule of the reference's flash_moe kernels
 * (prime_kernels/flash_moe/csrc/kernels/fused_moe_mxfp8_kernel.cu:4-20, mx_block_scale + store_fp8x16):
 * e = clamp(biased_exponent(amax) - 8, 0, 254), i.e. scale 2^(floor(log2 amax) - 8); values w * 2^(127 - e)
 * converted from fp32 with round-to-nearest-even and finite saturation (a block's largest values may saturate
 * at 448).  Same packed format as the round-up recipe.
 */
int pk_oracle_quantise_weight_floor(const uint16_t* w, int64_t rows, int K, uint8_t* vals, uint8_t* scales) {
    if (K % 32) return 1;
    for (int64_t r = 0; r < rows; ++r) {
        for (int g = 0; g < K; g += 32) {
            float amax = 0.f;
            for (int k = 0; k < 32; ++k) amax = fmaxf(amax, fabsf(pk_bf16_to_float(w[r * K + g + k])));
            int e = (int)((f2u(amax) >> 23) & 0xffu) - 8;
            e = e < 0 ? 0 : (e > 254 ? 254 : e);
            const float inv = u2f((uint32_t)(254 - e) << 23);
            for (int k = 0; k < 32; ++k)
                vals[r * K + g + k] = pk_float_to_e4m3(pk_bf16_to_float(w[r * K + g + k]) * inv);
            scales[r * (K / 32) + g / 32] = (uint8_t)e;
        }
    }
    return 0;
}
