// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// Builds the reference project's own CPU `reference()` for the fused RMSNorm + residual +
// MXFP8 quantiser, straight from the reference checkout (prime_kernels/rmsnorm/test.cu:82-150),
// into a small shared library with a C entry point.  Nothing is copied: the reference source
// file is #included from where it lies (path given by -DREF_TEST_CU=...), its `main` is renamed
// away, and the GPU launchers its variant table names are satisfied by empty stubs because only
// the host-side reference() is ever called here.
//
// Build recipe: oracle/build_ref.sh.  Output: oracle/_ref/libref_rmsnorm.so
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#define main ref_test_main_unused
#include REF_TEST_CU
#undef main

// Stubs for the GPU launchers referenced by the reference's variant table (never called).
#define PK_STUB(name) void name(RMSNORM_LAUNCH_PARAMS) {}
PK_STUB(launch_rmsnorm_loop)
PK_STUB(launch_rmsnorm_epi)
PK_STUB(launch_rmsnorm_fixed_c)
PK_STUB(launch_rmsnorm_32pt)
PK_STUB(launch_rmsnorm_pers32)
PK_STUB(launch_rmsnorm_tma_simple)
PK_STUB(launch_rmsnorm_tma_simple_swz)
int rmsnorm_tma_simple_max_c() { return 0; }

// math: 0 = bf16 scale math, 1 = fp32 scale math (prime_kernels/rmsnorm/test.cu:71-74).
// `s` is the per-row reciprocal RMS the quantiser is driven with (test.cu:105-106).
// scales must hold (N/128)*(C/128)*512 bytes; N and C multiples of 128 (reference contract).
extern "C" int ref_rmsnorm_mxfp8(const uint16_t* branch, const uint16_t* residual,
                                 const uint16_t* weight, const float* s, float epsilon, int N,
                                 int C, int math, int group_size, uint8_t* vals, uint8_t* scales,
                                 double* rrms) {
    std::vector<nv_bfloat16> b((size_t)N * C), r((size_t)N * C), w(C);
    std::memcpy(b.data(), branch, b.size() * 2);
    std::memcpy(r.data(), residual, r.size() * 2);
    std::memcpy(w.data(), weight, w.size() * 2);
    std::vector<float> sv(s, s + N);
    RefResult out = reference(b, r, w, sv, epsilon, N, C,
                              math ? ScaleMath::Fp32 : ScaleMath::Bf16, group_size);
    std::memcpy(vals, out.vals.data(), out.vals.size());
    std::memcpy(scales, out.scales.data(), out.scales.size());
    std::memcpy(rrms, out.rrms.data(), out.rrms.size() * sizeof(double));
    return 0;
}

// Element-level probes of the CUDA host conversion intrinsics the reference oracle uses, so
// the plain-C restatement can be pinned exhaustively (all 65536 bf16 patterns, float sweeps).
extern "C" uint8_t ref_bf16_to_e4m3(uint16_t bits) {
    __nv_bfloat16_raw raw; raw.x = bits;
    return __nv_cvt_bfloat16raw_to_fp8(raw, __NV_SATFINITE, __NV_E4M3);
}
extern "C" uint8_t ref_float_to_e8m0_rp(float x) {
    return __nv_cvt_float_to_e8m0(x, __NV_SATFINITE, cudaRoundPosInf);
}
extern "C" uint16_t ref_e8m0_to_bf16(uint8_t e) {
    return __nv_cvt_e8m0_to_bf16raw(e).x;
}
extern "C" uint16_t ref_float_to_bf16(float x) {
    return __nv_bfloat16_raw(__float2bfloat16(x)).x;
}
extern "C" long long ref_sf_offset_c(int m, int k, int num_k_tiles) { return ref_sf_offset(m, k, num_k_tiles); }
