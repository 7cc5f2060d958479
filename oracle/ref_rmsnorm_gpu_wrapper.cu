// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// C entry points around the reference project's own GPU launchers for the fused RMSNorm +
// residual + MXFP8 quantiser (prime_kernels/rmsnorm/rmsnorm.cuh: `fused_rmsnorm_residual_forward`
// and the per-variant `launch_*` functions).  The reference's kernels are compiled from the
// reference checkout where they lie and linked with this file into
// oracle/_ref/libref_rmsnorm_gpu.so (recipe: oracle/build_ref.sh); nothing is copied.
// The GPU parity tests call it on the same device buffers as the product kernel.
#include "rmsnorm.cuh"

#include <cstring>

namespace {
using Launch = void (*)(RMSNORM_LAUNCH_PARAMS);
Launch pick(const char* name) {
    if (!name || !std::strcmp(name, "auto")) return &fused_rmsnorm_residual_forward;
    if (!std::strcmp(name, "loop")) return &launch_rmsnorm_loop;
    if (!std::strcmp(name, "epi")) return &launch_rmsnorm_epi;
    if (!std::strcmp(name, "fixed_c")) return &launch_rmsnorm_fixed_c;
    if (!std::strcmp(name, "fixed_32pt")) return &launch_rmsnorm_32pt;
    if (!std::strcmp(name, "pers_32pt")) return &launch_rmsnorm_pers32;
    if (!std::strcmp(name, "tma_simple")) return &launch_rmsnorm_tma_simple;
    if (!std::strcmp(name, "tma_simple_swz")) return &launch_rmsnorm_tma_simple_swz;
    return nullptr;
}
}  // namespace

// Device pointers; N and C multiples of 128 (the reference's contract; it exits the process on other
// shapes, so the caller checks first).  Returns 0, -1 for an unknown variant, -2 for a shape the
// reference does not accept, else the cudaError_t of the launch.
extern "C" int ref_rmsnorm_gpu(const char* variant, void* vals, void* scales, float* rrms, const void* branch,
                               const void* residual, const void* weight, float epsilon, int N, int C,
                               void* stream) {
    Launch fn = pick(variant);
    if (!fn) return -1;
    if (N <= 0 || C <= 0 || N % 128 || C % 128) return -2;
    fn(static_cast<__nv_fp8_e4m3*>(vals), static_cast<__nv_fp8_e8m0*>(scales), rrms,
       static_cast<const nv_bfloat16*>(branch), static_cast<const nv_bfloat16*>(residual),
       static_cast<const nv_bfloat16*>(weight), epsilon, N, C, static_cast<cudaStream_t>(stream));
    return (int)cudaGetLastError();
}
