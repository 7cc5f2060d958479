// TEST INFRASTRUCTURE ONLY (never linked into the product library).
//
// Builds one of the reference project's own decode megakernels (SmolLM2-135M:
// prime_kernels/decode_megakernel/csrc/megakernel.cu; SmolLM2-360M:
// prime_kernels/decode_megakernel_360m/csrc/block360.cu with block360_kernel.inc) for sm_100a, straight from the reference checkout: the
// source file is #included from where it lies (path given by -DREF_MEGAKERNEL_CU=...), nothing is copied
// or edited.  The reference entries refuse every device that is not sm_89 (megakernel.cu:873,
// block360_kernel.inc:884); its kernel
// itself is plain CUDA C++ (cooperative launch of 24 CTAs, cooperative-groups grid.sync between phases in
// the default build), so the only change needed to run it on a B200 is what its capability query reports.
// That query is redirected, for this translation unit only, to a shim that returns the real properties with
// the compute capability reported as 8.9.  The exported C symbols (mk_query, mk_workspace_bytes, mk_decode,
// mk_status_string) are the reference's own.
//
// Used by the GPU parity tests as a second decode oracle (the reference's own kernel on the same device
// buffers) and for a same-box timing of the reference design.  Build recipe: oracle/build_ref.sh.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#include <mma.h>

#include <cfloat>   // FLT_MAX, which the 360M source uses without including it

static inline cudaError_t pk_ref_device_properties(cudaDeviceProp* prop, int device) {
    cudaError_t e = cudaGetDeviceProperties(prop, device);
    if (e == cudaSuccess) {
        prop->major = 8;
        prop->minor = 9;
    }
    return e;
}
#undef cudaGetDeviceProperties
#define cudaGetDeviceProperties pk_ref_device_properties
#include REF_MEGAKERNEL_CU
