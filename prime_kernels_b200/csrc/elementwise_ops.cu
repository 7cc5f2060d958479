// Forward-only CUDA replacements for the reference's Triton elementwise ops (bf16, sm_100a):
//   apply_rotary      prime_kernels/triton_rope/__init__.py:41-82,373-377
//   rmsnorm           prime_kernels/triton_rmsnorm/rmsnorm.py:43-104,701-708
//   residual_rmsnorm  prime_kernels/triton_rmsnorm/rmsnorm.py:239-297,711-722
//   swiglu            prime_kernels/triton_swiglu/swiglu.py:31-59,195-202
// Same rounding points as the reference (which follow HuggingFace): every product / sum that the
// eager model materialises in bf16 is rounded to bf16 here too.  All kernels are HBM-bound streaming
// kernels: 16-byte accesses, one row per warp (norms) or one 8-element vector per thread.
#include <cuda_runtime.h>

#include <cstdint>

#include "pk_common.cuh"

namespace pk {

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
    f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
    f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// ---- RoPE: x [rows, D] where row = (b, h, s) flattened as given by (heads, seq, head-major or seq-major);
// cos/sin [B or 1, S, rot].  y[d] = bf16( bf16(x[d] c[d]) + bf16(sign x[partner] s[d]) ) for d < rot, else x[d].
__global__ void __launch_bounds__(256) rope_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y,
                                                   const uint16_t* __restrict__ cs, const uint16_t* __restrict__ sn,
                                                   long long rows, int D, int rot, int heads, int seq, int head_major,
                                                   int cos_batch) {
    const int vpr = D >> 3;                                     // 8-element vectors per row
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * vpr) return;
    const long long row = gid / vpr;
    const int d0 = (int)(gid - row * vpr) * 8;
    // row -> (b, s): head_major: row = (b*heads + h)*seq + s; else row = (b*seq + s)*heads + h
    long long b, s;
    if (head_major) {
        s = row % seq;
        b = row / ((long long)heads * seq);
    } else {
        s = (row / heads) % seq;
        b = row / ((long long)heads * seq);
    }
    const uint16_t* xr = x + row * D;
    float xv[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + d0), xv);
    float out[8];
    if (d0 < rot) {
        const int half = rot >> 1;
        const int p0 = d0 < half ? d0 + half : d0 - half;       // partner vector (rot/2 is a multiple of 8)
        float pv[8], cv[8], sv[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + p0), pv);
        const long long crow = ((cos_batch > 1 ? b : 0) * seq + s) * rot;
        unpack8(*reinterpret_cast<const uint4*>(cs + crow + d0), cv);
        unpack8(*reinterpret_cast<const uint4*>(sn + crow + d0), sv);
        const float sign = d0 < half ? -1.f : 1.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = round_bf16(__fmul_rn(xv[i], cv[i]));
            const float bb = round_bf16(__fmul_rn(__fmul_rn(sign, pv[i]), sv[i]));
            out[i] = __fadd_rn(a, bb);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = xv[i];
    }
    *reinterpret_cast<uint4*>(y + row * D + d0) = pack8(out);
}

// ---- RMSNorm (optionally fused with the residual add): one warp per row.
//   sum = bf16(branch + residual) (if residual), rstd = rsqrt(mean(sum^2) + eps), out = bf16( w * bf16(sum * rstd) )
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ res,
                                                           const uint16_t* __restrict__ w, uint16_t* __restrict__ out,
                                                           uint16_t* __restrict__ sum_out, long long rows, int H, float eps) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const int nv = H >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + row * H) : nullptr;
    float ss = 0.f;
    for (int v = lane; v < nv; v += 32) {
        float a[8];
        unpack8(ld_stream_16(xr + v), a);
        if (rr) {
            float r8[8];
            unpack8(ld_stream_16(rr + v), r8);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = round_bf16(__fadd_rn(a[i], r8[i]));
            if (sum_out) *reinterpret_cast<uint4*>(sum_out + row * H + v * 8) = pack8(a);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(a[i], a[i], ss);
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    // second pass re-reads the row (L1/L2 resident: a row is a few KB)
    for (int v = lane; v < nv; v += 32) {
        float a[8], wv[8];
        if (rr && sum_out) {
            unpack8(*reinterpret_cast<const uint4*>(sum_out + row * H + v * 8), a);
        } else {
            unpack8(xr[v], a);
            if (rr) {
                float r8[8];
                unpack8(rr[v], r8);
#pragma unroll
                for (int i = 0; i < 8; ++i) a[i] = round_bf16(__fadd_rn(a[i], r8[i]));
            }
        }
        unpack8(__ldg(reinterpret_cast<const uint4*>(w) + v), wv);
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = __fmul_rn(wv[i], round_bf16(__fmul_rn(a[i], rstd)));
        st_stream_16(out + row * H + v * 8, pack8(o));
    }
}

// ---- SwiGLU: out = bf16( bf16(silu(gate)) * up ), silu(x) = x / (1 + exp(-x)) in fp32
__global__ void __launch_bounds__(256) swiglu_kernel(const uint16_t* __restrict__ gate, const uint16_t* __restrict__ up,
                                                     uint16_t* __restrict__ out, long long rows, int cols,
                                                     long long gate_stride, long long up_stride) {
    const int vpr = cols >> 3;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * vpr) return;
    const long long row = gid / vpr;
    const int c0 = (int)(gid - row * vpr) * 8;
    float g[8], u[8], o[8];
    unpack8(ld_stream_16(gate + row * gate_stride + c0), g);
    unpack8(ld_stream_16(up + row * up_stride + c0), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float silu = round_bf16(__fdiv_rn(g[i], 1.f + expf(-g[i])));
        o[i] = __fmul_rn(silu, u[i]);
    }
    st_stream_16(out + row * cols + c0, pack8(o));
}

}  // namespace pk

using namespace pk;

// q/k rotary embedding, one call per tensor.  x, y: bf16 [rows, D] contiguous with rows = B*heads*S laid out
// head-major ([B, heads, S, D], unsqueeze_dim 1) or sequence-major ([B, S, heads, D], unsqueeze_dim 2);
// cos, sin: bf16 [cos_batch (1 or B), S, rot].  Replaces the forward of triton_rope.apply_rotary.
extern "C" int pk_apply_rotary(const void* x, void* y, const void* cos, const void* sin, long long batch, int heads,
                               int seq, int D, int rot, int head_major, int cos_batch, void* stream) {
    if (batch < 0 || heads <= 0 || seq <= 0 || D <= 0 || (D % 8) || rot <= 0 || rot > D || (rot % 16)) return kErrShape;
    if (batch == 0) return kOk;
    if (!x || !y || !cos || !sin) return kErrNull;
    const long long rows = batch * heads * seq;
    const long long threads = rows * (D / 8);
    rope_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x), static_cast<uint16_t*>(y), static_cast<const uint16_t*>(cos),
        static_cast<const uint16_t*>(sin), rows, D, rot, heads, seq, head_major, cos_batch);
    return (int)cudaPeekAtLastError();
}

// RMSNorm forward; residual and sum_out may be null (plain rmsnorm).  Replaces the forward of
// triton_rmsnorm.rmsnorm / residual_rmsnorm.
extern "C" int pk_rmsnorm_forward(const void* x, const void* residual, const void* weight, void* out, void* sum_out,
                                  long long rows, int H, float eps, void* stream) {
    if (rows < 0 || H <= 0 || (H % 8)) return kErrShape;
    if (rows == 0) return kOk;
    if (!x || !weight || !out) return kErrNull;
    rmsnorm_rows_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(residual), static_cast<const uint16_t*>(weight),
        static_cast<uint16_t*>(out), static_cast<uint16_t*>(sum_out), rows, H, eps);
    return (int)cudaPeekAtLastError();
}

// SwiGLU forward; gate/up rows may be strided views (row strides in elements).  Replaces triton_swiglu.swiglu.
extern "C" int pk_swiglu_forward(const void* gate, const void* up, void* out, long long rows, int cols,
                                 long long gate_stride, long long up_stride, void* stream) {
    if (rows < 0 || cols <= 0 || (cols % 8) || (gate_stride % 8) || (up_stride % 8)) return kErrShape;
    if (rows == 0) return kOk;
    if (!gate || !up || !out) return kErrNull;
    const long long threads = rows * (cols / 8);
    swiglu_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(gate), static_cast<const uint16_t*>(up), static_cast<uint16_t*>(out), rows, cols,
        gate_stride, up_stride);
    return (int)cudaPeekAtLastError();
}
