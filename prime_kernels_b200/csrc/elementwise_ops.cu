// CUDA replacements for the reference's Triton elementwise ops (bf16, sm_100a), forward and backward:
//   apply_rotary      prime_kernels/triton_rope/__init__.py:41-82,373-377       backward :85-123
//   rmsnorm           prime_kernels/triton_rmsnorm/rmsnorm.py:43-104,701-708    backward :107-193, 459-476
//   residual_rmsnorm  prime_kernels/triton_rmsnorm/rmsnorm.py:239-297,711-722   backward :300-392
//   swiglu            prime_kernels/triton_swiglu/swiglu.py:31-59,195-202       backward :62-97
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

// ---- RoPE backward: gx[d] = bf16( bf16(g[d] c[d]) + sign bf16(g[partner] s[partner]) ), sign = +1 for d < rot/2
__global__ void __launch_bounds__(256) rope_bwd_kernel(const uint16_t* __restrict__ g, uint16_t* __restrict__ gx,
                                                       const uint16_t* __restrict__ cs, const uint16_t* __restrict__ sn,
                                                       long long rows, int D, int rot, int heads, int seq, int head_major,
                                                       int cos_batch) {
    const int vpr = D >> 3;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * vpr) return;
    const long long row = gid / vpr;
    const int d0 = (int)(gid - row * vpr) * 8;
    long long b, s;
    if (head_major) {
        s = row % seq;
        b = row / ((long long)heads * seq);
    } else {
        s = (row / heads) % seq;
        b = row / ((long long)heads * seq);
    }
    const uint16_t* gr = g + row * D;
    float gv[8], out[8];
    unpack8(*reinterpret_cast<const uint4*>(gr + d0), gv);
    if (d0 < rot) {
        const int half = rot >> 1;
        const int p0 = d0 < half ? d0 + half : d0 - half;
        float pv[8], cv[8], sv[8];
        unpack8(*reinterpret_cast<const uint4*>(gr + p0), pv);
        const long long crow = ((cos_batch > 1 ? b : 0) * seq + s) * rot;
        unpack8(*reinterpret_cast<const uint4*>(cs + crow + d0), cv);
        unpack8(*reinterpret_cast<const uint4*>(sn + crow + p0), sv);
        const float sign = d0 < half ? 1.f : -1.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float a = round_bf16(__fmul_rn(gv[i], cv[i]));
            const float bb = __fmul_rn(round_bf16(__fmul_rn(pv[i], sv[i])), sign);
            out[i] = __fadd_rn(a, bb);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = gv[i];
    }
    *reinterpret_cast<uint4*>(gx + row * D + d0) = pack8(out);
}

// ---- SwiGLU backward: d_up = bf16(grad * bf16(silu(gate))); d_gate = bf16( bf16(grad * up) * sig * (1 + gate (1 - sig)) )
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint16_t* __restrict__ grad, const uint16_t* __restrict__ gate,
                                                         const uint16_t* __restrict__ up, uint16_t* __restrict__ d_gate,
                                                         uint16_t* __restrict__ d_up, long long rows, int cols,
                                                         long long gate_stride, long long up_stride) {
    const int vpr = cols >> 3;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= rows * vpr) return;
    const long long row = gid / vpr;
    const int c0 = (int)(gid - row * vpr) * 8;
    float gr[8], g[8], u[8], dg[8], du[8];
    unpack8(ld_stream_16(grad + row * cols + c0), gr);
    unpack8(ld_stream_16(gate + row * gate_stride + c0), g);
    unpack8(ld_stream_16(up + row * up_stride + c0), u);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float e = expf(-g[i]);
        const float silu = round_bf16(__fdiv_rn(g[i], 1.f + e));
        du[i] = __fmul_rn(gr[i], silu);
        const float d_silu = round_bf16(__fmul_rn(gr[i], u[i]));
        const float sig = __fdiv_rn(1.f, 1.f + e);
        dg[i] = d_silu * sig * (1.f + g[i] * (1.f - sig));
    }
    st_stream_16(d_gate + row * cols + c0, pack8(dg));
    st_stream_16(d_up + row * cols + c0, pack8(du));
}

// ---- RMSNorm backward (x is the normed input: the sum for the residual variant).  A block owns groups of 8 rows
// (group index strided by the grid).  Per group: one warp per row computes rstd, dot = sum bf16(g w) x and
//   dx = bf16( bf16(g w) rstd + (-0.5 dot rstd^3 / H) 2x )          (+ grad_sum, rounded again, when given);
// then the 256 threads walk the columns and add the group's bf16(g bf16(x rstd)) into per-thread fp32 sums of the
// weight gradient (rows in a fixed order).  The block writes one partial row; rmsnorm_dw_reduce_kernel adds the
// partial rows in a fixed order, so the result does not depend on scheduling.
constexpr int kBwdMaxVec = 4;      // 8-element column vectors per thread: H <= 8 * 256 * 4 = 8192
__global__ void __launch_bounds__(256) rmsnorm_bwd_kernel(const uint16_t* __restrict__ go, const uint16_t* __restrict__ gsum,
                                                          const uint16_t* __restrict__ x, const uint16_t* __restrict__ w,
                                                          uint16_t* __restrict__ dx, float* __restrict__ dw_part,
                                                          long long rows, int H, float eps) {
    __shared__ float rstd_s[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nv = H >> 3;
    const float inv_h = 1.f / (float)H;
    float dw[kBwdMaxVec][8];
#pragma unroll
    for (int k = 0; k < kBwdMaxVec; ++k)
#pragma unroll
        for (int i = 0; i < 8; ++i) dw[k][i] = 0.f;
    const long long groups = (rows + 7) / 8;
    for (long long grp = blockIdx.x; grp < groups; grp += gridDim.x) {
        const long long row = grp * 8 + warp;
        if (row < rows) {
            const uint4* xr = reinterpret_cast<const uint4*>(x + row * H);
            const uint4* gr = reinterpret_cast<const uint4*>(go + row * H);
            float ss = 0.f, dot = 0.f;
            for (int v = lane; v < nv; v += 32) {
                float a[8], g8[8], wv[8];
                unpack8(xr[v], a);
                unpack8(gr[v], g8);
                unpack8(__ldg(reinterpret_cast<const uint4*>(w) + v), wv);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    ss = fmaf(a[i], a[i], ss);
                    dot = __fadd_rn(dot, __fmul_rn(round_bf16(__fmul_rn(g8[i], wv[i])), a[i]));
                }
            }
            ss = warp_sum(ss);
            dot = warp_sum(dot);
            const float rstd = rsqrtf(ss * inv_h + eps);
            if (lane == 0) rstd_s[warp] = rstd;
            const float grad_mean = __fmul_rn(__fmul_rn(__fmul_rn(-0.5f, dot), __fmul_rn(__fmul_rn(rstd, rstd), rstd)), inv_h);
            for (int v = lane; v < nv; v += 32) {
                float a[8], g8[8], wv[8], o[8];
                unpack8(xr[v], a);
                unpack8(gr[v], g8);
                unpack8(__ldg(reinterpret_cast<const uint4*>(w) + v), wv);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float dn = round_bf16(__fmul_rn(g8[i], wv[i]));
                    o[i] = __fadd_rn(__fmul_rn(dn, rstd), __fmul_rn(grad_mean, __fmul_rn(2.f, a[i])));
                }
                if (gsum) {
                    float s8[8];
                    unpack8(ld_stream_16(gsum + row * H + v * 8), s8);
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = __fadd_rn(round_bf16(o[i]), s8[i]);
                }
                st_stream_16(dx + row * H + v * 8, pack8(o));
            }
        }
        __syncthreads();
        const int nr = (int)((rows - grp * 8) < 8 ? (rows - grp * 8) : 8);
#pragma unroll
        for (int k = 0; k < kBwdMaxVec; ++k) {
            const int v = threadIdx.x + k * 256;
            if (v < nv) {
                for (int r = 0; r < nr; ++r) {
                    const long long rr = grp * 8 + r;
                    float a[8], g8[8];
                    unpack8(*(reinterpret_cast<const uint4*>(x + rr * H) + v), a);
                    unpack8(*(reinterpret_cast<const uint4*>(go + rr * H) + v), g8);
                    const float rstd = rstd_s[r];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        dw[k][i] = __fadd_rn(dw[k][i], round_bf16(__fmul_rn(g8[i], round_bf16(__fmul_rn(a[i], rstd)))));
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < kBwdMaxVec; ++k) {
        const int v = threadIdx.x + k * 256;
        if (v < nv) {
            float* dst = dw_part + (size_t)blockIdx.x * H + v * 8;
            *reinterpret_cast<float4*>(dst) = make_float4(dw[k][0], dw[k][1], dw[k][2], dw[k][3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(dw[k][4], dw[k][5], dw[k][6], dw[k][7]);
        }
    }
}
__global__ void __launch_bounds__(256) rmsnorm_dw_reduce_kernel(const float* __restrict__ dw_part, uint16_t* __restrict__ dw,
                                                                int parts, int H) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= H) return;
    float acc = 0.f;
    for (int p = 0; p < parts; ++p) acc = __fadd_rn(acc, dw_part[(size_t)p * H + c]);
    dw[c] = (uint16_t)f32_to_bf16_bits(acc);
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

// Backward of pk_apply_rotary for one tensor: g, gx bf16 [rows, D] in the layout of the forward's output.
extern "C" int pk_apply_rotary_backward(const void* g, void* gx, const void* cos, const void* sin, long long batch, int heads,
                                        int seq, int D, int rot, int head_major, int cos_batch, void* stream) {
    if (batch < 0 || heads <= 0 || seq <= 0 || D <= 0 || (D % 8) || rot <= 0 || rot > D || (rot % 16)) return kErrShape;
    if (batch == 0) return kOk;
    if (!g || !gx || !cos || !sin) return kErrNull;
    const long long rows = batch * heads * seq;
    const long long threads = rows * (D / 8);
    rope_bwd_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(g), static_cast<uint16_t*>(gx), static_cast<const uint16_t*>(cos),
        static_cast<const uint16_t*>(sin), rows, D, rot, heads, seq, head_major, cos_batch);
    return (int)cudaPeekAtLastError();
}

// Backward of pk_swiglu_forward: grad, d_gate, d_up contiguous [rows, cols]; gate / up rows may be strided.
extern "C" int pk_swiglu_backward(const void* grad, const void* gate, const void* up, void* d_gate, void* d_up, long long rows,
                                  int cols, long long gate_stride, long long up_stride, void* stream) {
    if (rows < 0 || cols <= 0 || (cols % 8) || (gate_stride % 8) || (up_stride % 8)) return kErrShape;
    if (rows == 0) return kOk;
    if (!grad || !gate || !up || !d_gate || !d_up) return kErrNull;
    const long long threads = rows * (cols / 8);
    swiglu_bwd_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(grad), static_cast<const uint16_t*>(gate), static_cast<const uint16_t*>(up),
        static_cast<uint16_t*>(d_gate), static_cast<uint16_t*>(d_up), rows, cols, gate_stride, up_stride);
    return (int)cudaPeekAtLastError();
}

// Partial rows of the weight gradient pk_rmsnorm_backward needs in `dw_partials` (fp32 [parts][H]).
extern "C" int pk_rmsnorm_backward_parts(long long rows) {
    const long long groups = (rows + 7) / 8;
    return (int)(groups < 1 ? 1 : (groups > 592 ? 592 : groups));
}

// Backward of pk_rmsnorm_forward.  x: the normed input (the sum for the residual variant); grad_sum: gradient that
// arrives through the returned sum (null for plain rmsnorm); dx: gradient of x (= of branch and of residual);
// dw: bf16 [H]; dw_partials: fp32 scratch [pk_rmsnorm_backward_parts(rows)][H].  H % 8 == 0, H <= 8192.
extern "C" int pk_rmsnorm_backward(const void* grad_out, const void* grad_sum, const void* x, const void* weight, void* dx,
                                   void* dw, void* dw_partials, long long rows, int H, float eps, void* stream) {
    if (rows < 0 || H <= 0 || (H % 8) || H > 8 * 256 * kBwdMaxVec) return kErrShape;
    if (!grad_out || !x || !weight || !dx || !dw || !dw_partials) return kErrNull;
    const int parts = pk_rmsnorm_backward_parts(rows);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        cudaError_t e = cudaMemsetAsync(dw, 0, (size_t)H * 2, st);
        return (int)e;
    }
    rmsnorm_bwd_kernel<<<parts, 256, 0, st>>>(static_cast<const uint16_t*>(grad_out), static_cast<const uint16_t*>(grad_sum),
                                              static_cast<const uint16_t*>(x), static_cast<const uint16_t*>(weight),
                                              static_cast<uint16_t*>(dx), static_cast<float*>(dw_partials), rows, H, eps);
    rmsnorm_dw_reduce_kernel<<<(H + 255) / 256, 256, 0, st>>>(static_cast<const float*>(dw_partials), static_cast<uint16_t*>(dw),
                                                              parts, H);
    return (int)cudaPeekAtLastError();
}
