// Fused RMSNorm + residual + MXFP8 quantisation for sm_100a.
//
// Two kernels share the arithmetic:
//  * rmsnorm_pipe_kernel (large power-of-two shapes): persistent CTAs; a producer warp streams tiles of
//    whole rows into a 3-stage shared-memory ring with bulk async copies (completion on mbarriers), the
//    consumer warps take one 1024-element unit each -- a lane owns one 32-element MXFP8 group, so the group
//    amax needs no shuffle -- and the fp8 bytes leave through a bulk shared->global store.  The bytes in
//    flight are set by the ring (two stages), not by registers or occupancy.
//  * rmsnorm_mxfp8_kernel (every other shape): the row stays in registers, described next.
//
// One row is handled by a team of W warps.  Every thread owns U 16-byte chunks (8 bf16) of the
// row at chunk indices t, t+T, t+2T, ... (T = 32*W), so every load and store instruction of a
// warp touches one contiguous 512-byte (loads) / 256-byte (fp8 stores) span: fully coalesced
// 128-bit accesses with no 32-byte-sector over-fetch.  A 32-element MXFP8 group is 4 adjacent
// lanes; the group amax takes two shuffles.  The whole row stays in registers between the
// sum-of-squares reduction and the quantisation, so each input byte is read from HBM exactly once.
// Scale bytes are written four at a time (one 32-bit store per 16 lanes) straight into the
// blocked [mTile, kTile, 32, 4, 4] layout a block-scaled tensor-core GEMM reads.
//
// Arithmetic contract (bit-exact with the reference quantiser,
// prime_kernels/rmsnorm/src/kernels/rmsnorm_03_fixed_32pt.cu:67-98 and test.cu:108-146):
//   s   = rsqrtf(sum(x^2) * (1/C) + eps)
//   res = bf16( s * (branch * w) + residual )      product exact in fp32, no FMA contraction
//   sf  = e8m0_roundup( amax32(|res|) / 448 ),  q = e4m3_rn_sat( res * 2^(127 - sf) )
// Extensions: C only needs to be a multiple of 32 and N is arbitrary (padded scale bytes are
// written as 0); mode 1 adds the residual before the norm and can return the bf16 sum.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "pk_common.cuh"

namespace pk {

struct RmsParams {
    uint8_t* vals;            // [N, C] e4m3
    uint8_t* scales;          // ceil(N/128) * ceil(C/128) * 512 e8m0, blocked
    float* rrms;              // [N]
    uint16_t* res_out;        // optional [N, C] bf16 (mode 0: pre-quant value; mode 1: branch+residual)
    const uint4* branch;      // [N, C] bf16
    const uint4* residual;    // [N, C] bf16
    const uint4* weight;      // [C] bf16
    float eps;
    float inv_c;
    int n;
    int c;
    int n_pad;                // N rounded up to 128
    int nkt;                  // ceil(C/128)
    int warps_per_row;        // W
    int rows_per_block;
    int mode;                 // 0: residual added after the norm; 1: before
};

__device__ __forceinline__ uint32_t e8m0_roundup(float x) {
    // cvt.rp.satfinite.ue8m0x2.f32 packs two results; the low byte is the conversion of the 2nd operand
    uint16_t r;
    asm("cvt.rp.satfinite.ue8m0x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(x));
    return r & 0xffu;
}

__device__ __forceinline__ uint32_t e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// d = a * b + c per packed bf16 half (a, b: two bf16 each; product exact, fp32 add, one rounding) with the
// sm_100 mixed-precision FMA -- no unpacking of the bf16 operands.
__device__ __forceinline__ void fma2_bf16(uint32_t a, uint32_t b, float c_lo, float c_hi, float& d_lo, float& d_hi) {
    asm("{\n.reg .b16 al, ah, bl, bh;\nmov.b32 {al, ah}, %2;\nmov.b32 {bl, bh}, %3;\n"
        "fma.rn.f32.bf16 %0, al, bl, %4;\nfma.rn.f32.bf16 %1, ah, bh, %5;\n}"
        : "=f"(d_lo), "=f"(d_hi)
        : "r"(a), "r"(b), "f"(c_lo), "f"(c_hi));
}
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
constexpr uint32_t kOnesBf16x2 = 0x3f803f80u;

// LW: fetch the norm weights after the reduction (fewer live registers while the row's loads are in flight:
// better for large inputs) instead of together with the row (shorter dependent chain: better when one
// wave of blocks covers the whole input).
template <int U, int LW>
__global__ void __launch_bounds__(256, U == 4 ? 4 : 2) rmsnorm_mxfp8_kernel(const RmsParams p) {
    extern __shared__ float red_s[];   // [rows_per_block][W]
    const int W = p.warps_per_row;
    const int T = W * 32;
    const int team = threadIdx.x / T;
    const int tt = threadIdx.x - team * T;       // thread index inside the team
    const int lane = threadIdx.x & 31;
    const int warp_in_team = tt >> 5;
    const int row = blockIdx.x * p.rows_per_block + team;
    const int nch = p.c >> 3;                    // 16-byte chunks per row
    const bool live = row < p.n;

    uint4 br[U], rs[U], wt[U];
    float ss = 0.f, ss2 = 0.f;
    if (live) {
        const uint4* bp = p.branch + (size_t)row * nch;
        const uint4* rp = p.residual + (size_t)row * nch;
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int c = tt + i * T;
            if (c < nch) {
                br[i] = ld_stream_16(bp + c);
                rs[i] = ld_stream_16(rp + c);
            }
        }
        if (!LW) {
#pragma unroll
            for (int i = 0; i < U; ++i) {
                const int c = tt + i * T;
                if (c < nch) wt[i] = __ldg(p.weight + c);
            }
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int c = tt + i * T;
            if (c < nch) {
                uint32_t a[4] = {br[i].x, br[i].y, br[i].z, br[i].w};
                if (p.mode) {
                    // sum = bf16(branch + residual): both addends exact in fp32, one rounding
                    const uint32_t r4[4] = {rs[i].x, rs[i].y, rs[i].z, rs[i].w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float lo, hi;
                        fma2_bf16(r4[k], kOnesBf16x2, 0.f, 0.f, lo, hi);
                        fma2_bf16(a[k], kOnesBf16x2, lo, hi, lo, hi);
                        a[k] = pack_bf16x2(lo, hi);
                    }
                    br[i] = make_uint4(a[0], a[1], a[2], a[3]);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) fma2_bf16(a[k], a[k], ss, ss2, ss, ss2);
            }
        }
    }
    ss = warp_sum(ss + ss2);
    if (W > 1) {
        if (lane == 0) red_s[team * W + warp_in_team] = ss;
        // one named barrier per team: the rows of a block do not wait for each other
        asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(T) : "memory");
        float tot = 0.f;
        for (int w = 0; w < W; ++w) tot += red_s[team * W + w];
        ss = tot;
    }
    const float s = rsqrtf(ss * p.inv_c + p.eps);

    if (row >= p.n_pad) return;
    // late weights (an L1/L2 hit): holding them across the reduction would cost 4*U registers during
    // the phase in which the row's loads are in flight
    if (LW && live) {
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const int c = tt + i * T;
            if (c < nch) wt[i] = __ldg(p.weight + c);
        }
    }
    uint32_t* sc32 = reinterpret_cast<uint32_t*>(p.scales);
#pragma unroll
    for (int i = 0; i < U; ++i) {
        const int c = tt + i * T;
        const bool has = live && c < nch;       // uniform over each aligned group of 4 lanes
        uint32_t packed[4] = {0u, 0u, 0u, 0u};
        uint32_t amax2 = 0u;                    // packed bf16 pair, both halves >= 0
        if (has) {
            const uint32_t a[4] = {br[i].x, br[i].y, br[i].z, br[i].w};
            const uint32_t r4[4] = {rs[i].x, rs[i].y, rs[i].z, rs[i].w};
            const uint32_t w4[4] = {wt[i].x, wt[i].y, wt[i].z, wt[i].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float pl, ph;
                fma2_bf16(a[k], w4[k], 0.f, 0.f, pl, ph);          // exact bf16 x bf16 products
                float ol = __fmul_rn(s, pl), oh = __fmul_rn(s, ph);
                // residual added after the norm in fp32 (r * 1 + x: exact product, one rounding, the same
                // as widening r and adding; never contracted with the multiply above)
                if (!p.mode) fma2_bf16(r4[k], kOnesBf16x2, ol, oh, ol, oh);
                packed[k] = pack_bf16x2(ol, oh);
                amax2 = max_bf16x2(amax2, packed[k] & 0x7fff7fffu);    // |x| by mask: abs.bf16x2 issues at half rate
            }
            if (p.res_out) {
                const uint4 o = p.mode ? br[i] : make_uint4(packed[0], packed[1], packed[2], packed[3]);
                st_stream_16(p.res_out + ((size_t)row * nch + c) * 8, o);
            }
        }
        // group amax over the 4 lanes of a 32-element group (executed by the whole warp)
        float amax = fmaxf(bf16_lo(amax2), bf16_hi(amax2));
        amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, 2));
        uint32_t sf = 0;
        if (has) {
            sf = e8m0_roundup(__fmul_rn(amax, 1.f / 448.f));
            const uint32_t e = 254u - sf;
            const uint32_t invb = e ? (e << 7) : 0x0040u;          // bf16 bits of 2^(127 - sf)
            const uint32_t inv2 = invb | (invb << 16);
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) fma2_bf16(packed[k], inv2, 0.f, 0.f, v[2 * k], v[2 * k + 1]);   // exact scaling
            uint2 q;
            q.x = e4m3x2(v[0], v[1]) | (e4m3x2(v[2], v[3]) << 16);
            q.y = e4m3x2(v[4], v[5]) | (e4m3x2(v[6], v[7]) << 16);
            st_stream_8(p.vals + ((size_t)row * nch + c) * 8, q);
        }
        // four consecutive groups (16 lanes) -> one 32-bit store of scale bytes; groups past the
        // end of the row and rows past N get 0 so that padded tiles are fully defined
        const int base = lane & 16;
        const uint32_t b0 = __shfl_sync(kFullMask, sf, base + 0);
        const uint32_t b1 = __shfl_sync(kFullMask, sf, base + 4);
        const uint32_t b2 = __shfl_sync(kFullMask, sf, base + 8);
        const uint32_t b3 = __shfl_sync(kFullMask, sf, base + 12);
        if ((lane & 15) == 0 && c < p.nkt * 16) {
            const int k = c >> 2;                 // group index, multiple of 4
            const size_t off = ((size_t)(row >> 7) * p.nkt + (k >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
            sc32[off >> 2] = b0 | (b1 << 8) | (b2 << 16) | (b3 << 24);
        }
    }
    if (live && tt == 0) p.rrms[row] = s;
}


// ---------------------------------------------------------------- pipelined kernel
constexpr int kPipeStages = 3;
constexpr int kPipeUnit = 1024;                 // elements per consumer warp and tile
constexpr unsigned kPipeSpinLimit = 1u << 26;   // bounded mbarrier waits (~seconds)
__device__ unsigned int g_rms_wait_timeouts;    // waits that gave up (results of that launch are invalid)

__device__ __forceinline__ void pipe_wait(uint64_t* bar, uint32_t parity) {
    for (unsigned spins = 0; !mbar_test(bar, parity); ++spins)
        if (spins > kPipeSpinLimit) {
            atomicAdd(&g_rms_wait_timeouts, 1u);
            return;
        }
}
// global -> this CTA's shared memory (never multicast), completion counted in bytes on an mbarrier
__device__ __forceinline__ void pipe_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void pipe_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

struct PipeShared {
    uint64_t full[kPipeStages], empty[kPipeStages];
    float part[2][16];            // per-unit sums of squares, double-buffered by tile parity
};
constexpr size_t pipe_smem_bytes(int pw) { return 256 + (size_t)kPipeStages * pw * kPipeUnit * 4 + (size_t)pw * 2048; }

// C = 1024 * M; PW consumer warps (one unit each) + one producer warp; a tile is PW / M consecutive rows, so
// its branch and residual bytes are one contiguous range each.  16 / PW CTAs per SM.
template <int M, int PW>
__global__ void __launch_bounds__(PW * 32 + 32, 16 / PW) rmsnorm_pipe_kernel(const RmsParams p, int ntiles) {
    constexpr int kTile = PW * kPipeUnit;
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    PipeShared& sh = *reinterpret_cast<PipeShared*>(pipe_smem);
    unsigned char* stages = pipe_smem + 256;                                  // kPipeStages x (branch, residual)
    unsigned char* outs = stages + (size_t)kPipeStages * kTile * 4;           // PW x 2 x 1 KB of fp8
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < kPipeStages; ++s) {
            mbar_init(&sh.full[s], 1);
            mbar_init(&sh.empty[s], PW);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == PW) {
        if (lane == 0) {
            int it = 0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
                const int s = it % kPipeStages;
                if (it >= kPipeStages) pipe_wait(&sh.empty[s], ((it / kPipeStages) - 1) & 1);
                mbar_expect_tx(&sh.full[s], kTile * 4);
                unsigned char* dst = stages + (size_t)s * kTile * 4;
                pipe_g2s(dst, reinterpret_cast<const uint16_t*>(p.branch) + (size_t)t * kTile, kTile * 2, &sh.full[s]);
                pipe_g2s(dst + kTile * 2, reinterpret_cast<const uint16_t*>(p.residual) + (size_t)t * kTile, kTile * 2,
                         &sh.full[s]);
            }
        }
        return;
    }
    constexpr int R = PW / M;                         // rows per tile
    const int row_in_tile = warp / M, seg = warp % M;
    // A lane owns 64 contiguous bytes (one 32-element group) of each input.  Its four 16-byte chunks are
    // visited in an order rotated by lane / 2, which makes every 8-lane phase of a 128-bit shared-memory
    // access hit eight different 16-byte bank groups.
    const int rot = lane >> 1;
    const uint4* wsrc = p.weight + seg * 128 + 4 * lane;
    uint32_t* sc32 = reinterpret_cast<uint32_t*>(p.scales);
    unsigned char* myout = outs + (size_t)warp * 2048;
    int it = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
        const int s = it % kPipeStages;
        pipe_wait(&sh.full[s], (it / kPipeStages) & 1);
        const uint4* sb = reinterpret_cast<const uint4*>(stages + (size_t)s * kTile * 4) + warp * 128 + 4 * lane;
        const uint4* sr = sb + kTile / 8;
        uint4 br[4], rs[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cj = (j + rot) & 3;
            br[j] = sb[cj];
            rs[j] = sr[cj];
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.empty[s]);      // the unit is in registers: the stage can be refilled
        float ss = 0.f, ss2 = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            fma2_bf16(br[j].x, br[j].x, ss, ss2, ss, ss2);
            fma2_bf16(br[j].y, br[j].y, ss, ss2, ss, ss2);
            fma2_bf16(br[j].z, br[j].z, ss, ss2, ss, ss2);
            fma2_bf16(br[j].w, br[j].w, ss, ss2, ss, ss2);
        }
        ss = warp_sum(ss + ss2);
        if (M > 1) {
            // the M warps of a row meet on the row's own named barrier; partials are summed in unit order
            if (lane == 0) sh.part[it & 1][warp] = ss;
            asm volatile("bar.sync %0, %1;" ::"r"(1 + row_in_tile), "n"(32 * M) : "memory");
            float tot = 0.f;
#pragma unroll
            for (int j = 0; j < M; ++j) tot += sh.part[it & 1][row_in_tile * M + j];
            ss = tot;
        }
        const float sc = rsqrtf(ss * p.inv_c + p.eps);
        uint4 wt[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) wt[j] = __ldg(wsrc + ((j + rot) & 3));
        uint32_t amax2 = 0u;
        uint32_t res[16];                              // bf16 pairs of the pre-quantisation values
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t a[4] = {br[j].x, br[j].y, br[j].z, br[j].w};
            const uint32_t r4[4] = {rs[j].x, rs[j].y, rs[j].z, rs[j].w};
            const uint32_t w4[4] = {wt[j].x, wt[j].y, wt[j].z, wt[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float pl, ph;
                fma2_bf16(a[k], w4[k], 0.f, 0.f, pl, ph);                 // exact bf16 x bf16 products
                float ol = __fmul_rn(sc, pl), oh = __fmul_rn(sc, ph);
                fma2_bf16(r4[k], kOnesBf16x2, ol, oh, ol, oh);            // + residual in fp32, one rounding
                res[4 * j + k] = pack_bf16x2(ol, oh);
                amax2 = max_bf16x2(amax2, res[4 * j + k] & 0x7fff7fffu);
            }
        }
        const float amax = fmaxf(bf16_lo(amax2), bf16_hi(amax2));
        const uint32_t sf = e8m0_roundup(__fmul_rn(amax, 1.f / 448.f));
        const uint32_t e = 254u - sf;
        const uint32_t invb = e ? (e << 7) : 0x0040u;                     // bf16 bits of 2^(127 - sf)
        const uint32_t inv2 = invb | (invb << 16);
        // the bulk store issued from this output buffer two tiles ago must have finished reading it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
        unsigned char* ob = myout + (it & 1) * 1024 + lane * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) fma2_bf16(res[4 * j + k], inv2, 0.f, 0.f, v[2 * k], v[2 * k + 1]);
            uint2 q;
            q.x = e4m3x2(v[0], v[1]) | (e4m3x2(v[2], v[3]) << 16);
            q.y = e4m3x2(v[4], v[5]) | (e4m3x2(v[6], v[7]) << 16);
            *reinterpret_cast<uint2*>(ob + 8 * ((j + rot) & 3)) = q;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) pipe_s2g(p.vals + (size_t)t * kTile + warp * kPipeUnit, myout + (it & 1) * 1024, 1024);
        // scale bytes of four adjacent groups -> one 32-bit store into the blocked layout
        uint32_t w2 = sf | (__shfl_xor_sync(kFullMask, sf, 1) << 8);
        w2 |= __shfl_xor_sync(kFullMask, w2, 2) << 16;
        const int row = t * R + row_in_tile;
        if ((lane & 3) == 0) {
            const int k = seg * 32 + lane;
            const size_t off = ((size_t)(row >> 7) * p.nkt + (k >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
            sc32[off >> 2] = w2;
        }
        if (seg == 0 && lane == 0) p.rrms[row] = sc;
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

template <int M, int PW>
static int launch_pipe_mp(const RmsParams& p, cudaStream_t stream) {
    static int sms[64] = {0};        // per device: SM count, read once (and the kernel's shared-memory opt-in)
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return kErrShape;
    constexpr size_t smem = pipe_smem_bytes(PW);
    if (!sms[dev]) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cudaError_t e = cudaFuncSetAttribute(rmsnorm_pipe_kernel<M, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        sms[dev] = n;
    }
    const int ntiles = p.n / (PW / M);
    const int grid = ntiles < sms[dev] * (16 / PW) ? ntiles : sms[dev] * (16 / PW);
    rmsnorm_pipe_kernel<M, PW><<<grid, PW * 32 + 32, smem, stream>>>(p, ntiles);
    return (int)cudaPeekAtLastError();
}

// Shapes the pipelined kernel takes (chosen by measurement against the lane-owns-group kernel): reference
// semantics only (mode 0, no residual output), whole 128-row tiles, C = 8192 or 16384, and enough rows to give
// every CTA several tiles.  The templates also cover C = 1024, 2048 and 4096, where the other kernel is as fast.
static bool pipe_eligible(const RmsParams& p) {
    if (p.mode != 0 || p.res_out != nullptr || (p.n % 128) != 0) return false;
    // bulk copies in both directions (global -> shared for branch / residual, shared -> global for vals) need
    // 16-byte aligned global addresses; the C entries only guarantee 8 bytes for vals
    auto a16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!a16(p.vals) || !a16(p.branch) || !a16(p.residual)) return false;
    if (p.c == 8192) return p.n >= 8192;
    if (p.c == 16384) return p.n >= 2048;
    return false;
}
static int launch_pipe(const RmsParams& p, cudaStream_t stream) {
    switch (p.c) {
        case 1024: return launch_pipe_mp<1, 8>(p, stream);
        case 2048: return launch_pipe_mp<2, 8>(p, stream);
        case 4096: return launch_pipe_mp<4, 8>(p, stream);
        case 8192: return launch_pipe_mp<8, 8>(p, stream);
        default: return launch_pipe_mp<16, 16>(p, stream);
    }
}


// ---------------------------------------------------------------- lane-owns-group kernel (256-bit accesses)
// A row is handled by M = ceil(C / 1024) warps and a lane owns one whole 32-element MXFP8 group: it reads the
// group's 64 bytes of each input with two 256-bit loads (sm_100 `ld.global.v8.b32`), needs no cross-lane
// traffic for the amax, the E8M0 conversion or the scale byte, and writes its 32 fp8 bytes with one 256-bit
// store.  Blocks are small (ROWS rows of M warps, at most TMAX threads), so a launch fills the machine at
// once and its tail is short.  Handles every shape of the op (ragged N, C % 32 == 0 up to 16384, both modes,
// optional bf16 output); needs 32-byte aligned pointers.
struct u32x8 {
    uint32_t v[8];
};
__device__ __forceinline__ u32x8 ld_stream_32(const void* p) {
    u32x8 r;
    asm volatile("ld.global.cs.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
                   "=r"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ u32x8 ld_keep_32(const void* p) {
    u32x8 r;
    asm volatile("ld.global.nc.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
                   "=r"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st_stream_32(void* p, const u32x8& r) {
    asm volatile("st.global.cs.v8.u32 [%8], {%0,%1,%2,%3,%4,%5,%6,%7};" ::"r"(r.v[0]), "r"(r.v[1]), "r"(r.v[2]),
                 "r"(r.v[3]), "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7]), "l"(p)
                 : "memory");
}

// MT > 0: C == 1024 * MT, N % 128 == 0, reference semantics -- every lane is live and nothing is optional
// (the common large shapes); MT == 0: the general form with a run-time warp count and masks.
template <int TMAX, int MT>
__global__ void __launch_bounds__(TMAX, 1024 / TMAX) rmsnorm_group_kernel(const RmsParams p) {
    __shared__ float part[16];
    constexpr bool kFull = MT > 0;
    const int M = kFull ? MT : p.warps_per_row;
    const int mode = kFull ? 0 : p.mode;
    uint16_t* const res_out = kFull ? nullptr : p.res_out;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_in_block = warp / M, seg = warp - row_in_block * M;
    const int row = blockIdx.x * p.rows_per_block + row_in_block;
    const int g = seg * 32 + lane;                     // group index inside the row
    const bool live = kFull || row < p.n;
    const bool has = kFull || (live && g < (p.c >> 5));
    const size_t ebase = (size_t)row * p.c + (size_t)g * 32;
    u32x8 br[2], rs[2], wt[2];
    if (has) {
        const uint16_t* gb = reinterpret_cast<const uint16_t*>(p.branch) + ebase;
        const uint16_t* gr = reinterpret_cast<const uint16_t*>(p.residual) + ebase;
        const uint16_t* gw = reinterpret_cast<const uint16_t*>(p.weight) + g * 32;
        br[0] = ld_stream_32(gb);
        br[1] = ld_stream_32(gb + 16);
        rs[0] = ld_stream_32(gr);
        rs[1] = ld_stream_32(gr + 16);
        wt[0] = ld_keep_32(gw);
        wt[1] = ld_keep_32(gw + 16);
    } else {
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) br[j].v[k] = rs[j].v[k] = wt[j].v[k] = 0u;
    }
    if (mode) {
        // sum = bf16(branch + residual): both addends exact in fp32, one rounding
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float lo, hi;
                fma2_bf16(rs[j].v[k], kOnesBf16x2, 0.f, 0.f, lo, hi);
                fma2_bf16(br[j].v[k], kOnesBf16x2, lo, hi, lo, hi);
                br[j].v[k] = pack_bf16x2(lo, hi);
            }
    }
    float ss = 0.f, ss2 = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int k = 0; k < 8; ++k) fma2_bf16(br[j].v[k], br[j].v[k], ss, ss2, ss, ss2);
    ss = warp_sum(ss + ss2);
    if (M > 1) {
        // the warps of a row meet on the row's own named barrier; partials are added in segment order
        if (lane == 0) part[warp] = ss;
        // Barrier ids are immediates: a barrier id held in a register makes the compiler reserve all 16
        // hardware barriers for the block, which caps the number of resident blocks per SM.
        if (p.rows_per_block == 1) {
            __syncthreads();
        } else {
            switch (row_in_block) {
                case 0: asm volatile("bar.sync 1, %0;" ::"r"(32 * M) : "memory"); break;
                case 1: asm volatile("bar.sync 2, %0;" ::"r"(32 * M) : "memory"); break;
                case 2: asm volatile("bar.sync 3, %0;" ::"r"(32 * M) : "memory"); break;
                default: asm volatile("bar.sync 4, %0;" ::"r"(32 * M) : "memory"); break;
            }
        }
        float tot = 0.f;
#pragma unroll
        for (int j = 0; j < (kFull ? MT : 16); ++j)
            if (kFull || j < M) tot += part[row_in_block * M + j];
        ss = tot;
    }
    const float sc = rsqrtf(ss * p.inv_c + p.eps);
    if (!kFull && row >= p.n_pad) return;
    uint32_t sf = 0u;
    if (has) {
        uint32_t amax2 = 0u;
        uint32_t res[16];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float pl, ph;
                fma2_bf16(br[j].v[k], wt[j].v[k], 0.f, 0.f, pl, ph);             // exact bf16 x bf16 products
                float ol = __fmul_rn(sc, pl), oh = __fmul_rn(sc, ph);
                if (!mode) fma2_bf16(rs[j].v[k], kOnesBf16x2, ol, oh, ol, oh);   // + residual in fp32, one rounding
                res[8 * j + k] = pack_bf16x2(ol, oh);
                amax2 = max_bf16x2(amax2, res[8 * j + k] & 0x7fff7fffu);
            }
        if (res_out) {
            u32x8 o0, o1;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                o0.v[k] = mode ? br[0].v[k] : res[k];
                o1.v[k] = mode ? br[1].v[k] : res[8 + k];
            }
            st_stream_32(res_out + ebase, o0);
            st_stream_32(res_out + ebase + 16, o1);
        }
        const float amax = fmaxf(bf16_lo(amax2), bf16_hi(amax2));
        sf = e8m0_roundup(__fmul_rn(amax, 1.f / 448.f));
        const uint32_t e = 254u - sf;
        const uint32_t invb = e ? (e << 7) : 0x0040u;                            // bf16 bits of 2^(127 - sf)
        const uint32_t inv2 = invb | (invb << 16);
        u32x8 q;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float v0, v1, v2, v3;
            fma2_bf16(res[2 * k], inv2, 0.f, 0.f, v0, v1);                       // exact scaling
            fma2_bf16(res[2 * k + 1], inv2, 0.f, 0.f, v2, v3);
            q.v[k] = e4m3x2(v0, v1) | (e4m3x2(v2, v3) << 16);
        }
        st_stream_32(p.vals + ebase, q);
    }
    // scale bytes of four adjacent groups -> one 32-bit store into the blocked layout; groups past the end of
    // the row and rows past N carry 0, so padded tiles are fully defined
    uint32_t w2 = sf | (__shfl_xor_sync(kFullMask, sf, 1) << 8);
    w2 |= __shfl_xor_sync(kFullMask, w2, 2) << 16;
    if ((lane & 3) == 0 && (kFull || g < p.nkt * 4)) {
        const size_t off = ((size_t)(row >> 7) * p.nkt + (g >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4;
        reinterpret_cast<uint32_t*>(p.scales)[off >> 2] = w2;
    }
    if (live && seg == 0 && lane == 0) p.rrms[row] = sc;
}

static bool aligned32(const void* q) { return (reinterpret_cast<uintptr_t>(q) & 31) == 0; }
static bool group_eligible(const RmsParams& p) {
    return p.c <= 16384 && aligned32(p.vals) && aligned32(p.branch) && aligned32(p.residual) && aligned32(p.weight) &&
           (p.res_out == nullptr || aligned32(p.res_out));
}
static int launch_group(const RmsParams& p0, cudaStream_t stream) {
    RmsParams p = p0;
    const int M = (p.c + 1023) / 1024;
    // rows per block, chosen by measurement: small blocks; 2048-wide rows prefer four rows per block once
    // the input is large
    int rows = 1;
    if (M == 1) rows = 2;
    else if (M == 2 && p.n >= 16384) rows = 4;
    p.warps_per_row = M;
    p.rows_per_block = rows;
    const int threads = rows * M * 32;
    const int grid = (p.n_pad + rows - 1) / rows;
    if (grid == 0) return kOk;
    const bool full = p.mode == 0 && p.res_out == nullptr && (p.n % 128) == 0 && (p.c % 1024) == 0;
    if (full && M == 1) rmsnorm_group_kernel<64, 1><<<grid, threads, 0, stream>>>(p);
    else if (full && M == 2 && rows == 1) rmsnorm_group_kernel<64, 2><<<grid, threads, 0, stream>>>(p);
    else if (full && M == 2) rmsnorm_group_kernel<256, 2><<<grid, threads, 0, stream>>>(p);
    else if (full && M == 4) rmsnorm_group_kernel<128, 4><<<grid, threads, 0, stream>>>(p);
    else if (full && M == 8) rmsnorm_group_kernel<256, 8><<<grid, threads, 0, stream>>>(p);
    else if (full && M == 16) rmsnorm_group_kernel<512, 16><<<grid, threads, 0, stream>>>(p);
    else if (threads <= 64) rmsnorm_group_kernel<64, 0><<<grid, threads, 0, stream>>>(p);
    else if (threads <= 128) rmsnorm_group_kernel<128, 0><<<grid, threads, 0, stream>>>(p);
    else if (threads <= 256) rmsnorm_group_kernel<256, 0><<<grid, threads, 0, stream>>>(p);
    else rmsnorm_group_kernel<512, 0><<<grid, threads, 0, stream>>>(p);
    return (int)cudaPeekAtLastError();
}

static int launch_rmsnorm(const RmsParams& p0, cudaStream_t stream) {
    if (pipe_eligible(p0)) return launch_pipe(p0, stream);
    if (group_eligible(p0)) return launch_group(p0, stream);
    RmsParams p = p0;
    const int nch = p.c / 8;
    // a team is at most 8 warps (256 threads): 4 chunks per thread up to C = 8192, 8 chunks up to 16384
    int U = nch <= 1024 ? 4 : 8;
    const int W = (nch + 32 * U - 1) / (32 * U);
    if (W > 8) return kErrShape;
    // teams must tile the block exactly: W rounded up to a power of two
    int Wp = 1;
    while (Wp < W) Wp <<= 1;
    p.warps_per_row = Wp;
    p.rows_per_block = 8 / Wp;
    const int threads = p.rows_per_block * Wp * 32;
    const int grid = (p.n_pad + p.rows_per_block - 1) / p.rows_per_block;
    if (grid == 0) return kOk;
    const size_t smem = (size_t)p.rows_per_block * Wp * sizeof(float);
    const bool late = (long long)p.n * p.c >= (1ll << 23);
    if (U == 4) {
        if (late) rmsnorm_mxfp8_kernel<4, 1><<<grid, threads, smem, stream>>>(p);
        else rmsnorm_mxfp8_kernel<4, 0><<<grid, threads, smem, stream>>>(p);
    } else {
        rmsnorm_mxfp8_kernel<8, 0><<<grid, threads, smem, stream>>>(p);
    }
    return (int)cudaPeekAtLastError();
}

}  // namespace pk

// ---------------------------------------------------------------- C ABI
// Replaces prime_kernels/rmsnorm/rmsnorm.cuh:15-18,85 (fused_rmsnorm_residual_forward): same
// argument order and meaning, but plain pointers, a status return instead of assert/exit, and
// relaxed shapes (any N >= 0, C a positive multiple of 32).
extern "C" int pk_fused_rmsnorm_residual_forward(void* vals, void* scales, float* rrms, const void* branch,
                                                 const void* residual, const void* weight, float epsilon,
                                                 int N, int C, void* stream) {
    using namespace pk;
    if (N < 0 || C <= 0 || (C % 32) != 0) return kErrShape;
    if (N == 0) return kOk;
    if (!vals || !scales || !rrms || !branch || !residual || !weight) return kErrNull;
    if ((reinterpret_cast<uintptr_t>(vals) % 8) || (reinterpret_cast<uintptr_t>(scales) % 4) ||
        (reinterpret_cast<uintptr_t>(branch) % 16) || (reinterpret_cast<uintptr_t>(residual) % 16) ||
        (reinterpret_cast<uintptr_t>(weight) % 16))
        return kErrAlign;
    RmsParams p{};
    p.vals = static_cast<uint8_t*>(vals);
    p.scales = static_cast<uint8_t*>(scales);
    p.rrms = rrms;
    p.res_out = nullptr;
    p.branch = static_cast<const uint4*>(branch);
    p.residual = static_cast<const uint4*>(residual);
    p.weight = static_cast<const uint4*>(weight);
    p.eps = epsilon;
    p.inv_c = 1.f / (float)C;
    p.n = N;
    p.c = C;
    p.n_pad = (N + 127) / 128 * 128;
    p.nkt = (C + 127) / 128;
    p.mode = 0;
    return launch_rmsnorm(p, static_cast<cudaStream_t>(stream));
}

// Host-side view of the dispatcher for the reference-semantics entry (no launch, no device needed): 2 = pipelined
// bulk-copy kernel, 1 = lane-owns-group kernel, 0 = register kernel, negative = the status the entry would return.
// Lets callers and tests see that pointers that are not 16-byte aligned never reach the bulk-copy kernel.
extern "C" int pk_rmsnorm_dispatch(const void* vals, const void* branch, const void* residual, const void* weight,
                                   int N, int C) {
    using namespace pk;
    if (N <= 0 || C <= 0 || (C % 32) != 0) return -kErrShape;
    if ((reinterpret_cast<uintptr_t>(vals) % 8) || (reinterpret_cast<uintptr_t>(branch) % 16) ||
        (reinterpret_cast<uintptr_t>(residual) % 16) || (reinterpret_cast<uintptr_t>(weight) % 16))
        return -kErrAlign;
    RmsParams p{};
    p.vals = static_cast<uint8_t*>(const_cast<void*>(vals));
    p.branch = static_cast<const uint4*>(branch);
    p.residual = static_cast<const uint4*>(residual);
    p.weight = static_cast<const uint4*>(weight);
    p.n = N;
    p.c = C;
    return pipe_eligible(p) ? 2 : (group_eligible(p) ? 1 : 0);
}

// Extended entry: mode 0 = residual added after the norm (reference semantics), mode 1 = residual
// added before the norm (the semantics of the reference's Triton residual-RMSNorm op,
// prime_kernels/triton_rmsnorm/rmsnorm.py:711-722, followed by the same quantiser).
// res_out (optional, bf16 [N, C]) receives the updated residual stream.
extern "C" int pk_fused_rmsnorm_residual_forward_ex(void* vals, void* scales, float* rrms, void* res_out,
                                                    const void* branch, const void* residual,
                                                    const void* weight, float epsilon, int N, int C, int mode,
                                                    void* stream) {
    using namespace pk;
    if (N < 0 || C <= 0 || (C % 32) != 0 || mode < 0 || mode > 1) return kErrShape;
    if (N == 0) return kOk;
    if (!vals || !scales || !rrms || !branch || !residual || !weight) return kErrNull;
    if ((reinterpret_cast<uintptr_t>(vals) % 8) || (reinterpret_cast<uintptr_t>(scales) % 4) ||
        (reinterpret_cast<uintptr_t>(branch) % 16) || (reinterpret_cast<uintptr_t>(residual) % 16) ||
        (reinterpret_cast<uintptr_t>(weight) % 16) || (res_out && reinterpret_cast<uintptr_t>(res_out) % 16))
        return kErrAlign;
    RmsParams p{};
    p.vals = static_cast<uint8_t*>(vals);
    p.scales = static_cast<uint8_t*>(scales);
    p.rrms = rrms;
    p.res_out = static_cast<uint16_t*>(res_out);
    p.branch = static_cast<const uint4*>(branch);
    p.residual = static_cast<const uint4*>(residual);
    p.weight = static_cast<const uint4*>(weight);
    p.eps = epsilon;
    p.inv_c = 1.f / (float)C;
    p.n = N;
    p.c = C;
    p.n_pad = (N + 127) / 128 * 128;
    p.nkt = (C + 127) / 128;
    p.mode = mode;
    return launch_rmsnorm(p, static_cast<cudaStream_t>(stream));
}

// Number of bounded shared-memory-barrier waits of the pipelined kernel that gave up since the library was
// loaded (0 in normal operation; a launch that counted one produced invalid output).  Synchronises the device.
extern "C" long long pk_rmsnorm_wait_timeouts(void) {
    unsigned int n = 0;
    if (cudaMemcpyFromSymbol(&n, pk::g_rms_wait_timeouts, sizeof(n)) != cudaSuccess) return -1;
    return (long long)n;
}

extern "C" long long pk_rmsnorm_scale_bytes(int N, int C) {
    return (long long)((N + 127) / 128) * ((C + 127) / 128) * 512;
}

// ---------------------------------------------------------------- MXFP8 weight packing
// Quantises a row-major bf16 matrix [rows, K] with the same per-32 recipe as the activation quantiser
// (scale = 2^ceil(log2(amax/448)), value = e4m3(bf16(w * 2^-scale))) along K and writes the packed-row
// format the decode GEMV streams: [K e4m3][K/32 e8m0][zero pad to a multiple of 16 bytes].
// One warp per row; lane owns whole 32-element groups (group g handled by lane g % 32).
namespace pk {

// floor_mode: the block-scale rule of the reference's flash_moe kernels instead
// (prime_kernels/flash_moe/csrc/kernels/fused_moe_mxfp8_kernel.cu:4-20): e = clamp(biased_exponent(amax) - 8, 0, 254),
// values w * 2^(127 - e) converted from fp32 with finite saturation (the largest values of a group may saturate).
__global__ void __launch_bounds__(256) pack_weights_mxfp8_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ out,
                                                                 long long rows, int K, int rowbytes, int floor_mode) {
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    const uint16_t* src = w + row * K;
    uint8_t* dst = out + row * rowbytes;
    const int groups = K >> 5;
    for (int g = lane; g < groups; g += 32) {
        const uint4* p = reinterpret_cast<const uint4*>(src + g * 32);
        uint32_t v[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 q = __ldg(p + i);
            v[4 * i] = q.x; v[4 * i + 1] = q.y; v[4 * i + 2] = q.z; v[4 * i + 3] = q.w;
        }
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fmaxf(fabsf(bf16_lo(v[i])), fabsf(bf16_hi(v[i]))));
        uint32_t sf;
        float inv;
        if (floor_mode) {
            int ef = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 8;
            ef = ef < 0 ? 0 : (ef > 254 ? 254 : ef);
            sf = (uint32_t)ef;
            inv = __uint_as_float((uint32_t)(254 - ef) << 23);
        } else {
            sf = e8m0_roundup(__fmul_rn(amax, 1.f / 448.f));
            const uint32_t e = 254u - sf;
            inv = __uint_as_float(e ? (e << 23) : 0x00400000u);
        }
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            q[i] = e4m3x2(bf16_lo(v[2 * i]) * inv, bf16_hi(v[2 * i]) * inv) |
                   (e4m3x2(bf16_lo(v[2 * i + 1]) * inv, bf16_hi(v[2 * i + 1]) * inv) << 16);
        uint4* o = reinterpret_cast<uint4*>(dst + g * 32);
        o[0] = make_uint4(q[0], q[1], q[2], q[3]);
        o[1] = make_uint4(q[4], q[5], q[6], q[7]);
        dst[K + g] = (uint8_t)sf;
    }
    for (int i = K + groups + lane; i < rowbytes; i += 32) dst[i] = 0;
}

}  // namespace pk

extern "C" long long pk_mxfp8_packed_row_bytes(int K) { return K % 32 ? -1 : ((long long)K + K / 32 + 15) / 16 * 16; }

// No counterpart in the reference (it consumes pre-quantised weights, flash_moe/__init__.py:165-170).
// scale_mode 0: round-up scales (the rmsnorm quantiser's rule, never saturates); 1: floor scales (flash_moe's rule).
extern "C" int pk_pack_weights_mxfp8_ex(const void* weights_bf16, void* packed, long long rows, int K, int scale_mode,
                                        void* stream) {
    using namespace pk;
    if (rows < 0 || K <= 0 || (K % 32) != 0 || (scale_mode != 0 && scale_mode != 1)) return kErrShape;
    if (rows == 0) return kOk;
    if (!weights_bf16 || !packed) return kErrNull;
    if ((reinterpret_cast<uintptr_t>(weights_bf16) % 16) || (reinterpret_cast<uintptr_t>(packed) % 16)) return kErrAlign;
    const int rowbytes = (int)pk_mxfp8_packed_row_bytes(K);
    const long long blocks = (rows + 7) / 8;
    if (blocks > 0x7fffffffLL) return kErrShape;
    pack_weights_mxfp8_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(weights_bf16), static_cast<uint8_t*>(packed), rows, K, rowbytes, scale_mode);
    return (int)cudaPeekAtLastError();
}

extern "C" int pk_pack_weights_mxfp8(const void* weights_bf16, void* packed, long long rows, int K, void* stream) {
    return pk_pack_weights_mxfp8_ex(weights_bf16, packed, rows, K, 0, stream);
}
