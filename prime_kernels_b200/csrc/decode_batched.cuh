// Batched decode step (up to 64 requests; the default from 4, or from 2 for wide models) with the projections on the
// 5th-generation tensor cores
// (included by decode_megakernel.cu).
//
// From a handful of requests on every projection is a real GEMM, C[rows, B] = W[rows, K] . X[B, K]^T.  It is mapped
// "swap-AB": the A operand is a tile of 128 weight rows (so a weight byte is streamed exactly once per step,
// like in the GEMV kernels), the B operand is the activation matrix with the batch padded to N = 16 / 32 / 64,
// and the fp32 accumulator tile (128 lanes x N columns) lives in tensor memory:
//
//   * operands are staged in shared memory in the K-major 128-byte-swizzle layout tcgen05.mma reads (rows of
//     64 bf16, eight-row groups of 1024 bytes, 16-byte chunks XOR-swizzled by the row).  bf16 weights and
//     activations arrive with 16-byte cp.async copies placed chunk by chunk; MXFP8 weights (E4M3 + one E8M0 per
//     32 along K) are de-quantised to bf16 in registers on their way in, which is exact;
//   * one elected thread issues tcgen05.mma (kind::f16, cta_group::1, M = 128, K = 16 per instruction) and
//     commits to an mbarrier; four warps read the accumulator back with tcgen05.ld (thread = weight row) and
//     run the epilogue;
//   * a phase has too few 128-row tiles to occupy 148 SMs, so K is split over work items as well; partial
//     tiles are added into an fp32 matrix in L2 with red.global.add and the rounding / residual / SwiGLU /
//     norm epilogues run after the grid barrier that ends the phase (the lm_head is not split: its epilogue
//     rounds the logits and takes the argmax directly);
//   * attention runs as split-KV items (request, kv head, chunk) on the CUDA cores like in the small-batch
//     kernels, followed by a log-sum-exp merge.
//
// One persistent cooperative launch per step; phases are separated by a counter-based grid barrier whose
// wait is bounded (status 9110 instead of a hang).  Rounding points are those of the small-batch kernels
// (HuggingFace eager); fp32 partial sums meet in a different order, which is within the parity tolerance.
//
// Behaviour of the reference's tensor-core code that was used as a map (nothing copied): descriptor fields
// and roles in prime_kernels/flash_moe/csrc/kernels/tcgen05_prelude.cuh:38-96,136-157,213-258 and
// fused_moe_bf16_kernel.cu:105-229; its waits are unbounded (tcgen05_prelude.cuh:404-414), these are not.
#pragma once

namespace pk {
namespace batched {

constexpr int kThreadsB = 256;        // warps 0-3: operand staging + epilogue; warp 4: MMA issue; all: SIMT phases
constexpr int kStages = 8;            // ring of staged 64-wide K blocks (A tile 16 KB + B tile NP x 128 bytes each)
constexpr int kDepth = 4;             // cp.async groups (K blocks) a producer thread keeps in flight
constexpr int kConv = 4;              // MXFP8 weights: de-quantised bf16 A slots (the raw bytes use a ring of kStages)
constexpr int kNcB = 32;              // max split-KV chunks per (request, kv head): one lane per chunk in the merge
constexpr int kMaxReq = 64;
constexpr int kAStage = 128 * 128;    // bytes of one A stage (128 rows x 64 bf16)
constexpr int kKvStages = 4;          // attention: runs of 16 positions in flight per warp
constexpr int kRunBytes = 16 * 256;   // K and V rows of one run
// the GEMM operand stages and the attention rings share the front of the dynamic shared memory
__host__ __device__ constexpr int staging_bytes(int np) {
    return kStages * kAStage + kStages * np * 128 > (kThreadsB / 32) * kKvStages * kRunBytes
               ? kStages * kAStage + kStages * np * 128
               : (kThreadsB / 32) * kKvStages * kRunBytes;
}

struct GemmDesc {
    int rows;            // weight rows (output features)
    int K;               // reduction length
    int widx;            // index in the per-layer pointer table, -1: embedding matrix
    int rowbytes;        // bytes per stored weight row
};

struct BParams {
    const unsigned long long* layers;   // device table [L][6]
    const unsigned long long* kv;       // device table [L]
    const unsigned char* embed;         // lm_head matrix (bf16 rows or packed MXFP8 rows)
    const uint16_t* embed_bf16;         // bf16 embedding rows for the input lookup
    const uint16_t* final_norm;
    const void* input_ids;
    const long long* positions;
    const int* seq_lens;
    const int* block_table;
    const long long* slot_mapping;
    const void* cos_sin;
    uint16_t* out_hidden;
    uint16_t* logits;
    long long* next_ids;
    uint16_t* layer_outputs;
    unsigned long long* profile;        // optional [ctas][L][kProfSlots] globaltimer stamps (thread 0, after every phase)
    unsigned int* ctrl;                 // control words shared with the other kernels (status)
    unsigned int* bctrl;                // this kernel's words: [0] barrier counter, [1] completion counter
    unsigned long long* argkey;         // [kMaxReq]
    float* c_qkv;                       // [NP][NQKV]   fp32 sums of the split-K partial tiles
    float* c_o;                         // [NP][H]
    float* c_gu;                        // [NP][2I]
    float* c_down;                      // [NP][H]
    uint16_t* x;                        // [NP][H]   residual stream (bf16)
    uint16_t* h1;                       // [NP][H]
    uint16_t* xn;                       // [NP][H]   normed input of the QKV / gate-up / lm_head GEMMs
    uint16_t* attn;                     // [NP][AD]
    uint16_t* act;                      // [NP][I]
    float* part;                        // [B][KVH][kNcB][G][66]
    long long k_off, v_off, block_stride, token_stride, head_stride;
    int block_size, bt_stride, ids_i64, cs_fp32;
    int bs_shift;                       // log2(block_size) when it is a power of two, else -1 (the run loop then divides)
    int H, I, L, QH, KVH, V, G, nb, wfmt, lm_head, advance, max_seq_len;
    unsigned spin_limit;
    float eps;
    GemmDesc gd[kNumPhaseTypes];
};

struct BShared {
    uint64_t full[kStages];      // 128 producer threads arrive
    uint64_t empty[kStages];     // tcgen05.commit arrives when the MMAs that read the stage have completed
    uint64_t accum;
    uint64_t kvbar[kThreadsB / 32][kKvStages];
    uint32_t tmem_base;
    volatile int abort_flag;
    uint32_t bar_gen;
    int seq[kMaxReq], pos[kMaxReq], nc[kMaxReq];
    long long tok[kMaxReq], slot_off[kMaxReq];
    int lc, ncmax;
    float red[8];
    unsigned long long lm_key[4][kMaxReq];
};

// ------------------------------------------------------------------ small helpers
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t n = valid ? 16u : 0u;      // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
// global -> shared bulk copy without a cache hint, completion counted in bytes on an mbarrier; never multicast
__device__ __forceinline__ void bulk_g2s_plain(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }

// K-major, 128-byte swizzle: start address, stride between eight-row groups = 1024 bytes, descriptor version 1
__device__ __forceinline__ uint64_t smem_desc_sw128(const void* p) {
    const uint64_t addr = smem_u32(p);
    return ((addr >> 4) & 0x3fffull) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// kind::f16: D = f32, A = B = bf16, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
    const uint32_t acc = accumulate ? 1u : 0u;
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
template <int NP>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, float (&v)[NP]);
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, float (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
          "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
        : "r"(taddr)
        : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<32>(uint32_t taddr, float (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
        "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
          "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]), "=f"(v[16]),
          "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]), "=f"(v[24]),
          "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
        : "r"(taddr)
        : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld<64>(uint32_t taddr, float (&v)[64]) {
    float a[32], b[32];
    tmem_ld<32>(taddr, a);
    tmem_ld<32>(taddr + 32u, b);
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = a[i];
        v[32 + i] = b[i];
    }
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct BC {
    const BParams& p;
    BShared& sh;
    unsigned char* stage_a;     // kStages x 16 KB, 1024-byte aligned
    unsigned char* stage_b;     // kStages x NP x 128 bytes (MXFP8 weights: followed by the raw ring, kStages x 8 KB)
    float* scratch;             // attention scratch (floats)
    int tid, warp, lane, cta, ncta;
    uint32_t uses;              // accumulator tiles finished so far (parity of the accumulator barrier)
    uint32_t prod, cons;        // K blocks this thread has produced / consumed so far (stage and parity of the ring)
    unsigned char* kvring;      // attention: kThreadsB/32 rings of kKvStages runs (over the GEMM stages)
    uint32_t kvi, kvc;          // runs this warp has issued / consumed so far (stage and parity of the ring)
};

__device__ __forceinline__ bool b_aborted(const BC& c) { return c.sh.abort_flag != 0; }
__device__ __forceinline__ void b_raise(BC& c, int code) {
    c.sh.abort_flag = 1;
    atomicCAS(c.p.ctrl + kCtrlStatus, 0u, (unsigned)code);
}
__device__ __forceinline__ bool b_wait_mbar(BC& c, uint64_t* bar, uint32_t parity) {
    if (mbar_probe(bar, parity)) return true;
    unsigned spins = 0;
    while (!mbar_test(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (b_aborted(c)) return false;
            if (spins >= c.p.spin_limit) {
                b_raise(c, kErrBarrierTimeout);
                return false;
            }
        }
    }
    return true;
}

// Grid barrier: every CTA adds one to a counter and waits until it reaches generation * grid size.  Global
// writes made before the barrier are visible to every CTA after it.  The wait is bounded; after a failure all
// later barriers fall through at once (the status word is checked first).
__device__ __forceinline__ void grid_barrier(BC& c) {
    __syncthreads();
    if (c.tid == 0) {
        const uint32_t target = (++c.sh.bar_gen) * (uint32_t)c.ncta;
        __threadfence();
        atomicAdd(c.p.bctrl, 1u);
        unsigned spins = 0;
        while (!b_aborted(c)) {
            uint32_t v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(c.p.bctrl) : "memory");
            if (v >= target) break;
            if ((++spins & 255u) == 0) {
                if (*((volatile unsigned int*)(c.p.ctrl + kCtrlStatus)) != 0) c.sh.abort_flag = 1;
                else if (spins >= c.p.spin_limit) b_raise(c, kErrBarrierTimeout);
            }
        }
    }
    __syncthreads();
}

// ------------------------------------------------------------------ tensor-core GEMM phase
// A phase is the flat sequence of (128-row tile, 64-wide K block) units of its weight matrix; CTA c owns the
// contiguous range [c U / n, (c+1) U / n), so every CTA streams the same number of weight bytes (+-1 block) and
// touches at most two or three row tiles.  Warps 0-3 produce (stage the operands of one K block per ring slot),
// lane 0 of warp 4 issues the MMAs and releases each slot with tcgen05.commit, warps 4-7 read a finished
// accumulator tile back (thread = weight row) and add it into the fp32 sums; the ring keeps the loads of the
// next tile going while a tile's epilogue runs.
__device__ __forceinline__ unsigned char* a_slot(BC& c, int st) { return c.stage_a + st * kAStage; }

// bf16 weights: 16-byte cp.async copies placed chunk by chunk in the swizzled layout.  Threads 0..127.
template <int NP>
__device__ __forceinline__ void stage_a_bf16(BC& c, int st, const unsigned char* wbase, int rowbytes, int r0, int nrows, int kblk) {
    unsigned char* sa = a_slot(c, st);
    const int t = c.tid;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        const int idx = t + u * 128;              // 128 rows x 8 chunks of 16 bytes
        const int row = idx >> 3, ch = idx & 7;
        const bool ok = r0 + row < nrows;
        const unsigned char* src = wbase + (size_t)(ok ? r0 + row : 0) * rowbytes + (size_t)kblk * 128 + ch * 16;
        cp_async16(sa + (row >> 3) * 1024 + (row & 7) * 128 + ((ch ^ (row & 7)) << 4), src, ok);
    }
}
// activations of one K block: NP rows x 128 bytes (requests >= nb are zero).  Threads 0..127.
template <int NP>
__device__ __forceinline__ void stage_b(BC& c, int st, const uint16_t* xmat, int xstride, int kblk) {
    unsigned char* sb = c.stage_b + st * NP * 128;
    const int t = c.tid;
#pragma unroll
    for (int u = 0; u < (NP * 8 + 127) / 128; ++u) {
        const int idx = t + u * 128;
        if (idx < NP * 8) {
            const int row = idx >> 3, ch = idx & 7;
            const bool ok = row < c.p.nb;
            const uint16_t* src = xmat + (size_t)(ok ? row : 0) * xstride + kblk * 64 + ch * 8;
            cp_async16(sb + (row >> 3) * 1024 + (row & 7) * 128 + ((ch ^ (row & 7)) << 4), src, ok);
        }
    }
}
// MXFP8 weights (rows [K e4m3][K/32 e8m0][pad]): a K block of a row is four 16-byte pieces.  Thread t owns pieces
// (row, pc) = ((t + 128 u) >> 2, (t + 128 u) & 3), u = 0..3: it copies them raw into the raw ring with cp.async
// (piece idx at byte 16 idx of the slot), keeps their E8M0 bytes in a register, and later de-quantises its own
// pieces (exact) into the swizzled bf16 tile - no other thread reads the raw ring.
__device__ __forceinline__ uint32_t copy_raw(BC& c, unsigned char* raw_slot, const unsigned char* wbase, int rowbytes, int K, int r0,
                                             int nrows, int kblk) {
    uint32_t scales = 0u;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int idx = c.tid + u * 128;
        const int row = idx >> 2, pc = idx & 3;
        const bool ok = r0 + row < nrows;
        const unsigned char* rp = wbase + (size_t)(ok ? r0 + row : 0) * rowbytes;
        cp_async16(raw_slot + idx * 16, rp + (size_t)kblk * 64 + pc * 16, ok);
        if (ok) scales |= (uint32_t)__ldg(rp + K + kblk * 2 + (pc >> 1)) << (8 * u);
    }
    return scales;
}
__device__ __forceinline__ void store_dequant(BC& c, unsigned char* sa, const unsigned char* raw_slot, uint32_t scales) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int idx = c.tid + u * 128;
        const int row = idx >> 2, pc = idx & 3;
        const uint32_t sbyte = (scales >> (8 * u)) & 0xffu;
        const float scale = __uint_as_float(sbyte ? (sbyte << 23) : 0x00400000u);
        const uint4 q = *reinterpret_cast<const uint4*>(raw_slot + idx * 16);
        uint4 lo, hi;
        float f[4];
        e4m3x4_to_f32(q.x, f);
        lo.x = pack_bf16x2(f[0] * scale, f[1] * scale); lo.y = pack_bf16x2(f[2] * scale, f[3] * scale);
        e4m3x4_to_f32(q.y, f);
        lo.z = pack_bf16x2(f[0] * scale, f[1] * scale); lo.w = pack_bf16x2(f[2] * scale, f[3] * scale);
        e4m3x4_to_f32(q.z, f);
        hi.x = pack_bf16x2(f[0] * scale, f[1] * scale); hi.y = pack_bf16x2(f[2] * scale, f[3] * scale);
        e4m3x4_to_f32(q.w, f);
        hi.z = pack_bf16x2(f[0] * scale, f[1] * scale); hi.w = pack_bf16x2(f[2] * scale, f[3] * scale);
        unsigned char* rowp = sa + (row >> 3) * 1024 + (row & 7) * 128;
        *reinterpret_cast<uint4*>(rowp + (((2 * pc) ^ (row & 7)) << 4)) = lo;
        *reinterpret_cast<uint4*>(rowp + (((2 * pc + 1) ^ (row & 7)) << 4)) = hi;
    }
}

// producers, bf16 weights: up to kDepth cp.async groups in flight per thread; a slot is published (proxy fence +
// arrive) when its group has landed
template <int NP>
__device__ void gemm_produce_bf16(BC& c, const GemmDesc& gd, const unsigned char* wbase, const uint16_t* xmat, int g0, int g1, int nk64) {
    BShared& sh = c.sh;
    int inflight = 0;
    for (int g = g0; g < g1; ++g) {
        const int rt = g / nk64, kb = g - rt * nk64;
        const int st = (int)(c.prod % kStages);
        if (!b_wait_mbar(c, &sh.empty[st], ((c.prod / kStages) & 1u) ^ 1u)) break;
        stage_a_bf16<NP>(c, st, wbase, gd.rowbytes, rt * 128, gd.rows, kb);
        stage_b<NP>(c, st, xmat, gd.K, kb);
        cp_async_commit();
        ++c.prod;
        if (++inflight == kDepth) {
            cp_async_wait<kDepth - 1>();
            fence_async_smem();
            mbar_arrive(&sh.full[(c.prod - kDepth) % kStages]);
            --inflight;
        }
    }
    while (inflight > 0) {
        switch (inflight - 1) {
            case 3: cp_async_wait<3>(); break;
            case 2: cp_async_wait<2>(); break;
            case 1: cp_async_wait<1>(); break;
            default: cp_async_wait<0>(); break;
        }
        fence_async_smem();
        mbar_arrive(&sh.full[(c.prod - inflight) % kStages]);
        --inflight;
    }
}
// producers, MXFP8 weights: raw pieces and activations of the next kDepth K blocks are in flight (cp.async into the
// raw ring / the B ring, kStages slots each) while the current block is de-quantised into one of the kConv bf16
// A slots.  B slot of block n + kDepth is rewritten after the MMAs of block n - kConv have completed (the
// empty-wait of block n), and kDepth + kConv <= kStages.
template <int NP>
__device__ void gemm_produce_mxfp8(BC& c, const GemmDesc& gd, const unsigned char* wbase, const uint16_t* xmat, int g0, int g1, int nk64) {
    BShared& sh = c.sh;
    static_assert(kDepth == 4 && kDepth + kConv <= kStages, "ring arithmetic");
    unsigned char* raw = c.stage_b + kStages * NP * 128;
    uint32_t sc0 = 0u, sc1 = 0u, sc2 = 0u, sc3 = 0u;
    auto issue = [&](int g, int ahead) -> uint32_t {
        const int slot = (int)((c.prod + (uint32_t)ahead) % kStages);
        const uint32_t scales = copy_raw(c, raw + slot * (kAStage / 2), wbase, gd.rowbytes, gd.K, (g / nk64) * 128, gd.rows, g % nk64);
        stage_b<NP>(c, slot, xmat, gd.K, g % nk64);
        cp_async_commit();
        return scales;
    };
    if (g0 < g1) sc0 = issue(g0, 0);
    if (g0 + 1 < g1) sc1 = issue(g0 + 1, 1);
    if (g0 + 2 < g1) sc2 = issue(g0 + 2, 2);
    if (g0 + 3 < g1) sc3 = issue(g0 + 3, 3);
#pragma unroll 1
    for (int g = g0; g < g1; ++g) {
        switch (min(kDepth - 1, g1 - 1 - g)) {      // groups issued after block g's
            case 3: cp_async_wait<3>(); break;
            case 2: cp_async_wait<2>(); break;
            case 1: cp_async_wait<1>(); break;
            default: cp_async_wait<0>(); break;
        }
        const int cs = (int)(c.prod % kConv);
        if (!b_wait_mbar(c, &sh.empty[cs], ((c.prod / kConv) & 1u) ^ 1u)) break;
        store_dequant(c, a_slot(c, cs), raw + (c.prod % kStages) * (kAStage / 2), sc0);
        fence_async_smem();
        mbar_arrive(&sh.full[cs]);
        ++c.prod;
        sc0 = sc1;
        sc1 = sc2;
        sc2 = sc3;
        if (g + kDepth < g1) sc3 = issue(g + kDepth, kDepth - 1);
    }
    cp_async_wait<0>();
}

// `mode` 0: partial tiles are added into cmat ([NP][rows] fp32); mode 1 (lm_head, whole row tiles per CTA): bf16
// logits and the per-request argmax.
template <int NP, int WF>
__device__ void gemm_phase(BC& c, const GemmDesc& gd, const unsigned char* wbase, const uint16_t* xmat, float* cmat, int mode) {
    const BParams& p = c.p;
    BShared& sh = c.sh;
    const int rtiles = (gd.rows + 127) / 128;
    const int nk64 = gd.K / 64;
    int g0, g1;
    if (mode == 1) {
        g0 = (int)((long long)c.cta * rtiles / c.ncta) * nk64;
        g1 = (int)((long long)(c.cta + 1) * rtiles / c.ncta) * nk64;
    } else {
        const long long units = (long long)rtiles * nk64;
        g0 = (int)(units * c.cta / c.ncta);
        g1 = (int)(units * (c.cta + 1) / c.ncta);
    }
    if (mode == 1 && c.tid < 4 * kMaxReq) (&sh.lm_key[0][0])[c.tid] = 0ull;
    if (mode == 1) __syncthreads();
    if (c.warp < 4) {
        if (WF == 0) gemm_produce_bf16<NP>(c, gd, wbase, xmat, g0, g1, nk64);
        else gemm_produce_mxfp8<NP>(c, gd, wbase, xmat, g0, g1, nk64);
    } else {
        const uint32_t idesc = idesc_bf16(128, NP);
        const int q4 = c.warp - 4;                 // this warp's quarter of the tensor-memory lanes
        int g = g0;
        while (g < g1) {
            const int rt = g / nk64;
            const int gend = min(g1, (rt + 1) * nk64);
            if (c.warp == 4 && c.lane == 0) {
                for (int q = g; q < gend; ++q) {
                    constexpr int kARing = WF ? kConv : kStages;
                    const int st = (int)(c.cons % kARing);
                    if (!b_wait_mbar(c, &sh.full[st], (c.cons / kARing) & 1u)) break;
                    tc_fence_after();
                    const uint64_t da = smem_desc_sw128(a_slot(c, st));
                    const uint64_t db = smem_desc_sw128(c.stage_b + (c.cons % kStages) * NP * 128);
#pragma unroll
                    for (int k = 0; k < 4; ++k)      // 16 bf16 = 32 bytes per instruction: start address + 2 (16-byte units)
                        mma_bf16(sh.tmem_base, da + 2 * k, db + 2 * k, idesc, q > g || k > 0);
                    mma_commit(&sh.empty[st]);       // the slot is free when these MMAs have read it
                    ++c.cons;
                }
                mma_commit(&sh.accum);               // arrives when every MMA issued so far has completed
            }
            __syncwarp();
            b_wait_mbar(c, &sh.accum, c.uses & 1u);
            ++c.uses;
            tc_fence_after();
            float v[NP];
            tmem_ld<NP>(sh.tmem_base + ((uint32_t)(q4 * 32) << 16), v);
            tmem_ld_wait();
            tc_fence_before();
            asm volatile("bar.sync 2, 128;" ::: "memory");      // all four quarters are read: the next tile may start
            const int row = rt * 128 + q4 * 32 + c.lane;
            if (mode == 0) {
                if (row < gd.rows && !b_aborted(c)) {
#pragma unroll
                    for (int j = 0; j < NP; ++j)
                        if (j < p.nb) atomicAdd(cmat + (size_t)j * gd.rows + row, v[j]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < NP; ++j) {
                    if (j < p.nb) {
                        const uint32_t lb = f32_to_bf16_bits(v[j]);
                        unsigned long long key = 0ull;
                        if (row < gd.rows) {
                            if (p.logits) p.logits[(size_t)j * gd.rows + row] = (uint16_t)lb;
                            const uint32_t ord = (lb & 0x8000u) ? (~lb & 0xffffu) : (lb | 0x8000u);
                            key = ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - (uint32_t)row);
                        }
#pragma unroll
                        for (int off = 16; off >= 1; off >>= 1) {
                            const unsigned long long o = __shfl_xor_sync(kFullMask, key, off);
                            key = o > key ? o : key;
                        }
                        if (c.lane == 0 && key > sh.lm_key[q4][j]) sh.lm_key[q4][j] = key;
                    }
                }
            }
            g = gend;
        }
    }
    if (mode == 1 && p.next_ids) {
        __syncthreads();
        if (c.tid < p.nb) {
            unsigned long long k = sh.lm_key[0][c.tid];
#pragma unroll
            for (int w = 1; w < 4; ++w) k = sh.lm_key[w][c.tid] > k ? sh.lm_key[w][c.tid] : k;
            if (k) atomicMax(p.argkey + c.tid, k);
        }
    }
}

// ------------------------------------------------------------------ SIMT phases between the GEMMs
// Residual add + RMSNorm of whole rows: request b is handled by one CTA.
//   which 0: x = embedding row (layer 0)            -> xn = norm(x, w)
//   which 1: x = bf16(h1 + bf16(c_down))            -> xn = norm(x, w)   (also layer_outputs, final hidden)
//   which 2: h1 = bf16(x + bf16(c_o))               -> xn = norm(h1, w)
__device__ void norm_phase(BC& c, int which, int layer, const uint16_t* weight, bool write_hidden) {
    const BParams& p = c.p;
    BShared& sh = c.sh;
    const int H = p.H, H8 = H >> 3;           // a thread handles 8 consecutive elements at a time
    for (int b = c.cta; b < p.nb; b += c.ncta) {
        float ss = 0.f;
        float* row = c.scratch;               // H floats
        for (int i8 = c.tid; i8 < H8; i8 += kThreadsB) {
            const size_t off = (size_t)b * H + 8 * i8;
            float v[8];
            uint4 bits;
            if (which == 0) {
                bits = __ldg(reinterpret_cast<const uint4*>(p.embed_bf16 + (size_t)sh.tok[b] * H + 8 * i8));
                const uint32_t w[4] = {bits.x, bits.y, bits.z, bits.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    v[2 * k] = bf16_lo(w[k]);
                    v[2 * k + 1] = bf16_hi(w[k]);
                }
                *reinterpret_cast<uint4*>(p.x + off) = bits;
            } else {
                // which 1: x = bf16(h1 + bf16(c_down));  which 2: h1 = bf16(x + bf16(c_o))
                float* sums = (which == 1 ? p.c_down : p.c_o) + off;
                const uint4 rb = __ldcg(reinterpret_cast<const uint4*>((which == 1 ? p.h1 : p.x) + off));
                const float4 s0 = __ldcg(reinterpret_cast<const float4*>(sums));
                const float4 s1 = __ldcg(reinterpret_cast<const float4*>(sums) + 1);
                const uint32_t w[4] = {rb.x, rb.y, rb.z, rb.w};
                const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                uint32_t o[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    v[2 * k] = round_bf16(__fadd_rn(bf16_lo(w[k]), round_bf16(sv[2 * k])));
                    v[2 * k + 1] = round_bf16(__fadd_rn(bf16_hi(w[k]), round_bf16(sv[2 * k + 1])));
                    o[k] = (__float_as_uint(v[2 * k]) >> 16) | (__float_as_uint(v[2 * k + 1]) & 0xffff0000u);
                }
                bits = make_uint4(o[0], o[1], o[2], o[3]);
                reinterpret_cast<float4*>(sums)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
                reinterpret_cast<float4*>(sums)[1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (which == 1) {
                    *reinterpret_cast<uint4*>(p.x + off) = bits;
                    if (p.layer_outputs) *reinterpret_cast<uint4*>(p.layer_outputs + ((size_t)(layer - 1) * p.nb + b) * H + 8 * i8) = bits;
                } else {
                    *reinterpret_cast<uint4*>(p.h1 + off) = bits;
                }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                row[8 * i8 + k] = v[k];
                ss = fmaf(v[k], v[k], ss);
            }
        }
        ss = warp_sum(ss);
        if (c.lane == 0) sh.red[c.warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kThreadsB / 32; ++w) tot += sh.red[w];
        const float s = rsqrtf(tot * (1.f / (float)H) + p.eps);
        for (int i8 = c.tid; i8 < H8; i8 += kThreadsB) {
            const uint4 wb = __ldg(reinterpret_cast<const uint4*>(weight) + i8);
            const uint32_t w[4] = {wb.x, wb.y, wb.z, wb.w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float n0 = round_bf16(__fmul_rn(row[8 * i8 + 2 * k], s));
                const float n1 = round_bf16(__fmul_rn(row[8 * i8 + 2 * k + 1], s));
                o[k] = pack_bf16x2(__fmul_rn(n0, bf16_lo(w[k])), __fmul_rn(n1, bf16_hi(w[k])));
            }
            const uint4 ob = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(p.xn + (size_t)b * H + 8 * i8) = ob;
            if (write_hidden) *reinterpret_cast<uint4*>(p.out_hidden + (size_t)b * H + 8 * i8) = ob;
        }
        __syncthreads();
    }
    if (which == 2) {
        // the q / k / v sums were consumed by the attention items two barriers ago: clear them for the next layer
        // (the CTAs without a row to normalise do most of it)
        const int total4 = p.nb * (p.QH + 2 * p.KVH) * (kD / 4);
        for (int e = c.cta * kThreadsB + c.tid; e < total4; e += c.ncta * kThreadsB)
            reinterpret_cast<float4*>(p.c_qkv)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// act = bf16( bf16(silu(bf16 gate)) * bf16 up ) over [nb][I]; clears the gate/up sums.  Four elements per thread
// and step, two steps' loads in flight.
__device__ void swiglu_phase(BC& c) {
    const BParams& p = c.p;
    const int I4 = p.I >> 2;
    const int total = p.nb * I4;
    const int stride = c.ncta * kThreadsB;
    auto fetch = [&](int e, float4& g, float4& u) {
        const int b = e / I4, j4 = e - b * I4;
        const float4* gp = reinterpret_cast<const float4*>(p.c_gu + (size_t)b * 2 * p.I) + j4;
        g = __ldcg(gp);
        u = __ldcg(gp + I4);
    };
    auto finish = [&](int e, const float4& g, const float4& u) {
        const int b = e / I4, j4 = e - b * I4;
        float4* gp = reinterpret_cast<float4*>(p.c_gu + (size_t)b * 2 * p.I) + j4;
        gp[0] = make_float4(0.f, 0.f, 0.f, 0.f);
        gp[I4] = make_float4(0.f, 0.f, 0.f, 0.f);
        const float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {u.x, u.y, u.z, u.w};
        float a[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gr = round_bf16(gv[k]);
            const float silu = round_bf16(__fdividef(gr, 1.f + __expf(-gr)));
            a[k] = __fmul_rn(silu, round_bf16(uv[k]));
        }
        *reinterpret_cast<uint2*>(p.act + (size_t)b * p.I + 4 * j4) = make_uint2(pack_bf16x2(a[0], a[1]), pack_bf16x2(a[2], a[3]));
    };
    for (int e = c.cta * kThreadsB + c.tid; e < total; e += 2 * stride) {
        float4 g0, u0, g1 = make_float4(0.f, 0.f, 0.f, 0.f), u1 = g1;
        fetch(e, g0, u0);
        const bool two = e + stride < total;
        if (two) fetch(e + stride, g1, u1);
        finish(e, g0, u0);
        if (two) finish(e + stride, g1, u1);
    }
}

// Split-KV attention item: one WARP, (request b, kv head, chunk), no CTA-wide synchronisation.  The K and V rows
// of a run of 16 positions are brought into the warp's shared-memory ring by bulk copies (one 4 KB copy per run
// where a block's K and V rows are adjacent, else one 128-byte copy per row) that complete on the run's
// mbarrier; kKvStages runs are in flight per warp, so eight warps keep about 100 KB per SM outstanding, which is
// what the HBM latency-bandwidth product asks for.  Scores: lane = (position, half of the head dim), 16-byte
// chunks read in an order rotated by the position so that the 256-byte row stride does not collide on banks;
// P.V: lane = two output dims.  The prologue rounds this head group's q / k / v sums to bf16, rotates q and k
// (lane j owns dims j and j + 32, HF rounding) and appends the new token, whose row is patched into the staged
// run instead of being read back.
template <int G>
__device__ void attention_item_b(BC& c, int layer, int b, int kvh, int chunk) {
    const BParams& p = c.p;
    BShared& sh = c.sh;
    const int lane = c.lane;
    const int seq = sh.seq[b], pos = sh.pos[b];
    const int ws = chunk * sh.lc;
    const int we = min(ws + sh.lc, seq);
    const int wcopy = (we == seq) ? seq - 1 : we;      // position seq-1 is this step's token: never read from the cache
    const int nruns = (we - ws + 15) >> 4;
    const uint16_t* kvr = reinterpret_cast<const uint16_t*>(__ldg(p.kv + layer));
    const long long hs = (long long)kvh * p.head_stride;
    const int pl = lane >> 1, half = lane & 1;
    const int nqkv = (p.QH + 2 * p.KVH) * kD;
    // per-warp shared memory: packed bf16 q (G heads, rotated), k (rotated), v; probabilities of a run
    uint32_t* qkvb_s = reinterpret_cast<uint32_t*>(c.scratch) + c.warp * ((G + 2) * 32 + G * 16);
    float* prob_s = reinterpret_cast<float*>(qkvb_s + (G + 2) * 32);
    unsigned char* ring = c.kvring + (size_t)c.warp * (kKvStages * kRunBytes);
    uint64_t* bars = sh.kvbar[c.warp];

    // a window of 32 block-table entries, one per lane, refreshed as the runs move along
    const int* bt = p.block_table + (size_t)b * p.bt_stride;
    const int bs = p.block_size, bsh = p.bs_shift;
    // position -> (block-table index, position inside the block): shifts for the usual power-of-two block sizes
    auto blk_of = [&](int pos) { return bsh >= 0 ? (pos >> bsh) : pos / bs; };
    auto in_blk = [&](int pos) { return bsh >= 0 ? (pos & (bs - 1)) : pos % bs; };
    int bt_base = blk_of(ws);
    int btc = __ldg(bt + min(bt_base + lane, p.bt_stride - 1));
    const bool packed = p.token_stride == 2 * kD && p.v_off == p.k_off + kD;
    auto issue = [&](int r0) {
        const int st = (int)(c.kvi % kKvStages);
        const int n = max(0, min(16, wcopy - r0));
        if (blk_of(r0 + 15) >= bt_base + 32) {
            bt_base = blk_of(r0);
            btc = __ldg(bt + min(bt_base + lane, p.bt_stride - 1));
        }
        const int j = lane & 15, pj = r0 + j, pin = in_blk(pj);
        const int blk = __shfl_sync(kFullMask, btc, (blk_of(pj) - bt_base) & 31);
        if (lane == 0) mbar_expect_tx(&bars[st], (uint32_t)n * 256u);      // n == 0: the phase completes at once
        __syncwarp();
        unsigned char* dst = ring + st * kRunBytes + j * 256;
        const long long e = (long long)blk * p.block_stride + (long long)pin * p.token_stride + hs;
        if (packed) {
            // one copy per piece of a block: lane j starts a piece when position j is the first of the run or of a block
            if (lane < 16 && j < n && (j == 0 || pin == 0))
                bulk_g2s_plain(dst, kvr + p.k_off + e, (uint32_t)min(bs - pin, n - j) * 256u, &bars[st]);
        } else if (j < n) {
            const bool isv = lane >= 16;
            bulk_g2s_plain(dst + (isv ? 128 : 0), kvr + (isv ? p.v_off : p.k_off) + e, 128u, &bars[st]);
        }
        ++c.kvi;
    };
    fence_async_smem();      // the previous item's generic writes to the ring (patched rows) before new bulk copies
    for (int k = 0; k < min(nruns, kKvStages); ++k) issue(ws + 16 * k);      // in flight during the prologue

    // ---- prologue: q (G heads), k, v of the new token; lane j owns dims j and j + 32
    {
        float cs, sn;
        if (p.cs_fp32) {
            cs = __ldg(reinterpret_cast<const float*>(p.cos_sin) + (size_t)pos * kD + lane);
            sn = __ldg(reinterpret_cast<const float*>(p.cos_sin) + (size_t)pos * kD + 32 + lane);
        } else {
            cs = __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.cos_sin) + (size_t)pos * kD + lane) << 16);
            sn = __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.cos_sin) + (size_t)pos * kD + 32 + lane) << 16);
        }
        uint16_t* q16 = reinterpret_cast<uint16_t*>(qkvb_s);
#pragma unroll
        for (int which = 0; which < G + 2; ++which) {
            const int row = which < G ? (kvh * G + which) * kD : (which == G ? (p.QH + kvh) * kD : (p.QH + p.KVH + kvh) * kD);
            const float* src = p.c_qkv + (size_t)b * nqkv + row;
            float x0 = round_bf16(__ldcg(src + lane)), x1 = round_bf16(__ldcg(src + 32 + lane));   // projection output dtype
            if (which <= G) {
                const float y0 = rope_elem(x0, x1, cs, sn, true);
                x1 = rope_elem(x1, x0, cs, sn, false);
                x0 = y0;
            }
            q16[which * kD + lane] = (uint16_t)f32_to_bf16_bits(x0);
            q16[which * kD + 32 + lane] = (uint16_t)f32_to_bf16_bits(x1);
        }
    }
    __syncwarp();
    if (we == seq && lane < 16 && sh.slot_off[b] >= 0) {      // this chunk holds position seq-1: append K/V
        uint16_t* kvw = const_cast<uint16_t*>(kvr);
        const int l8 = lane & 7;
        const long long e = sh.slot_off[b] + hs + 8 * l8;
        if (lane < 8) *reinterpret_cast<uint4*>(kvw + p.k_off + e) = *reinterpret_cast<const uint4*>(qkvb_s + G * 32 + 4 * l8);
        else *reinterpret_cast<uint4*>(kvw + p.v_off + e) = *reinterpret_cast<const uint4*>(qkvb_s + (G + 1) * 32 + 4 * l8);
    }

    float m[G], l[G], acc[G][2];
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        m[hh] = -INFINITY;
        l[hh] = 0.f;
        acc[hh][0] = acc[hh][1] = 0.f;
    }
    // this lane's half of every query head, in the lane's (rotated) chunk order: loop-invariant, kept in registers
    uint4 qreg[G][4];
#pragma unroll
    for (int hh = 0; hh < G; ++hh)
#pragma unroll
        for (int i = 0; i < 4; ++i)
            qreg[hh][i] = *reinterpret_cast<const uint4*>(qkvb_s + hh * 32 + 16 * half + 4 * ((i + pl) & 3));
    bool alive = true;
#pragma unroll 1
    for (int k = 0; k < nruns; ++k) {
        const int r0 = ws + 16 * k;
        const int st = (int)(c.kvc % kKvStages);
        // after a failed wait the remaining runs are still waited for (each wait bounded), nothing is computed
        alive = b_wait_mbar(c, &bars[st], (c.kvc / kKvStages) & 1u) && alive;
        unsigned char* data = ring + st * kRunBytes;
        if (alive) {
        if (we == seq && seq - 1 >= r0 && seq - 1 < r0 + 16) {      // the new token's row, from the prologue
            uint32_t* rowp = reinterpret_cast<uint32_t*>(data + (seq - 1 - r0) * 256);
            rowp[lane] = qkvb_s[G * 32 + lane];
            rowp[32 + lane] = qkvb_s[(G + 1) * 32 + lane];
            __syncwarp();
        }
        const int pp = r0 + pl;
        const bool valid = pp < we;
        float d0[G], d1[G];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) d0[hh] = d1[hh] = 0.f;
        const unsigned char* krow = data + pl * 256 + half * 64;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int ii = (i + pl) & 3;
            const uint4 k4 = *reinterpret_cast<const uint4*>(krow + ii * 16);
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                const uint4 q4 = qreg[hh][i];
                d0[hh] = fma2_bf16(k4.x, q4.x, d0[hh]);
                d1[hh] = fma2_bf16(k4.y, q4.y, d1[hh]);
                d0[hh] = fma2_bf16(k4.z, q4.z, d0[hh]);
                d1[hh] = fma2_bf16(k4.w, q4.w, d1[hh]);
            }
        }
        float sc[G], mx[G], pr[G];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            sc[hh] = d0[hh] + d1[hh];
            sc[hh] += __shfl_xor_sync(kFullMask, sc[hh], 1);
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            sc[hh] = valid ? round_bf16(sc[hh]) * 0.125f : -INFINITY;    // bf16 matmul output, exact 1/8 scale
            int key = __float_as_int(sc[hh]);
            key ^= (key >> 31) & 0x7fffffff;
            key = __reduce_max_sync(kFullMask, key);
            mx[hh] = __int_as_float(key ^ ((key >> 31) & 0x7fffffff));
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            const float mn = fmaxf(m[hh], mx[hh]);
            const float alpha = (mn == -INFINITY) ? 1.f : __expf(m[hh] - mn);
            pr[hh] = (sc[hh] == -INFINITY) ? 0.f : __expf(sc[hh] - mn);
            m[hh] = mn;
            l[hh] = l[hh] * alpha + (half == 0 ? pr[hh] : 0.f);
            acc[hh][0] *= alpha;
            acc[hh][1] *= alpha;
            if (half == 0) prob_s[hh * 16 + pl] = pr[hh];
        }
        __syncwarp();
        const int jn = we - r0;               // positions of this run that exist (the rest of the stage is stale)
        float a0[G], a1[G];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            a0[hh] = acc[hh][0];
            a1[hh] = acc[hh][1];
        }
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
            uint32_t v[4];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int j = 4 * j4 + jj;
                v[jj] = *reinterpret_cast<const uint32_t*>(data + j * 256 + 128 + lane * 4);
                if (j >= jn) v[jj] = 0u;
            }
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                const float4 p4 = *reinterpret_cast<const float4*>(prob_s + hh * 16 + 4 * j4);
                a0[hh] = fmaf(p4.x, bf16_lo(v[0]), a0[hh]); a1[hh] = fmaf(p4.x, bf16_hi(v[0]), a1[hh]);
                a0[hh] = fmaf(p4.y, bf16_lo(v[1]), a0[hh]); a1[hh] = fmaf(p4.y, bf16_hi(v[1]), a1[hh]);
                a0[hh] = fmaf(p4.z, bf16_lo(v[2]), a0[hh]); a1[hh] = fmaf(p4.z, bf16_hi(v[2]), a1[hh]);
                a0[hh] = fmaf(p4.w, bf16_lo(v[3]), a0[hh]); a1[hh] = fmaf(p4.w, bf16_hi(v[3]), a1[hh]);
            }
        }
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            acc[hh][0] = a0[hh];
            acc[hh][1] = a1[hh];
        }
        }
        __syncwarp();                          // every lane is done with the stage before it is refilled
        ++c.kvc;
        if (k + kKvStages < nruns) issue(ws + 16 * (k + kKvStages));
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
        for (int hh = 0; hh < G; ++hh) l[hh] += __shfl_xor_sync(kFullMask, l[hh], off);
    if (sh.ncmax == 1) {
        // every request of the step is a single chunk: the item's result is final (what the merge would compute
        // from one partial), and the step runs without the merge phase and its barrier
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            const float inv = 1.f / l[hh];
            reinterpret_cast<uint32_t*>(p.attn + (size_t)b * p.QH * kD + (kvh * G + hh) * kD)[lane] =
                pack_bf16x2(acc[hh][0] * inv, acc[hh][1] * inv);
        }
        __syncwarp();
        return;
    }
    float* part = p.part + ((size_t)(b * p.KVH + kvh) * kNcB + chunk) * G * 66;
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        float* dst = part + hh * 66;
        if (lane == 0) {
            dst[0] = m[hh];
            dst[1] = l[hh];
        }
        *reinterpret_cast<float2*>(dst + 2 + 2 * lane) = make_float2(acc[hh][0], acc[hh][1]);
    }
    __syncwarp();
}

// log-sum-exp merge of the chunk partials: one warp per (request, query head); bf16 output into attn[b][hq*64 + d]
__device__ void merge_phase(BC& c) {
    const BParams& p = c.p;
    BShared& sh = c.sh;
    const int G = p.G, lane = c.lane;
    const int gw = c.cta * (kThreadsB / 32) + c.warp, nw = c.ncta * (kThreadsB / 32);
    for (int t = gw; t < p.nb * p.QH; t += nw) {
        const int b = t / p.QH, hq = t - b * p.QH;
        const int kvh = hq / G, g = hq - kvh * G;
        const int nc = sh.nc[b];
        const float* part = p.part + ((size_t)(b * p.KVH + kvh) * kNcB * G + g) * 66;
        const size_t cs = (size_t)G * 66;
        const float mc = lane < nc ? __ldcg(part + lane * cs) : -INFINITY;
        const float lc = lane < nc ? __ldcg(part + lane * cs + 1) : 0.f;
        const float M = warp_max(mc);
        const float wc = __expf(mc - M);
        const float den = warp_sum(lc * wc);
        float a0 = 0.f, a1 = 0.f;
        for (int ch = 0; ch < nc; ++ch) {
            const float wgt = __shfl_sync(kFullMask, wc, ch);
            const float2 a = __ldcg(reinterpret_cast<const float2*>(part + ch * cs + 2) + lane);
            a0 = fmaf(wgt, a.x, a0);
            a1 = fmaf(wgt, a.y, a1);
        }
        const float inv = 1.f / den;
        reinterpret_cast<uint32_t*>(p.attn + (size_t)b * p.QH * kD + hq * kD)[lane] = pack_bf16x2(a0 * inv, a1 * inv);
    }
}

// ------------------------------------------------------------------ the kernel
template <int NP, int G, int WF>
__global__ void __launch_bounds__(kThreadsB, 1) decode_batched_kernel(const BParams p) {
    extern __shared__ __align__(128) unsigned char smem_dyn[];
    // layout: A stages (1024-byte aligned: the swizzle pattern repeats every 1024 bytes), B stages, shared struct,
    // scratch floats; the launcher asks for 1024 bytes more than the sum so the base can be rounded up
    unsigned char* smem_raw = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char* stage_a = smem_raw;
    unsigned char* stage_b = stage_a + (WF ? kConv : kStages) * kAStage;      // MXFP8: bf16 A slots, B ring, raw ring
    BShared& sh = *reinterpret_cast<BShared*>(stage_a + staging_bytes(NP));
    float* scratch = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(&sh) + ((sizeof(BShared) + 127) & ~size_t(127)));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    BC c{p, sh, stage_a, stage_b, scratch, tid, warp, lane, (int)blockIdx.x, (int)gridDim.x, 0u, 0u, 0u, stage_a, 0u, 0u};

    if (tid == 0) {
        sh.abort_flag = (p.ctrl[kCtrlStatus] != 0u) ? 1 : 0;
        sh.bar_gen = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sh.full[s], 128);
            mbar_init(&sh.empty[s], 1);
        }
        mbar_init(&sh.accum, 1);
        for (int w = 0; w < kThreadsB / 32; ++w)
            for (int s = 0; s < kKvStages; ++s) mbar_init(&sh.kvbar[w][s], 1);
        int smax = 1;
        for (int b = 0; b < p.nb; ++b) {
            if (p.seq_lens[b] > p.max_seq_len) {
                sh.abort_flag = 1;
                atomicCAS(p.ctrl + kCtrlStatus, 0u, (unsigned)kErrMaxSeq);
            }
            smax = max(smax, min(max(p.seq_lens[b], 1), p.max_seq_len));
        }
        // chunks per (request, kv head): the split that minimises rounds x (runs per item + a prologue's worth),
        // counted for the longest request; at most kNcB chunks, at least 64 positions each.  With one chunk the
        // items write the final attention output and the merge phase is skipped.
        const int units = p.nb * p.KVH, nwarps = (int)gridDim.x * (kThreadsB / 32);
        int lc = 64;
        long long best = -1;
        for (int nc = 1; nc <= kNcB; ++nc) {
            const int l = max(64, (((smax + nc - 1) / nc) + 15) & ~15);
            const int ncr = (smax + l - 1) / l;
            const long long rounds = ((long long)units * ncr + nwarps - 1) / nwarps;
            // more than one chunk adds the merge phase and its grid barrier (about eight runs' worth of time)
            const long long cost = rounds * (l / 16 + 3) + (ncr > 1 ? 8 : 0);
            if (best < 0 || cost < best) {
                best = cost;
                lc = l;
            }
        }
        sh.lc = lc;
        sh.ncmax = (smax + lc - 1) / lc;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    if (tid < p.nb) {
        const int seq = min(max(p.seq_lens[tid], 1), p.max_seq_len);
        sh.seq[tid] = seq;
        sh.pos[tid] = (int)max(p.positions[tid], 0LL);
        sh.nc[tid] = (seq + sh.lc - 1) / sh.lc;
        const long long tok = p.ids_i64 ? reinterpret_cast<const long long*>(p.input_ids)[tid]
                                        : (long long)reinterpret_cast<const int*>(p.input_ids)[tid];
        sh.tok[tid] = tok < 0 ? 0 : (tok >= p.V ? p.V - 1 : tok);
        const long long slot = p.slot_mapping[tid];
        sh.slot_off[tid] = slot < 0 ? -1 : (slot / p.block_size) * p.block_stride + (slot % p.block_size) * p.token_stride;
    }
    if (warp == 4) {
        // tensor memory for one accumulator tile: 128 lanes x NP fp32 columns (allocation unit: power of two >= 32)
        const uint32_t ncols = NP < 32 ? 32u : (uint32_t)NP;
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh.tmem_base)), "r"(ncols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (c.cta == 0 && tid < p.nb) p.argkey[tid] = 0ull;

    auto wptr = [&](int layer, int widx) { return reinterpret_cast<const unsigned char*>(__ldg(p.layers + layer * 6 + widx)); };
    // stamps: slot 2k = the CTA's own work of phase k done, slot 2k+1 = the grid barrier behind it passed
    int slot = 0;
    unsigned long long* prof = nullptr;
    auto stamp = [&]() {
        if (prof && slot < kProfSlots) prof[slot] = global_ns();
        ++slot;
    };
    auto sync_phase = [&]() {
        stamp();
        grid_barrier(c);
        stamp();
    };
    for (int layer = 0; layer < p.L; ++layer) {
        prof = (p.profile && tid == 0) ? p.profile + ((size_t)c.cta * p.L + layer) * kProfSlots : nullptr;
        slot = 0;
        stamp();
        norm_phase(c, layer == 0 ? 0 : 1, layer, reinterpret_cast<const uint16_t*>(wptr(layer, 0)), false);
        sync_phase();
        gemm_phase<NP, WF>(c, p.gd[kQKV], wptr(layer, 1), p.xn, p.c_qkv, 0);
        sync_phase();
        {
            // attention items (chunk, request, kv head), chunk-major, dealt to the warps of the grid
            const int nslots = sh.ncmax * p.nb * p.KVH;
            const int nwarps = c.ncta * (kThreadsB / 32);
            for (int s = c.warp * c.ncta + c.cta; s < nslots; s += nwarps) {
                const int kvh = s % p.KVH, rest = s / p.KVH;
                const int b = rest % p.nb, chunk = rest / p.nb;
                if (chunk >= sh.nc[b]) continue;
                attention_item_b<G>(c, layer, b, kvh, chunk);
            }
        }
        sync_phase();
        if (sh.ncmax > 1) {
            merge_phase(c);
            sync_phase();
        } else {        // single-chunk step: the items wrote the attention output themselves
            stamp();
            stamp();
        }
        gemm_phase<NP, WF>(c, p.gd[kO], wptr(layer, 2), p.attn, p.c_o, 0);
        sync_phase();
        norm_phase(c, 2, layer, reinterpret_cast<const uint16_t*>(wptr(layer, 3)), false);
        sync_phase();
        gemm_phase<NP, WF>(c, p.gd[kGU], wptr(layer, 4), p.xn, p.c_gu, 0);
        sync_phase();
        swiglu_phase(c);
        sync_phase();
        gemm_phase<NP, WF>(c, p.gd[kDown], wptr(layer, 5), p.act, p.c_down, 0);
        sync_phase();
    }
    norm_phase(c, 1, p.L, p.final_norm, true);
    if (p.lm_head) {
        grid_barrier(c);
        gemm_phase<NP, WF>(c, p.gd[kLM], p.embed, p.xn, nullptr, 1);
    }

    __syncthreads();
    tc_fence_before();
    __syncthreads();
    if (warp == 4) {
        const uint32_t ncols = NP < 32 ? 32u : (uint32_t)NP;
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sh.tmem_base), "r"(ncols) : "memory");
    }
    // the last CTA to finish publishes the greedy ids, optionally advances the step inputs, resets the counters
    if (tid == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(p.bctrl + 1, 1u);
        if (prev == (unsigned)c.ncta - 1u) {
            __threadfence();
            const bool ok = *((volatile unsigned int*)(p.ctrl + kCtrlStatus)) == 0;
            if (p.next_ids && p.lm_head && ok) {
                for (int b = 0; b < p.nb; ++b) {
                    const unsigned long long key = *((volatile unsigned long long*)(p.argkey + b));
                    const long long id = (long long)(0xffffffffu - (uint32_t)key);
                    p.next_ids[b] = id;
                    if (p.advance) {
                        if (p.ids_i64) reinterpret_cast<long long*>(const_cast<void*>(p.input_ids))[b] = id;
                        else reinterpret_cast<int*>(const_cast<void*>(p.input_ids))[b] = (int)id;
                        const long long np = p.positions[b] + 1;
                        const_cast<long long*>(p.positions)[b] = np;
                        const_cast<int*>(p.seq_lens)[b] = p.seq_lens[b] + 1;
                        if (p.slot_mapping[b] >= 0 && np < (long long)p.max_seq_len) {
                            const long long blk = p.block_table[(size_t)b * p.bt_stride + (int)(np / p.block_size)];
                            const_cast<long long*>(p.slot_mapping)[b] = blk * p.block_size + np % p.block_size;
                        }
                    }
                }
            }
            p.bctrl[0] = 0u;
            p.bctrl[1] = 0u;
            __threadfence();
        }
    }
}

}  // namespace batched
}  // namespace pk
