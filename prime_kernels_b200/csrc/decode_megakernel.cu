// Single-launch decode step for Llama-style small LMs (SmolLM2 135M / 360M / 1.7B) on sm_100a.
//
// One persistent cooperative kernel, one CTA per SM, runs every layer of one decode step:
//   RMSNorm -> QKV GEMV -> RoPE + paged-KV append + split-KV attention -> merge -> O GEMV + residual
//   -> RMSNorm -> gate/up GEMV + SwiGLU -> down GEMV + residual -> ... -> final norm
//   -> tied lm_head GEMV + argmax (optional extension; the reference op stops at the final norm,
//      prime_kernels/decode_megakernel/csrc/megakernel.cu:786-798).
//
// B200 design (not a translation of the reference's 24-CTA grid.sync design):
//  * Weight streaming is decoupled from the dependency chain.  Weights do not depend on
//    activations, so a producer warp runs ahead of the math through the whole step and keeps
//    ~190 KB of weights per SM in flight / staged in shared memory with bulk async copies
//    (cp.async.bulk + mbarrier complete_tx, L2 evict-first).  Each of the kNW (7) consumer warps owns a
//    private single-producer/single-consumer byte ring; one producer lane serves each ring, and
//    the lanes advance in lock step so copy issue is kNW-way parallel.  The row -> CTA -> warp
//    schedule is a pure function of the geometry, evaluated identically on both sides.
//  * There is no grid barrier.  Activations cross CTAs through "flagged word" buffers in L2:
//    every 64-bit word carries 32 bits of payload and a 32-bit tag (launch epoch, layer), written
//    and polled with single 8-byte relaxed accesses, so a consumer needs one L2 round trip per
//    hand-off instead of barrier + fence + reload.  Buffers are double-buffered by layer parity;
//    every wait is bounded and reports kErrBarrierTimeout instead of hanging.
//  * GEMVs are warp-per-row-group SIMT fp32 FMA on bf16 (or MXFP8: E4M3 + E8M0 per 32 along K,
//    de-quantised in registers) with 128-bit shared-memory reads; results are rounded to bf16 at
//    the points HuggingFace eager rounds (see the rounding notes at each epilogue).
//
// Reference behaviour followed (file:line inside the reference project):
//   prime_kernels/decode_megakernel/csrc/megakernel.cu:294-799      phase structure, paged KV contract
//   prime_kernels/decode_megakernel_360m_lossless/csrc/block360.cu:121-166,239-255  norm / RoPE rounding
//   prime_kernels/decode_megakernel_360m_lossless/csrc/block360_kernel.inc:114-234,360-436  split-KV + merge
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "pk_common.cuh"

namespace pk {

constexpr int kNW = 7;                     // consumer warps per CTA (+1 producer = 256 threads: 255 registers each)
constexpr int kCT = kNW * 32;              // consumer threads
constexpr int kThreads = kCT + 32;         // + one producer warp
constexpr int kD = 64;                     // head dim (fixed)
constexpr int kE = 8;                      // ring entries in flight per consumer warp
// max weight rows staged per ring entry (8 was measured slower: more registers live across the phase)
__host__ __device__ constexpr int row_cap(int) { return 4; }
constexpr int kMaxB = 8;
constexpr int kNCMax = 64;                 // max split-KV chunks per (request, kv head)
constexpr int kMaxSeq = 8192;
constexpr int kMaxLayerEntries = 40;       // ring entries per consumer warp and layer
constexpr int kMaxLmEntries = 56;          // ring entries per consumer warp for the lm_head
constexpr int kNormRegs = 10;              // norm weights held per thread: hidden <= kNormRegs * kCT
constexpr int kDirectWords = 2048;         // direct-merge limit: partial words every CTA stages per layer
constexpr int kAttnScratchWords = 3072;        // staged partials + merge weights; also >= kNW * 4 * 66 + staging
constexpr int kMaxLayers = 120;
constexpr unsigned kSpinLimit = 1u << 22;  // default bound of every device-side wait: ~1-2 s of L2 polling

enum PhaseType { kQKV = 0, kO = 1, kGU = 2, kDown = 3, kLM = 4, kNumPhaseTypes = 5 };

struct PhaseDesc {
    int nrows;          // output rows of the phase (row pairs for gate/up)
    int kchunks;        // 16-byte chunks per stored row
    int rowbytes;       // bytes per stored row (multiple of 16)
    int rows_per_entry; // rows (pairs) per ring entry when nseg == 1
    int nseg;           // K segments per row; > 1 only when a row does not fit an entry
    int segchunks;      // chunks per segment (multiple of 32 when nseg > 1)
    int pair;           // 1: every entry stages a gate part and an up part
    int widx;           // index in the per-layer pointer table, -1 = embedding matrix (lm_head)
    long long pair_off; // byte offset from a gate row to its up row
    int kact;           // activation length K (elements)
    int pad;
};

struct DecodeParams {
    // model
    const unsigned long long* layers;   // device table [L][6]: norm1, qkv, o, norm2, gate_up, down
    const unsigned long long* kv;       // device table [L]
    const uint16_t* embed;              // [V, H] bf16 (or packed MXFP8 rows when wfmt == 1)
    const uint16_t* embed_bf16;         // [V, H] bf16 embedding rows for the input lookup
    const uint16_t* final_norm;         // [H]
    // step inputs
    const void* input_ids;
    const long long* positions;
    const int* seq_lens;
    const int* block_table;
    const long long* slot_mapping;
    const void* cos_sin;
    // outputs
    uint16_t* out_hidden;               // [B, H] bf16, final-normed
    uint16_t* logits;                   // optional [B, V] bf16
    long long* next_ids;                // optional [B]
    uint16_t* layer_outputs;            // optional [L, B, H]
    unsigned long long* profile;        // optional [ncta][L][kProfSlots] globaltimer stamps (ns)
    // workspace
    unsigned int* ctrl;                 // control words (see Ctrl* below)
    unsigned long long* argkey;         // [2][kMaxB]
    unsigned long long* ll_x;           // [2][B*H]
    unsigned long long* ll_qkv;         // [2][B*NQKV]
    unsigned long long* ll_attn;        // [2][B*QH*32]      (two bf16 per word)
    unsigned long long* ll_h1;          // [2][B*H]
    unsigned long long* ll_act;         // [2][B*I]
    unsigned long long* ll_part;        // [2][B*KVH*kNCMax*G*66]
    long long k_off, v_off, block_stride, token_stride, head_stride;
    int block_size, bt_stride, ids_i64, cs_fp32;
    int H, I, L, QH, KVH, V, B, G;       // B = batch the kernel is instantiated for
    int nb;                             // requests actually present (<= B); rows nb..B-1 are padding
    int wfmt;                           // 0 = bf16 weights, 1 = MXFP8 packed rows
    int lm_head, advance;
    int max_seq_len;
    int ring_bytes;                     // per consumer warp
    int act_elems;                      // max(H, I)
    unsigned spin_limit;                // bound of every device-side wait (polling rounds)
    float eps;
    PhaseDesc ph[kNumPhaseTypes];
};

constexpr int kProfSlots = 24;
constexpr int kKvPtrCache = 64;            // per-layer KV base pointers kept in shared memory (deeper models read the table)
constexpr int kPreRuns = 4;                // runs per warp whose block-table look-ups are resolved at kernel start
constexpr unsigned kProducerIdleNs = 100;   // producer back-off when its rings are full
enum CtrlWord { kCtrlEpoch = 0, kCtrlStatus = 1, kCtrlDone = 2, kCtrlWords = 16 };

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
// global -> this CTA's shared memory, completion counted in bytes on an mbarrier; never multicast
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}
__device__ __forceinline__ unsigned long long ld_flagged(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_flagged(unsigned long long* p, uint32_t payload, uint32_t tag) {
    const unsigned long long v = ((unsigned long long)tag << 32) | payload;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kCT) : "memory"); }

// ------------------------------------------------------------------ shared state
struct Shared {
    uint64_t full[kNW][kE];
    uint64_t empty[kNW][kE];
    uint32_t ent_off[kNW][kE];
    uint32_t ent_foot[kNW][kE];
    uint2 ent_table[kNW][kMaxLayerEntries + kMaxLmEntries];   // per-warp ring schedule: one layer, then lm_head
    int ent_count[kNW][2];
    int row_a[kNumPhaseTypes][kNW];
    int row_b[kNumPhaseTypes][kNW];
    float red[kMaxB][kNW];
    int seq[kMaxB], pos[kMaxB], nc[kMaxB], lc[kMaxB];
    int ncmax, two_level;
    PhaseDesc ph[kNumPhaseTypes];       // copy of the phase descriptors (indexed with a run-time phase type)
    unsigned long long kv_ptr[kKvPtrCache];   // copy of the per-layer KV base pointers: no dependent global load per layer
    uint32_t lm_best[kNW][32];          // lm_head: running argmax per consumer lane
    // This CTA's first attention item, resolved once per launch (nothing in it depends on the layer):
    int item0_b, item0_kvh, item0_chunk;   // its coordinates; item0_b < 0: this CTA has no item
    int item0_all;                         // 1 when kv_off covers every position of the item's chunk
    long long slot_off[kMaxB];             // cache element offset (without the kv-head term) of each request's new token; -1 = skip
    long long kv_off[kNW][kPreRuns * 16];  // cache element offsets (without the kv-head term) of the first kPreRuns
                                           // 16-position runs of each warp's share of the item; -1 = none
    long long slot[kMaxB];
    long long tok[kMaxB];
    volatile int abort_flag;
    uint32_t epoch;
};

struct Ctx {
    const DecodeParams& p;
    Shared& sh;
    uint4* act;        // [B][act_elems/8] bf16 activations of the current phase
    float* res;        // [B][H] residual stream copy (x or h1) for the epilogues
    float* attn;       // attention scratch: per-warp partials / staged chunk partials (kAttnScratchWords)
    unsigned char* ring;  // this warp's ring (consumer) / ring of warp `lane` (producer)
    uint32_t tag_base;
    int warp, lane, cta, ncta;
    unsigned long long* prof;   // non-null only in thread 0 while profiling: stamps of the current layer
};

__device__ __forceinline__ void raise_abort(Ctx& c, int code) {
    c.sh.abort_flag = 1;
    atomicCAS(c.p.ctrl + kCtrlStatus, 0u, (unsigned)code);
}
__device__ __forceinline__ bool aborted(const Ctx& c) { return c.sh.abort_flag != 0; }

// Bounded poll of one flagged word.  Returns the payload; on timeout raises the abort flag.
__device__ __forceinline__ uint32_t wait_flagged(Ctx& c, const unsigned long long* p, uint32_t tag) {
    if (aborted(c)) return 0;
    unsigned spins = 0;
    for (;;) {
        const unsigned long long v = ld_flagged(p);
        if ((uint32_t)(v >> 32) == tag) return (uint32_t)v;
        if ((++spins & 1023u) == 0) {
            if (aborted(c)) return 0;
            if (*((volatile unsigned int*)(c.p.ctrl + kCtrlStatus)) != 0) {
                c.sh.abort_flag = 1;
                return 0;
            }
            if (spins >= c.p.spin_limit) {
                raise_abort(c, kErrBarrierTimeout);
                return 0;
            }
        }
    }
}

// Wait for up to N flagged words at once.  Every round re-issues the loads of all words that are still
// missing before checking any of them, so a round costs one L2 round trip no matter how many words
// are outstanding (re-polling them one after the other would cost one round trip each).
// ptr(u) returns the address of word u, or nullptr when slot u is unused.
template <int N, typename PtrFn>
__device__ __forceinline__ void wait_flagged_multi(Ctx& c, PtrFn ptr, uint32_t tag, uint32_t (&out)[N]) {
    unsigned need = 0;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        out[u] = 0;
        if (ptr(u) != nullptr) need |= 1u << u;
    }
    if (aborted(c)) return;
    unsigned spins = 0;
    while (need) {
        unsigned long long v[N];
#pragma unroll
        for (int u = 0; u < N; ++u)
            if (need & (1u << u)) v[u] = ld_flagged(ptr(u));
#pragma unroll
        for (int u = 0; u < N; ++u)
            if ((need & (1u << u)) && (uint32_t)(v[u] >> 32) == tag) {
                out[u] = (uint32_t)v[u];
                need &= ~(1u << u);
            }
        if (need && (++spins & 255u) == 0) {
            if (aborted(c)) return;
            if (*((volatile unsigned int*)(c.p.ctrl + kCtrlStatus)) != 0) {
                c.sh.abort_flag = 1;
                return;
            }
            if (spins >= c.p.spin_limit) {
                raise_abort(c, kErrBarrierTimeout);
                return;
            }
        }
    }
}

// Up to N words at indices first, first+stride, ... (< n), fetched in one round.
template <int N>
__device__ __forceinline__ void wait_flagged_strided(Ctx& c, const unsigned long long* base, int first, int stride,
                                                     int n, uint32_t tag, uint32_t (&out)[N]) {
    wait_flagged_multi<N>(
        c, [&](int u) { const int idx = first + u * stride; return idx < n ? base + idx : nullptr; }, tag, out);
}

__device__ __forceinline__ bool wait_mbar(Ctx& c, uint64_t* bar, uint32_t parity) {
    if (mbar_probe(bar, parity)) return true;      // the common case: the entry landed long ago
    if (aborted(c)) return false;
    unsigned spins = 0;
    while (!mbar_test(bar, parity)) {
        if ((++spins & 255u) == 0) {
            if (aborted(c)) return false;
            if (spins >= c.p.spin_limit) {
                raise_abort(c, kErrBarrierTimeout);
                return false;
            }
        }
    }
    return true;
}

// ------------------------------------------------------------------ schedule (shared by both sides)
// Rows of phase type t owned by (cta, warp): the CTA takes an even contiguous share of the rows,
// and its warps take even contiguous shares of that.
__device__ __forceinline__ void warp_rows(int nrows, int cta, int ncta, int warp, int& a, int& b) {
    const int r0 = (int)((long long)nrows * cta / ncta);
    const int r1 = (int)((long long)nrows * (cta + 1) / ncta);
    const int n = r1 - r0;
    a = r0 + n * warp / kNW;
    b = r0 + n * (warp + 1) / kNW;
}

// Ring entries of phase type t for a warp that owns rows [a, b): count, and the e-th entry in closed
// form (no sequential state), so the per-warp entry tables can be filled by all lanes in parallel.
// Descriptor: x = byte offset inside the weight matrix; y = part bytes | (widx + 1) << 16 | pair << 20.
__device__ __forceinline__ int phase_entries(const PhaseDesc& d, int a, int b) {
    const int n = b - a;
    if (n <= 0) return 0;
    return d.nseg == 1 ? (n + d.rows_per_entry - 1) / d.rows_per_entry : n * d.nseg;
}
__device__ __forceinline__ uint2 phase_entry(const PhaseDesc& d, int a, int b, int e) {
    uint32_t off, bytes;
    if (d.nseg == 1) {
        const int row = a + e * d.rows_per_entry;
        const int nre = min(d.rows_per_entry, b - row);
        bytes = (uint32_t)nre * (uint32_t)d.rowbytes;
        off = (uint32_t)row * (uint32_t)d.rowbytes;
    } else {
        const int row = a + e / d.nseg, seg = e % d.nseg;
        const int sc = min(d.segchunks, d.kchunks - seg * d.segchunks);
        bytes = (uint32_t)sc * 16u;
        off = (uint32_t)row * (uint32_t)d.rowbytes + (uint32_t)seg * (uint32_t)d.segchunks * 16u;
    }
    return make_uint2(off, bytes | ((uint32_t)(d.widx + 1) << 16) | ((uint32_t)d.pair << 20));
}

// ------------------------------------------------------------------ producer warp
// Lane w (< kNW) feeds the ring of consumer warp w from that warp's entry table (one list per layer,
// reused for every layer, plus the lm_head list).  All lanes run the same loop in lock step; every
// iteration a lane retires up to two consumed entries (non-blocking probes) and issues up to two new
// ones if the ring has room.  Nothing here blocks, so one slow ring never stalls the others.
__device__ void producer_loop(Ctx& c, unsigned char* ring_base) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const int w = c.lane;
    const bool active = w < kNW;
    const uint32_t RW = (uint32_t)p.ring_bytes;
    unsigned char* ring = ring_base + (size_t)(active ? w : 0) * RW;
    const uint64_t pol = evict_first_policy();
    const int n_layer = active ? sh.ent_count[w][0] : 0;
    const int n_lm = (active && p.lm_head) ? sh.ent_count[w][1] : 0;
    const uint32_t total = (uint32_t)n_layer * (uint32_t)p.L + (uint32_t)n_lm;
    const uint2* table = sh.ent_table[active ? w : 0];
    const long long pair_off = p.ph[kGU].pair_off;
    int li = 0, layer = 0;             // position in the schedule: entry li of `layer` (layer == L: lm_head list)
    if (n_layer == 0) layer = p.L;
    uint32_t issued = 0, tail = 0, head = 0, used = 0;
    unsigned idle = 0;
    for (;;) {
        bool progressed = false;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (tail < issued) {
                const uint32_t slot = tail % kE;
                if (mbar_probe(&sh.empty[w][slot], (tail / kE) & 1)) {
                    used -= sh.ent_foot[w][slot];
                    ++tail;
                    progressed = true;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (issued < total) {
                const uint2 dsc = table[layer < p.L ? li : kMaxLayerEntries + li];
                const uint32_t part = dsc.y & 0xffffu;
                const int widx = (int)((dsc.y >> 16) & 0xfu) - 1;
                const bool pair = (dsc.y >> 20) & 1u;
                const uint32_t bytes = pair ? 2 * part : part;
                const uint32_t gap = (head + bytes > RW) ? RW - head : 0;
                const uint32_t foot = bytes + gap;
                if (issued - tail < (uint32_t)kE && used + foot <= RW) {
                    const unsigned char* base =
                        widx < 0 ? reinterpret_cast<const unsigned char*>(p.embed)
                                 : reinterpret_cast<const unsigned char*>(__ldg(p.layers + layer * 6 + widx));
                    const unsigned char* src = base + dsc.x;
                    const uint32_t off = gap ? 0 : head;
                    const uint32_t slot = issued % kE;
                    sh.ent_off[w][slot] = off;
                    sh.ent_foot[w][slot] = foot;
                    mbar_expect_tx(&sh.full[w][slot], bytes);
                    bulk_g2s(ring + off, src, part, &sh.full[w][slot], pol);
                    if (pair) bulk_g2s(ring + off + part, src + pair_off, part, &sh.full[w][slot], pol);
                    head = off + bytes;
                    if (head >= RW) head = 0;
                    used += foot;
                    ++issued;
                    if (++li == (layer < p.L ? n_layer : n_lm)) {
                        li = 0;
                        ++layer;
                    }
                    progressed = true;
                }
            }
        }
        const bool done = issued >= total;      // everything issued; outstanding copies are drained below
        if (__all_sync(kFullMask, done)) break;
        idle = (progressed || done) ? 0 : idle + 1;
        // nothing to retire or issue: yield the issue slots to the consumer warp that shares this scheduler
        if (!__any_sync(kFullMask, progressed)) __nanosleep(kProducerIdleNs);
        if ((idle & 255u) == 255u) {
            if (idle >= c.p.spin_limit) raise_abort(c, kErrBarrierTimeout);
        }
        if (__any_sync(kFullMask, aborted(c))) break;
    }
    // Drain: never leave the CTA while bulk copies into its shared memory are still in flight.
    if (active) {
        for (uint32_t n = tail; n < issued; ++n) {
            const uint32_t slot = n % kE;
            unsigned spins = 0;
            while (!mbar_probe(&sh.full[w][slot], (n / kE) & 1)) {
                if (++spins >= c.p.spin_limit) break;
            }
        }
    }
}

// ------------------------------------------------------------------ math helpers
// acc += w.lo * a.lo + w.hi * a.hi for one packed bf16 pair per operand, with the sm_100 mixed-precision
// FMA (bf16 x bf16 product exact, fp32 accumulate, one rounding: the same result as widening both
// operands and using an fp32 FMA, without the four unpack instructions).
__device__ __forceinline__ float fma2_bf16(uint32_t w, uint32_t a, float acc) {
    asm("{\n.reg .b16 wl, wh, al, ah;\nmov.b32 {wl, wh}, %1;\nmov.b32 {al, ah}, %2;\n"
        "fma.rn.f32.bf16 %0, wl, al, %0;\nfma.rn.f32.bf16 %0, wh, ah, %0;\n}"
        : "+f"(acc)
        : "r"(w), "r"(a));
    return acc;
}
__device__ __forceinline__ float dot8_bf16(const uint4 w, const uint4 a, float acc) {
    acc = fma2_bf16(w.x, a.x, acc);
    acc = fma2_bf16(w.y, a.y, acc);
    acc = fma2_bf16(w.z, a.z, acc);
    acc = fma2_bf16(w.w, a.w, acc);
    return acc;
}

// four E4M3 bytes (one 32-bit word) -> four fp32 (exact)
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t v, float (&f)[4]) {
    uint32_t h0, h1;
    asm("{\n.reg .b16 lo, hi;\nmov.b32 {lo, hi}, %2;\ncvt.rn.f16x2.e4m3x2 %0, lo;\ncvt.rn.f16x2.e4m3x2 %1, hi;\n}"
        : "=r"(h0), "=r"(h1)
        : "r"(v));
    const __half2 a = *reinterpret_cast<__half2*>(&h0);
    const __half2 b = *reinterpret_cast<__half2*>(&h1);
    const float2 fa = __half22float2(a), fb = __half22float2(b);
    f[0] = fa.x;
    f[1] = fa.y;
    f[2] = fb.x;
    f[3] = fb.y;
}

__device__ __forceinline__ float dot16_e4m3(const uint4 w, const uint4 a0, const uint4 a1, float acc) {
    float f[4];
    e4m3x4_to_f32(w.x, f);
    acc = fmaf(f[0], bf16_lo(a0.x), acc);
    acc = fmaf(f[1], bf16_hi(a0.x), acc);
    acc = fmaf(f[2], bf16_lo(a0.y), acc);
    acc = fmaf(f[3], bf16_hi(a0.y), acc);
    e4m3x4_to_f32(w.y, f);
    acc = fmaf(f[0], bf16_lo(a0.z), acc);
    acc = fmaf(f[1], bf16_hi(a0.z), acc);
    acc = fmaf(f[2], bf16_lo(a0.w), acc);
    acc = fmaf(f[3], bf16_hi(a0.w), acc);
    e4m3x4_to_f32(w.z, f);
    acc = fmaf(f[0], bf16_lo(a1.x), acc);
    acc = fmaf(f[1], bf16_hi(a1.x), acc);
    acc = fmaf(f[2], bf16_lo(a1.y), acc);
    acc = fmaf(f[3], bf16_hi(a1.y), acc);
    e4m3x4_to_f32(w.w, f);
    acc = fmaf(f[0], bf16_lo(a1.z), acc);
    acc = fmaf(f[1], bf16_hi(a1.z), acc);
    acc = fmaf(f[2], bf16_lo(a1.w), acc);
    acc = fmaf(f[3], bf16_hi(a1.w), acc);
    return acc;
}

__device__ __forceinline__ uint32_t layer_tag(const Ctx& c, int layer) { return c.tag_base + (uint32_t)layer + 1u; }

__host__ __device__ constexpr int pow2_ceil(int n) { return n <= 1 ? 1 : 2 * pow2_ceil((n + 1) / 2); }
__host__ __device__ constexpr int ilog2(int n) { return n <= 1 ? 0 : 1 + ilog2(n / 2); }

// Warp reduction of NV values per lane that also transposes: on return lane L holds the sum over
// all lanes of v[L >> (5 - log2 NV)].  Step t exchanges one half of the remaining values with the
// lane at distance 16 >> t and keeps the other half, so the number of live values halves each step.
template <int NV>
__device__ __forceinline__ float transpose_reduce(float (&v)[NV], int lane) {
    static_assert(NV >= 1 && NV <= 32 && (NV & (NV - 1)) == 0, "NV must be a power of two up to 32");
#pragma unroll
    for (int k = NV / 2; k >= 1; k >>= 1) {
        const int off = 16 / (NV / (2 * k));
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < k; ++i) {
            const float send = upper ? v[i] : v[i + k];
            const float keep = upper ? v[i + k] : v[i];
            v[i] = keep + __shfl_xor_sync(kFullMask, send, off);
        }
    }
    float r = v[0];
#pragma unroll
    for (int off = 16 / NV; off >= 1; off >>= 1) r += __shfl_xor_sync(kFullMask, r, off);
    return r;
}

// ------------------------------------------------------------------ GEMV row kernels
// NR staged rows (row r at ep + r * stride chunks) times B activation vectors, K-split over the lanes.
// A lone warp cannot hide instruction latency behind other warps, so the loops are unrolled four
// lane-chunks deep: every shared-memory load of a 128-chunk span is issued first, then the FMAs run
// as independent chains (two accumulators per row and request).
template <int B, int NR>
__device__ __forceinline__ void gemv_rows_bf16(const uint4* ep, int sc, const uint4* act, int actc, int kc0, int lane,
                                               float (&acc)[row_cap(B)][B], float (&acc2)[row_cap(B)][B], int nlive = NR) {
    constexpr int U = (NR * B <= 2) ? 4 : (NR * B <= 8 ? 2 : 1);     // lane-chunks in flight; bounded by the register budget
    for (int it0 = 0; it0 < sc; it0 += 32 * U) {
        uint4 av[U][B], wv[NR][U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int ch = it0 + 32 * u + lane;
            const bool ok = ch < sc;
#pragma unroll
            for (int b = 0; b < B; ++b) av[u][b] = ok ? act[b * actc + kc0 + ch] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int r = 0; r < NR; ++r) wv[r][u] = (ok && r < nlive) ? ep[r * sc + ch] : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int r = 0; r < NR; ++r)
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    // the second accumulator set (more independent chains) is only affordable at small batch:
                    // at batch >= 4 it would cost RM * B registers that the kernel does not have
                    if ((u & 1) && B < 4) acc2[r][b] = dot8_bf16(wv[r][u], av[u][b], acc2[r][b]);
                    else acc[r][b] = dot8_bf16(wv[r][u], av[u][b], acc[r][b]);
                }
    }
}

// MXFP8 packed rows: [K e4m3][K/32 e8m0][pad to 16 B]; one lane-chunk = 16 values, scale per 32.
template <int B, int NR>
__device__ __forceinline__ void gemv_rows_mxfp8(const uint4* ep, int rc, int kact, const uint4* act, int actc, int lane,
                                                float (&acc)[row_cap(B)][B], float (&acc2)[row_cap(B)][B], int nlive = NR) {
    const int vc = kact >> 4;
    for (int it0 = 0; it0 < vc; it0 += 64) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int ch = it0 + 32 * u + lane;
            if (ch < vc) {
                uint4 a0[B], a1[B];
#pragma unroll
                for (int b = 0; b < B; ++b) {
                    a0[b] = act[b * actc + 2 * ch];
                    a1[b] = act[b * actc + 2 * ch + 1];
                }
#pragma unroll
                for (int r = 0; r < NR; ++r) {
                    if (r >= nlive) continue;
                    const uint4 wq = ep[r * rc + ch];
                    const unsigned char sb = reinterpret_cast<const unsigned char*>(ep + r * rc)[kact + (ch >> 1)];
                    const float scale = __uint_as_float(sb ? ((uint32_t)sb << 23) : 0x00400000u);
#pragma unroll
                    for (int b = 0; b < B; ++b) {
                        const float part = dot16_e4m3(wq, a0[b], a1[b], 0.f);
                        if ((u & 1) && B < 4) acc2[r][b] = fmaf(scale, part, acc2[r][b]);
                        else acc[r][b] = fmaf(scale, part, acc[r][b]);
                    }
                }
            }
        }
    }
}

// ------------------------------------------------------------------ GEMV phase (consumer warps)
// Consumes this warp's ring entries of phase type T at `layer`, multiplying the staged rows with
// the bf16 activations in c.act, and hands each finished row to the phase epilogue.
template <int B, int WF>
__device__ void gemv_phase(Ctx& c, const int T, int layer, uint32_t& consumed) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const PhaseDesc& d = sh.ph[T];      // shared-memory copy: T is a run-time index
    const int w = c.warp, lane = c.lane;
    const int ra = sh.row_a[T][w], rb = sh.row_b[T][w];
    const int actc = p.act_elems >> 3;                 // uint4 per request in c.act
    const uint32_t tag = layer_tag(c, layer);
    const int par = layer & 1;
    const bool kPair = (T == kGU);
    // lm_head: running argmax over this lane's rows in one word: bf16 order key << 16 | (0xffff - local row).
    // One atomic per warp at the end instead of one per vocabulary row (49152 atomics on one address
    // serialise in L2 and took longer than streaming the embedding matrix).
    // The running value lives in shared memory, not in a register, so that the other phases (which share this
    // code) do not carry it.
    uint32_t& best = sh.lm_best[w][lane];
    if (T == kLM) best = 0u;
    for (int row = ra; row < rb; row += d.rows_per_entry) {
        const int nre = min(d.rows_per_entry, rb - row);
        constexpr int RM = row_cap(B);
        float acc[RM][B], acc2[RM][B];
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int b = 0; b < B; ++b) acc[i][b] = acc2[i][b] = 0.f;
        for (int seg = 0; seg < d.nseg; ++seg) {
            const uint32_t slot = consumed % kE;
            if (!__all_sync(kFullMask, wait_mbar(c, &sh.full[w][slot], (consumed / kE) & 1))) return;
            if (T == kGU && c.prof) c.prof[16] = global_ns();
            const uint4* ep = reinterpret_cast<const uint4*>(c.ring + sh.ent_off[w][slot]);
            // accumulator r <- staged row r; a gate/up entry stages nre gate rows, then nre up rows
            const int nmem = kPair ? 2 * nre : nre;
            if (WF == 0) {
                const int sc = d.nseg == 1 ? d.kchunks : min(d.segchunks, d.kchunks - seg * d.segchunks);
                const int kc0 = seg * d.segchunks;
                switch (nmem) {
                    case 1: gemv_rows_bf16<B, 1>(ep, sc, c.act, actc, kc0, lane, acc, acc2); break;
                    case 2: gemv_rows_bf16<B, 2>(ep, sc, c.act, actc, kc0, lane, acc, acc2); break;
                    case 3: gemv_rows_bf16<B, 3>(ep, sc, c.act, actc, kc0, lane, acc, acc2); break;
                    case 4: gemv_rows_bf16<B, 4>(ep, sc, c.act, actc, kc0, lane, acc, acc2); break;
                    default:
                        if constexpr (RM > 4) {
                            if (nmem <= 6) gemv_rows_bf16<B, 6>(ep, sc, c.act, actc, kc0, lane, acc, acc2, nmem);
                            else gemv_rows_bf16<B, 8>(ep, sc, c.act, actc, kc0, lane, acc, acc2, nmem);
                        }
                        break;
                }
            } else {
                switch (nmem) {
                    case 1: gemv_rows_mxfp8<B, 1>(ep, d.kchunks, d.kact, c.act, actc, lane, acc, acc2); break;
                    case 2: gemv_rows_mxfp8<B, 2>(ep, d.kchunks, d.kact, c.act, actc, lane, acc, acc2); break;
                    case 3: gemv_rows_mxfp8<B, 3>(ep, d.kchunks, d.kact, c.act, actc, lane, acc, acc2); break;
                    case 4: gemv_rows_mxfp8<B, 4>(ep, d.kchunks, d.kact, c.act, actc, lane, acc, acc2); break;
                    default:
                        if constexpr (RM > 4) {
                            if (nmem <= 6) gemv_rows_mxfp8<B, 6>(ep, d.kchunks, d.kact, c.act, actc, lane, acc, acc2, nmem);
                            else gemv_rows_mxfp8<B, 8>(ep, d.kchunks, d.kact, c.act, actc, lane, acc, acc2, nmem);
                        }
                        break;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty[w][slot]);
            ++consumed;
            if (T == kGU && c.prof) c.prof[17] = global_ns();
        }
        // Transposing warp reduction: afterwards lane L holds the total of value L >> SH, where value
        // j = (request j / RM, staged row j % RM), so every (row, request) pair is finished by its
        // own lane at once (no dynamic register indexing, 31 shuffles at most instead of 5 per value).
        constexpr int NV = pow2_ceil(RM * B);
        constexpr int SH = 5 - ilog2(NV);
        float v[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int bb = j / RM < B ? j / RM : 0;     // NV > RM * B only for batch 3: those values are zero
            v[j] = (j / RM < B) ? acc[j % RM][bb] + acc2[j % RM][bb] : 0.f;
        }
        const float mine = transpose_reduce<NV>(v, lane);
        if (T == kGU && c.prof) c.prof[18] = global_ns();
        const int vj = lane >> SH;
        const int ri = vj % RM, b = vj / RM;
        // gate/up entries: the lane that owns gate row ri also needs up row ri, staged at nre + ri
        const float mine_up = __shfl_sync(kFullMask, mine, ((vj + nre) << SH) & 31);
        if ((lane & ((1 << SH) - 1)) == 0 && b < B && ri < nre) {
            const int r = row + ri;
            {
                if (T == kQKV) {
                    // projection output rounded to bf16 (HF linear output dtype)
                    st_flagged(p.ll_qkv + (size_t)par * B * d.nrows + b * d.nrows + r, f32_to_bf16_bits(mine), tag);
                } else if (T == kO) {
                    // h1 = bf16( x + bf16(o_proj) )
                    const float o = round_bf16(mine);
                    const float h = round_bf16(__fadd_rn(c.res[b * p.H + r], o));
                    st_flagged(p.ll_h1 + (size_t)par * B * p.H + b * p.H + r, f32_to_bf16_bits(h), tag);
                } else if (T == kGU) {
                    // act = bf16( bf16(silu(bf16 gate)) * bf16 up )   (HF LlamaMLP rounding)
                    const float g = round_bf16(mine);
                    const float u = round_bf16(mine_up);
                    const float silu = round_bf16(__fdividef(g, 1.f + __expf(-g)));
                    const float a = round_bf16(__fmul_rn(silu, u));
                    st_flagged(p.ll_act + (size_t)par * B * p.I + b * p.I + r, f32_to_bf16_bits(a), tag);
                } else if (T == kDown) {
                    // x' = bf16( h1 + bf16(down_proj) ), handed to the next layer's parity slot
                    const float dn = round_bf16(mine);
                    const uint32_t xb = f32_to_bf16_bits(__fadd_rn(c.res[b * p.H + r], dn));
                    st_flagged(p.ll_x + (size_t)((layer + 1) & 1) * B * p.H + b * p.H + r, xb, layer_tag(c, layer + 1));
                    if (p.layer_outputs && b < p.nb) p.layer_outputs[((size_t)layer * p.nb + b) * p.H + r] = (uint16_t)xb;
                } else {
                    // logits rounded to bf16; argmax breaks ties toward the lowest index
                    const uint32_t lb = f32_to_bf16_bits(mine);
                    if (p.logits && b < p.nb) p.logits[(size_t)b * p.V + r] = (uint16_t)lb;
                    if (p.next_ids && b < p.nb) {
                        const uint32_t ord = (lb & 0x8000u) ? (~lb & 0xffffu) : (lb | 0x8000u);
                        best = max(best, (ord << 16) | (0xffffu - (uint32_t)(r - ra)));
                    }
                }
            }
        }
    }
    if (T == kLM && p.next_ids) {
        // lanes that hold rows of the same request sit in one aligned group of RM << SH lanes
        constexpr int RM = row_cap(B);
        constexpr int SH = 5 - ilog2(pow2_ceil(RM * B));
        constexpr int kGroup = (RM << SH) < 32 ? (RM << SH) : 32;
        uint32_t top = best;
#pragma unroll
        for (int off = 1; off < kGroup; off <<= 1) top = max(top, __shfl_xor_sync(kFullMask, top, off));
        const int b = (lane >> SH) / RM;
        if ((lane & (kGroup - 1)) == 0 && b < p.nb && top != 0u) {
            const uint32_t r = (uint32_t)ra + (0xffffu - (top & 0xffffu));
            const unsigned long long key = ((unsigned long long)(top >> 16) << 32) | (unsigned long long)(0xffffffffu - r);
            atomicMax(p.argkey + (size_t)(sh.epoch & 1u) * kMaxB + b, key);
        }
    }
}

// ------------------------------------------------------------------ activation staging
// Load the residual stream (embedding row for layer 0, flagged X words otherwise), keep an fp32
// copy for the residual add, and write bf16( bf16(x * rsqrt(mean x^2 + eps)) * w ) to c.act.
// HF LlamaRMSNorm: fp32 statistics, cast to bf16, then multiply by the bf16 weight.
template <int B>
__device__ void stage_norm(Ctx& c, const unsigned long long* src_words, uint32_t tag, const uint16_t* weight,
                           bool from_embed) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const int ct = threadIdx.x;
    const int H = p.H;
    // the norm weight does not depend on the activations: fetch it before waiting for them
    float wreg[kNormRegs];
#pragma unroll
    for (int u = 0; u < kNormRegs; ++u) {
        const int i = ct + u * kCT;
        wreg[u] = i < H ? __uint_as_float((uint32_t)__ldg(weight + i) << 16) : 0.f;
    }
    consumer_bar();   // everyone is done with the previous phase's act/res
    // Up to RG requests are polled in one round, so the wait costs one L2 round trip per RG requests
    // instead of one per request.
    constexpr int RG = B < 4 ? B : 4;
    float ss[B];
#pragma unroll
    for (int b = 0; b < B; ++b) ss[b] = 0.f;
    for (int i0 = ct; i0 < H; i0 += 8 * kCT) {
#pragma unroll
        for (int bg = 0; bg < B; bg += RG) {
            uint32_t xv[RG * 8];
            if (from_embed) {
#pragma unroll
                for (int u = 0; u < RG * 8; ++u) {
                    const int i = i0 + (u & 7) * kCT;
                    xv[u] = i < H ? (uint32_t)p.embed_bf16[(size_t)sh.tok[bg + (u >> 3)] * H + i] : 0u;
                }
            } else {
                wait_flagged_multi<RG * 8>(
                    c,
                    [&](int u) {
                        const int i = i0 + (u & 7) * kCT;
                        return i < H ? src_words + (bg + (u >> 3)) * H + i : nullptr;
                    },
                    tag, xv);
            }
#pragma unroll
            for (int u = 0; u < RG * 8; ++u) {
                const int i = i0 + (u & 7) * kCT;
                const int b = bg + (u >> 3);
                if (i < H) {
                    const float x = __uint_as_float(xv[u] << 16);
                    c.res[b * H + i] = x;
                    ss[b] = fmaf(x, x, ss[b]);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
        ss[b] = warp_sum(ss[b]);
        if (c.lane == 0) sh.red[b][c.warp] = ss[b];
    }
    consumer_bar();
    uint16_t* act16 = reinterpret_cast<uint16_t*>(c.act);
    if constexpr (B > 1) {
        // Batched: requests are normalised in pairs; all shared-memory loads of a pair are issued before its
        // stores (the compiler must assume they alias), so the two dependent chains overlap.
#pragma unroll
        for (int bg = 0; bg < B; bg += 2) {
            float s2[2], xr[2][kNormRegs];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int bb = bg + j < B ? bg + j : B - 1;
                float tot = 0.f;
#pragma unroll
                for (int w = 0; w < kNW; ++w) tot += sh.red[bb][w];
                s2[j] = rsqrtf(tot * (1.f / (float)H) + p.eps);
#pragma unroll
                for (int u = 0; u < kNormRegs; ++u) {
                    const int i = ct + u * kCT;
                    xr[j][u] = i < H ? c.res[bb * H + i] : 0.f;
                }
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                if (bg + j >= B) continue;
#pragma unroll
                for (int u = 0; u < kNormRegs; ++u) {
                    const int i = ct + u * kCT;
                    if (i < H) {
                        const float n = round_bf16(__fmul_rn(xr[j][u], s2[j]));
                        act16[(size_t)(bg + j) * p.act_elems + i] = (uint16_t)f32_to_bf16_bits(__fmul_rn(n, wreg[u]));
                    }
                }
            }
        }
        consumer_bar();
        return;
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kNW; ++w) tot += sh.red[b][w];
        const float s = rsqrtf(tot * (1.f / (float)H) + p.eps);
        // all loads first: the stores below may alias them as far as the compiler knows
        float xr[kNormRegs];
#pragma unroll
        for (int u = 0; u < kNormRegs; ++u) {
            const int i = ct + u * kCT;
            xr[u] = i < H ? c.res[b * H + i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < kNormRegs; ++u) {
            const int i = ct + u * kCT;
            if (i < H) {
                const float n = round_bf16(__fmul_rn(xr[u], s));
                act16[(size_t)b * p.act_elems + i] = (uint16_t)f32_to_bf16_bits(__fmul_rn(n, wreg[u]));
            }
        }
    }
    consumer_bar();
}

// Copy flagged bf16 words into c.act.  `packed` words carry two bf16 values each.
template <int B>
__device__ void stage_copy(Ctx& c, const unsigned long long* src_words, uint32_t tag, int n, bool packed) {
    const DecodeParams& p = c.p;
    const int ct = threadIdx.x;
    consumer_bar();
    if constexpr (B > 1) {
        // Batched: two requests are polled per round (one L2 round trip per pair of requests, not per request).
        // Words are 32-bit payloads holding two bf16 values (packed) or one.
        const int nw = packed ? n >> 1 : n;
        constexpr int N = 8;                     // words per request and round
        uint32_t* act32 = reinterpret_cast<uint32_t*>(c.act);
        uint16_t* act16 = reinterpret_cast<uint16_t*>(c.act);
        for (int i0 = ct; i0 < nw; i0 += N * kCT) {
#pragma unroll
            for (int bg = 0; bg < B; bg += 2) {
                constexpr int kPairs = 2;
                uint32_t v[kPairs * N];
                wait_flagged_multi<kPairs * N>(
                    c,
                    [&](int u) {
                        const int i = i0 + (u % N) * kCT;
                        const int bb = bg + u / N;
                        return (i < nw && bb < B) ? src_words + bb * nw + i : nullptr;
                    },
                    tag, v);
#pragma unroll
                for (int u = 0; u < kPairs * N; ++u) {
                    const int i = i0 + (u % N) * kCT;
                    const int bb = bg + u / N;
                    if (i < nw && bb < B) {
                        if (packed) act32[(size_t)bb * (p.act_elems >> 1) + i] = v[u];
                        else act16[(size_t)bb * p.act_elems + i] = (uint16_t)v[u];
                    }
                }
            }
        }
        consumer_bar();
        return;
    }
    if (packed) {
        uint32_t* act32 = reinterpret_cast<uint32_t*>(c.act);
        const int nw = n >> 1;
        for (int b = 0; b < B; ++b)
            for (int i0 = ct; i0 < nw; i0 += 4 * kCT) {
                uint32_t v[4];
                wait_flagged_strided<4>(c, src_words + b * nw, i0, kCT, nw, tag, v);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i0 + u * kCT < nw) act32[(size_t)b * (p.act_elems >> 1) + i0 + u * kCT] = v[u];
            }
    } else {
        uint16_t* act16 = reinterpret_cast<uint16_t*>(c.act);
        for (int b = 0; b < B; ++b)
            for (int i0 = ct; i0 < n; i0 += 16 * kCT) {
                uint32_t v[16];
                wait_flagged_strided<16>(c, src_words + b * n, i0, kCT, n, tag, v);
#pragma unroll
                for (int u = 0; u < 16; ++u)
                    if (i0 + u * kCT < n) act16[(size_t)b * p.act_elems + i0 + u * kCT] = (uint16_t)v[u];
            }
    }
    consumer_bar();
}

// ------------------------------------------------------------------ attention
// HF apply_rotary_pos_emb rounding: bf16( bf16(x*cos) + bf16(rotate_half(x)*sin) ).
__device__ __forceinline__ float rope_elem(float x, float partner, float cs, float sn, bool first_half) {
    const float xc = round_bf16(__fmul_rn(x, cs));
    const float ys = round_bf16(__fmul_rn(partner, sn));
    return round_bf16(__fadd_rn(xc, first_half ? -ys : ys));
}

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x);
    f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z);
    f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}

// One CTA = one (request b, kv head, chunk) item over cache positions [start, end); the consumer warps
// split the chunk into runs of 16 positions.  Each run is processed in two phases so that no value
// has to be reduced across more than two lanes:
//   scores: lane = (position, half) -- a lane reads 32 dims of its position's K row (four 16-byte
//           loads; a lane pair covers the 128-byte row) and dots them with the G rotated queries kept
//           as packed bf16 in shared memory (mixed-precision FMA, no unpacking); one shuffle joins the
//           halves.  The softmax statistics of the run are warp reductions over the 16 positions.
//   P.V:    lane = two output dims -- the V rows of the 16 positions are read as coalesced 128-byte
//           rows (one 4-byte load per lane and position) and accumulated with the probabilities
//           broadcast from shared memory.
// All K and V loads of a run are issued before the new token's q/k/v words are waited for.  Warps are
// combined through shared memory with log-sum-exp and one partial (m, l, acc[64]) per query head of the
// GQA group leaves the CTA as flagged words.
template <int G>
__device__ void attention_item(Ctx& c, int layer, int b, int kvh, int chunk, bool first_item) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const int lane = c.lane;
    const uint32_t tag = layer_tag(c, layer);
    const int par = layer & 1;
    const int nqkv = (p.QH + 2 * p.KVH) * kD;
    const unsigned long long* qkv = p.ll_qkv + (size_t)par * p.B * nqkv + (size_t)b * nqkv;
    const int seq = sh.seq[b], pos = sh.pos[b];
    const int start = chunk * sh.lc[b];
    const int end = min(start + sh.lc[b], seq);
    // this warp's share of the chunk, a multiple of 16 positions
    const int ppw = (((end - start + kNW - 1) / kNW) + 15) & ~15;
    const int ws = min(start + c.warp * ppw, end);
    const int we = min(ws + ppw, end);
    const bool has_new = (seq - 1 >= ws) && (seq - 1 < we);
    const uint16_t* kvr = reinterpret_cast<const uint16_t*>(layer < kKvPtrCache ? sh.kv_ptr[layer] : p.kv[layer]);
    const int pl = lane >> 1, half = lane & 1;      // scores phase: position in the run, half of the head dim

    // shared-memory staging (all on 16-byte boundaries)
    constexpr int kPartWords = (kNW * G * 66 + 3) & ~3;
    static_assert(kPartWords + (G + 2) * kD + (G + 2) * 32 + kNW * G * 16 <= kAttnScratchWords, "attention scratch too small");
    float* raw_s = c.attn + kPartWords;                                  // [(G+2)*64] un-rotated q, k, v
    uint32_t* qkvb_s = reinterpret_cast<uint32_t*>(raw_s + (G + 2) * kD);   // [(G+2)*32] packed bf16: rotated q, k; v
    float* prob_s = reinterpret_cast<float*>(qkvb_s + (G + 2) * 32) + c.warp * G * 16;   // [G][16] per warp

    // element offset of position pp of this (request, kv head) in the paged cache
    auto kv_offset = [&](int pp) -> long long {
        // padding rows read the block-table row of the last real request
        const int blk = __ldg(p.block_table + min(b, p.nb - 1) * p.bt_stride + pp / p.block_size);
        return (long long)blk * p.block_stride + (long long)(pp % p.block_size) * p.token_stride +
               (long long)kvh * p.head_stride;
    };
    // loads of one run of 16 positions starting at r0: K (this lane's position and half), V (all 16
    // positions, this lane's two dims); the position seq-1 is taken from shared memory later
    uint4 kq[4];
    uint32_t vw[16];
    auto fetch_run = [&](int r0) {
        const int pp = r0 + pl;
        long long e_own = 0;
        const bool own_ok = pp < we && pp != seq - 1;
        if (first_item && r0 - ws < kPreRuns * 16) {
            // offsets resolved at kernel start (shared memory, no dependent global load)
            const long long hs = (long long)kvh * p.head_stride;
            const long long* pre = sh.kv_off[c.warp] + (r0 - ws);
            if (pp < we) e_own = pre[pl] + hs;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                kq[i] = own_ok ? __ldcg(reinterpret_cast<const uint4*>(kvr + p.k_off + e_own + 32 * half) + i)
                               : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int pj = r0 + j;
                const long long ej = pre[j] + hs;
                vw[j] = (pj < we && pj != seq - 1)
                            ? __ldcg(reinterpret_cast<const uint32_t*>(kvr + p.v_off + ej) + lane)
                            : 0u;
            }
            return;
        }
        if (pp < we) e_own = kv_offset(pp);
#pragma unroll
        for (int i = 0; i < 4; ++i)
            kq[i] = own_ok ? __ldcg(reinterpret_cast<const uint4*>(kvr + p.k_off + e_own + 32 * half) + i)
                           : make_uint4(0u, 0u, 0u, 0u);
        // V rows: when the run lies inside one cache block the offsets are an arithmetic sequence
        const bool one_block = (r0 % p.block_size) + 15 < p.block_size;
        const long long e0 = __shfl_sync(kFullMask, e_own, 0);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int pj = r0 + j;
            long long ej;
            if (one_block) {
                ej = e0 + (long long)j * p.token_stride;
            } else {
                ej = __shfl_sync(kFullMask, e_own, 2 * j);
            }
            vw[j] = (pj < we && pj != seq - 1)
                        ? __ldcg(reinterpret_cast<const uint32_t*>(kvr + p.v_off + ej) + lane)
                        : 0u;
        }
    };
    if (c.prof) c.prof[10] = global_ns();
    if (ws < we) fetch_run(ws);

    // q of the G heads sharing this kv head plus the new token's k and v: (G + 2) * 64 flagged words
    {
        constexpr int kPer = ((G + 2) * kD + kCT - 1) / kCT;      // words per thread
        auto word_row = [&](int t) {
            const int which = t / kD, d = t % kD;     // which: 0..G-1 = q head, G = k, G+1 = v
            return which < G ? (kvh * G + which) * kD + d
                             : (which == G ? (p.QH + kvh) * kD + d : (p.QH + p.KVH + kvh) * kD + d);
        };
        uint32_t bits[kPer];
        wait_flagged_multi<kPer>(
            c,
            [&](int u) -> const unsigned long long* {
                const int t = (int)threadIdx.x + u * kCT;
                return t < (G + 2) * kD ? qkv + word_row(t) : nullptr;
            },
            tag, bits);
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int t = (int)threadIdx.x + u * kCT;
            if (t < (G + 2) * kD) raw_s[t] = __uint_as_float(bits[u] << 16);
        }
    }
    consumer_bar();
    if (c.prof) c.prof[11] = global_ns();
    // rotate q and k (two adjacent dims per thread) and pack everything to bf16 pairs
    for (int t = threadIdx.x; t < (G + 2) * 32; t += kCT) {
        const int which = t >> 5, dp = t & 31, d = 2 * dp;
        float o0 = raw_s[which * kD + d], o1 = raw_s[which * kD + d + 1];
        if (which <= G) {
            float c0, s0, c1, s1;
            const int ci = pos * kD + (d & 31);
            if (p.cs_fp32) {
                const float* t32 = reinterpret_cast<const float*>(p.cos_sin);
                c0 = __ldg(t32 + ci); c1 = __ldg(t32 + ci + 1);
                s0 = __ldg(t32 + ci + 32); s1 = __ldg(t32 + ci + 33);
            } else {
                const uint32_t cw = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.cos_sin) + ci));
                const uint32_t sw = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.cos_sin) + ci + 32));
                c0 = bf16_lo(cw); c1 = bf16_hi(cw);
                s0 = bf16_lo(sw); s1 = bf16_hi(sw);
            }
            const float p0 = raw_s[which * kD + (d ^ 32)], p1 = raw_s[which * kD + ((d + 1) ^ 32)];
            o0 = rope_elem(o0, p0, c0, s0, d < 32);
            o1 = rope_elem(o1, p1, c1, s1, d < 32);
        }
        qkvb_s[t] = pack_bf16x2(o0, o1);
    }
    consumer_bar();
    if (c.prof) c.prof[12] = global_ns();
    if (has_new) {   // warp-uniform: append the new token's K/V to the paged cache (slot -1 = padded row: skip)
        const long long so = sh.slot_off[b];
        if (so >= 0 && lane < 8) {
            uint16_t* kvw = reinterpret_cast<uint16_t*>(layer < kKvPtrCache ? sh.kv_ptr[layer] : p.kv[layer]);
            const long long e = so + (long long)kvh * p.head_stride + 8 * lane;
            *reinterpret_cast<uint4*>(kvw + p.k_off + e) = *reinterpret_cast<const uint4*>(qkvb_s + G * 32 + 4 * lane);
            *reinterpret_cast<uint4*>(kvw + p.v_off + e) = *reinterpret_cast<const uint4*>(qkvb_s + (G + 1) * 32 + 4 * lane);
        }
    }

    float m[G], l[G], acc[G][2];
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        m[hh] = -INFINITY;
        l[hh] = 0.f;
        acc[hh][0] = acc[hh][1] = 0.f;
    }
    for (int r0 = ws; r0 < we; r0 += 16) {
        if (r0 != ws) fetch_run(r0);
        const int pp = r0 + pl;
        const bool valid = pp < we;
        // ---- scores of this lane's position (half of the dims), joined with the other half
        uint32_t kwd[16];
        if (pp == seq - 1) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 t4 = *reinterpret_cast<const uint4*>(qkvb_s + G * 32 + 16 * half + 4 * i);
                kwd[4 * i] = t4.x; kwd[4 * i + 1] = t4.y; kwd[4 * i + 2] = t4.z; kwd[4 * i + 3] = t4.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                kwd[4 * i] = kq[i].x; kwd[4 * i + 1] = kq[i].y; kwd[4 * i + 2] = kq[i].z; kwd[4 * i + 3] = kq[i].w;
            }
        }
        float sc[G];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            float d0 = 0.f, d1 = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 q4 = *reinterpret_cast<const uint4*>(qkvb_s + hh * 32 + 16 * half + 4 * i);
                d0 = fma2_bf16(kwd[4 * i], q4.x, d0);
                d1 = fma2_bf16(kwd[4 * i + 1], q4.y, d1);
                d0 = fma2_bf16(kwd[4 * i + 2], q4.z, d0);
                d1 = fma2_bf16(kwd[4 * i + 3], q4.w, d1);
            }
            float dsum = d0 + d1;
            dsum += __shfl_xor_sync(kFullMask, dsum, 1);
            // bf16 matmul output, then the exact 1/8 scale (HF eager_attention_forward)
            sc[hh] = valid ? round_bf16(dsum) * 0.125f : -INFINITY;
        }
        // ---- running softmax statistics over the 16 positions of the run
        float pr[G];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            float mx = sc[hh];
#pragma unroll
            for (int o = 2; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(kFullMask, mx, o));
            const float mn = fmaxf(m[hh], mx);
            const float alpha = (mn == -INFINITY) ? 1.f : __expf(m[hh] - mn);
            pr[hh] = (sc[hh] == -INFINITY) ? 0.f : __expf(sc[hh] - mn);
            float ps = pr[hh];
#pragma unroll
            for (int o = 2; o < 32; o <<= 1) ps += __shfl_xor_sync(kFullMask, ps, o);
            l[hh] = l[hh] * alpha + ps;
            m[hh] = mn;
            acc[hh][0] *= alpha;
            acc[hh][1] *= alpha;
            if (half == 0) prob_s[hh * 16 + pl] = pr[hh];
        }
        __syncwarp();
        // ---- P.V: this lane accumulates dims 2*lane, 2*lane+1 over the 16 positions
        const uint32_t vnew = qkvb_s[(G + 1) * 32 + lane];
#pragma unroll
        for (int hh = 0; hh < G; ++hh) {
            float a0 = acc[hh][0], a1 = acc[hh][1];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
                const float4 p4 = *reinterpret_cast<const float4*>(prob_s + hh * 16 + 4 * j4);
                const float pj[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) {
                    const int j = 4 * j4 + jj;
                    const uint32_t v = (r0 + j == seq - 1) ? vnew : vw[j];
                    a0 = fmaf(pj[jj], bf16_lo(v), a0);
                    a1 = fmaf(pj[jj], bf16_hi(v), a1);
                }
            }
            acc[hh][0] = a0;
            acc[hh][1] = a1;
        }
        __syncwarp();
    }
    if (c.prof) c.prof[13] = global_ns();
    // park the warp's partial in shared memory: lanes hold two dims each, nothing to shuffle
    float* wpart = c.attn + (size_t)c.warp * G * 66;
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        float* dst = wpart + hh * 66;
        if (lane == 0) {
            dst[0] = m[hh];
            dst[1] = l[hh];
        }
        *reinterpret_cast<float2*>(dst + 2 + 2 * lane) = make_float2(acc[hh][0], acc[hh][1]);
    }
    consumer_bar();
    if (c.prof) c.prof[14] = global_ns();
    // combine the warps; thread (hh, d) publishes one accumulator word, d == 0 also m and l
    const size_t item = ((size_t)(b * p.KVH + kvh) * kNCMax + chunk) * G;
    unsigned long long* part = p.ll_part + ((size_t)par * p.B * p.KVH * kNCMax * G + item) * 66;
    for (int t = threadIdx.x; t < G * kD; t += kCT) {
        const int hh = t / kD, d = t % kD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kNW; ++w) M = fmaxf(M, c.attn[(w * G + hh) * 66]);
        float lt = 0.f, a = 0.f;
#pragma unroll
        for (int w = 0; w < kNW; ++w) {
            const float* src = c.attn + (w * G + hh) * 66;
            const float f = (src[0] == -INFINITY) ? 0.f : __expf(src[0] - M);
            lt = fmaf(src[1], f, lt);
            a = fmaf(src[2 + d], f, a);
        }
        unsigned long long* dst = part + hh * 66;
        if (d == 0) {
            st_flagged(dst + 0, __float_as_uint(M), tag);
            st_flagged(dst + 1, __float_as_uint(lt), tag);
        }
        st_flagged(dst + 2 + d, __float_as_uint(a), tag);
    }
    consumer_bar();   // c.attn is reused by the next item / the merge staging
    if (c.prof) c.prof[15] = global_ns();
}

// Two-level mode only: log-sum-exp merge of the chunk partials of one (request, query head) by one
// warp; output rounded to bf16 (the attention output dtype), two values per flagged word.
__device__ void merge_task(Ctx& c, int layer, int b, int hq) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const int lane = c.lane;
    const uint32_t tag = layer_tag(c, layer);
    const int par = layer & 1;
    const int G = p.G;
    const int kvh = hq / G, hh = hq - kvh * G;
    const int nc = sh.nc[b];
    const unsigned long long* part =
        p.ll_part + ((size_t)par * p.B * p.KVH * kNCMax * G + ((size_t)(b * p.KVH + kvh) * kNCMax) * G + hh) * 66;
    const size_t cstride = (size_t)G * 66;
    // one round of loads: m and l of chunks lane, lane+32, and this lane's accumulator pair of the
    // first 8 chunks
    uint32_t w20[20];
    wait_flagged_multi<20>(
        c,
        [&](int u) -> const unsigned long long* {
            if (u < 4) {
                const int ch = lane + 32 * (u >> 1);
                return ch < nc ? part + ch * cstride + (u & 1) : nullptr;
            }
            const int ch = (u - 4) >> 1;
            return ch < nc ? part + ch * cstride + 2 + 2 * lane + (u & 1) : nullptr;
        },
        tag, w20);
    float mc[2], lc[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int ch = lane + 32 * u;
        mc[u] = ch < nc ? __uint_as_float(w20[2 * u]) : -INFINITY;
        lc[u] = ch < nc ? __uint_as_float(w20[2 * u + 1]) : 0.f;
    }
    const float M = warp_max(fmaxf(mc[0], mc[1]));
    float wc[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) wc[u] = (mc[u] == -INFINITY) ? 0.f : __expf(mc[u] - M);
    const float den = warp_sum(lc[0] * wc[0] + lc[1] * wc[1]);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        if (u < nc) {   // warp-uniform
            const float wgt = __shfl_sync(kFullMask, wc[0], u);
            a0 = fmaf(wgt, __uint_as_float(w20[4 + 2 * u]), a0);
            a1 = fmaf(wgt, __uint_as_float(w20[5 + 2 * u]), a1);
        }
    }
    for (int ch0 = 8; ch0 < nc; ch0 += 8) {
        uint32_t av[16];
        wait_flagged_multi<16>(
            c,
            [&](int u) -> const unsigned long long* {
                const int ch = ch0 + (u >> 1);
                return ch < nc ? part + ch * cstride + 2 + 2 * lane + (u & 1) : nullptr;
            },
            tag, av);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int ch = ch0 + u;
            if (ch < nc) {   // warp-uniform
                const float wgt = __shfl_sync(kFullMask, ch < 32 ? wc[0] : wc[1], ch & 31);
                a0 = fmaf(wgt, __uint_as_float(av[2 * u]), a0);
                a1 = fmaf(wgt, __uint_as_float(av[2 * u + 1]), a1);
            }
        }
    }
    const float inv = 1.f / den;
    const uint32_t packed = pack_bf16x2(a0 * inv, a1 * inv);
    const int nattn = p.QH * kD / 2;
    st_flagged(p.ll_attn + (size_t)par * p.B * nattn + (size_t)b * nattn + hq * (kD / 2) + lane, packed, tag);
}

// Top of a layer: the CTAs that own attention items pull their chunk's K/V rows (256 contiguous bytes
// per position and kv head) towards L2 while the QKV projection is still being computed.
__device__ void attention_prefetch(Ctx& c, int layer) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const int nslots = kNCMax * p.B * p.KVH;
    const unsigned char* kvr = reinterpret_cast<const unsigned char*>(layer < kKvPtrCache ? sh.kv_ptr[layer] : p.kv[layer]);
    int first = c.cta;
    if (sh.item0_all) {
        // first item, offsets already resolved: thread = (warp share, position, K or V), no look-ups
        const long long hs = (long long)sh.item0_kvh * p.head_stride;
        for (int t = (int)threadIdx.x; t < kNW * kPreRuns * 32; t += kCT) {
            const long long off = sh.kv_off[t / (kPreRuns * 32)][(t % (kPreRuns * 32)) >> 1];
            if (off >= 0) {
                const long long e = off + hs;
                const unsigned char* a = kvr + ((t & 1) ? p.v_off + e : p.k_off + e) * 2;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
            }
        }
        first += c.ncta;
    } else if (sh.item0_b < 0) {
        first += c.ncta;       // the first slot holds no item (a short request); later slots are still visited
    }
    for (int s = first; s < nslots; s += c.ncta) {
        const int kvh = s % p.KVH;
        const int rest = s / p.KVH;
        const int b = rest % p.B;
        const int chunk = rest / p.B;
        if (chunk >= sh.ncmax) break;
        if (chunk >= sh.nc[b]) continue;
        const int start = chunk * sh.lc[b];
        const int end = min(start + sh.lc[b], sh.seq[b] - 1);
        for (int i = start * 2 + (int)threadIdx.x; i < end * 2; i += kCT) {
            const int pp = i >> 1;
            const int blk = __ldg(p.block_table + min(b, p.nb - 1) * p.bt_stride + pp / p.block_size);
            const long long e = (long long)blk * p.block_stride + (long long)(pp % p.block_size) * p.token_stride +
                                (long long)kvh * p.head_stride;
            const unsigned char* a = kvr + ((i & 1) ? p.v_off + e : p.k_off + e) * 2;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(a));
        }
    }
}

template <int G>
__device__ void attention_phase(Ctx& c, int layer) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    // items (chunk-major so that the always-present chunk 0 of every (request, kv head) comes first),
    // dealt round-robin to CTAs
    const int nslots = kNCMax * p.B * p.KVH;
    // one call site (the item code is large): the first slot takes its coordinates from shared memory
    for (int s = c.cta; s < nslots; s += c.ncta) {
        const bool first = (s == c.cta);
        int b = sh.item0_b, kvh = sh.item0_kvh, chunk = sh.item0_chunk;
        if (first) {
            if (b < 0) continue;
        } else {
            kvh = s % p.KVH;
            const int rest = s / p.KVH;
            b = rest % p.B;
            chunk = rest / p.B;
            if (chunk >= sh.ncmax) break;
            if (chunk >= sh.nc[b]) continue;
        }
        attention_item<G>(c, layer, b, kvh, chunk, first);
    }
    if (sh.two_level) {
        const int total_warps = c.ncta * kNW;
        const int gm = (kNW - 1 - c.warp) * c.ncta + c.cta;
        for (int t = gm; t < p.B * p.QH; t += total_warps) merge_task(c, layer, t / p.QH, t % p.QH);
    }
}

// Direct mode: every CTA pulls all chunk partials (at most kDirectWords words), merges them with
// log-sum-exp in shared memory and writes the bf16 attention output straight into c.act -- one
// hand-off between the attention items and the O projection instead of two.
template <int B>
__device__ void stage_attn_direct(Ctx& c, int layer) {
    const DecodeParams& p = c.p;
    Shared& sh = c.sh;
    const int ct = threadIdx.x;
    const uint32_t tag = layer_tag(c, layer);
    const int par = layer & 1;
    const int G = p.G;
    const unsigned long long* base = p.ll_part + (size_t)par * p.B * p.KVH * kNCMax * G * 66;
    float* wts = c.attn + kDirectWords;          // [B * QH * nc] merge weights (<= 512 words)
    consumer_bar();
    // stage: shared layout [b][kvh][chunk < nc_b][hh][66], source layout [b][kvh][kNCMax][hh][66]
    int soff = 0;
    for (int b = 0; b < B; ++b) {
        const int nc = sh.nc[b];
        const int per_kvh = nc * G * 66;
        const int n = p.KVH * per_kvh;
        for (int i0 = ct; i0 < n; i0 += 8 * kCT) {
            uint32_t bits[8];
            wait_flagged_multi<8>(
                c,
                [&](int u) -> const unsigned long long* {
                    const int i = i0 + u * kCT;
                    if (i >= n) return nullptr;
                    const int kvh = i / per_kvh, r = i - kvh * per_kvh;
                    return base + ((size_t)(b * p.KVH + kvh) * kNCMax) * G * 66 + r;
                },
                tag, bits);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int i = i0 + u * kCT;
                if (i < n) c.attn[soff + i] = __uint_as_float(bits[u]);
            }
        }
        soff += n;
    }
    consumer_bar();
    // merge weights once per (request, head, chunk): w = exp(m_c - M) / sum_c l_c exp(m_c - M)
    soff = 0;
    int woff = 0;
    for (int b = 0; b < B; ++b) {
        const int nc = sh.nc[b];
        for (int hq = ct; hq < p.QH; hq += kCT) {
            const int kvh = hq / G, hh = hq - kvh * G;
            const float* src = c.attn + soff + ((kvh * nc) * G + hh) * 66;
            const int cs = G * 66;
            float M = -INFINITY;
            for (int ch = 0; ch < nc; ++ch) M = fmaxf(M, src[ch * cs]);
            float den = 0.f;
            for (int ch = 0; ch < nc; ++ch) {
                const float w = (src[ch * cs] == -INFINITY) ? 0.f : __expf(src[ch * cs] - M);
                wts[woff + hq * nc + ch] = w;
                den = fmaf(src[ch * cs + 1], w, den);
            }
            const float inv = 1.f / den;
            for (int ch = 0; ch < nc; ++ch) wts[woff + hq * nc + ch] *= inv;
        }
        soff += p.KVH * nc * G * 66;
        woff += p.QH * nc;
    }
    consumer_bar();
    uint16_t* act16 = reinterpret_cast<uint16_t*>(c.act);
    soff = 0;
    woff = 0;
    for (int b = 0; b < B; ++b) {
        const int nc = sh.nc[b];
        for (int o = ct; o < p.QH * kD; o += kCT) {
            const int hq = o / kD, d = o - hq * kD;
            const int kvh = hq / G, hh = hq - kvh * G;
            const float* src = c.attn + soff + ((kvh * nc) * G + hh) * 66 + 2 + d;
            const float* w = wts + woff + hq * nc;
            const int cs = G * 66;
            float a = 0.f;
            for (int ch = 0; ch < nc; ++ch) a = fmaf(src[ch * cs], w[ch], a);
            act16[(size_t)b * p.act_elems + o] = (uint16_t)f32_to_bf16_bits(a);
        }
        soff += p.KVH * nc * G * 66;
        woff += p.QH * nc;
    }
    consumer_bar();
}

// ------------------------------------------------------------------ the kernel
template <int B, int G, int WF>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const DecodeParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    Shared& sh = *reinterpret_cast<Shared*>(smem_raw);
    size_t off = (sizeof(Shared) + 127) & ~size_t(127);
    uint4* act = reinterpret_cast<uint4*>(smem_raw + off);
    off += ((size_t)B * p.act_elems * 2 + 127) & ~size_t(127);
    float* res = reinterpret_cast<float*>(smem_raw + off);
    off += ((size_t)B * p.H * 4 + 127) & ~size_t(127);
    float* attn_scratch = reinterpret_cast<float*>(smem_raw + off);
    off += (size_t)kAttnScratchWords * 4;
    unsigned char* ring_base = smem_raw + off;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, ncta = gridDim.x;

    if (tid == 0) {
        sh.abort_flag = (p.ctrl[kCtrlStatus] != 0u) ? 1 : 0;   // an earlier failure on this workspace: fall through
        sh.epoch = p.ctrl[kCtrlEpoch];
    }
    if (tid < kNW * kE) {
        mbar_init(&sh.full[tid / kE][tid % kE], 1);
        mbar_init(&sh.empty[tid / kE][tid % kE], 1);
    }
    if (tid < kNumPhaseTypes) sh.ph[tid] = p.ph[tid];
    for (int l = tid; l < p.L && l < kKvPtrCache; l += kThreads) sh.kv_ptr[l] = p.kv[l];
    if (tid < kNumPhaseTypes * kNW) {
        const int t = tid / kNW, w = tid % kNW;
        int a = 0, b = 0;
        if (t != kLM || p.lm_head) warp_rows(p.ph[t].nrows, cta, ncta, w, a, b);
        sh.row_a[t][w] = a;
        sh.row_b[t][w] = b;
    }
    if (tid < B) {
        // padding rows (batch 5..7 run on the batch-8 kernel) mirror the last real request and write nothing
        const int src = min(tid, p.nb - 1);
        // a sequence length beyond the block table's capacity would index past its row: clamp and report
        const int seq = min(max(p.seq_lens[src], 1), p.max_seq_len);
        sh.seq[tid] = seq;
        sh.pos[tid] = (int)max(p.positions[src], 0LL);
        sh.slot[tid] = tid < p.nb ? p.slot_mapping[src] : -1LL;
        const long long tok = p.ids_i64 ? reinterpret_cast<const long long*>(p.input_ids)[src]
                                        : (long long)reinterpret_cast<const int*>(p.input_ids)[src];
        sh.tok[tid] = tok < 0 ? 0 : (tok >= p.V ? p.V - 1 : tok);   // an out-of-range id must not become a wild read
        // Split-KV chunking: one CTA per (request, kv head, chunk) item.  The chunk length is the
        // shortest multiple of 16 positions, at least one 16-position run per warp, that keeps the
        // number of items within one round of the grid (and the chunks per request within kNCMax);
        // when there are more (request, kv head) pairs than CTAs a chunk covers the whole context.
        // With few partials (short contexts) every CTA merges them itself while staging the O
        // projection input (direct mode, one hand-off); otherwise one warp per (request, head) merges
        // and publishes the result (two hand-offs, but no redundant staging).  The mode is decided on
        // the longest request so it is CTA-uniform.
        int smax = 1;
        for (int bb = 0; bb < p.nb; ++bb) smax = max(smax, min(max(p.seq_lens[bb], 1), p.max_seq_len));
        const int nct = min(max(ncta / (B * p.KVH), 1), kNCMax);
        const int lc = max(16 * kNW, (((smax + nct - 1) / nct) + 15) & ~15);
        const int two = (B * p.QH * ((smax + lc - 1) / lc) * 66 > kDirectWords) ? 1 : 0;
        sh.lc[tid] = lc;
        sh.nc[tid] = (seq + lc - 1) / lc;
        if (tid == 0) {
            sh.two_level = two;
            sh.ncmax = (smax + lc - 1) / lc;
        }
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
        for (int bb = 0; bb < p.nb; ++bb)
            if (p.seq_lens[bb] > p.max_seq_len) {
                sh.abort_flag = 1;
                atomicCAS(p.ctrl + kCtrlStatus, 0u, (unsigned)kErrMaxSeq);
            }
    }
    if (warp < kNW) {
        // The block-table look-ups of an attention item do not depend on the layer: resolve them once per
        // launch for this CTA's first item (the only one at moderate contexts), so that a layer's K/V loads
        // can be issued without a dependent global load and integer divisions in front of them.
        {
            const int sidx = cta;
            int ib = -1, ikvh = 0, ichunk = 0, ws = 0, we = 0, ppw = 0;
            if (sidx < kNCMax * B * p.KVH) {
                const int rest = sidx / p.KVH;
                const int b = rest % B, chunk = rest / B;
                if (chunk < sh.nc[b]) {
                    ib = b;
                    ikvh = sidx % p.KVH;
                    ichunk = chunk;
                    const int seq = sh.seq[b];
                    const int start = chunk * sh.lc[b];
                    const int end = min(start + sh.lc[b], seq);
                    ppw = (((end - start + kNW - 1) / kNW) + 15) & ~15;
                    ws = min(start + warp * ppw, end);
                    we = min(ws + ppw, end);
                }
            }
            for (int j = lane; j < kPreRuns * 16; j += 32) {
                long long off = -1;
                const int pp = ws + j;
                if (ib >= 0 && pp < we) {
                    const int blk = p.block_table[min(ib, p.nb - 1) * p.bt_stride + pp / p.block_size];
                    off = (long long)blk * p.block_stride + (long long)(pp % p.block_size) * p.token_stride;
                }
                sh.kv_off[warp][j] = off;
            }
            if (warp == 0 && lane == 0) {
                sh.item0_b = ib;
                sh.item0_kvh = ikvh;
                sh.item0_chunk = ichunk;
                sh.item0_all = (ib >= 0 && ppw <= kPreRuns * 16) ? 1 : 0;
            }
            if (warp == 0 && lane < B) {
                const long long slot = sh.slot[lane];
                sh.slot_off[lane] = slot < 0 ? -1
                                             : (slot / p.block_size) * p.block_stride + (slot % p.block_size) * p.token_stride;
            }
        }
        // this warp's entry table: lanes fill entries in parallel (closed form per entry)
        int base = 0;
        for (int t = 0; t < 4; ++t) {
            const int n = phase_entries(p.ph[t], sh.row_a[t][warp], sh.row_b[t][warp]);
            for (int e = lane; e < n; e += 32)
                if (base + e < kMaxLayerEntries)
                    sh.ent_table[warp][base + e] = phase_entry(p.ph[t], sh.row_a[t][warp], sh.row_b[t][warp], e);
            base += n;
        }
        const int nlm = p.lm_head ? phase_entries(p.ph[kLM], sh.row_a[kLM][warp], sh.row_b[kLM][warp]) : 0;
        for (int e = lane; e < nlm; e += 32)
            if (e < kMaxLmEntries)
                sh.ent_table[warp][kMaxLayerEntries + e] = phase_entry(p.ph[kLM], sh.row_a[kLM][warp], sh.row_b[kLM][warp], e);
        if (lane == 0) {
            sh.ent_count[warp][0] = base;
            sh.ent_count[warp][1] = nlm;
            if (base > kMaxLayerEntries || nlm > kMaxLmEntries) {
                sh.abort_flag = 1;
                atomicCAS(p.ctrl + kCtrlStatus, 0u, (unsigned)kErrShape);
            }
        }
    }
    __syncthreads();

    Ctx c{p, sh, act, res, attn_scratch, ring_base + (size_t)(warp < kNW ? warp : 0) * p.ring_bytes, 0u, warp, lane, cta, ncta, nullptr};
    c.tag_base = (sh.epoch + 1u) << 7;

    if (warp == kNW) {
        producer_loop(c, ring_base);
    } else {
        // reset the argmax cells the *next* launch will use
        // (unconditionally: a launch without next_ids must not leave an older launch's keys behind)
        if (cta == 0 && tid < kMaxB) p.argkey[(size_t)((sh.epoch + 1u) & 1u) * kMaxB + tid] = 0ull;
        uint32_t consumed = 0;
        // One loop over the global phase index (4 per layer, then the lm_head) with a single call site
        // for every building block, so each is instantiated once and the instruction footprint of a
        // layer stays small enough for the instruction cache.
        const int nphases = p.L * 4 + 1;
        for (int gp = 0; gp < nphases; ++gp) {
            const int layer = gp >> 2;
            const int t = gp < p.L * 4 ? (gp & 3) : (int)kLM;
            if (t == kLM && !(p.lm_head || cta == 0)) break;
            const uint32_t tag = layer_tag(c, layer);
            const int par = layer & 1;
            unsigned long long* prof = nullptr;
            if (p.profile && tid == 0 && t != kLM) prof = p.profile + ((size_t)cta * p.L + layer) * kProfSlots;
            c.prof = prof;
            if (t == kQKV) {
                if (prof) prof[0] = global_ns();
                attention_prefetch(c, layer);
            }
            if (t == kO) {
                attention_phase<G>(c, layer);
                if (prof) prof[3] = global_ns();
            }
            // ---- stage the phase input into c.act
            const bool norm = (t == kQKV || t == kGU || t == kLM);
            if (norm) {
                const unsigned long long* src =
                    (t == kGU) ? p.ll_h1 + (size_t)par * B * p.H : p.ll_x + (size_t)par * B * p.H;
                const uint16_t* w = (t == kLM) ? p.final_norm
                                               : reinterpret_cast<const uint16_t*>(p.layers[layer * 6 + (t == kQKV ? 0 : 3)]);
                stage_norm<B>(c, src, tag, w, gp == 0);
            } else if (t == kO && !sh.two_level) {
                stage_attn_direct<B>(c, layer);
            } else {
                const bool attn = (t == kO);
                stage_copy<B>(c, attn ? p.ll_attn + (size_t)par * B * (p.QH * kD / 2) : p.ll_act + (size_t)par * B * p.I, tag,
                              attn ? p.QH * kD : p.I, attn);
            }
            if (prof) prof[1 + 2 * t + (t >= kO ? 1 : 0)] = global_ns();     // slots 1, 4, 6, 8
            if (t == kLM && cta == 0) {
                const uint16_t* act16 = reinterpret_cast<const uint16_t*>(c.act);
                for (int b = 0; b < p.nb; ++b)
                    for (int i = tid; i < p.H; i += kCT) p.out_hidden[b * p.H + i] = act16[(size_t)b * p.act_elems + i];
            }
            if (t != kLM || p.lm_head) gemv_phase<B, WF>(c, t, layer, consumed);
            if (prof) prof[2 + 2 * t + (t >= kO ? 1 : 0)] = global_ns();     // slots 2, 5, 7, 9
        }
    }
    __syncthreads();
    // The last CTA to finish publishes the greedy ids, optionally advances the step inputs in
    // place (device-driven generation), and opens the next launch's epoch.
    if (tid == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(p.ctrl + kCtrlDone, 1u);
        if (prev == (unsigned)ncta - 1u) {
            __threadfence();
            const bool ok = *((volatile unsigned int*)(p.ctrl + kCtrlStatus)) == 0;
            if (p.next_ids && p.lm_head && ok) {
                for (int b = 0; b < p.nb; ++b) {
                    const unsigned long long key =
                        *((volatile unsigned long long*)(p.argkey + (size_t)(sh.epoch & 1u) * kMaxB + b));
                    const long long id = (long long)(0xffffffffu - (uint32_t)key);
                    p.next_ids[b] = id;
                    if (p.advance) {
                        if (p.ids_i64) reinterpret_cast<long long*>(const_cast<void*>(p.input_ids))[b] = id;
                        else reinterpret_cast<int*>(const_cast<void*>(p.input_ids))[b] = (int)id;
                        const long long np = p.positions[b] + 1;
                        const_cast<long long*>(p.positions)[b] = np;
                        const_cast<int*>(p.seq_lens)[b] = p.seq_lens[b] + 1;
                        if (p.slot_mapping[b] >= 0 && np < (long long)p.max_seq_len) {
                            const long long blk = p.block_table[b * p.bt_stride + (int)(np / p.block_size)];
                            const_cast<long long*>(p.slot_mapping)[b] = blk * p.block_size + np % p.block_size;
                        }
                    }
                }
            }
            p.ctrl[kCtrlDone] = 0u;
            p.ctrl[kCtrlEpoch] = sh.epoch + 1u;
            __threadfence();
        }
    }
}


}  // namespace pk
#include "decode_fast.cuh"
#include "decode_batched.cuh"
namespace pk {

// One-CTA helper for tests of the failure path: polls a flagged word that nothing writes with the same
// bounded wait the decode kernels use; the wait runs out after `spin_limit` rounds and the status word
// of the workspace receives kErrBarrierTimeout.  It cannot hang.
__global__ void wait_probe_kernel(unsigned int* ctrl, const unsigned long long* never_written, unsigned spin_limit) {
    unsigned spins = 0;
    const uint32_t tag = 0xfffffff1u;       // no launch produces this tag
    for (;;) {
        const unsigned long long v = ld_flagged(never_written);
        if ((uint32_t)(v >> 32) == tag) return;
        if (++spins >= spin_limit) {
            atomicCAS(ctrl + kCtrlStatus, 0u, (unsigned)kErrBarrierTimeout);
            return;
        }
    }
}

// ------------------------------------------------------------------ host side
struct ModelGeom {
    int H, I, L, QH, KVH, V, wfmt;
    float eps;
};

struct WsLayout {
    size_t ctrl, argkey, x, qkv, attn, h1, act, part, fast, total;
};
// Region of the tensor-core batched kernel.
struct BatchedLayout {
    size_t bctrl, argkey, c_qkv, c_o, c_gu, c_down, x, h1, xn, attn, act, part, total;
};
// Region of the batch-1 fast kernel (its own words; never shared with the generic kernel's buffers).
struct FastLayout {
    size_t fctrl, argkey, x, qkv, h1, act, part, gate, total;
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static int fast_nc(const ModelGeom& g) {
    const int kvh = g.KVH > 0 ? g.KVH : 1;
    const int nc = g.QH == g.KVH ? fast::kNominalCtas / kvh : (fast::kNominalCtas - g.QH) / kvh;      // Widths::NC
    return nc < 16 ? nc : 16;
}

static FastLayout fast_layout(const ModelGeom& g) {
    FastLayout l{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += align_up(bytes, 256);
        return at;
    };
    const size_t nqkv = (size_t)(g.QH + 2 * g.KVH) * kD;
    const int G = g.QH / (g.KVH > 0 ? g.KVH : 1);
    l.fctrl = take(256);
    l.argkey = take(256);
    l.x = take(2 * (size_t)g.H * 4);
    l.qkv = take(2 * nqkv * 4);
    l.h1 = take(2 * (size_t)g.H * 4);
    l.act = take(2 * (size_t)g.I * 4);
    l.part = take(2 * (size_t)g.KVH * fast_nc(g) * G * 66 * 8);
    l.gate = take(2 * (size_t)g.QH * kD * 4);       // merged attention output words
    l.total = off;
    return l;
}

static int batched_np(int B) { return B <= 16 ? 16 : (B <= 32 ? 32 : 64); }

// One layout for every batch size (sized for the maximum): the fp32 sums must be zero when a launch starts, and the
// kernel leaves them zero, which only holds across launches of different batch sizes if a buffer never moves.
static BatchedLayout batched_layout(const ModelGeom& g, int /*B*/) {
    const int B = batched::kMaxReq;
    BatchedLayout l{};
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t at = off;
        off += align_up(bytes, 256);
        return at;
    };
    const size_t NP = (size_t)batched_np(B);
    const size_t nqkv = (size_t)(g.QH + 2 * g.KVH) * kD;
    const int G = g.QH / (g.KVH > 0 ? g.KVH : 1);
    l.bctrl = take(256);
    l.argkey = take(8 * batched::kMaxReq);
    l.c_qkv = take(NP * nqkv * 4);
    l.c_o = take(NP * g.H * 4);
    l.c_gu = take(NP * 2 * g.I * 4);
    l.c_down = take(NP * g.H * 4);
    l.x = take(NP * g.H * 2);
    l.h1 = take(NP * g.H * 2);
    l.xn = take(NP * g.H * 2);
    l.attn = take(NP * g.QH * kD * 2);
    l.act = take(NP * g.I * 2);
    l.part = take((size_t)B * g.KVH * batched::kNcB * G * 66 * 4);
    l.total = off;
    return l;
}

static WsLayout ws_layout(const ModelGeom& g, int B) {
    WsLayout l{};
    size_t off = 0;
    l.ctrl = off;
    off += 256;
    l.argkey = off;
    off += align_up(sizeof(unsigned long long) * 2 * kMaxB, 256);
    const int G = g.QH / g.KVH;
    const size_t nqkv = (size_t)(g.QH + 2 * g.KVH) * kD;
    auto take = [&](size_t words) {
        const size_t at = off;
        off += align_up(words * 2 * sizeof(unsigned long long), 256);   // x2: layer parity
        return at;
    };
    l.x = take((size_t)B * g.H);
    l.qkv = take((size_t)B * nqkv);
    l.attn = take((size_t)B * g.QH * kD / 2);
    l.h1 = take((size_t)B * g.H);
    l.act = take((size_t)B * g.I);
    l.part = take((size_t)B * g.KVH * kNCMax * G * 66);
    l.fast = off;
    off += fast_layout(g).total;
    l.total = off;
    return l;
}

// The tensor-core kernel's region lies behind the CUDA-core kernels' region (batch 8), so one workspace serves every
// kernel and a caller may alternate batch sizes on it; the control words at the front are shared.
static size_t tc_offset(const ModelGeom& g) { return align_up(ws_layout(g, kMaxB).total, 256); }
static size_t batched_ws_bytes(const ModelGeom& g, int B) { return tc_offset(g) + batched_layout(g, B).total; }
static bool batched_eligible(const ModelGeom& g) {
    if (g.KVH <= 0 || g.QH % g.KVH) return false;
    const int G = g.QH / g.KVH;
    return (G == 1 || G == 3) && g.H % 64 == 0 && g.I % 64 == 0 && (g.QH * kD) % 64 == 0 && g.H <= 4096;
}

struct DeviceInfo {
    bool valid = false;
    int sm_count = 0, coop = 0, major = 0, minor = 0, smem_optin = 0;
};
static std::mutex g_mu;
static unsigned long long* g_profile = nullptr;   // optional stage-timestamp buffer (debug aid)
static size_t g_profile_bytes = 0;
static std::unordered_map<int, DeviceInfo> g_devinfo;
struct WsState {
    size_t bytes = 0;               // zeroed size
    unsigned long long sig = 0;     // geometry the workspace was last used with
    unsigned long long launches = 0;
    int kb = 0;                     // kernel batch of the last CUDA-core launch (fixes the offsets of its buffers)
};
static std::unordered_map<const void*, WsState> g_ws_ready;     // workspace pointers already zeroed
// largest dynamic shared memory opted in, per (device, kernel): the attribute belongs to the device's context
static std::unordered_map<unsigned long long, int> g_kernel_smem;
static unsigned g_spin_limit = kSpinLimit;
static int g_tc_min_batch = 0;       // smallest batch pk_decode_step hands to the tensor-core kernel; 0: by model size (below)
static int g_fast_warps = -1;        // batch-1 fast path: -1 = not decided yet (environment), 0 = off, 7 / 8 = consumer warps per CTA

static unsigned long long geom_sig(const ModelGeom& g) {
    unsigned long long h = 1469598103934665603ull;
    const int v[7] = {g.H, g.I, g.L, g.QH, g.KVH, g.V, g.wfmt};
    for (int i = 0; i < 7; ++i) h = (h ^ (unsigned long long)(unsigned)v[i]) * 1099511628211ull;
    return h | 1ull;
}

static unsigned long long smem_key(int dev, const void* fn) {
    return ((unsigned long long)(unsigned)dev << 56) ^ (unsigned long long)reinterpret_cast<uintptr_t>(fn);
}

// Opt a kernel in to `smem` bytes of dynamic shared memory on the current device (once per device and size).
static int ensure_smem(const void* fn, size_t smem) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lk(g_mu);
    int& cur = g_kernel_smem[smem_key(dev, fn)];
    if ((int)smem > cur) {
        e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        cur = (int)smem;
    }
    return 0;
}

// Zero the workspace in stream order when it is new, when it was last used with another geometry (the
// fast kernel's 16-bit tags only tell consecutive launches of one geometry apart), when the CUDA-core kernels'
// buffers move because the kernel batch changed (`kb`: 1, 2, 3, 4 or 8; their offsets depend on it, and stale
// words of another layout must never be mistaken for tagged words; 0 = the tensor-core kernel, whose region
// is fixed) and every 2^24 launches (so that the launch epoch inside the tags never wraps).
static int ensure_workspace(void* ws, size_t ws_bytes, size_t need, const ModelGeom& g, cudaStream_t stream, int kb = 0) {
    std::lock_guard<std::mutex> lk(g_mu);
    WsState& st = g_ws_ready[ws];
    const unsigned long long sig = geom_sig(g);
    const bool moved = kb != 0 && st.kb != 0 && st.kb != kb;
    if (st.bytes < need || st.sig != sig || moved || st.launches >= (1ull << 24)) {
        cudaError_t e = cudaMemsetAsync(ws, 0, ws_bytes, stream);
        if (e != cudaSuccess) return (int)e;
        st.bytes = ws_bytes;
        st.sig = sig;
        st.launches = 0;
    }
    if (kb != 0) st.kb = kb;
    ++st.launches;
    return 0;
}

static int device_info(DeviceInfo& out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceInfo& d = g_devinfo[dev];
    if (!d.valid) {
        if ((e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&d.coop, cudaDevAttrCooperativeLaunch, dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&d.major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&d.minor, cudaDevAttrComputeCapabilityMinor, dev)) != cudaSuccess) return (int)e;
        if ((e = cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess)
            return (int)e;
        d.valid = true;
    }
    out = d;
    return 0;
}

typedef void (*KernelFn)(const DecodeParams);
static KernelFn pick_kernel(int B, int G, int WF) {
#define PK_CASE(b, g)                                            \
    if (B == b && G == g && WF == 0) return decode_step_kernel<b, g, 0>; \
    if (B == b && G == g && WF == 1) return decode_step_kernel<b, g, 1>;
#ifndef PK_DECODE_FAST_ONLY      // development builds that only need the batch-1 fast kernel compile in seconds
    PK_CASE(1, 1) PK_CASE(2, 1) PK_CASE(3, 1) PK_CASE(4, 1) PK_CASE(8, 1)
    PK_CASE(1, 3) PK_CASE(2, 3) PK_CASE(3, 3) PK_CASE(4, 3) PK_CASE(8, 3)
#endif
#undef PK_CASE
    return nullptr;
}

// Fill the per-phase staging descriptors for a ring of `rw` bytes per consumer warp.
static int make_phases_with(const ModelGeom& g, int entry_max, int rm, PhaseDesc (&ph)[kNumPhaseTypes]) {
    auto rowbytes = [&](int K) { return g.wfmt ? (int)align_up((size_t)K + K / 32, 16) : K * 2; };
    struct Spec { int nrows, K, pair, widx; long long pair_rows; };
    const int nqkv = (g.QH + 2 * g.KVH) * kD;
    const Spec spec[kNumPhaseTypes] = {
        {nqkv, g.H, 0, 1, 0}, {g.H, g.QH * kD, 0, 2, 0}, {g.I, g.H, 1, 4, g.I}, {g.H, g.I, 0, 5, 0}, {g.V, g.H, 0, -1, 0}};
    for (int t = 0; t < kNumPhaseTypes; ++t) {
        PhaseDesc& d = ph[t];
        d = PhaseDesc{};
        d.nrows = spec[t].nrows;
        d.kact = spec[t].K;
        if (spec[t].K % 32) return kErrShape;
        d.rowbytes = rowbytes(spec[t].K);
        d.kchunks = d.rowbytes / 16;
        d.pair = spec[t].pair;
        d.widx = spec[t].widx;
        d.pair_off = spec[t].pair_rows * (long long)d.rowbytes;
        const int unit = d.rowbytes * (d.pair ? 2 : 1);
        int R = entry_max / unit;
        const int rcap = d.pair ? rm / 2 : rm;
        if (R > rcap) R = rcap;
        if (R >= 1) {
            d.rows_per_entry = R;
            d.nseg = 1;
            d.segchunks = d.kchunks;
        } else {
            if (g.wfmt) return kErrShape;   // packed MXFP8 rows are not split along K
            const int part_max_chunks = entry_max / (d.pair ? 2 : 1) / 16 / 32 * 32;
            if (part_max_chunks < 32) return kErrResidency;
            int nseg = (d.kchunks + part_max_chunks - 1) / part_max_chunks;
            int segc = ((d.kchunks + nseg - 1) / nseg + 31) / 32 * 32;
            nseg = (d.kchunks + segc - 1) / segc;
            d.rows_per_entry = 1;
            d.nseg = nseg;
            d.segchunks = segc;
        }
    }
    return 0;
}

// Entries per consumer warp (worst CTA) for one layer / for the lm_head under the given descriptors.
static void worst_entry_counts(const PhaseDesc (&ph)[kNumPhaseTypes], int ncta, int& per_layer, int& lm) {
    auto count = [&](const PhaseDesc& d) {
        const int rows_cta = (d.nrows + ncta - 1) / ncta;
        const int rpw = (rows_cta + kNW - 1) / kNW;
        return d.nseg == 1 ? (rpw + d.rows_per_entry - 1) / d.rows_per_entry : rpw * d.nseg;
    };
    per_layer = 0;
    for (int t = 0; t < 4; ++t) per_layer += count(ph[t]);
    lm = count(ph[kLM]);
}

// Pick the smallest entry size (small entries lose little ring space at the wrap point, which an
// entry never straddles) whose per-warp schedule still fits the in-kernel entry tables.
static int make_phases(const ModelGeom& g, int rw, int ncta, int rm, PhaseDesc (&ph)[kNumPhaseTypes]) {
    int rc = kErrShape;
    int first = rw / 2 / 512 * 512;
    if (first > 8192) first = 8192;
    if (first < 1024) return kErrResidency;
    for (int entry_max = first; entry_max <= rw / 2; entry_max *= 2) {
        rc = make_phases_with(g, entry_max, rm, ph);
        if (rc) continue;
        int per_layer = 0, lm = 0;
        worst_entry_counts(ph, ncta, per_layer, lm);
        if (per_layer <= kMaxLayerEntries && lm <= kMaxLmEntries) return 0;
        rc = kErrShape;
    }
    return rc;
}

struct StepArgs {
    cudaStream_t stream;
    int B;
    const void* input_ids; int ids_i64;
    const void* positions; const void* seq_lens; const void* block_table; int bt_stride; const void* slot_mapping;
    const void* layers; const void* embed; const void* embed_lookup; const void* final_norm; const void* kv;
    long long k_off, v_off, block_stride, token_stride, head_stride; int block_size;
    const void* cos_sin; int cs_fp32;
    void* out_hidden; void* logits; void* next_ids; void* layer_outputs;
    void* ws; size_t ws_bytes; int max_seq_len; int lm_head; int advance;
    int path = 0;         // 0: chosen by batch size, 1: tensor-core kernel, 2: CUDA-core kernels
};

// ---- batch-1 fast path (decode_fast.cuh) --------------------------------------------------------
constexpr int kFastNotEligible = -7777;

static int fast_warps() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_fast_warps < 0) {
        const char* e = std::getenv("PK_DECODE_FAST");        // "0" = generic kernel only, "7" / "8" = consumer warps per CTA
        g_fast_warps = e ? std::atoi(e) : 7;
        if (g_fast_warps != 0 && g_fast_warps != 7 && g_fast_warps != 8) g_fast_warps = 7;
    }
    return g_fast_warps;
}

template <class W, int NW, int WF>
static int fast_launch_t(const ModelGeom& g, const StepArgs& a, const DeviceInfo& di, const WsLayout& lay) {
    using namespace fast;
    // the attention items take the first NC * KVH CTAs, the head merges the last QH
    if (di.sm_count < kNominalCtas || di.sm_count < W::NC * W::KVH + (W::G == 1 ? 0 : W::QH)) return kFastNotEligible;
    constexpr int ACT = W::H > W::I ? W::H : W::I;
    constexpr size_t kAttnWords = (size_t)attn_words<W, NW>();
    const size_t fixed = align_up(sizeof(FShared<NW>), 128) + align_up((size_t)W::H * 2, 128) + align_up((size_t)ACT * 2, 128) +
                         2 * align_up((size_t)W::H * 4, 128) + align_up(kAttnWords * 4, 128);
    if ((size_t)di.smem_optin < fixed + (size_t)NW * 4096) return kFastNotEligible;
    const int rw = (int)(((size_t)di.smem_optin - fixed) / NW / 128 * 128);
    // every entry must fit the ring (an empty ring restarts at its base)
#define PK_ENT(T) (fast_row_bytes<WF>(Ph<W, NW, T>::K) * Ph<W, NW, T>::RPE * (Ph<W, NW, T>::PAIR ? 2 : 1))
    const int ent[5] = {PK_ENT(kQKV), PK_ENT(kO), PK_ENT(kGU), PK_ENT(kDown) / down_ks<W, WF>(), PK_ENT(kLM)};
#undef PK_ENT
    for (int t = 0; t < 5; ++t)
        if (ent[t] > rw) return kFastNotEligible;
    const size_t smem = fixed + (size_t)NW * rw;
    auto fn = decode_fast_kernel<W, NW, WF>;
    int rc = ensure_smem(reinterpret_cast<const void*>(fn), smem);
    if (rc) return rc;
    rc = ensure_workspace(a.ws, a.ws_bytes, lay.total, g, a.stream, 1);      // the batch-1 layout
    if (rc) return rc;

    const FastLayout fl = fast_layout(g);
    unsigned char* ws = static_cast<unsigned char*>(a.ws);
    unsigned char* fw = ws + lay.fast;
    FastParams p{};
    p.layers = static_cast<const unsigned long long*>(a.layers);
    p.kv = static_cast<const unsigned long long*>(a.kv);
    p.embed = a.embed;
    p.embed_bf16 = static_cast<const uint16_t*>(a.embed_lookup ? a.embed_lookup : a.embed);
    p.final_norm = static_cast<const uint16_t*>(a.final_norm);
    p.input_ids = a.input_ids;
    p.positions = static_cast<const long long*>(a.positions);
    p.seq_lens = static_cast<const int*>(a.seq_lens);
    p.block_table = static_cast<const int*>(a.block_table);
    p.slot_mapping = static_cast<const long long*>(a.slot_mapping);
    p.cos_sin = a.cos_sin;
    p.out_hidden = static_cast<uint16_t*>(a.out_hidden);
    p.logits = static_cast<uint16_t*>(a.logits);
    p.next_ids = static_cast<long long*>(a.next_ids);
    p.layer_outputs = static_cast<uint16_t*>(a.layer_outputs);
    p.profile = (g_profile && g_profile_bytes >= (size_t)di.sm_count * g.L * kProfSlots * 8) ? g_profile : nullptr;
    p.ctrl = reinterpret_cast<unsigned int*>(ws + lay.ctrl);
    p.fctrl = reinterpret_cast<unsigned int*>(fw + fl.fctrl);
    p.argkey = reinterpret_cast<unsigned long long*>(fw + fl.argkey);
    p.w_x = reinterpret_cast<uint32_t*>(fw + fl.x);
    p.w_qkv = reinterpret_cast<uint32_t*>(fw + fl.qkv);
    p.w_h1 = reinterpret_cast<uint32_t*>(fw + fl.h1);
    p.w_act = reinterpret_cast<uint32_t*>(fw + fl.act);
    p.w_part = reinterpret_cast<unsigned long long*>(fw + fl.part);
    p.w_attn = reinterpret_cast<uint32_t*>(fw + fl.gate);
    p.k_off = a.k_off;
    p.v_off = a.v_off;
    p.block_stride = a.block_stride;
    p.token_stride = a.token_stride;
    p.head_stride = a.head_stride;
    p.block_size = a.block_size;
    p.bt_stride = a.bt_stride;
    p.ids_i64 = a.ids_i64 ? 1 : 0;
    p.cs_fp32 = a.cs_fp32 ? 1 : 0;
    p.L = g.L;
    p.V = g.V;
    p.lm_head = (a.lm_head && (a.logits || a.next_ids)) ? 1 : 0;
    p.advance = (a.advance && p.lm_head && a.next_ids) ? 1 : 0;
    p.max_seq_len = a.max_seq_len;
    p.ring_bytes = rw;
    p.spin_limit = g_spin_limit;
    p.eps = g.eps;
    void* args[] = {&p};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(fn), dim3(di.sm_count), dim3((NW + 1) * 32), args,
                                                smem, a.stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return e == cudaErrorCooperativeLaunchTooLarge ? (int)kErrResidency : (int)e;
    }
    return (int)cudaPeekAtLastError();
}

// Batch 1, bf16 weights, one of the model widths the fast kernel is instantiated for: returns the launch
// status, or kFastNotEligible when the generic kernel has to take the step.
static int fast_launch(const ModelGeom& g, const StepArgs& a, const DeviceInfo& di, const WsLayout& lay) {
    const int nw = fast_warps();
    if (nw == 0 || g.L > kMaxLayers) return kFastNotEligible;
    using W135 = fast::Widths<576, 1536, 9, 3>;
    using W360 = fast::Widths<960, 2560, 15, 5>;
    using W17 = fast::Widths<2048, 8192, 32, 32>;
    const bool is135 = g.H == 576 && g.I == 1536 && g.QH == 9 && g.KVH == 3;
    const bool is360 = g.H == 960 && g.I == 2560 && g.QH == 15 && g.KVH == 5;
    const bool is17 = g.H == 2048 && g.I == 8192 && g.QH == 32 && g.KVH == 32;
    if (g.wfmt) {       // MXFP8 weights: seven consumer warps only
        if (is135) return fast_launch_t<W135, 7, 1>(g, a, di, lay);
        if (is360) return fast_launch_t<W360, 7, 1>(g, a, di, lay);
        if (is17) return fast_launch_t<W17, 7, 1>(g, a, di, lay);
        return kFastNotEligible;
    }
    if (is17) return fast_launch_t<W17, 7, 0>(g, a, di, lay);
    if (is135) return nw == 8 ? fast_launch_t<W135, 8, 0>(g, a, di, lay) : fast_launch_t<W135, 7, 0>(g, a, di, lay);
    if (is360) return nw == 8 ? fast_launch_t<W360, 8, 0>(g, a, di, lay) : fast_launch_t<W360, 7, 0>(g, a, di, lay);
    return kFastNotEligible;
}

// ---- tensor-core batched path (decode_batched.cuh): up to 64 requests in one launch -------------------
template <int NP, int G, int WF>
static int batched_launch_t(const ModelGeom& g, const StepArgs& a, const DeviceInfo& di) {
    using namespace batched;
    const size_t need = batched_ws_bytes(g, a.B);
    if (a.ws_bytes < need) return kErrScratch;
    constexpr int NW = kThreadsB / 32;
    const size_t item_words = (size_t)NW * ((G + 2) * 32 + G * 16);      // per-warp q/k/v + probabilities
    const size_t scratch_words = item_words > (size_t)g.H ? item_words : (size_t)g.H;
    const size_t smem = 1024 + (size_t)staging_bytes(NP) + align_up(sizeof(BShared), 128) +
                        align_up(scratch_words * 4, 128);
    if (smem > (size_t)di.smem_optin) return kErrResidency;
    auto fn = decode_batched_kernel<NP, G, WF>;
    int rc = ensure_smem(reinterpret_cast<const void*>(fn), smem);
    if (rc) return rc;
    rc = ensure_workspace(a.ws, a.ws_bytes, need, g, a.stream);
    if (rc) return rc;
    const BatchedLayout bl = batched_layout(g, a.B);
    unsigned char* ws = static_cast<unsigned char*>(a.ws);
    unsigned char* bw = ws + tc_offset(g);
    BParams p{};
    p.layers = static_cast<const unsigned long long*>(a.layers);
    p.kv = static_cast<const unsigned long long*>(a.kv);
    p.embed = static_cast<const unsigned char*>(a.embed);
    p.embed_bf16 = static_cast<const uint16_t*>(a.embed_lookup ? a.embed_lookup : a.embed);
    p.final_norm = static_cast<const uint16_t*>(a.final_norm);
    p.input_ids = a.input_ids;
    p.positions = static_cast<const long long*>(a.positions);
    p.seq_lens = static_cast<const int*>(a.seq_lens);
    p.block_table = static_cast<const int*>(a.block_table);
    p.slot_mapping = static_cast<const long long*>(a.slot_mapping);
    p.cos_sin = a.cos_sin;
    p.out_hidden = static_cast<uint16_t*>(a.out_hidden);
    p.logits = static_cast<uint16_t*>(a.logits);
    p.next_ids = static_cast<long long*>(a.next_ids);
    p.layer_outputs = static_cast<uint16_t*>(a.layer_outputs);
    p.profile = (g_profile && g_profile_bytes >= (size_t)di.sm_count * g.L * kProfSlots * 8) ? g_profile : nullptr;
    p.ctrl = reinterpret_cast<unsigned int*>(ws);
    p.bctrl = reinterpret_cast<unsigned int*>(bw + bl.bctrl);
    p.argkey = reinterpret_cast<unsigned long long*>(bw + bl.argkey);
    p.c_qkv = reinterpret_cast<float*>(bw + bl.c_qkv);
    p.c_o = reinterpret_cast<float*>(bw + bl.c_o);
    p.c_gu = reinterpret_cast<float*>(bw + bl.c_gu);
    p.c_down = reinterpret_cast<float*>(bw + bl.c_down);
    p.x = reinterpret_cast<uint16_t*>(bw + bl.x);
    p.h1 = reinterpret_cast<uint16_t*>(bw + bl.h1);
    p.xn = reinterpret_cast<uint16_t*>(bw + bl.xn);
    p.attn = reinterpret_cast<uint16_t*>(bw + bl.attn);
    p.act = reinterpret_cast<uint16_t*>(bw + bl.act);
    p.part = reinterpret_cast<float*>(bw + bl.part);
    p.k_off = a.k_off;
    p.v_off = a.v_off;
    p.block_stride = a.block_stride;
    p.token_stride = a.token_stride;
    p.head_stride = a.head_stride;
    p.block_size = a.block_size;
    p.bs_shift = -1;
    for (int sft = 0; sft < 16; ++sft)
        if ((1 << sft) == a.block_size) p.bs_shift = sft;
    p.bt_stride = a.bt_stride;
    p.ids_i64 = a.ids_i64 ? 1 : 0;
    p.cs_fp32 = a.cs_fp32 ? 1 : 0;
    p.H = g.H; p.I = g.I; p.L = g.L; p.QH = g.QH; p.KVH = g.KVH; p.V = g.V; p.G = G;
    p.nb = a.B;
    p.wfmt = g.wfmt;
    p.lm_head = (a.lm_head && (a.logits || a.next_ids)) ? 1 : 0;
    p.advance = (a.advance && p.lm_head && a.next_ids) ? 1 : 0;
    p.max_seq_len = a.max_seq_len;
    p.spin_limit = g_spin_limit;
    p.eps = g.eps;
    // GEMM phases: rows, K and row pitch of each weight matrix
    const int nqkv = (g.QH + 2 * g.KVH) * kD;
    const int rows[5] = {nqkv, g.H, 2 * g.I, g.H, g.V};
    const int Ks[5] = {g.H, g.QH * kD, g.H, g.I, g.H};
    const int widx[5] = {1, 2, 4, 5, -1};
    for (int t = 0; t < 5; ++t) {
        GemmDesc& d = p.gd[t];
        d.rows = rows[t];
        d.K = Ks[t];
        d.widx = widx[t];
        d.rowbytes = g.wfmt ? (int)align_up((size_t)Ks[t] + Ks[t] / 32, 16) : Ks[t] * 2;
    }
    void* args[] = {&p};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(fn), dim3(di.sm_count), dim3(kThreadsB), args,
                                                smem, a.stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return e == cudaErrorCooperativeLaunchTooLarge ? (int)kErrResidency : (int)e;
    }
    return (int)cudaPeekAtLastError();
}

static int batched_launch(const ModelGeom& g, const StepArgs& a, const DeviceInfo& di) {
    const int G = g.QH / g.KVH;
    if ((G != 1 && G != 3) || g.H % 64 || g.I % 64 || (g.QH * kD) % 64 || g.H > 4096) return kErrShape;
    const int NP = batched_np(a.B);
#define PK_BCASE(np, gg)                                                                      \
    if (NP == np && G == gg) return g.wfmt ? batched_launch_t<np, gg, 1>(g, a, di) : batched_launch_t<np, gg, 0>(g, a, di);
    PK_BCASE(16, 1) PK_BCASE(32, 1) PK_BCASE(64, 1) PK_BCASE(16, 3) PK_BCASE(32, 3) PK_BCASE(64, 3)
#undef PK_BCASE
    return kErrShape;
}

static int decode_launch(const ModelGeom& g, const StepArgs& a) {
    if (a.B < 1 || a.B > batched::kMaxReq) return kErrBatch;
    if (a.path == 2 && a.B > kMaxB) return kErrBatch;
    // measured cross-over: 4 requests for the small models, 2 where a layer's weights are large enough to hide the
    // grid barriers (hidden >= 2048: SmolLM2-1.7B)
    const int tc_min = g_tc_min_batch > 0 ? g_tc_min_batch : (g.H >= 2048 ? 2 : 4);
    const bool tc = a.path == 1 || a.B > kMaxB ||
                    (a.path == 0 && a.B >= tc_min && batched_eligible(g) && a.ws_bytes >= batched_ws_bytes(g, a.B));
    if (tc) {
        // the tensor-core kernel: always from 9 requests on, from g_tc_min_batch on when the geometry and the
        // workspace allow it (same argument checks as below)
        if (a.max_seq_len < 1 || a.max_seq_len > kMaxSeq) return kErrMaxSeq;
        if (!a.input_ids || !a.positions || !a.seq_lens || !a.block_table || !a.slot_mapping || !a.layers || !a.embed ||
            !a.final_norm || !a.kv || !a.cos_sin || !a.out_hidden || !a.ws)
            return kErrNull;
        if (g.H <= 0 || g.I <= 0 || g.L < 1 || g.L > kMaxLayers || g.QH <= 0 || g.KVH <= 0 || g.QH % g.KVH || g.V <= 0 ||
            (g.wfmt != 0 && g.wfmt != 1))
            return kErrShape;
        if (a.block_size <= 0 || a.bt_stride < 1 || (long long)a.bt_stride * a.block_size < a.max_seq_len) return kErrBlock;
        if (a.k_off % 8 || a.v_off % 8 || a.block_stride % 8 || a.token_stride % 8 || a.head_stride % 8 || a.k_off < 0 ||
            a.v_off < 0 || a.block_stride < 0 || a.token_stride < 0 || a.head_stride < 0)
            return kErrAlign;
        auto mis = [](const void* q) { return q && (reinterpret_cast<uintptr_t>(q) % 16) != 0; };
        if (mis(a.layers) || mis(a.embed) || mis(a.final_norm) || mis(a.ws) || mis(a.out_hidden) || mis(a.kv) ||
            mis(a.embed_lookup) || mis(a.layer_outputs) || mis(a.logits))
            return kErrAlign;
        DeviceInfo dib;
        int rcb = device_info(dib);
        if (rcb) return rcb;
        if (dib.major != 10) return kErrArch;
        if (!dib.coop) return kErrCoop;
        return batched_launch(g, a, dib);
    }
    const int KB = a.B <= 4 ? a.B : kMaxB;      // kernel batch: exact up to 4, the batch-8 kernel (padded) beyond
    if (a.max_seq_len < 1 || a.max_seq_len > kMaxSeq) return kErrMaxSeq;
    if (!a.input_ids || !a.positions || !a.seq_lens || !a.block_table || !a.slot_mapping || !a.layers || !a.embed ||
        !a.final_norm || !a.kv || !a.cos_sin || !a.out_hidden || !a.ws)
        return kErrNull;
    if (g.H <= 0 || g.I <= 0 || g.L < 1 || g.L > kMaxLayers || g.QH <= 0 || g.KVH <= 0 || g.QH % g.KVH || g.V <= 0 ||
        g.H % 32 || g.I % 32 || (g.QH * kD) % 32 || g.H > kNormRegs * kCT)
        return kErrShape;
    const int G = g.QH / g.KVH;
    if (g.wfmt != 0 && g.wfmt != 1) return kErrShape;
    KernelFn fn = pick_kernel(KB, G, g.wfmt);
    if (!fn) return kErrShape;
    if (a.block_size <= 0 || a.bt_stride < 1 || (long long)a.bt_stride * a.block_size < a.max_seq_len) return kErrBlock;
    if (a.k_off % 8 || a.v_off % 8 || a.block_stride % 8 || a.token_stride % 8 || a.head_stride % 8 || a.k_off < 0 ||
        a.v_off < 0 || a.block_stride < 0 || a.token_stride < 0 || a.head_stride < 0)
        return kErrAlign;
    auto mis16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) % 16) != 0; };
    if (mis16(a.layers) || mis16(a.embed) || mis16(a.final_norm) || mis16(a.ws) || mis16(a.out_hidden) || mis16(a.kv) ||
        (a.embed_lookup && mis16(a.embed_lookup)) || (a.layer_outputs && mis16(a.layer_outputs)) ||
        (a.logits && mis16(a.logits)))
        return kErrAlign;
    const WsLayout lay = ws_layout(g, KB);
    if (a.ws_bytes < lay.total) return kErrScratch;

    DeviceInfo di;
    int rc = device_info(di);
    if (rc) return rc;
    if (di.major != 10) return kErrArch;
    if (!di.coop) return kErrCoop;

    // batch 1: the kernel specialised for the SmolLM2-135M / 360M / 1.7B widths (bf16 weights with the tied embedding as
    // lm_head, or MXFP8 weights with the bf16 embedding rows given separately)
    if (a.B == 1 && ((g.wfmt == 0 && (!a.embed_lookup || a.embed_lookup == a.embed)) || (g.wfmt == 1 && a.embed_lookup))) {
        rc = fast_launch(g, a, di, lay);
        if (rc != kFastNotEligible) return rc;
    }

    // shared memory: fixed part + per-warp rings
    const int act_elems = g.H > g.I ? g.H : g.I;
    const size_t fixed = align_up(sizeof(Shared), 128) + align_up((size_t)KB * act_elems * 2, 128) +
                         align_up((size_t)KB * g.H * 4, 128) + (size_t)kAttnScratchWords * 4;
    if ((size_t)di.smem_optin < fixed + (size_t)kNW * 2048) return kErrResidency;
    int rw = (int)(((size_t)di.smem_optin - fixed) / kNW / 512 * 512);
    DecodeParams p{};
    // grid: one CTA per SM, but never more CTAs than rows in the smallest projection, so every
    // CTA takes part in every hand-off (which bounds how far any CTA can run ahead of another)
    int ncta = di.sm_count;
    {
        const int rows[4] = {(g.QH + 2 * g.KVH) * kD, g.H, g.I, g.H};
        for (int t = 0; t < 4; ++t) ncta = rows[t] < ncta ? rows[t] : ncta;
    }
    if (ncta < 1) return kErrShape;
    rc = make_phases(g, rw, ncta, row_cap(KB), p.ph);
    if (rc) return rc;
    const size_t smem = fixed + (size_t)kNW * rw;

    rc = ensure_smem(reinterpret_cast<const void*>(fn), smem);
    if (rc) return rc;
    rc = ensure_workspace(a.ws, a.ws_bytes, lay.total, g, a.stream, KB);
    if (rc) return rc;

    unsigned char* ws = static_cast<unsigned char*>(a.ws);
    p.layers = static_cast<const unsigned long long*>(a.layers);
    p.kv = static_cast<const unsigned long long*>(a.kv);
    p.embed = static_cast<const uint16_t*>(a.embed);
    p.embed_bf16 = static_cast<const uint16_t*>(a.embed_lookup ? a.embed_lookup : a.embed);
    p.final_norm = static_cast<const uint16_t*>(a.final_norm);
    p.input_ids = a.input_ids;
    p.positions = static_cast<const long long*>(a.positions);
    p.seq_lens = static_cast<const int*>(a.seq_lens);
    p.block_table = static_cast<const int*>(a.block_table);
    p.slot_mapping = static_cast<const long long*>(a.slot_mapping);
    p.cos_sin = a.cos_sin;
    p.out_hidden = static_cast<uint16_t*>(a.out_hidden);
    p.logits = static_cast<uint16_t*>(a.logits);
    p.next_ids = static_cast<long long*>(a.next_ids);
    p.layer_outputs = static_cast<uint16_t*>(a.layer_outputs);
    p.ctrl = reinterpret_cast<unsigned int*>(ws + lay.ctrl);
    p.argkey = reinterpret_cast<unsigned long long*>(ws + lay.argkey);
    p.ll_x = reinterpret_cast<unsigned long long*>(ws + lay.x);
    p.ll_qkv = reinterpret_cast<unsigned long long*>(ws + lay.qkv);
    p.ll_attn = reinterpret_cast<unsigned long long*>(ws + lay.attn);
    p.ll_h1 = reinterpret_cast<unsigned long long*>(ws + lay.h1);
    p.ll_act = reinterpret_cast<unsigned long long*>(ws + lay.act);
    p.ll_part = reinterpret_cast<unsigned long long*>(ws + lay.part);
    p.k_off = a.k_off;
    p.v_off = a.v_off;
    p.block_stride = a.block_stride;
    p.token_stride = a.token_stride;
    p.head_stride = a.head_stride;
    p.block_size = a.block_size;
    p.bt_stride = a.bt_stride;
    p.ids_i64 = a.ids_i64 ? 1 : 0;
    p.cs_fp32 = a.cs_fp32 ? 1 : 0;
    p.H = g.H; p.I = g.I; p.L = g.L; p.QH = g.QH; p.KVH = g.KVH; p.V = g.V; p.B = KB; p.G = G;
    p.nb = a.B;
    p.wfmt = g.wfmt;
    p.lm_head = (a.lm_head && (a.logits || a.next_ids)) ? 1 : 0;
    p.advance = (a.advance && p.lm_head && a.next_ids) ? 1 : 0;
    p.max_seq_len = a.max_seq_len;
    p.ring_bytes = rw;
    p.profile = (g_profile && g_profile_bytes >= (size_t)ncta * g.L * kProfSlots * 8) ? g_profile : nullptr;
    p.act_elems = act_elems;
    p.spin_limit = g_spin_limit;
    p.eps = g.eps;

    void* args[] = {&p};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(fn), dim3(ncta), dim3(kThreads), args,
                                                smem, a.stream);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return e == cudaErrorCooperativeLaunchTooLarge ? (int)kErrResidency : (int)e;
    }
    return (int)cudaPeekAtLastError();
}

static const char* status_string(int status) {
    switch (status) {
        case kOk: return "ok";
        case kErrBatch: return "batch_must_be_1_to_64";
        case kErrMaxSeq: return "max_seq_len_must_be_1_to_8192";
        case kErrNull: return "null_device_pointer";
        case kErrCoop: return "cooperative_launch_unsupported";
        case kErrResidency: return "grid_exceeds_resident_capacity_or_shared_memory";
        case kErrArch: return "kernel_requires_sm100";
        case kErrAlign: return "kv_offsets_or_pointers_not_16_byte_aligned";
        case kErrScratch: return "scratch_smaller_than_workspace_bytes";
        case kErrBlock: return "block_size_or_stride_invalid";
        case kErrBarrierTimeout: return "device_wait_timed_out";
        case kErrShape: return "unsupported_model_geometry";
        case kErrStaticScratch: return "request_needs_more_than_the_2_MiB_built_in_scratch";
        default: return cudaGetErrorString(static_cast<cudaError_t>(status));
    }
}

static const ModelGeom kGeom135{576, 1536, 30, 9, 3, 49152, 0, 1e-5f};
static const ModelGeom kGeom360{960, 2560, 32, 15, 5, 49152, 0, 1e-5f};

}  // namespace pk

// ================================================================== C ABI
using namespace pk;

struct PkDecodeModel {
    int hidden, intermediate, layers, q_heads, kv_heads, vocab;
    int weight_format;   // 0 = bf16, 1 = MXFP8 packed rows
    float eps;
};

struct PkDecodeArgs {
    void* stream;
    int batch;
    const void* input_ids; int ids_i64;
    const void* positions; const void* seq_lens; const void* block_table; int bt_stride; const void* slot_mapping;
    const void* layers; const void* embed; const void* embed_lookup; const void* final_norm; const void* kv_layers;
    long long k_off, v_off, block_stride, token_stride, head_stride; int block_size;
    const void* cos_sin; int cs_fp32;
    void* out_hidden; void* logits; void* next_ids; void* layer_outputs;
    void* workspace; size_t workspace_bytes; int max_seq_len; int lm_head; int advance;
};

static ModelGeom to_geom(const PkDecodeModel* m) {
    return ModelGeom{m->hidden, m->intermediate, m->layers, m->q_heads, m->kv_heads, m->vocab, m->weight_format, m->eps};
}

extern "C" size_t pk_decode_workspace_bytes(const PkDecodeModel* m, int max_batch) {
    if (!m || max_batch < 1 || max_batch > batched::kMaxReq || m->kv_heads <= 0) return 0;
    // below the tensor-core cross-over (4 requests; 2 for hidden >= 2048) only the CUDA-core kernels run; from there on
    // the workspace also holds the tensor-core kernel's region (behind the CUDA-core kernels' batch-8 region, which batches 5..7 need anyway)
    const ModelGeom g = to_geom(m);
    if (max_batch < (g.H >= 2048 ? 2 : 4)) return ws_layout(g, max_batch).total;
    return batched_ws_bytes(g, max_batch);
}

extern "C" int pk_decode_step(const PkDecodeModel* m, const PkDecodeArgs* a) {
    if (!m || !a) return kErrNull;
    StepArgs s{static_cast<cudaStream_t>(a->stream), a->batch, a->input_ids, a->ids_i64, a->positions, a->seq_lens,
               a->block_table, a->bt_stride, a->slot_mapping, a->layers, a->embed, a->embed_lookup, a->final_norm,
               a->kv_layers, a->k_off, a->v_off, a->block_stride, a->token_stride, a->head_stride, a->block_size,
               a->cos_sin, a->cs_fp32, a->out_hidden, a->logits, a->next_ids, a->layer_outputs, a->workspace,
               a->workspace_bytes, a->max_seq_len, a->lm_head, a->advance};
    return decode_launch(to_geom(m), s);
}

// Same step on the tensor-core kernel whatever the batch (pk_decode_step picks it from
// pk_decode_set_tc_min_batch requests on, default 4, and always above 8).  The workspace must have
// pk_decode_workspace_bytes(model, n) bytes for some n >= max(4, batch).
extern "C" int pk_decode_step_tc(const PkDecodeModel* m, const PkDecodeArgs* a) {
    if (!m || !a) return kErrNull;
    StepArgs s{static_cast<cudaStream_t>(a->stream), a->batch, a->input_ids, a->ids_i64, a->positions, a->seq_lens,
               a->block_table, a->bt_stride, a->slot_mapping, a->layers, a->embed, a->embed_lookup, a->final_norm,
               a->kv_layers, a->k_off, a->v_off, a->block_stride, a->token_stride, a->head_stride, a->block_size,
               a->cos_sin, a->cs_fp32, a->out_hidden, a->logits, a->next_ids, a->layer_outputs, a->workspace,
               a->workspace_bytes, a->max_seq_len, a->lm_head, a->advance};
    s.path = 1;
    return decode_launch(to_geom(m), s);
}

// Same step on the CUDA-core kernels only (1..8 requests), whatever pk_decode_set_tc_min_batch says.
extern "C" int pk_decode_step_cc(const PkDecodeModel* m, const PkDecodeArgs* a) {
    if (!m || !a) return kErrNull;
    StepArgs s{static_cast<cudaStream_t>(a->stream), a->batch, a->input_ids, a->ids_i64, a->positions, a->seq_lens,
               a->block_table, a->bt_stride, a->slot_mapping, a->layers, a->embed, a->embed_lookup, a->final_norm,
               a->kv_layers, a->k_off, a->v_off, a->block_stride, a->token_stride, a->head_stride, a->block_size,
               a->cos_sin, a->cs_fp32, a->out_hidden, a->logits, a->next_ids, a->layer_outputs, a->workspace,
               a->workspace_bytes, a->max_seq_len, a->lm_head, a->advance};
    s.path = 2;
    return decode_launch(to_geom(m), s);
}

// Smallest batch pk_decode_step / mk_decode hand to the tensor-core kernel (1..9; 9 = only above 8 requests;
// 0 = the default: 2 for hidden >= 2048, else 4).
extern "C" void pk_decode_set_tc_min_batch(int n) { g_tc_min_batch = n < 0 ? 0 : (n > kMaxB + 1 ? kMaxB + 1 : n); }

// Zero a workspace in stream order and mark it ready (also done implicitly on first use).
extern "C" int pk_decode_workspace_init(void* workspace, size_t bytes, void* stream) {
    if (!workspace) return kErrNull;
    cudaError_t e = cudaMemsetAsync(workspace, 0, bytes, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lk(g_mu);
    WsState& st = g_ws_ready[workspace];
    st = WsState{};
    st.bytes = bytes;
    return 0;
}

// Forget a workspace pointer (call before freeing it, so a later allocation at the same address is re-zeroed).
extern "C" void pk_decode_workspace_forget(void* workspace) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_ws_ready.erase(workspace);
}

// Synchronise the stream and return the device-side status word of the workspace (0 = ok,
// 9110 = a bounded device wait gave up).  The word is cleared so the workspace can be reused.
extern "C" int pk_decode_status(void* workspace, void* stream) {
    if (!workspace) return kErrNull;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned int word = 0;
    cudaError_t e = cudaMemcpyAsync(&word, static_cast<unsigned int*>(workspace) + kCtrlStatus, sizeof(word),
                                    cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return (int)e;
    if (word) {
        e = cudaMemsetAsync(workspace, 0, 256, s);   // control words only; tags stay monotonic via the epoch reset to 0
        if (e != cudaSuccess) return (int)e;
        std::lock_guard<std::mutex> lk(g_mu);
        g_ws_ready.erase(workspace);                 // force a full re-zero before the next launch
    }
    return (int)word;
}

extern "C" const char* pk_status_string(int status) { return status_string(status); }

// Tuning / test knobs (process-wide).
// Batch-1 steps of the SmolLM2-135M / 360M / 1.7B widths run on the specialised kernel with `warps` (7 or 8)
// consumer warps per CTA; 0 sends every step to the generic kernel.  Default: environment PK_DECODE_FAST, else 7
// (7 consumer warps + the producer warp = 256 threads measured 8 % faster than 8 + 1).
extern "C" int pk_decode_set_fast_path(int warps) {
    if (warps != 0 && warps != 7 && warps != 8) return kErrShape;
    std::lock_guard<std::mutex> lk(g_mu);
    g_fast_warps = warps;
    return 0;
}
// Bound (polling rounds) of every device-side wait of later launches; 0 restores the default.
extern "C" void pk_decode_set_spin_limit(unsigned rounds) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_spin_limit = rounds ? rounds : kSpinLimit;
}
// Failure-path probe: one CTA polls a word of `workspace` that nothing writes, with the decode kernels'
// bounded wait; after `rounds` polls it gives up and the workspace status becomes 9110, which
// pk_decode_status() then returns (and clears).  Never hangs; touches nothing else.
extern "C" int pk_decode_wait_probe(void* workspace, size_t bytes, unsigned rounds, void* stream) {
    if (!workspace) return kErrNull;
    if (bytes < 512 || (reinterpret_cast<uintptr_t>(workspace) % 16) != 0) return kErrScratch;
    if (rounds < 1 || rounds > (1u << 20)) return kErrShape;
    unsigned int* ctrl = static_cast<unsigned int*>(workspace);
    const unsigned long long* word = reinterpret_cast<const unsigned long long*>(static_cast<unsigned char*>(workspace) + 128);
    wait_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(ctrl, word, rounds);
    return (int)cudaGetLastError();
}

// Debug aid: when set (device buffer of at least ctas * layers * 24 * 8 bytes), thread 0 of every CTA
// stamps %globaltimer at each phase boundary of each layer: [cta][layer][12].  Pass null to disable.
extern "C" void pk_decode_set_profile(void* buffer, size_t bytes) {
    std::lock_guard<std::mutex> lk(g_mu);
    g_profile = static_cast<unsigned long long*>(buffer);
    g_profile_bytes = buffer ? bytes : 0;
}

extern "C" int pk_decode_query(int* sm_count, int* coop, int* major, int* minor, int* smem_optin, int* threads,
                               int* consumer_warps) {
    DeviceInfo di;
    const int rc = device_info(di);
    if (rc) return rc;
    if (sm_count) *sm_count = di.sm_count;
    if (coop) *coop = di.coop;
    if (major) *major = di.major;
    if (minor) *minor = di.minor;
    if (smem_optin) *smem_optin = di.smem_optin;
    if (threads) *threads = kThreads;
    if (consumer_warps) *consumer_warps = kNW;
    return 0;
}

// ---- drop-in entry points with the reference's signatures -------------------------------------
// SmolLM2-135M: prime_kernels/decode_megakernel/csrc/megakernel.cu:833-927
extern "C" int mk_query(int* sm_count, int* coop, int* active_per_sm, int* major, int* minor, int* regs,
                        int* static_smem) {
    DeviceInfo di;
    const int rc = device_info(di);
    if (rc) return rc;
    cudaFuncAttributes fa{};
    cudaError_t e = cudaFuncGetAttributes(&fa, reinterpret_cast<const void*>(pick_kernel(4, 3, 0)));
    if (e != cudaSuccess) return (int)e;
    *sm_count = di.sm_count;
    *coop = di.coop;
    *active_per_sm = 1;
    *major = di.major;
    *minor = di.minor;
    *regs = fa.numRegs;
    *static_smem = (int)fa.sharedSizeBytes;
    return 0;
}

extern "C" size_t mk_workspace_bytes(int B, int max_seq_len) {
    (void)B;
    (void)max_seq_len;
    return batched_ws_bytes(kGeom135, kMaxB);      // batches 4..8 run on the tensor-core kernel when the scratch has this size
}

extern "C" int mk_decode(void* stream, int B, const void* input_ids, int ids_i64, const void* positions,
                         const void* seq_lens, const void* block_table, int bt_stride, const void* slot_mapping,
                         const void* layers, const void* embed, const void* final_norm, void* const* kv_layers,
                         long long k_off, long long v_off, long long block_stride, long long token_stride,
                         long long head_stride, int block_size, const void* cos_sin, int cs_fp32, void* out_hidden,
                         void* scratch, size_t scratch_bytes, int max_seq_len) {
    if (B < 1 || B > kMaxB) return kErrBatch;      // the reference's entry takes 1..8 requests
    StepArgs s{static_cast<cudaStream_t>(stream), B, input_ids, ids_i64, positions, seq_lens, block_table, bt_stride,
               slot_mapping, layers, embed, nullptr, final_norm, kv_layers, k_off, v_off, block_stride, token_stride,
               head_stride, block_size, cos_sin, cs_fp32, out_hidden, nullptr, nullptr, nullptr, scratch, scratch_bytes,
               max_seq_len, 0, 0};
    return decode_launch(kGeom135, s);
}

extern "C" const char* mk_status_string(int status) { return status_string(status); }

// SmolLM2-360M: prime_kernels/decode_megakernel_360m/csrc/block360_kernel.inc:849-938
extern "C" size_t decode360_workspace_bytes() { return ws_layout(kGeom360, kMaxB).total; }
extern "C" size_t decode360_debug_bytes() { return 16; }   // stage dumps are not produced; accepted and ignored

extern "C" int decode360(void* stream, int B, const void* input_ids, const void* embed, const void* final_norm,
                         const void* positions, const void* seq_lens, const void* block_table, int bt_stride,
                         const void* slot_mapping, const void* layers, void* const* kv, long long k_off, long long v_off,
                         long long block_stride, long long token_stride, long long head_stride, int block_size,
                         const void* cos_sin, int cs_fp32, void* out_hidden, void* layer_outputs, void* scratch,
                         size_t scratch_bytes, void* debug, size_t debug_bytes, int max_seq_len,
                         int debug_layer_index) {
    (void)debug;
    (void)debug_bytes;
    if (debug_layer_index < -1 || debug_layer_index >= kGeom360.L) return kErrBlock;
    if (B < 1 || B > kMaxB) return kErrBatch;      // the reference's entry takes 1..8 requests
    StepArgs s{static_cast<cudaStream_t>(stream), B, input_ids, 0, positions, seq_lens, block_table, bt_stride,
               slot_mapping, layers, embed, nullptr, final_norm, kv, k_off, v_off, block_stride, token_stride,
               head_stride, block_size, cos_sin, cs_fp32, out_hidden, nullptr, nullptr, layer_outputs, scratch,
               scratch_bytes, max_seq_len, 0, 0};
    return decode_launch(kGeom360, s);
}

extern "C" const char* decode360_status_string(int status) { return status_string(status); }

// ---- decode step for callers that must not allocate device memory ------------------------------
// The workspace of pk_decode_step normally comes from the caller (the Python surface allocates it with
// torch).  Inference servers typically hand every byte that is left after start-up to their KV-cache
// pool, and some embedders call the C ABI from places where the CUDA allocator is off limits (for
// example a pre-sized arena with no allocator behind it); neither can produce a scratch buffer later.
// For them the library carries a small scratch area of its own: a file-scope device array, resident on
// every GPU that loads the library until the process exits.
//
// Limits and rules:
//  * the step's workspace must fit kStaticScratchBytes (2 MiB): SmolLM2-360M at batch 1 and SmolLM2-135M
//    up to batch 2 fit, SmolLM2-1.7B does not; larger requests are refused with status 9112;
//  * the first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
//    device current) and remembers it; make that first call outside any stream capture;
//  * all calls on a device share the one array.  It keeps what the previous call left (the launch epoch
//    must survive from call to call); the status and completion words are cleared in stream order on
//    every call.  Calls that overlap on the GPU (different streams) race on it: serialise them;
//  * nothing on this path calls cudaMalloc, cudaFree or any allocating library routine.
namespace pk {
constexpr size_t kStaticScratchBytes = size_t(2) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static std::unordered_map<int, void*> g_static_scratch_addr;   // device ordinal -> device address
}  // namespace pk

extern "C" size_t pk_decode_static_scratch_bytes() { return kStaticScratchBytes; }

extern "C" int pk_decode_step_static(const PkDecodeModel* m, const PkDecodeArgs* a) {
    if (!m || !a) return kErrNull;
    if (m->kv_heads <= 0 || a->batch < 1) return kErrBatch;
    const ModelGeom g = to_geom(m);
    if (a->batch > kMaxB) return kErrBatch;
    if (ws_layout(g, a->batch <= 4 ? a->batch : kMaxB).total > kStaticScratchBytes) return kErrStaticScratch;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_static_scratch_addr.find(dev);
        if (it == g_static_scratch_addr.end()) {
            // In host code the array's name is only a handle; the kernel needs its device address.
            e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess) return (int)e;
            g_static_scratch_addr[dev] = ptr;
            g_ws_ready[ptr].bytes = kStaticScratchBytes;   // zero-initialised at module load
        } else {
            ptr = it->second;
        }
    }
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    // status and completion counter start every call at zero; the epoch word before them is kept
    e = cudaMemsetAsync(static_cast<unsigned int*>(ptr) + kCtrlStatus, 0, 2 * sizeof(unsigned int), stream);
    if (e != cudaSuccess) return (int)e;
    StepArgs s{stream, a->batch, a->input_ids, a->ids_i64, a->positions, a->seq_lens, a->block_table, a->bt_stride,
               a->slot_mapping, a->layers, a->embed, a->embed_lookup, a->final_norm, a->kv_layers, a->k_off, a->v_off,
               a->block_stride, a->token_stride, a->head_stride, a->block_size, a->cos_sin, a->cs_fp32, a->out_hidden,
               a->logits, a->next_ids, a->layer_outputs, ptr, kStaticScratchBytes, a->max_seq_len, a->lm_head, a->advance};
    s.path = 2;      // the static scratch holds the CUDA-core kernels' workspace only
    return decode_launch(g, s);
}

// Status word of the built-in scratch on the current device (synchronises `stream`).
extern "C" int pk_decode_static_status(void* stream) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    void* ptr = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_static_scratch_addr.find(dev);
        if (it == g_static_scratch_addr.end()) return 0;
        ptr = it->second;
    }
    unsigned int word = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    e = cudaMemcpyAsync(&word, static_cast<unsigned int*>(ptr) + kCtrlStatus, sizeof(word), cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return (int)e;
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return (int)e;
    return (int)word;
}
