// Batch-1 bf16 decode step with compile-time model widths (included by decode_megakernel.cu).
//
// Same arithmetic contract and the same dataflow idea as decode_step_kernel (weights streamed through
// per-warp shared-memory rings with bulk async copies, activations handed from CTA to CTA through
// self-validating words in L2, no grid barrier, every wait bounded), specialised so that one step of a
// small model is a short chain of short phases:
//
//  * hidden / intermediate / head counts are template constants: every loop bound, divisor and stride
//    folds, and the whole kernel is a few thousand instructions, so a layer iteration stays inside the
//    instruction cache (the generic kernel is ~200 KB of code per instantiation and refetches it from L2
//    every layer);
//  * a producer warp feeds the per-warp weight rings (one lane per ring; issuing bulk copies can block for
//    a while when the copy engine's queue is full at a phase boundary, which must not happen to a warp on
//    the dependent chain: letting every consumer warp refill its own ring was measured 5 % slower);
//  * bf16 activations travel as 32-bit words [tag:16 | bf16:16] and are polled with 16-byte loads: four
//    values per load, each word validating itself (no reliance on 16-byte atomicity).  fp32 split-KV
//    partials travel as 64-bit words [tag:32 | fp32] polled two per 16-byte load;
//  * five hand-offs per layer instead of six: split-KV partials are always merged by the consumers while
//    they stage the O-projection input (at most Widths::NC chunks per kv head; longer contexts get
//    longer chunks), so there is no separate merge stage;
//  * activation and residual staging buffers alternate between phases, which removes the barrier that
//    protected them from the previous phase's stragglers (two barriers per norm phase, one per copy phase).
//
// Reference behaviour followed: see the header of decode_megakernel.cu (same rounding points).
#pragma once

namespace pk {
namespace fast {

constexpr int kFE = 8;             // ring entries in flight per warp
constexpr int kPre = 4;            // 16-position runs per warp whose cache offsets are resolved at kernel start
constexpr int kKvPtrs = 64;        // per-layer KV base pointers cached in shared memory
constexpr int kNominalCtas = 128;  // compile-time lower bound of the grid (the host checks it)

template <int H_, int I_, int QH_, int KVH_>
struct Widths {
    static constexpr int H = H_, I = I_, QH = QH_, KVH = KVH_, G = QH_ / KVH_;
    static constexpr int NQKV = (QH_ + 2 * KVH_) * kD;
    static constexpr int AD = QH_ * kD;                           // attention output width (K of the O projection)
    // max chunks per kv head: a chunk is one run of 16 positions per warp up to 16 x NW x NC positions, longer beyond.
    // Grouped-query widths keep the QH merging CTAs free of attention items; with one query head per kv head the
    // items may use every CTA (a merging CTA then merges after its own item, which no other item waits for).
    static constexpr int NCRAW = (QH_ == KVH_) ? kNominalCtas / KVH_ : (kNominalCtas - QH_) / KVH_;
    static constexpr int NC = NCRAW < 16 ? NCRAW : 16;
    static_assert(QH_ % KVH_ == 0 && H_ % 32 == 0 && I_ % 32 == 0, "unsupported widths");
};

// Floats of the attention scratch: an item's working set (per-warp partials, staged q/k/v, probabilities).
template <class W, int NW>
__host__ __device__ constexpr int attn_words() {
    return (((NW * W::G * 66 + 3) & ~3) + (W::G + 2) * kD + (W::G + 2) * 32 + NW * W::G * 16 + 3) & ~3;
}

struct FastParams {
    const unsigned long long* layers;   // device table [L][6]
    const unsigned long long* kv;       // device table [L]
    const void* embed;                  // lm_head matrix: [V, H] bf16, or packed MXFP8 rows
    const uint16_t* embed_bf16;         // [V, H] bf16 rows for the input look-up (= embed for bf16 weights)
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
    unsigned long long* profile;
    unsigned int* ctrl;                 // control words shared with the generic kernel (status)
    unsigned int* fctrl;                // this kernel's own control words: epoch, completion counter
    unsigned long long* argkey;         // [2]
    uint32_t* w_x;                      // [2][H]      words [tag16 | bf16]
    uint32_t* w_qkv;                    // [2][NQKV]
    uint32_t* w_h1;                     // [2][H]
    uint32_t* w_act;                    // [2][I]
    unsigned long long* w_part;         // [2][KVH][NC][G][66]  words [tag32 | fp32]
    uint32_t* w_attn;                   // [2][QH * 64]         merged attention output, words [tag16 | bf16]
    long long k_off, v_off, block_stride, token_stride, head_stride;
    int block_size, bt_stride, ids_i64, cs_fp32;
    int L, V, lm_head, advance, max_seq_len, ring_bytes;
    unsigned spin_limit;
    float eps;
};

enum { kFctrlEpoch = 0, kFctrlDone = 1 };

template <int NW>
struct FShared {
    uint64_t full[NW][kFE];
    uint64_t empty[NW][kFE];
    uint32_t ent_off[NW][kFE];
    uint32_t ent_foot[NW][kFE];
    int row_a[kNumPhaseTypes][NW];
    int row_b[kNumPhaseTypes][NW];
    float red[NW];
    float cs[64];                          // cos[32], sin[32] of this step's position
    unsigned long long lm_key[NW];
    unsigned long long kv_ptr[kKvPtrs];
    unsigned long long norm_ptr[2 * kMaxLayers + 1];   // norm1 / norm2 weight pointers of every layer, then the final norm
    unsigned long long mat_ptr[kMaxLayers][4];         // qkv, o, gate_up, down weight pointers of every layer
    long long kv_off[NW][kPre * 16];       // cache element offsets (without the kv-head term) of the warp's first runs
    long long slot_off;                    // cache element offset of the new token; -1 = skip the write
    long long tok;
    int seq, pos, nc, lc;
    int item_kvh, item_chunk;              // this CTA's attention item; item_kvh < 0: none
    volatile int abort_flag;
    uint32_t epoch;
};

// ------------------------------------------------------------------ hand-off words
__device__ __forceinline__ uint4 ld_packet(const void* p) {
    uint4 v;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_word(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void ld_flagged2(const unsigned long long* p, unsigned long long& a, unsigned long long& b) {
    asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// all four words of a packet carry the tag T (= tag16 << 16)
__device__ __forceinline__ bool packet_ok(const uint4 v, uint32_t T) {
    return ((((v.x ^ T) | (v.y ^ T)) | ((v.z ^ T) | (v.w ^ T))) >> 16) == 0u;
}

// ------------------------------------------------------------------ per-thread kernel state
template <int NW>
struct FC {
    const FastParams& p;
    FShared<NW>& sh;
    uint4* act[2];      // bf16 activations of the current phase, alternating between phases
    float* res[2];      // fp32 copy of the residual stream: [0] = x (layer input), [1] = h1
    float* attn;        // attention scratch / staged split-KV partials
    unsigned char* ring;
    uint32_t T16;       // ((epoch % 511) + 1) << 23: the epoch part of a 16-bit tag, already in the high half
    uint32_t T32;       // (epoch + 1) << 7: the epoch part of a 32-bit tag
    int warp, lane, cta, ncta;
    uint32_t consumed;          // ring entries this warp has used so far
    uint2 nwv[3];               // this thread's norm weights of the *next* norm phase (fetched one phase ahead)
    uint32_t pre_off;           // ring offset of the upcoming phase's first entry, valid when pre_ok
    bool pre_ok;                // that entry has landed (checked before the staging of the phase)
    unsigned long long* prof;
};

// barrier of the NW consumer warps (the producer warp does not take part)
template <int NW>
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory"); }

template <int NW>
__device__ __forceinline__ bool f_aborted(const FC<NW>& c) { return c.sh.abort_flag != 0; }
template <int NW>
__device__ __forceinline__ void f_raise(FC<NW>& c, int code) {
    c.sh.abort_flag = 1;
    atomicCAS(c.p.ctrl + kCtrlStatus, 0u, (unsigned)code);
}
// periodic check inside a spin loop; returns true when the wait must be given up
template <int NW>
__device__ __forceinline__ bool f_give_up(FC<NW>& c, unsigned spins) {
    if (f_aborted(c)) return true;
    if (*((volatile unsigned int*)(c.p.ctrl + kCtrlStatus)) != 0) {
        c.sh.abort_flag = 1;
        return true;
    }
    if (spins >= c.p.spin_limit) {
        f_raise(c, kErrBarrierTimeout);
        return true;
    }
    return false;
}

template <int NW>
__device__ __forceinline__ uint32_t tag16(const FC<NW>& c, int layer) { return c.T16 | ((uint32_t)(layer + 1) << 16); }
template <int NW>
__device__ __forceinline__ uint32_t tag32(const FC<NW>& c, int layer) { return c.T32 + (uint32_t)layer + 1u; }

// Wait for up to N packets (ptr[u] == nullptr: slot unused).  While nothing has arrived only the first
// packet is polled (the CTAs that have no other work in a phase would otherwise multiply the polling
// traffic in L2 by N); once it is there all remaining ones are fetched together.
// `mid` runs once, warp-converged, after the first round of loads has been issued and before it is looked
// at: work that may block for a while (the ring refill: the copy engine's queue fills up when every warp
// refills at a phase boundary) then overlaps the L2 round trip of the poll instead of preceding it.
template <int N, int NW, typename Mid>
__device__ __forceinline__ void poll_packets(FC<NW>& c, const uint32_t* const (&ptr)[N], uint32_t T, uint4 (&out)[N], Mid mid) {
    unsigned need = 0;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        out[u] = make_uint4(0u, 0u, 0u, 0u);
        if (ptr[u] != nullptr) need |= 1u << u;
    }
    bool first_only = N > 1;
    unsigned cur = first_only ? (need & (0u - need)) : need;
    uint4 v[N];
#pragma unroll
    for (int u = 0; u < N; ++u)
        if (cur & (1u << u)) v[u] = ld_packet(ptr[u]);
    mid();
    if (f_aborted(c)) return;
    unsigned spins = 0;
    while (need) {
#pragma unroll
        for (int u = 0; u < N; ++u)
            if ((cur & (1u << u)) && packet_ok(v[u], T)) {
                out[u] = v[u];
                need &= ~(1u << u);
                first_only = false;
            }
        if (!need) break;
        if ((++spins & 255u) == 0 && f_give_up(c, spins)) return;
        cur = first_only ? (need & (0u - need)) : need;
#pragma unroll
        for (int u = 0; u < N; ++u)
            if (cur & (1u << u)) v[u] = ld_packet(ptr[u]);
    }
}
template <int N, int NW>
__device__ __forceinline__ void poll_packets(FC<NW>& c, const uint32_t* const (&ptr)[N], uint32_t T, uint4 (&out)[N]) {
    poll_packets<N>(c, ptr, T, out, [] {});
}

// Same for pairs of 64-bit flagged words [tag32 | fp32]; out[2u], out[2u+1] receive the payloads.
template <int N, int NW>
__device__ __forceinline__ void poll_flagged_pairs(FC<NW>& c, const unsigned long long* const (&ptr)[N], uint32_t tag,
                                                   uint32_t (&out)[2 * N], bool first_only = false) {
    unsigned need = 0;
#pragma unroll
    for (int u = 0; u < N; ++u) {
        out[2 * u] = out[2 * u + 1] = 0u;
        if (ptr[u] != nullptr) need |= 1u << u;
    }
    if (f_aborted(c)) return;
    unsigned spins = 0;
    while (need) {
        const unsigned cur = first_only ? (need & (0u - need)) : need;
        unsigned long long a[N], b[N];
#pragma unroll
        for (int u = 0; u < N; ++u)
            if (cur & (1u << u)) ld_flagged2(ptr[u], a[u], b[u]);
#pragma unroll
        for (int u = 0; u < N; ++u)
            if ((cur & (1u << u)) && (uint32_t)(a[u] >> 32) == tag && (uint32_t)(b[u] >> 32) == tag) {
                out[2 * u] = (uint32_t)a[u];
                out[2 * u + 1] = (uint32_t)b[u];
                need &= ~(1u << u);
                first_only = false;
            }
        if (need && (++spins & 255u) == 0 && f_give_up(c, spins)) return;
    }
}

template <int NW>
__device__ __forceinline__ bool f_wait_mbar(FC<NW>& c, uint64_t* bar, uint32_t parity) {
    if (mbar_probe(bar, parity)) return true;
    if (f_aborted(c)) return false;
    unsigned spins = 0;
    while (!mbar_test(bar, parity)) {
        if ((++spins & 255u) == 0 && f_give_up(c, spins)) return false;
    }
    return true;
}

// ------------------------------------------------------------------ weight schedule
// Phase constants.  Rows are dealt in contiguous shares: CTA, then warp (same rule as the generic kernel).
template <class W, int NW, int T>
struct Ph;
template <class W, int NW>
struct Ph<W, NW, kQKV> { static constexpr int K = W::H, WIDX = 1, PAIR = 1, RPE = 1; };   // unit = rows (d, d + 32) of a head
template <class W, int NW>
struct Ph<W, NW, kO> { static constexpr int K = W::AD, WIDX = 2, PAIR = 0, RPE = 2; };
template <class W, int NW>
struct Ph<W, NW, kGU> { static constexpr int K = W::H, WIDX = 4, PAIR = 1, RPE = ((NW >= 12 || W::H * 2 >= 4096) ? 1 : 3); };
template <class W, int NW>
struct Ph<W, NW, kDown> { static constexpr int K = W::I, WIDX = 5, PAIR = 0, RPE = (W::I * 2 > 4096 ? 1 : 2); };
template <class W, int NW>
struct Ph<W, NW, kLM> { static constexpr int K = W::H, WIDX = -1, PAIR = 0, RPE = ((NW >= 12 || W::H * 2 >= 4096) ? 2 : 4); };

// A bf16 row of the down projection longer than 8 KB travels as KS ring entries of K / KS weights each (a ring
// holds three 8 KB entries at the widest model); the consumer adds the parts' dot products before the epilogue.
template <class W, int WF>
__host__ __device__ constexpr int down_ks() { return (WF == 0 && W::I * 2 > 8192) ? 2 : 1; }

// bytes of one stored weight row: bf16, or packed MXFP8 ([K e4m3][K/32 e8m0], padded to 16 bytes)
template <int WF>
__host__ __device__ constexpr int fast_row_bytes(int K) { return WF ? ((K + K / 32 + 15) & ~15) : K * 2; }

template <class W, int NW, int WF>
__device__ __forceinline__ void phase_consts(int t, int& rowbytes, int& rpe, int& widx, int& ks) {
    ks = t == kDown ? down_ks<W, WF>() : 1;
    switch (t) {
        case kQKV: rowbytes = fast_row_bytes<WF>(Ph<W, NW, kQKV>::K); rpe = Ph<W, NW, kQKV>::RPE; widx = Ph<W, NW, kQKV>::WIDX; break;
        case kO: rowbytes = fast_row_bytes<WF>(Ph<W, NW, kO>::K); rpe = Ph<W, NW, kO>::RPE; widx = Ph<W, NW, kO>::WIDX; break;
        case kGU: rowbytes = fast_row_bytes<WF>(Ph<W, NW, kGU>::K); rpe = Ph<W, NW, kGU>::RPE; widx = Ph<W, NW, kGU>::WIDX; break;
        case kDown: rowbytes = fast_row_bytes<WF>(Ph<W, NW, kDown>::K); rpe = Ph<W, NW, kDown>::RPE; widx = Ph<W, NW, kDown>::WIDX; break;
        default: rowbytes = fast_row_bytes<WF>(Ph<W, NW, kLM>::K); rpe = Ph<W, NW, kLM>::RPE; widx = Ph<W, NW, kLM>::WIDX; break;
    }
}

template <int NW>
__device__ __forceinline__ void warp_share(int nrows, int cta, int ncta, int warp, int& a, int& b) {
    const int r0 = (int)((long long)nrows * cta / ncta);
    const int r1 = (int)((long long)nrows * (cta + 1) / ncta);
    const int n = r1 - r0;
    a = r0 + n * warp / NW;
    b = r0 + n * (warp + 1) / NW;
}

// Producer warp: lane w (< NW) feeds the ring of consumer warp w with that warp's entries in schedule
// order (4 phases per layer, then the lm_head), in closed form from the row shares.  All lanes run the same
// loop; every iteration a lane retires up to two consumed entries (non-blocking probes) and issues up to two
// new ones if its ring has room.  Nothing here waits on a consumer, so one slow ring never stalls the others.
template <class W, int NW, int WF>
__device__ void producer_loop(const FastParams& p, FShared<NW>& sh, unsigned char* ring_base, int lane) {
    const bool active = lane < NW;
    const int w = active ? lane : 0;
    const uint32_t RW = (uint32_t)p.ring_bytes;
    unsigned char* ring = ring_base + (size_t)w * RW;
    const uint64_t pol = evict_first_policy();
    int layer = 0, t = -1, row = 0, sub = 0;   // cursor: next entry is part `sub` of unit `row` of phase t in `layer`
    bool more = active;
    auto next_phase = [&]() {
        for (;;) {
            if (t == kLM) { more = false; return; }
            if (++t == 4) {
                ++layer;
                if (layer < p.L) t = 0;
                else if (p.lm_head) t = kLM;
                else { more = false; return; }
            }
            row = sh.row_a[t][w];
            if (row < sh.row_b[t][w]) return;
        }
    };
    if (more) next_phase();
    uint32_t issued = 0, tail = 0, head = 0, used = 0;
    unsigned idle = 0;
    for (;;) {
        bool progressed = false;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (tail < issued) {
                const uint32_t slot = tail % kFE;
                if (mbar_probe(&sh.empty[w][slot], (tail / kFE) & 1)) {
                    used -= sh.ent_foot[w][slot];
                    ++tail;
                    progressed = true;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            if (more) {
                int rowbytes, rpe, widx, ks;
                phase_consts<W, NW, WF>(t, rowbytes, rpe, widx, ks);
                const int nre = min(rpe, sh.row_b[t][w] - row);
                const uint32_t part = (uint32_t)(nre * rowbytes / ks);        // ks > 1 only with one row per entry
                const bool pair = t == kGU || t == kQKV;
                const uint32_t bytes = pair ? 2u * part : part;
                if (issued == tail) head = 0;      // empty ring: restart at its base, so any entry <= RW fits
                const uint32_t gap = (head + bytes > RW) ? RW - head : 0u;
                const uint32_t foot = bytes + gap;
                if (issued - tail < (uint32_t)kFE && used + foot <= RW) {
                    const uint32_t off = gap ? 0u : head;
                    const uint32_t slot = issued % kFE;
                    sh.ent_off[w][slot] = off;
                    sh.ent_foot[w][slot] = foot;
                    // weight pointers come from the shared-memory copy of the table: no global load in front of the copy
                    const unsigned char* base = widx < 0 ? reinterpret_cast<const unsigned char*>(p.embed)
                                                         : reinterpret_cast<const unsigned char*>(sh.mat_ptr[layer][t]);
                    // QKV units pair row d with row d + 32 of the same head; gate/up units pair row r with row I + r
                    const int row0 = t == kQKV ? ((row >> 5) << 6) + (row & 31) : row;
                    const size_t pair_off = (size_t)(t == kQKV ? 32 : W::I) * rowbytes;
                    const unsigned char* src = base + (size_t)row0 * rowbytes + (size_t)sub * part;
                    mbar_expect_tx(&sh.full[w][slot], bytes);
                    bulk_g2s(ring + off, src, part, &sh.full[w][slot], pol);
                    if (pair) bulk_g2s(ring + off + part, src + pair_off, part, &sh.full[w][slot], pol);
                    head = off + bytes;
                    if (head >= RW) head = 0;
                    used += foot;
                    ++issued;
                    if (++sub == ks) {
                        sub = 0;
                        row += rpe;
                        if (row >= sh.row_b[t][w]) next_phase();
                    }
                    progressed = true;
                }
            }
        }
        const bool done = !more;                 // everything issued; outstanding copies are drained below
        if (__all_sync(kFullMask, done)) break;
        idle = (progressed || done) ? 0 : idle + 1;
        // nothing to retire or issue: yield the issue slots to the consumer warp that shares this scheduler
        if (!__any_sync(kFullMask, progressed)) __nanosleep(kProducerIdleNs);
        if ((idle & 255u) == 255u && idle >= p.spin_limit) {
            sh.abort_flag = 1;
            atomicCAS(p.ctrl + kCtrlStatus, 0u, (unsigned)kErrBarrierTimeout);
        }
        if (__any_sync(kFullMask, sh.abort_flag != 0)) break;
    }
    // Drain: never leave the CTA while bulk copies into its shared memory are still in flight.
    if (active) {
        for (uint32_t n = tail; n < issued; ++n) {
            const uint32_t slot = n % kFE;
            unsigned spins = 0;
            while (!mbar_probe(&sh.full[w][slot], (n / kFE) & 1))
                if (++spins >= p.spin_limit) break;
        }
    }
}

// ------------------------------------------------------------------ GEMV
// NR staged rows of KC 16-byte chunks each times the activation vector, K split over the lanes.
template <int KC, int NR>
__device__ __forceinline__ void gemv_rows(const uint4* ep, const uint4* act, int lane, int nlive, float (&v)[8]) {
    constexpr int IT = (KC + 31) / 32;
    float acc[NR], acc2[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = acc2[r] = 0.f;
#pragma unroll 4
    for (int it = 0; it < IT; ++it) {
        const int ch = it * 32 + lane;
        const bool ok = (it + 1) * 32 <= KC || ch < KC;
        const uint4 a = ok ? act[ch] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint4 wv = (ok && r < nlive) ? ep[r * KC + ch] : make_uint4(0u, 0u, 0u, 0u);
            if (it & 1) acc2[r] = dot8_bf16(wv, a, acc2[r]);
            else acc[r] = dot8_bf16(wv, a, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) v[r] += acc[r] + acc2[r];     // v: zero, or the sum over the row's earlier parts
}

// The same for packed MXFP8 rows ([K e4m3][K/32 e8m0][pad]): a 16-byte chunk is 16 weights against two activation
// chunks; the chunk's partial sum is scaled by its E8M0 (one per 32 along K, i.e. per two chunks) - exact
// de-quantisation, fp32 accumulation.
template <int K, int NR, int RB>
__device__ __forceinline__ void gemv_rows_fp8(const uint4* ep, const uint4* act, int lane, int nlive, float (&v)[8]) {
    constexpr int KC = K / 16;
    constexpr int IT = (KC + 31) / 32;
    float acc[NR], acc2[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = acc2[r] = 0.f;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
        const int ch = it * 32 + lane;
        const bool ok = (it + 1) * 32 <= KC || ch < KC;
        const uint4 a0 = ok ? act[2 * ch] : make_uint4(0u, 0u, 0u, 0u);
        const uint4 a1 = ok ? act[2 * ch + 1] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            if (ok && r < nlive) {
                const unsigned char* row = reinterpret_cast<const unsigned char*>(ep) + r * RB;
                const uint4 wq = *reinterpret_cast<const uint4*>(row + ch * 16);
                const uint32_t sb = row[K + (ch >> 1)];
                const float scale = __uint_as_float(sb ? (sb << 23) : 0x00400000u);
                const float part = dot16_e4m3(wq, a0, a1, 0.f);
                if (it & 1) acc2[r] = fmaf(scale, part, acc2[r]);
                else acc[r] = fmaf(scale, part, acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) v[r] = acc[r] + acc2[r];
}

// One GEMV phase of one warp: its ring entries of phase type t at `layer`.  One body for all phase types
// (run-time t) so that the wait, the reduction and the ring refill exist once in the instruction stream;
// only the dot products (compile-time K) and the epilogues are switched.
template <class W, int NW, int WF>
__device__ __forceinline__ void gemv_phase(FC<NW>& c, const int t, int layer, const uint4* act, const float* res) {
    const FastParams& p = c.p;
    FShared<NW>& sh = c.sh;
    const int w = c.warp, lane = c.lane;
    const int ra = sh.row_a[t][w], rb = sh.row_b[t][w];
    const int par = layer & 1;
    int rowbytes, rpe, widx, ks;
    phase_consts<W, NW, WF>(t, rowbytes, rpe, widx, ks);
    uint32_t best = 0u;      // lm_head: bf16 order key << 16 | (0xffff - local row)
    bool gone = false;
#pragma unroll 1
    for (int row = ra; row < rb; row += rpe) {
        const int nre = min(rpe, rb - row);
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int part = 0; part < ks; ++part) {
            const uint32_t slot = c.consumed % kFE;
            uint32_t eoff = c.pre_off;
            if (!(row == ra && part == 0 && c.pre_ok)) {
                // after an abort the staged bytes are undefined: leave the phase (warp-uniform)
                if (!__all_sync(kFullMask, f_wait_mbar(c, &sh.full[w][slot], (c.consumed / kFE) & 1))) {
                    gone = true;
                    break;
                }
                eoff = sh.ent_off[w][slot];
            }
            const uint4* ep = reinterpret_cast<const uint4*>(c.ring + eoff);
            if constexpr (WF == 0) {
                constexpr int KSD = down_ks<W, 0>();
                constexpr int KCD = Ph<W, NW, kDown>::K / 8 / KSD;
                switch (t) {
                    case kQKV: gemv_rows<Ph<W, NW, kQKV>::K / 8, 2 * Ph<W, NW, kQKV>::RPE>(ep, act, lane, 2 * nre, v); break;
                    case kO: gemv_rows<Ph<W, NW, kO>::K / 8, Ph<W, NW, kO>::RPE>(ep, act, lane, nre, v); break;
                    case kGU: gemv_rows<Ph<W, NW, kGU>::K / 8, 2 * Ph<W, NW, kGU>::RPE>(ep, act, lane, 2 * nre, v); break;
                    case kDown: gemv_rows<KCD, Ph<W, NW, kDown>::RPE>(ep, act + part * KCD, lane, nre, v); break;
                    default: gemv_rows<Ph<W, NW, kLM>::K / 8, Ph<W, NW, kLM>::RPE>(ep, act, lane, nre, v); break;
                }
            } else {
                constexpr int nq = 2 * Ph<W, NW, kQKV>::RPE, no = Ph<W, NW, kO>::RPE, ng = 2 * Ph<W, NW, kGU>::RPE,
                              nd = Ph<W, NW, kDown>::RPE, nl = Ph<W, NW, kLM>::RPE;
                constexpr int kq = Ph<W, NW, kQKV>::K, ko = Ph<W, NW, kO>::K, kg = Ph<W, NW, kGU>::K, kd = Ph<W, NW, kDown>::K,
                              kl = Ph<W, NW, kLM>::K;
                switch (t) {
                    case kQKV: gemv_rows_fp8<kq, nq, fast_row_bytes<1>(kq)>(ep, act, lane, 2 * nre, v); break;
                    case kO: gemv_rows_fp8<ko, no, fast_row_bytes<1>(ko)>(ep, act, lane, nre, v); break;
                    case kGU: gemv_rows_fp8<kg, ng, fast_row_bytes<1>(kg)>(ep, act, lane, 2 * nre, v); break;
                    case kDown: gemv_rows_fp8<kd, nd, fast_row_bytes<1>(kd)>(ep, act, lane, nre, v); break;
                    default: gemv_rows_fp8<kl, nl, fast_row_bytes<1>(kl)>(ep, act, lane, nre, v); break;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.empty[w][slot]);      // every lane's loads of this entry have been consumed
            ++c.consumed;
        }
        if (gone) break;
        // lane 4 j ends up with the total of staged row j (j < 8)
        const float mine = transpose_reduce<8>(v, lane);
        const int vj = lane >> 2;
        // pair entries stage nre first rows (gate / dim d), then nre second rows (up / dim d + 32)
        const float mine_up = __shfl_sync(kFullMask, mine, ((vj + nre) << 2) & 31);
        if ((lane & 3) == 0 && vj < nre) {
            const int r = row + vj;
            if (t == kQKV) {
                // unit r = (head, j): projection outputs of dims j and j + 32 rounded to bf16 (HF linear output),
                // q and k heads rotated here (HF apply_rotary_pos_emb rounding), v passed through
                const int hd = r >> 5, j = r & 31;
                float x0 = round_bf16(mine), x1 = round_bf16(mine_up);
                if (hd < W::QH + W::KVH) {
                    const float cs = sh.cs[j], sn = sh.cs[32 + j];
                    const float y0 = rope_elem(x0, x1, cs, sn, true);
                    x1 = rope_elem(x1, x0, cs, sn, false);
                    x0 = y0;
                }
                uint32_t* dst = p.w_qkv + par * W::NQKV + hd * kD + j;
                st_word(dst, f32_to_bf16_bits(x0) | tag16(c, layer));
                st_word(dst + 32, f32_to_bf16_bits(x1) | tag16(c, layer));
            } else if (t == kO) {
                // h1 = bf16( x + bf16(o_proj) )
                const float h = __fadd_rn(res[r], round_bf16(mine));
                st_word(p.w_h1 + par * W::H + r, f32_to_bf16_bits(h) | tag16(c, layer));
            } else if (t == kGU) {
                // act = bf16( bf16(silu(bf16 gate)) * bf16 up )   (HF LlamaMLP rounding)
                const float g = round_bf16(mine);
                const float u = round_bf16(mine_up);
                const float silu = round_bf16(__fdividef(g, 1.f + __expf(-g)));
                st_word(p.w_act + par * W::I + r, f32_to_bf16_bits(__fmul_rn(silu, u)) | tag16(c, layer));
            } else if (t == kDown) {
                // x' = bf16( h1 + bf16(down_proj) ), handed to the next layer
                const uint32_t xb = f32_to_bf16_bits(__fadd_rn(res[r], round_bf16(mine)));
                st_word(p.w_x + ((layer + 1) & 1) * W::H + r, xb | tag16(c, layer + 1));
                if (p.layer_outputs) p.layer_outputs[(size_t)layer * W::H + r] = (uint16_t)xb;
            } else {
                const uint32_t lb = f32_to_bf16_bits(mine);
                if (p.logits) p.logits[r] = (uint16_t)lb;
                const uint32_t ord = (lb & 0x8000u) ? (~lb & 0xffffu) : (lb | 0x8000u);
                best = max(best, (ord << 16) | (0xffffu - (uint32_t)(r - ra)));
            }
        }
    }
    if (t == kLM) {
        // greedy argmax: highest logit, ties toward the lowest index; one atomic per CTA
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) best = max(best, __shfl_xor_sync(kFullMask, best, off));
        if (lane == 0) {
            const uint32_t r = (uint32_t)ra + (0xffffu - (best & 0xffffu));
            sh.lm_key[w] = best ? (((unsigned long long)(best >> 16) << 32) | (unsigned long long)(0xffffffffu - r)) : 0ull;
        }
        csync<NW>();
        if (w == 0) {
            unsigned long long k = lane < NW ? sh.lm_key[lane] : 0ull;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) {
                const unsigned long long o = __shfl_xor_sync(kFullMask, k, off);
                k = o > k ? o : k;
            }
            if (lane == 0 && k != 0ull && p.next_ids) atomicMax(p.argkey + (sh.epoch & 1u), k);
        }
    }
}

// ------------------------------------------------------------------ activation staging
// Residual stream in (embedding row, or H words [tag16 | bf16]), fp32 copy to `res`, and
// bf16( bf16(x * rsqrt(mean x^2 + eps)) * w ) to `act`.  HF LlamaRMSNorm rounding.
template <class W, int NW>
__device__ __forceinline__ void stage_norm(FC<NW>& c, const uint32_t* src_words, uint32_t T, const uint16_t* next_weight,
                                           bool from_embed, uint4* act, float* res) {
    constexpr int NT = NW * 32;
    constexpr int NP = W::H / 4;                    // packets of four values
    constexpr int PPT = (NP + NT - 1) / NT;
    const int tid = threadIdx.x;
    FShared<NW>& sh = c.sh;
    static_assert(PPT <= 3, "norm weights are carried in three register pairs per thread");
    // the norm weights were fetched during the previous phase (c.nwv): nothing here waits for DRAM
    uint2 wv[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) wv[u] = c.nwv[u];
    float x[PPT][4];
    if (from_embed) {
#pragma unroll
        for (int u = 0; u < PPT; ++u) {
            const int pk = tid + u * NT;
            const uint2 e = pk < NP ? __ldg(reinterpret_cast<const uint2*>(c.p.embed_bf16 + (size_t)sh.tok * W::H) + pk)
                                    : make_uint2(0u, 0u);
            x[u][0] = bf16_lo(e.x); x[u][1] = bf16_hi(e.x);
            x[u][2] = bf16_lo(e.y); x[u][3] = bf16_hi(e.y);
        }
    } else {
        uint4 pkt[PPT];
        const uint32_t* ptr[PPT];
#pragma unroll
        for (int u = 0; u < PPT; ++u) ptr[u] = (tid + u * NT) < NP ? src_words + 4 * (tid + u * NT) : nullptr;
        poll_packets<PPT>(c, ptr, T, pkt);
#pragma unroll
        for (int u = 0; u < PPT; ++u) {
            x[u][0] = __uint_as_float(pkt[u].x << 16); x[u][1] = __uint_as_float(pkt[u].y << 16);
            x[u][2] = __uint_as_float(pkt[u].z << 16); x[u][3] = __uint_as_float(pkt[u].w << 16);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
        const int pk = tid + u * NT;
        if (pk < NP) {
            *reinterpret_cast<float4*>(res + 4 * pk) = make_float4(x[u][0], x[u][1], x[u][2], x[u][3]);
#pragma unroll
            for (int j = 0; j < 4; ++j) ss = fmaf(x[u][j], x[u][j], ss);
        }
    }
    ss = warp_sum(ss);
    if (c.lane == 0) sh.red[c.warp] = ss;
    csync<NW>();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) tot += sh.red[w];
    const float s = rsqrtf(tot * (1.f / (float)W::H) + c.p.eps);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
        const int pk = tid + u * NT;
        if (pk < NP) {
            const float n0 = round_bf16(__fmul_rn(x[u][0], s)), n1 = round_bf16(__fmul_rn(x[u][1], s));
            const float n2 = round_bf16(__fmul_rn(x[u][2], s)), n3 = round_bf16(__fmul_rn(x[u][3], s));
            uint2 o;
            o.x = pack_bf16x2(__fmul_rn(n0, bf16_lo(wv[u].x)), __fmul_rn(n1, bf16_hi(wv[u].x)));
            o.y = pack_bf16x2(__fmul_rn(n2, bf16_lo(wv[u].y)), __fmul_rn(n3, bf16_hi(wv[u].y)));
            reinterpret_cast<uint2*>(act)[pk] = o;
        }
    }
    // weights of the next norm phase: in flight while the phases in between run
    if (next_weight) {
#pragma unroll
        for (int u = 0; u < PPT; ++u) {
            const int pk = tid + u * NT;
            if (pk < NP) c.nwv[u] = __ldg(reinterpret_cast<const uint2*>(next_weight) + pk);
        }
    }
    csync<NW>();
}

// Copy N words [tag16 | bf16] into `act` (input of the down projection).
template <class W, int N, int NW>
__device__ __forceinline__ void stage_copy(FC<NW>& c, const uint32_t* src_words, uint32_t T, uint4* act) {
    constexpr int NT = NW * 32;
    constexpr int NP = N / 4;
    constexpr int PPT = (NP + NT - 1) / NT;
    const int tid = threadIdx.x;
    uint4 pkt[PPT];
    const uint32_t* ptr[PPT];
#pragma unroll
    for (int u = 0; u < PPT; ++u) ptr[u] = (tid + u * NT) < NP ? src_words + 4 * (tid + u * NT) : nullptr;
    poll_packets<PPT>(c, ptr, T, pkt);
#pragma unroll
    for (int u = 0; u < PPT; ++u) {
        const int pk = tid + u * NT;
        if (pk < NP) {
            uint2 o;
            o.x = (pkt[u].x & 0xffffu) | (pkt[u].y << 16);
            o.y = (pkt[u].z & 0xffffu) | (pkt[u].w << 16);
            reinterpret_cast<uint2*>(act)[pk] = o;
        }
    }
    csync<NW>();
}

// One warp merges the split-KV partials of one query head with log-sum-exp and publishes that head's bf16
// attention output (64 words [tag16 | bf16]).  Only QH warps of the grid poll the partials, so the lines the
// attention items are writing are not read by the whole grid; everybody else waits for the 64-word results,
// which are written once (pulling all partials into every CTA cost 6 MB of L2 traffic per layer and ~1 us).
// Lane = two output dims; lane c also owns the (m, l) statistics of chunk c.
template <class W, int NW>
__device__ __forceinline__ void merge_head(FC<NW>& c, int layer, int hq) {
    constexpr int G = W::G;
    static_assert(W::NC <= 32, "one lane per chunk");
    const int lane = c.lane, nc = c.sh.nc;
    const int kvh = hq / G, g = hq - kvh * G;
    const unsigned long long* part =
        c.p.w_part + ((size_t)(layer & 1) * W::KVH * W::NC + (size_t)kvh * W::NC) * G * 66 + g * 66;
    constexpr size_t cstride = (size_t)G * 66;
    const unsigned long long* ptr[1 + W::NC];
    ptr[0] = lane < nc ? part + lane * cstride : nullptr;                       // words 0, 1: m and l of chunk `lane`
#pragma unroll
    for (int ch = 0; ch < W::NC; ++ch) ptr[1 + ch] = ch < nc ? part + ch * cstride + 2 + 2 * lane : nullptr;
    uint32_t bits[2 * (1 + W::NC)];
    poll_flagged_pairs<1 + W::NC>(c, ptr, tag32(c, layer), bits);
    const float mc = lane < nc ? __uint_as_float(bits[0]) : -INFINITY;
    const float lc = lane < nc ? __uint_as_float(bits[1]) : 0.f;
    const float M = warp_max(mc);                          // chunk 0 always holds at least one position
    const float wc = __expf(mc - M);                       // exp(-inf) = 0 for empty / absent chunks
    const float den = warp_sum(lc * wc);
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int ch = 0; ch < W::NC; ++ch) {
        const float wgt = __shfl_sync(kFullMask, wc, ch);
        if (ch < nc) {
            a0 = fmaf(wgt, __uint_as_float(bits[2 + 2 * ch]), a0);
            a1 = fmaf(wgt, __uint_as_float(bits[3 + 2 * ch]), a1);
        }
    }
    const float inv = 1.f / den;
    const uint32_t T = tag16(c, layer);
    uint32_t* dst = c.p.w_attn + (layer & 1) * W::AD + hq * kD + 2 * lane;
    // two self-validating words in one 8-byte store: a head's 64 words are two stores of 16 lanes' worth each
    const uint32_t w0 = f32_to_bf16_bits(a0 * inv) | T, w1 = f32_to_bf16_bits(a1 * inv) | T;
    asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(w0), "r"(w1) : "memory");
}

// K (this lane's position and half of the head dim) and V (all 16 positions, this lane's two dims) of one
// run of 16 cache positions starting at r0, into registers.  The position seq-1 (the new token) is never
// read from the cache.  ws / we: this warp's share of its CTA's chunk.
template <int NW>
__device__ __forceinline__ void fetch_kv_run(FC<NW>& c, int layer, int r0, int ws, int we, bool pre_ok, uint4 (&kq)[4],
                                             uint32_t (&vw)[16]) {
    const FastParams& p = c.p;
    FShared<NW>& sh = c.sh;
    const int lane = c.lane, pl = lane >> 1, half = lane & 1;
    const int seq = sh.seq;
    const uint16_t* kvr = reinterpret_cast<const uint16_t*>(layer < kKvPtrs ? sh.kv_ptr[layer] : __ldg(p.kv + layer));
    const long long hs = (long long)sh.item_kvh * p.head_stride;
    long long* offs = sh.kv_off[c.warp] + (((r0 - ws) >> 4) & (kPre - 1)) * 16;
    if (!pre_ok) {
        // long context: resolve this run's block-table entries now (lanes 0..15, one position each)
        if (lane < 16) {
            const int pp = r0 + lane;
            long long off = -1;
            if (pp < we) {
                const int blk = __ldg(p.block_table + pp / p.block_size);
                off = (long long)blk * p.block_stride + (long long)(pp % p.block_size) * p.token_stride;
            }
            offs[lane] = off;
        }
        __syncwarp();
    }
    const int pp = r0 + pl;
    const bool own_ok = pp < we && pp != seq - 1;
    const long long e_own = own_ok ? offs[pl] + hs : 0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
        kq[i] = own_ok ? __ldcg(reinterpret_cast<const uint4*>(kvr + p.k_off + e_own + 32 * half) + i)
                       : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int pj = r0 + j;
        const bool ok = pj < we && pj != seq - 1;
        vw[j] = ok ? __ldcg(reinterpret_cast<const uint32_t*>(kvr + p.v_off + offs[j] + hs) + lane) : 0u;
    }
    if (!pre_ok) __syncwarp();
}

// ------------------------------------------------------------------ attention item
// One CTA = one (kv head, chunk) item over cache positions [start, end); its warps split the chunk into
// runs of 16 positions.  Scores: lane = (position, half of the head dim); P.V: lane = two output dims.
// All K and V loads of the first run are issued before the new token's q/k/v words are waited for.
template <class W, int NW>
__device__ __forceinline__ void attention_item(FC<NW>& c, int layer, const int ws, const int we, const bool pre_ok,
                                               uint4 (&kq)[4], uint32_t (&vw)[16]) {
    constexpr int G = W::G;
    constexpr int NT = NW * 32;
    const FastParams& p = c.p;
    FShared<NW>& sh = c.sh;
    const int lane = c.lane, tid = threadIdx.x;
    const int kvh = sh.item_kvh, chunk = sh.item_chunk;
    const int seq = sh.seq;
    const int end = min((chunk + 1) * sh.lc, seq);
    const uint16_t* kvr = reinterpret_cast<const uint16_t*>(layer < kKvPtrs ? sh.kv_ptr[layer] : __ldg(p.kv + layer));
    const long long hs = (long long)kvh * p.head_stride;
    const int pl = lane >> 1, half = lane & 1;

    constexpr int kPartWords = (NW * G * 66 + 3) & ~3;
    uint32_t* qkvb_s = reinterpret_cast<uint32_t*>(c.attn + kPartWords);       // [(G+2)*32] packed bf16: rotated q, k; v
    float* prob_s = reinterpret_cast<float*>(qkvb_s + (G + 2) * 32) + c.warp * G * 16;

    if (c.prof) c.prof[10] = global_ns();
    float m[G], l[G], acc[G][2];
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        m[hh] = -INFINITY;
        l[hh] = 0.f;
        acc[hh][0] = acc[hh][1] = 0.f;
    }
    // One loop over the warp's runs with a single site for the K/V loads; the first iteration (executed by
    // every warp, also one without positions) contains the CTA-wide part: wait for the new token's q/k/v,
    // rotate, append.  The K/V loads of the first run are therefore issued before that wait.
    int r0 = ws;
#pragma unroll 1
    do {
        if (r0 != ws) fetch_kv_run<NW>(c, layer, r0, ws, we, pre_ok, kq, vw);   // the first run was fetched at the top of the layer
        if (r0 == ws) {
            // rotated q of the G heads of this kv head, then rotated k and v of the new token: (G + 2) * 16 packets
            {
                const uint32_t* qkv = p.w_qkv + (layer & 1) * W::NQKV;
                uint4 pkt[1];
                const int which = tid >> 4, d4 = (tid & 15) * 4;
                const int qrow = which < G ? (kvh * G + which) * kD : (which == G ? (W::QH + kvh) * kD : (W::QH + W::KVH + kvh) * kD);
                const uint32_t* ptr[1] = {tid < (G + 2) * 16 ? qkv + qrow + d4 : nullptr};
                poll_packets<1>(c, ptr, tag16(c, layer), pkt);
                if (tid < (G + 2) * 16)
                    *reinterpret_cast<uint2*>(qkvb_s + 2 * tid) =
                        make_uint2((pkt[0].x & 0xffffu) | (pkt[0].y << 16), (pkt[0].z & 0xffffu) | (pkt[0].w << 16));
            }
            csync<NW>();
            if (c.prof) c.prof[11] = global_ns();
            // the item that holds position seq-1 appends the new token's K/V to the paged cache (slot -1: skip)
            if (end == seq && c.warp == 0 && lane < 16 && sh.slot_off >= 0) {
                uint16_t* kvw = const_cast<uint16_t*>(kvr);
                const int l8 = lane & 7;
                const long long e = sh.slot_off + hs + 8 * l8;
                if (lane < 8) *reinterpret_cast<uint4*>(kvw + p.k_off + e) = *reinterpret_cast<const uint4*>(qkvb_s + G * 32 + 4 * l8);
                else *reinterpret_cast<uint4*>(kvw + p.v_off + e) = *reinterpret_cast<const uint4*>(qkvb_s + (G + 1) * 32 + 4 * l8);
            }
        }
        if (r0 < we) {
            if (c.prof && r0 == ws) c.prof[16] = global_ns();
            const int pp = r0 + pl;
            const bool valid = pp < we;
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
            // The G heads are processed side by side in every step (shuffles keep their program order, so
            // a head-by-head loop would run the three dependent chains one after the other).
            float sc[G], mx[G], pr[G];
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
                sc[hh] = d0 + d1;
            }
            if (c.prof && r0 == ws) c.prof[17] = global_ns();
#pragma unroll
            for (int hh = 0; hh < G; ++hh) sc[hh] += __shfl_xor_sync(kFullMask, sc[hh], 1);
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                // bf16 matmul output, then the exact 1/8 scale (HF eager_attention_forward)
                sc[hh] = valid ? round_bf16(sc[hh]) * 0.125f : -INFINITY;
                mx[hh] = sc[hh];
            }
            // warp maximum with one redux per head: floats compare like these integer keys
#pragma unroll
            for (int hh = 0; hh < G; ++hh) {
                int key = __float_as_int(mx[hh]);
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
                // per-lane share of the denominator (one lane of every position pair); summed over the warp after
                // the last run -- the rescale factor is warp-uniform, so the order does not matter
                l[hh] = l[hh] * alpha + (half == 0 ? pr[hh] : 0.f);
                acc[hh][0] *= alpha;
                acc[hh][1] *= alpha;
                if (half == 0) prob_s[hh * 16 + pl] = pr[hh];
            }
            __syncwarp();
            if (c.prof && r0 == ws) c.prof[18] = global_ns();
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
        r0 += 16;
    } while (r0 < we);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1)
#pragma unroll
        for (int hh = 0; hh < G; ++hh) l[hh] += __shfl_xor_sync(kFullMask, l[hh], off);
    if (c.prof) c.prof[12] = global_ns();
    // park the warp's partial: lanes hold two dims each
    float* wpart = c.attn + c.warp * G * 66;
#pragma unroll
    for (int hh = 0; hh < G; ++hh) {
        float* dst = wpart + hh * 66;
        if (lane == 0) {
            dst[0] = m[hh];
            dst[1] = l[hh];
        }
        *reinterpret_cast<float2*>(dst + 2 + 2 * lane) = make_float2(acc[hh][0], acc[hh][1]);
    }
    csync<NW>();
    if (c.prof) c.prof[13] = global_ns();
    // combine the warps; thread (hh, d) publishes one accumulator word, d == 0 also m and l
    unsigned long long* part =
        p.w_part + ((size_t)(layer & 1) * W::KVH * W::NC + (size_t)(kvh * W::NC + chunk)) * G * 66;
    const uint32_t tag = tag32(c, layer);
    for (int t = tid; t < G * kD; t += NT) {
        const int hh = t / kD, d = t % kD;
        float M = -INFINITY;
#pragma unroll 8
        for (int w = 0; w < NW; ++w) M = fmaxf(M, c.attn[(w * G + hh) * 66]);
        float lt = 0.f, a = 0.f;
#pragma unroll 8
        for (int w = 0; w < NW; ++w) {
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
    csync<NW>();     // c.attn is reused by the merge staging
    if (c.prof) c.prof[14] = global_ns();
}

// ------------------------------------------------------------------ the kernel
template <class W, int NW, int WF>
__global__ void __launch_bounds__((NW + 1) * 32, 1) decode_fast_kernel(const FastParams p) {
    constexpr int NT = (NW + 1) * 32;      // NW consumer warps + the producer warp
    constexpr int NTC = NW * 32;           // consumer threads
    constexpr int G = W::G;
    constexpr int ACT = W::H > W::I ? W::H : W::I;
    constexpr int kAttnWords = attn_words<W, NW>();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    FShared<NW>& sh = *reinterpret_cast<FShared<NW>*>(smem_raw);
    size_t off = (sizeof(FShared<NW>) + 127) & ~size_t(127);
    uint4* act0 = reinterpret_cast<uint4*>(smem_raw + off);      // norm outputs (H); act1: attention output / SwiGLU product
    off += ((size_t)W::H * 2 + 127) & ~size_t(127);
    uint4* act1 = reinterpret_cast<uint4*>(smem_raw + off);
    off += ((size_t)ACT * 2 + 127) & ~size_t(127);
    float* res0 = reinterpret_cast<float*>(smem_raw + off);
    off += ((size_t)W::H * 4 + 127) & ~size_t(127);
    float* res1 = reinterpret_cast<float*>(smem_raw + off);
    off += ((size_t)W::H * 4 + 127) & ~size_t(127);
    float* attn = reinterpret_cast<float*>(smem_raw + off);
    off += ((size_t)kAttnWords * 4 + 127) & ~size_t(127);
    unsigned char* ring_base = smem_raw + off;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x, ncta = gridDim.x;

    if (tid == 0) {
        sh.abort_flag = (p.ctrl[kCtrlStatus] != 0u) ? 1 : 0;     // an earlier failure on this workspace: fall through
        sh.epoch = p.fctrl[kFctrlEpoch];
        const int seq = min(max(p.seq_lens[0], 1), p.max_seq_len);
        if (p.seq_lens[0] > p.max_seq_len) {
            sh.abort_flag = 1;
            atomicCAS(p.ctrl + kCtrlStatus, 0u, (unsigned)kErrMaxSeq);
        }
        sh.seq = seq;
        sh.pos = (int)max(p.positions[0], 0LL);
        const long long tok = p.ids_i64 ? reinterpret_cast<const long long*>(p.input_ids)[0]
                                        : (long long)reinterpret_cast<const int*>(p.input_ids)[0];
        sh.tok = tok < 0 ? 0 : (tok >= p.V ? p.V - 1 : tok);      // an out-of-range id must not become a wild read
        const long long slot = p.slot_mapping[0];
        sh.slot_off = slot < 0 ? -1 : (slot / p.block_size) * p.block_stride + (slot % p.block_size) * p.token_stride;
        // split-KV: one run of 16 positions per warp while that needs at most W::NC chunks, longer chunks beyond
        int nc = (seq + NW * 16 - 1) / (NW * 16);
        nc = nc < 1 ? 1 : (nc > W::NC ? W::NC : nc);
        const int lc = (((seq + nc - 1) / nc) + 15) & ~15;
        sh.lc = lc;
        sh.nc = (seq + lc - 1) / lc;
        const bool has = cta < sh.nc * W::KVH;
        sh.item_kvh = has ? cta % W::KVH : -1;
        sh.item_chunk = has ? cta / W::KVH : 0;
    }
    if (tid < NW * kFE) {
        mbar_init(&sh.full[tid / kFE][tid % kFE], 1);
        mbar_init(&sh.empty[tid / kFE][tid % kFE], 1);
        sh.ent_off[tid / kFE][tid % kFE] = 0u;
        sh.ent_foot[tid / kFE][tid % kFE] = 0u;
    }
    for (int l = tid; l < p.L && l < kKvPtrs; l += NT) sh.kv_ptr[l] = p.kv[l];
    for (int i = tid; i < 4 * p.L; i += NT) {
        const int l = i >> 2, m = i & 3;
        sh.mat_ptr[l][m] = p.layers[l * 6 + (m == 0 ? 1 : (m == 1 ? 2 : (m == 2 ? 4 : 5)))];
    }
    for (int i = tid; i <= 2 * p.L; i += NT)
        sh.norm_ptr[i] = i == 2 * p.L ? reinterpret_cast<unsigned long long>(p.final_norm) : p.layers[(i >> 1) * 6 + ((i & 1) ? 3 : 0)];
    if (tid < kNumPhaseTypes * NW) {
        const int t = tid / NW, w = tid % NW;
        // units: QKV row pairs (d, d + 32), gate/up row pairs, single rows elsewhere
        const int nrows = t == kQKV ? W::NQKV / 2 : (t == kGU ? W::I : (t == kLM ? (p.lm_head ? p.V : 0) : W::H));
        int a = 0, b = 0;
        warp_share<NW>(nrows, cta, ncta, w, a, b);
        sh.row_a[t][w] = a;
        sh.row_b[t][w] = b;
    }
    if (tid >= 64 && tid < 128) {
        const int j = tid - 64;
        const long long pos = max(p.positions[0], 0LL);
        sh.cs[j] = p.cs_fp32 ? __ldg(reinterpret_cast<const float*>(p.cos_sin) + pos * kD + j)
                             : __uint_as_float((uint32_t)__ldg(reinterpret_cast<const uint16_t*>(p.cos_sin) + pos * kD + j) << 16);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    __syncthreads();

    FC<NW> c{p, sh, {act0, act1}, {res0, res1}, attn, ring_base + (size_t)warp * p.ring_bytes, 0u, 0u, warp, lane, cta, ncta,
             0u, {make_uint2(0u, 0u), make_uint2(0u, 0u), make_uint2(0u, 0u)}, 0u, false, nullptr};
    c.T16 = ((sh.epoch % 511u) + 1u) << 23;
    c.T32 = (sh.epoch + 1u) << 7;
    if (warp == NW) {
        producer_loop<W, NW, WF>(p, sh, ring_base, lane);
    } else {

    // block-table look-ups of this CTA's attention item do not depend on the layer: resolve them once
    {
        int ws = 0, we = 0;
        if (sh.item_kvh >= 0) {
            const int start = sh.item_chunk * sh.lc;
            const int end = min(start + sh.lc, sh.seq);
            const int ppw = (((end - start + NW - 1) / NW) + 15) & ~15;
            ws = min(start + warp * ppw, end);
            we = min(ws + ppw, end);
        }
        for (int j = lane; j < kPre * 16; j += 32) {
            long long o = -1;
            const int pp = ws + j;
            if (pp < we) {
                const int blk = p.block_table[pp / p.block_size];
                o = (long long)blk * p.block_stride + (long long)(pp % p.block_size) * p.token_stride;
            }
            sh.kv_off[warp][j] = o;
        }
    }
    // this warp's share of the CTA's attention item (layer-invariant) and the registers its first run lives in
    int item_ws = 0, item_we = 0;
    bool item_pre_ok = true;
    if (sh.item_kvh >= 0) {
        const int start = sh.item_chunk * sh.lc;
        const int end = min(start + sh.lc, sh.seq);
        const int ppw = (((end - start + NW - 1) / NW) + 15) & ~15;
        item_ws = min(start + warp * ppw, end);
        item_we = min(item_ws + ppw, end);
        item_pre_ok = ppw <= kPre * 16;      // every run's offsets were resolved above
    }
    uint4 kq[4];
    uint32_t vw[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) kq[i] = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int j = 0; j < 16; ++j) vw[j] = 0u;
    // reset the argmax cell the *next* launch will use
    if (cta == 0 && tid == 0) p.argkey[(sh.epoch + 1u) & 1u] = 0ull;
    // norm weights of the first norm phase (every later phase fetches the next one's ahead of time)
    {
        constexpr int NP = W::H / 4;
        const uint2* nw0 = reinterpret_cast<const uint2*>(sh.norm_ptr[0]);
#pragma unroll
        for (int u = 0; u < 3; ++u)
            if (tid + u * NTC < NP) c.nwv[u] = __ldg(nw0 + tid + u * NTC);
    }
    csync<NW>();

    // One loop over the global phase index (4 per layer, then the final norm + lm_head) with a single call
    // site for every building block, so each exists once in the instruction stream.
    const int nph = p.L * 4 + 1;
#pragma unroll 1
    for (int gp = 0; gp < nph; ++gp) {
        const int layer = gp >> 2;
        const bool last = gp == nph - 1;
        const int t = last ? (int)kLM : (gp & 3);
        if (last && !(p.lm_head || cta == 0)) break;
        const int par = layer & 1;
        unsigned long long* prof = nullptr;
        if (p.profile && tid == 0 && !last) prof = p.profile + ((size_t)cta * p.L + layer) * kProfSlots;
        c.prof = prof;
        uint4* act = (t == kO || t == kDown) ? act1 : act0;
        const float* res = (t == kGU || t == kDown) ? res1 : res0;
        // The weights of this phase normally landed long ago: confirm it now, before the activations are waited
        // for, so that the first dot product can start right behind the staging barrier.
        c.pre_ok = false;
        if (sh.row_a[t][warp] < sh.row_b[t][warp] && !(last && !p.lm_head)) {
            const uint32_t slot = c.consumed % kFE;
            c.pre_ok = __all_sync(kFullMask, f_wait_mbar(c, &sh.full[warp][slot], (c.consumed / kFE) & 1));
            c.pre_off = sh.ent_off[warp][slot];
        }
        if (t == kQKV || t == kGU || last) {
            if (t == kQKV) {
                if (prof) prof[0] = global_ns();
                // K/V of the first run of this warp's share go into registers now: they have the whole norm + QKV
                // phase to arrive, and no burst of loads sits in front of the q poll of the attention item
                // (20 loads per thread issued right before that poll delayed its answer by ~0.7 us)
                if (sh.item_kvh >= 0 && item_ws < item_we) fetch_kv_run<NW>(c, layer, item_ws, item_ws, item_we, item_pre_ok, kq, vw);
            }
            // RMSNorm: input norm (x -> res0), post-attention norm (h1 -> res1) or the final norm
            const uint32_t* src = (t == kGU ? p.w_h1 : p.w_x) + par * W::H;
            const int ni = 2 * layer + (t == kGU ? 1 : 0);          // index of this norm; the next one is fetched now
            const uint16_t* next_w = ni < 2 * p.L ? reinterpret_cast<const uint16_t*>(sh.norm_ptr[ni + 1]) : nullptr;
            stage_norm<W, NW>(c, src, tag16(c, layer), next_w, gp == 0, act0, t == kGU ? res1 : res0);
        } else if (t == kO) {
            if (sh.item_kvh >= 0) attention_item<W, NW>(c, layer, item_ws, item_we, item_pre_ok, kq, vw);
            if (prof) prof[3] = global_ns();
            // the last QH CTAs (never attention items) merge one query head each; everybody stages the result
            if (cta >= ncta - W::QH && warp == 0) merge_head<W, NW>(c, layer, ncta - 1 - cta);
            stage_copy<W, W::AD, NW>(c, p.w_attn + par * W::AD, tag16(c, layer), act1);
        } else {
            stage_copy<W, W::I, NW>(c, p.w_act + par * W::I, tag16(c, layer), act1);
        }
        if (prof) prof[1 + 2 * t + (t >= kO ? 1 : 0)] = global_ns();     // slots 1, 4, 6, 8
        if (last) {
            if (cta == 0)
                for (int i = tid; i < W::H / 2; i += NTC)
                    reinterpret_cast<uint32_t*>(p.out_hidden)[i] = reinterpret_cast<const uint32_t*>(act0)[i];
            if (!p.lm_head) break;
        }
        gemv_phase<W, NW, WF>(c, t, layer, act, res);
        // Nobody in this CTA polls the next hand-off before the CTA's own results are on their way: reads of a
        // line that is still being written slow the writes down (measured: several microseconds per hand-off
        // when the warps without rows in a phase started polling at once).
        csync<NW>();
        if (prof) prof[2 + 2 * t + (t >= kO ? 1 : 0)] = global_ns();     // slots 2, 5, 7, 9
    }

    }   // consumer warps
    __syncthreads();
    // The last CTA to finish publishes the greedy id, optionally advances the step inputs in place
    // (device-driven generation), and opens the next launch's epoch.
    if (tid == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(p.fctrl + kFctrlDone, 1u);
        if (prev == (unsigned)ncta - 1u) {
            __threadfence();
            const bool ok = *((volatile unsigned int*)(p.ctrl + kCtrlStatus)) == 0;
            if (p.next_ids && p.lm_head && ok) {
                const unsigned long long key = *((volatile unsigned long long*)(p.argkey + (sh.epoch & 1u)));
                const long long id = (long long)(0xffffffffu - (uint32_t)key);
                p.next_ids[0] = id;
                if (p.advance) {
                    if (p.ids_i64) reinterpret_cast<long long*>(const_cast<void*>(p.input_ids))[0] = id;
                    else reinterpret_cast<int*>(const_cast<void*>(p.input_ids))[0] = (int)id;
                    const long long np = p.positions[0] + 1;
                    const_cast<long long*>(p.positions)[0] = np;
                    const_cast<int*>(p.seq_lens)[0] = p.seq_lens[0] + 1;
                    if (p.slot_mapping[0] >= 0 && np < (long long)p.max_seq_len) {
                        const long long blk = p.block_table[(int)(np / p.block_size)];
                        const_cast<long long*>(p.slot_mapping)[0] = blk * p.block_size + np % p.block_size;
                    }
                }
            }
            p.fctrl[kFctrlDone] = 0u;
            p.fctrl[kFctrlEpoch] = sh.epoch + 1u;
            __threadfence();
        }
    }
}

}  // namespace fast
}  // namespace pk
