/*
 * C ABI of libprime_kernels_b200.so -- the drop-in boundary of the B200-native decode hot path.
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer unless stated otherwise,
 * `stream` is a cudaStream_t passed as void*.  Every function that can fail returns an int:
 * 0 = ok, 9101..9112 = contract violations (see pk_status_string), any other value is a
 * cudaError_t.  Nothing here allocates device memory; nothing here falls back to the CPU.
 *
 * Each entry cites the reference interface it replaces (paths inside the reference project).
 */
#ifndef PRIME_KERNELS_B200_H
#define PRIME_KERNELS_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- fused RMSNorm + residual + MXFP8 */

/* Replaces fused_rmsnorm_residual_forward (prime_kernels/rmsnorm/rmsnorm.cuh:15-18,85):
 * vals e4m3 [N,C]; scales e8m0, blocked 128x4 layout, pk_rmsnorm_scale_bytes(N,C) bytes;
 * rrms fp32 [N]; branch/residual bf16 [N,C]; weight bf16 [C].
 * out = rmsnorm(branch) * weight + residual, quantised per 32 elements.
 * Differences: returns a status instead of assert/exit; N may be any size >= 0 and C any positive
 * multiple of 32 (bytes of partially covered scale tiles are written as 0). */
int pk_fused_rmsnorm_residual_forward(void* vals, void* scales, float* rrms, const void* branch,
                                      const void* residual, const void* weight, float epsilon, int N, int C,
                                      void* stream);

/* Extension of the above.  mode 0: as above; mode 1: residual added before the norm (forward
 * semantics of triton_residual_rmsnorm, prime_kernels/triton_rmsnorm/rmsnorm.py:711-722) followed by
 * the same quantiser.  res_out (nullable, bf16 [N,C]) receives the updated residual stream
 * (mode 0: the bf16 value that was quantised; mode 1: bf16(branch + residual)). */
int pk_fused_rmsnorm_residual_forward_ex(void* vals, void* scales, float* rrms, void* res_out, const void* branch,
                                         const void* residual, const void* weight, float epsilon, int N, int C,
                                         int mode, void* stream);

/* Which kernel pk_fused_rmsnorm_residual_forward would launch for these pointers and this shape, without launching:
 * 2 = pipelined bulk-copy kernel (needs 16-byte aligned vals / branch / residual), 1 = lane-owns-group kernel
 * (32-byte aligned pointers), 0 = register kernel; a negative value is minus the status the entry would return.
 * Replaces the shape-only dispatch rule of prime_kernels/rmsnorm/rmsnorm.cu:15-31.  Host only. */
int pk_rmsnorm_dispatch(const void* vals, const void* branch, const void* residual, const void* weight, int N, int C);
/* Size in bytes of the blocked scale buffer: ceil(N/128) * ceil(C/128) * 512
 * (scale_numel in prime_kernels/rmsnorm/csrc/torch_interface.cpp:18-20, extended to ragged shapes). */
long long pk_rmsnorm_scale_bytes(int N, int C);
/* Bounded barrier waits of the pipelined kernel that expired since load (0 = healthy; -1 = CUDA error).
 * No counterpart in the reference (its TMA kernels wait without a bound, rmsnorm_05_tma.cu). Synchronises. */
long long pk_rmsnorm_wait_timeouts(void);

/* ---------------------------------------------------------------- forward ops the megakernel absorbs, standalone */

/* Forward of triton_rope.apply_rotary (prime_kernels/triton_rope/__init__.py:41-82,373-377) for one tensor:
 * x, y bf16 [batch*heads*seq, D] contiguous, head-major ([B, heads, S, D]; unsqueeze_dim 1) or sequence-major
 * ([B, S, heads, D]; unsqueeze_dim 2); cos, sin bf16 [cos_batch (1 or B), S, rot]; the first `rot` dims rotate. */
int pk_apply_rotary(const void* x, void* y, const void* cos, const void* sin, long long batch, int heads, int seq,
                    int D, int rot, int head_major, int cos_batch, void* stream);
/* Forward of triton_rmsnorm.rmsnorm / residual_rmsnorm (prime_kernels/triton_rmsnorm/rmsnorm.py:701-722):
 * out = bf16(w * bf16(v * rstd)), v = x or bf16(x + residual); residual and sum_out may be NULL. */
int pk_rmsnorm_forward(const void* x, const void* residual, const void* weight, void* out, void* sum_out,
                       long long rows, int H, float eps, void* stream);
/* Forward of triton_swiglu.swiglu (prime_kernels/triton_swiglu/swiglu.py:31-59,195-202):
 * out = bf16(bf16(silu(gate)) * up); gate/up row strides in elements. */
int pk_swiglu_forward(const void* gate, const void* up, void* out, long long rows, int cols, long long gate_stride,
                      long long up_stride, void* stream);
/* Backward passes of the three ops above (bf16; same rounding points as the reference's Triton backward kernels:
 * prime_kernels/triton_rope/__init__.py:85-123, triton_swiglu/swiglu.py:62-97, triton_rmsnorm/rmsnorm.py:107-193
 * and :300-392).  pk_rmsnorm_backward: `x` is the normed input (the returned sum for the residual variant), `grad_sum`
 * the gradient arriving through that sum (NULL for plain rmsnorm), `dx` the gradient of x (of branch and of residual),
 * `dw` bf16 [H], `dw_partials` fp32 scratch [pk_rmsnorm_backward_parts(rows)][H]; H % 8 == 0, H <= 8192; the weight
 * gradient is summed in a fixed order (deterministic). */
int pk_apply_rotary_backward(const void* g, void* gx, const void* cos, const void* sin, long long batch, int heads, int seq,
                             int D, int rot, int head_major, int cos_batch, void* stream);
int pk_swiglu_backward(const void* grad, const void* gate, const void* up, void* d_gate, void* d_up, long long rows, int cols,
                       long long gate_stride, long long up_stride, void* stream);
int pk_rmsnorm_backward_parts(long long rows);
int pk_rmsnorm_backward(const void* grad_out, const void* grad_sum, const void* x, const void* weight, void* dx, void* dw,
                        void* dw_partials, long long rows, int H, float eps, void* stream);

/* MXFP8 weight packing for the decode GEMVs.  No counterpart in the reference (its kernels take
 * pre-quantised weights, prime_kernels/flash_moe/__init__.py:165-170).  Quantises bf16 [rows, K] along K
 * with the quantiser above (one E8M0 scale per 32 values, round-up scale) into packed rows
 * [K e4m3][K/32 e8m0][zero pad to 16 B]; pk_mxfp8_packed_row_bytes(K) is the row stride (-1: bad K). */
long long pk_mxfp8_packed_row_bytes(int K);
int pk_pack_weights_mxfp8(const void* weights_bf16, void* packed, long long rows, int K, void* stream);
/* Same with the scale rule chosen: 0 = round-up (above), 1 = floor: e = clamp(biased_exponent(amax) - 8, 0, 254), values
 * converted from fp32 with finite saturation - the block-scale rule of the reference's flash_moe kernels
 * (prime_kernels/flash_moe/csrc/kernels/fused_moe_mxfp8_kernel.cu:4-20).  The packed format is the same. */
int pk_pack_weights_mxfp8_ex(const void* weights_bf16, void* packed, long long rows, int K, int scale_mode, void* stream);

/* ---------------------------------------------------------------- decode megakernel, generic geometry */

typedef struct PkDecodeModel {
    int hidden, intermediate, layers, q_heads, kv_heads, vocab; /* head_dim is 64 */
    int weight_format; /* 0 = bf16 row-major; 1 = MXFP8 packed rows: [K e4m3][K/32 e8m0][pad to 16 B] */
    float eps;
} PkDecodeModel;

/* Argument block of one decode step.  Field meaning follows the reference's Params
 * (prime_kernels/decode_megakernel/csrc/megakernel.cu:125-154) and mk_decode (:844-851):
 * layers = device table int64 [L][6] (norm1, qkv, o, norm2, gate_up, down); kv_layers = device table
 * int64 [L]; KV strides in elements of a [blocks, kv_heads, block_size, 128] bf16 cache; seq_lens
 * include the token being decoded; slot_mapping -1 skips the cache write.
 * Extensions: logits (nullable, bf16 [B, vocab]) and next_ids (nullable, int64 [B]) enable the fused
 * tied lm_head + argmax when lm_head != 0; advance != 0 additionally rewrites input_ids, positions,
 * seq_lens and slot_mapping in place for the next step (device-driven greedy generation);
 * embed_lookup (nullable) is the bf16 embedding used for the input lookup when `embed` is MXFP8. */
typedef struct PkDecodeArgs {
    void* stream;
    int batch;
    const void* input_ids; int ids_i64;
    const void* positions; const void* seq_lens; const void* block_table; int bt_stride; const void* slot_mapping;
    const void* layers; const void* embed; const void* embed_lookup; const void* final_norm; const void* kv_layers;
    long long k_off, v_off, block_stride, token_stride, head_stride; int block_size;
    const void* cos_sin; int cs_fp32;
    void* out_hidden; void* logits; void* next_ids; void* layer_outputs;
    void* workspace; size_t workspace_bytes; int max_seq_len; int lm_head; int advance;
} PkDecodeArgs;

/* Generic form of mk_workspace_bytes / decode360_workspace_bytes; max_batch 1..64.  One workspace serves every kernel and
 * every batch up to max_batch: from the tensor-core cross-over on (4 requests; 2 for hidden >= 2048) it also holds the
 * tensor-core kernel's region (same size whatever the batch), behind the CUDA-core kernels' region. */
size_t pk_decode_workspace_bytes(const PkDecodeModel* model, int max_batch);
/* Generic form of mk_decode / decode360 (one cooperative launch on args->stream), 1..64 requests.  Small batches run on
 * the CUDA-core kernels (batch 1 of the SmolLM2-135M / 360M / 1.7B widths, bf16 or MXFP8 weights, on a kernel specialised for
 * them); from the cross-over on (pk_decode_set_tc_min_batch) and always above 8 requests the step runs on the
 * tensor-core kernel: projections as tcgen05 GEMMs with the weight tile as the 128-row operand, batch padded to
 * 16 / 32 / 64, accumulators in tensor memory, every weight streamed once per step. */
int pk_decode_step(const PkDecodeModel* model, const PkDecodeArgs* args);
/* Same step on the tensor-core kernel whatever the batch (1..64); pk_decode_step picks it by itself from
 * pk_decode_set_tc_min_batch requests on (default: the measured cross-over, 4 requests, 2 for hidden >= 2048) when the
 * workspace has pk_decode_workspace_bytes(model, n >= 4) bytes, and always above 8.  No counterpart in the reference
 * (its decode kernels have no tensor-core path beyond wmma at batch 2,
 * prime_kernels/decode_megakernel_360m/csrc/block360.cu:312-364).  One workspace serves all kernels. */
int pk_decode_step_tc(const PkDecodeModel* model, const PkDecodeArgs* args);
/* Same step on the CUDA-core kernels only (1..8 requests). */
int pk_decode_step_cc(const PkDecodeModel* model, const PkDecodeArgs* args);
/* Smallest batch pk_decode_step and mk_decode hand to the tensor-core kernel (1..9; 9 = only above 8 requests;
 * 0 = the default, the measured cross-over: 2 requests for hidden >= 2048, else 4). */
void pk_decode_set_tc_min_batch(int n);
/* Zero a workspace in stream order (also done implicitly the first time a pointer is seen). */
int pk_decode_workspace_init(void* workspace, size_t bytes, void* stream);
void pk_decode_workspace_forget(void* workspace);
/* Synchronise `stream` and return the device-side status word (9110 = a bounded wait gave up). */
int pk_decode_status(void* workspace, void* stream);
/* Decode step for callers that cannot allocate device memory.  No counterpart in the reference (its
 * Python surface always allocates the scratch with torch).  Inference servers usually give all memory
 * left after start-up to their KV-cache pool, and some embedders run where the CUDA allocator must not
 * be called; for them the library holds a scratch area of its own, a 2 MiB device array that every GPU
 * loading the library keeps until the process exits.  Same arguments as pk_decode_step except that
 * args->workspace / workspace_bytes are ignored.  Status 9112 when the step needs more than
 * pk_decode_static_scratch_bytes() (fits: SmolLM2-360M at batch 1, SmolLM2-135M up to batch 2).
 * The first call on a device resolves the array's device address: make it before any stream capture.
 * All calls on a device share the array (it keeps the previous call's contents; status and completion
 * words are cleared per call), so calls that overlap on the GPU race -- serialise them.
 * Nothing on this path calls cudaMalloc, cudaFree or an allocating library routine. */
int pk_decode_step_static(const PkDecodeModel* model, const PkDecodeArgs* args);
size_t pk_decode_static_scratch_bytes(void);
/* Synchronise `stream` and return the status word of the built-in scratch of the current device. */
int pk_decode_static_status(void* stream);
/* Generic form of mk_query (prime_kernels/decode_megakernel/csrc/megakernel.cu:833-836). */
int pk_decode_query(int* sm_count, int* coop, int* major, int* minor, int* smem_optin, int* threads,
                    int* consumer_warps);
/* Debug aid modelled on the reference's private stage profiler
 * (research/smollm2_360m_decode/experiments/r28-fast-stage-profile-r1/README.md:7-9): when a device
 * buffer of at least ctas * layers * 24 * 8 bytes is set, thread 0 of every CTA stamps %globaltimer at
 * each phase boundary of each layer ([cta][layer][24] uint64 ns).  Pass NULL to disable. */
void pk_decode_set_profile(void* buffer, size_t bytes);
/* Replaces mk_status_string / decode360_status_string for every code above. */
const char* pk_status_string(int status);
/* Tuning and test knobs, process-wide; no counterpart in the reference.
 * pk_decode_set_fast_path: batch-1 steps of the SmolLM2-135M / 360M / 1.7B widths run on a kernel specialised
 * for those widths with `warps` (7 or 8) consumer warps per CTA; 0 sends every step to the generic kernel
 * (default: environment variable PK_DECODE_FAST, else 7).  Both kernels keep the same rounding points.
 * pk_decode_set_spin_limit: bound, in polling rounds, of every device-side wait of later launches (the
 * reference spins without a bound, prime_kernels/decode_megakernel/csrc/megakernel.cu:109-122); 0 = default.
 * pk_decode_wait_probe: failure-path check in the form of the reference's harness watchdog
 * (prime_kernels/rmsnorm/test.cu:180-192) moved onto the device: one CTA polls a word of `workspace` that
 * nothing writes, gives up after `rounds` polls and records status 9110, which pk_decode_status() then
 * returns and clears.  It cannot hang and writes nothing else. */
int pk_decode_set_fast_path(int warps);
void pk_decode_set_spin_limit(unsigned rounds);
int pk_decode_wait_probe(void* workspace, size_t bytes, unsigned rounds, void* stream);

/* ---------------------------------------------------------------- drop-in signatures of the reference */

/* SmolLM2-135M: prime_kernels/decode_megakernel/csrc/megakernel.cu:833-927 (same arguments, same
 * status numbers; 9106 now means "requires sm_100"; 9110/9111 are new). */
int mk_query(int* sm_count, int* coop, int* active_per_sm, int* major, int* minor, int* regs, int* static_smem);
size_t mk_workspace_bytes(int B, int max_seq_len);
int mk_decode(void* stream, int B, const void* input_ids, int ids_i64, const void* positions, const void* seq_lens,
              const void* block_table, int bt_stride, const void* slot_mapping, const void* layers, const void* embed,
              const void* final_norm, void* const* kv_layers, long long k_off, long long v_off, long long block_stride,
              long long token_stride, long long head_stride, int block_size, const void* cos_sin, int cs_fp32,
              void* out_hidden, void* scratch, size_t scratch_bytes, int max_seq_len);
const char* mk_status_string(int status);

/* SmolLM2-360M: prime_kernels/decode_megakernel_360m/csrc/block360_kernel.inc:849-938.  The debug
 * stage dump is accepted and ignored (nothing is written to it). */
size_t decode360_workspace_bytes(void);
size_t decode360_debug_bytes(void);
int decode360(void* stream, int B, const void* input_ids, const void* embed, const void* final_norm,
              const void* positions, const void* seq_lens, const void* block_table, int bt_stride,
              const void* slot_mapping, const void* layers, void* const* kv, long long k_off, long long v_off,
              long long block_stride, long long token_stride, long long head_stride, int block_size,
              const void* cos_sin, int cs_fp32, void* out_hidden, void* layer_outputs, void* scratch,
              size_t scratch_bytes, void* debug, size_t debug_bytes, int max_seq_len, int debug_layer_index);
const char* decode360_status_string(int status);

#ifdef __cplusplus
}
#endif
#endif /* PRIME_KERNELS_B200_H */
