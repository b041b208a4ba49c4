/*
 * rl_b200.h -- C ABI of the B200 (sm_100a) hybrid-attention operators.
 *
 * Drop-in surface for the attention / DeltaNet hot path of RapidLLM's qwen3_5
 * engine.  Each entry point names the reference interface it replaces
 * (paths relative to the RapidLLM tree).  Conventions follow the reference's C
 * API (include/rapidllm/api.h:11-25, src/api/rapidllm_c.cpp:46-50): nothing
 * throws across this boundary, every call returns an rl_status, and
 * rl_last_error() gives the message of the last failure on the calling thread.
 *
 * Unless a name ends in _host, every pointer is a DEVICE pointer owned by the
 * caller and `stream` is a cudaStream_t passed as void* (NULL = default
 * stream).  Work is enqueued asynchronously; bad device-side data (a page id
 * outside the pool, a slot outside the cache, a length beyond the page table)
 * never faults: the kernel skips the access and records a code that
 * rl_device_error() returns.
 */
#ifndef RL_B200_H
#define RL_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#define RL_B200_ABI_VERSION 2

/* Same values as RapidStatus, include/rapidllm/api.h:11-20. */
typedef enum rl_status {
    RL_OK = 0,
    RL_ERR_IO,
    RL_ERR_FORMAT,
    RL_ERR_NOMEM,
    RL_ERR_UNSUPPORTED,
    RL_ERR_DEVICE,
    RL_ERR_RANGE,
    RL_ERR_INTERNAL
} rl_status;

/* KV cache element formats (the reference's --kv-type f16 | q8k_tq3v,
 * src/cli/main.cpp:137-155). */
enum { RL_KV_F16 = 0, RL_KV_Q8K_TQ3V = 1 };
/* layer_types[] entries (LayerKind, include/rapidllm/ir/model_desc.h). */
enum { RL_LAYER_LINEAR_ATTENTION = 0, RL_LAYER_FULL_ATTENTION = 1 };
/* How DeltaNet value head h finds its key/query head
 * (src/kernels/ops_fused.cpp:117-119, cuda_engine.cu:78-89). */
enum { RL_HEADS_PER_VALUE = 0, RL_HEADS_GROUPED = 1, RL_HEADS_TILED = 2 };

/* cuda_gen::available(), include/rapidllm/runtime/cuda_engine.h:11:
 * 1 when a CUDA device of compute capability 10.x is present, else 0. */
int rl_b200_available(void);
int rl_b200_abi_version(void);
/* Message of the last failing call on this thread (RapidError.message). */
const char* rl_last_error(void);
/* Synchronises `stream`, returns the device error word (0 = none; see
 * rl_device_error_string) and clears it. */
int rl_device_error(void* stream);
const char* rl_device_error_string(int code);

/* ------------------------------------------------------------------------- */
/* Gated attention, decode                                                    */
/* ------------------------------------------------------------------------- */

/* AttnDecodeParams {n_q, n_kv, head_dim, seq, pos, kv_dtype, rms_eps}
 * (include/rapidllm/backend/params.h:17) extended to a ragged batch on a paged
 * cache: `seq`/`pos` become the device arrays passed to the call. */
typedef struct rl_attn_decode_params {
    int n_q, n_kv, head_dim;     /* 24, 4, 256; n_q/n_kv <= 8, head_dim must be 256 */
    int kv_dtype;                /* RL_KV_F16 or RL_KV_Q8K_TQ3V */
    int batch;                   /* sequences in this call */
    int page_tokens;             /* must be 64 */
    int n_pages;                 /* pages in the pool */
    int max_pages_per_seq;       /* row stride of page_table */
    int max_seq_len;             /* host-side upper bound of every seq_lens[b] + len_add (sizing only) */
    int len_add;                 /* tokens attended = seq_lens[b] + len_add (1 when seq_lens holds `pos`) */
    int chunk_pages;             /* least pages a persistent CTA should own (bounds the grid); 0 = 1 */
    int wht_len;                 /* TQ3 transform length: 128 (reference layout) or 256 */
    const float* tq_signs;       /* device [256] +-1 sign vector of the 256 layout, or NULL */
} rl_attn_decode_params;

/* Bytes of scratch rl_attn_decode needs for these parameters. */
size_t rl_attn_decode_workspace_bytes(const rl_attn_decode_params* p);

/* ops::attn_decode (include/rapidllm/kernels/ops.h:130-131,
 * src/kernels/ops.cpp:575-605) for every sequence of a batch, followed by the
 * sigmoid output gate o *= sigmoid(gate) (src/kernels/ops_fused.cpp:178) when
 * gate != NULL.  Replaces qk_attn_decode_gqa_k / flash_attn_decode_f16_hd256
 * (src/kernels/cuda/cuda_engine.cu:5802-5862, 303-375).
 *   k_pool, v_pool  F16: fp16 pools [n_pages][n_kv] of 64x256 slices in the tile
 *                   format written by rl_kv_append (opaque; read back with
 *                   rl_kv_gather).  Q8K_TQ3V: k_pool is the record pool written by
 *                   rl_kv_compact_append, v_pool is ignored; replaces
 *                   qk_attn_decode_tq_gqa_k (cuda_engine.cu:8382-8454).
 *   page_table      int32 [batch][max_pages_per_seq]
 *   seq_lens        int32 [batch], device resident so a step can be graph-captured
 *   q, gate, o      fp32 [batch][n_q][head_dim]; softmax scale 1/sqrt(head_dim) */
int rl_attn_decode(const void* k_pool, const void* v_pool, const int32_t* page_table,
                   const int32_t* seq_lens, const float* q, const float* gate, float* o,
                   void* workspace, size_t workspace_bytes, const rl_attn_decode_params* p,
                   void* stream);

/* rl_attn_decode for callers that must not allocate device memory and have none to lend:
 * code running inside a memory-pool-managed or fixed-budget process where every cudaMalloc
 * is forbidden or already spoken for (a serving engine that sized its pools at start-up,
 * a plug-in loaded into someone else's allocator regime).  This entry point has no
 * counterpart in the reference.  The split-KV partials go to a 4 MiB array that lives in
 * the library's own device image (every GPU that loads the library holds it until exit)
 * instead of a caller workspace; inputs and outputs are still the caller's.  Limits and rules:
 *   - the call needs (SM count + batch * n_kv) * (n_q / n_kv) * 1032 bytes of that array,
 *     rounded up to 512; anything beyond 4 MiB (for 24Q/4KV heads on a 148-SM part:
 *     batch > 132) is refused with RL_ERR_RANGE and a message, nothing is launched;
 *   - the first call of any entry point on a device does the library's one-time set-up for that
 *     device (kernel attributes, a synchronising clear of the 4-byte error word) and this entry
 *     point's first call also looks up the array's device address; make that first call outside
 *     any stream capture.  Every later call allocates nothing: no cudaMalloc / cudaFree, no
 *     stream or event creation, no allocating library routine;
 *   - all calls on a device share the array, which keeps the previous call's contents.
 *     Nothing in it has to start at zero (every slot a call reads, that call wrote first),
 *     but two calls that overlap on the GPU (different streams, or a graph replayed while
 *     another call runs) race on it: serialise them. */
int rl_attn_decode_noalloc(const void* k_pool, const void* v_pool, const int32_t* page_table,
                           const int32_t* seq_lens, const float* q, const float* gate, float* o,
                           const rl_attn_decode_params* p, void* stream);

/* Merge n_parts split-KV partials per row and apply the gate: the grid-level
 * (and cross-GPU) form of the warp merge at cuda_engine.cu:347-374.
 *   part_o  fp32 [n_parts][rows][256] unnormalised sums
 *   part_ml fp32 [n_parts][rows][2]   (running max of scaled scores, sum of exp)
 *   gate    fp32 [rows][256] or NULL;  o fp32 [rows][256]
 *   wht_len 0 for F16 partials; 128 / 256 (+ tq_signs) when the partials come from the
 *           compact cache and are still in the rotated domain of the V transform */
int rl_lse_combine(const float* part_o, const float* part_ml, const float* gate, float* o,
                   int n_parts, int rows, int head_dim, int wht_len, const float* tq_signs,
                   void* stream);

/* Same as rl_attn_decode but stops before the merge across sequences' chunks
 * is normalised: writes one partial (unnormalised o, max, sum) per
 * (sequence, query head) so that partials of several GPUs holding different
 * token ranges can be merged with rl_lse_combine.
 *   part_o fp32 [batch][n_q][256], part_ml fp32 [batch][n_q][2] */
int rl_attn_decode_partial(const void* k_pool, const void* v_pool, const int32_t* page_table,
                           const int32_t* seq_lens, const float* q, float* part_o, float* part_ml,
                           void* workspace, size_t workspace_bytes,
                           const rl_attn_decode_params* p, void* stream);

/* ------------------------------------------------------------------------- */
/* Gated attention, chunked prefill                                           */
/* ------------------------------------------------------------------------- */

/* AttnPrefillParams {n_q, n_kv, head_dim, seq, br, bc} (params.h:18) + chunk position and
 * paging.  br / bc are the row / column tile sizes; this kernel uses 128 / 64 and ignores
 * other requests. */
typedef struct rl_attn_prefill_params {
    int n_q, n_kv, head_dim;     /* 24, 4, 256 */
    int seq;                     /* T: query rows in this chunk */
    int br, bc;
    int pos0;                    /* position of the first row; the cache holds [0, pos0) already */
    int page_tokens, n_pages;    /* 64, pages in the pool */
    int n_table;                 /* entries in page_table_row (>= ceil((pos0 + seq) / 64)) */
} rl_attn_prefill_params;

/* ops::attn_prefill (ops.h:128-129, src/kernels/ops.cpp:542-573) for one chunk of one
 * sequence, the way launch_prefill_chunk drives it (cuda_engine.cu:18338-18590): first the
 * chunk's K,V rows (bf16 [seq][n_kv][256], norm and RoPE applied) are appended to the F16
 * cache at pos0.. (skipped when k_rows is NULL), then row t attends to cache rows
 * [0, pos0 + t] and the result is multiplied by sigmoid(gate) when gate != NULL.
 *   q bf16 [seq][n_q][256];  gate, o fp32 [seq][n_q][256] */
int rl_attn_prefill(void* k_pool, void* v_pool, const int32_t* page_table_row, const void* q_bf16,
                    const void* k_rows_bf16, const void* v_rows_bf16, const float* gate, float* o,
                    const rl_attn_prefill_params* p, void* stream);
/* The same with a workspace: short chunks (the reference's chunks are at most 1024 rows) and the
 * few rows of a speculative verify leave SMs idle when every (query tile, head) is one CTA.  With a
 * workspace of rl_attn_prefill_workspace_bytes() a call with fewer items than SMs divides the KV
 * range of each among several CTAs, and a call whose last wave of CTAs is at most half full (192
 * items of a 1024-row chunk on 148 SMs) divides the items of that wave only; the partials are
 * merged (log-sum-exp, then the gate) by a second kernel.
 * 0 bytes = this call would not be divided; rl_attn_prefill_ws then equals rl_attn_prefill. */
size_t rl_attn_prefill_workspace_bytes(const rl_attn_prefill_params* p);
int rl_attn_prefill_ws(void* k_pool, void* v_pool, const int32_t* page_table_row, const void* q_bf16,
                       const void* k_rows_bf16, const void* v_rows_bf16, const float* gate, float* o,
                       void* workspace, size_t workspace_bytes, const rl_attn_prefill_params* p,
                       void* stream);

/* ------------------------------------------------------------------------- */
/* KV cache maintenance                                                       */
/* ------------------------------------------------------------------------- */

typedef struct rl_kv_append_params {
    int n_kv, head_dim;          /* 4, 256 */
    int batch;                   /* sequences */
    int n_tok;                   /* rows per sequence in this call (1 for decode) */
    int page_tokens, n_pages, max_pages_per_seq;
    int pos0;                    /* first position when pos == NULL */
    int rows_fp16;               /* row element type: 0 fp32 (rounded to nearest even), 1 fp16, 2 bf16 */
    int wht_len;                 /* compact cache only: 128 or 256 */
    int pos_limit;               /* F16 cache only, > 0: rows at positions >= pos_limit are left out (used
                                  * for the F16 window beside a compact cache); 0 = write every row */
} rl_kv_append_params;

/* DualCache::append_kv (src/runtime/dual_cache.cpp:74-79) / store_kv_batch_h_k
 * (cuda_engine.cu:8216-8221): write K and V rows [batch][n_tok][n_kv][256] of
 * each sequence at positions pos[b] (device int32, or pos0 when NULL) + 0..n_tok-1. */
int rl_kv_append(void* k_pool, void* v_pool, const int32_t* page_table, const int32_t* pos,
                 const void* k_rows, const void* v_rows, const rl_kv_append_params* p,
                 void* stream);

/* Read tokens [0, n_tok) of one sequence (its page-table row) of one pool back as
 * contiguous fp16 [n_tok][n_kv][256] -- the reference's cache layout
 * (src/runtime/dual_cache.cpp:49-60). */
int rl_kv_gather(const void* pool, const int32_t* page_table_row, void* out_f16, int n_tok,
                 int n_kv, int head_dim, int n_pages, void* stream);

/* Compact cache (--kv-type q8k_tq3v): K int8 + fp16 scale per row, V Walsh-Hadamard
 * rotated + 3-bit Lloyd-Max codes + fp16 RMS scale per block of wht_len.  Codes and
 * scales are those of store_k_q8_th_k / store_v_tq3_th_k (cuda_engine.cu:8224-8284)
 * evaluated in IEEE fp32.  The pool is n_pages * n_kv * rl_kv_compact_page_bytes()
 * bytes, 358 bytes per token and head as in the reference (cuda_engine.cu:18305-18318). */
size_t rl_kv_compact_page_bytes(void);
/* k_rows, v_rows [batch][n_tok][n_kv][256], fp32 (rows_fp16 == 0) or bf16 (rows_fp16 == 2, widened
 * exactly before quantising); tq_signs device [256] or NULL. */
int rl_kv_compact_append(void* pool, const int32_t* page_table, const int32_t* pos,
                         const void* k_rows, const void* v_rows, const float* tq_signs,
                         const rl_kv_append_params* p, void* stream);
/* Tokens [0, n_tok) of one sequence in the reference's packing: k_q int8 [n_tok][n_kv][256],
 * k_sc fp16 [n_tok][n_kv], v_codes u8 [n_tok][n_kv][96], v_sc fp16 [n_tok][n_kv][256/wht_len]. */
int rl_kv_compact_gather(const void* pool, const int32_t* page_table_row, void* k_q, void* k_sc,
                         void* v_codes, void* v_sc, int n_tok, int n_kv, int n_pages, int wht_len,
                         void* stream);
/* Dequantise tokens [src_pos0, src_pos0 + n_tok) of one sequence of the compact cache into
 * paged F16 pools at positions dst_pos0 ..: the rebuild of the F16 compute window the
 * reference does for prefill chunks and verify rows over a compact cache (dequant_k_q8_k /
 * dequant_v_tq3_256, cuda_engine.cu:8286-8314, 293-299).  Afterwards rl_attn_prefill /
 * rl_attn_decode run over the F16 pools.  Tables are one sequence's rows. */
int rl_kv_compact_to_f16(const void* pool, const int32_t* src_table_row, int src_pos0, int n_src_pages,
                         void* k_pool, void* v_pool, const int32_t* dst_table_row, int dst_pos0,
                         int n_dst_pages, int n_tok, int n_kv, int wht_len, const float* tq_signs,
                         void* stream);

/* ------------------------------------------------------------------------- */
/* Gated DeltaNet                                                             */
/* ------------------------------------------------------------------------- */

/* DeltaRecurrentParams {n_v, dk, dv, eps_l2} (params.h:20) + batch/slot fields. */
typedef struct rl_delta_recurrent_params {
    int n_v, dk, dv;             /* 48, 128, 128 (dk = dv = 128 required) */
    float eps_l2;                /* 1e-6 */
    int batch;                   /* sequences in this call */
    int n_slots;                 /* state slots in S */
    int n_qk;                    /* heads present in q and k */
    int head_map;                /* RL_HEADS_*; PER_VALUE requires n_qk == n_v */
    long long q_stride, k_stride, v_stride; /* floats between sequences; 0 = dense */
} rl_delta_recurrent_params;

/* ops::delta_recurrent_step (ops.h:126-128, src/kernels/ops.cpp:495-540) for a
 * batch: S fp32 [n_slots][n_v][128][128] updated in place (FP32 in HBM, as
 * DualCache keeps it, src/runtime/dual_cache.cpp:29-33); sequence b uses slot
 * slot_ids[b] (or b when NULL).  q,k fp32 [batch][n_qk][128] are L2-normalised
 * inside (q also scaled by 1/sqrt(dk)), v [batch][n_v][128], beta/g_log
 * [batch][n_v], o [batch][n_v][128].  Replaces gdn_decode_t1_k
 * (cuda_engine.cu:5166-5286). */
int rl_delta_recurrent(float* S, const int32_t* slot_ids, const float* q, const float* k,
                       const float* v, const float* beta, const float* g_log, float* o,
                       const rl_delta_recurrent_params* p, void* stream);

/* n_tok consecutive tokens per sequence in one pass with the state kept on chip: the
 * speculative-verify form of the step (gdn_decode_tn_k, cuda_engine.cu:5289-5536;
 * gdn_t12.cu:100-220; Engine::spec_verify, cuda_engine.h:69-77).  q,k [batch][n_tok][n_qk][128],
 * v [batch][n_tok][n_v][128], beta/g_log [batch][n_tok][n_v], o [batch][n_tok][n_v][128];
 * the strides of p are between sequences (0 = dense), qk_tok_stride / v_tok_stride between
 * tokens (0 = dense).  When S_backup != NULL (same shape as S) the state of every touched
 * (slot, head) as it was BEFORE the first token is written there: to roll back to k accepted
 * tokens, copy those heads back and run k tokens.  The result equals n_tok calls of
 * rl_delta_recurrent bit for bit.  n_tok <= 64. */
int rl_delta_recurrent_multi(float* S, float* S_backup, const int32_t* slot_ids, const float* q,
                             const float* k, const float* v, const float* beta, const float* g_log,
                             float* o, const rl_delta_recurrent_params* p, int n_tok,
                             long long qk_tok_stride, long long v_tok_stride, void* stream);

/* DeltaChunkParams {n_v, dk, dv, seq, chunk, eps_l2} (params.h:21; declared but never
 * implemented in the reference) + the key/query head layout. */
typedef struct rl_delta_chunk_params {
    int n_v, dk, dv;             /* 48, 128, 128 */
    int seq;                     /* T tokens of this call */
    int chunk;                   /* must be 64 */
    float eps_l2;                /* 1e-6 */
    int n_qk, head_map;          /* as in rl_delta_recurrent_params */
    long long qk_tok_stride;     /* floats between tokens in q and k; 0 = dense (n_qk * dk) */
    long long v_tok_stride;      /* floats between tokens in v; 0 = dense (n_v * dv).  With both set
                                  * q, k, v can be column ranges of the conv output [T][conv_dim] */
} rl_delta_chunk_params;

size_t rl_delta_chunk_workspace_bytes(const rl_delta_chunk_params* p);
/* Floating-point operations of the tensor-core MMAs rl_delta_chunk_prefill issues per (chunk of 64
 * tokens, value head) in its sequential scan: the figure a tensor roofline of the call is computed
 * from (2 * M * N * K per MMA as issued, the hi + lo operand splits counted as issued). */
double rl_delta_chunk_mma_flops(void);

/* T consecutive delta-rule steps of ONE sequence in chunked (WY) form on the tensor cores:
 * the result of calling ops::delta_recurrent_step (src/kernels/ops.cpp:495-540) T times, which
 * is the reference's only prefill form (src/runtime/session.cpp:232-248; CUDA
 * gdn_prefill_split2_k, cuda_engine.cu:4911-4974).  S fp32 [n_v][128][128] (one slot of the state
 * cache) is read as the initial state and overwritten with the final one; q,k fp32
 * [seq][n_qk][128], v [seq][n_v][128], beta/g_log [seq][n_v], o [seq][n_v][128]. */
int rl_delta_chunk_prefill(float* S, const float* q, const float* k, const float* v, const float* beta,
                           const float* g_log, float* o, void* workspace, size_t workspace_bytes,
                           const rl_delta_chunk_params* p, void* stream);

/* Conv1dParams {dim, k, silu} (params.h:19) + batch/slot fields. */
typedef struct rl_conv1d_params {
    int dim, k, silu;            /* 10240, 4, 1 (silu must be 1) */
    int batch, n_slots;
} rl_conv1d_params;

/* ops::conv1d_update (ops.h:121, src/kernels/ops.cpp:458-468): shift the
 * [dim][k] window of each sequence's slot, append x, dot with w, SiLU.
 * x,y fp32 [batch][dim]; w [dim][k]; state [n_slots][dim][k]. */
int rl_conv1d_update(const float* x, const float* w, float* state, const int32_t* slot_ids,
                     float* y, const rl_conv1d_params* p, void* stream);

/* ops::conv1d_causal_prefill (ops.h:120, src/kernels/ops.cpp:443-456) over
 * x,y fp32 [seq][dim].  state_io (NULL or [dim][k]) receives the window after
 * the last row; when use_state_in != 0 it also supplies the rows before row 0
 * (a later chunk of a chunked prefill). */
int rl_conv1d_causal(const float* x, const float* w, float* y, float* state_io, int seq,
                     const rl_conv1d_params* p, int use_state_in, void* stream);

/* The whole Gated DeltaNet decode step of one layer in one kernel, as the reference's CUDA engine
 * runs it (gdn_decode_t1_k, src/kernels/cuda/cuda_engine.cu:5166-5286): ops::conv1d_update on the
 * q | k | v channels (src/kernels/ops.cpp:458-468), l2 norms, then ops::delta_recurrent_step
 * (495-540), with the CPU operators' arithmetic (double conv accumulator, FP32 state).
 *   qkv       fp32 [batch][conv_dim] channels before the conv, conv_dim = 2 * n_qk * 128 + n_v * 128
 *   conv_w    fp32 [conv_dim][4] taps, oldest first
 *   conv_ring fp32 [n_slots][conv_dim][4] windows kept as RINGS: nothing is shifted, tap slot
 *             (t & 3) holds input x_t, so that the value heads sharing a key head can all read its
 *             channels while one of them stores the new tap.  conv_phase int32 [n_slots] holds
 *             t & 3 of each slot's next token; this call only reads it.  After the layer's step
 *             call rl_gdn_phase_advance once.  rl_conv_ring_export / _import convert to and from
 *             the reference's shifted [conv_dim][4] window (oldest tap first).
 * The other arguments are those of rl_delta_recurrent; conv k must be 4. */
typedef struct rl_gdn_decode_params {
    int n_v, n_qk, dk, dv;       /* 48, 16, 128, 128 */
    int conv_k;                  /* 4 */
    int batch, n_slots;
    int head_map;                /* RL_HEADS_* */
    float eps_l2;                /* 1e-6 */
} rl_gdn_decode_params;
int rl_gdn_decode(float* S, float* conv_ring, const int32_t* conv_phase, const int32_t* slot_ids,
                  const float* qkv, const float* conv_w, const float* beta, const float* g_log, float* o,
                  const rl_gdn_decode_params* p, void* stream);
/* conv_phase[l][slot_ids[b]] = (phase + n_tok) & 3 for l < n_layers, b < batch; conv_phase int32
 * [n_layers][n_slots]. */
int rl_gdn_phase_advance(int32_t* conv_phase, const int32_t* slot_ids, int n_layers, int n_slots, int batch,
                         int n_tok, void* stream);
/* Rings [n_layers][n_slots][conv_dim][4] <-> the reference's windows (ops::conv1d_update's state,
 * DualCache::conv_ptr, src/runtime/dual_cache.cpp:67-70) of slot `slot`, or of every slot when
 * slot < 0: canon fp32 [n_layers][n_slots or 1][conv_dim][4].  Import resets the phases it covers. */
int rl_conv_ring_export(const float* conv_ring, const int32_t* conv_phase, float* canon, int n_layers,
                        int n_slots, int slot, int conv_dim, void* stream);
int rl_conv_ring_import(float* conv_ring, int32_t* conv_phase, const float* canon, int n_layers, int n_slots,
                        int slot, int conv_dim, void* stream);

/* ---- element-wise steps around the mixers (the "next" ring of the path) ---- */

typedef struct rl_attn_qk_prepare_params {
    int n_q, n_kv, head_dim;     /* head_dim 256 */
    int rotary_dim;              /* 64: even, <= head_dim */
    int rows;                    /* tokens: batch at decode, chunk length at prefill */
    int pos0;                    /* used when pos == NULL: row r is at position pos0 + r */
    float theta;                 /* 1e7 */
    float eps;                   /* 1e-6 */
} rl_attn_qk_prepare_params;

/* What fused_attn_decode does between its projections and the cache append
 * (src/kernels/ops_fused.cpp:154-171; cuda_engine.cu:5819-5839, 93-115): split
 * qg [rows][n_q][2*hd] ([q | gate] per head) into q_out and gate_out, head RMSNorm
 * with weight (1 + gamma) on q and on k (ops::qwen3_rmsnorm, ops.cpp:107-127; q_norm,
 * k_norm [hd] or NULL), partial RoPE at pos[row] on the first rotary_dim dims
 * (ops::rope_partial, ops.cpp:470-493).  k [rows][n_kv][hd] is updated in place. */
int rl_attn_qk_prepare(const float* qg, float* k, const float* q_norm, const float* k_norm,
                       const int32_t* pos, float* q_out, float* gate_out,
                       const rl_attn_qk_prepare_params* p, void* stream);

/* ops::qwen3_rmsnorm (ops.h, ops.cpp:107-127) over rows of n values: the norm in front of a
 * mixer's projections (ops_fused.cpp:99, 151): y = x / rms(x) * (1 + gamma); gamma [n] or NULL.
 * x and y may be the same buffer. */
int rl_rmsnorm(const float* x, const float* gamma, float* y, int rows, int n, float eps, void* stream);

/* ops::gated_rmsnorm in its per-head form (ops.h:22, ops.cpp:129-157), applied to
 * the delta-rule output (ops_fused.cpp:131): y = gamma * (x / rms(x)) * silu(z) per
 * head.  x, z, y [rows][n_heads][head_dim] (head_dim 128); gamma [head_dim] or NULL. */
int rl_gated_rmsnorm(const float* x, const float* z, const float* gamma, float* y, int rows,
                     int n_heads, int head_dim, float eps, void* stream);

/* fp32 -> bf16 (round to nearest even) over n values: the reference's prefill keeps its chunk
 * activations in fp32 (cuda_engine.cu:18338-18590) while rl_attn_prefill takes bf16 rows. */
int rl_cast_f32_to_bf16(const float* x, void* y_bf16, size_t n, void* stream);

/* The gate maths in front of the delta rule (ops_fused.cpp:12-13, 122-123):
 * beta = sigmoid(b), g_log = -exp(A_log) * softplus(a + dt_bias).  a, b, beta, g_log
 * [rows][n_v]; A_log, dt_bias [n_v]. */
int rl_delta_gates(const float* a, const float* b, const float* A_log, const float* dt_bias,
                   float* beta, float* g_log, int rows, int n_v, void* stream);


/* ------------------------------------------------------------------------- */
/* Caches and the layer_types[] dispatch                                      */
/* ------------------------------------------------------------------------- */

/* Device-side replacement of DualCache (include/rapidllm/runtime/dual_cache.h:
 * 11-39): a paged KV pool per full-attention layer and, per linear-attention
 * layer, the FP32 recurrent state and conv window of every sequence slot. */
typedef struct rl_cache rl_cache;

typedef struct rl_cache_config {
    int n_layers;                /* length of layer_types */
    const int* layer_types;      /* RL_LAYER_* per layer (ModelDesc.layers[i].kind) */
    int n_q, n_kv, head_dim;     /* attention: 24, 4, 256 */
    int kv_dtype;                /* RL_KV_F16, or RL_KV_Q8K_TQ3V (then see wht_len, window_tokens below) */
    int page_tokens, n_pages;    /* 64, pool size shared by all attention layers */
    int n_v, n_k, dk, dv;        /* DeltaNet: 48, 16, 128, 128 */
    int conv_k;                  /* must be 4; conv_dim = 2*n_k*dk + n_v*dv */
    int head_map;                /* RL_HEADS_GROUPED (HF) or RL_HEADS_TILED (GGUF) */
    int n_slots;                 /* sequences that can hold DeltaNet state */
    int max_batch, max_pages_per_seq, max_seq_len;
    /* RL_KV_Q8K_TQ3V only (the engine's compact cache, cuda_engine.cu:20106-20165): every token
     * persists as q8 K + TQ3 V; beside it an F16 compute window holds the first window_tokens
     * tokens of every slot (rl_plan_cache gives the size; 0 = no window).  Decode steps attend
     * over the window while the caller says every sequence is inside it (rl_stack_io.kv_window_ok,
     * the engine's rule at 18948-18953, 19048), else over the compact pages; a prefill chunk
     * [pos0, pos0 + T) attends over the window when it ends inside it, else over F16 scratch
     * pages rebuilt from the compact pages (18487-18497, 18331-18336). */
    int wht_len;                 /* 128 (the reference's layout) or 256 */
    int window_tokens;
    const float* tq_signs;       /* HOST [256] +-1 sign vector for wht_len 256, else NULL */
} rl_cache_config;

/* One chunk of one sequence's prompt through every layer: the reference's chunked-prefill driver
 * (launch_prefill / launch_prefill_chunk, src/kernels/cuda/cuda_engine.cu:18854-18873, 18338-18590)
 * for the mixers.  Attention layers append the chunk's K/V rows at pos0 .. pos0+T-1 and attend
 * causally over cache rows [0, pos0+t] (rl_attn_prefill); DeltaNet layers run the causal conv with
 * the slot's window carried from the previous chunk (rl_conv1d_causal) and T delta-rule steps in
 * chunked form on the slot's state (rl_delta_chunk_prefill; q | k | v are column ranges of the conv
 * output).  pos0 == 0 starts the sequence: the slot's state is zeroed and its conv window ignored.
 * Per-layer tensors are stacked over the layers of a kind, like rl_stack_io:
 *   attn_q bf16 [n_attn][T][n_q][256], attn_k, attn_v bf16 [n_attn][T][n_kv][256] (normed, rotated),
 *   attn_gate fp32 [n_attn][T][n_q][256] or NULL, attn_o fp32 [n_attn][T][n_q][256];
 *   delta_qkv fp32 [n_delta][T][conv_dim] (before the conv), delta_beta, delta_g fp32 [n_delta][T][n_v],
 *   delta_o fp32 [n_delta][T][n_v][128]; conv_w fp32 [n_delta][conv_dim][k].
 * After the last chunk rl_stack_decode continues at pos = prompt length with the same page table row
 * and slot.  workspace: rl_stack_prefill_workspace_bytes(cache, pos0, T) bytes, 256-byte aligned. */
typedef struct rl_stack_prefill_io {
    const void* attn_q;
    const void* attn_k;
    const void* attn_v;
    const float* attn_gate;
    float* attn_o;
    const float* delta_qkv;
    const float* delta_beta;
    const float* delta_g;
    float* delta_o;
    const float* conv_w;
    const int32_t* page_table_row;   /* int32 [max_pages_per_seq] of this sequence, on the device */
    int slot;                        /* DeltaNet state slot of this sequence */
    int pos0, T;
} rl_stack_prefill_io;
size_t rl_stack_prefill_workspace_bytes(const rl_cache* c, int pos0, int T);
int rl_stack_prefill(rl_cache* c, const rl_stack_prefill_io* io, void* workspace, size_t workspace_bytes,
                     void* stream);

/* One DeltaNet layer of rl_stack_prefill on its own, for a host that runs the layers one after the
 * other with its projections in between (launch_gdn, cuda_engine.cu:10584-10606, inside
 * launch_prefill_chunk): causal conv over the chunk's T rows with slot's window carried (pos0 > 0) or
 * empty (pos0 == 0, which also zeroes the slot's state), then T delta-rule steps in chunked form.
 * qkv fp32 [T][conv_dim] before the conv, conv_w [conv_dim][4], beta / g_log [T][n_v], o [T][n_v][dv].
 * workspace: rl_cache_delta_prefill_workspace_bytes(c, T) bytes, 256-byte aligned. */
size_t rl_cache_delta_prefill_workspace_bytes(const rl_cache* c, int T);
int rl_cache_delta_prefill(rl_cache* c, int delta_index, int slot, int pos0, int T, const float* qkv,
                           const float* conv_w, const float* beta, const float* g_log, float* o,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Memory plan for a cache: PlannerInput / PlannerResult / plan_memory
 * (include/rapidllm/runtime/planner.h:11-33, src/runtime/planner.cpp:28-44) plus the engine's
 * KV-type policy (RAPIDLLM_KV_TQ / automatic switch to the compact cache for long contexts,
 * src/kernels/cuda/cuda_engine.cu:20106-20118), restated for paged pools: pages come out of
 * what is left of `available_bytes` after weights, DeltaNet state, conv windows and padding. */
#define RL_KV_POLICY_AUTO 0      /* F16 when it fits, else the compact cache (RAPIDLLM_KV_TQ unset) */
#define RL_KV_POLICY_F16 1       /* RAPIDLLM_KV_TQ=0 */
#define RL_KV_POLICY_COMPACT 2   /* RAPIDLLM_KV_TQ=1 */
typedef struct rl_plan_input {
    unsigned long long weight_bytes;     /* what else must stay resident */
    unsigned long long available_bytes;  /* budget; 0 = do not check (plan_memory's convention) */
    unsigned long long pad_bytes;        /* head-room; the reference uses 64 MiB */
    int ctx;                     /* tokens per sequence asked for */
    int max_batch;               /* sequences (KV page sets and DeltaNet slots) */
    int n_attn_layers, n_kv, head_dim;
    int n_delta_layers, n_v, dk, dv, conv_dim, conv_k;
    int page_tokens;             /* 64 */
    int kv_policy;               /* RL_KV_POLICY_* */
    int allow_shrink;            /* != 0: reduce ctx to what fits instead of refusing */
    int prefill_chunk;           /* longest prefill chunk (the engine's pf_cap_); 0 = 1024 */
} rl_plan_input;
typedef struct rl_plan_result {
    int ok;                      /* 0: does not fit (message says why), like PlannerResult.ok */
    int kv_dtype;                /* RL_KV_F16 or RL_KV_Q8K_TQ3V */
    int ctx;                     /* granted tokens per sequence (a multiple of page_tokens when shrunk) */
    int max_pages_per_seq;
    int n_pages;                 /* per attention layer pool: max_batch * max_pages_per_seq */
    unsigned long long kv_bytes, state_bytes, need_bytes;
    /* With the compact cache the engine also keeps an F16 compute window over the first
     * min(ctx, max(8192, 2 * prefill_chunk)) tokens of every sequence and attends over it while
     * a sequence still fits (cuda_engine.cu:20118-20123, 18948, 18487-18493); 0 with F16 KV.
     * kv_bytes counts both. */
    int window_tokens, window_pages_per_seq;
    unsigned long long window_bytes;
    char message[160];
} rl_plan_result;
/* Host-only arithmetic (no device call); returns RL_OK when the plan was computed (see
 * result->ok for whether it fits) and RL_ERR_RANGE for nonsensical input. */
int rl_plan_cache(const rl_plan_input* in, rl_plan_result* out);

/* DualCache::DualCache (src/runtime/dual_cache.cpp:7-41): allocates and zeroes. */
int rl_cache_create(const rl_cache_config* cfg, rl_cache** out);
void rl_cache_destroy(rl_cache* c);
size_t rl_cache_bytes(const rl_cache* c);
/* DualCache::k_ptr / v_ptr / state_ptr / conv_ptr (dual_cache.cpp:49-70), by
 * the index among layers of the same kind (ModelDesc::mixer_slot,
 * src/ir/model_desc.cpp:12-22). */
void* rl_cache_k_pool(rl_cache* c, int attn_index);
void* rl_cache_v_pool(rl_cache* c, int attn_index);
/* Compact cache: k_pool above is the layer's record pool (rl_kv_compact_append's format) and v_pool is
 * NULL; these are the F16 window pools [n_slots * window pages][n_kv] of 64x256 slices (slot s owns
 * pages [s * wp, (s + 1) * wp), wp = ceil(window_tokens / 64)), NULL without a window. */
void* rl_cache_window_k_pool(rl_cache* c, int attn_index);
void* rl_cache_window_v_pool(rl_cache* c, int attn_index);
float* rl_cache_state(rl_cache* c, int delta_index);
/* The conv windows of a layer as stored: rings [n_slots][conv_dim][4] (see rl_gdn_decode); equal to
 * the reference's shifted windows only while no token has been consumed since creation, rl_cache_zero
 * or rl_cache_conv_import.  rl_cache_conv_export / _import convert: canon fp32
 * [n_slots][conv_dim][conv_k], oldest tap first (DualCache::conv_ptr). */
float* rl_cache_conv(rl_cache* c, int delta_index);
int32_t* rl_cache_conv_phase(rl_cache* c, int delta_index);     /* int32 [n_slots], see rl_gdn_decode */
int rl_cache_conv_export(rl_cache* c, int delta_index, float* canon, void* stream);
int rl_cache_conv_import(rl_cache* c, int delta_index, const float* canon, void* stream);
/* DualCache::zero (dual_cache.cpp:43-47). */
int rl_cache_zero(rl_cache* c, void* stream);

/* Optional: the element-wise steps on either side of the operators run inside the step, as the
 * reference fuses them into its decode kernels (q/gate split + head RMSNorm + partial RoPE before the
 * attention, cuda_engine.cu:5819-5850; the gate maths before and the gated RMSNorm after the delta
 * rule, 5644-5653, 4400-4424): rl_attn_qk_prepare, rl_delta_gates, rl_gated_rmsnorm.  The step then
 * takes the raw projections instead of the prepared tensors.  Indexing as in rl_stack_io. */
typedef struct rl_stack_glue {
    const float* attn_qg;        /* [n_attn][batch][n_q][2*256] ([q | gate] per head): replaces attn_q, attn_gate */
    float* attn_k_raw;           /* [n_attn][batch][n_kv][256] K rows before norm and RoPE, updated in place:
                                  * replaces attn_k (attn_v is still read from rl_stack_io) */
    const float* q_norm;         /* [n_attn][256] or NULL */
    const float* k_norm;         /* [n_attn][256] or NULL */
    int rotary_dim;              /* 64 */
    float theta;                 /* 1e7 */
    float rms_eps;               /* 1e-6 */
    const float* delta_a;        /* [n_delta][batch][n_v]: with delta_b replaces delta_beta, delta_g */
    const float* delta_b;
    const float* A_log;          /* [n_delta][n_v] */
    const float* dt_bias;        /* [n_delta][n_v] */
    const float* delta_z;        /* [n_delta][batch][n_v][dv] or NULL: delta_o = gated RMSNorm(o, z) */
    const float* gnorm;          /* [n_delta][dv] or NULL */
} rl_stack_glue;

/* Inputs of one decode step of the attention/DeltaNet-only stack.  Arrays are
 * indexed by the layer's index among its kind, then by sequence. */
typedef struct rl_stack_io {
    const float* attn_q;         /* [n_attn][batch][n_q][256] */
    const float* attn_gate;      /* [n_attn][batch][n_q][256] pre-activation */
    const float* attn_k;         /* [n_attn][batch][n_kv][256] new K row (norm + RoPE applied) */
    const float* attn_v;         /* [n_attn][batch][n_kv][256] */
    float* attn_o;               /* [n_attn][batch][n_q][256] */
    const float* delta_qkv;      /* [n_delta][batch][conv_dim] pre-conv q|k|v channels */
    const float* delta_beta;     /* [n_delta][batch][n_v] */
    const float* delta_g;        /* [n_delta][batch][n_v]  log decay */
    float* delta_o;              /* [n_delta][batch][n_v][dv] */
    const float* conv_w;         /* [n_delta][conv_dim][conv_k] (weights, read only) */
    const int32_t* page_table;   /* [batch][max_pages_per_seq] */
    const int32_t* pos;          /* [batch] position of the token being decoded */
    const int32_t* slot_ids;     /* [batch] DeltaNet slot per sequence or NULL */
    int batch;
    /* Split-KV across devices (each device holds a token range of every sequence): with
     * attn_ml != NULL the attention layers emit one partial per (sequence, query head) instead
     * of the final output -- attn_o unnormalised and ungated, attn_ml [n_attn][batch][n_q][2]
     * (max in natural-log units, sum) -- to be gathered over the devices and merged with
     * rl_lse_combine (which applies the gate).  no_append != 0: this device does not hold the
     * sequences' tail, so nothing is appended and the layer attends over pos tokens instead
     * of pos + 1. */
    float* attn_ml;
    int no_append;
    /* Compact cache only: != 0 = the caller (who knows the positions on the host, like the engine's
     * decode_tokens(tokens, poss, B)) asserts that every pos[b] < window_tokens, so the attention
     * layers read the F16 window; 0 = they read the compact pages (always valid). */
    int kv_window_ok;
    const rl_stack_glue* glue;   /* NULL, or the raw projections and the small weights (device step only) */
} rl_stack_io;

/* One decode step over layer_types[]: the scheduler loop of
 * Session::forward_hidden (src/runtime/session.cpp:325-411) / launch_decode_batch
 * (cuda_engine.cu:18999-19106) restricted to the mixer operators.  Per
 * full-attention layer: append K,V at pos, attend over pos+1 tokens, gate.
 * Per linear-attention layer: conv1d_update on the q|k|v channels, then the
 * delta rule, in one kernel (rl_gdn_decode).  All pointers in io are device pointers. */
int rl_stack_decode(rl_cache* c, const rl_stack_io* io, void* stream);
/* Graph replay of rl_stack_decode, the counterpart of the reference's captured decode step
 * (cuda_engine.cu:18787-18789 keeps positions on the device for that purpose).  Enabled by
 * default: the first step with a given io (same pointers and batch) runs as plain launches,
 * the second is captured into a CUDA graph, later ones replay it.  Positions, page table and
 * slot ids are read from device memory at run time, so the caller may advance them between
 * steps; a different io re-captures.  rl_stack_decode_host does the same with its copies in and
 * out included (pinned host buffers; with pageable ones it stays on plain launches).  Disabled
 * while rl_stack_set_timing is on. */
int rl_stack_set_graph(rl_cache* c, int enable);

/* ---- one batch on several GPUs of one node ---------------------------------------------------
 * The reference engine is single-GPU (one Engine per process, cuda_engine.h:13-83); this part has
 * no counterpart there.  The mixers shard without moving KV or state: every rank (one process per
 * GPU) owns a slice of the KV heads / DeltaNet value heads (its rl_cache is created with the local
 * head counts), and/or a subset of the sequences, and/or a token range of every sequence
 * (rl_stack_io.attn_ml / no_append).  The one exchange is an all-gather of the per-layer outputs,
 * issued by rl_stack_decode on an internal side stream right after the layer that produced them,
 * so it runs beside the following layers; the step's stream waits for the last exchange at the end
 * of the step.  Transport: NCCL (ncclAllGather over NVLink / NVSwitch), bound at run time from
 * libnccl.so.2; no peer pointers, no multicast loads. */
#define RL_COMM_ID_BYTES 128
typedef struct rl_comm rl_comm;
/* ncclGetUniqueId: called by one rank; the host program hands the RL_COMM_ID_BYTES bytes to every
 * rank (any transport: a file, MPI, torch.distributed ...). */
int rl_comm_unique_id(void* id);
/* ncclCommInitRank on the current device; collective over the n_ranks processes. */
int rl_comm_create(const void* id, int rank, int n_ranks, rl_comm** out);
void rl_comm_destroy(rl_comm* comm);

/* Where the gathered outputs of a sharded step go (all device pointers, owned by the caller, fixed
 * for the life of the setting).  n_q, n_v below are this rank's LOCAL head counts and batch the
 * LOCAL batch, as in rl_stack_io; every rank must use the same local shapes.
 *   attn_o_all   [n_attn][n_ranks][batch][n_q][256]   block r = rank r's attn_o of that layer
 *   delta_o_all  [n_delta][n_ranks][batch][n_v][dv]
 *   attn_ml_all  [n_attn][n_ranks][batch][n_q][2]     split-KV only (io.attn_ml != NULL)
 *   attn_o_final [n_attn][batch][n_q][256]            split-KV only: the partials of all ranks merged
 *                                                     (log-sum-exp) and gated, on every rank
 * layers_per_exchange: how many layers' outputs one grouped exchange carries; 0 = 4 (one exchange
 * per attention layer of the 3 + 1 pattern); n_layers = a single exchange at the end of the step. */
typedef struct rl_stack_gather {
    rl_comm* comm;
    float* attn_o_all;
    float* delta_o_all;
    float* attn_ml_all;
    float* attn_o_final;
    int layers_per_exchange;
    int reserve_sms;             /* SMs the step's persistent kernels leave free so that the exchange kernels
                                  * run beside them instead of between them; 0 = none */
} rl_stack_gather;
/* Attach (or, with g == NULL, detach) the exchange to every following rl_stack_decode[_host] of
 * this cache.  Every rank of the communicator must then call the step the same number of times. */
int rl_stack_set_gather(rl_cache* c, const rl_stack_gather* g);

/* The same step for a caller that keeps its tensors in HOST memory (pinned for
 * full speed): copies every input of io (host pointers) to staging buffers on
 * the device, runs the step and copies attn_o / delta_o back, overlapping the
 * copies with the layers on internal streams.  conv_w is taken from the last
 * rl_stack_set_conv_w call.  Returns after the outputs are in host memory. */
int rl_stack_decode_host(rl_cache* c, const rl_stack_io* host_io);
/* Upload the conv weights [n_delta][conv_dim][conv_k] (host pointer) once. */
int rl_stack_set_conv_w(rl_cache* c, const float* host_conv_w);
/* Number of kernels rl_stack_decode enqueues for a batch of this cache's shape. */
int rl_stack_launches_per_step(const rl_cache* c);
/* Phase timing with CUDA events on the launching stream, the counterpart of the
 * reference's RAPIDLLM_PF_PROFILE brackets (cuda_engine.cu:18362-18380,
 * 18581-18589).  While enabled every rl_stack_decode[_host] records events
 * between its kernels; rl_stack_timing waits for the last step and returns the
 * summed milliseconds over the layers in ms[5]: [0] KV append, [1] split-KV
 * decode kernel, [2] merge + gate, [3] conv1d update, [4] delta rule. */
int rl_stack_set_timing(rl_cache* c, int enable);
int rl_stack_timing(rl_cache* c, float* ms);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* RL_B200_H */
