// Launch-side declarations shared by the kernels and the C ABI (api.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace rl {

// ---- decode attention over the paged F16 cache ------------------------------
struct AttnDecodeArgs {
    const __half* k_pool;        // [n_pages][n_kv] slices, see kv_slice_offset()
    const __half* v_pool;
    const int32_t* page_table;   // [batch][max_pages_per_seq]
    const int32_t* seq_lens;     // [batch] device resident; tokens attended = seq_lens[b] + len_add
    const float* q;              // [batch][n_q][256]
    float* part_o;               // [grid + batch*n_kv][G][256] unnormalised partial outputs
    float* part_ml;              // [grid + batch*n_kv][G][2]   (max in natural-log units, sum)
    int* err;                    // device error word
    int batch, n_q, n_kv, n_pages, max_pages_per_seq;
    int len_add;
    float scale;                 // 1/sqrt(head_dim)
    int seg_weight;              // charge per (sequence, head) boundary in the division of the units (attn_split.cuh)
    // 1 (F16 kernel, inside a step): lengths, page table and every page but a sequence's last are the caller's or an
    // earlier step's, so the producer streams them before it waits for the kernel in front (the append of this
    // step's token, which writes into the last page)
    int stream_before_wait;
};
__global__ void attn_decode_f16_kernel(AttnDecodeArgs a);
// same arguments over the compact cache: k_pool = record pool (kv_compact.cu), v_pool unused
__global__ void attn_decode_tq_kernel(AttnDecodeArgs a);
size_t attn_decode_tq_smem_bytes();
int attn_decode_tq_threads();
size_t attn_decode_f16_smem_bytes();
int attn_decode_f16_threads();
int attn_decode_max_batch();

// ---- chunked causal attention prefill (tcgen05) ------------------------------------------
struct AttnPrefillArgs {
    const __half* k_pool;
    const __half* v_pool;
    const int32_t* page_table;   // this sequence's row
    const __nv_bfloat16* q;      // [T][n_q][256]
    const float* gate;           // [T][n_q][256] or null
    float* o;                    // [T][n_q][256]
    int* err;
    int T, pos0, n_q, n_kv, n_pages;
    float scale;
    // kv_parts > 1: the KV tiles of every (query tile, head) are divided among kv_parts CTAs; part p
    // writes its unnormalised, ungated output to part_o [p][T][n_q][256] and (max in natural-log
    // units, sum) to part_ml [p][T][n_q][2] for lse_combine_kernel, which applies the gate
    int kv_parts;
    float* part_o;
    float* part_ml;
    int packed;                  // T * (n_q / n_kv) <= 128: one item per KV head, MMA rows = (token, head of the group)
    int wave;                    // CTAs resident at a time (one per SM): CTA i + wave is taken to follow CTA i on its SM
    // tail_parts > 1 (with kv_parts <= 1): the first n_full items of the launch order run whole; each
    // later item is divided among tail_parts CTAs, launched after all whole items, so that the last,
    // partly filled wave is spread over every SM.  Unit u = (item - n_full) * tail_parts + part writes
    // part_o [u][128][256] and part_ml [u][128][2]; attn_prefill_tail_merge_kernel finishes those rows.
    int n_full, tail_parts;
    // order of the items along the grid: 0 = one KV head after the other, inside it the longest jobs first;
    // 1 = by size over all heads (all query heads of the last query tile, then of the one before, ...), for calls
    // of fewer than two waves, whose second wave should hold the shortest items
    int by_size;
};
__global__ void attn_prefill_kernel(AttnPrefillArgs a);
__global__ void attn_prefill_tail_merge_kernel(AttnPrefillArgs a);
size_t attn_prefill_smem_bytes();
int attn_prefill_threads();
int attn_prefill_q_rows();

// ---- merge of split-KV partials + sigmoid gate -----------------------------------
struct AttnCombineArgs {
    const float* part_o;
    const float* part_ml;
    const int32_t* seq_lens;
    const float* gate;           // [batch][n_q][256] pre-activation, may be null
    float* o;                    // [batch][n_q][256]; unnormalised when out_ml != null
    float* out_ml;               // null, or [batch][n_q][2] (max, sum): emit one partial per row
    int batch, n_q, n_kv, len_add;
    int n_ctas;                  // grid size of the decode kernel that wrote the partials
    int seg_weight;              // the decode kernel's charge per (sequence, head) boundary, in units (attn_split.cuh)
    int max_len;                 // lengths outside [0, max_len] count as 0, as in the decode kernel
    int wht_len;                 // 0, or 128 / 256: the partials are in the rotated domain of TQ3 V
    const float* signs;          // [256] +-1 applied after the inverse transform, or null
};
__global__ void attn_combine_kernel(AttnCombineArgs a);

// Generic merge of n_parts partials per row (used across GPUs):
// part_o [n_parts][rows][256], part_ml [n_parts][rows][2]
__global__ void lse_combine_kernel(const float* part_o, const float* part_ml, const float* gate,
                                   float* o, int n_parts, int rows, int wht_len, const float* signs);

// ---- KV cache maintenance ------------------------------------------------------------
// Write rows [n_tok][n_kv][256] (fp32 or fp16) of sequence b at positions pos0.. into the pool.
struct KvWriteArgs {
    __half* k_pool;
    __half* v_pool;
    const int32_t* page_table;   // [batch][max_pages_per_seq]
    const int32_t* pos;          // [batch] device positions (decode append) or null
    const void* k_rows;          // [batch][n_tok][n_kv][256]
    const void* v_rows;
    int* err;
    int batch, n_tok, n_kv, n_pages, max_pages_per_seq;
    int pos0;                    // used when pos == null
    int rows_fp16;               // row element type: 0 fp32 (rounded to nearest even), 1 fp16, 2 bf16
    int pos_limit;               // > 0: rows at positions >= pos_limit are left out (the F16 window of a compact cache)
    // 1: nothing this kernel reads or writes is touched by the kernels in front of it in the step (its rows are the
    // caller's, its pages belong to its own layer), so it works first and waits for the kernel in front afterwards
    int early;
};
__global__ void kv_write_kernel(KvWriteArgs a);
// rows[b][j] = slot_ids[b] * pages_per_slot + j: the page-table rows of a step's sequences in a pool
// where slot s owns pages [s * pages_per_slot, (s + 1) * pages_per_slot); grid (batch), any block
__global__ void kv_slot_rows_kernel(int32_t* rows, const int32_t* slot_ids, int pages_per_slot, int n_slots, int* err);
// Read tokens [0, n_tok) of one sequence back as contiguous fp16 [n_tok][n_kv][256].
__global__ void kv_gather_kernel(const __half* pool, const int32_t* table, __half* out, int n_tok,
                                 int n_kv, int n_pages, int* err);

// ---- compact KV (q8 K + TQ3 V) ---------------------------------------------------------
struct KvCompactWriteArgs {
    unsigned char* pool;         // [n_pages][n_kv][2] records of kCompactRecordBytes
    const int32_t* page_table;
    const int32_t* pos;          // [batch] or null
    const void* k_rows;          // [batch][n_tok][n_kv][256] fp32 (or bf16 when rows_bf16)
    const void* v_rows;
    const float* signs;          // [256] +-1 (wht_len 256) or null
    int* err;
    int batch, n_tok, n_kv, n_pages, max_pages_per_seq, pos0, wht_len;
    int rows_bf16;               // rows are bf16 (a prefill chunk's rows), widened exactly before quantising
};
__global__ void kv_compact_write_kernel(KvCompactWriteArgs a);
__global__ void kv_compact_gather_kernel(const unsigned char* pool, const int32_t* table, signed char* k_q,
                                         __half* k_sc, unsigned char* v_codes, __half* v_sc, int n_tok,
                                         int n_kv, int n_pages, int wht_len, int* err);
__global__ void kv_compact_to_f16_kernel(const unsigned char* pool, const int32_t* src_table, int src_pos0,
                                         int n_src_pages, __half* k_pool, __half* v_pool, const int32_t* dst_table,
                                         int dst_pos0, int n_dst_pages, int n_kv, int wht_len, const float* signs,
                                         int* err);

// ---- Gated DeltaNet decode step ----------------------------------------------------
struct DeltaDecodeArgs {
    float* S;                    // [n_slots][n_v][128][128] fp32 recurrent state
    const int32_t* slot_ids;     // [batch] state slot of each sequence, or null (slot = b)
    const float* q;              // [batch][n_qk][128]
    const float* k;              // [batch][n_qk][128]
    const float* v;              // [batch][n_v][128]
    const float* beta;           // [batch][n_v]
    const float* g_log;          // [batch][n_v]
    float* o;                    // [batch][n_v][128]
    int* err;
    int batch, n_v, n_qk, n_slots;
    int head_map;                // 0: q/k given per value head; 1: grouped h/(n_v/n_qk); 2: tiled h%n_qk
    float eps_l2;
    long long q_stride, k_stride, v_stride;   // floats between sequences
};
void launch_delta_decode(const DeltaDecodeArgs& a, int sms, cudaStream_t st);
// n_tok consecutive tokens per sequence with the state kept on chip; a.beta, a.g_log
// [batch][n_tok][n_v], a.o [batch][n_tok][n_v][128]; q/k/v token t at + t * tstride floats
void launch_delta_decode_multi(const DeltaDecodeArgs& a, float* S_backup, int n_tok, long long qk_tstride,
                               long long v_tstride, cudaStream_t st);
size_t delta_decode_stream_smem_bytes();
const void* delta_decode_stream_kernel_ptr();

// ---- fused Gated DeltaNet decode step: conv window + SiLU + l2 norms + delta rule (gdn_decode.cu) ----
// The conv windows of the cache are kept as rings: tap slot (t & 3) of a channel holds input x_t,
// nothing is shifted.  conv_phase [n_slots] = t & 3 of the NEXT token of each slot; a step reads the
// three older taps, writes x into slot phase, and gdn_phase_advance_kernel bumps the phase once
// after the layer's last reader is done.
struct GdnDecodeArgs {
    float* S;                    // [n_slots][n_v][128][128] fp32 recurrent state
    float* conv;                 // [n_slots][conv_dim][4] ring windows
    const int32_t* conv_phase;   // [n_slots]
    const int32_t* slot_ids;     // [batch] or null (slot = b)
    const float* x;              // [batch][conv_dim] q | k | v channels before the conv
    const float* w;              // [conv_dim][4] taps, oldest first
    const float* beta;           // [batch][n_v]
    const float* g_log;          // [batch][n_v]
    float* o;                    // [batch][n_v][128]
    int* err;
    int batch, n_v, n_qk, n_slots, head_map, conv_dim;
    float eps_l2;
    // 1 (inside a step whose DeltaNet inputs are the caller's): nothing the kernel touches belongs to a kernel in
    // front of it in the step, so it works at once -- filling the SMs the previous layer's last round leaves idle --
    // and waits for the kernel in front only before it ends
    int early;
};
// heads (items) from which the streaming form is used instead of one CTA per column slice
void launch_gdn_decode(const GdnDecodeArgs& a, int sms, cudaStream_t st, int stream_min_items, int grid_override = 0);
int gdn_stream_grid(int items, int sms);
size_t gdn_decode_stream_smem_bytes();
const void* gdn_decode_stream_kernel_ptr();
// phase[l][slot_ids[b]] = (phase + n_tok) & 3 for l < n_layers, b < batch (phase [n_layers][n_slots])
void launch_gdn_phase_advance(int32_t* phase, const int32_t* slot_ids, int n_layers, int n_slots, int batch, int n_tok,
                              int* err, cudaStream_t st);
// ring [n_layers][n_slots][dim][4] <-> oldest-first windows for slot `slot` (or every slot when slot < 0):
// canon [n_layers][n_slots or 1][dim][4]; import also resets the phases it covers to 0
void launch_conv_ring_export(const float* ring, const int32_t* phase, float* canon, int n_layers, int n_slots, int slot,
                             int dim, cudaStream_t st);
void launch_conv_ring_import(float* ring, int32_t* phase, const float* canon, int n_layers, int n_slots, int slot,
                             int dim, cudaStream_t st);

// ---- element-wise steps around the mixers (layer_glue.cu) ------------------------------------
struct AttnQkPrepareArgs {
    const float* qg;             // [rows][n_q][2 * 256]  ([q | gate] per head)
    float* k;                    // [rows][n_kv][256] in place
    const float* q_norm;         // [256] or null
    const float* k_norm;         // [256] or null
    const int32_t* pos;          // [rows] or null (then pos0 + row)
    float* q_out;                // [rows][n_q][256]
    float* gate_out;             // [rows][n_q][256]
    int n_q, n_kv, rotary_dim, pos0;
    float eps;
    float inv_freq[128];         // 1 / theta^(i / pairs), i < rotary_dim / 2, computed on the host
};
__global__ void attn_qk_prepare_kernel(AttnQkPrepareArgs a);
struct GatedRmsnormArgs {
    const float* x;              // [rows][n_heads][head_dim]
    const float* z;
    const float* gamma;          // [head_dim] or null
    float* y;
    int n_heads, head_dim;
    float eps;
};
__global__ void gated_rmsnorm_kernel(GatedRmsnormArgs a);
__global__ void rmsnorm_kernel(const float* x, const float* gamma, float* y, int n, float eps);
__global__ void cast_f32_bf16_kernel(const float* x, __nv_bfloat16* y, size_t n);
__global__ void delta_gates_kernel(const float* a_in, const float* b_in, const float* A_log, const float* dt_bias,
                                   float* beta, float* g_log, int n_v, int rows);

// ---- chunked (WY-form) DeltaNet prefill (tcgen05) --------------------------------------------
struct DeltaChunkArgs {
    float* S;                    // [n_v][128][128] fp32 state of one sequence, in place
    const float* q;              // [T][n_qk][128]
    const float* k;              // [T][n_qk][128]
    const float* v;              // [T][n_v][128]
    const float* beta;           // [T][n_v]
    const float* g_log;          // [T][n_v]
    float* o;                    // [T][n_v][128]
    unsigned char* work;         // [n_chunks][n_v] records of delta_chunk_record_bytes()
    float* chunk_decay;          // [n_chunks][n_v]
    float* keys;                 // [n_chunks][n_qk] records of delta_chunk_keys_bytes(): what a key head's value heads share
    int* err;
    int T, n_v, n_qk, head_map;
    float eps_l2;
    long long qk_tok_stride, v_tok_stride;   // floats between tokens in q/k and in v
    int chunk0, chunks;          // this launch covers chunks [chunk0, chunk0 + chunks) of the T tokens
};
__global__ void delta_chunk_keys_kernel(DeltaChunkArgs a);
__global__ void delta_chunk_prepare_kernel(DeltaChunkArgs a);
size_t delta_chunk_keys_bytes();
__global__ void delta_chunk_scan_kernel(DeltaChunkArgs a);
size_t delta_chunk_record_bytes();
size_t delta_chunk_prepare_smem_bytes();
int delta_chunk_prepare_threads();
size_t delta_chunk_scan_smem_bytes();
int delta_chunk_scan_threads();
double delta_chunk_scan_mma_flops();     // flops of the MMAs the scan issues per (chunk, head)

// ---- causal depthwise conv1d + SiLU ------------------------------------------------
struct ConvUpdateArgs {
    const float* x;              // [batch][dim]
    const float* w;              // [dim][k]
    float* state;                // [n_slots][dim][k]
    const int32_t* slot_ids;     // may be null
    float* y;                    // [batch][dim]
    int* err;
    int batch, dim, k, n_slots;
};
void launch_conv1d_update(const ConvUpdateArgs& a, cudaStream_t st);
// x,y [seq][dim]; state_out (may be null) receives the last k inputs [dim][k]
void launch_conv1d_prefill(const float* x, const float* w, float* y, float* state_io, int seq,
                           int dim, int k, int use_state_in, cudaStream_t st);

}  // namespace rl
