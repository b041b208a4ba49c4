// Compact KV cache: K as int8 with one fp16 scale per row, V as TurboQuant-3
// (Walsh-Hadamard rotation + 3-bit Lloyd-Max codes + fp16 RMS scale per block).
//
// The arithmetic follows the reference's store kernels
// (src/kernels/cuda/cuda_engine.cu:8224-8249 store_k_q8_th_k, 8252-8284
// store_v_tq3_th_k, helpers 199-254) in IEEE fp32: true division, sqrtf,
// first-minimum ties, sum of squares as a xor butterfly inside groups of 32 and
// the groups added in ascending order.  This file is compiled with -fmad=false
// so no multiply-add is fused: the codes must equal the CPU restatement bit for
// bit.  wht_len 128 = two independent blocks per head without signs (the
// reference layout); wht_len 256 = one block per head with a +-1 sign vector
// applied before the transform.
//
// Storage is paged like the F16 cache, in records of half a page (32 tokens) per
// KV head, kCompactRecordBytes each, laid out for the decode kernel:
//   [0, 8192)        K int8 [32 rows][256], 16-byte chunk index ^ ((row & 1) << 2)
//   [8192, 11264)    V codes of 16 token pairs (even row, odd row), 192 B per pair, placed by
//                    compact_v_offset(): 24 B per (pair, g = 0..7) holding 16 fields of 12 bits,
//                    field 4j+i = codes of dims d = 64j + 8g + 2i and d+1 for the even and the
//                    odd token of the pair: even(d) | odd(d) << 3 | even(d+1) << 6 | odd(d+1) << 9
//   [11264, 11328)   K scales fp16 [32]
//   [11328, 11456)   V scales fp16 [32][2] (wht_len 256: the one scale in both slots)
// 358 bytes per token and head, the same as the reference's layout
// (cuda_engine.cu:18305-18318).
#include "common.cuh"
#include "kernels.h"

namespace rl {

namespace {

// The 8 reconstruction levels of the 3-bit Lloyd-Max quantiser for a unit normal variable
// (the values the reference's dequantiser maps codes to, cuda_engine.cu:204-208).
__constant__ float kTq3Levels[8] = {-2.152f, -1.344f, -0.756f, -0.245f, 0.245f, 0.756f, 1.344f, 2.152f};

// Code of the level nearest to x.  The scan visits the levels in ascending order and only a
// strictly smaller distance replaces the current choice, so an exact tie keeps the lower code:
// the rule the bit-exact contract with the CPU restatement fixes.
__device__ __forceinline__ int tq3_code(float x) {
    int code = 0;
    float nearest = fabsf(x - kTq3Levels[0]);
#pragma unroll
    for (int level = 1; level < 8; ++level) {
        const float dist = fabsf(x - kTq3Levels[level]);
        const bool closer = dist < nearest;
        nearest = closer ? dist : nearest;
        code = closer ? level : code;
    }
    return code;
}

}  // namespace

// grid (n_tok, n_kv, batch), 256 threads: thread = dim.
__global__ void __launch_bounds__(256) kv_compact_write_kernel(KvCompactWriteArgs a) {
    const int t = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    __shared__ float xs[256];
    __shared__ float wred[8];
    __shared__ float s_scale[2];
    __shared__ unsigned char s_idx[256];

    const int pos = (a.pos ? a.pos[b] : a.pos0) + t;
    const int pi = pos / kPageTokens;
    if (pos < 0 || pi >= a.max_pages_per_seq) {
        if (tid == 0) set_err(a.err, DEV_ERR_BAD_LEN);
        return;
    }
    const int page = a.page_table[size_t(b) * a.max_pages_per_seq + pi];
    if (page < 0 || page >= a.n_pages) {
        if (tid == 0) set_err(a.err, DEV_ERR_BAD_PAGE);
        return;
    }
    const int row64 = pos % kPageTokens;
    const int half = row64 >> 5, row = row64 & 31;
    unsigned char* rec = a.pool + ((size_t(page) * a.n_kv + h) * 2 + half) * kCompactRecordBytes;
    const size_t src = ((size_t(b) * a.n_tok + t) * a.n_kv + h) * kHeadDim;

    // ---------------- K: int8 + fp16 scale ----------------
    const float kx = a.rows_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.k_rows)[src + tid])
                                 : static_cast<const float*>(a.k_rows)[src + tid];
    float amax = fabsf(kx);
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    if (lane == 0) wred[warp] = amax;
    __syncthreads();
    if (tid == 0) {
        float m = wred[0];
        for (int w = 1; w < 8; ++w) m = fmaxf(m, wred[w]);
        const float s = m / 127.f + 1e-8f;
        s_scale[0] = s;
        reinterpret_cast<__half*>(rec + kCompactKScaleOff)[row] = __float2half_rn(s);
    }
    __syncthreads();
    {
        const float s = s_scale[0];
        const float u = fminf(fmaxf(kx / s, -127.f), 127.f);
        const int chunk = (tid >> 4) ^ ((row & 1) << 2);
        reinterpret_cast<signed char*>(rec)[row * 256 + chunk * 16 + (tid & 15)] =
            static_cast<signed char>(__float2int_rn(u));
    }
    __syncthreads();

    // ---------------- V: signs, Walsh-Hadamard, RMS scale, 3-bit codes ----------------
    float v = a.rows_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.v_rows)[src + tid])
                          : static_cast<const float*>(a.v_rows)[src + tid];
    if (a.wht_len == 256 && a.signs) v = v * a.signs[tid];
    v = wht32_in_warp(v, lane);
    xs[tid] = v;
    __syncthreads();
    for (int s = 32; s < a.wht_len; s <<= 1) {
        const int j = tid ^ s;
        const float x0 = xs[tid], x1 = xs[j];
        __syncthreads();
        xs[tid] = (tid < j) ? (x0 + x1) : (x1 - x0);
        __syncthreads();
    }
    v = xs[tid] * (a.wht_len == 128 ? 0.08838834764831845f : 0.0625f);
    float ss = __fmul_rn(v, v);
    for (int off = 16; off > 0; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
    if (lane == 0) wred[warp] = ss;
    __syncthreads();
    const int nblk = kHeadDim / a.wht_len;
    if (tid < nblk) {
        const int w0 = tid * (a.wht_len / 32);
        float tot = wred[w0];
        for (int w = 1; w < a.wht_len / 32; ++w) tot = __fadd_rn(tot, wred[w0 + w]);
        const float rms = __fadd_rn(sqrtf(tot / float(a.wht_len)), 1e-8f);
        s_scale[tid] = rms;
        __half* vs = reinterpret_cast<__half*>(rec + kCompactVScaleOff) + row * 2;
        const __half hs = __float2half_rn(rms);
        if (nblk == 2) vs[tid] = hs;
        else vs[0] = vs[1] = hs;
    }
    __syncthreads();
    s_idx[tid] = static_cast<unsigned char>(tq3_code(v / s_scale[tid / a.wht_len]));
    __syncthreads();
    // pack: thread (g, j) owns dims 64j + 8g .. +7 = 4 fields = 48 bits of this token's parity
    if (tid < 32) {
        const int g = tid & 7, j = tid >> 3;
        const int e = row & 1;
        unsigned long long bits = 0, mask = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int d = 64 * j + 8 * g + 2 * i;
            const unsigned long long f = (unsigned long long)(s_idx[d]) << (3 * e) |
                                         (unsigned long long)(s_idx[d + 1]) << (6 + 3 * e);
            const unsigned long long m = (7ull << (3 * e)) | (7ull << (6 + 3 * e));
            bits |= f << (12 * i);
            mask |= m << (12 * i);
        }
        // The partner token of the pair may be written by another block of this launch: update
        // only this token's bits, with word atomics (the 48 bits span two aligned 32-bit words).
        const int o = compact_v_offset(row, g, j);
        const int sh = (o & 3) * 8;
        unsigned int* w = reinterpret_cast<unsigned int*>(rec + (o & ~3));
        const unsigned long long b64 = bits << sh, m64 = mask << sh;
        atomicAnd(w, ~static_cast<unsigned int>(m64));
        atomicOr(w, static_cast<unsigned int>(b64));
        atomicAnd(w + 1, ~static_cast<unsigned int>(m64 >> 32));
        atomicOr(w + 1, static_cast<unsigned int>(b64 >> 32));
    }
}

// Read tokens [0, n_tok) of one sequence back in the reference's packing
// (cuda_engine.cu:18305-18318): k_q int8 [n_tok][n_kv][256], k_sc fp16 [n_tok][n_kv],
// v_codes u8 [n_tok][n_kv][96] (8 indices LSB-first per 3 bytes, blocks in order),
// v_sc fp16 [n_tok][n_kv][nblk].  grid (n_tok, n_kv), 256 threads.
__global__ void __launch_bounds__(256)
kv_compact_gather_kernel(const unsigned char* pool, const int32_t* table, signed char* k_q, __half* k_sc,
                         unsigned char* v_codes, __half* v_sc, int n_tok, int n_kv, int n_pages, int wht_len,
                         int* err) {
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    __shared__ unsigned char s_idx[256];
    const int page = table[t / kPageTokens];
    if (page < 0 || page >= n_pages) {
        if (tid == 0) set_err(err, DEV_ERR_BAD_PAGE);
        return;
    }
    const int row64 = t % kPageTokens, half = row64 >> 5, row = row64 & 31;
    const unsigned char* rec = pool + ((size_t(page) * n_kv + h) * 2 + half) * kCompactRecordBytes;
    const size_t th = size_t(t) * n_kv + h;
    const int chunk = (tid >> 4) ^ ((row & 1) << 2);
    k_q[th * 256 + tid] = reinterpret_cast<const signed char*>(rec)[row * 256 + chunk * 16 + (tid & 15)];
    const int nblk = kHeadDim / wht_len;
    if (tid == 0) k_sc[th] = reinterpret_cast<const __half*>(rec + kCompactKScaleOff)[row];
    if (tid < nblk) v_sc[th * nblk + tid] = reinterpret_cast<const __half*>(rec + kCompactVScaleOff)[row * 2 + tid];
    {
        const int d = tid;
        const int j = d >> 6, g = (d >> 3) & 7, i = (d >> 1) & 3, odd_dim = d & 1, e = row & 1;
        const unsigned char* p = rec + compact_v_offset(row, g, j);
        unsigned long long w48 = 0;
        for (int x = 0; x < 6; ++x) w48 |= (unsigned long long)p[x] << (8 * x);
        s_idx[d] = static_cast<unsigned char>((w48 >> (12 * i + 6 * odd_dim + 3 * e)) & 7ull);
    }
    __syncthreads();
    if (tid < 32) {
        unsigned int w = 0;
        for (int x = 0; x < 8; ++x) w |= (unsigned int)(s_idx[tid * 8 + x]) << (3 * x);
        unsigned char* dst = v_codes + th * 96 + tid * 3;
        dst[0] = (unsigned char)w;
        dst[1] = (unsigned char)(w >> 8);
        dst[2] = (unsigned char)(w >> 16);
    }
}

// Dequantise tokens [src_pos0, src_pos0 + n_tok) of one sequence into paged F16 pools at
// positions dst_pos0 .. : what the reference does when it rebuilds its F16 compute window from
// the compact cache (dequant_k_q8_k / dequant_v_tq3_256, src/kernels/cuda/cuda_engine.cu:
// 8286-8314, 293-299) so that prefill chunks and verify rows can attend over it.
// K = half2float(scale) * int8; V = inverse transform of centroid[code] * half2float(scale)
// (the orthonormal Walsh-Hadamard transform is its own inverse), times the signs for the
// 256-point layout; both rounded to fp16 (RNE) into the tile-swizzled page format.
// grid (n_tok, n_kv), 256 threads: thread = dim.
__global__ void __launch_bounds__(256)
kv_compact_to_f16_kernel(const unsigned char* pool, const int32_t* src_table, int src_pos0, int n_src_pages,
                         __half* k_pool, __half* v_pool, const int32_t* dst_table, int dst_pos0, int n_dst_pages,
                         int n_kv, int wht_len, const float* signs, int* err) {
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    __shared__ float xs[256];
    const int sp = src_pos0 + t, dp = dst_pos0 + t;
    const int spage = src_table[sp / kPageTokens], dpage = dst_table[dp / kPageTokens];
    if (spage < 0 || spage >= n_src_pages || dpage < 0 || dpage >= n_dst_pages) {
        if (tid == 0) set_err(err, DEV_ERR_BAD_PAGE);
        return;
    }
    const int row64 = sp % kPageTokens, half = row64 >> 5, row = row64 & 31;
    const unsigned char* rec = pool + ((size_t(spage) * n_kv + h) * 2 + half) * kCompactRecordBytes;
    const size_t dst = (size_t(dpage) * n_kv + h) * kv_slice_elems() + kv_slice_offset(dp % kPageTokens, tid);
    // K
    {
        const int chunk = (tid >> 4) ^ ((row & 1) << 2);
        const float q = float(reinterpret_cast<const signed char*>(rec)[row * 256 + chunk * 16 + (tid & 15)]);
        const float s = __half2float(reinterpret_cast<const __half*>(rec + kCompactKScaleOff)[row]);
        k_pool[dst] = __float2half_rn(s * q);
    }
    // V
    const int d = tid;
    const int j = d >> 6, g = (d >> 3) & 7, i = (d >> 1) & 3, odd_dim = d & 1, e = row & 1;
    const unsigned char* p = rec + compact_v_offset(row, g, j);
    unsigned long long w48 = 0;
    for (int x = 0; x < 6; ++x) w48 |= (unsigned long long)p[x] << (8 * x);
    const int idx = int((w48 >> (12 * i + 6 * odd_dim + 3 * e)) & 7ull);
    const float sc = __half2float(reinterpret_cast<const __half*>(rec + kCompactVScaleOff)[row * 2 + d / wht_len]);
    float v = kTq3Levels[idx] * sc;
    v = wht32_in_warp(v, lane);
    xs[tid] = v;
    __syncthreads();
    for (int s = 32; s < wht_len; s <<= 1) {
        const int jj = tid ^ s;
        const float x0 = xs[tid], x1 = xs[jj];
        __syncthreads();
        xs[tid] = (tid < jj) ? (x0 + x1) : (x1 - x0);
        __syncthreads();
    }
    v = xs[tid] * (wht_len == 128 ? 0.08838834764831845f : 0.0625f);
    if (wht_len == 256 && signs) v *= signs[tid];
    v_pool[dst] = __float2half_rn(v);
}

}  // namespace rl
