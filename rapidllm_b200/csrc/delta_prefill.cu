// Chunked (WY-form) Gated DeltaNet prefill on tcgen05 / TMEM (sm_100a).
//
// The reference has only the token-by-token recurrence (ops::delta_recurrent_step,
// src/kernels/ops.cpp:495-540, driven per token by Session::layer_delta, src/runtime/
// session.cpp:232-248; CUDA gdn_prefill_split2_k, src/kernels/cuda/cuda_engine.cu:
// 4911-4974); DeltaChunkParams is declared but unused (include/rapidllm/backend/params.h:21).
// This file derives the chunked form from that recurrence.  Per value head, with S [dk][dv],
// k^ = l2norm(k), q^ = l2norm(q)/sqrt(dk), decay g_t = exp(glog_t), for a chunk of C = 64
// tokens with G_t = sum_{i<=t} glog_i (so prod g = exp(G)):
//   S_t = exp(G_t) S_0 + sum_{i<=t} exp(G_t - G_i) k^_i d_i^T
//   d_t = beta_t (v_t - exp(G_t) S_0^T k^_t - sum_{i<t} exp(G_t - G_i) (k^_i . k^_t) d_i)
// i.e. (I + A) D = diag(beta) (V - diag(exp G) K S_0) with the strictly lower triangular
// A_ti = beta_t exp(G_t - G_i) (k^_t . k^_i).  With T = (I + A)^-1 diag(beta):
//   D   = T V - W S_0,            W  = T diag(exp G) K
//   O   = Qg S_0 + P D,           Qg = diag(exp G) Q,  P_ti = exp(G_t - G_i) (q^_t . k^_i), i <= t
//   S_C = exp(G_C) S_0 + Kt^T D,  Kt = diag(exp(G_C - G)) K
// (the diagonal of P is included because the reference reads o_t from the updated state).
//
// Kernel 0 (delta_chunk_keys_kernel) computes, per (chunk, key head), what the value heads of a key
// head share: k^, q^ and their dot products.
// Kernel 1 (delta_chunk_prepare_kernel) computes everything else that does not depend on S for
// all (chunk, value head) pairs in parallel, one CTA each: W, Kt (each as an fp16 high part and
// an fp16 residual, ~22 bits together), Qg, P (fp16) as tiles already in the 128-byte-swizzled
// operand format of the tensor cores, and the product T V in fp32; 120 KiB per pair.
// Kernel 2 (delta_chunk_scan_kernel), one CTA per value head, walks the chunks in order.
// Everything is transposed so that the 128 value dims are the MMA M dimension (TMEM lanes):
// S^T lives in tensor memory in fp32 for the whole sequence, and its fp16 high and low
// parts are the tensor-memory A operands of -S^T W^T and O^T = S^T Qg^T + D^T P^T;
// D^T = (T V)^T - S^T W^T is formed by the worker threads (fp32 T V from shared memory plus
// the accumulator) and, again as hi + lo, is the A operand of S^T += D^T Kt.  Every product
// that feeds the state (S W^T, D Kt) runs as hi*hi + lo*hi + hi*lo, so the state keeps fp32
// accuracy; the two that only feed the output (S Qg^T, D P^T) use a single fp16 B operand.
// The tiles of a chunk arrive by three linear TMA bulk copies into three buffers, one per stage
// of the chunk's work (before D, for D, after D; the first is double), each refilled for the next
// chunk as soon as the products that read it have completed.
#include "common.cuh"
#include "kernels.h"
#include "tcgen05.cuh"

namespace rl {

namespace {

constexpr int kC = 64;                    // chunk length
constexpr int kD = 128;                   // dk = dv
constexpr int kTileWide = kC * kD * 2;    // 16 KiB: 64 x 128 fp16
constexpr int kTileSq = kC * kC * 2;      // 8 KiB: 64 x 64 fp16
// record of one (chunk, head): three parts, one per ring of the scan kernel
//   part A (needed first):  W hi, W lo, Qg                 48 KiB
//   part B (for D):         T V, fp32 [64 tokens][128]     32 KiB
//   part C (after D):       P, Kt hi, Kt lo                40 KiB
constexpr int kOffW = 0, kOffWlo = kTileWide, kOffQg = 2 * kTileWide;
constexpr int kPartABytes = 3 * kTileWide;
constexpr int kOffTV = kPartABytes;
constexpr int kPartBBytes = kC * kD * 4;
constexpr int kOffPartC = kOffTV + kPartBBytes;
constexpr int kOffP = 0, kOffKt = kTileSq, kOffKtlo = kTileSq + kTileWide;      // inside part C
constexpr int kPartCBytes = kTileSq + 2 * kTileWide;
constexpr int kRecordBytes = kPartABytes + kPartBBytes + kPartCBytes;            // 122880

// byte offset of element (row, x) in a swizzled tile whose rows are 64-element (128-byte) atoms
__device__ __forceinline__ int tile_off(int row, int x) {
    return (x >> 6) * (kC * 128) + row * 128 + ((((x & 63) >> 3) ^ (row & 7)) << 4) + (x & 7) * 2;
}

constexpr int kPrepThreads = 256;
constexpr int kPad = kD + 4;                // row stride = 4 (mod 32) floats: the MMA fragment loads spread over the banks
constexpr int kSq = kC + 4;                 // same for the 64 x 64 arrays
constexpr int kB = 16;                    // block size of the triangular inverse

// fp32 -> tf32 high part and tf32 residual: a x b ~= ah bh + ah bl + al bh to fp32 accuracy
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(x - __uint_as_float(hi)));
}
// warp MMA m16n8k8, tf32 inputs, fp32 accumulate.  A row-major 16 x 8: a0 (g, c), a1 (g+8, c), a2 (g, c+4),
// a3 (g+8, c+4); B 8 x 8: b0 (k = c, n = g), b1 (k = c+4, n = g); D: d0 (g, 2c), d1 (g, 2c+1), d2 (g+8, 2c),
// d3 (g+8, 2c+1), with g = lane / 4, c = lane % 4.
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// One 16 x 8 output tile of a small product on the tensor cores with fp32 accuracy (3 x TF32):
// d += A[16][K] B[K][8], a_at(row, k) and b_at(k, col) give the elements (row, col inside the tile);
// g = lane / 4, c = lane % 4; d follows the accumulator layout of mma_tf32.
template <int K, class FA, class FB>
__device__ __forceinline__ void tile_mma3(float (&d)[4], FA a_at, FB b_at, int g, int c) {
#pragma unroll
    for (int k0 = 0; k0 < K; k0 += 8) {
        uint32_t ah[4], al[4], bh[2], bl[2];
        split_tf32(a_at(g, k0 + c), ah[0], al[0]);
        split_tf32(a_at(g + 8, k0 + c), ah[1], al[1]);
        split_tf32(a_at(g, k0 + c + 4), ah[2], al[2]);
        split_tf32(a_at(g + 8, k0 + c + 4), ah[3], al[3]);
        split_tf32(b_at(k0 + c, g), bh[0], bl[0]);
        split_tf32(b_at(k0 + c + 4, g), bh[1], bl[1]);
        mma_tf32(d, al, bh);
        mma_tf32(d, ah, bl);
        mma_tf32(d, ah, bh);
    }
}

struct PrepSmem {
    float kn[kC][kPad];       // k^
    union {
        float qn[kC][kPad];   // q^, dead once q^.k^ and the Qg tile are out
        struct {
            float m[kC][kSq];         // (I + A)^-1
            float tmp[kC][kSq];
        } inv;
    } u;
    union {
        struct {
            float l[kC][kSq];     // k^_t . k^_i, then in place A (strictly lower part of I + A)
            float qk[kC][kSq];    // q^_t . k^_i
        } d;
        float v[kC][kPad];        // the chunk's value rows in fp32, once l and qk are no longer needed
    } w;
    float G[kC], beta[kC], eg[kC];
    uint64_t bar;             // the key head's record has landed
};
// the struct from its start to the end of qk, padding included, is what the key head's pass hands to its
// value heads (k^, q^, a gap where the union is larger than q^, k^.k^, q^.k^)
constexpr int kKeysBytes = (kC * kPad + 2 * kC * kSq + 2 * kC * kSq) * 4;     // 103 424
static_assert(offsetof(PrepSmem, w) + 2 * kC * kSq * 4 == kKeysBytes && kKeysBytes % 64 == 0,
              "k^, q^, k^.k^, q^.k^ lie at the start of PrepSmem");

// fp32 -> (fp16 high part, fp16 residual), two values per register
__device__ __forceinline__ void split_h2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    const __half2 hh = __halves2half2(h0, h1);
    hi = *reinterpret_cast<const uint32_t*>(&hh);
    lo = pack_h2(x0 - __half2float(h0), x1 - __half2float(h1));
}

}  // namespace

size_t delta_chunk_record_bytes() { return kRecordBytes; }

// What a chunk's value heads share: per (chunk, key head) the normalised keys and queries and their
// dot products.  Record: k^ [64][132], q^ [64][132], k^.k^ [64][68], q^.k^ [64][68], fp32 -- laid out
// exactly as in shared memory (PrepSmem), so that a value head's CTA fetches the record with bulk copies.
constexpr int kKeysFloats = kKeysBytes / 4;

// grid (n_chunks, n_qk), 256 threads: l2 norms and the two 64 x 64 x 128 products once per key head
// (the value heads that share it, 3 in qwen3_5, read the result instead of recomputing it).
__global__ void __launch_bounds__(kPrepThreads, 2) delta_chunk_keys_kernel(DeltaChunkArgs a) {
    extern __shared__ unsigned char smem_raw[];
    PrepSmem& s = *reinterpret_cast<PrepSmem*>(smem_raw);
    griddep_launch();
    griddep_wait();
    const int chunk = a.chunk0 + blockIdx.x, hs = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = chunk * kC;
    const int n_tok = min(kC, a.T - t0);
    float* rec = a.keys + (size_t(chunk) * a.n_qk + hs) * kKeysFloats;
    // ---- l2 norms (double accumulators as ops::l2norm); padded tokens are all zero.  A warp owns
    // 8 tokens; all 16 row loads are issued before the first reduction so their latencies overlap ----
    {
        constexpr int kPer = kC / (kPrepThreads / 32);
        float4 kx[kPer], qx[kPer];
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int t = warp + u * (kPrepThreads / 32);
            kx[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            qx[u] = kx[u];
            if (t < n_tok) {
                kx[u] = *reinterpret_cast<const float4*>(a.k + size_t(t0 + t) * a.qk_tok_stride + size_t(hs) * kD + lane * 4);
                qx[u] = *reinterpret_cast<const float4*>(a.q + size_t(t0 + t) * a.qk_tok_stride + size_t(hs) * kD + lane * 4);
            }
        }
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int t = warp + u * (kPrepThreads / 32);
            double ks = double(kx[u].x) * kx[u].x + double(kx[u].y) * kx[u].y + double(kx[u].z) * kx[u].z + double(kx[u].w) * kx[u].w;
            double qs = double(qx[u].x) * qx[u].x + double(qx[u].y) * qx[u].y + double(qx[u].z) * qx[u].z + double(qx[u].w) * qx[u].w;
            for (int off = 16; off > 0; off >>= 1) {
                ks += __shfl_xor_sync(0xffffffffu, ks, off);
                qs += __shfl_xor_sync(0xffffffffu, qs, off);
            }
            float ki = 1.f / sqrtf(float(ks) + a.eps_l2);
            float qi = 1.f / sqrtf(float(qs) + a.eps_l2) * (1.f / sqrtf(float(kD)));
            if (t >= n_tok) ki = qi = 0.f;
            s.kn[t][lane * 4 + 0] = kx[u].x * ki; s.kn[t][lane * 4 + 1] = kx[u].y * ki;
            s.kn[t][lane * 4 + 2] = kx[u].z * ki; s.kn[t][lane * 4 + 3] = kx[u].w * ki;
            s.u.qn[t][lane * 4 + 0] = qx[u].x * qi; s.u.qn[t][lane * 4 + 1] = qx[u].y * qi;
            s.u.qn[t][lane * 4 + 2] = qx[u].z * qi; s.u.qn[t][lane * 4 + 3] = qx[u].w * qi;
        }
    }
    __syncthreads();
    // ---- k^.k^ and q^.k^ on the tensor cores (3 x TF32 = fp32 accuracy).  Only the 8-column tiles that
    // touch the lower triangle are computed: 2, 4, 6, 8 of them for the four 16-row blocks.  Warp -> (row
    // block, first tile, tiles): at most three tiles each; the rest of l and qk is zero-filled first (nobody
    // reads more than their zero) ----
    for (int idx = tid; idx < kC * kC / 4; idx += kPrepThreads) {
        const int t = idx >> 4, i = (idx & 15) * 4;
        if (i >= (t & ~15) + 16) {
            *reinterpret_cast<float4*>(&s.w.d.l[t][i]) = make_float4(0.f, 0.f, 0.f, 0.f);
            *reinterpret_cast<float4*>(&s.w.d.qk[t][i]) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
    {
        const int g = lane >> 2, c = lane & 3;
        // warps 0..7 -> row blocks 0, 1, 1, 2, 2, 3, 3, 3; first tiles 0, 0, 2, 0, 3, 0, 3, 6; tiles 2, 2, 2, 3, 3, 3, 3, 2
        const int rb = (0x33322110u >> (4 * warp)) & 15, tile0 = (0x63030200u >> (4 * warp)) & 15;
        const int n_tiles = (0x23333222u >> (4 * warp)) & 15;
        const int t_base = rb * 16, i_base = tile0 * 8;
        float ck[3][4] = {}, cq[3][4] = {};
        for (int k0 = 0; k0 < kD; k0 += 8) {
            uint32_t akh[4], akl[4], aqh[4], aql[4];
            split_tf32(s.kn[t_base + g][k0 + c], akh[0], akl[0]);
            split_tf32(s.kn[t_base + g + 8][k0 + c], akh[1], akl[1]);
            split_tf32(s.kn[t_base + g][k0 + c + 4], akh[2], akl[2]);
            split_tf32(s.kn[t_base + g + 8][k0 + c + 4], akh[3], akl[3]);
            split_tf32(s.u.qn[t_base + g][k0 + c], aqh[0], aql[0]);
            split_tf32(s.u.qn[t_base + g + 8][k0 + c], aqh[1], aql[1]);
            split_tf32(s.u.qn[t_base + g][k0 + c + 4], aqh[2], aql[2]);
            split_tf32(s.u.qn[t_base + g + 8][k0 + c + 4], aqh[3], aql[3]);
            // B fragments of all column tiles first, then the three TF32 passes with the accumulators
            // interleaved: consecutive MMAs never depend on each other
            uint32_t bh[3][2], bl[3][2];
#pragma unroll
            for (int nt = 0; nt < 3; ++nt) {
                if (nt < n_tiles) {
                    split_tf32(s.kn[i_base + 8 * nt + g][k0 + c], bh[nt][0], bl[nt][0]);
                    split_tf32(s.kn[i_base + 8 * nt + g][k0 + c + 4], bh[nt][1], bl[nt][1]);
                }
            }
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
#pragma unroll
                for (int nt = 0; nt < 3; ++nt) {
                    if (nt < n_tiles) {
                        mma_tf32(ck[nt], pass == 0 ? akl : akh, pass == 1 ? bl[nt] : bh[nt]);
                        mma_tf32(cq[nt], pass == 0 ? aql : aqh, pass == 1 ? bl[nt] : bh[nt]);
                    }
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 3; ++nt) {
            if (nt < n_tiles) {
                const int i0 = i_base + 8 * nt + 2 * c;
                s.w.d.l[t_base + g][i0] = ck[nt][0];      s.w.d.l[t_base + g][i0 + 1] = ck[nt][1];
                s.w.d.l[t_base + g + 8][i0] = ck[nt][2];  s.w.d.l[t_base + g + 8][i0 + 1] = ck[nt][3];
                s.w.d.qk[t_base + g][i0] = cq[nt][0];     s.w.d.qk[t_base + g][i0 + 1] = cq[nt][1];
                s.w.d.qk[t_base + g + 8][i0] = cq[nt][2]; s.w.d.qk[t_base + g + 8][i0 + 1] = cq[nt][3];
            }
        }
    }
    __syncthreads();
    // the four arrays out as they lie (the padding columns carry whatever shared memory held; nobody reads them)
    const float4* src = reinterpret_cast<const float4*>(smem_raw);
    for (int idx = tid; idx < kKeysBytes / 16; idx += kPrepThreads) reinterpret_cast<float4*>(rec)[idx] = src[idx];
}

// grid (n_chunks, n_v), 256 threads: one CTA per chunk and value head.  103 KB of shared memory, so
// two CTAs share an SM and hide each other's barriers.
__global__ void __launch_bounds__(kPrepThreads, 2) delta_chunk_prepare_kernel(DeltaChunkArgs a) {
    extern __shared__ unsigned char smem_raw[];
    PrepSmem& s = *reinterpret_cast<PrepSmem*>(smem_raw);
    const int chunk = a.chunk0 + blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int rep = a.head_map == 0 ? 1 : a.n_v / a.n_qk;
    const int hs = a.head_map == 0 ? h : (a.head_map == 1 ? h / rep : h % a.n_qk);
    const int t0 = chunk * kC;
    const int n_tok = min(kC, a.T - t0);
    unsigned char* rec = a.work + (size_t(chunk) * a.n_v + h) * kRecordBytes;
    griddep_launch();
    griddep_wait();

    // ---- what the key head's pass left (k^, q^, k^.k^, q^.k^) comes in by bulk copies beside the gates ----
    if (tid == 0) {
        mbar_init(&s.bar, 1);
        mbar_fence_init();
        mbar_arrive_expect_tx(&s.bar, kKeysBytes);
        const unsigned char* keys = reinterpret_cast<const unsigned char*>(a.keys + (size_t(chunk) * a.n_qk + hs) * kKeysFloats);
        constexpr int kPiece = kKeysBytes / 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) bulk_g2s(smem_raw + i * kPiece, keys + i * kPiece, kPiece, &s.bar);
    }
    // ---- cumulative log decay, beta (needed by every tile) ----
    if (tid < kC) {
        const bool live = tid < n_tok;
        s.beta[tid] = live ? a.beta[size_t(t0 + tid) * a.n_v + h] : 0.f;
        float gl = live ? a.g_log[size_t(t0 + tid) * a.n_v + h] : 0.f;
        // inclusive scan over 64 values held by two warps
        for (int off = 1; off < 32; off <<= 1) {
            const float o = __shfl_up_sync(0xffffffffu, gl, off);
            if (lane >= off) gl += o;
        }
        s.G[tid] = gl;
    }
    __syncthreads();
    if (tid >= 32 && tid < kC) s.G[tid] += s.G[31];
    if (!mbar_wait(&s.bar, 0)) {
        set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
        return;
    }
    __syncthreads();
    if (tid < kC) s.eg[tid] = expf(s.G[tid]);
    if (tid == 0) a.chunk_decay[size_t(chunk) * a.n_v + h] = expf(s.G[kC - 1]);
    __syncthreads();
    // ---- tiles that need q^: Qg (fp16); with it Kt as fp16 hi + lo (64 x 128, swizzled) ----
    const float gC = s.G[kC - 1];
    {
        constexpr int kPer = kC * kD / 4 / kPrepThreads;      // 8 groups of 4 dims per thread
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int idx = tid + u * kPrepThreads;
            const int t = idx >> 5, d = (idx & 31) * 4;
            const int o = tile_off(t, d);
            const float e = s.eg[t];
            *reinterpret_cast<uint2*>(rec + kOffQg + o) =
                make_uint2(pack_h2(e * s.u.qn[t][d], e * s.u.qn[t][d + 1]), pack_h2(e * s.u.qn[t][d + 2], e * s.u.qn[t][d + 3]));
            const float kt = expf(gC - s.G[t]);
            uint32_t h0, l0, h1, l1;
            split_h2(kt * s.kn[t][d], kt * s.kn[t][d + 1], h0, l0);
            split_h2(kt * s.kn[t][d + 2], kt * s.kn[t][d + 3], h1, l1);
            *reinterpret_cast<uint2*>(rec + kOffPartC + kOffKt + o) = make_uint2(h0, h1);
            *reinterpret_cast<uint2*>(rec + kOffPartC + kOffKtlo + o) = make_uint2(l0, l1);
        }
    }
    __syncthreads();                                  // q^ is dead from here on: its space becomes m and tmp
    float (*m)[kSq] = s.u.inv.m;
    float (*tmp)[kSq] = s.u.inv.tmp;
    // ---- A_ti = beta_t exp(G_t - G_i) (k^_t . k^_i), i < t, in place (four columns per thread and pass) ----
    for (int idx = tid; idx < kC * kC / 4; idx += kPrepThreads) {
        const int t = idx >> 4, i = (idx & 15) * 4;
        const float4 kk = *reinterpret_cast<const float4*>(&s.w.d.l[t][i]);
        const float4 gi = *reinterpret_cast<const float4*>(&s.G[i]);
        const float gt = s.G[t], bt = s.beta[t];
        float4 av;
        av.x = i < t ? bt * expf(gt - gi.x) * kk.x : 0.f;
        av.y = i + 1 < t ? bt * expf(gt - gi.y) * kk.y : 0.f;
        av.z = i + 2 < t ? bt * expf(gt - gi.z) * kk.z : 0.f;
        av.w = i + 3 < t ? bt * expf(gt - gi.w) * kk.w : 0.f;
        *reinterpret_cast<float4*>(&s.w.d.l[t][i]) = av;
        *reinterpret_cast<float4*>(&m[t][i]) = make_float4(t == i ? 1.f : 0.f, t == i + 1 ? 1.f : 0.f, t == i + 2 ? 1.f : 0.f,
                                                           t == i + 3 ? 1.f : 0.f);
    }
    __syncthreads();
    // ---- M = (I + A)^-1 on the tensor cores (3 x TF32 = fp32 accuracy), a dozen barriers ----
    // Every product is cut into 16 x 8 output tiles, one per warp (tile_mma3).
    {
        const int g = lane >> 2, c = lane & 3;
        float (*L)[kSq] = s.w.d.l;
        auto ld_tile = [&](const float (*X)[kSq], int r0, int n0, float (&d)[4]) {
            const float2 lo = *reinterpret_cast<const float2*>(&X[r0 + g][n0 + 2 * c]);
            const float2 hi = *reinterpret_cast<const float2*>(&X[r0 + g + 8][n0 + 2 * c]);
            d[0] = lo.x; d[1] = lo.y; d[2] = hi.x; d[3] = hi.y;
        };
        auto st_tile = [&](float (*X)[kSq], int r0, int n0, const float (&d)[4]) {
            *reinterpret_cast<float2*>(&X[r0 + g][n0 + 2 * c]) = make_float2(d[0], d[1]);
            *reinterpret_cast<float2*>(&X[r0 + g + 8][n0 + 2 * c]) = make_float2(d[2], d[3]);
        };
        // (1) the four 16 x 16 diagonal blocks: N = strictly lower part is nilpotent (N^16 = 0), so
        //     (I + N)^-1 = (I - N)(I + N^2)(I + N^4)(I + N^8): six products per block, block = warp / 2,
        //     the warp's tile = 8 of its 16 columns.
        {
            const int bb = (warp >> 1) * kB, nb = bb + (warp & 1) * 8;
            float d[4];
            // tmp = N^2
            d[0] = d[1] = d[2] = d[3] = 0.f;
            tile_mma3<kB>(d, [&](int r, int k) { return L[bb + r][bb + k]; }, [&](int k, int n) { return L[bb + k][nb + n]; }, g, c);
            st_tile(tmp, bb, nb, d);
            __syncthreads();
            // m = (I - N) + (I - N) N^2
            ld_tile(L, bb, nb, d);
            d[0] = (bb + g == nb + 2 * c ? 1.f : 0.f) - d[0];
            d[1] = (bb + g == nb + 2 * c + 1 ? 1.f : 0.f) - d[1];
            d[2] = (bb + g + 8 == nb + 2 * c ? 1.f : 0.f) - d[2];
            d[3] = (bb + g + 8 == nb + 2 * c + 1 ? 1.f : 0.f) - d[3];
            tile_mma3<kB>(d, [&](int r, int k) { return (r == k ? 1.f : 0.f) - L[bb + r][bb + k]; },
                          [&](int k, int n) { return tmp[bb + k][nb + n]; }, g, c);
            st_tile(m, bb, nb, d);
            __syncthreads();
            // l = N^4
            d[0] = d[1] = d[2] = d[3] = 0.f;
            tile_mma3<kB>(d, [&](int r, int k) { return tmp[bb + r][bb + k]; }, [&](int k, int n) { return tmp[bb + k][nb + n]; }, g, c);
            st_tile(L, bb, nb, d);
            __syncthreads();
            // tmp = m + m N^4
            ld_tile(m, bb, nb, d);
            tile_mma3<kB>(d, [&](int r, int k) { return m[bb + r][bb + k]; }, [&](int k, int n) { return L[bb + k][nb + n]; }, g, c);
            st_tile(tmp, bb, nb, d);
            __syncthreads();
            // m = N^8
            d[0] = d[1] = d[2] = d[3] = 0.f;
            tile_mma3<kB>(d, [&](int r, int k) { return L[bb + r][bb + k]; }, [&](int k, int n) { return L[bb + k][nb + n]; }, g, c);
            st_tile(m, bb, nb, d);
            __syncthreads();
            // m = tmp + tmp N^8: the inverse of the block (kept in registers until every warp has read m)
            ld_tile(tmp, bb, nb, d);
            tile_mma3<kB>(d, [&](int r, int k) { return tmp[bb + r][bb + k]; }, [&](int k, int n) { return m[bb + k][nb + n]; }, g, c);
            __syncthreads();
            st_tile(m, bb, nb, d);
            __syncthreads();
        }
        // (2) off-diagonal blocks from inv [[P, 0], [C, Q]] = [[P^-1, 0], [-Q^-1 C P^-1, Q^-1]], first
        //     for the two 32 x 32 halves (C = a 16 x 16 block of A; four tiles, warps 0-3), then for the whole
        //     (C = 32 x 32; eight tiles)
        {
            const int u = warp >> 1, bi = (2 * u + 1) * kB, bj = 2 * u * kB, nb = bj + (warp & 1) * 8;
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            if (warp < 4) {
                tile_mma3<kB>(d, [&](int r, int k) { return L[bi + r][bj + k]; }, [&](int k, int n) { return m[bj + k][nb + n]; }, g, c);
                st_tile(tmp, bi, nb, d);
            }
            __syncthreads();
            if (warp < 4) {
                d[0] = d[1] = d[2] = d[3] = 0.f;
                tile_mma3<kB>(d, [&](int r, int k) { return m[bi + r][bi + k]; }, [&](int k, int n) { return tmp[bi + k][nb + n]; }, g, c);
                d[0] = -d[0]; d[1] = -d[1]; d[2] = -d[2]; d[3] = -d[3];
                st_tile(m, bi, nb, d);
            }
            __syncthreads();
        }
        {
            const int r0 = 32 + (warp >> 2) * 16, n0 = (warp & 3) * 8;
            float d[4] = {0.f, 0.f, 0.f, 0.f};
            tile_mma3<32>(d, [&](int r, int k) { return L[r0 + r][k]; }, [&](int k, int n) { return m[k][n0 + n]; }, g, c);
            st_tile(tmp, r0, n0, d);
            __syncthreads();
            d[0] = d[1] = d[2] = d[3] = 0.f;
            tile_mma3<32>(d, [&](int r, int k) { return m[r0 + r][32 + k]; }, [&](int k, int n) { return tmp[32 + k][n0 + n]; }, g, c);
            d[0] = -d[0]; d[1] = -d[1]; d[2] = -d[2]; d[3] = -d[3];
            st_tile(m, r0, n0, d);
            __syncthreads();
        }
    }
    // ---- tile P (64 x 64, fp16, swizzled), four columns per thread and pass ----
    for (int idx = tid; idx < kC * kC / 4; idx += kPrepThreads) {
        const int t = idx >> 4, i = (idx & 15) * 4;
        const float4 qk = *reinterpret_cast<const float4*>(&s.w.d.qk[t][i]);
        const float4 gi = *reinterpret_cast<const float4*>(&s.G[i]);
        const float gt = s.G[t];
        const float p0 = i <= t ? expf(gt - gi.x) * qk.x : 0.f;
        const float p1 = i + 1 <= t ? expf(gt - gi.y) * qk.y : 0.f;
        const float p2 = i + 2 <= t ? expf(gt - gi.z) * qk.z : 0.f;
        const float p3 = i + 3 <= t ? expf(gt - gi.w) * qk.w : 0.f;
        *reinterpret_cast<uint2*>(rec + kOffPartC + kOffP + tile_off(t, i)) = make_uint2(pack_h2(p0, p1), pack_h2(p2, p3));
    }
    // T = M diag(beta) in place, and tmp[t][i] = T[t][i] exp(G_i) for W
    for (int idx = tid; idx < kC * kC / 4; idx += kPrepThreads) {
        const int t = idx >> 4, i = (idx & 15) * 4;
        const float4 mv = *reinterpret_cast<const float4*>(&m[t][i]);
        const float4 bv = *reinterpret_cast<const float4*>(&s.beta[i]);
        const float4 ev = *reinterpret_cast<const float4*>(&s.eg[i]);
        const float4 tv = make_float4(mv.x * bv.x, mv.y * bv.y, mv.z * bv.z, mv.w * bv.w);
        *reinterpret_cast<float4*>(&m[t][i]) = tv;
        *reinterpret_cast<float4*>(&tmp[t][i]) = make_float4(tv.x * ev.x, tv.y * ev.y, tv.z * ev.z, tv.w * ev.w);
    }
    __syncthreads();                                  // l and qk are dead: their space takes the value rows
    {
        constexpr int kPer = kC * kD / 4 / kPrepThreads;
        float4 vv[kPer];
#pragma unroll
        for (int u = 0; u < kPer; ++u) {                      // all value loads in flight together
            const int idx = tid + u * kPrepThreads;
            const int t = idx >> 5, d = (idx & 31) * 4;
            vv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t < n_tok) vv[u] = *reinterpret_cast<const float4*>(a.v + size_t(t0 + t) * a.v_tok_stride + size_t(h) * kD + d);
        }
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int idx = tid + u * kPrepThreads;
            const int t = idx >> 5, d = (idx & 31) * 4;
            *reinterpret_cast<float4*>(&s.w.v[t][d]) = vv[u];
        }
    }
    __syncthreads();
    // W[t][d] = sum_{i<=t} tmp[t][i] k^[i][d] and (T V)[t][d] = sum_{i<=t} T[t][i] v[i][d] (tmp and T are zero
    // above the diagonal), 3 x TF32 MMAs.  K steps beyond a row block's diagonal are skipped, so the four
    // 16-row blocks cost 2, 4, 6 and 8 steps: a warp takes blocks {0, 3} or {1, 2} (10 steps either way) of
    // one 32-dim column group.  W leaves as fp16 hi + lo tiles, T V as plain fp32 rows.
    {
        const int g = lane >> 2, c = lane & 3;
        const int d_base = (warp >> 1) * 32;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
            const float (*A)[kSq] = which == 0 ? tmp : m;
            const float (*B)[kPad] = which == 0 ? s.kn : s.w.v;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                const int t_base = (half == 0 ? (warp & 1) : 3 - (warp & 1)) * 16;
                float acc[4][4] = {};
                for (int k0 = 0; k0 < t_base + 16; k0 += 8) {
                    uint32_t ah[4], al[4];
                    split_tf32(A[t_base + g][k0 + c], ah[0], al[0]);
                    split_tf32(A[t_base + g + 8][k0 + c], ah[1], al[1]);
                    split_tf32(A[t_base + g][k0 + c + 4], ah[2], al[2]);
                    split_tf32(A[t_base + g + 8][k0 + c + 4], ah[3], al[3]);
                    uint32_t bh[4][2], bl[4][2];
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        split_tf32(B[k0 + c][d_base + 8 * nt + g], bh[nt][0], bl[nt][0]);
                        split_tf32(B[k0 + c + 4][d_base + 8 * nt + g], bh[nt][1], bl[nt][1]);
                    }
#pragma unroll
                    for (int pass = 0; pass < 3; ++pass)
#pragma unroll
                        for (int nt = 0; nt < 4; ++nt) mma_tf32(acc[nt], pass == 0 ? al : ah, pass == 1 ? bl[nt] : bh[nt]);
                }
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const int d0 = d_base + 8 * nt + 2 * c;
                    if (which == 0) {
                        uint32_t h0, l0, h1, l1;
                        split_h2(acc[nt][0], acc[nt][1], h0, l0);
                        split_h2(acc[nt][2], acc[nt][3], h1, l1);
                        *reinterpret_cast<uint32_t*>(rec + kOffW + tile_off(t_base + g, d0)) = h0;
                        *reinterpret_cast<uint32_t*>(rec + kOffWlo + tile_off(t_base + g, d0)) = l0;
                        *reinterpret_cast<uint32_t*>(rec + kOffW + tile_off(t_base + g + 8, d0)) = h1;
                        *reinterpret_cast<uint32_t*>(rec + kOffWlo + tile_off(t_base + g + 8, d0)) = l1;
                    } else {
                        float* tv = reinterpret_cast<float*>(rec + kOffTV);
                        *reinterpret_cast<float2*>(tv + (t_base + g) * kD + d0) = make_float2(acc[nt][0], acc[nt][1]);
                        *reinterpret_cast<float2*>(tv + (t_base + g + 8) * kD + d0) = make_float2(acc[nt][2], acc[nt][3]);
                    }
                }
            }
        }
    }
}

size_t delta_chunk_prepare_smem_bytes() { return sizeof(PrepSmem); }
size_t delta_chunk_keys_bytes() { return size_t(kKeysFloats) * sizeof(float); }
int delta_chunk_prepare_threads() { return kPrepThreads; }

// ================================================================================================
namespace {

constexpr int kScanWorkers = 256;         // 8 worker warps: TMEM lane = value dim, two warps per lane quadrant split the columns
constexpr int kScanOutput = 128;          // 4 output warps (one per lane quadrant) write o while the chain goes on
constexpr int kScanThreads = kScanWorkers + kScanOutput + 64;   // + loader warp + MMA warp
constexpr int kWarpScanOut0 = kScanWorkers / 32, kWarpScanLoader = (kScanWorkers + kScanOutput) / 32, kWarpScanMma = kWarpScanLoader + 1;
constexpr int kStagesA = 2, kStagesC = 1;
// tensor memory map (columns); lane = value dim
constexpr uint32_t kColSt = 0;            // S^T fp32, 128 columns (column = key dim)
constexpr uint32_t kColShi = 128;         // fp16 pairs: 64 columns
constexpr uint32_t kColSlo = 192;
constexpr uint32_t kColD = 256;           // -S^T W^T fp32, 64 columns (column = token)
constexpr uint32_t kColO = 320;           // O^T fp32, 64 columns
constexpr uint32_t kColDhi = 384;         // D^T as fp16 pairs: 32 columns
constexpr uint32_t kColDlo = 416;

struct ScanSmem {
    alignas(1024) unsigned char pa[kStagesA][kPartABytes];   // W hi, W lo, Qg
    alignas(1024) unsigned char pc[kStagesC][kPartCBytes];   // P, Kt hi, Kt lo
    alignas(1024) unsigned char pb[kPartBBytes];             // T V fp32
    alignas(16) float ostage[kC][kD];                        // O of a chunk, token-major, on its way out
    uint64_t full_a[kStagesA], empty_a[kStagesA], full_c[kStagesC], empty_c[kStagesC], full_b, empty_b;
    uint64_t bar_s[2];   // workers -> MMA: S hi/lo of the chunk are in tensor memory ([0]: key dims 0-31 and 64-95, [1]: the rest)
    uint64_t bar_w;      // MMA -> workers: -S^T W^T is complete
    uint64_t bar_d;      // workers -> MMA: D hi/lo are in tensor memory
    uint64_t bar_k;      // MMA -> workers: S^T += D^T Kt is complete
    uint64_t bar_o;      // MMA -> workers: O^T of the chunk is complete
    uint64_t bar_oread;  // workers -> MMA: O^T has been read out (its columns may be overwritten)
    uint32_t tmem_base;
    int failed;
};

}  // namespace

// grid (n_v), 448 threads.  o [T][n_v][128]; S [n_v][128][128] fp32 in place (row = key dim).  A launch
// walks chunks [chunk0, chunk0 + chunks): S is read at its start and written back at its end, so a
// sequence can be scanned in several launches while later chunks are still being prepared.
//
// The chain from one chunk's state to the next is: 24 MMAs (-S^T W^T) -> workers form D -> 12 MMAs
// (S^T += D^T Kt) -> workers split the new S^T.  The output products (S^T Qg^T before D is known,
// D^T P^T after the state update) are issued behind the chain's MMAs and read out by four output warps
// while the next chunk's first MMAs run.
__global__ void __launch_bounds__(kScanThreads, 1) delta_chunk_scan_kernel(DeltaChunkArgs a) {
    extern __shared__ unsigned char smem_raw[];
    ScanSmem& s = *reinterpret_cast<ScanSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int h = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_chunks = a.chunks;            // of this launch; c below counts from a.chunk0
    float* Sg = a.S + size_t(h) * kD * kD;

    if (tid == 0) {
        for (int i = 0; i < kStagesA; ++i) {
            mbar_init(&s.full_a[i], 1);
            mbar_init(&s.empty_a[i], 1);
        }
        for (int i = 0; i < kStagesC; ++i) {
            mbar_init(&s.full_c[i], 1);
            mbar_init(&s.empty_c[i], 1);
        }
        mbar_init(&s.full_b, 1);
        // the worker and output warps arrive once per warp (lane 0, behind a __syncwarp): 256 single arrivals on
        // one barrier word took ~600 clocks of every hand-over
        mbar_init(&s.empty_b, kScanWorkers / 32);
        mbar_init(&s.bar_s[0], kScanWorkers / 32);
        mbar_init(&s.bar_s[1], kScanWorkers / 32);
        mbar_init(&s.bar_w, 1);
        mbar_init(&s.bar_d, kScanWorkers / 32);
        mbar_init(&s.bar_k, 1);
        mbar_init(&s.bar_o, 1);
        mbar_init(&s.bar_oread, kScanOutput / 32);
        s.failed = 0;
        mbar_fence_init();
    }
    if (warp == kWarpScanMma) tc::tmem_alloc(&s.tmem_base, 512);
    griddep_launch();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    griddep_wait();       // barriers and tensor memory were set up beside the tail of the kernel in front
    const uint32_t tmem = s.tmem_base;

    if (warp == kWarpScanLoader) {
        // ------------------------------ loader ------------------------------
        if (lane == 0) {
            for (int c = 0; c < n_chunks; ++c) {
                const unsigned char* rec = a.work + (size_t(a.chunk0 + c) * a.n_v + h) * kRecordBytes;
                const int sa = c % kStagesA, sc = c % kStagesC;
                if (!mbar_wait(&s.empty_a[sa], ((c / kStagesA) & 1) ^ 1)) { s.failed = 1; break; }
                mbar_arrive_expect_tx(&s.full_a[sa], kPartABytes);
                bulk_g2s(s.pa[sa], rec, kPartABytes, &s.full_a[sa]);
                if (!mbar_wait(&s.empty_b, (c & 1) ^ 1)) { s.failed = 1; break; }
                mbar_arrive_expect_tx(&s.full_b, kPartBBytes);
                bulk_g2s(s.pb, rec + kOffTV, kPartBBytes, &s.full_b);
                if (!mbar_wait(&s.empty_c[sc], ((c / kStagesC) & 1) ^ 1)) { s.failed = 1; break; }
                mbar_arrive_expect_tx(&s.full_c[sc], kPartCBytes);
                bulk_g2s(s.pc[sc], rec + kOffPartC, kPartCBytes, &s.full_c[sc]);
            }
            if (s.failed) set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
        }
    } else if (warp == kWarpScanMma) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t id_n64 = tc::idesc_f16(128, kC, false, false);           // A from TMEM, B K-major
            constexpr uint32_t id_n64_neg = id_n64 | (1u << 13);                        // -A
            constexpr uint32_t id_n128 = tc::idesc_f16(128, kD, false, true);          // B = Kt MN-major
            bool ok = true;
            // Descriptors are built once per ring stage and advanced by constants (their address
            // field counts 16-byte units): the issuing thread must spend only a few instructions
            // per tcgen05.mma or it, not the tensor pipe, sets the pace.
            uint64_t a_desc[kStagesA], ck_desc[kStagesC], cmn_desc[kStagesC];
#pragma unroll
            for (int i = 0; i < kStagesA; ++i) a_desc[i] = tc::smem_desc(smem_u32(s.pa[i]), 16, 1024);        // W, Qg: K-major
#pragma unroll
            for (int i = 0; i < kStagesC; ++i) {
                ck_desc[i] = tc::smem_desc(smem_u32(s.pc[i]), 16, 1024);                                       // P: K-major
                cmn_desc[i] = tc::smem_desc(smem_u32(s.pc[i]), kC * 128, 1024);                                // Kt: 64 contiguous along N
            }
            const uint32_t t_d = tmem + kColD, t_o = tmem + kColO, t_st = tmem + kColSt;
            const uint32_t t_shi = tmem + kColShi, t_slo = tmem + kColSlo, t_dhi = tmem + kColDhi, t_dlo = tmem + kColDlo;
            for (int c = 0; c < n_chunks && ok; ++c) {
                const int sa = c % kStagesA, sc = c % kStagesC;
                if (!mbar_wait(&s.full_a[sa], (c / kStagesA) & 1)) { ok = false; break; }
                const uint64_t ka = a_desc[kStagesA > 1 ? sa : 0];
                // -S^T W^T with hi*hi + lo*hi + hi*lo: K = 128 key dims in 8 steps, taken in the order in which
                // the workers hand the split state over (each warp its first 32 key dims, then its second 32)
#pragma unroll
                for (int grp = 0; grp < 2; ++grp) {
                    if (!mbar_wait(&s.bar_s[grp], c & 1)) { ok = false; break; }        // S hi/lo of these key dims ready
                    tc::fence_after_sync();
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int kk = (u >> 1) * 4 + grp * 2 + (u & 1);                // 0, 1, 4, 5 then 2, 3, 6, 7
                        const uint64_t off = uint64_t(((kk >> 2) * (kC * 128) + (kk & 3) * 32) >> 4);
                        const uint64_t bw = ka + uint64_t(kOffW >> 4) + off, bwl = ka + uint64_t(kOffWlo >> 4) + off;
                        tc::mma_ts(t_d, t_shi + kk * 8, bw, id_n64_neg, (grp | u) > 0);
                        tc::mma_ts(t_d, t_slo + kk * 8, bw, id_n64_neg, 1);
                        tc::mma_ts(t_d, t_shi + kk * 8, bwl, id_n64_neg, 1);
                    }
                }
                if (!ok) break;
                tc::commit(&s.bar_w);
                // O^T = S^T Qg^T: behind the chain's MMAs, while the workers form D.  The previous chunk's
                // O^T must have been read out first.
                if (c > 0 && !mbar_wait(&s.bar_oread, (c - 1) & 1)) { ok = false; break; }
                tc::fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t bq = ka + uint64_t((kOffQg + (kk >> 2) * (kC * 128) + (kk & 3) * 32) >> 4);
                    tc::mma_ts(t_o, t_shi + kk * 8, bq, id_n64, kk > 0);
                    tc::mma_ts(t_o, t_slo + kk * 8, bq, id_n64, 1);
                }
                tc::commit(&s.empty_a[sa]);                                             // part A free once these are done
                if (!mbar_wait(&s.full_c[sc], (c / kStagesC) & 1)) { ok = false; break; }
                if (!mbar_wait(&s.bar_d, c & 1)) { ok = false; break; }                 // D hi/lo ready, S^T decayed
                tc::fence_after_sync();
                const uint64_t kc = ck_desc[kStagesC > 1 ? sc : 0];
                const uint64_t mc = cmn_desc[kStagesC > 1 ? sc : 0];
                // S^T += D^T Kt with hi*hi + lo*hi + hi*lo: K = 64 tokens in 4 steps
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t bk = mc + uint64_t((kOffKt + kk * 2048) >> 4), bkl = mc + uint64_t((kOffKtlo + kk * 2048) >> 4);
                    tc::mma_ts(t_st, t_dhi + kk * 8, bk, id_n128, 1);
                    tc::mma_ts(t_st, t_dlo + kk * 8, bk, id_n128, 1);
                    tc::mma_ts(t_st, t_dhi + kk * 8, bkl, id_n128, 1);
                }
                tc::commit(&s.bar_k);
                // O^T += D^T P^T
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {
                    const uint64_t bp = kc + uint64_t((kOffP + kk * 32) >> 4);
                    tc::mma_ts(t_o, t_dhi + kk * 8, bp, id_n64, 1);
                    tc::mma_ts(t_o, t_dlo + kk * 8, bp, id_n64, 1);
                }
                tc::commit(&s.empty_c[sc]);
                tc::commit(&s.bar_o);
            }
            if (!ok) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                s.failed = 1;
            }
        }
    } else if (warp >= kWarpScanOut0) {
        // ------------------------------ output warps: o[t][h][j] = O^T[j][t], off the chain ------------------------------
        const int wq = warp & 3;
        const int j = wq * 32 + lane;
        const uint32_t lane_addr = tmem + (uint32_t(wq * 32) << 16);
        bool ok = true;
        for (int c = 0; c < n_chunks; ++c) {
            if (ok && !mbar_wait(&s.bar_o, c & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            const int t0 = (a.chunk0 + c) * kC;
            uint32_t f[2][32];
            tc::tmem_ld32(lane_addr + kColO, f[0]);
            tc::tmem_ld32(lane_addr + kColO + 32, f[1]);
            tc::tmem_wait_ld();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.bar_oread);          // O^T is in registers: its columns may be overwritten
            // through shared memory, so that a warp writes whole 512-byte rows of o (one request per token
            // instead of four, a quarter of the store instructions)
            named_bar_sync(1, kScanOutput);                    // the previous chunk's rows have left the stage
#pragma unroll
            for (int q = 0; q < 2; ++q)
#pragma unroll
                for (int i = 0; i < 32; ++i) s.ostage[32 * q + i][j] = __uint_as_float(f[q][i]);
            named_bar_sync(2, kScanOutput);
            if (ok && !s.failed) {
#pragma unroll
                for (int i = 0; i < kC / 4; ++i) {
                    const int t = wq * (kC / 4) + i;
                    if (t0 + t < a.T)
                        __stcs(reinterpret_cast<float4*>(a.o + (size_t(t0 + t) * a.n_v + h) * kD) + lane,
                               *reinterpret_cast<const float4*>(&s.ostage[t][lane * 4]));
                }
            }
        }
    } else {
        // ------------------------------ workers: thread = (value dim j = TMEM lane, half of the columns) ------------------------------
        // A warp reaches the 32 lanes of its quadrant (warp % 4); the two warps of a quadrant take one half
        // of every pass's columns each, so a pass is half as long as with one thread per lane.  Every pass
        // issues all its tensor-memory loads before it waits once.
        const int wq = warp & 3, half = warp >> 2;
        const int j = wq * 32 + lane;
        const uint32_t lane_addr = tmem + (uint32_t(wq * 32) << 16);
        bool ok = true;
        // S_0^T into tensor memory: hi/lo of S_0 for the first chunk's products, and S_0 exp(G_C) of the
        // first chunk as the accumulator S^T += D^T Kt adds to.  Column i of lane j = S[i][j].
        {
            const float decay0 = a.chunk_decay[size_t(a.chunk0) * a.n_v + h];
#pragma unroll 1
            for (int c0 = 64 * half; c0 < 64 * half + 64; c0 += 32) {
                uint32_t f[32], hi[16], lo[16];
#pragma unroll
                for (int i = 0; i < 32; ++i) f[i] = __float_as_uint(Sg[size_t(c0 + i) * kD + j]);
#pragma unroll
                for (int i = 0; i < 16; ++i) split_h2(__uint_as_float(f[2 * i]), __uint_as_float(f[2 * i + 1]), hi[i], lo[i]);
#pragma unroll
                for (int i = 0; i < 32; ++i) f[i] = __float_as_uint(__uint_as_float(f[i]) * decay0);
                tc::tmem_st32(lane_addr + kColSt + c0, f);
                tc::tmem_st16(lane_addr + kColShi + c0 / 2, hi);
                tc::tmem_st16(lane_addr + kColSlo + c0 / 2, lo);
            }
        }
        tc::tmem_wait_st();
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) {
            mbar_arrive(&s.bar_s[0]);
            mbar_arrive(&s.bar_s[1]);
        }
        const float* tv = reinterpret_cast<const float*>(s.pb);
        for (int c = 0; c < n_chunks; ++c) {
            const bool last = c == n_chunks - 1;
            // exp(G_C) of the NEXT chunk: folded into the pass that splits the new state
            const float next_decay = last ? 1.f : a.chunk_decay[size_t(a.chunk0 + c + 1) * a.n_v + h];
            if (ok && !mbar_wait(&s.full_b, c & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            if (ok && !mbar_wait(&s.bar_w, c & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            // D^T = (T V)^T - S^T W^T -> hi/lo A operands; (T V)[t][j] comes from shared memory in fp32
            {
                uint32_t f[32], hi[16], lo[16];
                tc::tmem_ld32(lane_addr + kColD + 32 * half, f);
                tc::tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    split_h2(__uint_as_float(f[2 * i]) + tv[(32 * half + 2 * i) * kD + j],
                             __uint_as_float(f[2 * i + 1]) + tv[(32 * half + 2 * i + 1) * kD + j], hi[i], lo[i]);
                tc::tmem_st16(lane_addr + kColDhi + 16 * half, hi);
                tc::tmem_st16(lane_addr + kColDlo + 16 * half, lo);
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&s.bar_d);
                mbar_arrive(&s.empty_b);                       // T V has been read: the next chunk's may land
            }
            if (ok && !mbar_wait(&s.bar_k, c & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            // the new S^T: hi/lo for the next chunk's products and, times the next chunk's exp(G_C), the
            // accumulator its state update adds to (or back to the cache after the last chunk)
            {
                uint32_t f[2][32];
#pragma unroll
                for (int q = 0; q < 2; ++q) tc::tmem_ld32(lane_addr + kColSt + 32 * (2 * half + q), f[q]);
                tc::tmem_wait_ld();
                if (last) {
                    if (ok && !s.failed) {
#pragma unroll
                        for (int q = 0; q < 2; ++q)
#pragma unroll
                            for (int i = 0; i < 32; ++i) Sg[size_t(32 * (2 * half + q) + i) * kD + j] = __uint_as_float(f[q][i]);
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        uint32_t hi[16], lo[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            split_h2(__uint_as_float(f[q][2 * i]), __uint_as_float(f[q][2 * i + 1]), hi[i], lo[i]);
                        tc::tmem_st16(lane_addr + kColShi + 16 * (2 * half + q), hi);
                        tc::tmem_st16(lane_addr + kColSlo + 16 * (2 * half + q), lo);
#pragma unroll
                        for (int i = 0; i < 32; ++i) f[q][i] = __float_as_uint(__uint_as_float(f[q][i]) * next_decay);
                        tc::tmem_st32(lane_addr + kColSt + 32 * (2 * half + q), f[q]);
                        // hand these 32 key dims over: the first product's K steps over them start while the
                        // other 32 are being split
                        tc::tmem_wait_st();
                        tc::fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&s.bar_s[q]);
                    }
                }
            }
            tc::fence_before_sync();
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == kWarpScanMma) tc::tmem_dealloc(tmem, 512);
}

size_t delta_chunk_scan_smem_bytes() { return sizeof(ScanSmem) + 1024; }
int delta_chunk_scan_threads() { return kScanThreads; }
// per (chunk, head), M = 128, K = 16 each: -S^T W^T 24 and O^T 16 + 8 MMAs of N = 64, S^T += D^T Kt 12 MMAs of N = 128
double delta_chunk_scan_mma_flops() { return 2.0 * 128 * 16 * ((24 + 16 + 8) * 64 + 12 * 128); }

}  // namespace rl
