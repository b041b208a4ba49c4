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
// Kernel 1 (delta_chunk_prepare_kernel) computes everything that does not depend on S for
// all (chunk, value head) pairs in parallel, one CTA each, and writes W, Qg, Kt, V, T, P as fp16
// tiles already in the 128-byte-swizzled operand format of the tensor cores, 80 KiB per pair.
// Kernel 2 (delta_chunk_scan_kernel), one CTA per value head, walks the chunks in order.
// Everything is transposed so that the 128 value dims are the MMA M dimension (TMEM lanes):
// S^T lives in tensor memory in fp32 for the whole sequence, and its fp16 high and low
// parts (S = hi + lo, ~22 bits) are the tensor-memory A operands of D^T = V^T T^T - S^T W^T
// and O^T = S^T Qg^T + D^T P^T; D^T (again hi + lo) is the A operand of S^T += D^T Kt.  A
// chunk's six tiles arrive with ONE linear TMA bulk copy into a two-stage ring.
#include "kernels.h"
#include "tcgen05.cuh"

namespace rl {

namespace {

constexpr int kC = 64;                    // chunk length
constexpr int kD = 128;                   // dk = dv
constexpr int kTileWide = kC * kD * 2;    // 16 KiB: 64 x 128 fp16
constexpr int kTileSq = kC * kC * 2;      // 8 KiB: 64 x 64 fp16
// record of one (chunk, head): byte offsets of the tiles
constexpr int kOffW = 0, kOffQg = kTileWide, kOffKt = 2 * kTileWide, kOffV = 3 * kTileWide;
constexpr int kOffT = 4 * kTileWide, kOffP = 4 * kTileWide + kTileSq;
constexpr int kRecordBytes = 4 * kTileWide + 2 * kTileSq;   // 81920

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

struct PrepSmem {
    float kn[kC][kPad];       // k^
    union {
        float qn[kC][kPad];   // q^, dead once q^.k^ and the Qg tile are out
        struct {
            float m[kC][kSq];         // (I + A)^-1
            float tmp[kC][kSq];
        } inv;
    } u;
    float l[kC][kSq];         // k^_t . k^_i, then in place A (strictly lower part of I + A)
    float qk[kC][kSq];        // q^_t . k^_i
    float G[kC], beta[kC], eg[kC];
};

}  // namespace

size_t delta_chunk_record_bytes() { return kRecordBytes; }

// grid (n_chunks, n_v), 256 threads: one CTA per chunk and value head.  98 KB of shared memory, so
// two CTAs share an SM and hide each other's barriers; the dot products k^.k^ and q^.k^ are
// recomputed by the value heads that share a key head (cheap next to the latency they hide).
__global__ void __launch_bounds__(kPrepThreads, 2) delta_chunk_prepare_kernel(DeltaChunkArgs a) {
    extern __shared__ unsigned char smem_raw[];
    PrepSmem& s = *reinterpret_cast<PrepSmem*>(smem_raw);
    const int chunk = a.chunk0 + blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rep = a.head_map == 0 ? 1 : a.n_v / a.n_qk;
    const int hs = a.head_map == 0 ? h : (a.head_map == 1 ? h / rep : h % a.n_qk);
    const int t0 = chunk * kC;
    const int n_tok = min(kC, a.T - t0);
    unsigned char* rec = a.work + (size_t(chunk) * a.n_v + h) * kRecordBytes;

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
    if (tid >= 32 && tid < kC) s.G[tid] += s.G[31];
    __syncthreads();
    if (tid < kC) s.eg[tid] = expf(s.G[tid]);
    if (tid == 0) a.chunk_decay[size_t(chunk) * a.n_v + h] = expf(s.G[kC - 1]);
    // ---- k^.k^ and q^.k^ on the tensor cores (3 x TF32 = fp32 accuracy): warp w owns rows
    // 16 (w & 3) .. +15 and columns 32 (w >> 2) .. +31; column tiles entirely above the diagonal
    // are skipped (and zero-filled, nobody reads more than their zero) ----
    {
        const int g = lane >> 2, c = lane & 3;
        const int t_base = (warp & 3) * 16, i_base = (warp >> 2) * 32;
        float ck[4][4] = {}, cq[4][4] = {};
        const int n_tiles = min(4, max(0, (t_base + 15 - i_base) / 8 + 1));   // tiles with i0 <= t_base + 15
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
            uint32_t bh[4][2], bl[4][2];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                if (nt < n_tiles) {
                    split_tf32(s.kn[i_base + 8 * nt + g][k0 + c], bh[nt][0], bl[nt][0]);
                    split_tf32(s.kn[i_base + 8 * nt + g][k0 + c + 4], bh[nt][1], bl[nt][1]);
                }
            }
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    if (nt < n_tiles) {
                        mma_tf32(ck[nt], pass == 0 ? akl : akh, pass == 1 ? bl[nt] : bh[nt]);
                        mma_tf32(cq[nt], pass == 0 ? aql : aqh, pass == 1 ? bl[nt] : bh[nt]);
                    }
                }
            }
        }
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const int i0 = i_base + 8 * nt + 2 * c;
            s.l[t_base + g][i0] = ck[nt][0];      s.l[t_base + g][i0 + 1] = ck[nt][1];
            s.l[t_base + g + 8][i0] = ck[nt][2];  s.l[t_base + g + 8][i0 + 1] = ck[nt][3];
            s.qk[t_base + g][i0] = cq[nt][0];     s.qk[t_base + g][i0 + 1] = cq[nt][1];
            s.qk[t_base + g + 8][i0] = cq[nt][2]; s.qk[t_base + g + 8][i0 + 1] = cq[nt][3];
        }
    }
    __syncthreads();
    // ---- tiles that need q^: Qg; with it Kt and V (64 x 128, fp16, swizzled) ----
    const float gC = s.G[kC - 1];
    {
        constexpr int kPer = kC * kD / 4 / kPrepThreads;      // 8 groups of 4 dims per thread
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
            const int o = tile_off(t, d);
            const float e = s.eg[t];
            *reinterpret_cast<uint2*>(rec + kOffQg + o) =
                make_uint2(pack_h2(e * s.u.qn[t][d], e * s.u.qn[t][d + 1]), pack_h2(e * s.u.qn[t][d + 2], e * s.u.qn[t][d + 3]));
            const float kt = expf(gC - s.G[t]);
            *reinterpret_cast<uint2*>(rec + kOffKt + o) =
                make_uint2(pack_h2(kt * s.kn[t][d], kt * s.kn[t][d + 1]), pack_h2(kt * s.kn[t][d + 2], kt * s.kn[t][d + 3]));
            *reinterpret_cast<uint2*>(rec + kOffV + o) = make_uint2(pack_h2(vv[u].x, vv[u].y), pack_h2(vv[u].z, vv[u].w));
        }
    }
    __syncthreads();                                  // q^ is dead from here on: its space becomes m and tmp
    float (*m)[kSq] = s.u.inv.m;
    float (*tmp)[kSq] = s.u.inv.tmp;
    // ---- A_ti = beta_t exp(G_t - G_i) (k^_t . k^_i), i < t, in place ----
    for (int idx = tid; idx < kC * kC; idx += kPrepThreads) {
        const int t = idx >> 6, i = idx & 63;
        s.l[t][i] = i < t ? s.beta[t] * expf(s.G[t] - s.G[i]) * s.l[t][i] : 0.f;
        m[t][i] = t == i ? 1.f : 0.f;
    }
    __syncthreads();
    // ---- M = (I + A)^-1 with all 256 threads and a dozen barriers ----
    // (1) the four 16 x 16 diagonal blocks: N = strictly lower part is nilpotent (N^16 = 0), so
    //     (I + N)^-1 = (I - N)(I + N^2)(I + N^4)(I + N^8): five small products, element (x, y) of
    //     block u per thread.  L, T, M below are the block's tiles of s.l, tmp, m.
    {
        const int x = tid >> 4, y = tid & 15;
#define RL_L(r, c) s.l[bb + (r)][bb + (c)]
#define RL_T(r, c) tmp[bb + (r)][bb + (c)]
#define RL_M(r, c) m[bb + (r)][bb + (c)]
#define RL_BLOCKS(BODY)                    \
    _Pragma("unroll") for (int u = 0; u < 4; ++u) { \
        const int bb = u * kB;             \
        BODY                               \
    }                                      \
    __syncthreads();
        RL_BLOCKS({ float acc = 0.f; for (int k = 0; k < kB; ++k) acc += RL_L(x, k) * RL_L(k, y); RL_T(x, y) = acc; })          // T = N^2
        RL_BLOCKS({ float acc = (x == y ? 1.f : 0.f) - RL_L(x, y);
                    for (int k = 0; k < kB; ++k) acc += ((x == k ? 1.f : 0.f) - RL_L(x, k)) * RL_T(k, y);
                    RL_M(x, y) = acc; })                                                                                    // M = (I - N)(I + N^2)
        RL_BLOCKS({ float acc = 0.f; for (int k = 0; k < kB; ++k) acc += RL_T(x, k) * RL_T(k, y); RL_L(x, y) = acc; })          // L = N^4
        RL_BLOCKS({ float acc = RL_M(x, y); for (int k = 0; k < kB; ++k) acc += RL_M(x, k) * RL_L(k, y); RL_T(x, y) = acc; })   // T = M (I + N^4)
        RL_BLOCKS({ float acc = 0.f; for (int k = 0; k < kB; ++k) acc += RL_L(x, k) * RL_L(k, y); RL_M(x, y) = acc; })          // M = N^8
        RL_BLOCKS({ float acc = RL_T(x, y); for (int k = 0; k < kB; ++k) acc += RL_T(x, k) * RL_M(k, y); RL_L(x, y) = acc; })   // L = T (I + N^8): the inverse
        RL_BLOCKS({ RL_M(x, y) = RL_L(x, y); })
#undef RL_BLOCKS
#undef RL_M
#undef RL_T
#undef RL_L
        // (2) off-diagonal blocks from inv [[P, 0], [C, Q]] = [[P^-1, 0], [-Q^-1 C P^-1, Q^-1]], first
        //     for the two 32 x 32 halves (C = a 16 x 16 block of A), then for the whole (C = 32 x 32)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int bi = (2 * u + 1) * kB, bj = 2 * u * kB;
            float acc = 0.f;
            for (int k = 0; k < kB; ++k) acc += s.l[bi + x][bj + k] * m[bj + k][bj + y];
            tmp[bi + x][bj + y] = acc;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int bi = (2 * u + 1) * kB, bj = 2 * u * kB;
            float acc = 0.f;
            for (int k = 0; k < kB; ++k) acc -= m[bi + x][bi + k] * tmp[bi + k][bj + y];
            m[bi + x][bj + y] = acc;
        }
        __syncthreads();
        const int x2 = tid >> 5, y2 = tid & 31;                 // rows 32 + x2 + 8 u, column y2
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int r = 32 + x2 + 8 * u;
            float acc = 0.f;
            for (int k = 0; k < 32; ++k) acc += s.l[r][k] * m[k][y2];
            tmp[r][y2] = acc;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int r = 32 + x2 + 8 * u;
            float acc = 0.f;
            for (int k = 0; k < 32; ++k) acc -= m[r][32 + k] * tmp[32 + k][y2];
            m[r][y2] = acc;
        }
        __syncthreads();
    }
    // ---- tiles: T = M diag(beta), P (64 x 64), fp16, swizzled ----
    for (int idx = tid; idx < kC * kC / 2; idx += kPrepThreads) {
        const int t = idx >> 5, i = (idx & 31) * 2;
        *reinterpret_cast<uint32_t*>(rec + kOffT + tile_off(t, i)) =
            pack_h2(m[t][i] * s.beta[i], m[t][i + 1] * s.beta[i + 1]);
        const float p0 = i <= t ? expf(s.G[t] - s.G[i]) * s.qk[t][i] : 0.f;
        const float p1 = i + 1 <= t ? expf(s.G[t] - s.G[i + 1]) * s.qk[t][i + 1] : 0.f;
        *reinterpret_cast<uint32_t*>(rec + kOffP + tile_off(t, i)) = pack_h2(p0, p1);
    }
    // fold beta_i exp(G_i) into M once: tmp[t][i] = M[t][i] beta_i exp(G_i)
    for (int idx = tid; idx < kC * kC; idx += kPrepThreads) {
        const int t = idx >> 6, i = idx & 63;
        tmp[t][i] = m[t][i] * s.beta[i] * s.eg[i];
    }
    __syncthreads();
    // W[t][d] = sum_{i<=t} tmp[t][i] k^[i][d] (tmp is zero above the diagonal), 3 x TF32 MMAs: warp w
    // owns rows 16 (w & 3) .. +15 and dims 64 (w >> 2) .. +63; K steps beyond the rows' diagonal skipped.
    {
        const int g = lane >> 2, c = lane & 3;
        const int t_base = (warp & 3) * 16, d_base = (warp >> 2) * 64;
        float acc[8][4] = {};
        for (int k0 = 0; k0 < t_base + 16; k0 += 8) {
            uint32_t ah[4], al[4];
            split_tf32(tmp[t_base + g][k0 + c], ah[0], al[0]);
            split_tf32(tmp[t_base + g + 8][k0 + c], ah[1], al[1]);
            split_tf32(tmp[t_base + g][k0 + c + 4], ah[2], al[2]);
            split_tf32(tmp[t_base + g + 8][k0 + c + 4], ah[3], al[3]);
            uint32_t bh[8][2], bl[8][2];
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                split_tf32(s.kn[k0 + c][d_base + 8 * nt + g], bh[nt][0], bl[nt][0]);
                split_tf32(s.kn[k0 + c + 4][d_base + 8 * nt + g], bh[nt][1], bl[nt][1]);
            }
#pragma unroll
            for (int pass = 0; pass < 3; ++pass)
#pragma unroll
                for (int nt = 0; nt < 8; ++nt) mma_tf32(acc[nt], pass == 0 ? al : ah, pass == 1 ? bl[nt] : bh[nt]);
        }
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const int d0 = d_base + 8 * nt + 2 * c;
            *reinterpret_cast<uint32_t*>(rec + kOffW + tile_off(t_base + g, d0)) = pack_h2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<uint32_t*>(rec + kOffW + tile_off(t_base + g + 8, d0)) = pack_h2(acc[nt][2], acc[nt][3]);
        }
    }
}

size_t delta_chunk_prepare_smem_bytes() { return sizeof(PrepSmem); }
int delta_chunk_prepare_threads() { return kPrepThreads; }

// ================================================================================================
namespace {

constexpr int kScanThreads = 192;         // 4 worker warps (lane = value dim) + loader warp + MMA warp
constexpr int kScanStages = 2;
// tensor memory map (columns); lane = value dim
constexpr uint32_t kColSt = 0;            // S^T fp32, 128 columns (column = key dim)
constexpr uint32_t kColShi = 128;         // fp16 pairs: 64 columns
constexpr uint32_t kColSlo = 192;
constexpr uint32_t kColD = 256;           // D^T fp32, 64 columns (column = token)
constexpr uint32_t kColO = 320;           // O^T fp32, 64 columns
constexpr uint32_t kColDhi = 384;         // fp16 pairs: 32 columns
constexpr uint32_t kColDlo = 416;

struct ScanSmem {
    alignas(1024) unsigned char rec[kScanStages][kRecordBytes];
    uint64_t full[kScanStages], empty[kScanStages];
    uint64_t bar_s, bar_g1, bar_d, bar_g3;
    uint32_t tmem_base;
    int failed;
};

// fp32 -> (fp16 high part, fp16 residual), two values per register
__device__ __forceinline__ void split_h2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    const __half2 hh = __halves2half2(h0, h1);
    hi = *reinterpret_cast<const uint32_t*>(&hh);
    lo = pack_h2(x0 - __half2float(h0), x1 - __half2float(h1));
}

}  // namespace

// grid (n_v), 192 threads.  o [T][n_v][128]; S [n_v][128][128] fp32 in place (row = key dim).  A launch
// walks chunks [chunk0, chunk0 + chunks): S is read at its start and written back at its end, so a
// sequence can be scanned in several launches while later chunks are still being prepared.
__global__ void __launch_bounds__(kScanThreads, 1) delta_chunk_scan_kernel(DeltaChunkArgs a) {
    extern __shared__ unsigned char smem_raw[];
    ScanSmem& s = *reinterpret_cast<ScanSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int h = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_chunks = a.chunks;            // of this launch; c below counts from a.chunk0
    float* Sg = a.S + size_t(h) * kD * kD;

    if (tid == 0) {
        for (int i = 0; i < kScanStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        mbar_init(&s.bar_s, 128);
        mbar_init(&s.bar_g1, 1);
        mbar_init(&s.bar_d, 128);
        mbar_init(&s.bar_g3, 1);
        s.failed = 0;
        mbar_fence_init();
    }
    if (warp == 5) tc::tmem_alloc(&s.tmem_base, 512);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s.tmem_base;

    if (warp == 4) {
        // ------------------------------ loader ------------------------------
        if (lane == 0) {
            for (int c = 0; c < n_chunks; ++c) {
                const int st = c % kScanStages;
                if (!mbar_wait(&s.empty[st], ((c / kScanStages) & 1) ^ 1)) { s.failed = 1; break; }
                mbar_arrive_expect_tx(&s.full[st], kRecordBytes);
                bulk_g2s(s.rec[st], a.work + (size_t(a.chunk0 + c) * a.n_v + h) * kRecordBytes, kRecordBytes, &s.full[st]);
            }
            if (s.failed) set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t id_n64 = tc::idesc_f16(128, kC, false, false);           // A K-major/TMEM, B K-major
            constexpr uint32_t id_n64_neg = id_n64 | (1u << 13);                        // -A
            constexpr uint32_t id_vt = tc::idesc_f16(128, kC, true, false);            // A = V^T MN-major (smem)
            constexpr uint32_t id_n128 = tc::idesc_f16(128, kD, false, true);          // B = Kt MN-major
            bool ok = true;
            // Descriptors are built once per ring stage and advanced by constants (their address
            // field counts 16-byte units): the issuing thread must spend only a few instructions
            // per tcgen05.mma or it, not the tensor pipe, sets the pace.
            uint64_t mn_desc[kScanStages], k_desc[kScanStages];
#pragma unroll
            for (int i = 0; i < kScanStages; ++i) {
                mn_desc[i] = tc::smem_desc(smem_u32(s.rec[i]), kC * 128, 1024);   // V^T, Kt: 64 contiguous along M/N
                k_desc[i] = tc::smem_desc(smem_u32(s.rec[i]), 16, 1024);          // T, W, Qg, P: K-major
            }
            const uint32_t t_d = tmem + kColD, t_o = tmem + kColO, t_st = tmem + kColSt;
            const uint32_t t_shi = tmem + kColShi, t_slo = tmem + kColSlo, t_dhi = tmem + kColDhi, t_dlo = tmem + kColDlo;
            for (int c = 0; c < n_chunks && ok; ++c) {
                const int st = c % kScanStages;
                if (!mbar_wait(&s.full[st], (c / kScanStages) & 1)) { ok = false; break; }
                if (!mbar_wait(&s.bar_s, c & 1)) { ok = false; break; }                 // S hi/lo ready
                tc::fence_after_sync();
                const uint64_t mn = st == 0 ? mn_desc[0] : mn_desc[1];
                const uint64_t km = st == 0 ? k_desc[0] : k_desc[1];
                // D^T = V^T T^T - S^T W^T
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)                                         // K = 64 tokens i
                    tc::mma_ss(t_d, mn + uint64_t((kOffV + kk * 2048) >> 4), km + uint64_t((kOffT + kk * 32) >> 4), id_vt,
                               kk > 0);
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {                                       // K = 128 key dims
                    const uint64_t bw = km + uint64_t((kOffW + (kk >> 2) * (kC * 128) + (kk & 3) * 32) >> 4);
                    tc::mma_ts(t_d, t_shi + kk * 8, bw, id_n64_neg, 1);
                    tc::mma_ts(t_d, t_slo + kk * 8, bw, id_n64_neg, 1);
                }
                // O^T = S^T Qg^T (+ D^T P^T below)
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    const uint64_t bq = km + uint64_t((kOffQg + (kk >> 2) * (kC * 128) + (kk & 3) * 32) >> 4);
                    tc::mma_ts(t_o, t_shi + kk * 8, bq, id_n64, kk > 0);
                    tc::mma_ts(t_o, t_slo + kk * 8, bq, id_n64, 1);
                }
                tc::commit(&s.bar_g1);
                if (!mbar_wait(&s.bar_d, c & 1)) { ok = false; break; }                 // D hi/lo ready, S^T decayed
                tc::fence_after_sync();
#pragma unroll
                for (int kk = 0; kk < 4; ++kk) {                                       // K = 64 tokens
                    const uint64_t bp = km + uint64_t((kOffP + kk * 32) >> 4);
                    tc::mma_ts(t_o, t_dhi + kk * 8, bp, id_n64, 1);
                    tc::mma_ts(t_o, t_dlo + kk * 8, bp, id_n64, 1);
                    const uint64_t bk = mn + uint64_t((kOffKt + kk * 2048) >> 4);
                    tc::mma_ts(t_st, t_dhi + kk * 8, bk, id_n128, 1);
                    tc::mma_ts(t_st, t_dlo + kk * 8, bk, id_n128, 1);
                }
                tc::commit(&s.empty[st]);
                tc::commit(&s.bar_g3);
            }
            if (!ok) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                s.failed = 1;
            }
        }
    } else {
        // ------------------------------ workers: thread = value dim j = TMEM lane ------------------------------
        const int j = tid;
        const uint32_t lane_addr = tmem + (uint32_t(warp * 32) << 16);
        bool ok = true;
        // S_0^T into tensor memory (fp32 and hi/lo): column i of lane j = S[i][j]
#pragma unroll 1
        for (int c0 = 0; c0 < kD; c0 += 32) {
            uint32_t f[32], hi[16], lo[16];
#pragma unroll
            for (int i = 0; i < 32; ++i) f[i] = __float_as_uint(Sg[size_t(c0 + i) * kD + j]);
#pragma unroll
            for (int i = 0; i < 16; ++i) split_h2(__uint_as_float(f[2 * i]), __uint_as_float(f[2 * i + 1]), hi[i], lo[i]);
            tc::tmem_st32(lane_addr + kColSt + c0, f);
            tc::tmem_st16(lane_addr + kColShi + c0 / 2, hi);
            tc::tmem_st16(lane_addr + kColSlo + c0 / 2, lo);
        }
        tc::tmem_wait_st();
        tc::fence_before_sync();
        mbar_arrive(&s.bar_s);
        for (int c = 0; c < n_chunks; ++c) {
            const float decay = a.chunk_decay[size_t(a.chunk0 + c) * a.n_v + h];
            // S^T *= exp(G_C) while the tensor core works from the hi/lo copies
#pragma unroll 1
            for (int c0 = 0; c0 < kD; c0 += 32) {
                uint32_t f[32];
                tc::tmem_ld32(lane_addr + kColSt + c0, f);
                tc::tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) f[i] = __float_as_uint(__uint_as_float(f[i]) * decay);
                tc::tmem_st32(lane_addr + kColSt + c0, f);
            }
            tc::tmem_wait_st();
            if (ok && !mbar_wait(&s.bar_g1, c & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            // D^T -> hi/lo A operands
#pragma unroll 1
            for (int c0 = 0; c0 < kC; c0 += 32) {
                uint32_t f[32], hi[16], lo[16];
                tc::tmem_ld32(lane_addr + kColD + c0, f);
                tc::tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) split_h2(__uint_as_float(f[2 * i]), __uint_as_float(f[2 * i + 1]), hi[i], lo[i]);
                tc::tmem_st16(lane_addr + kColDhi + c0 / 2, hi);
                tc::tmem_st16(lane_addr + kColDlo + c0 / 2, lo);
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
            mbar_arrive(&s.bar_d);
            if (ok && !mbar_wait(&s.bar_g3, c & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            // o[t][h][j] = O^T[j][t]
            const int t0 = (a.chunk0 + c) * kC;
#pragma unroll 1
            for (int c0 = 0; c0 < kC; c0 += 32) {
                uint32_t f[32];
                tc::tmem_ld32(lane_addr + kColO + c0, f);
                tc::tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    if (ok && t0 + c0 + i < a.T) a.o[(size_t(t0 + c0 + i) * a.n_v + h) * kD + j] = __uint_as_float(f[i]);
            }
            // new S^T -> hi/lo for the next chunk (or back to the cache after the last one)
            const bool last = c == n_chunks - 1;
#pragma unroll 1
            for (int c0 = 0; c0 < kD; c0 += 32) {
                uint32_t f[32], hi[16], lo[16];
                tc::tmem_ld32(lane_addr + kColSt + c0, f);
                tc::tmem_wait_ld();
                if (last) {
                    if (ok && !s.failed)
#pragma unroll
                        for (int i = 0; i < 32; ++i) Sg[size_t(c0 + i) * kD + j] = __uint_as_float(f[i]);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) split_h2(__uint_as_float(f[2 * i]), __uint_as_float(f[2 * i + 1]), hi[i], lo[i]);
                    tc::tmem_st16(lane_addr + kColShi + c0 / 2, hi);
                    tc::tmem_st16(lane_addr + kColSlo + c0 / 2, lo);
                }
            }
            tc::tmem_wait_st();
            tc::fence_before_sync();
            if (!last) mbar_arrive(&s.bar_s);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 5) tc::tmem_dealloc(tmem, 512);
}

size_t delta_chunk_scan_smem_bytes() { return sizeof(ScanSmem) + 1024; }
int delta_chunk_scan_threads() { return kScanThreads; }
// per (chunk, head), M = 128, K = 16 each: D^T 4 + 16 and O^T 16 + 8 MMAs of N = 64, S^T 8 MMAs of N = 128
double delta_chunk_scan_mma_flops() { return 2.0 * 128 * 16 * ((4 + 16 + 16 + 8) * 64 + 8 * 128); }

}  // namespace rl
