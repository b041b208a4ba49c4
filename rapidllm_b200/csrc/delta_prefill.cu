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
constexpr int kPad = kD + 1;
constexpr int kB = 16;                    // block size of the triangular inverse

struct PrepSmem {
    float kn[kC][kPad];       // k^
    union {
        float qn[kC][kPad];   // q^, dead once q^.k^ and the Qg tile are out
        struct {
            float m[kC][kC + 1];      // (I + A)^-1
            float tmp[kC][kC + 1];
        } inv;
    } u;
    float l[kC][kC + 1];      // k^_t . k^_i, then in place A (strictly lower part of I + A)
    float qk[kC][kC + 1];     // q^_t . k^_i
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
    const int chunk = blockIdx.x, h = blockIdx.y;
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
    // ---- l2 norms (double accumulators as ops::l2norm); padded tokens are all zero ----
    for (int t = warp; t < kC; t += kPrepThreads / 32) {
        float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), qx = kx;
        if (t < n_tok) {
            kx = *reinterpret_cast<const float4*>(a.k + (size_t(t0 + t) * a.n_qk + hs) * kD + lane * 4);
            qx = *reinterpret_cast<const float4*>(a.q + (size_t(t0 + t) * a.n_qk + hs) * kD + lane * 4);
        }
        double ks = double(kx.x) * kx.x + double(kx.y) * kx.y + double(kx.z) * kx.z + double(kx.w) * kx.w;
        double qs = double(qx.x) * qx.x + double(qx.y) * qx.y + double(qx.z) * qx.z + double(qx.w) * qx.w;
        for (int off = 16; off > 0; off >>= 1) {
            ks += __shfl_xor_sync(0xffffffffu, ks, off);
            qs += __shfl_xor_sync(0xffffffffu, qs, off);
        }
        float ki = 1.f / sqrtf(float(ks) + a.eps_l2);
        float qi = 1.f / sqrtf(float(qs) + a.eps_l2) * (1.f / sqrtf(float(kD)));
        if (t >= n_tok) ki = qi = 0.f;
        s.kn[t][lane * 4 + 0] = kx.x * ki; s.kn[t][lane * 4 + 1] = kx.y * ki;
        s.kn[t][lane * 4 + 2] = kx.z * ki; s.kn[t][lane * 4 + 3] = kx.w * ki;
        s.u.qn[t][lane * 4 + 0] = qx.x * qi; s.u.qn[t][lane * 4 + 1] = qx.y * qi;
        s.u.qn[t][lane * 4 + 2] = qx.z * qi; s.u.qn[t][lane * 4 + 3] = qx.w * qi;
    }
    __syncthreads();
    if (tid >= 32 && tid < kC) s.G[tid] += s.G[31];
    __syncthreads();
    if (tid < kC) s.eg[tid] = expf(s.G[tid]);
    if (tid == 0) a.chunk_decay[size_t(chunk) * a.n_v + h] = expf(s.G[kC - 1]);
    // ---- k^.k^ and q^.k^ (lower triangle), 4 x 4 outputs per thread ----
    {
        const int tb = (tid >> 4) * 4, ib = (tid & 15) * 4;
        float kk[4][4] = {}, qk[4][4] = {};
        if (ib <= tb + 3) {
            for (int d = 0; d < kD; ++d) {
                float kt[4], qt[4], ki[4];
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                    kt[x] = s.kn[tb + x][d];
                    qt[x] = s.u.qn[tb + x][d];
                    ki[x] = s.kn[ib + x][d];
                }
#pragma unroll
                for (int x = 0; x < 4; ++x)
#pragma unroll
                    for (int y = 0; y < 4; ++y) {
                        kk[x][y] += kt[x] * ki[y];
                        qk[x][y] += qt[x] * ki[y];
                    }
            }
        }
#pragma unroll
        for (int x = 0; x < 4; ++x)
#pragma unroll
            for (int y = 0; y < 4; ++y) {
                s.l[tb + x][ib + y] = kk[x][y];
                s.qk[tb + x][ib + y] = qk[x][y];
            }
    }
    __syncthreads();
    // ---- tiles that need q^: Qg; with it Kt and V (64 x 128, fp16, swizzled) ----
    const float gC = s.G[kC - 1];
    for (int idx = tid; idx < kC * kD / 4; idx += kPrepThreads) {
        const int t = idx >> 5, d = (idx & 31) * 4;
        const int o = tile_off(t, d);
        const float e = s.eg[t];
        *reinterpret_cast<uint2*>(rec + kOffQg + o) =
            make_uint2(pack_h2(e * s.u.qn[t][d], e * s.u.qn[t][d + 1]), pack_h2(e * s.u.qn[t][d + 2], e * s.u.qn[t][d + 3]));
        const float kt = expf(gC - s.G[t]);
        *reinterpret_cast<uint2*>(rec + kOffKt + o) =
            make_uint2(pack_h2(kt * s.kn[t][d], kt * s.kn[t][d + 1]), pack_h2(kt * s.kn[t][d + 2], kt * s.kn[t][d + 3]));
        float4 vv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (t < n_tok) vv = *reinterpret_cast<const float4*>(a.v + (size_t(t0 + t) * a.n_v + h) * kD + d);
        *reinterpret_cast<uint2*>(rec + kOffV + o) = make_uint2(pack_h2(vv.x, vv.y), pack_h2(vv.z, vv.w));
    }
    __syncthreads();                                  // q^ is dead from here on: its space becomes m and tmp
    float (*m)[kC + 1] = s.u.inv.m;
    float (*tmp)[kC + 1] = s.u.inv.tmp;
    // ---- A_ti = beta_t exp(G_t - G_i) (k^_t . k^_i), i < t, in place ----
    for (int idx = tid; idx < kC * kC; idx += kPrepThreads) {
        const int t = idx >> 6, i = idx & 63;
        s.l[t][i] = i < t ? s.beta[t] * expf(s.G[t] - s.G[i]) * s.l[t][i] : 0.f;
        m[t][i] = t == i ? 1.f : 0.f;
    }
    __syncthreads();
    // ---- M = (I + A)^-1, blocked: 16 x 16 diagonal blocks by forward substitution ... ----
    if (tid < kC) {
        const int bb = (tid >> 4) * kB, c = tid & 15;           // thread owns column c of block bb
        for (int t = c + 1; t < kB; ++t) {
            float acc = 0.f;
            for (int i = c; i < t; ++i) acc -= s.l[bb + t][bb + i] * m[bb + i][bb + c];
            m[bb + t][bb + c] = acc;
        }
    }
    __syncthreads();
    // ... then block row by block row: M_ij = -M_ii (sum_{j<=k<i} A_ik M_kj), j < i
    for (int bi = 1; bi < kC / kB; ++bi) {
        for (int idx = tid; idx < bi * kB * kB; idx += kPrepThreads) {
            const int bj = idx / (kB * kB), x = (idx >> 4) & 15, y = idx & 15;
            float acc = 0.f;
            for (int kx = bj * kB; kx < bi * kB; ++kx) acc += s.l[bi * kB + x][kx] * m[kx][bj * kB + y];
            tmp[bi * kB + x][bj * kB + y] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < bi * kB * kB; idx += kPrepThreads) {
            const int bj = idx / (kB * kB), x = (idx >> 4) & 15, y = idx & 15;
            float acc = 0.f;
            for (int kx = 0; kx <= x; ++kx) acc -= m[bi * kB + x][bi * kB + kx] * tmp[bi * kB + kx][bj * kB + y];
            m[bi * kB + x][bj * kB + y] = acc;
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
    // W[t][d] = sum_{i<=t} tmp[t][i] k^[i][d] (tmp is zero above the diagonal).  Warp w owns rows
    // w, w+8, ..., in two groups of four that share the k^ loads; lane owns dims 2l, 2l+1 (+64).
    for (int grp = 0; grp < 2; ++grp) {
        const int tr0 = warp + 8 * (4 * grp);
        float acc[4][4] = {};
        const int i_max = tr0 + 24;
        for (int i = 0; i <= i_max; ++i) {
            const float k0 = s.kn[i][2 * lane], k1 = s.kn[i][2 * lane + 1];
            const float k2 = s.kn[i][2 * lane + 64], k3 = s.kn[i][2 * lane + 65];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float c = tmp[tr0 + 8 * r][i];
                acc[r][0] += c * k0; acc[r][1] += c * k1; acc[r][2] += c * k2; acc[r][3] += c * k3;
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int t = tr0 + 8 * r;
            *reinterpret_cast<uint32_t*>(rec + kOffW + tile_off(t, 2 * lane)) = pack_h2(acc[r][0], acc[r][1]);
            *reinterpret_cast<uint32_t*>(rec + kOffW + tile_off(t, 2 * lane + 64)) = pack_h2(acc[r][2], acc[r][3]);
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

// grid (n_v), 192 threads.  o [T][n_v][128]; S [n_v][128][128] fp32 in place (row = key dim).
__global__ void __launch_bounds__(kScanThreads, 1) delta_chunk_scan_kernel(DeltaChunkArgs a) {
    extern __shared__ unsigned char smem_raw[];
    ScanSmem& s = *reinterpret_cast<ScanSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int h = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_chunks = (a.T + kC - 1) / kC;
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
                bulk_g2s(s.rec[st], a.work + (size_t(c) * a.n_v + h) * kRecordBytes, kRecordBytes, &s.full[st]);
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
            const float decay = a.chunk_decay[size_t(c) * a.n_v + h];
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
            const int t0 = c * kC;
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

}  // namespace rl
