// Split-KV GQA decode attention over the compact KV cache: q8 K + TurboQuant-3 V (sm_100a).
//
// Replaces qk_attn_decode_tq_gqa_k (src/kernels/cuda/cuda_engine.cu:8382-8454), which
// walks the whole context with four thread blocks, dequantising every V row with two
// Walsh-Hadamard transforms (dequant_v_tq3_256, 293-299).  Two identities remove the
// per-token work:
//   * q . (s_k * k_int8) = s_k * (q . k_int8): the query is quantised once per segment to two
//     int8 levels (q ~ s1*q1 + s2*q2, 16-bit effective precision) and the scores come from
//     int8 tensor-core MMAs (m16n8k32) straight off the stored bytes, level 1 in MMA rows
//     0-7 and level 2 in rows 8-15;
//   * the transform is linear and orthonormal: sum_t p_t H(s_t c_t) = H(sum_t p_t s_t c_t), so
//     P.V accumulates in the rotated domain -- the codes of a token pair are stored
//     interleaved, so 6 bits index a lane-private shared-memory table that returns one
//     fp16x2 MMA operand register; the per-token scale is folded into P -- and ONE inverse
//     transform per output head is applied by the merge kernel.
// The persistent producer/consumer structure, the work division and the segment merge are those
// of attn_decode_f16.cu; a stage is one 32-token record (11 456 B, see kv_compact.cu).
#include "attn_split.cuh"
#include "kernels.h"

namespace rl {

namespace {

constexpr int kStages = 14;
constexpr int kConsumerWarps = 7;                  // each consumes whole records, round-robin
constexpr int kThreads = 256;                      // 7 consumer warps + 1 producer warp
using split::kNegBig;
using split::Segment;

struct Smem {
    alignas(128) unsigned char stage[kStages][kCompactRecordBytes];
    // 6-bit index (code of the even token | code of the odd token << 3) -> fp16x2 centroids;
    // one copy per lane ([index][lane]) so that a warp's 32 lookups never share a bank
    alignas(128) uint32_t lut[64][32];
    split::Shared<kConsumerWarps> sp;
    uint64_t full[kStages];
    uint64_t empty[kStages];
};

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_s8x4(int a, int b, int c, int d) {
    return (uint32_t(a) & 0xffu) | ((uint32_t(b) & 0xffu) << 8) | ((uint32_t(c) & 0xffu) << 16) |
           ((uint32_t(d) & 0xffu) << 24);
}

// The 6 bits starting at bit BIT of a 24-byte group held in six words, times 128 (the byte
// stride between table indices).
template <int BIT>
__device__ __forceinline__ uint32_t index_offset(const uint32_t (&w)[6]) {
    constexpr int word = BIT >> 5, sh = BIT & 31;
    uint32_t x;
    if constexpr (sh + 6 <= 32) {
        if constexpr (sh >= 7) x = w[word] >> (sh - 7);
        else x = w[word] << (7 - sh);
    } else {
        x = __funnelshift_r(w[word], w[word + 1], sh - 7);
    }
    return x & 0x1f80u;
}

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) attn_decode_tq_kernel(AttnDecodeArgs a) {
    extern __shared__ unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int G = a.n_q / a.n_kv;

    griddep_launch();     // the merge kernel behind this one may be scheduled; it waits for this grid
    griddep_wait();
    if (warp == 0)
        split::build_prefix(s.sp, a.seq_lens, a.len_add, a.batch, a.max_pages_per_seq, a.err, lane);
    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        mbar_fence_init();
    }
    {   // centroid table (3-bit Lloyd-Max for N(0,1), cuda_engine.cu:205-209), fp16
        const float cent[8] = {-2.152f, -1.344f, -0.756f, -0.245f, 0.245f, 0.756f, 1.344f, 2.152f};
        for (int x = tid; x < 64 * 32; x += kThreads) s.lut[x >> 5][x & 31] = pack_h2(cent[(x >> 5) & 7], cent[x >> 8]);
    }
    __syncthreads();
    int u_begin, u_end;
    split::cta_range(s.sp, a.batch, a.n_kv, u_begin, u_end, a.seg_weight);

    if (warp == kConsumerWarps) {
        // ------------------------------ producer ------------------------------
        // The warp reads 32 page ids at a time (one per lane), so that the page-table latency is
        // paid once per 16 pages; lane 0 waits for free stages and issues the copies.
        uint32_t it = 0;
        bool ok = true;
        for (int pos = u_begin; pos < u_end;) {
            const Segment w = split::segment_at(s.sp, pos, u_end, a.batch, a.n_kv, a.seq_lens, a.len_add);
            pos += w.hp1 - w.hp0;
            for (int hp_base = w.hp0; hp_base < w.hp1; hp_base += 32) {
                int my_page = 0;
                if (hp_base + lane < w.hp1) {
                    my_page = a.page_table[size_t(w.b) * a.max_pages_per_seq + ((hp_base + lane) >> 1)];
                    if (my_page < 0 || my_page >= a.n_pages) {
                        set_err(a.err, DEV_ERR_BAD_PAGE);
                        my_page = 0;
                    }
                }
                const int n = min(32, w.hp1 - hp_base);
                for (int j = 0; j < n; ++j, ++it) {
                    const int page = __shfl_sync(0xffffffffu, my_page, j);
                    if (lane != 0 || !ok) continue;
                    const int hp = hp_base + j;
                    const int st = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait(&s.empty[st], ph ^ 1)) {
                        set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                        ok = false;
                        continue;
                    }
                    const unsigned char* src = reinterpret_cast<const unsigned char*>(a.k_pool) +
                                               ((size_t(page) * a.n_kv + w.h) * 2 + (hp & 1)) * kCompactRecordBytes;
                    mbar_arrive_expect_tx(&s.full[st], kCompactRecordBytes);
                    bulk_g2s(s.stage[st], src, kCompactRecordBytes, &s.full[st]);
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    // A warp takes every 7th record (32 tokens): scores for all 32 tokens first (four independent
    // int8 MMA chains), one online-softmax update, then the two 16-token halves of P.V.
    const int g = lane >> 2;
    const int c = lane & 3;
    const float scale_log2 = a.scale * 1.4426950408889634f;
    const uint32_t lut = smem_u32(&s.lut[0][lane]);
    const uint32_t stage0 = smem_u32(s.stage[0]);

    uint32_t it = 0;
    bool alive = true;
    for (int pos = u_begin; pos < u_end;) {
        const Segment w = split::segment_at(s.sp, pos, u_end, a.batch, a.n_kv, a.seq_lens, a.len_add);
        pos += w.hp1 - w.hp0;

        // Query of head g in two int8 levels.  MMA (L, z) contracts dims 64L + 16c + 8z + 0..7
        // of this lane: qa[L][z][0] level 1 dims +0..3, [1] level 2 dims +0..3, [2] level 1 dims
        // +4..7, [3] level 2 dims +4..7.
        uint32_t qa[4][2][4];
        float s1 = 0.f, s2 = 0.f;
        {
            const bool live = g < G;
            const float* qp = a.q + (size_t(w.b) * a.n_q + w.h * G + (live ? g : 0)) * kHeadDim;
            float qv[4][2][8];
            float amax = 0.f;
#pragma unroll
            for (int L = 0; L < 4; ++L)
#pragma unroll
                for (int z = 0; z < 2; ++z) {
                    float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
                    if (live) {
                        x0 = *reinterpret_cast<const float4*>(qp + 64 * L + 16 * c + 8 * z);
                        x1 = *reinterpret_cast<const float4*>(qp + 64 * L + 16 * c + 8 * z + 4);
                    }
                    const float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        qv[L][z][e] = v[e];
                        amax = fmaxf(amax, fabsf(v[e]));
                    }
                }
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            s1 = amax / 127.f + 1e-20f;
            s2 = s1 / 254.f;
            const float i1 = 1.f / s1, i2 = 1.f / s2;
#pragma unroll
            for (int L = 0; L < 4; ++L)
#pragma unroll
                for (int z = 0; z < 2; ++z) {
                    int q1[8], q2[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        q1[e] = __float2int_rn(fminf(fmaxf(qv[L][z][e] * i1, -127.f), 127.f));
                        const float r = qv[L][z][e] - s1 * float(q1[e]);
                        q2[e] = __float2int_rn(fminf(fmaxf(r * i2, -127.f), 127.f));
                    }
                    qa[L][z][0] = pack_s8x4(q1[0], q1[1], q1[2], q1[3]);
                    qa[L][z][1] = pack_s8x4(q2[0], q2[1], q2[2], q2[3]);
                    qa[L][z][2] = pack_s8x4(q1[4], q1[5], q1[6], q1[7]);
                    qa[L][z][3] = pack_s8x4(q2[4], q2[5], q2[6], q2[7]);
                }
        }

        float acc[4][4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][i][e] = 0.f;
        float m_run = kNegBig;
        float l_run = 0.f;

        for (int hp = w.hp0; hp < w.hp1; ++hp, ++it) {
            if (int(it % kConsumerWarps) != warp) continue;
            const int st = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (alive && !mbar_wait(&s.full[st], ph)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                alive = false;
            }
            const int n_valid = min(kCompactHalfTokens, w.len - hp * kCompactHalfTokens);
            if (alive) {
                const uint32_t rec = stage0 + st * kCompactRecordBytes;
                // ---- scores from the stored int8 rows: n-tile nt = tokens 8nt .. 8nt+7 ----
                int sc[4][4];
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) sc[nt][e] = 0;
#pragma unroll
                for (int L = 0; L < 4; ++L) {
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt) {
                        const int r = 8 * nt + g;
                        const int chunk = (4 * L + c) ^ ((r & 1) << 2);
                        const uint4 kk = lds128(rec + r * 256 + chunk * 16);
                        mma_s8(sc[nt], qa[L][0][0], qa[L][0][1], qa[L][0][2], qa[L][0][3], kk.x, kk.y);
                        mma_s8(sc[nt], qa[L][1][0], qa[L][1][1], qa[L][1][2], qa[L][1][3], kk.z, kk.w);
                    }
                }
                // ---- online softmax; columns 2c, 2c+1 of n-tile nt are tokens 8nt + 2c (+1) ----
                float p[8];
                float mx = kNegBig;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    const uint32_t ks_raw = lds32(rec + kCompactKScaleOff + (8 * nt + 2 * c) * 2);
                    const float2 ks = __half22float2(*reinterpret_cast<const __half2*>(&ks_raw));
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float sv = (e ? ks.y : ks.x) * (s1 * float(sc[nt][e]) + s2 * float(sc[nt][e + 2]));
                        const int tok = 8 * nt + 2 * c + e;
                        p[nt * 2 + e] = tok < n_valid ? sv * scale_log2 : kNegBig;
                        mx = fmaxf(mx, p[nt * 2 + e]);
                    }
                }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run, mx);
                if (__any_sync(0xffffffffu, m_new > m_run)) {
                    const float alpha = fast_exp2(m_run - m_new);
                    l_run *= alpha;
                    const float a0 = __shfl_sync(0xffffffffu, alpha, 8 * c);
                    const float a1 = __shfl_sync(0xffffffffu, alpha, 8 * c + 4);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            acc[j][i][0] *= a0;
                            acc[j][i][1] *= a1;
                            acc[j][i][2] *= a0;
                            acc[j][i][3] *= a1;
                        }
                    m_run = m_new;
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    p[e] = p[e] > 0.5f * kNegBig ? fast_exp2(p[e] - m_run) : 0.f;
                    l_run += p[e];
                }
                // ---- the two 16-token halves: acc[dims][heads] += centroids(V codes)^T (P * scale)^T ----
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    // fold the V scales into P: one B operand per transform block (dims 0-127 / 128-255)
                    uint32_t pb[2][2];
#pragma unroll
                    for (int q2 = 0; q2 < 2; ++q2) {
                        const int nt = 2 * blk + q2;
                        const uint2 raw = lds64(rec + kCompactVScaleOff + (8 * nt + 2 * c) * 4);
                        const float2 t0 = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));  // even token
                        const float2 t1 = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));  // odd token
                        // rows beyond the sequence may hold anything: their p is 0, keep the product 0
                        const float p0 = p[nt * 2], p1 = p[nt * 2 + 1];
                        pb[0][q2] = pack_h2(p0 > 0.f ? p0 * t0.x : 0.f, p1 > 0.f ? p1 * t1.x : 0.f);
                        pb[1][q2] = pack_h2(p0 > 0.f ? p0 * t0.y : 0.f, p1 > 0.f ? p1 * t1.y : 0.f);
                    }
                    uint32_t wa[6], wb[6];
                    {
                        const uint32_t va = rec + kCompactVOff + blk * 1536 + g * 96 + c * 24;
                        const uint2 a0 = lds64(va), a1 = lds64(va + 8), a2 = lds64(va + 16);
                        const uint2 b0 = lds64(va + 768), b1 = lds64(va + 776), b2 = lds64(va + 784);
                        wa[0] = a0.x; wa[1] = a0.y; wa[2] = a1.x; wa[3] = a1.y; wa[4] = a2.x; wa[5] = a2.y;
                        wb[0] = b0.x; wb[1] = b0.y; wb[2] = b1.x; wb[3] = b1.y; wb[4] = b2.x; wb[5] = b2.y;
                    }
                    // codes of rows past the end are arbitrary but finite table entries; with p = 0
                    // they contribute exactly 0, nothing to clear
#define RL_TQ_LUT(W, BIT) lds32(lut + index_offset<(BIT)>(W))
#define RL_TQ_MMA(J, I)                                                                              \
    mma_f16(acc[J][I], RL_TQ_LUT(wa, 12 * (4 * (J) + (I))), RL_TQ_LUT(wa, 12 * (4 * (J) + (I)) + 6), \
            RL_TQ_LUT(wb, 12 * (4 * (J) + (I))), RL_TQ_LUT(wb, 12 * (4 * (J) + (I)) + 6),            \
            pb[(J) >> 1][0], pb[(J) >> 1][1]);
                    RL_TQ_MMA(0, 0) RL_TQ_MMA(0, 1) RL_TQ_MMA(0, 2) RL_TQ_MMA(0, 3)
                    RL_TQ_MMA(1, 0) RL_TQ_MMA(1, 1) RL_TQ_MMA(1, 2) RL_TQ_MMA(1, 3)
                    RL_TQ_MMA(2, 0) RL_TQ_MMA(2, 1) RL_TQ_MMA(2, 2) RL_TQ_MMA(2, 3)
                    RL_TQ_MMA(3, 0) RL_TQ_MMA(3, 1) RL_TQ_MMA(3, 2) RL_TQ_MMA(3, 3)
#undef RL_TQ_MMA
#undef RL_TQ_LUT
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.empty[st]);
        }
        split::merge_segment(s.sp, acc, m_run, l_run, warp, lane, g, G, a.part_o, a.part_ml,
                             size_t(blockIdx.x) + size_t(w.b) * a.n_kv + w.h);
    }
}

size_t attn_decode_tq_smem_bytes() { return sizeof(Smem) + 128; }
int attn_decode_tq_threads() { return kThreads; }

}  // namespace rl
