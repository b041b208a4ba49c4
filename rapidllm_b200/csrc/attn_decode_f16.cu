// Split-KV GQA decode attention over the paged F16 KV cache (sm_100a).
//
// Replaces the reference's one-block-per-head context walk
// (src/kernels/cuda/cuda_engine.cu:303-375 flash_attn_decode_f16_hd256, called
// from qk_attn_decode_gqa_k 5802-5862) and computes what ops::attn_decode
// (src/kernels/ops.cpp:575-605) computes, for a batch of ragged sequences.
//
// Structure: a persistent grid (one CTA per SM).  The (sequence, KV head, half
// page) units of the whole batch form one list and every CTA owns an equal
// contiguous share of it (attn_split.cuh), cut into segments at (sequence, head)
// boundaries.  One producer thread streams half pages (32 tokens of K and of V,
// 32 KiB) into a ring of shared-memory stages with TMA bulk copies that complete
// on mbarriers; it runs ahead across segment boundaries so the HBM stream never
// drains.  Six consumer warps (three pairs, one pair per stage in flight) each
// own 16 tokens of a stage: scores for the whole GQA group (<= 8 query heads)
// come from m16n8k16 tensor-core MMAs with the fp32 query split into an fp16
// high part (MMA rows 0-7) and its fp16 residual (rows 8-15, otherwise idle), the
// online softmax runs in registers, and P.V accumulates transposed (dims x
// heads) so that P feeds the second MMA straight from the score registers.  At
// the end of a segment the warps' (m, l, acc) merge in shared memory into one
// partial per (segment, head); attn_combine.cu merges the few partials of a
// (sequence, head) and applies the sigmoid gate.
#include "attn_split.cuh"
#include "kernels.h"

namespace rl {

namespace {

constexpr int kStageTokens = 32;                 // half a page
constexpr int kStages = 6;
constexpr int kSlots = 3;                        // consumer warp pairs
constexpr int kConsumerWarps = 6;
static_assert(kConsumerWarps == 2 * kSlots, "two warps per stage in flight");
// 6 consumer warps + 1 producer warp + 1 idle warp: 256 threads lets every thread have 255 registers
constexpr int kThreads = 256;
constexpr int kSubTiles = kHeadDim / 64;         // 4
constexpr int kStageKBytes = kStageTokens * kHeadDim * 2;  // 16 KiB
constexpr int kStageBytes = 2 * kStageKBytes;              // K + V
constexpr int kSubTileStageBytes = kStageTokens * 128;     // 4 KiB
constexpr int kSubTilePageBytes = kPageTokens * 128;       // 8 KiB
using split::kNegBig;
using split::Segment;

struct Smem {
    alignas(128) unsigned char stage[kStages][kStageBytes];
    split::Shared<kConsumerWarps> sp;
    uint64_t full[kStages];
    uint64_t empty[kStages];
};

}  // namespace

__global__ void __launch_bounds__(kThreads, 1)
attn_decode_f16_kernel(AttnDecodeArgs a) {
    extern __shared__ unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int G = a.n_q / a.n_kv;

    griddep_launch();
    // the appended rows, the query and the workspace belong to kernels in front of this one
    if (!a.stream_before_wait) griddep_wait();
    // chunk prefix over the batch (every CTA computes the same table)
    if (warp == 0)
        split::build_prefix(s.sp, a.seq_lens, a.len_add, a.batch, a.max_pages_per_seq, a.err, lane);
    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 2);
        }
        mbar_fence_init();
    }
    __syncthreads();
    int u_begin, u_end;
    split::cta_range(s.sp, a.batch, a.n_kv, u_begin, u_end, a.seg_weight);

    if (a.stream_before_wait && warp != kConsumerWarps) griddep_wait();
    if (warp > kConsumerWarps) return;
    if (warp == kConsumerWarps) {
        // ------------------------------ producer ------------------------------
        // The warp reads 32 page ids at a time (one per lane), so that the page-table latency is
        // paid once per 16 pages; lane 0 waits for free stages and issues the copies.
        uint32_t it = 0;
        bool ok = true;
        bool waited = !a.stream_before_wait;      // lane 0: the kernel in front has completed
        for (int pos = u_begin; pos < u_end;) {
            const Segment w = split::segment_at(s.sp, pos, u_end, a.batch, a.n_kv, a.seq_lens, a.len_add);
            pos += w.hp1 - w.hp0;
            const int last_page = (w.len - 1) >> 6;   // where this step's token was appended
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
                    if (!waited && (hp >> 1) >= last_page) {
                        griddep_wait();
                        waited = true;
                    }
                    if (!mbar_wait(&s.empty[st], ph ^ 1)) {
                        set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                        ok = false;
                        continue;
                    }
                    const size_t slice = (size_t(page) * a.n_kv + w.h) * kv_slice_elems();
                    const unsigned char* ksrc = reinterpret_cast<const unsigned char*>(a.k_pool + slice) +
                                                (hp & 1) * kSubTileStageBytes;
                    const unsigned char* vsrc = reinterpret_cast<const unsigned char*>(a.v_pool + slice) +
                                                (hp & 1) * kSubTileStageBytes;
                    unsigned char* dst = s.stage[st];
                    mbar_arrive_expect_tx(&s.full[st], kStageBytes);
#pragma unroll
                    for (int sub = 0; sub < kSubTiles; ++sub) {
                        bulk_g2s(dst + sub * kSubTileStageBytes, ksrc + sub * kSubTilePageBytes,
                                 kSubTileStageBytes, &s.full[st]);
                        bulk_g2s(dst + kStageKBytes + sub * kSubTileStageBytes,
                                 vsrc + sub * kSubTilePageBytes, kSubTileStageBytes, &s.full[st]);
                    }
                }
            }
        }
        return;
    }

    // -------------------------------- consumers --------------------------------
    const int g = lane >> 2;                       // MMA group id: query head / token column
    const int c = lane & 3;
    const int pg = ((g & 1) << 2) | (g >> 1);      // bank-conflict-free permutation of 0..7
    const int slot = warp >> 1;
    const int tb = (warp & 1) * 16;                // this warp's tokens inside a stage
    const float scale_log2 = a.scale * 1.4426950408889634f;

    uint32_t it = 0;
    bool alive = true;   // false after a wait gave up: keep arriving at barriers, touch no data
    for (int pos = u_begin; pos < u_end;) {
        const Segment w = split::segment_at(s.sp, pos, u_end, a.batch, a.n_kv, a.seq_lens, a.len_add);
        pos += w.hp1 - w.hp0;

        // query fragments: rows 0-7 fp16(q), rows 8-15 fp16(q - fp16(q))
        uint32_t qhi[8][4], qlo[8][4];
        {
            const bool live = g < G;
            const float* qp = a.q + (size_t(w.b) * a.n_q + w.h * G + (live ? g : 0)) * kHeadDim;
#pragma unroll
            for (int L = 0; L < 8; ++L) {
                float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
                if (live) {
                    x0 = *reinterpret_cast<const float4*>(qp + 32 * L + 8 * c);
                    x1 = *reinterpret_cast<const float4*>(qp + 32 * L + 8 * c + 4);
                }
                const float v[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __half h0 = __float2half_rn(v[2 * e]);
                    const __half h1 = __float2half_rn(v[2 * e + 1]);
                    const __half2 hh = __halves2half2(h0, h1);
                    qhi[L][e] = *reinterpret_cast<const uint32_t*>(&hh);
                    qlo[L][e] = pack_h2(v[2 * e] - __half2float(h0), v[2 * e + 1] - __half2float(h1));
                }
            }
        }

        float acc[4][4][4];                          // [sub-tile j][pair i][c0..c3]
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[j][i][e] = 0.f;
        float m_run = kNegBig;                       // log2 domain, head g
        float l_run = 0.f;                           // this lane's share of the row sum

        for (int hp = w.hp0; hp < w.hp1; ++hp, ++it) {
            if (int(it % kSlots) != slot) continue;
            const int st = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (alive && !mbar_wait(&s.full[st], ph)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                alive = false;
            }
            const int n_valid = min(kStageTokens, w.len - hp * kStageTokens) - tb;  // in this warp's 16
            if (alive && n_valid > 0) {
                const uint32_t kst = smem_u32(s.stage[st]);
                const uint32_t vsa = kst + kStageKBytes;
                unsigned char* vst = s.stage[st] + kStageKBytes;
                if (n_valid < 16) {
                    // rows past the end of the sequence may hold anything: clear V
                    for (int r = tb + n_valid; r < tb + 16; ++r)
                        for (int x = lane; x < kSubTiles * 8; x += 32)
                            *reinterpret_cast<uint4*>(vst + (x >> 3) * kSubTileStageBytes + r * 128 +
                                                      (x & 7) * 16) = make_uint4(0, 0, 0, 0);
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                }
                // ---- scores: S[heads][16 tokens], two n-tiles, two chains each ----
                float sc[2][2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int z = 0; z < 2; ++z)
#pragma unroll
                        for (int e = 0; e < 4; ++e) sc[nt][z][e] = 0.f;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const int r = tb + 8 * nt + pg;
                    const uint32_t rowp = kst + r * 128;
#pragma unroll
                    for (int L = 0; L < 8; ++L) {
                        const int chunk = (4 * (L & 1) + c) ^ (r & 7);
                        const uint4 kk = lds128(rowp + (L >> 1) * kSubTileStageBytes + chunk * 16);
                        mma_f16(sc[nt][0], qhi[L][0], qlo[L][0], qhi[L][1], qlo[L][1], kk.x, kk.y);
                        mma_f16(sc[nt][1], qhi[L][2], qlo[L][2], qhi[L][3], qlo[L][3], kk.z, kk.w);
                    }
                }
                // ---- online softmax (columns: tokens tb+c, tb+4+c, tb+8+c, tb+12+c) ----
                float p[4];
                float mx = kNegBig;
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float sv = (sc[nt][0][e] + sc[nt][1][e]) + (sc[nt][0][e + 2] + sc[nt][1][e + 2]);
                        const int tok = 8 * nt + 4 * e + c;
                        p[nt * 2 + e] = tok < n_valid ? sv * scale_log2 : kNegBig;
                        mx = fmaxf(mx, p[nt * 2 + e]);
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
                for (int e = 0; e < 4; ++e) {
                    p[e] = p[e] > 0.5f * kNegBig ? fast_exp2(p[e] - m_run) : 0.f;
                    l_run += p[e];
                }
                const uint32_t pb0 = pack_h2(p[0], p[1]);   // tokens tb+c, tb+4+c
                const uint32_t pb1 = pack_h2(p[2], p[3]);   // tokens tb+8+c, tb+12+c
                // ---- acc[dims][heads] += V^T P^T ----
                const int r0 = tb + c, r1 = tb + 4 + c, r8 = tb + 8 + c, r9 = tb + 12 + c;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t sub = vsa + j * kSubTileStageBytes;
                    const uint4 v0 = lds128(sub + r0 * 128 + ((pg ^ (r0 & 7)) << 4));
                    const uint4 v1 = lds128(sub + r1 * 128 + ((pg ^ (r1 & 7)) << 4));
                    const uint4 v8 = lds128(sub + r8 * 128 + ((pg ^ (r8 & 7)) << 4));
                    const uint4 v9 = lds128(sub + r9 * 128 + ((pg ^ (r9 & 7)) << 4));
                    const uint32_t x0[4] = {v0.x, v0.y, v0.z, v0.w};
                    const uint32_t x1[4] = {v1.x, v1.y, v1.z, v1.w};
                    const uint32_t x8[4] = {v8.x, v8.y, v8.z, v8.w};
                    const uint32_t x9[4] = {v9.x, v9.y, v9.z, v9.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        mma_f16(acc[j][i], __byte_perm(x0[i], x1[i], 0x5410),
                                __byte_perm(x0[i], x1[i], 0x7632), __byte_perm(x8[i], x9[i], 0x5410),
                                __byte_perm(x8[i], x9[i], 0x7632), pb0, pb1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.empty[st]);
        }

        split::merge_segment(s.sp, acc, m_run, l_run, warp, lane, pg, G, a.part_o, a.part_ml,
                             size_t(blockIdx.x) + size_t(w.b) * a.n_kv + w.h);
    }
}

size_t attn_decode_f16_smem_bytes() { return sizeof(Smem) + 128; }
int attn_decode_f16_threads() { return kThreads; }
int attn_decode_max_batch() { return split::kMaxBatch; }

}  // namespace rl
