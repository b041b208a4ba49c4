// Chunked causal attention prefill over the paged F16 KV cache on tcgen05 / TMEM (sm_100a).
//
// Computes what ops::attn_prefill (src/kernels/ops.cpp:542-573) computes for the query rows
// of one chunk -- T rows at positions pos0 .. pos0+T-1 attending to cache rows [0, pos] with
// the causal offset of the reference's chunk driver (src/kernels/cuda/cuda_engine.cu:
// 8963-8975, launch_prefill_chunk 18338-18590) -- followed by the sigmoid output gate.  It
// replaces the reference's CUDA-core prefill kernels and its cuBLAS TF32 path
// (launch_attn_gqa_gemm, 9038-9125).
//
// One CTA = 128 query rows of one query head.  Q (bf16 -> fp16) is written once into tensor
// memory.  KV tiles are whole pages: a (page, head) slice is stored in HBM in exactly the
// tensor-core tile format (kv_slice_offset), so a tile moves with linear TMA bulk copies and is
// consumed in place: K as the K-major B operand of S = Q K^T (M 128, N 64, 16 MMAs of K 16), V
// as the MN-major B operand of O += P V (M 128, N 256, 4 MMAs).  Q and P are A operands read
// from tensor memory, so shared memory carries only the K/V tiles (fills + one read each).
// Tensor memory: S (64 columns), two P buffers (fp16 pairs, 32 columns each), O (256), Q (128).
//
// Warps: 16 softmax warps in two groups that take alternate KV tiles (TMEM lane = query row; the
// two warps of a group that share a lane quadrant split a row's 64 scores and exchange the row
// maximum through shared memory); a loader warp streaming pages; one thread issuing the S MMAs
// and one thread of another warp issuing the P.V MMAs -- two issuers keep the in-order tensor
// pipe fed while either waits, and each spends only a few instructions per tcgen05.mma
// (descriptors are prebuilt per ring stage).  S is released as soon as a group has it in
// registers, so the next S = Q K^T runs under the current tile's exponentials.  The running
// row maximum is handed from tile to tile through shared memory (mrow/bar_m) and is only
// raised when it grows by more than 2^8; then the deciding group rescales O in tensor memory.
// Each thread keeps its partial row sum relative to the maximum it last saw.  Epilogue: O / l
// goes through shared memory so that the gate is read and the output written by whole rows.
// Completion is signalled through tcgen05.commit on mbarriers; all waits are bounded.
//
// Two variations for calls with few query rows (short chunks, the rows of a speculative verify):
// kv_parts > 1 divides the KV tiles of an item among several CTAs that write partials for the
// log-sum-exp merge kernel; packed makes the 128 MMA rows (token, query head of the GQA group)
// pairs, one item per KV head, so the group's heads share a single pass over K/V.
// A third for item counts a little above a multiple of the SM count (192 items of a 1 024-row chunk
// on 148 SMs): tail_parts > 1 divides only the items of the last, partly filled wave, so that the
// wave's work is spread over every SM; attn_prefill_tail_merge_kernel merges those items' partials.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"
#include "tcgen05.cuh"

namespace rl {

namespace {

constexpr int kQRows = 128;
constexpr int kKvTile = kPageTokens;              // 64
constexpr int kKStages = 3, kVStages = 3;         // K tiles and V tiles are staged in separate rings
constexpr int kSliceBytes = kPageTokens * kHeadDim * 2;   // 32 KiB
constexpr int kGroupThreads = 256;                // one softmax group: 8 warps
constexpr int kSoftmaxThreads = 512;              // two groups, alternating KV tiles
constexpr int kThreads = 608;                     // + loader warp + two MMA-issuing warps
constexpr int kWarpLoader = 16, kWarpQK = 17, kWarpPV = 18;
constexpr uint32_t kTmemCols = 512;
// Tensor memory map (512 columns x 128 lanes, lane = query row): S in columns [0,64), two P
// buffers (fp16 pairs, 32 columns each) in [64,128), O in [128,384), Q (fp16 pairs) in [384,512).
constexpr uint32_t kColS = 0, kColP = 64, kColO = 128, kColQ = 384;
constexpr float kRescaleThreshold = 8.f;          // log2 units
// Q rows arrive by one bulk copy per row into V stages 1 and 2 (not needed before the second P.V), rows
// 528 bytes apart so that the thread-per-row reads spread over all banks.
constexpr int kQRowStride = kHeadDim * 2 + 16;
constexpr int kQStageBytes = kQRows * kQRowStride;            // 67 584
static_assert(kQStageBytes > 2 * kSliceBytes && kVStages >= 3, "Q staging = V stages 1, 2 + q_pad");

// item of the launch order -> (query tile, query head)
__device__ __forceinline__ void item_tile(const AttnPrefillArgs& a, int item, int n_qtiles, int& qt, int& hq) {
    const int G = a.n_q / a.n_kv;
    if (a.by_size) {
        qt = n_qtiles - 1 - item / a.n_q;
        hq = item % a.n_q;
    } else {
        const int per_kv = n_qtiles * G, hkv = item / per_kv, rem = item - hkv * per_kv;
        qt = n_qtiles - 1 - rem / G;
        hq = hkv * G + rem % G;
    }
}

struct Smem {
    alignas(1024) unsigned char k[kKStages][kSliceBytes];     // K page slices
    alignas(1024) unsigned char v[kVStages][kSliceBytes];     // V page slices
    unsigned char q_pad[kQStageBytes - 2 * kSliceBytes];      // with v[1], v[2]: where the Q rows land first
    uint64_t k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages];
    uint64_t bar_s[2], bar_sfree[2], bar_p[2], bar_pv[2], bar_m[2], bar_q, bar_done, bar_qload, bar_qfree;
    float xch[2][2][kQRows][2];                       // [group][use parity] row maxima of the two column halves
    float mrow[2][kQRows];                            // [tile parity] running maximum after that tile
    alignas(16) float lsum[kQRows][4];                 // read back as one float4 per row
    uint32_t tmem_base;
    int failed;
};

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) attn_prefill_kernel(AttnPrefillArgs a) {
    extern __shared__ unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_qtiles = (a.T + kQRows - 1) / kQRows;
    // 1-D grid; launch order = one KV head after the other (its K/V stay hot in L2 and the CTAs
    // running side by side read the same tiles), inside a KV head the longest jobs first: the
    // group's query heads of the last (heaviest) query tile, then of the one before, ...
    const int G = a.n_q / a.n_kv;
    const bool tail = a.tail_parts > 1 && int(blockIdx.x) >= a.n_full;
    const int tail_unit = int(blockIdx.x) - a.n_full;
    const int parts = tail ? a.tail_parts : (a.kv_parts > 1 ? a.kv_parts : 1);
    const int item = tail ? a.n_full + tail_unit / parts : int(blockIdx.x) / parts;
    const int part = tail ? tail_unit % parts : int(blockIdx.x) - item * parts;
    // packed (a few rows, e.g. a speculative verify): one item per KV head, its MMA rows are
    // (token, query head of the group) pairs, so the group's heads share one pass over K/V
    int qt = 0, hq = item * G;
    if (!a.packed) item_tile(a, item, n_qtiles, qt, hq);
    const int hkv = hq / G;
    const int q0 = qt * kQRows;                               // first query row of this CTA
    const int rows = a.packed ? a.T * G : min(kQRows, a.T - q0);
    const int last_pos = a.packed ? a.pos0 + a.T - 1 : a.pos0 + q0 + rows - 1;   // position of the last query row
    // MMA row r -> row of the [T][n_q] tensors, and its position
    auto flat_row = [&](int r) { return a.packed ? size_t(r / G) * a.n_q + hkv * G + r % G : size_t(q0 + r) * a.n_q + hq; };
    auto row_pos = [&](int r) { return a.packed ? a.pos0 + r / G : a.pos0 + q0 + r; };
    const int n_tiles_all = last_pos / kKvTile + 1;           // KV tiles [0, n_tiles_all) of this query tile
    // this CTA's share [j0, j0 + n_tiles); below j counts from 0 inside the share
    const int j0 = int(1LL * part * n_tiles_all / parts);
    const int n_tiles = int(1LL * (part + 1) * n_tiles_all / parts) - j0;

    if (tid == 0) {
        for (int i = 0; i < kKStages; ++i) {
            mbar_init(&s.k_full[i], 1);
            mbar_init(&s.k_empty[i], 1);
        }
        for (int i = 0; i < kVStages; ++i) {
            mbar_init(&s.v_full[i], 1);
            mbar_init(&s.v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.bar_s[i], 1);
            mbar_init(&s.bar_sfree[i], kGroupThreads);
            mbar_init(&s.bar_p[i], kGroupThreads);
            mbar_init(&s.bar_pv[i], 1);
            mbar_init(&s.bar_m[i], kGroupThreads);
        }
        mbar_init(&s.bar_q, kSoftmaxThreads);
        mbar_init(&s.bar_done, 1);
        mbar_init(&s.bar_qload, 1);
        mbar_init(&s.bar_qfree, kSoftmaxThreads);
        s.failed = 0;
        mbar_fence_init();
    }
    if (warp == kWarpQK) tc::tmem_alloc(&s.tmem_base, kTmemCols);
    griddep_launch();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    griddep_wait();       // the barriers and the tensor memory were set up beside the tail of the kernel before
    const uint32_t tmem = s.tmem_base;
    // Q rows -> tensor memory as the A operand of S = Q K^T (bf16 -> fp16 is exact for
    // normal-range values): lane = row, column c holds dims 2c, 2c+1; each of the four threads
    // of a row stores 64 dims.  The rows come in by bulk copies (one per row), issued by the loader warp
    // ahead of its first K/V tiles.
    unsigned char* qstage = s.v[1];
    if (warp == kWarpLoader) {
        if (lane == 0) mbar_arrive_expect_tx(&s.bar_qload, uint32_t(rows) * kHeadDim * 2);
        __syncwarp();
        for (int r = lane; r < rows; r += 32)
            bulk_g2s(qstage + r * kQRowStride, a.q + flat_row(r) * kHeadDim, kHeadDim * 2, &s.bar_qload);
        __syncwarp();
        // The CTA that follows this one on the SM is, to a good approximation, the one a wave further down
        // the launch order: start its Q rows on their way into L2.
        const int nxt = int(blockIdx.x) + int(a.wave);
        if (!a.packed && parts == 1 && nxt < (a.tail_parts > 1 ? a.n_full : int(gridDim.x))) {
            int n_qt, n_hq;
            item_tile(a, nxt, n_qtiles, n_qt, n_hq);
            const int n_q0 = n_qt * kQRows;
            const int n_rows = min(kQRows, a.T - n_q0);
            for (int i = lane; i < n_rows * 4; i += 32) {     // 4 lines of 128 bytes per row
                const __nv_bfloat16* pq = a.q + (size_t(n_q0 + (i >> 2)) * a.n_q + n_hq) * kHeadDim + (i & 3) * 64;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(pq));
            }
        }
    }
    if (tid < kSoftmaxThreads) {
        const int qpart = warp >> 2, r = (warp & 3) * 32 + lane;
        const uint32_t lane_addr = tmem + (uint32_t((warp & 3) * 32) << 16);
        uint32_t regs[32];
        bool got = mbar_wait(&s.bar_qload, 0);
        if (!got) {
            set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
            s.failed = 1;
        }
        uint4 in[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch)
            in[ch] = (got && r < rows) ? *reinterpret_cast<const uint4*>(qstage + r * kQRowStride + qpart * 128 + ch * 16)
                                       : make_uint4(0, 0, 0, 0);
        mbar_arrive(&s.bar_qfree);                            // V stages 1, 2 may be filled once all have read
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&in[ch]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(b2[e]);
                regs[ch * 4 + e] = pack_h2(f.x, f.y);
            }
        }
        tc::tmem_st32(lane_addr + kColQ + qpart * 32, regs);
        tc::tmem_wait_st();
        tc::fence_before_sync();
        mbar_arrive(&s.bar_q);                                // Q is in tensor memory (awaited by the S issuer)
        // the epilogue's gate rows: start them on their way into L2 now (2 of the row's 8 lines each)
        if (a.gate && parts <= 1 && r < rows) {
            const float* gp = a.gate + flat_row(r) * kHeadDim + qpart * 64;
            asm volatile("prefetch.global.L2 [%0];" ::"l"(gp));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(gp + 32));
        }
    }

    if (warp == kWarpLoader) {
        // ------------------------------ page loader ------------------------------
        // K_j is needed early (S_j = Q K_j^T is issued one tile ahead), V_j late (O += P_j V_j):
        // two rings, each freed by the MMA that last read it.
        if (lane == 0) {
            for (int j = 0; j < n_tiles; ++j) {
                const int ks = j % kKStages, vs = j % kVStages;
                int page = a.page_table[j0 + j];
                if (page < 0 || page >= a.n_pages) {
                    set_err(a.err, DEV_ERR_BAD_PAGE);
                    page = 0;
                }
                const size_t slice = (size_t(page) * a.n_kv + hkv) * kv_slice_elems();
                if (!mbar_wait(&s.k_empty[ks], ((j / kKStages) & 1) ^ 1)) { s.failed = 1; break; }
                mbar_arrive_expect_tx(&s.k_full[ks], kSliceBytes);
                bulk_g2s(s.k[ks], a.k_pool + slice, kSliceBytes, &s.k_full[ks]);
                if (!mbar_wait(&s.v_empty[vs], ((j / kVStages) & 1) ^ 1)) { s.failed = 1; break; }
                if (j == 1 && !mbar_wait(&s.bar_qfree, 0)) { s.failed = 1; break; }   // the Q rows were staged in V stages 1, 2
                mbar_arrive_expect_tx(&s.v_full[vs], kSliceBytes);
                bulk_g2s(s.v[vs], a.v_pool + slice, kSliceBytes, &s.v_full[vs]);
            }
            if (s.failed) set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
        }
    } else if (warp == kWarpQK) {
        // ------------------------------ S = Q K^T issuer ------------------------------
        // Two issuing threads (this one and the next warp) feed the one in-order tensor pipe: while one
        // is waiting on a barrier the other keeps the pipe busy.
        // The issuing thread must spend only a few instructions per tcgen05.mma (a 128x64x16 MMA
        // retires in about 45 clocks): descriptors are built once per ring stage and advanced by
        // constants (their address field counts 16-byte units).
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::idesc_f16(kQRows, kKvTile, false, false);
            uint64_t k_desc[kKStages];
#pragma unroll
            for (int i = 0; i < kKStages; ++i) k_desc[i] = tc::smem_desc(smem_u32(s.k[i]), 16, 1024);
            const uint32_t q_tmem = tmem + kColQ;
            bool ok = mbar_wait(&s.bar_q, 0);
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int st = j % kKStages;
                if (!mbar_wait(&s.k_full[st], (j / kKStages) & 1)) { ok = false; break; }
                // the S buffer is free once every softmax thread of the previous tile has read it out
                if (j >= 1 && !mbar_wait(&s.bar_sfree[(j - 1) & 1], ((j - 1) >> 1) & 1)) { ok = false; break; }
                tc::fence_after_sync();
                const uint64_t kd = st == 0 ? k_desc[0] : (st == 1 ? k_desc[1] : k_desc[2]);
                const uint32_t s_tmem = tmem + kColS;
                // 16 K-steps of 16 dims: A = 8 columns of Q in tensor memory, B = 32 bytes further
                // into the 64-dim sub-tile of the K slice
#pragma unroll
                for (int kk = 0; kk < 16; ++kk)
                    tc::mma_ts(s_tmem, q_tmem + kk * 8, kd + uint64_t(((kk >> 2) * (kKvTile * 128) + (kk & 3) * 32) >> 4),
                               idesc_qk, kk > 0);
                tc::commit(&s.k_empty[st]);           // K stage free once S_j is done
                tc::commit(&s.bar_s[j & 1]);
            }
            if (!ok) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                s.failed = 1;
            }
        }
    } else if (warp == kWarpPV) {
        // ------------------------------ O += P V issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_pv = tc::idesc_f16(kQRows, kHeadDim, false, true);
            uint64_t v_desc[kVStages];
#pragma unroll
            for (int i = 0; i < kVStages; ++i) v_desc[i] = tc::smem_desc(smem_u32(s.v[i]), kKvTile * 128, 1024);
            bool ok = true;
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % kVStages;
                if (!mbar_wait(&s.v_full[st], (j / kVStages) & 1)) { ok = false; break; }
                if (!mbar_wait(&s.bar_p[j & 1], (j >> 1) & 1)) { ok = false; break; }
                tc::fence_after_sync();
                const uint64_t vd = st == 0 ? v_desc[0] : (st == 1 ? v_desc[1] : v_desc[2]);
                const uint32_t p_tmem = tmem + kColP + (j & 1) * 32;
                // 4 K-steps of 16 tokens: A = 8 columns of P in tensor memory, B = 16 rows of V
                tc::mma_ts(tmem + kColO, p_tmem, vd, idesc_pv, j > 0);
#pragma unroll
                for (int kk = 1; kk < 4; ++kk)
                    tc::mma_ts(tmem + kColO, p_tmem + kk * 8, vd + uint64_t((kk * 16 * 128) >> 4), idesc_pv, 1);
                tc::commit(&s.v_empty[st]);           // V stage free
                tc::commit(&s.bar_pv[j & 1]);         // this P buffer free, O consistent
            }
            if (!ok) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                s.failed = 1;
            }
            tc::commit(&s.bar_done);
        }
    } else {
        // ------------------------------ softmax warps ------------------------------
        // Group g (warps 8g .. 8g+7) owns the tiles j with j & 1 == g, so two tiles are in flight:
        // the latency of one tile (TMEM load, maxima, exponentials, P store) overlaps the other's.
        // The only hand-over between consecutive tiles is the running row maximum (mrow + bar_m).
        const int grp = warp >> 3, half = (warp >> 2) & 1, quad = warp & 3;   // column half, TMEM lane quadrant
        const int r = quad * 32 + lane;                       // query row = TMEM lane
        const int pos = row_pos(r);                           // its position (rows >= `rows` are padding)
        const uint32_t lane_addr = tmem + (uint32_t(quad * 32) << 16);
        const float scale_log2 = a.scale * 1.4426950408889634f;
        float m_known = -1e30f, l_part = 0.f;                 // l_part is relative to m_known
        bool ok = true;
        for (int j = grp; j < n_tiles; j += 2) {
            const uint32_t par = (j >> 1) & 1;                // phase of this tile on the [j & 1] barriers
            if (ok && !mbar_wait(&s.bar_s[grp], par)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            uint32_t raw[32];
            if (ok) {
                tc::tmem_ld32(lane_addr + kColS + half * 32, raw);
                tc::tmem_wait_ld();
            }
            tc::fence_before_sync();
            mbar_arrive(&s.bar_sfree[grp]);                   // the scores are in registers: S buffer free
            const int tok0 = (j0 + j) * kKvTile;
            if (j0 + j == n_tiles_all - 1 && last_pos + 1 - tok0 < kKvTile) {
                // V rows past the last position may hold anything (0 * NaN would poison O): clear them
                if (ok && !mbar_wait(&s.v_full[j % kVStages], (j / kVStages) & 1)) {
                    set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                    ok = false;
                }
                const int first = last_pos + 1 - tok0;
                unsigned char* vt = s.v[j % kVStages];
                for (int idx = tid - grp * kGroupThreads; idx < (kKvTile - first) * 32; idx += kGroupThreads) {
                    const int row = first + (idx >> 5), c16 = idx & 31;
                    *reinterpret_cast<uint4*>(vt + (c16 >> 3) * (kKvTile * 128) + row * 128 + (c16 & 7) * 16) =
                        make_uint4(0, 0, 0, 0);
                }
                tc::fence_async_smem();
            }
            // raw scores -> maximum (scale > 0, so the maximum can be taken before scaling);
            // only tiles that reach past the first row's position need the causal mask
            const bool masked = tok0 + kKvTile - 1 > row_pos(0);
            float mx = -1e30f;
            if (masked) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    if (tok0 + half * 32 + i > pos) raw[i] = 0xff800000u;      // -inf
                    mx = fmaxf(mx, __uint_as_float(raw[i]));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(raw[i]));
            }
            // the row maximum over both halves: exchange with the partner warp of this quadrant
            s.xch[grp][par][r][half] = mx;
            named_bar_sync(1 + grp * 4 + quad, 64);
            mx = fmaxf(mx, s.xch[grp][par][r][half ^ 1]);
            mx = fmaxf(mx * scale_log2, -1e30f);
            // running maximum after the previous tile (owned by the other group)
            float m_prev = -1e30f;
            if (j > 0) {
                if (ok && !mbar_wait(&s.bar_m[grp ^ 1], ((j - 1) >> 1) & 1)) {
                    set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                    ok = false;
                }
                m_prev = s.mrow[grp ^ 1][r];
            }
            // raise it only when it grew by more than the threshold
            float m_new = m_prev, alpha = 1.f;
            if (mx > m_prev + kRescaleThreshold) {
                alpha = fast_exp2(m_prev - mx);                   // 0 on the first tile
                m_new = mx;
            }
            if (half == 0) s.mrow[grp][r] = m_new;
            mbar_arrive(&s.bar_m[grp]);                       // release: the next tile may read mrow[grp]
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                // O must not be in use by the tensor core: wait for P.V of tile j-1 (P_j is not
                // published before this is done, so P.V of tile j and later come after it)
                if (ok && !mbar_wait(&s.bar_pv[grp ^ 1], ((j - 1) >> 1) & 1)) {
                    set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                    ok = false;
                }
                tc::fence_after_sync();
                if (ok) {
#pragma unroll 1
                    for (int c0 = 0; c0 < kHeadDim / 2; c0 += 32) {
                        uint32_t o[32];
                        tc::tmem_ld32(lane_addr + kColO + half * 128 + c0, o);
                        tc::tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tc::tmem_st32(lane_addr + kColO + half * 128 + c0, o);
                    }
                    tc::tmem_wait_st();
                }
            }
            // this thread's partial row sum follows the maximum (it may have moved twice since
            // this group's previous tile)
            if (m_new != m_known) {
                l_part *= fast_exp2(m_known - m_new);
                m_known = m_new;
            }
            // p = 2^(s * scale - m): one FFMA + one EX2 per score (-inf gives exactly 0)
            uint32_t ph[16];
            float lsum0 = 0.f, lsum1 = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float p0 = fast_exp2(fmaf(__uint_as_float(raw[2 * i]), scale_log2, -m_new));
                const float p1 = fast_exp2(fmaf(__uint_as_float(raw[2 * i + 1]), scale_log2, -m_new));
                lsum0 += p0;
                lsum1 += p1;
                ph[i] = pack_h2(p0, p1);
            }
            l_part += lsum0 + lsum1;
            // P row -> tensor memory, the A operand of O += P V: this thread's 32 tokens are fp16
            // columns [16 half, 16 half + 16) of P buffer grp, last read by P.V of tile j-2
            if (ok && j >= 2 && !mbar_wait(&s.bar_pv[grp], ((j - 2) >> 1) & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            tc::fence_after_sync();
            if (ok) {
                tc::tmem_st16(lane_addr + kColP + grp * 32 + half * 16, ph);
                tc::tmem_wait_st();
            }
            tc::fence_before_sync();
            mbar_arrive(&s.bar_p[grp]);
        }
        // ------------------------------ epilogue ------------------------------
        // final maximum = after the last tile; the four partial sums of a row are brought to it
        float m_fin = -1e30f;
        if (n_tiles > 0) {
            if (ok && !mbar_wait(&s.bar_m[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                ok = false;
            }
            m_fin = s.mrow[(n_tiles - 1) & 1][r];
        }
        s.lsum[r][grp * 2 + half] = l_part * fast_exp2(m_known - m_fin);
        named_bar_sync(9, kSoftmaxThreads);
        const float4 lp = *reinterpret_cast<const float4*>(s.lsum[r]);
        const float l_run = (lp.x + lp.y) + (lp.z + lp.w);
        if (n_tiles > 0 && ok && !mbar_wait(&s.bar_done, 0)) {
            set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
            ok = false;
        }
        tc::fence_after_sync();
        // O / l -> shared memory (the K and V rings are free now: every MMA has completed), row
        // stride 260 floats so that the thread-per-row stores spread over the banks; then each
        // warp takes whole rows, so the gate is read and the output written in full 512-byte
        // requests.  With kv_parts > 1 the output stays unnormalised and ungated.
        float* stage = reinterpret_cast<float*>(s.k[0]);
        constexpr int kStageStride = kHeadDim + 4;
        static_assert(sizeof(float) * kQRows * kStageStride <= sizeof(s.k) + sizeof(s.v), "O staging must fit the rings");
        const bool good = ok && !s.failed;
        const bool split = parts > 1;
        if (good) {
            const float inv = split ? 1.f : (l_run > 0.f ? 1.f / l_run : 0.f);
            const int col0 = (half * 2 + grp) * 64;           // this thread's 64 output columns
#pragma unroll 1
            for (int c0 = 0; c0 < 64; c0 += 32) {
                uint32_t o[32];
                if (n_tiles > 0) {
                    tc::tmem_ld32(lane_addr + kColO + col0 + c0, o);
                    tc::tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = 0u;   // no tile: O was never written
                }
#pragma unroll
                for (int i = 0; i < 32; i += 4)
                    *reinterpret_cast<float4*>(stage + r * kStageStride + col0 + c0 + i) =
                        make_float4(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv,
                                    __uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
            }
            if (split && grp == 0 && half == 0 && r < rows) {
                float* ml = a.part_ml + (tail ? size_t(tail_unit) * kQRows + r : size_t(part) * a.T * a.n_q + flat_row(r)) * 2;
                ml[0] = m_fin * 0.6931471805599453f;          // log2 domain -> natural-log units
                ml[1] = l_run;
            }
        }
        // The gate values this warp needs (rows warp, warp + 16, ...: 8 rows x 2 x float4 per lane; the
        // prologue started them towards L2) are all requested before the first is used.
        const bool gated = a.gate && parts <= 1;
        constexpr int kRowsPerWarp = kQRows / (kSoftmaxThreads / 32);
        float4 gq[kRowsPerWarp][2];
        if (gated && good) {
#pragma unroll
            for (int i = 0; i < kRowsPerWarp; ++i) {
                const int row = warp + i * (kSoftmaxThreads / 32);
                if (row < rows) {
                    const float* gp = a.gate + flat_row(row) * kHeadDim + lane * 4;
                    gq[i][0] = __ldcs(reinterpret_cast<const float4*>(gp));
                    gq[i][1] = __ldcs(reinterpret_cast<const float4*>(gp + 128));
                }
            }
        }
        named_bar_sync(9, kSoftmaxThreads);
        if (good) {
            // sigmoid(g) = 1 / (1 + 2^(-g log2 e)) with the hardware exponential and reciprocal: a few
            // 1e-7 relative from expf, far inside the tolerance of an fp16 attention
            auto sig = [](float g) { return __frcp_rn(1.f + fast_exp2(g * -1.4426950408889634f)); };
#pragma unroll
            for (int i = 0; i < kRowsPerWarp; ++i) {
                const int row = warp + i * (kSoftmaxThreads / 32);
                if (row >= rows) break;
                float* dst = !split ? a.o + flat_row(row) * kHeadDim
                             : a.part_o + (tail ? size_t(tail_unit) * kQRows + row : size_t(part) * a.T * a.n_q + flat_row(row)) * kHeadDim;
#pragma unroll
                for (int hcol = 0; hcol < 2; ++hcol) {
                    const int c = hcol * 128 + lane * 4;
                    float4 v = *reinterpret_cast<const float4*>(stage + row * kStageStride + c);
                    if (gated) {
                        v.x *= sig(gq[i][hcol].x);
                        v.y *= sig(gq[i][hcol].y);
                        v.z *= sig(gq[i][hcol].z);
                        v.w *= sig(gq[i][hcol].w);
                    }
                    __stcs(reinterpret_cast<float4*>(dst + c), v);
                }
            }
        }
        tc::fence_before_sync();
    }
    __syncthreads();
    if (warp == kWarpQK) tc::tmem_dealloc(tmem, kTmemCols);
}

// Rows of the items the main kernel divided (tail_parts > 1): block = (8 rows of the item, item - n_full), one
// warp per row, a lane 2 x 4 output dims.  Log-sum-exp merge of the item's partials, 1 / l and the sigmoid
// gate; every load of a row is requested before the first is used.
constexpr int kMergeRows = 8, kMergeMaxParts = 8;
__global__ void __launch_bounds__(kMergeRows * 32) attn_prefill_tail_merge_kernel(AttnPrefillArgs a) {
    griddep_launch();
    griddep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * kMergeRows + warp;
    const int n_qtiles = (a.T + kQRows - 1) / kQRows;
    int qt, hq;
    item_tile(a, a.n_full + int(blockIdx.y), n_qtiles, qt, hq);
    const int q0 = qt * kQRows;
    if (q0 + r >= a.T) return;
    const int parts = min(a.tail_parts, kMergeMaxParts);
    const size_t u0 = size_t(blockIdx.y) * a.tail_parts;
    const size_t oi = (size_t(q0 + r) * a.n_q + hq) * kHeadDim + lane * 4;
    float2 ml[kMergeMaxParts];
    float4 o0[kMergeMaxParts], o1[kMergeMaxParts];
    float4 g0 = make_float4(0.f, 0.f, 0.f, 0.f), g1 = g0;
#pragma unroll
    for (int p = 0; p < kMergeMaxParts; ++p) {
        if (p < parts) {
            const size_t row = (u0 + p) * kQRows + r;
            ml[p] = *reinterpret_cast<const float2*>(a.part_ml + row * 2);
            o0[p] = __ldcs(reinterpret_cast<const float4*>(a.part_o + row * kHeadDim + lane * 4));
            o1[p] = __ldcs(reinterpret_cast<const float4*>(a.part_o + row * kHeadDim + 128 + lane * 4));
        }
    }
    if (a.gate) {
        g0 = __ldcs(reinterpret_cast<const float4*>(a.gate + oi));
        g1 = __ldcs(reinterpret_cast<const float4*>(a.gate + oi + 128));
    }
    float mm = -1e30f;
#pragma unroll
    for (int p = 0; p < kMergeMaxParts; ++p)
        if (p < parts) mm = fmaxf(mm, ml[p].x);
    float l = 0.f;
    float4 x0 = make_float4(0.f, 0.f, 0.f, 0.f), x1 = x0;
#pragma unroll
    for (int p = 0; p < kMergeMaxParts; ++p) {
        if (p < parts) {
            const float al = expf(ml[p].x - mm);
            l += ml[p].y * al;
            x0.x += o0[p].x * al; x0.y += o0[p].y * al; x0.z += o0[p].z * al; x0.w += o0[p].w * al;
            x1.x += o1[p].x * al; x1.y += o1[p].y * al; x1.z += o1[p].z * al; x1.w += o1[p].w * al;
        }
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    auto fin = [&](float v, float g) { return a.gate ? v * inv * (1.f / (1.f + expf(-g))) : v * inv; };
    __stcs(reinterpret_cast<float4*>(a.o + oi), make_float4(fin(x0.x, g0.x), fin(x0.y, g0.y), fin(x0.z, g0.z), fin(x0.w, g0.w)));
    __stcs(reinterpret_cast<float4*>(a.o + oi + 128),
           make_float4(fin(x1.x, g1.x), fin(x1.y, g1.y), fin(x1.z, g1.z), fin(x1.w, g1.w)));
}

size_t attn_prefill_smem_bytes() { return sizeof(Smem) + 1024; }
int attn_prefill_threads() { return kThreads; }
int attn_prefill_q_rows() { return kQRows; }

}  // namespace rl
