// Pieces shared by the split-KV decode kernels (F16 and compact KV): the division of
// the work among the persistent CTAs, and the fixed-order merge of the consumer warps
// of a CTA.
#pragma once
#include "common.cuh"

namespace rl {
namespace split {

constexpr int kMaxBatch = 1024;
constexpr float kNegBig = -1e30f;
constexpr int kMergeStride = kHeadDim + 1;   // row stride 257 floats: conflict-free

// NW = consumer warps of the kernel (6..8); the merge tree needs NW - 4 buffers
template <int NW>
struct Shared {
    static_assert(NW >= 6 && NW <= 8, "merge tree written for 6..8 consumer warps");
    float o[NW - 4][8][kMergeStride];   // segment merge buffers
    float m[NW][8];
    float l[NW][8];
    int prefix[kMaxBatch + 1];          // half pages (32 tokens) before sequence b, per KV head
};

// The work of a launch is the list of all (sequence b, KV head h, half page hp) units in the
// order b, h, hp.  CTA k of a grid of n CTAs owns the contiguous units [k*Q, (k+1)*Q), Q =
// ceil(total / n): equal work per CTA, and a CTA streams consecutive half pages of one head.
// A CTA's range is cut into segments at (b, h) boundaries; each segment yields one partial
// (unnormalised output, max, sum) in workspace slot k + (b * n_kv + h).  Along the unit list
// either k or the (b, h) index grows from one segment to the next, so the slots are distinct
// and there are fewer than n + batch * n_kv of them.
struct Segment {
    int b, h;
    int hp0, hp1;                   // half pages [hp0, hp1) of sequence b
    int len;                        // tokens of sequence b
};

__device__ __forceinline__ int half_pages(int len) { return (len + 31) >> 5; }

// Warp 0 fills s.prefix; lengths outside [0, max_pages_per_seq * 64] count as 0 and are reported.
template <int NW>
__device__ __forceinline__ void build_prefix(Shared<NW>& s, const int32_t* seq_lens, int len_add, int batch,
                                             int max_pages_per_seq, int* err, int lane) {
    int run = 0;
    for (int b0 = 0; b0 < batch; b0 += 32) {
        const int b = b0 + lane;
        int n = 0;
        if (b < batch) {
            int len = seq_lens[b] + len_add;
            if (len < 0 || len > max_pages_per_seq * kPageTokens) {
                set_err(err, DEV_ERR_BAD_LEN);
                len = 0;
            }
            n = half_pages(len);
        }
        int inc = n;
        for (int off = 1; off < 32; off <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, inc, off);
            if (lane >= off) inc += t;
        }
        if (b < batch) s.prefix[b] = run + inc - n;
        run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) s.prefix[batch] = run;
}

// Units in front of cost position c when every (b, h) segment sg = b * n_kv + h is charged
// `seg_weight` extra positions in front of its own units (cost of unit u of segment sg = u +
// seg_weight * sg).
template <int NW>
__device__ __forceinline__ int units_below_cost(const Shared<NW>& s, int c, int batch, int n_kv, int seg_weight) {
    auto seg_units0 = [&](int sg, int& hpb) {
        const int b = sg / n_kv, h = sg - b * n_kv;
        hpb = s.prefix[b + 1] - s.prefix[b];
        return s.prefix[b] * n_kv + h * hpb;
    };
    int lo = 0, hi = batch * n_kv, hpb;       // largest segment whose cost range starts at or before c
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (seg_units0(mid, hpb) + seg_weight * mid <= c) lo = mid; else hi = mid;
    }
    const int u0 = seg_units0(lo, hpb);
    return u0 + min(max(c - (u0 + seg_weight * lo), 0), hpb);
}

// seg_weight = 0: CTA k owns units [k*Q, (k+1)*Q), Q = ceil(total / n).  seg_weight > 0: a CTA
// whose range runs over a (b, h) boundary closes one segment and opens the next (a merge, a new
// query), which costs it about as long as streaming seg_weight units; the division is equal in
// cost instead: CTA k owns the units whose cost position lies in [k*Qc, (k+1)*Qc), Qc =
// ceil((total + seg_weight * batch * n_kv) / n).  attn_combine_kernel inverts the same formula.
template <int NW>
__device__ __forceinline__ void cta_range(const Shared<NW>& s, int batch, int n_kv, int& begin, int& end,
                                          int seg_weight = 0) {
    const int total = s.prefix[batch] * n_kv;
    if (seg_weight > 0) {
        const int qc = max(1, (total + seg_weight * batch * n_kv + int(gridDim.x) - 1) / int(gridDim.x));
        begin = units_below_cost(s, int(blockIdx.x) * qc, batch, n_kv, seg_weight);
        end = units_below_cost(s, (int(blockIdx.x) + 1) * qc, batch, n_kv, seg_weight);
        return;
    }
    const int q = (total + int(gridDim.x) - 1) / int(gridDim.x);
    begin = min(int(blockIdx.x) * q, total);
    end = min(begin + q, total);
}

// The segment that starts at unit `pos` (pos < end <= total).
template <int NW>
__device__ __forceinline__ Segment segment_at(const Shared<NW>& s, int pos, int end, int batch, int n_kv,
                                              const int32_t* seq_lens, int len_add) {
    Segment g;
    int lo = 0, hi = batch;         // largest b with prefix[b] * n_kv <= pos
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s.prefix[mid] * n_kv <= pos) lo = mid; else hi = mid;
    }
    g.b = lo;
    const int hpb = s.prefix[lo + 1] - s.prefix[lo];
    const int rem = pos - s.prefix[lo] * n_kv;
    g.h = rem / hpb;
    g.hp0 = rem - g.h * hpb;
    g.hp1 = min(hpb, g.hp0 + (end - pos));
    g.len = seq_lens[lo] + len_add;
    return g;
}

// Merge the consumer warps' partial results of one segment and write its partial to `slot`.
// acc[j][i][0..3] of lane (g, c) holds dims d = 64j + 8*dsel + 2i (+1 for [2],[3]) of heads
// 2c ([0],[2]) and 2c+1 ([1],[3]); m_run is the running maximum (log2 domain) of head g and
// l_run this lane's share of the row sum.  All consumer threads must call this.
template <int NW>
__device__ __forceinline__ void merge_segment(Shared<NW>& s, float (&acc)[4][4][4], float m_run, float l_run,
                                              int warp, int lane, int dsel, int G, float* part_o,
                                              float* part_ml, size_t item) {
    constexpr int kThreads = NW * 32;
    const int g = lane >> 2, c = lane & 3;
    const int tid = warp * 32 + lane;
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    if (c == 0) {
        s.m[warp][g] = m_run;
        s.l[warp][g] = l_run;
    }
    named_bar_sync(1, kThreads);
    {   // scale this warp's accumulators to the segment-wide maximum
        float f[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float mm = kNegBig;
#pragma unroll
            for (int ww = 0; ww < NW; ++ww) mm = fmaxf(mm, s.m[ww][2 * c + e]);
            f[e] = fast_exp2(s.m[warp][2 * c + e] - mm);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[j][i][0] *= f[0];
                acc[j][i][2] *= f[0];
                acc[j][i][1] *= f[1];
                acc[j][i][3] *= f[1];
            }
    }
    // Fixed-order binary tree (bit-reproducible, unlike atomics): at stride 4, 2, 1 the warps
    // [stride, 2 stride) store their accumulators and the warps below add them.  Lanes with
    // dsel >= 4 touch the odd dim first so a warp's 32 accesses hit 32 banks.
    const int odd = dsel >> 2;
    auto put = [&](float (*buf)[kMergeStride]) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = 64 * j + 8 * dsel + 2 * i;
                buf[2 * c][d + odd] = odd ? acc[j][i][2] : acc[j][i][0];
                buf[2 * c][d + 1 - odd] = odd ? acc[j][i][0] : acc[j][i][2];
                buf[2 * c + 1][d + odd] = odd ? acc[j][i][3] : acc[j][i][1];
                buf[2 * c + 1][d + 1 - odd] = odd ? acc[j][i][1] : acc[j][i][3];
            }
    };
    auto add = [&](const float (*buf)[kMergeStride]) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int d = 64 * j + 8 * dsel + 2 * i;
                const float x0 = buf[2 * c][d + odd], x1 = buf[2 * c][d + 1 - odd];
                const float y0 = buf[2 * c + 1][d + odd], y1 = buf[2 * c + 1][d + 1 - odd];
                acc[j][i][0] += odd ? x1 : x0;
                acc[j][i][2] += odd ? x0 : x1;
                acc[j][i][1] += odd ? y1 : y0;
                acc[j][i][3] += odd ? y0 : y1;
            }
    };
#pragma unroll
    for (int stride = 4; stride >= 1; stride >>= 1) {
        if (warp >= stride && warp < 2 * stride) put(s.o[warp - stride]);
        named_bar_sync(1, kThreads);
        if (warp < stride && warp + stride < NW) add(s.o[warp]);
        named_bar_sync(1, kThreads);
    }
    if (warp == 0) put(s.o[0]);
    named_bar_sync(1, kThreads);
    float* po = part_o + item * G * kHeadDim;
    for (int x = tid; x < G * kHeadDim; x += kThreads) po[x] = s.o[0][x >> 8][x & (kHeadDim - 1)];
    if (tid < G) {
        float mm = kNegBig;
        for (int ww = 0; ww < NW; ++ww) mm = fmaxf(mm, s.m[ww][tid]);
        float ll = 0.f;
        for (int ww = 0; ww < NW; ++ww) ll += s.l[ww][tid] * fast_exp2(s.m[ww][tid] - mm);
        part_ml[(item * G + tid) * 2 + 0] = mm * 0.6931471805599453f;   // natural-log units
        part_ml[(item * G + tid) * 2 + 1] = ll;
    }
    named_bar_sync(1, kThreads);
}

}  // namespace split
}  // namespace rl
