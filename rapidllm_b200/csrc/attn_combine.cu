// Log-sum-exp merge of split-KV partials, fused with the sigmoid output gate.
//
// Generalises the reference's merge of its 8 warp partials
// (src/kernels/cuda/cuda_engine.cu:347-374) to grid-level chunks and, through
// lse_combine_kernel, to partials gathered from other GPUs.  The gate is
// o *= sigmoid(gate) (src/kernels/ops_fused.cpp:178, cuda_engine.cu:6229-6232).
#include "common.cuh"
#include "kernels.h"

namespace rl {

namespace {

// Orthonormal Walsh-Hadamard transform of the 256 values held one per thread (blocks of
// wht_len = 128 or 256), same stage order as the store kernel; then the +-1 signs.
__device__ __forceinline__ float block_wht(float v, int wht_len, const float* signs, float* xs) {
    const int tid = threadIdx.x, lane = tid & 31;
    v = wht32_in_warp(v, lane);
    xs[tid] = v;
    __syncthreads();
    for (int s = 32; s < wht_len; s <<= 1) {
        const int j = tid ^ s;
        const float x0 = xs[tid], x1 = xs[j];
        __syncthreads();
        xs[tid] = (tid < j) ? (x0 + x1) : (x1 - x0);
        __syncthreads();
    }
    v = xs[tid] * (wht_len == 128 ? 0.08838834764831845f : 0.0625f);
    if (signs) v *= signs[tid];
    return v;
}

}  // namespace

__global__ void __launch_bounds__(256) attn_combine_kernel(AttnCombineArgs a) {
    griddep_launch();
    const int hq = blockIdx.x;
    const int b = blockIdx.y;
    const int G = a.n_q / a.n_kv;
    const int h = hq / G, gi = hq - h * G;
    const int d = threadIdx.x;
    __shared__ int red[2][8];
    __shared__ float xs[256];
    // half pages of the sequences before b, and of all sequences (the unit list of attn_split.cuh)
    int before = 0, total = 0;
    for (int bb = d; bb < a.batch; bb += 256) {
        int len = a.seq_lens[bb] + a.len_add;
        if (len < 0 || len > a.max_len) len = 0;
        const int n = (len + 31) >> 5;
        total += n;
        if (bb < b) before += n;
    }
    for (int off = 16; off > 0; off >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, off);
        total += __shfl_xor_sync(0xffffffffu, total, off);
    }
    if ((d & 31) == 0) {
        red[0][d >> 5] = before;
        red[1][d >> 5] = total;
    }
    __syncthreads();
    before = total = 0;
    for (int w = 0; w < 8; ++w) {
        before += red[0][w];
        total += red[1][w];
    }
    int len = a.seq_lens[b] + a.len_add;
    if (len < 0 || len > a.max_len) len = 0;
    const int hpb = (len + 31) >> 5;
    // this head's units are [u0, u0 + hpb); CTA k of the decode kernel owned [k*q, (k+1)*q)
    const int u0 = before * a.n_kv + h * hpb;
    // (equal in cost when seg_weight > 0: unit u of segment sg sits at cost position u + seg_weight * sg)
    const int c0 = u0 + a.seg_weight * (b * a.n_kv + h);
    const int q = max(1, (total * a.n_kv + a.seg_weight * a.batch * a.n_kv + a.n_ctas - 1) / a.n_ctas);
    const int k0 = c0 / q;
    const int k1 = hpb > 0 ? (c0 + hpb - 1) / q : k0 - 1;
    const size_t unit = size_t(b) * a.n_kv + h;
    // Up to here only the sequence lengths were read, which the step's kernels never write: which CTAs hold
    // this head's partials is worked out beside the tail of the decode kernel.  The partials need it finished.
    griddep_wait();

    // A long sequence at a small batch is spread over many CTAs: fetch all their (m, l) pairs at
    // once (one per thread), reduce the maximum across the block, keep the weights in shared
    // memory and let the accumulation loop run with several independent loads in flight.
    const int n = k1 - k0 + 1;
    float mm = -1e30f, acc = 0.f, l = 0.f;
    if (n <= 256) {
        __shared__ float s_w[256];
        __shared__ float s_red[2][8];
        float my_m = -1e30f, my_l = 0.f;
        if (d < n) {
            const size_t row = (k0 + d + unit) * G + gi;
            my_m = a.part_ml[row * 2];
            my_l = a.part_ml[row * 2 + 1];
        }
        float wm = my_m;
        for (int off = 16; off > 0; off >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, off));
        if ((d & 31) == 0) s_red[0][d >> 5] = wm;
        __syncthreads();
        for (int w = 0; w < 8; ++w) mm = fmaxf(mm, s_red[0][w]);
        const float al = d < n ? expf(my_m - mm) : 0.f;
        s_w[d] = al;
        float wl = my_l * al;
        for (int off = 16; off > 0; off >>= 1) wl += __shfl_xor_sync(0xffffffffu, wl, off);
        if ((d & 31) == 0) s_red[1][d >> 5] = wl;
        __syncthreads();
        for (int w = 0; w < 8; ++w) l += s_red[1][w];
        const float* po = a.part_o + ((k0 + unit) * G + gi) * kHeadDim + d;
        const size_t stride = size_t(G) * kHeadDim;       // next CTA's slot of this head
#pragma unroll 8
        for (int i = 0; i < n; ++i) acc += po[i * stride] * s_w[i];
    } else {
        for (int k = k0; k <= k1; ++k) mm = fmaxf(mm, a.part_ml[((k + unit) * G + gi) * 2]);
        for (int k = k0; k <= k1; ++k) {
            const size_t row = (k + unit) * G + gi;
            const float al = expf(a.part_ml[row * 2] - mm);
            l += a.part_ml[row * 2 + 1] * al;
            acc += a.part_o[row * kHeadDim + d] * al;
        }
    }
    const size_t oi = (size_t(b) * a.n_q + hq) * kHeadDim + d;
    if (a.out_ml) {
        a.o[oi] = acc;
        if (d == 0) {
            a.out_ml[(size_t(b) * a.n_q + hq) * 2] = mm;
            a.out_ml[(size_t(b) * a.n_q + hq) * 2 + 1] = l;
        }
        return;
    }
    float out = l > 0.f ? acc / l : 0.f;
    if (a.wht_len) out = block_wht(out, a.wht_len, a.signs, xs);
    if (a.gate) out *= 1.f / (1.f + expf(-a.gate[oi]));
    a.o[oi] = out;
}

__global__ void __launch_bounds__(256)
lse_combine_kernel(const float* part_o, const float* part_ml, const float* gate, float* o,
                   int n_parts, int rows, int wht_len, const float* signs) {
    __shared__ float xs[256];
    const int row = blockIdx.x;
    const int d = threadIdx.x;
    float mm = -1e30f;
    for (int p = 0; p < n_parts; ++p) mm = fmaxf(mm, part_ml[(size_t(p) * rows + row) * 2]);
    float acc = 0.f, l = 0.f;
    for (int p = 0; p < n_parts; ++p) {
        const size_t r = size_t(p) * rows + row;
        const float al = expf(part_ml[r * 2] - mm);
        l += part_ml[r * 2 + 1] * al;
        acc += part_o[r * kHeadDim + d] * al;
    }
    float out = l > 0.f ? acc / l : 0.f;
    if (wht_len) out = block_wht(out, wht_len, signs, xs);
    const size_t oi = size_t(row) * kHeadDim + d;
    if (gate) out *= 1.f / (1.f + expf(-gate[oi]));
    o[oi] = out;
}

}  // namespace rl
