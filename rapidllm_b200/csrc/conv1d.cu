// Depthwise causal conv1d (k taps, oldest first) + SiLU for the DeltaNet q/k/v
// channels: the decode form keeps a [dim][k] fp32 window per sequence
// (ops::conv1d_update, src/kernels/ops.cpp:458-468) and the prefill form walks
// a [seq][dim] block (ops::conv1d_causal_prefill, 443-456).
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace rl {

namespace {

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }

// k == 4: one channel per thread, window as one float4.
__global__ void __launch_bounds__(256) conv1d_update4_kernel(ConvUpdateArgs a) {
    griddep_launch();
    griddep_wait();       // x, the window and y's previous reader belong to earlier kernels
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= a.dim) return;
    const int slot = a.slot_ids ? a.slot_ids[b] : b;
    if (slot < 0 || slot >= a.n_slots) {
        set_err(a.err, DEV_ERR_BAD_SLOT);
        return;
    }
    float4* st = reinterpret_cast<float4*>(a.state + (size_t(slot) * a.dim + c) * 4);
    const float4 old = *st;
    const float4 w = *reinterpret_cast<const float4*>(a.w + size_t(c) * 4);
    const float4 nw = make_float4(old.y, old.z, old.w, a.x[size_t(b) * a.dim + c]);
    *st = nw;
    // double accumulator, taps in order, as the reference does
    double acc = double(w.x) * nw.x;
    acc += double(w.y) * nw.y;
    acc += double(w.z) * nw.z;
    acc += double(w.w) * nw.w;
    a.y[size_t(b) * a.dim + c] = silu(float(acc));
}

__global__ void __launch_bounds__(256) conv1d_update_generic_kernel(ConvUpdateArgs a) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int b = blockIdx.y;
    if (c >= a.dim) return;
    const int slot = a.slot_ids ? a.slot_ids[b] : b;
    if (slot < 0 || slot >= a.n_slots) {
        set_err(a.err, DEV_ERR_BAD_SLOT);
        return;
    }
    float* st = a.state + (size_t(slot) * a.dim + c) * a.k;
    double acc = 0.0;
    for (int p = 0; p < a.k - 1; ++p) {
        const float t = st[p + 1];
        st[p] = t;
        acc += double(a.w[size_t(c) * a.k + p]) * t;
    }
    const float xn = a.x[size_t(b) * a.dim + c];
    st[a.k - 1] = xn;
    acc += double(a.w[size_t(c) * a.k + a.k - 1]) * xn;
    a.y[size_t(b) * a.dim + c] = silu(float(acc));
}

// Prefill: thread = channel, walks a tile of time steps with the window in
// registers (k <= 8).  grid (ceil(dim/256), ceil(seq/tile)).
constexpr int kMaxTaps = 8;
__global__ void __launch_bounds__(256)
conv1d_prefill_kernel(const float* x, const float* w, float* y, const float* state_in, int seq,
                      int dim, int k, int tile) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= dim) return;
    const int t0 = blockIdx.y * tile;
    const int t1 = min(seq, t0 + tile);
    float win[kMaxTaps], wt[kMaxTaps];
    for (int p = 0; p < k; ++p) wt[p] = w[size_t(c) * k + p];
    // window before t0: inputs t0-k+1 .. t0-1 (index p = 0..k-2), from x, state_in or zero
    for (int p = 0; p < k - 1; ++p) {
        const int src = t0 - (k - 1) + p;
        float v = 0.f;
        if (src >= 0) v = x[size_t(src) * dim + c];
        else if (state_in) v = state_in[size_t(c) * k + (k + src)];   // src = -1 -> newest tap k-1
        win[p + 1] = v;
    }
    for (int t = t0; t < t1; ++t) {
        for (int p = 0; p < k - 1; ++p) win[p] = win[p + 1];
        win[k - 1] = x[size_t(t) * dim + c];
        double acc = 0.0;
        for (int p = 0; p < k; ++p) acc += double(wt[p]) * win[p];
        y[size_t(t) * dim + c] = silu(float(acc));
    }
}

// The same for k = 4 and an even dim: thread = 2 adjacent channels x 8 time steps, every input of the
// tile requested before the first is used (the walk above has one load in flight per thread and is bound
// by their latency); small enough per thread that three CTAs fit an SM (the fp64 copies of the inputs are
// what costs registers).  Taps are accumulated in the same order and width.
constexpr int kVecSteps = 8;
__global__ void __launch_bounds__(256, 3)
conv1d_prefill4_kernel(const float* x, const float* w, float* y, const float* state_in, float* state_out, int seq,
                       int dim) {
    griddep_launch();
    griddep_wait();
    const int c = (blockIdx.x * 256 + threadIdx.x) * 2;
    if (c >= dim) return;
    const int t0 = blockIdx.y * kVecSteps;
    float2 in[kVecSteps + 3];
#pragma unroll
    for (int i = 0; i < kVecSteps + 3; ++i) {
        const int src = t0 - 3 + i;
        float2 v = make_float2(0.f, 0.f);
        if (src >= 0) {
            if (src < seq) v = *reinterpret_cast<const float2*>(x + size_t(src) * dim + c);
        } else if (state_in) {
            // src = -1 is the newest tap (index 3) of each channel's window
            const float* sp = state_in + size_t(c) * 4 + (4 + src);
            v = make_float2(sp[0], sp[4]);
        }
        in[i] = v;
    }
    const float4 w0 = *reinterpret_cast<const float4*>(w + size_t(c) * 4);
    const float4 w1 = *reinterpret_cast<const float4*>(w + size_t(c + 1) * 4);
    if (state_out && blockIdx.y == 0) {
        // seq >= 4: the window after the call is the last four inputs.  The thread that read this channel
        // pair's old window (above, first tile) is the one that replaces it.
        float2 last[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) last[p] = *reinterpret_cast<const float2*>(x + size_t(seq - 4 + p) * dim + c);
        *reinterpret_cast<float4*>(state_out + size_t(c) * 4) = make_float4(last[0].x, last[1].x, last[2].x, last[3].x);
        *reinterpret_cast<float4*>(state_out + size_t(c + 1) * 4) = make_float4(last[0].y, last[1].y, last[2].y, last[3].y);
    }
#pragma unroll
    for (int i = 0; i < kVecSteps; ++i) {
        if (t0 + i >= seq) break;
        auto one = [&](const float4& wj, float a0, float a1, float a2, float a3) {
            double acc = 0.0;
            acc += double(wj.x) * a0;
            acc += double(wj.y) * a1;
            acc += double(wj.z) * a2;
            acc += double(wj.w) * a3;
            // hardware exponential and reciprocal: a few 1e-7 relative from expf and a true division, far inside the
            // 2e-6 the operator is checked to, and a quarter of the instructions of a kernel that is otherwise issue-bound
            const float x = float(acc);
            return __fdividef(x, 1.f + __expf(-x));
        };
        *reinterpret_cast<float2*>(y + size_t(t0 + i) * dim + c) =
            make_float2(one(w0, in[i].x, in[i + 1].x, in[i + 2].x, in[i + 3].x),
                        one(w1, in[i].y, in[i + 1].y, in[i + 2].y, in[i + 3].y));
    }
}

__global__ void __launch_bounds__(256)
conv1d_state_tail_kernel(const float* x, float* state_io, int seq, int dim, int k, int use_state_in) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= dim) return;
    float old[kMaxTaps];
    for (int p = 0; p < k; ++p) old[p] = use_state_in ? state_io[size_t(c) * k + p] : 0.f;
    for (int p = 0; p < k; ++p) {
        const int src = seq - k + p;   // input index that ends at tap p
        state_io[size_t(c) * k + p] = src >= 0 ? x[size_t(src) * dim + c] : old[p + seq < k ? p + seq : k - 1];
    }
}

}  // namespace

void launch_conv1d_update(const ConvUpdateArgs& a, cudaStream_t st) {
    if (a.batch <= 0 || a.dim <= 0) return;
    dim3 grid((a.dim + 255) / 256, a.batch);
    if (a.k == 4) launch_step(conv1d_update4_kernel, grid, dim3(256), 0, st, a);
    else conv1d_update_generic_kernel<<<grid, 256, 0, st>>>(a);
}

void launch_conv1d_prefill(const float* x, const float* w, float* y, float* state_io, int seq,
                           int dim, int k, int use_state_in, cudaStream_t st) {
    if (seq <= 0 || dim <= 0) return;
    const float* state_in = (use_state_in && state_io) ? state_io : nullptr;
    const bool vec = k == 4 && dim % 2 == 0 && reinterpret_cast<uintptr_t>(x) % 8 == 0 &&
                     reinterpret_cast<uintptr_t>(y) % 8 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
    if (vec) {
        const bool tail_fused = state_io && seq >= 4 && reinterpret_cast<uintptr_t>(state_io) % 16 == 0;
        launch_step(conv1d_prefill4_kernel, dim3((dim / 2 + 255) / 256, (seq + kVecSteps - 1) / kVecSteps), dim3(256), 0, st,
                    x, w, y, state_in, tail_fused ? state_io : nullptr, seq, dim);
        if (tail_fused) return;
    } else {
        const int tile = 64;
        conv1d_prefill_kernel<<<dim3((dim + 255) / 256, (seq + tile - 1) / tile), 256, 0, st>>>(x, w, y, state_in, seq, dim,
                                                                                             k, tile);
    }
    if (state_io)
        conv1d_state_tail_kernel<<<(dim + 255) / 256, 256, 0, st>>>(x, state_io, seq, dim, k, use_state_in);
}

}  // namespace rl
