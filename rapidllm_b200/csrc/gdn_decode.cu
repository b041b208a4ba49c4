// Fused Gated DeltaNet decode step (sm_100a): causal conv window + SiLU, l2 norms and the delta
// rule in one kernel per layer -- what the reference's gdn_decode_t1_k does in one launch
// (src/kernels/cuda/cuda_engine.cu:5166-5286), with the arithmetic of its CPU operators:
// ops::conv1d_update (src/kernels/ops.cpp:458-468: taps oldest first, double accumulator, SiLU),
// ops::l2norm (158-163) and ops::delta_recurrent_step (495-540), FP32 state in HBM.
//
// Value head h needs the conv outputs of its own 128 v channels and of the 128 q and 128 k
// channels of its key head, which up to n_v / n_qk value heads share.  So that any number of
// CTAs can use a key head's channels in the same step, the windows are rings: tap slot (t & 3)
// holds input x_t and nothing is ever shifted.  A step reads the three older taps (no one
// writes them during the step), takes the newest input from x, and one designated head per key
// head stores x into slot `phase`; the phase moves on after the step (gdn_phase_advance_kernel).
//
// Two forms, as for the unfused delta rule (delta_decode.cu): with at least four heads per SM,
// persistent CTAs stream whole 64 KiB heads through a 3-stage TMA ring while three further warps
// run the conv + norms of the 384 channels of the items ahead and hand q, k, v over through
// shared memory; otherwise one CTA per 32-column slice of a head with the slice in registers.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace rl {

namespace {

constexpr int kDk = 128, kDv = 128;
constexpr int kTaps = 4;

__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }

// value head -> key/query head, and whether h is the head that stores its key head's new taps
__device__ __forceinline__ int key_head_of(int h, int n_v, int n_qk, int head_map) {
    return head_map == 0 ? h : (head_map == 1 ? h / (n_v / n_qk) : h % n_qk);
}
__device__ __forceinline__ bool stores_key_taps(int h, int n_v, int n_qk, int head_map) {
    return head_map == 0 ? true : (head_map == 1 ? h % (n_v / n_qk) == 0 : h < n_qk);
}

// Inputs of the conv of 4 consecutive channels, fetched one item ahead of their use.
struct ConvIn {
    float4 win[4];
    float4 w[4];
    float4 x;
    int ph;
};

__device__ __forceinline__ void conv_fetch(ConvIn& in, const GdnDecodeArgs& a, int b, int slot, int c0) {
    const float4* wp = reinterpret_cast<const float4*>(a.w) + c0;
    const float4* sp = reinterpret_cast<const float4*>(a.conv) + size_t(slot) * a.conv_dim + c0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        in.win[i] = sp[i];
        in.w[i] = wp[i];
    }
    in.x = *reinterpret_cast<const float4*>(a.x + size_t(b) * a.conv_dim + c0);
    in.ph = a.conv_phase[slot] & 3;
}

// One channel: the ring holds x_{t-3..t-1} in slots (ph+1, ph+2, ph+3) & 3; y = silu(sum_p w_p tap_p)
// with the accumulation order and width of ops::conv1d_update.
__device__ __forceinline__ float conv_one(const float4 win, const float4 w, float xn, int ph) {
    // rotate so that r.y, r.z, r.w are the three older taps in age order
    float4 r = win;
    if (ph & 1) r = make_float4(r.y, r.z, r.w, r.x);
    if (ph & 2) r = make_float4(r.z, r.w, r.x, r.y);
    double acc = double(w.x) * r.y;
    acc += double(w.y) * r.z;
    acc += double(w.z) * r.w;
    acc += double(w.w) * xn;
    return silu(float(acc));
}

__device__ __forceinline__ float4 conv_four(const ConvIn& in) {
    return make_float4(conv_one(in.win[0], in.w[0], in.x.x, in.ph), conv_one(in.win[1], in.w[1], in.x.y, in.ph),
                       conv_one(in.win[2], in.w[2], in.x.z, in.ph), conv_one(in.win[3], in.w[3], in.x.w, in.ph));
}

__device__ __forceinline__ void conv_store_taps(const ConvIn& in, const GdnDecodeArgs& a, int slot, int c0) {
    float* sp = a.conv + (size_t(slot) * a.conv_dim + c0) * kTaps + in.ph;
    sp[0] = in.x.x;
    sp[kTaps] = in.x.y;
    sp[2 * kTaps] = in.x.z;
    sp[3 * kTaps] = in.x.w;
}

// l2 norm over the 128 values a warp holds 4 per lane (double accumulator as ops::l2norm)
__device__ __forceinline__ float4 l2norm_warp(float4 y, float eps, float extra) {
    double ss = double(y.x) * y.x + double(y.y) * y.y + double(y.z) * y.z + double(y.w) * y.w;
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = 1.f / sqrtf(float(ss) + eps) * extra;
    return make_float4(y.x * inv, y.y * inv, y.z * inv, y.w * inv);
}

// first channel of the 4 this lane convolves: warp 0 = q, 1 = k of key head hs, 2 = v of head h
__device__ __forceinline__ int conv_channel0(int role, int hs, int h, int n_qk, int lane) {
    const int base = role == 0 ? hs * kDk : (role == 1 ? (n_qk + hs) * kDk : 2 * n_qk * kDk + h * kDv);
    return base + lane * 4;
}

// ------------------------------------------------------------------------------------------------
constexpr int kStreamStages = 3;
constexpr int kStreamThreads = 384;            // 8 consumer warps + TMA producer warp + 3 conv warps
constexpr int kHeadBytes = kDk * kDv * 4;      // 64 KiB
constexpr int kWarpProducer = 8, kWarpConv0 = 9;

struct StreamSmem {
    alignas(128) float S[kStreamStages][kDk * kDv];
    float q[2][kDk], k[2][kDk], v[2][kDv];
    float red[8][kDv], red2[8][kDv];
    uint64_t full[kStreamStages], empty[kStreamStages];
    uint64_t vec_ready[2], vec_free[2];        // q, k, v of an item: written by the conv warps, read by the consumers
};

__global__ void __launch_bounds__(kStreamThreads, 1) gdn_decode_stream_kernel(GdnDecodeArgs a) {
    extern __shared__ unsigned char smem_raw[];
    StreamSmem& s = *reinterpret_cast<StreamSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_items = a.batch * a.n_v;
    if (tid == 0) {
        for (int i = 0; i < kStreamStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s.vec_ready[i], 3);     // one arrival per conv warp
            mbar_init(&s.vec_free[i], 1);
        }
        mbar_fence_init();
    }
    griddep_launch();
    __syncthreads();
    // The producer warp only reads this layer's state, which no kernel since this layer's previous step has
    // written (the kernel in front belongs to another layer, or to the end of the previous step), so its first
    // copies are on their way while that kernel finishes.  Everything else -- the step's inputs, the conv
    // rings, every write -- waits for the kernel in front.
    if (warp != kWarpProducer && !a.early) griddep_wait();
    auto slot_of = [&](int b) {
        int slot = a.slot_ids ? a.slot_ids[b] : b;
        if (slot < 0 || slot >= a.n_slots) {
            set_err(a.err, DEV_ERR_BAD_SLOT);
            slot = -1;
        }
        return slot;
    };

    if (warp == kWarpProducer) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
                const int st = it % kStreamStages;
                if (!mbar_wait(&s.empty[st], ((it / kStreamStages) & 1) ^ 1)) {
                    set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                    break;
                }
                const int b = item / a.n_v, h = item - b * a.n_v;
                const int slot = slot_of(b);
                const float* src = a.S + (size_t(slot < 0 ? 0 : slot) * a.n_v + h) * (kDk * kDv);
                mbar_arrive_expect_tx(&s.full[st], kHeadBytes);
                bulk_g2s(s.S[st], src, kHeadBytes, &s.full[st]);
            }
        }
        if (a.early) griddep_wait();
        return;
    }
    if (warp >= kWarpConv0) {
        // ------------------------------ conv warps: q, k, v of the items, one item ahead ------------------------------
        const int role = warp - kWarpConv0;    // 0 = q, 1 = k (key head's channels), 2 = v (this head's channels)
        ConvIn cin;
        auto fetch = [&](int item) {
            if (item < n_items) {
                const int b = item / a.n_v, h = item - b * a.n_v;
                const int slot = slot_of(b);
                conv_fetch(cin, a, b, slot < 0 ? 0 : slot,
                           conv_channel0(role, key_head_of(h, a.n_v, a.n_qk, a.head_map), h, a.n_qk, lane));
            }
        };
        fetch(blockIdx.x);
        uint32_t it = 0;
        for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
            const int buf = it & 1;
            const int b = item / a.n_v, h = item - b * a.n_v;
            const int hs = key_head_of(h, a.n_v, a.n_qk, a.head_map);
            const int slot = slot_of(b);
            float4 y = conv_four(cin);
            if (slot >= 0 && (role == 2 || stores_key_taps(h, a.n_v, a.n_qk, a.head_map)))
                conv_store_taps(cin, a, slot, conv_channel0(role, hs, h, a.n_qk, lane));
            fetch(item + gridDim.x);           // the next item's inputs are on their way while this one is finished
            if (role == 0) y = l2norm_warp(y, a.eps_l2, 1.f / sqrtf(float(kDk)));
            if (role == 1) y = l2norm_warp(y, a.eps_l2, 1.f);
            // the buffer was last read for item it - 2
            if (it >= 2 && !mbar_wait(&s.vec_free[buf], ((it - 2) >> 1) & 1)) {
                set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
                break;
            }
            float* dst = role == 0 ? s.q[buf] : (role == 1 ? s.k[buf] : s.v[buf]);
            *reinterpret_cast<float4*>(dst + lane * 4) = y;
            __syncwarp();
            if (lane == 0) mbar_arrive(&s.vec_ready[buf]);
        }
        if (a.early) griddep_wait();
        return;
    }
    // ------------------------------ consumers ------------------------------
    const int cg = tid & 31;                  // columns 4cg .. 4cg+3
    const int rg = tid >> 5;                  // rows 16rg .. 16rg+15 (= warp)
    uint32_t it = 0;
    bool alive = true;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
        const int st = it % kStreamStages, buf = it & 1;
        const int b = item / a.n_v, h = item - b * a.n_v;
        const int slot = slot_of(b);
        const float g = expf(a.g_log[size_t(b) * a.n_v + h]);
        const float beta = a.beta[size_t(b) * a.n_v + h];
        if (alive && !mbar_wait(&s.vec_ready[buf], (it >> 1) & 1)) {
            set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
            alive = false;
        }
        if (alive && !mbar_wait(&s.full[st], (it / kStreamStages) & 1)) {
            set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
            alive = false;
        }
        const float4 vv = *reinterpret_cast<const float4*>(&s.v[buf][cg * 4]);
        const float* Sp = s.S[st];
        float* Sg = a.S + (size_t(slot < 0 ? 0 : slot) * a.n_v + h) * (kDk * kDv);
        const float* kq = s.k[buf];
        const float* qq = s.q[buf];
        // pass 1: kv = (g S)^T k over this warp's 16 rows
        float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (alive) {
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int i = 16 * rg + r;
                const float4 x = *reinterpret_cast<const float4*>(Sp + i * kDv + cg * 4);
                const float ki = kq[i] * g;
                kv.x += x.x * ki; kv.y += x.y * ki; kv.z += x.z * ki; kv.w += x.w * ki;
            }
        }
        *reinterpret_cast<float4*>(&s.red[rg][cg * 4]) = kv;
        named_bar_sync(1, 256);
        float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 t = *reinterpret_cast<const float4*>(&s.red[w][cg * 4]);
            tot.x += t.x; tot.y += t.y; tot.z += t.z; tot.w += t.w;
        }
        const float4 dl = make_float4((vv.x - tot.x) * beta, (vv.y - tot.y) * beta, (vv.z - tot.z) * beta,
                                      (vv.w - tot.w) * beta);
        // pass 2: S = g S + k (x) delta written back to HBM, o = S^T q
        float4 oo = make_float4(0.f, 0.f, 0.f, 0.f);
        if (alive) {
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int i = 16 * rg + r;
                float4 x = *reinterpret_cast<const float4*>(Sp + i * kDv + cg * 4);
                const float ki = kq[i], qi = qq[i];
                x.x = x.x * g + ki * dl.x; x.y = x.y * g + ki * dl.y; x.z = x.z * g + ki * dl.z; x.w = x.w * g + ki * dl.w;
                oo.x += x.x * qi; oo.y += x.y * qi; oo.z += x.z * qi; oo.w += x.w * qi;
                if (slot >= 0) __stcs(reinterpret_cast<float4*>(Sg + i * kDv + cg * 4), x);
            }
        }
        *reinterpret_cast<float4*>(&s.red2[rg][cg * 4]) = oo;
        named_bar_sync(1, 256);               // every thread is done reading this stage and this item's q, k, v
        if (tid < kDv) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += s.red2[w][tid];
            if (slot >= 0) a.o[(size_t(b) * a.n_v + h) * kDv + tid] = t;
        }
        if (tid == 0) {
            mbar_arrive(&s.empty[st]);
            mbar_arrive(&s.vec_free[buf]);
        }
    }
    if (a.early) griddep_wait();      // completes after the kernel in front, as every kernel of a step does
}

// ------------------------------------------------------------------------------------------------
// Few heads: one CTA per (32-column slice, head, sequence); the slice stays in registers between the
// two passes.  Every slice CTA runs the q and k conv of its key head itself (the ring makes that
// safe); slice 0 of the designated head stores the q/k taps, every slice its own v taps.
constexpr int kSliceCols = 32;
constexpr int kSlices = kDv / kSliceCols;   // 4

__global__ void __launch_bounds__(256) gdn_decode_kernel(GdnDecodeArgs a) {
    griddep_launch();
    const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __shared__ float sq[kDk], sk[kDk], sv[kSliceCols];
    __shared__ float red[8][kSliceCols];
    __shared__ float red2[8][kSliceCols];

    const int slot = a.slot_ids ? a.slot_ids[b] : b;
    if (slot < 0 || slot >= a.n_slots) {
        if (tid == 0) set_err(a.err, DEV_ERR_BAD_SLOT);
        return;
    }
    const int hs = key_head_of(h, a.n_v, a.n_qk, a.head_map);
    float* Sp = a.S + (size_t(slot) * a.n_v + h) * (kDk * kDv);
    const int rg = tid >> 3;           // rows 4rg .. 4rg+3
    const int cg = tid & 7;            // slice columns 4cg .. 4cg+3
    const int col0 = slice * kSliceCols + cg * 4;
    // the slice of the state is requested before the wait for the kernel in front: only this layer's own
    // step writes it (see the streaming form)
    float4 s[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) s[r] = *reinterpret_cast<const float4*>(Sp + (4 * rg + r) * kDv + col0);
    if (!a.early) griddep_wait();

    if (warp < 2 || (warp == 2 && lane < kSliceCols / 4)) {
        // warp 0: q, warp 1: k (128 channels each), warp 2 lanes 0..7: this slice's 32 v channels
        const int c0 = warp < 2 ? conv_channel0(warp, hs, h, a.n_qk, lane)
                                : 2 * a.n_qk * kDk + h * kDv + slice * kSliceCols + lane * 4;
        ConvIn cin;
        conv_fetch(cin, a, b, slot, c0);
        float4 y = conv_four(cin);
        if (warp == 2 || (slice == 0 && stores_key_taps(h, a.n_v, a.n_qk, a.head_map))) conv_store_taps(cin, a, slot, c0);
        if (warp == 0) y = l2norm_warp(y, a.eps_l2, 1.f / sqrtf(float(kDk)));
        if (warp == 1) y = l2norm_warp(y, a.eps_l2, 1.f);
        float* dst = warp == 0 ? sq : (warp == 1 ? sk : sv);
        *reinterpret_cast<float4*>(dst + lane * 4) = y;
    }
    const float g = expf(a.g_log[size_t(b) * a.n_v + h]);
    const float beta = a.beta[size_t(b) * a.n_v + h];
    __syncthreads();

    // pass 1: decay, kv = S^T k
    float kr[4], qr[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        kr[r] = sk[4 * rg + r];
        qr[r] = sq[4 * rg + r];
    }
    float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        s[r].x *= g; s[r].y *= g; s[r].z *= g; s[r].w *= g;
        kv.x += s[r].x * kr[r]; kv.y += s[r].y * kr[r]; kv.z += s[r].z * kr[r]; kv.w += s[r].w * kr[r];
    }
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
        kv.x += __shfl_xor_sync(0xffffffffu, kv.x, off);
        kv.y += __shfl_xor_sync(0xffffffffu, kv.y, off);
        kv.z += __shfl_xor_sync(0xffffffffu, kv.z, off);
        kv.w += __shfl_xor_sync(0xffffffffu, kv.w, off);
    }
    if (lane < 8) *reinterpret_cast<float4*>(&red[warp][lane * 4]) = kv;
    __syncthreads();
    float4 tot = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const float4 t = *reinterpret_cast<const float4*>(&red[w][cg * 4]);
        tot.x += t.x; tot.y += t.y; tot.z += t.z; tot.w += t.w;
    }
    const float4 vv = *reinterpret_cast<const float4*>(&sv[cg * 4]);
    const float4 dl = make_float4((vv.x - tot.x) * beta, (vv.y - tot.y) * beta, (vv.z - tot.z) * beta,
                                  (vv.w - tot.w) * beta);
    // pass 2: rank-1 update, o = S^T q, write S back
    float4 oo = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        s[r].x += kr[r] * dl.x; s[r].y += kr[r] * dl.y; s[r].z += kr[r] * dl.z; s[r].w += kr[r] * dl.w;
        oo.x += s[r].x * qr[r]; oo.y += s[r].y * qr[r]; oo.z += s[r].z * qr[r]; oo.w += s[r].w * qr[r];
        *reinterpret_cast<float4*>(Sp + (4 * rg + r) * kDv + col0) = s[r];
    }
#pragma unroll
    for (int off = 8; off <= 16; off <<= 1) {
        oo.x += __shfl_xor_sync(0xffffffffu, oo.x, off);
        oo.y += __shfl_xor_sync(0xffffffffu, oo.y, off);
        oo.z += __shfl_xor_sync(0xffffffffu, oo.z, off);
        oo.w += __shfl_xor_sync(0xffffffffu, oo.w, off);
    }
    if (lane < 8) *reinterpret_cast<float4*>(&red2[warp][lane * 4]) = oo;
    __syncthreads();
    if (tid < kSliceCols) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red2[w][tid];
        a.o[(size_t(b) * a.n_v + h) * kDv + slice * kSliceCols + tid] = t;
    }
    if (a.early) griddep_wait();
}

// phase[l][slot_ids[b]] += n_tok (mod 4): thread = (layer, sequence)
__global__ void gdn_phase_advance_kernel(int32_t* phase, const int32_t* slot_ids, int n_layers, int n_slots, int batch,
                                         int n_tok, int* err) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_layers * batch) return;
    const int l = i / batch, b = i - l * batch;
    const int slot = slot_ids ? slot_ids[b] : b;
    if (slot < 0 || slot >= n_slots) {
        set_err(err, DEV_ERR_BAD_SLOT);
        return;
    }
    int32_t* p = phase + size_t(l) * n_slots + slot;
    *p = (*p + n_tok) & 3;
}

// thread = channel; grid (ceil(dim / 256), slots covered, n_layers)
__global__ void conv_ring_export_kernel(const float* ring, const int32_t* phase, float* canon, int n_slots, int slot,
                                        int dim) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= dim) return;
    const int l = blockIdx.z, si = blockIdx.y, sl = slot < 0 ? si : slot;
    const int ph = phase[size_t(l) * n_slots + sl] & 3;
    float4 r = reinterpret_cast<const float4*>(ring)[(size_t(l) * n_slots + sl) * dim + c];
    // oldest-first: taps x_{t-4..t-1} sit in slots (ph, ph+1, ph+2, ph+3) & 3
    if (ph & 1) r = make_float4(r.y, r.z, r.w, r.x);
    if (ph & 2) r = make_float4(r.z, r.w, r.x, r.y);
    reinterpret_cast<float4*>(canon)[(size_t(l) * gridDim.y + si) * dim + c] = r;
}

__global__ void conv_ring_import_kernel(float* ring, int32_t* phase, const float* canon, int n_slots, int slot, int dim) {
    const int c = blockIdx.x * 256 + threadIdx.x;
    const int l = blockIdx.z, si = blockIdx.y, sl = slot < 0 ? si : slot;
    if (c == 0) phase[size_t(l) * n_slots + sl] = 0;
    if (c >= dim) return;
    reinterpret_cast<float4*>(ring)[(size_t(l) * n_slots + sl) * dim + c] =
        reinterpret_cast<const float4*>(canon)[(size_t(l) * gridDim.y + si) * dim + c];
}

}  // namespace

size_t gdn_decode_stream_smem_bytes() { return sizeof(StreamSmem) + 128; }
const void* gdn_decode_stream_kernel_ptr() { return reinterpret_cast<const void*>(&gdn_decode_stream_kernel); }

// Persistent CTAs for `items` heads: one per SM.  (A grid that divides the heads evenly -- 128 CTAs x 12
// heads instead of 148 CTAs with an eleventh round on 56 of them at batch 32 -- measured 5 % slower: one SM
// streams at most ~44 GB/s, so every SM has to take part.)
int gdn_stream_grid(int items, int sms) { return items < sms ? items : sms; }

void launch_gdn_decode(const GdnDecodeArgs& a, int sms, cudaStream_t st, int stream_min_items, int grid_override) {
    if (a.batch <= 0) return;
    const int items = a.batch * a.n_v;
    if (sms > 0 && items >= stream_min_items) {
        const int grid = grid_override > 0 ? (grid_override < items ? grid_override : items) : gdn_stream_grid(items, sms);
        launch_step(gdn_decode_stream_kernel, dim3(grid), dim3(kStreamThreads), gdn_decode_stream_smem_bytes(), st, a);
        return;
    }
    launch_step(gdn_decode_kernel, dim3(kSlices, a.n_v, a.batch), dim3(256), 0, st, a);
}

void launch_gdn_phase_advance(int32_t* phase, const int32_t* slot_ids, int n_layers, int n_slots, int batch, int n_tok,
                              int* err, cudaStream_t st) {
    const int n = n_layers * batch;
    if (n <= 0) return;
    launch_step(gdn_phase_advance_kernel, dim3((n + 127) / 128), dim3(128), 0, st, phase, slot_ids, n_layers, n_slots, batch,
                n_tok, err);
}

void launch_conv_ring_export(const float* ring, const int32_t* phase, float* canon, int n_layers, int n_slots, int slot,
                             int dim, cudaStream_t st) {
    if (n_layers <= 0 || dim <= 0) return;
    conv_ring_export_kernel<<<dim3((dim + 255) / 256, slot < 0 ? n_slots : 1, n_layers), 256, 0, st>>>(ring, phase, canon,
                                                                                                     n_slots, slot, dim);
}

void launch_conv_ring_import(float* ring, int32_t* phase, const float* canon, int n_layers, int n_slots, int slot, int dim,
                             cudaStream_t st) {
    if (n_layers <= 0 || dim <= 0) return;
    conv_ring_import_kernel<<<dim3((dim + 255) / 256, slot < 0 ? n_slots : 1, n_layers), 256, 0, st>>>(ring, phase, canon,
                                                                                                     n_slots, slot, dim);
}

}  // namespace rl
