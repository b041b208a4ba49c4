// Gated DeltaNet decode step on the FP32 recurrent state (sm_100a).
//
// Computes what ops::delta_recurrent_step (src/kernels/ops.cpp:495-540) computes
// per value head:  q^ = l2norm(q)/sqrt(dk), k^ = l2norm(k);  S *= exp(g);
// kv = S^T k^;  delta = beta (v - kv);  S += k^ (x) delta;  o = S^T q^,
// with S [dk=128][dv=128] fp32 row-major (row = key index), kept FP32 in HBM as
// the reference's CPU cache does (src/runtime/dual_cache.cpp:29-33), not BF16 as
// its CUDA kernel does (src/kernels/cuda/cuda_engine.cu:5166-5286).
//
// The step is a pure HBM stream: S is read once and written once.  Columns of S
// are independent, so a CTA owns a 128 x 32 column slice of one head, held in
// registers (4 x 4 per thread) between the two passes; 4 slices x n_v heads x
// batch CTAs keep all SMs busy even at batch 1.
#include "common.cuh"
#include "kernels.h"
#include "launch.cuh"

namespace rl {

namespace {

constexpr int kDk = 128, kDv = 128;
constexpr int kSliceCols = 32;
constexpr int kSlices = kDv / kSliceCols;   // 4

__global__ void __launch_bounds__(256) delta_decode_kernel(DeltaDecodeArgs a) {
    griddep_wait();
    const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __shared__ float sq[kDk], sk[kDk];
    __shared__ float red[8][kSliceCols];
    __shared__ float red2[8][kSliceCols];

    int slot = a.slot_ids ? a.slot_ids[b] : b;
    if (slot < 0 || slot >= a.n_slots) {
        if (tid == 0) set_err(a.err, DEV_ERR_BAD_SLOT);
        return;
    }
    const int rep = a.n_v / a.n_qk;
    const int hs = a.head_map == 0 ? h : (a.head_map == 1 ? h / rep : h % a.n_qk);
    float* Sp = a.S + (size_t(slot) * a.n_v + h) * (kDk * kDv);

    const int rg = tid >> 3;           // rows 4rg .. 4rg+3
    const int cg = tid & 7;            // slice columns 4cg .. 4cg+3
    const int col0 = slice * kSliceCols + cg * 4;
    float4 s[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) s[r] = *reinterpret_cast<const float4*>(Sp + (4 * rg + r) * kDv + col0);

    // l2 norms of this head's query and key (warp 0: q, warp 1: k)
    if (warp < 2) {
        const float* src = warp == 0 ? a.q + size_t(b) * a.q_stride + size_t(hs) * kDk
                                     : a.k + size_t(b) * a.k_stride + size_t(hs) * kDk;
        const float4 x = *reinterpret_cast<const float4*>(src + lane * 4);
        // double accumulator like ops::l2norm (src/kernels/ops.cpp:158-163)
        double ss = double(x.x) * x.x + double(x.y) * x.y + double(x.z) * x.z + double(x.w) * x.w;
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        float inv = 1.f / sqrtf(float(ss) + a.eps_l2);
        if (warp == 0) inv *= 1.f / sqrtf(float(kDk));
        float* dst = warp == 0 ? sq : sk;
        *reinterpret_cast<float4*>(dst + lane * 4) = make_float4(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
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
    const float4 vv = *reinterpret_cast<const float4*>(a.v + size_t(b) * a.v_stride + size_t(h) * kDv + col0);
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
}

// ---- several consecutive tokens per launch (speculative verify) ----
// The reference verifies T = 2..12 drafted tokens with one pass that keeps S on chip across the
// tokens and backs the state up for the rollback (gdn_decode_tn_k, src/kernels/cuda/
// cuda_engine.cu:5289-5536; gdn_t12.cu:100-220).  Same here: the column slice stays in registers
// for all n_tok steps (one read and one write of S however many tokens), every step's output is
// written, and the state as it was before the first token goes to S_backup when that is given.
// Rolling back to k accepted tokens = restore the backup and run k tokens.  Step arithmetic and
// its order are those of delta_decode_kernel, so n_tok steps here equal n_tok single launches bit
// for bit.
__global__ void __launch_bounds__(256) delta_decode_multi_kernel(DeltaDecodeArgs a, float* S_backup, int n_tok,
                                                                  long long qk_tstride, long long v_tstride) {
    const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    __shared__ float sq[kDk], sk[kDk];
    __shared__ float red[8][kSliceCols];
    __shared__ float red2[8][kSliceCols];

    int slot = a.slot_ids ? a.slot_ids[b] : b;
    if (slot < 0 || slot >= a.n_slots) {
        if (tid == 0) set_err(a.err, DEV_ERR_BAD_SLOT);
        return;
    }
    const int rep = a.n_v / a.n_qk;
    const int hs = a.head_map == 0 ? h : (a.head_map == 1 ? h / rep : h % a.n_qk);
    const size_t head_off = (size_t(slot) * a.n_v + h) * (kDk * kDv);
    float* Sp = a.S + head_off;
    const int rg = tid >> 3;           // rows 4rg .. 4rg+3
    const int cg = tid & 7;            // slice columns 4cg .. 4cg+3
    const int col0 = slice * kSliceCols + cg * 4;
    float4 s[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        s[r] = *reinterpret_cast<const float4*>(Sp + (4 * rg + r) * kDv + col0);
        if (S_backup) *reinterpret_cast<float4*>(S_backup + head_off + (4 * rg + r) * kDv + col0) = s[r];
    }
    for (int t = 0; t < n_tok; ++t) {
        if (warp < 2) {
            const float* src = warp == 0 ? a.q + size_t(b) * a.q_stride + size_t(t) * qk_tstride + size_t(hs) * kDk
                                         : a.k + size_t(b) * a.k_stride + size_t(t) * qk_tstride + size_t(hs) * kDk;
            const float4 x = *reinterpret_cast<const float4*>(src + lane * 4);
            double ss = double(x.x) * x.x + double(x.y) * x.y + double(x.z) * x.z + double(x.w) * x.w;
            for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            float inv = 1.f / sqrtf(float(ss) + a.eps_l2);
            if (warp == 0) inv *= 1.f / sqrtf(float(kDk));
            float* dst = warp == 0 ? sq : sk;
            *reinterpret_cast<float4*>(dst + lane * 4) = make_float4(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
        }
        const size_t bt = (size_t(b) * n_tok + t) * a.n_v + h;
        const float g = expf(a.g_log[bt]);
        const float beta = a.beta[bt];
        __syncthreads();
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
            const float4 x = *reinterpret_cast<const float4*>(&red[w][cg * 4]);
            tot.x += x.x; tot.y += x.y; tot.z += x.z; tot.w += x.w;
        }
        const float4 vv = *reinterpret_cast<const float4*>(a.v + size_t(b) * a.v_stride + size_t(t) * v_tstride +
                                                           size_t(h) * kDv + col0);
        const float4 dl = make_float4((vv.x - tot.x) * beta, (vv.y - tot.y) * beta, (vv.z - tot.z) * beta,
                                      (vv.w - tot.w) * beta);
        float4 oo = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            s[r].x += kr[r] * dl.x; s[r].y += kr[r] * dl.y; s[r].z += kr[r] * dl.z; s[r].w += kr[r] * dl.w;
            oo.x += s[r].x * qr[r]; oo.y += s[r].y * qr[r]; oo.z += s[r].z * qr[r]; oo.w += s[r].w * qr[r];
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
            float x = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) x += red2[w][tid];
            a.o[bt * kDv + slice * kSliceCols + tid] = x;
        }
        // sq, sk, red and red2 are rewritten by the next token only after its first barrier, which
        // every thread reaches after the reads above
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) *reinterpret_cast<float4*>(Sp + (4 * rg + r) * kDv + col0) = s[r];
}

// ---- large batches: persistent CTAs streaming whole heads through shared memory with TMA ----
// One work item = one (sequence, value head): its 64 KiB of S is contiguous in HBM.  A producer
// thread bulk-loads items into a 3-stage ring; 256 consumer threads decay, reduce S^T k, then
// apply the rank-1 update, reduce S^T q and stream the new state straight back to HBM.  While
// one item is computed two more are in flight, independent of registers or occupancy.
constexpr int kStreamStages = 3;
constexpr int kStreamThreads = 288;            // 8 consumer warps + producer warp
constexpr int kHeadBytes = kDk * kDv * 4;      // 64 KiB

struct StreamSmem {
    alignas(128) float S[kStreamStages][kDk * kDv];
    float q[2][kDk], k[2][kDk];
    float red[8][kDv], red2[8][kDv];
    uint64_t full[kStreamStages], empty[kStreamStages];
};

__global__ void __launch_bounds__(kStreamThreads, 1) delta_decode_stream_kernel(DeltaDecodeArgs a) {
    extern __shared__ unsigned char smem_raw[];
    StreamSmem& s = *reinterpret_cast<StreamSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_items = a.batch * a.n_v;
    if (tid == 0) {
        for (int i = 0; i < kStreamStages; ++i) {
            mbar_init(&s.full[i], 1);
            mbar_init(&s.empty[i], 1);
        }
        mbar_fence_init();
    }
    griddep_launch();
    __syncthreads();
    griddep_wait();       // barrier set-up above overlaps the tail of the kernel in front; nothing is read before this
    auto slot_of = [&](int b) {
        int slot = a.slot_ids ? a.slot_ids[b] : b;
        if (slot < 0 || slot >= a.n_slots) {
            set_err(a.err, DEV_ERR_BAD_SLOT);
            slot = -1;
        }
        return slot;
    };

    if (warp == 8) {
        // ------------------------------ producer ------------------------------
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
        return;
    }
    // ------------------------------ consumers ------------------------------
    const int rep = a.n_v / a.n_qk;
    const int cg = tid & 31;                  // columns 4cg .. 4cg+3
    const int rg = tid >> 5;                  // rows 16rg .. 16rg+15 (= warp)
    uint32_t it = 0;
    bool alive = true;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x, ++it) {
        const int st = it % kStreamStages;
        const int b = item / a.n_v, h = item - b * a.n_v;
        const int hs = a.head_map == 0 ? h : (a.head_map == 1 ? h / rep : h % a.n_qk);
        const int slot = slot_of(b);
        // l2 norms of q (warp 0) and k (warp 1) into buffer it & 1
        if (warp < 2) {
            const float* src = warp == 0 ? a.q + size_t(b) * a.q_stride + size_t(hs) * kDk
                                         : a.k + size_t(b) * a.k_stride + size_t(hs) * kDk;
            const float4 x = *reinterpret_cast<const float4*>(src + lane * 4);
            double ss = double(x.x) * x.x + double(x.y) * x.y + double(x.z) * x.z + double(x.w) * x.w;
            for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
            float inv = 1.f / sqrtf(float(ss) + a.eps_l2);
            if (warp == 0) inv *= 1.f / sqrtf(float(kDk));
            float* dst = warp == 0 ? s.q[it & 1] : s.k[it & 1];
            *reinterpret_cast<float4*>(dst + lane * 4) = make_float4(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
        }
        const float g = expf(a.g_log[size_t(b) * a.n_v + h]);
        const float beta = a.beta[size_t(b) * a.n_v + h];
        const float4 vv = *reinterpret_cast<const float4*>(a.v + size_t(b) * a.v_stride + size_t(h) * kDv + cg * 4);
        if (alive && !mbar_wait(&s.full[st], (it / kStreamStages) & 1)) {
            set_err(a.err, DEV_ERR_WAIT_TIMEOUT);
            alive = false;
        }
        named_bar_sync(1, 256);               // q, k of this item visible
        const float* Sp = s.S[st];
        float* Sg = a.S + (size_t(slot < 0 ? 0 : slot) * a.n_v + h) * (kDk * kDv);
        const float* kq = s.k[it & 1];
        const float* qq = s.q[it & 1];
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
        named_bar_sync(1, 256);               // every thread is done reading this stage
        if (tid < kDv) {
            float t = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) t += s.red2[w][tid];
            if (slot >= 0) a.o[(size_t(b) * a.n_v + h) * kDv + tid] = t;
        }
        if (tid == 0) mbar_arrive(&s.empty[st]);
    }
}

}  // namespace

void launch_delta_decode_multi(const DeltaDecodeArgs& a, float* S_backup, int n_tok, long long qk_tstride,
                               long long v_tstride, cudaStream_t st) {
    if (a.batch <= 0 || n_tok <= 0) return;
    dim3 grid(kSlices, a.n_v, a.batch);
    delta_decode_multi_kernel<<<grid, 256, 0, st>>>(a, S_backup, n_tok, qk_tstride, v_tstride);
}

size_t delta_decode_stream_smem_bytes() { return sizeof(StreamSmem) + 128; }
const void* delta_decode_stream_kernel_ptr() { return reinterpret_cast<const void*>(&delta_decode_stream_kernel); }

void launch_delta_decode(const DeltaDecodeArgs& a, int sms, cudaStream_t st) {
    if (a.batch <= 0) return;
    const int items = a.batch * a.n_v;
    if (sms > 0 && items >= 4 * sms) {
        // enough heads to keep every SM streaming: one persistent CTA per SM
        launch_step(delta_decode_stream_kernel, dim3(sms), dim3(kStreamThreads), delta_decode_stream_smem_bytes(), st, a);
        return;
    }
    dim3 grid(kSlices, a.n_v, a.batch);
    launch_step(delta_decode_kernel, grid, dim3(256), 0, st, a);
}

}  // namespace rl
