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

namespace rl {

namespace {

constexpr int kDk = 128, kDv = 128;
constexpr int kSliceCols = 32;
constexpr int kSlices = kDv / kSliceCols;   // 4

__global__ void __launch_bounds__(256) delta_decode_kernel(DeltaDecodeArgs a) {
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

}  // namespace

void launch_delta_decode(const DeltaDecodeArgs& a, cudaStream_t st) {
    if (a.batch <= 0) return;
    dim3 grid(kSlices, a.n_v, a.batch);
    delta_decode_kernel<<<grid, 256, 0, st>>>(a);
}

}  // namespace rl
