// The element-wise steps that sit directly around the mixers inside a layer:
//   * before attention (fused_attn_decode, src/kernels/ops_fused.cpp:154-171; CUDA twins
//     src/kernels/cuda/cuda_engine.cu:5819-5839, 93-115): split every query head's projected row
//     pair into q and the gate pre-activation, head RMSNorm with the (1 + gamma) weight on q and k
//     (ops::qwen3_rmsnorm, src/kernels/ops.cpp:107-127), partial RoPE on the first rotary_dim dims
//     with rotate-half pairing (ops::rope_partial, ops.cpp:470-493);
//   * before the delta rule (ops_fused.cpp:12-13, 122-123): beta = sigmoid(b),
//     g = -exp(A_log) * softplus(a + dt_bias);
//   * after the delta rule (ops::gated_rmsnorm per head, ops.cpp:129-157): y = gamma (x / rms) silu(z).
// All three are bandwidth-trivial; they exist so that a caller can go from its projections to the
// mixer operators and back without leaving the device.  Sums of squares are accumulated in double
// like the reference's; the RoPE frequencies 1 / theta^(i / pairs) come from the host (the same
// powf the reference's CPU path calls), the angle is the same fp32 product, and cosf / sinf are
// the accurate versions (no fast-math in this build), so the result follows the CPU path to a
// few ulp even at positions beyond 100 000.
#include "common.cuh"
#include "kernels.h"

namespace rl {

namespace {

// sum over the block's threads (blockDim.x a multiple of 32, at most 1024)
__device__ __forceinline__ double block_sum(double v, double* red) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < int(blockDim.x >> 5); ++w) t += red[w];
    __syncthreads();
    return t;
}

}  // namespace

// grid (n_q + n_kv, rows), block head_dim threads (head_dim = 256).  Row r is one token: position
// pos[r] (or pos0 + r when pos is null).  qg [rows][n_q][2 * hd] ([q | gate] per head),
// k [rows][n_kv][hd] in place, q_out / gate_out [rows][n_q][hd].
__global__ void __launch_bounds__(256) attn_qk_prepare_kernel(AttnQkPrepareArgs a) {
    __shared__ double red[8];
    __shared__ float ys[kHeadDim];
    const int hh = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
    const bool is_q = hh < a.n_q;
    float x;
    const float* gamma;
    float* out;
    if (is_q) {
        const float* src = a.qg + (size_t(r) * a.n_q + hh) * (2 * kHeadDim);
        x = src[d];
        a.gate_out[(size_t(r) * a.n_q + hh) * kHeadDim + d] = src[kHeadDim + d];
        gamma = a.q_norm;
        out = a.q_out + (size_t(r) * a.n_q + hh) * kHeadDim;
    } else {
        out = a.k + (size_t(r) * a.n_kv + (hh - a.n_q)) * kHeadDim;
        x = out[d];
        gamma = a.k_norm;
    }
    const double acc = block_sum(double(x) * x, red);
    const float inv = 1.f / sqrtf(float(acc / kHeadDim) + a.eps);
    const float y = x * inv * (gamma ? 1.f + gamma[d] : 1.f);
    const int pairs = a.rotary_dim / 2;
    if (d >= a.rotary_dim) {
        out[d] = y;
        return;
    }
    ys[d] = y;
    __syncthreads();
    if (d < pairs) {
        const int pos = a.pos ? a.pos[r] : a.pos0 + r;
        const float ang = float(pos) * a.inv_freq[d];
        const float c = cosf(ang), s = sinf(ang);
        const float x0 = ys[d], x1 = ys[d + pairs];
        out[d] = x0 * c - x1 * s;
        out[d + pairs] = x0 * s + x1 * c;
    }
}

// grid (n_heads, rows), block head_dim threads (128): y = gamma * (x * inv_rms) * silu(z), per head.
__global__ void __launch_bounds__(128) gated_rmsnorm_kernel(GatedRmsnormArgs a) {
    __shared__ double red[4];
    const int h = blockIdx.x, r = blockIdx.y, d = threadIdx.x;
    const size_t i = (size_t(r) * a.n_heads + h) * a.head_dim + d;
    const float x = a.x[i], z = a.z[i];
    const double acc = block_sum(double(x) * x, red);
    const float inv = 1.f / sqrtf(float(acc / a.head_dim) + a.eps);
    const float sz = z / (1.f + expf(-z));
    a.y[i] = (a.gamma ? a.gamma[d] : 1.f) * (x * inv) * sz;
}

// grid rows, block 256: y = x * inv_rms * (1 + gamma) over rows of n values (the pre-mixer norm of the hidden state).
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float* x, const float* gamma, float* y, int n, float eps) {
    __shared__ double red[8];
    const float* xr = x + size_t(blockIdx.x) * n;
    float* yr = y + size_t(blockIdx.x) * n;
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += double(xr[i]) * xr[i];
    acc = block_sum(acc, red);
    const float inv = 1.f / sqrtf(float(acc / n) + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x) yr[i] = xr[i] * inv * (gamma ? 1.f + gamma[i] : 1.f);
}

// one thread per (row, value head)
__global__ void delta_gates_kernel(const float* a_in, const float* b_in, const float* A_log, const float* dt_bias,
                                   float* beta, float* g_log, int n_v, int rows) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_v * rows) return;
    const int h = i % n_v;
    beta[i] = 1.f / (1.f + expf(-b_in[i]));
    const float x = a_in[i] + dt_bias[h];
    const float sp = log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f);
    g_log[i] = -expf(A_log[h]) * sp;
}

// fp32 rows -> bf16 (round to nearest even): the element type rl_attn_prefill takes its chunk rows in
__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* x, __nv_bfloat16* y, size_t n) {
    const size_t i = (size_t(blockIdx.x) * 256 + threadIdx.x) * 4;
    if (i + 3 < n) {
        const float4 v = *reinterpret_cast<const float4*>(x + i);
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 out;
        out.x = *reinterpret_cast<uint32_t*>(&a);
        out.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(y + i) = out;
    } else {
        for (size_t j = i; j < n; ++j) y[j] = __float2bfloat16_rn(x[j]);
    }
}

}  // namespace rl
