// ref_shim.cpp -- C entry points onto the UNMODIFIED RapidLLM CPU operators.
//
// TEST INFRASTRUCTURE ONLY.  Compiled by oracle/Makefile together with the
// reference's own source files, taken where they lie in the reference tree,
// into oracle/_ref/librl_ref.so.  It pins the C restatement in rl_oracle.c
// and serves as the timed CPU baseline.  Nothing here is copied from the
// reference: this file only forwards arguments.
#include "rapidllm/kernels/cpu_caps.h"
#include "rapidllm/kernels/ops.h"
#include "rapidllm/runtime/thread_pool.h"

#include <cstring>

using namespace rapidllm;

extern "C" {

void ref_attn_decode(const float* q, const float* k, const float* v, float* o, int pos, int n_q,
                     int n_kv, int hd) {
    ops::attn_decode(q, k, v, o, pos, n_q, n_kv, hd);
}

void ref_attn_prefill(const float* q, const float* k, const float* v, float* o, int seq, int n_q,
                      int n_kv, int hd) {
    ops::attn_prefill(q, k, v, o, seq, n_q, n_kv, hd);
}

void ref_delta_step_scalar(float* S, const float* q, const float* k, const float* v,
                           const float* beta, const float* g, float* o, int n_v, int dk, int dv,
                           float eps) {
    ops::delta_recurrent_step_scalar(S, q, k, v, beta, g, o, n_v, dk, dv, eps);
}

void ref_delta_step_simd(float* S, const float* q, const float* k, const float* v,
                         const float* beta, const float* g, float* o, int n_v, int dk, int dv,
                         float eps) {
    ops::delta_recurrent_step_simd(S, q, k, v, beta, g, o, n_v, dk, dv, eps);
}

void ref_conv1d_update(const float* x, const float* w, float* state, float* y, int dim, int k) {
    ops::conv1d_update(x, w, state, y, dim, k);
}

void ref_conv1d_causal_prefill(const float* x, const float* w, float* y, int seq, int dim, int k) {
    ops::conv1d_causal_prefill(x, w, y, seq, dim, k);
}

void ref_l2norm(const float* x, float* y, int n, float eps) { ops::l2norm(x, y, n, eps); }

void ref_qwen3_rmsnorm(const float* x, const float* gamma, float* y, int n, float eps) {
    ops::qwen3_rmsnorm(x, gamma, y, n, eps);
}

void ref_gated_rmsnorm(const float* x, const float* z, const float* gamma, float* y, int n, float eps,
                       int gamma_n) {
    ops::gated_rmsnorm(x, z, gamma, y, n, eps, gamma_n);
}

void ref_rope_partial(float* q, float* k, int n_q, int n_kv, int head_dim, int rotary_dim, int pos,
                      float theta) {
    ops::rope_partial(q, k, n_q, n_kv, head_dim, rotary_dim, pos, theta);
}

// The whole decode mixers (ops::fused_delta_decode / fused_attn_decode, ops_fused.cpp:84-182) with
// dense fp32 weights: norm, projections, the operator, output projection, residual.
static ops::QuantW dense(const float* w) {
    ops::QuantW q;
    q.data = reinterpret_cast<const uint8_t*>(w);
    return q;
}

void ref_fused_delta_decode(float* x, const float* rms_w, const float* Wqkv, const float* Wz, const float* Wa,
                            const float* Wb, const float* Wo, const float* A_log, const float* dt_bias,
                            const float* conv_w, const float* gnorm, float* S, float* conv_state, int hidden,
                            int nk, int nv, int dk, int dv, int conv_k, float eps, int use_simd, int v_tiled) {
    ops::FusedDeltaArgs a{};
    a.x = x;
    a.x_inout = x;
    a.rms_w = rms_w;
    a.Wqkv = dense(Wqkv);
    a.Wz = dense(Wz);
    a.Wa = dense(Wa);
    a.Wb = dense(Wb);
    a.Wo = dense(Wo);
    a.A_log = A_log;
    a.dt_bias = dt_bias;
    a.conv_w = conv_w;
    a.gnorm = gnorm;
    a.S = S;
    a.conv_state = conv_state;
    a.hidden = hidden;
    a.nk = nk;
    a.nv = nv;
    a.dk = dk;
    a.dv = dv;
    a.conv_k = conv_k;
    a.gnorm_n = dv;
    a.eps = eps;
    a.use_simd = use_simd != 0;
    a.v_tiled = v_tiled != 0;
    ops::fused_delta_decode(a);
}

void ref_fused_attn_decode(float* x, const float* rms_w, const float* Wq, const float* Wk, const float* Wv,
                           const float* Wo, const float* q_norm, const float* k_norm, float* k_cache,
                           float* v_cache, int hidden, int n_q, int n_kv, int head_dim, int rotary_dim, int pos,
                           float theta, float eps, int use_simd) {
    ops::FusedAttnArgs a{};
    a.x = x;
    a.x_inout = x;
    a.rms_w = rms_w;
    a.Wq = dense(Wq);
    a.Wk = dense(Wk);
    a.Wv = dense(Wv);
    a.Wo = dense(Wo);
    a.q_norm = q_norm;
    a.k_norm = k_norm;
    a.k_cache = k_cache;
    a.v_cache = v_cache;
    a.hidden = hidden;
    a.n_q = n_q;
    a.n_kv = n_kv;
    a.head_dim = head_dim;
    a.rotary_dim = rotary_dim;
    a.pos = pos;
    a.theta = theta;
    a.eps = eps;
    a.use_simd = use_simd != 0;
    ops::fused_attn_decode(a);
}

void ref_set_threads(int n) { set_num_threads(n); }
int ref_num_threads(void) { return num_threads(); }

int ref_simd_name(char* buf, int n) {
    const char* s = ops::simd_isa_name();
    std::strncpy(buf, s, n > 0 ? n - 1 : 0);
    if (n > 0) buf[n - 1] = 0;
    return static_cast<int>(std::strlen(s));
}

} // extern "C"
