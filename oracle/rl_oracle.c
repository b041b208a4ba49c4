/*
 * rl_oracle.c -- CPU restatement of the RapidLLM hybrid-attention operators.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels: it
 * is imported by tests/, by the smoke check and by the bench's cpu_baseline /
 * reference legs, and by nothing that ships.  The product library never links
 * or calls it.
 *
 * Every function restates, in plain C, one piece of the reference engine and
 * cites the file:line it follows (paths are relative to the RapidLLM tree).
 * Where the reference has CPU code (attention, delta rule, conv1d) the
 * restatement keeps the reference's operation order and accumulator widths, so
 * it is bit-identical to the reference when both are built without FMA
 * contraction; tests pin that against outputs of the reference itself.
 *
 * Where the reference has CUDA code only (q8 K / TQ3 V compact KV) no
 * reference test or CPU function exists: the restatement follows the cited
 * CUDA lines in IEEE fp32 (true division, sqrtf, no fast-math) with one
 * documented summation order, and is pinned on the reference's own CUDA
 * kernels run on a GPU (ref_cuda_shim.cu; tests/test_gpu_compact_ref_pin.py:
 * V codes and all scales equal, K codes equal but for ~1 in 10^6 that sit
 * on a rounding boundary of the reference's fast-math division).  The
 * 256-point layout with a sign vector has no reference kernel: that
 * variant alone stays unpinned.
 *
 * Build: gcc -O2 -ffp-contract=off -fno-fast-math (see oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define RLO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ */
/* fp16 <-> fp32, round-to-nearest-even (what __float2half does on the */
/* reference's KV append, cuda_engine.cu:5844-5850, 8216-8221).        */
/* ------------------------------------------------------------------ */
RLO_API uint16_t rlo_f32_to_f16(float f) {
    _Float16 h = (_Float16)f;
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}

RLO_API float rlo_f16_to_f32(uint16_t u) {
    _Float16 h;
    memcpy(&h, &u, 2);
    return (float)h;
}

RLO_API void rlo_f32_to_f16_n(const float* x, uint16_t* y, long n) {
    for (long i = 0; i < n; ++i) y[i] = rlo_f32_to_f16(x[i]);
}

RLO_API void rlo_f16_to_f32_n(const uint16_t* x, float* y, long n) {
    for (long i = 0; i < n; ++i) y[i] = rlo_f16_to_f32(x[i]);
}

static float silu_f(float x) { return x / (1.f + expf(-x)); } /* ops.cpp:13 */

/* ------------------------------------------------------------------ */
/* Gated attention                                                     */
/* ------------------------------------------------------------------ */

/* One query token against cache rows [0, pos].  src/kernels/ops.cpp:575-605.
 * q [n_q][hd], k_cache/v_cache [seq][n_kv][hd] fp32, o [n_q][hd]. */
RLO_API void rlo_attn_decode(const float* q, const float* k_cache, const float* v_cache, float* o,
                             int pos, int n_q, int n_kv, int hd) {
    const int seq = pos + 1;
    const int rep = n_q / n_kv;
    const float scale = 1.f / sqrtf((float)hd);
    float* scores = (float*)malloc(sizeof(float) * (size_t)seq);
    for (int hq = 0; hq < n_q; ++hq) {
        const int hkv = hq / rep;
        const float* qt = q + (size_t)hq * hd;
        float m = -1e30f;
        for (int s = 0; s < seq; ++s) {
            const float* ks = k_cache + ((size_t)s * n_kv + hkv) * hd;
            double acc = 0;
            for (int d = 0; d < hd; ++d) acc += (double)qt[d] * ks[d];
            scores[s] = (float)acc * scale;
            m = fmaxf(m, scores[s]);
        }
        double z = 0;
        for (int s = 0; s < seq; ++s) {
            scores[s] = expf(scores[s] - m);
            z += scores[s];
        }
        float* ot = o + (size_t)hq * hd;
        for (int d = 0; d < hd; ++d) ot[d] = 0.f;
        for (int s = 0; s < seq; ++s) {
            const float a = (float)(scores[s] / z);
            const float* vs = v_cache + ((size_t)s * n_kv + hkv) * hd;
            for (int d = 0; d < hd; ++d) ot[d] += a * vs[d];
        }
    }
    free(scores);
}

/* Causal prefill of a whole sequence.  src/kernels/ops.cpp:542-573.
 * q [seq][n_q][hd], k/v [seq][n_kv][hd], o [seq][n_q][hd]. */
RLO_API void rlo_attn_prefill(const float* q, const float* k, const float* v, float* o, int seq,
                              int n_q, int n_kv, int hd) {
    for (int t = 0; t < seq; ++t)
        rlo_attn_decode(q + (size_t)t * n_q * hd, k, v, o + (size_t)t * n_q * hd, t, n_q, n_kv, hd);
}

/* Chunked prefill: T query rows at positions pos0..pos0+T-1 against a cache
 * that already holds rows [0, pos0+T).  The reference's chunk driver applies
 * the same causal rule with an offset (cuda_engine.cu:8963-8975); on the CPU
 * it is attn_decode per row.  Only the listed rows are computed so a strided
 * sample of a long prefill stays cheap. */
RLO_API void rlo_attn_prefill_rows(const float* q_rows, const float* k_cache, const float* v_cache,
                                   float* o_rows, const int* row_pos, int n_rows, int n_q,
                                   int n_kv, int hd) {
    for (int r = 0; r < n_rows; ++r)
        rlo_attn_decode(q_rows + (size_t)r * n_q * hd, k_cache, v_cache,
                        o_rows + (size_t)r * n_q * hd, row_pos[r], n_q, n_kv, hd);
}

/* Sigmoid output gate, src/kernels/ops_fused.cpp:178 (session.cpp:318). */
RLO_API void rlo_sigmoid_gate(float* o, const float* gate, long n) {
    for (long j = 0; j < n; ++j) o[j] *= 1.f / (1.f + expf(-gate[j]));
}

/* Merge split-KV partials (m, l, acc) the way the reference merges its
 * 8 warp partials, cuda_engine.cu:347-374 (expf instead of __expf).
 * m,l [n_parts], acc [n_parts][hd]; o [hd]. */
RLO_API void rlo_lse_combine(const float* m, const float* l, const float* acc, int n_parts,
                             int hd, float* o) {
    float mm = -1e30f;
    for (int w = 0; w < n_parts; ++w) mm = fmaxf(mm, m[w]);
    float lsum = 0.f;
    for (int d = 0; d < hd; ++d) o[d] = 0.f;
    for (int w = 0; w < n_parts; ++w) {
        const float al = expf(m[w] - mm);
        lsum += l[w] * al;
        for (int d = 0; d < hd; ++d) o[d] += acc[(size_t)w * hd + d] * al;
    }
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    for (int d = 0; d < hd; ++d) o[d] *= inv;
}

/* Unnormalised partial over cache rows [s0, s1) for one query head: the
 * quantity a split-KV worker produces.  Same arithmetic as rlo_attn_decode. */
RLO_API void rlo_attn_partial(const float* qh, const float* k_cache, const float* v_cache,
                              int s0, int s1, int n_kv, int hkv, int hd, float* m_out,
                              float* l_out, float* acc) {
    const float scale = 1.f / sqrtf((float)hd);
    float m = -1e30f;
    const int n = s1 - s0;
    float* sc = (float*)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1));
    for (int s = s0; s < s1; ++s) {
        const float* ks = k_cache + ((size_t)s * n_kv + hkv) * hd;
        double a = 0;
        for (int d = 0; d < hd; ++d) a += (double)qh[d] * ks[d];
        sc[s - s0] = (float)a * scale;
        m = fmaxf(m, sc[s - s0]);
    }
    double z = 0;
    for (int d = 0; d < hd; ++d) acc[d] = 0.f;
    for (int s = s0; s < s1; ++s) {
        const float p = expf(sc[s - s0] - m);
        z += p;
        const float* vs = v_cache + ((size_t)s * n_kv + hkv) * hd;
        for (int d = 0; d < hd; ++d) acc[d] += p * vs[d];
    }
    *m_out = m;
    *l_out = (float)z;
    free(sc);
}

/* ------------------------------------------------------------------ */
/* Paged KV indexing.  The reference cache is contiguous                */
/* [pos][n_kv][hd] (src/runtime/dual_cache.cpp:49-60, append 74-79);   */
/* the paged pool is [page][n_kv][page_tokens][hd] and a sequence's     */
/* token s lives in page table[s / page_tokens], slot s % page_tokens.  */
/* Gathering through the table must reproduce the contiguous bytes.    */
/* ------------------------------------------------------------------ */
RLO_API void rlo_paged_gather_u16(const uint16_t* pool, const int32_t* table, int seq_len,
                                  int n_kv, int page_tokens, int hd, uint16_t* out) {
    for (int s = 0; s < seq_len; ++s) {
        const size_t page = (size_t)table[s / page_tokens];
        const int slot = s % page_tokens;
        for (int h = 0; h < n_kv; ++h)
            memcpy(out + ((size_t)s * n_kv + h) * hd,
                   pool + ((page * n_kv + h) * page_tokens + slot) * hd, sizeof(uint16_t) * hd);
    }
}

RLO_API void rlo_paged_scatter_u16(uint16_t* pool, const int32_t* table, int s0, int s1, int n_kv,
                                   int page_tokens, int hd, const uint16_t* rows) {
    for (int s = s0; s < s1; ++s) {
        const size_t page = (size_t)table[s / page_tokens];
        const int slot = s % page_tokens;
        for (int h = 0; h < n_kv; ++h)
            memcpy(pool + ((page * n_kv + h) * page_tokens + slot) * hd,
                   rows + ((size_t)(s - s0) * n_kv + h) * hd, sizeof(uint16_t) * hd);
    }
}

/* ------------------------------------------------------------------ */
/* Gated DeltaNet                                                      */
/* ------------------------------------------------------------------ */

/* src/kernels/ops.cpp:158-163 */
static void l2norm_f(const float* x, float* y, int n, float eps) {
    double acc = 0;
    for (int i = 0; i < n; ++i) acc += (double)x[i] * x[i];
    const float inv = 1.f / sqrtf((float)acc + eps);
    for (int i = 0; i < n; ++i) y[i] = x[i] * inv;
}

RLO_API void rlo_l2norm(const float* x, float* y, int n, float eps) { l2norm_f(x, y, n, eps); }

/* One decode step of the gated delta rule for n_v value heads.
 * src/kernels/ops.cpp:495-534.  S [n_v][dk][dv] in place; q,k [n_v][dk]
 * (already repeated per value head); v [n_v][dv]; beta,g_log [n_v]. */
RLO_API void rlo_delta_step(float* S, const float* q_in, const float* k_in, const float* v,
                            const float* beta, const float* g_log, float* o, int n_v, int dk,
                            int dv, float eps_l2) {
    float* q = (float*)malloc(sizeof(float) * (size_t)n_v * dk);
    float* k = (float*)malloc(sizeof(float) * (size_t)n_v * dk);
    float* kv = (float*)malloc(sizeof(float) * (size_t)dv);
    float* delta = (float*)malloc(sizeof(float) * (size_t)dv);
    for (int h = 0; h < n_v; ++h) {
        l2norm_f(q_in + (size_t)h * dk, q + (size_t)h * dk, dk, eps_l2);
        l2norm_f(k_in + (size_t)h * dk, k + (size_t)h * dk, dk, eps_l2);
        const float scale = 1.f / sqrtf((float)dk);
        for (int i = 0; i < dk; ++i) q[(size_t)h * dk + i] *= scale;
    }
    for (int h = 0; h < n_v; ++h) {
        const float g = expf(g_log[h]);
        float* Sh = S + (size_t)h * dk * dv;
        for (int i = 0; i < dk * dv; ++i) Sh[i] *= g;
        const float* kh = k + (size_t)h * dk;
        const float* qh = q + (size_t)h * dk;
        const float* vh = v + (size_t)h * dv;
        for (int j = 0; j < dv; ++j) kv[j] = 0.f;
        for (int i = 0; i < dk; ++i) {
            const float ki = kh[i];
            const float* srow = Sh + (size_t)i * dv;
            for (int j = 0; j < dv; ++j) kv[j] += srow[j] * ki;
        }
        for (int j = 0; j < dv; ++j) delta[j] = (vh[j] - kv[j]) * beta[h];
        for (int i = 0; i < dk; ++i) {
            float* srow = Sh + (size_t)i * dv;
            const float ki = kh[i];
            for (int j = 0; j < dv; ++j) srow[j] += ki * delta[j];
        }
        float* oh = o + (size_t)h * dv;
        for (int j = 0; j < dv; ++j) oh[j] = 0.f;
        for (int i = 0; i < dk; ++i) {
            const float qi = qh[i];
            const float* srow = Sh + (size_t)i * dv;
            for (int j = 0; j < dv; ++j) oh[j] += srow[j] * qi;
        }
    }
    free(q);
    free(k);
    free(kv);
    free(delta);
}

/* Value head h reads key/query head h / (n_v/n_k) (grouped, HF order) or
 * h % n_k (tiled, GGUF order): src/kernels/ops_fused.cpp:111-124,
 * cuda_engine.cu:78-89. */
RLO_API void rlo_repeat_heads(const float* x, float* y, int n_k, int n_v, int d, int tiled) {
    const int rep = n_v / n_k;
    for (int h = 0; h < n_v; ++h) {
        const int src = tiled ? (h % n_k) : (h / rep);
        memcpy(y + (size_t)h * d, x + (size_t)src * d, sizeof(float) * d);
    }
}

/* T sequential delta steps; the reference's only prefill form
 * (src/runtime/session.cpp:232-248).  q,k [T][n_v][dk], v,o [T][n_v][dv],
 * beta,g_log [T][n_v]. */
RLO_API void rlo_delta_prefill_seq(float* S, const float* q, const float* k, const float* v,
                                   const float* beta, const float* g_log, float* o, int T, int n_v,
                                   int dk, int dv, float eps_l2) {
    for (int t = 0; t < T; ++t)
        rlo_delta_step(S, q + (size_t)t * n_v * dk, k + (size_t)t * n_v * dk,
                       v + (size_t)t * n_v * dv, beta + (size_t)t * n_v, g_log + (size_t)t * n_v,
                       o + (size_t)t * n_v * dv, n_v, dk, dv, eps_l2);
}

/* Gate maths in front of the delta rule, src/kernels/ops_fused.cpp:12-13,
 * 122-123: beta = sigmoid(b), g = -exp(A_log) * softplus(a + dt_bias) with
 * softplus(x) = log1p(exp(-|x|)) + max(x, 0). */
RLO_API void rlo_delta_gates(const float* a, const float* b, const float* A_log,
                             const float* dt_bias, float* beta, float* g_log, int n_v) {
    for (int h = 0; h < n_v; ++h) {
        beta[h] = 1.f / (1.f + expf(-b[h]));
        const float x = a[h] + dt_bias[h];
        const float sp = log1pf(expf(-fabsf(x))) + fmaxf(x, 0.f);
        g_log[h] = -expf(A_log[h]) * sp;
    }
}

/* Dense projection, scalar path of src/kernels/ops.cpp:165-172 (gemv_f32_scalar, what
 * gemv_w calls without SIMD, ops_fused.cpp:36-41): y[i] = (float) sum_j (double) W[i][j] x[j],
 * summed in index order. */
RLO_API void rlo_gemv_f32(const float* W, const float* x, float* y, int m, int n) {
    for (int i = 0; i < m; ++i) {
        double acc = 0;
        const float* row = W + (size_t)i * n;
        for (int j = 0; j < n; ++j) acc += (double)row[j] * x[j];
        y[i] = (float)acc;
    }
}

/* Head RMSNorm with the (1 + gamma) weight, scalar path of src/kernels/ops.cpp:107-127:
 * double sum of squares, inv = 1 / sqrtf((float)(acc / n) + eps), y = x * inv * (1 + gamma). */
RLO_API void rlo_qwen3_rmsnorm(const float* x, const float* gamma, float* y, int n, float eps) {
    double acc = 0;
    for (int i = 0; i < n; ++i) acc += (double)x[i] * x[i];
    const float inv = 1.f / sqrtf((float)(acc / n) + eps);
    for (int i = 0; i < n; ++i) {
        const float g = gamma ? (1.f + gamma[i]) : 1.f;
        y[i] = x[i] * inv * g;
    }
}

/* Partial rotary embedding, src/kernels/ops.cpp:470-493: the first rotary_dim dims of every
 * head, rotate-half pairing (i, i + rotary_dim/2) for head_dim >= 64, adjacent pairs below;
 * freq_i = 1 / powf(theta, i / pairs), angle = (float)pos * freq_i. */
static void rope_heads(float* t, int n_heads, int head_dim, int rotary_dim, int pos, float theta) {
    const int pairs = rotary_dim / 2;
    for (int h = 0; h < n_heads; ++h) {
        float* v = t + (size_t)h * head_dim;
        for (int i = 0; i < pairs; ++i) {
            const float freq = 1.f / powf(theta, (float)i / (float)pairs);
            const float ang = (float)pos * freq;
            const float c = cosf(ang), s = sinf(ang);
            if (head_dim >= 64) {
                const float x0 = v[i], x1 = v[i + pairs];
                v[i] = x0 * c - x1 * s;
                v[i + pairs] = x0 * s + x1 * c;
            } else {
                const float x0 = v[2 * i], x1 = v[2 * i + 1];
                v[2 * i] = x0 * c - x1 * s;
                v[2 * i + 1] = x0 * s + x1 * c;
            }
        }
    }
}
RLO_API void rlo_rope_partial(float* q, float* k, int n_q, int n_kv, int head_dim, int rotary_dim,
                              int pos, float theta) {
    rope_heads(q, n_q, head_dim, rotary_dim, pos, theta);
    rope_heads(k, n_kv, head_dim, rotary_dim, pos, theta);
}

/* What fused_attn_decode does between the projections and the cache append,
 * src/kernels/ops_fused.cpp:154-171: split each query head's row pair into q and gate
 * (head_dim >= 64: [q | gate] per head; below: all q then all gate), head RMSNorm of q and k
 * with (1 + gamma), partial RoPE at pos.  qg [n_q * 2 * hd], k [n_kv * hd] in place. */
RLO_API void rlo_attn_qk_prepare(const float* qg, float* k, const float* q_norm, const float* k_norm,
                                 float* q, float* gate, int n_q, int n_kv, int hd, int rotary_dim,
                                 int pos, float theta, float eps) {
    const int qn = n_q * hd;
    if (hd >= 64) {
        for (int h = 0; h < n_q; ++h)
            for (int d = 0; d < hd; ++d) {
                q[h * hd + d] = qg[h * hd * 2 + d];
                gate[h * hd + d] = qg[h * hd * 2 + hd + d];
            }
    } else {
        for (int j = 0; j < qn; ++j) {
            q[j] = qg[j];
            gate[j] = qg[qn + j];
        }
    }
    for (int h = 0; h < n_q; ++h) rlo_qwen3_rmsnorm(q + h * hd, q_norm, q + h * hd, hd, eps);
    for (int h = 0; h < n_kv; ++h) rlo_qwen3_rmsnorm(k + h * hd, k_norm, k + h * hd, hd, eps);
    rlo_rope_partial(q, k, n_q, n_kv, hd, rotary_dim, pos, theta);
}

/* Gated RMSNorm after the delta rule, src/kernels/ops.cpp:129-157 (silu at line 13):
 * per head of gamma_n values when gamma_n < n divides n and n >= 256, else over all n:
 * y = gamma * (x * inv) * silu(z), silu(z) = z / (1 + expf(-z)). */
RLO_API void rlo_gated_rmsnorm(const float* x, const float* z, const float* gamma, float* y, int n,
                               float eps, int gamma_n) {
    if (gamma_n <= 0) gamma_n = n;
    const int per_head = gamma_n < n && (n % gamma_n) == 0 && n >= 256;
    const int span = per_head ? gamma_n : n;
    for (int h = 0; h < n / span; ++h) {
        const float* xh = x + (size_t)h * span;
        const float* zh = z + (size_t)h * span;
        float* yh = y + (size_t)h * span;
        double acc = 0;
        for (int i = 0; i < span; ++i) acc += (double)xh[i] * xh[i];
        const float inv = 1.f / sqrtf((float)(acc / span) + eps);
        for (int i = 0; i < span; ++i) {
            const float g = gamma ? gamma[per_head ? i : i % gamma_n] : 1.f;
            const float sz = zh[i] / (1.f + expf(-zh[i]));
            yh[i] = g * (xh[i] * inv) * sz;
        }
    }
}

/* Depthwise causal conv, decode form.  src/kernels/ops.cpp:458-468.
 * state [dim][k] (oldest tap first) shifted left, x appended, dot, SiLU. */
RLO_API void rlo_conv1d_update(const float* x_t, const float* w, float* state, float* y, int dim,
                               int k) {
    for (int c = 0; c < dim; ++c) {
        float* st = state + (size_t)c * k;
        for (int p = 0; p < k - 1; ++p) st[p] = st[p + 1];
        st[k - 1] = x_t[c];
        double acc = 0;
        for (int p = 0; p < k; ++p) acc += (double)w[(size_t)c * k + p] * st[p];
        y[c] = silu_f((float)acc);
    }
}

/* Prefill form.  src/kernels/ops.cpp:443-456.  x,y [seq][dim]. */
RLO_API void rlo_conv1d_causal_prefill(const float* x, const float* w, float* y, int seq, int dim,
                                       int k) {
    for (int t = 0; t < seq; ++t)
        for (int c = 0; c < dim; ++c) {
            double acc = 0;
            for (int p = 0; p < k; ++p) {
                const int src = t - (k - 1 - p);
                const float xv = src >= 0 ? x[(size_t)src * dim + c] : 0.f;
                acc += (double)w[(size_t)c * k + p] * xv;
            }
            y[(size_t)t * dim + c] = silu_f((float)acc);
        }
}

/* ------------------------------------------------------------------ */
/* Compact KV: q8 K + TurboQuant-3 V.  CUDA-only in the reference;      */
/* pinned on its own CUDA kernels (see the header of this file).        */
/* ------------------------------------------------------------------ */

/* 3-bit Lloyd-Max centroids for N(0,1), cuda_engine.cu:205-209. */
static const float kTq3Cent[8] = {-2.152f, -1.344f, -0.756f, -0.245f,
                                  0.245f,  0.756f,  1.344f,  2.152f};

RLO_API const float* rlo_tq3_centroids(void) { return kTq3Cent; }

/* K row -> int8 + fp16 scale.  cuda_engine.cu:8224-8249 (twin 6037-6054):
 * s = amax/127 + 1e-8 (fp32); stored scale = half(s);
 * q = lrintf(clamp(x / s, -127, 127)) with the fp32 s (round half to even). */
RLO_API void rlo_q8k_store(const float* x, int hd, int8_t* q, uint16_t* scale) {
    float amax = 0.f;
    for (int i = 0; i < hd; ++i) amax = fmaxf(amax, fabsf(x[i]));
    const float s = amax / 127.f + 1e-8f;
    *scale = rlo_f32_to_f16(s);
    for (int i = 0; i < hd; ++i) {
        const float u = fminf(fmaxf(x[i] / s, -127.f), 127.f);
        q[i] = (int8_t)lrintf(u);
    }
}

/* cuda_engine.cu:8286-8295: k_hat = half2float(scale) * q */
RLO_API void rlo_q8k_dequant(const int8_t* q, uint16_t scale, int hd, float* x) {
    const float s = rlo_f16_to_f32(scale);
    for (int i = 0; i < hd; ++i) x[i] = s * (float)q[i];
}

/* In-place Walsh-Hadamard butterflies, strides 1,2,..,n/2, then x 1/sqrt(n).
 * cuda_engine.cu:212-229 (the shuffle form 267-291 computes the same values:
 * every stage is one add or subtract per element). */
static void fwht_f(float* x, int n) {
    for (int stride = 1; stride < n; stride <<= 1)
        for (int i = 0; i < n; ++i) {
            const int j = i ^ stride;
            if (i < j) {
                const float a = x[i], b = x[j];
                x[i] = a + b;
                x[j] = a - b;
            }
        }
    const float inv = n == 128 ? 0.08838834764831845f : 1.f / sqrtf((float)n);
    for (int i = 0; i < n; ++i) x[i] *= inv;
}

RLO_API void rlo_fwht(float* x, int n) { fwht_f(x, n); }

/* Sum of squares in the order the store kernel uses (cuda_engine.cu:8266-8273):
 * inside each group of 32 a xor-butterfly (offsets 16,8,4,2,1), then the group
 * sums added in ascending order. */
static float sumsq_grouped(const float* x, int n) {
    float tot = 0.f;
    for (int g0 = 0; g0 < n; g0 += 32) {
        float v[32], t[32];
        for (int i = 0; i < 32; ++i) v[i] = x[g0 + i] * x[g0 + i];
        for (int off = 16; off > 0; off >>= 1) {
            for (int i = 0; i < 32; ++i) t[i] = v[i] + v[i ^ off];
            memcpy(v, t, sizeof v);
        }
        tot = g0 == 0 ? v[0] : tot + v[0];
    }
    return tot;
}

/* nearest centroid, strict '<' so the lowest index wins ties: 231-243 */
static int tq3_nn(float v) {
    int bi = 0;
    float bd = fabsf(v - kTq3Cent[0]);
    for (int i = 1; i < 8; ++i) {
        const float d = fabsf(v - kTq3Cent[i]);
        if (d < bd) {
            bd = d;
            bi = i;
        }
    }
    return bi;
}

/* V row -> TQ3 codes.  cuda_engine.cu:8252-8284 with IEEE division
 * (idx = nn(x / rms), as the decode-time twin at 6073 does).
 *   wht_len 128: the reference layout, hd/128 independent blocks, no signs.
 *   wht_len 256: one block per head; signs (+-1, length wht_len, may be NULL)
 *                multiply the input before the transform.
 * Per block: codes = wht_len*3/8 bytes (8 indices LSB-first per 24-bit word,
 * 245-254), scale = half(rms), rms = sqrtf(sumsq/wht_len) + 1e-8. */
RLO_API void rlo_tq3v_store(const float* x, int hd, int wht_len, const float* signs, uint8_t* codes,
                            uint16_t* scales) {
    const int nblk = hd / wht_len;
    const int cb = wht_len * 3 / 8;
    float buf[256];
    for (int b = 0; b < nblk; ++b) {
        for (int i = 0; i < wht_len; ++i)
            buf[i] = signs ? x[b * wht_len + i] * signs[i] : x[b * wht_len + i];
        fwht_f(buf, wht_len);
        const float tot = sumsq_grouped(buf, wht_len);
        const float rms = sqrtf(tot / (float)wht_len) + 1e-8f;
        scales[b] = rlo_f32_to_f16(rms);
        uint8_t* dst = codes + (size_t)b * cb;
        for (int g = 0; g < wht_len / 8; ++g) {
            uint32_t w = 0;
            for (int j = 0; j < 8; ++j) w |= (uint32_t)(tq3_nn(buf[g * 8 + j] / rms) & 7) << (3 * j);
            dst[g * 3 + 0] = (uint8_t)w;
            dst[g * 3 + 1] = (uint8_t)(w >> 8);
            dst[g * 3 + 2] = (uint8_t)(w >> 16);
        }
    }
}

/* cuda_engine.cu:256-262, 293-299, 8297-8314: centroid * half2float(scale),
 * inverse transform (= the same orthonormal transform), then signs. */
RLO_API void rlo_tq3v_dequant(const uint8_t* codes, const uint16_t* scales, int hd, int wht_len,
                              const float* signs, float* x) {
    const int nblk = hd / wht_len;
    const int cb = wht_len * 3 / 8;
    for (int b = 0; b < nblk; ++b) {
        const float s = rlo_f16_to_f32(scales[b]);
        const uint8_t* src = codes + (size_t)b * cb;
        float* xb = x + b * wht_len;
        for (int i = 0; i < wht_len; ++i) {
            const int g = i >> 3, j = i & 7;
            const uint32_t w = (uint32_t)src[g * 3] | ((uint32_t)src[g * 3 + 1] << 8) |
                               ((uint32_t)src[g * 3 + 2] << 16);
            xb[i] = kTq3Cent[(w >> (3 * j)) & 7u] * s;
        }
        fwht_f(xb, wht_len);
        if (signs)
            for (int i = 0; i < wht_len; ++i) xb[i] *= signs[i];
    }
}

/* Store / dequantise a whole [T][n_kv][hd] block (token-major compact layout
 * of the reference, cuda_engine.cu:18305-18318). */
RLO_API void rlo_compact_store(const float* k, const float* v, long T, int n_kv, int hd,
                               int wht_len, const float* signs, int8_t* k_q, uint16_t* k_sc,
                               uint8_t* v_codes, uint16_t* v_sc) {
    const int nblk = hd / wht_len;
    const int vb = hd * 3 / 8;
    for (long r = 0; r < T * n_kv; ++r) {
        rlo_q8k_store(k + r * hd, hd, k_q + r * hd, k_sc + r);
        rlo_tq3v_store(v + r * hd, hd, wht_len, signs, v_codes + r * vb, v_sc + r * nblk);
    }
}

RLO_API void rlo_compact_dequant(const int8_t* k_q, const uint16_t* k_sc, const uint8_t* v_codes,
                                 const uint16_t* v_sc, long T, int n_kv, int hd, int wht_len,
                                 const float* signs, float* k, float* v) {
    const int nblk = hd / wht_len;
    const int vb = hd * 3 / 8;
    for (long r = 0; r < T * n_kv; ++r) {
        rlo_q8k_dequant(k_q + r * hd, k_sc[r], hd, k + r * hd);
        rlo_tq3v_dequant(v_codes + r * vb, v_sc + r * nblk, hd, wht_len, signs, v + r * hd);
    }
}
