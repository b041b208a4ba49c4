// Runs EngineB200 (adapter/engine_b200.cpp) on a B200 against a stand-in dense side: the reference's
// own ModelDesc of the 27B qwen3_5 stack (make_qwen36_27b_desc, 64 layers, real mixer shapes; vocabulary
// and hidden size cut down, which the mixers never see) with projections replaced by seeded pseudo-random
// activations.  It checks that the adapter's walk over the layers -- chunked prefill of two prompts into
// two slots, batched decode steps, a one-sequence decode, replicate_slot0, zero_slots, spec_verify -- goes
// through every rl_* call without a host or device error and leaves finite outputs and the positions
// the Engine interface promises.  Test infrastructure; built by adapter/Makefile from the reference's
// headers and src/ir/model_desc.cpp where they lie.
#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <random>
#include <vector>

#include "engine_b200.h"

using namespace rapidllm;
using namespace rapidllm::cuda_gen;

namespace {

struct FakeDense final : DenseHooks {
    const ModelDesc& m;
    int rows_cap;
    float* pool = nullptr;          // seeded N(0,1) values the "projections" copy from
    size_t pool_n = 0;
    float* smalls = nullptr;
    int n_q, n_kv, hd, n_v, n_k, dk, dv, conv_dim;
    size_t cursor = 0;

    FakeDense(const ModelDesc& md, int rows) : m(md), rows_cap(rows) {
        const LayerDesc* A = nullptr;
        const LayerDesc* D = nullptr;
        for (const LayerDesc& L : m.layers) (L.kind == LayerKind::GatedDeltaNet ? D : A) = &L;
        n_q = A->attn.n_q, n_kv = A->attn.n_kv, hd = A->attn.head_dim;
        n_v = D->delta.n_v_heads, n_k = D->delta.n_k_heads, dk = D->delta.k_dim, dv = D->delta.v_dim;
        conv_dim = 2 * n_k * dk + n_v * dv;
        pool_n = size_t(rows) * (size_t(n_q) * 2 * hd + conv_dim) + (size_t(1) << 20);
        std::vector<float> h(pool_n);
        std::mt19937 rng(1234);
        std::normal_distribution<float> nd(0.f, 1.f);
        for (float& x : h) x = nd(rng);
        cudaMalloc(reinterpret_cast<void**>(&pool), pool_n * sizeof(float));
        cudaMemcpy(pool, h.data(), pool_n * sizeof(float), cudaMemcpyHostToDevice);
        std::vector<float> s(size_t(conv_dim) * 4 + 2 * hd + 2 * n_v + dv);
        for (float& x : s) x = 0.3f * nd(rng);
        cudaMalloc(reinterpret_cast<void**>(&smalls), s.size() * sizeof(float));
        cudaMemcpy(smalls, s.data(), s.size() * sizeof(float), cudaMemcpyHostToDevice);
    }
    ~FakeDense() override {
        cudaFree(pool);
        cudaFree(smalls);
    }
    // n values of the pool, from a position that moves with every call
    void fill(float* dst, size_t n, void* stream) {
        cursor = (cursor * 31 + 4099) % (pool_n - n);
        cursor -= cursor % 4;
        cudaMemcpyAsync(dst, pool + cursor, n * sizeof(float), cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    }
    void embed(const int32_t*, int rows, float* x, void* st) override { fill(x, size_t(rows) * m.hidden, st); }
    void attn_in(int, const float*, int rows, float* qg, float* k, float* v, void* st) override {
        fill(qg, size_t(rows) * n_q * 2 * hd, st);
        fill(k, size_t(rows) * n_kv * hd, st);
        fill(v, size_t(rows) * n_kv * hd, st);
    }
    void attn_out(int, const float*, int, float*, void*) override {}
    void delta_in(int, const float*, int rows, float* qkv, float* z, float* a, float* b, void* st) override {
        fill(qkv, size_t(rows) * conv_dim, st);
        fill(z, size_t(rows) * n_v * dv, st);
        fill(a, size_t(rows) * n_v, st);
        fill(b, size_t(rows) * n_v, st);
    }
    void delta_out(int, const float*, int, float*, void*) override {}
    void logits(const float*, int rows, float* lg, int32_t* greedy, void* st) override {
        fill(lg, size_t(rows) * m.vocab, st);
        cudaMemsetAsync(greedy, 0, sizeof(int32_t) * rows, static_cast<cudaStream_t>(st));
    }
    LayerSmall small(int) override {
        LayerSmall w;
        w.conv_w = smalls;
        w.q_norm = smalls + size_t(conv_dim) * 4;
        w.k_norm = w.q_norm + hd;
        w.A_log = w.k_norm + hd;
        w.dt_bias = w.A_log + n_v;
        w.gnorm = w.dt_bias + n_v;
        return w;
    }
};

int fail(const char* what) {
    std::printf("engine smoke FAILED: %s\n", what);
    return 1;
}

}  // namespace

int main() {
    if (!available()) return fail("no sm_100 device");
    WeightStore store;
    store.table().model = make_qwen36_27b_desc();
    store.table().model.vocab = 512;          // the dense side is a stand-in: keep its buffers small
    store.table().model.hidden = 256;
    const int ctx = 2048, max_batch = 4;
    try {
        EngineB200 eng(store, ctx, std::make_unique<FakeDense>(store.model(), 1024), max_batch);
        if (eng.max_batch() != max_batch || eng.vocab() != 512 || eng.hidden() != 256) return fail("shape getters");
        std::vector<int32_t> ids(1500);
        for (size_t i = 0; i < ids.size(); ++i) ids[i] = int32_t(i % 500);
        eng.prefill(ids.data(), 1500);                       // two chunks: 1024 + 476
        if (eng.pos() != 1500) return fail("pos after prefill");
        eng.prefill_slot(ids.data(), 70, 1);
        int32_t toks[2] = {5, 6};
        int poss[2] = {1500, 70};
        for (int step = 0; step < 3; ++step) {
            eng.decode_tokens(toks, poss, 2);
            ++poss[0], ++poss[1];
        }
        if (eng.pos() != 1503) return fail("pos after batched decode");
        eng.decode_token(7);
        if (eng.pos() != 1504) return fail("pos after decode_token");
        std::vector<float> logits(2 * 512);
        eng.copy_logits_n(logits.data(), 1);
        for (int i = 0; i < 512; ++i)
            if (!std::isfinite(logits[size_t(i)])) return fail("logits not finite");
        int32_t g[2] = {-1, -1};
        eng.copy_greedy_n(g, 1);
        if (g[0] != eng.greedy()) return fail("greedy");
        int32_t draft[3] = {1, 0, 0}, preds[3] = {-1, -1, -1};
        const int n = eng.spec_verify(draft, 3, preds);      // the stand-in argmax is always 0: all three drafted tokens pass
        if (n != 3 || eng.pos() != 1507) return fail("spec_verify");
        eng.replicate_slot0(3);
        int p3[3] = {1507, 1507, 1507};
        int32_t t3[3] = {1, 2, 3};
        eng.decode_tokens(t3, p3, 3);
        eng.zero_slots(max_batch);
        if (eng.pos() != 0) return fail("pos after zero_slots");
        eng.prefill(ids.data(), 33);
        eng.decode_token(1);
        if (eng.pos() != 34) return fail("pos after restart");
    } catch (const std::exception& e) {
        return fail(e.what());
    }
    std::printf("engine smoke ok\n");
    return 0;
}
