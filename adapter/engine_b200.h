// EngineB200: the reference's CUDA engine interface (rapidllm::cuda_gen::Engine,
// include/rapidllm/runtime/cuda_engine.h:13-83) implemented over the rl_* C ABI (include/rl_b200.h).
//
// Session selects a cuda_gen::Engine when `--device cuda` is given and available() holds
// (src/runtime/session.cpp:22-30).  This translation unit is what a RapidLLM build links in place
// of src/kernels/cuda/cuda_engine.cu (or of the stub, cuda_engine_stub.cpp:3-13) to run the
// qwen3_5 mixers -- Gated Attention over the paged KV cache and Gated DeltaNet over the FP32
// state cache -- on B200.  It owns the device-side cache (rl_cache = DualCache on the device),
// the page table and the walk over ModelDesc::layers[] (the scheduler dispatch of
// launch_decode_batch, cuda_engine.cu:18999-19106, and of the chunked prefill driver,
// 18854-18873).
//
// What it does NOT own is every dense linear: embedding, the in/out projections of the mixers,
// the MLP blocks, the final norm, lm_head and the argmax.  Those stay with the host engine's own
// GEMV / cuBLASLt code and weight loaders (FP8 safetensors, GGUF), which are outside this
// library; the adapter reaches them through DenseHooks.  All hook arguments are device pointers,
// fp32 row-major, enqueued on `stream`.
#pragma once

#include <cstdint>
#include <memory>
#include <vector>

#include "rapidllm/runtime/cuda_engine.h"
#include "rl_b200.h"

namespace rapidllm::cuda_gen {

struct DenseHooks {
    virtual ~DenseHooks() = default;
    // x [rows][hidden] = embedding rows of the tokens (device int32)
    virtual void embed(const int32_t* tokens, int rows, float* x, void* stream) = 0;
    // Gated Attention layer `layer` (index in ModelDesc::layers): input RMSNorm, then
    // qg [rows][n_q][2*hd] = wq x ([q | gate] per head), k, v [rows][n_kv][hd] = wk x, wv x
    // (src/kernels/ops_fused.cpp:151-162)
    virtual void attn_in(int layer, const float* x, int rows, float* qg, float* k, float* v, void* stream) = 0;
    // x += wo o, followed by the layer's post-attention norm + MLP block (ops_fused.cpp:180-182,
    // src/runtime/session.cpp:386-404); o [rows][n_q][hd] is already gated
    virtual void attn_out(int layer, const float* o, int rows, float* x, void* stream) = 0;
    // Gated DeltaNet layer: input RMSNorm, then qkv [rows][conv_dim] (q | k | v channels before the
    // conv), z [rows][n_v][dv], a, b [rows][n_v] (ops_fused.cpp:99-110)
    virtual void delta_in(int layer, const float* x, int rows, float* qkv, float* z, float* a, float* b,
                          void* stream) = 0;
    // x += out_proj y, then the MLP block; y [rows][n_v][dv] is the gated-normed delta-rule output
    virtual void delta_out(int layer, const float* y, int rows, float* x, void* stream) = 0;
    // final RMSNorm + lm_head over the given rows, argmax per row into greedy (device)
    virtual void logits(const float* x, int rows, float* logits, int32_t* greedy, void* stream) = 0;
    // device copies of the small per-layer tensors the mixers read themselves
    struct LayerSmall {
        const float* q_norm = nullptr;     // [hd]      attention
        const float* k_norm = nullptr;     // [hd]
        const float* conv_w = nullptr;     // [conv_dim][4]  DeltaNet, taps oldest first
        const float* A_log = nullptr;      // [n_v]
        const float* dt_bias = nullptr;    // [n_v]
        const float* gnorm = nullptr;      // [dv]      gated RMSNorm weight
    };
    virtual LayerSmall small(int layer) = 0;
};

// Provided by the host engine (its linear-algebra and weight-loading side).  A build without one
// links the weak default, which returns null: Engine::create then returns null and Session falls
// back to its CPU path, exactly as with the reference's stub.
std::unique_ptr<DenseHooks> make_dense_hooks(WeightStore& store, int max_rows);

class EngineB200 final : public Engine {
public:
    EngineB200(WeightStore& store, int ctx, std::unique_ptr<DenseHooks> dense, int max_batch);
    ~EngineB200() override;

    void prefill(const int32_t* ids, int n) override { prefill_slot(ids, n, 0); }
    void decode_token(int32_t token) override;
    void copy_logits(float* host) const override { copy_logits_n(host, 1); }
    int32_t greedy() const override { return greedy_host_.empty() ? 0 : greedy_host_[0]; }
    int pos() const override { return pos_host_.empty() ? 0 : pos_host_[0]; }
    int vocab() const override { return vocab_; }
    int hidden() const override { return hidden_; }
    int max_batch() const override { return max_batch_; }
    void decode_tokens(const int32_t* tokens, const int* poss, int B) override;
    void copy_logits_n(float* host, int B) const override;
    void copy_greedy_n(int32_t* host, int B) override;
    void replicate_slot0(int n_slots) override;
    void zero_slots(int n_slots) override;
    void prefill_slot(const int32_t* ids, int n, int slot) override;
    int spec_verify(const int32_t* toks, int T, int32_t* preds) override;

private:
    void step(const int32_t* tokens, const int* poss, const int* slots, int B);
    void chunk(const int32_t* ids, int T, int slot, int pos0);
    void check(int status, const char* what) const;

    const ModelDesc* m_ = nullptr;
    std::unique_ptr<DenseHooks> dense_;
    rl_cache* cache_ = nullptr;
    void* stream_ = nullptr;
    int ctx_ = 0, vocab_ = 0, hidden_ = 0, max_batch_ = 1, max_pages_per_seq_ = 0, pf_cap_ = 1024;
    int n_q_ = 0, n_kv_ = 0, hd_ = 0, n_v_ = 0, n_k_ = 0, dk_ = 0, dv_ = 0, conv_dim_ = 0, rotary_dim_ = 0;
    std::vector<int> types_, slot_of_layer_;
    // device buffers (sized for max(max_batch, pf_cap) rows)
    float *x_ = nullptr, *qg_ = nullptr, *k_ = nullptr, *v_ = nullptr, *q_ = nullptr, *gate_ = nullptr, *o_ = nullptr;
    float *qkv_ = nullptr, *z_ = nullptr, *a_ = nullptr, *b_ = nullptr, *beta_ = nullptr, *g_ = nullptr, *dy_ = nullptr;
    float* logits_ = nullptr;
    void *q16_ = nullptr, *k16_ = nullptr, *v16_ = nullptr, *ws_ = nullptr;
    size_t ws_bytes_ = 0;
    int32_t *tok_ = nullptr, *pos_ = nullptr, *slots_ = nullptr, *greedy_ = nullptr, *table_ = nullptr;
    std::vector<int32_t> greedy_host_, pos_host_;
    int last_rows_ = 0;
};

}  // namespace rapidllm::cuda_gen
