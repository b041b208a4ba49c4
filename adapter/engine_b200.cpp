// See engine_b200.h.  Built inside a RapidLLM tree in place of src/kernels/cuda/cuda_engine.cu:
//   g++ -std=c++20 -I<rapidllm>/include -I<this repo>/include -I<cuda>/include -c adapter/engine_b200.cpp
//   ... -L<this repo>/rapidllm_b200 -lrl_b200 -lcudart
#include "engine_b200.h"

#include <cuda_runtime_api.h>

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>

namespace rapidllm::cuda_gen {

namespace {

void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("CUDA: ") + what + ": " + cudaGetErrorString(e));
}

template <class T>
T* dev_alloc(size_t n) {
    void* p = nullptr;
    cuda_check(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)), "cudaMalloc");
    return static_cast<T*>(p);
}

}  // namespace

// cuda_gen::available() (cuda_engine.h:11): a B200-class device is present.
bool available() { return rl_b200_available() != 0; }

__attribute__((weak)) std::unique_ptr<DenseHooks> make_dense_hooks(WeightStore&, int) { return nullptr; }

// Engine::create (cuda_engine.h:15): null when the host engine supplies no dense side, like the stub.
std::unique_ptr<Engine> Engine::create(WeightStore& store, int ctx) {
    if (!available()) return nullptr;
    const int max_batch = 32;                 // the reference's continuous-batch ceiling is a build constant too
    std::unique_ptr<DenseHooks> dense = make_dense_hooks(store, std::max(max_batch, 1024));
    if (!dense) return nullptr;
    return std::make_unique<EngineB200>(store, ctx, std::move(dense), max_batch);
}

void EngineB200::check(int status, const char* what) const {
    if (status != RL_OK) throw std::runtime_error(std::string(what) + ": " + rl_last_error());
}

EngineB200::EngineB200(WeightStore& store, int ctx, std::unique_ptr<DenseHooks> dense, int max_batch)
    : m_(&store.model()), dense_(std::move(dense)), ctx_(ctx), max_batch_(max_batch) {
    const ModelDesc& m = *m_;
    vocab_ = m.vocab;
    hidden_ = m.hidden;
    int n_attn = 0, n_delta = 0;
    for (int i = 0; i < m.n_layers; ++i) {
        const LayerDesc& L = m.layers[static_cast<size_t>(i)];
        const bool attn = L.kind != LayerKind::GatedDeltaNet;
        types_.push_back(attn ? RL_LAYER_FULL_ATTENTION : RL_LAYER_LINEAR_ATTENTION);
        slot_of_layer_.push_back(m.mixer_slot(i));            // index among the layers of its kind
        if (attn) {
            ++n_attn;
            n_q_ = L.attn.n_q, n_kv_ = L.attn.n_kv, hd_ = L.attn.head_dim;
        } else {
            ++n_delta;
            n_v_ = L.delta.n_v_heads, n_k_ = L.delta.n_k_heads, dk_ = L.delta.k_dim, dv_ = L.delta.v_dim;
        }
    }
    conv_dim_ = 2 * n_k_ * dk_ + n_v_ * dv_;
    rotary_dim_ = static_cast<int>(hd_ * m.rope.partial_factor);
    // memory plan: pages out of what is free now (planner.cpp:28-44), F16 when it fits, else refuse
    size_t free_b = 0, total_b = 0;
    cuda_check(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo");
    rl_plan_input pin;
    std::memset(&pin, 0, sizeof pin);
    pin.available_bytes = free_b;
    pin.pad_bytes = 64ull << 20;
    pin.ctx = ctx;
    pin.max_batch = max_batch_;
    pin.n_attn_layers = n_attn, pin.n_kv = n_kv_, pin.head_dim = hd_;
    pin.n_delta_layers = n_delta, pin.n_v = n_v_, pin.dk = dk_, pin.dv = dv_, pin.conv_dim = conv_dim_, pin.conv_k = 4;
    pin.page_tokens = 64;
    pin.kv_policy = RL_KV_POLICY_F16;
    pin.allow_shrink = 1;
    pin.prefill_chunk = pf_cap_;
    rl_plan_result plan;
    check(rl_plan_cache(&pin, &plan), "rl_plan_cache");
    if (!plan.ok) throw std::runtime_error(std::string("KV plan: ") + plan.message);
    ctx_ = plan.ctx;
    max_pages_per_seq_ = plan.max_pages_per_seq;
    rl_cache_config cfg;
    std::memset(&cfg, 0, sizeof cfg);
    cfg.n_layers = m.n_layers;
    cfg.layer_types = types_.data();
    cfg.n_q = n_q_, cfg.n_kv = n_kv_, cfg.head_dim = hd_;
    cfg.kv_dtype = RL_KV_F16;
    cfg.page_tokens = 64, cfg.n_pages = plan.n_pages;
    cfg.n_v = n_v_, cfg.n_k = n_k_, cfg.dk = dk_, cfg.dv = dv_, cfg.conv_k = 4;
    cfg.head_map = m.gdn_v_tiled ? RL_HEADS_TILED : RL_HEADS_GROUPED;
    cfg.n_slots = max_batch_, cfg.max_batch = max_batch_;
    cfg.max_pages_per_seq = max_pages_per_seq_, cfg.max_seq_len = ctx_;
    check(rl_cache_create(&cfg, &cache_), "rl_cache_create");
    cudaStream_t st = nullptr;
    cuda_check(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking), "cudaStreamCreate");
    stream_ = st;
    const size_t rows = static_cast<size_t>(std::max(max_batch_, pf_cap_));
    x_ = dev_alloc<float>(rows * hidden_);
    qg_ = dev_alloc<float>(rows * n_q_ * 2 * hd_);
    k_ = dev_alloc<float>(rows * n_kv_ * hd_);
    v_ = dev_alloc<float>(rows * n_kv_ * hd_);
    q_ = dev_alloc<float>(rows * n_q_ * hd_);
    gate_ = dev_alloc<float>(rows * n_q_ * hd_);
    o_ = dev_alloc<float>(rows * n_q_ * hd_);
    qkv_ = dev_alloc<float>(rows * conv_dim_);
    z_ = dev_alloc<float>(rows * n_v_ * dv_);
    a_ = dev_alloc<float>(rows * n_v_);
    b_ = dev_alloc<float>(rows * n_v_);
    beta_ = dev_alloc<float>(rows * n_v_);
    g_ = dev_alloc<float>(rows * n_v_);
    dy_ = dev_alloc<float>(rows * n_v_ * dv_);
    logits_ = dev_alloc<float>(static_cast<size_t>(max_batch_) * vocab_);
    q16_ = dev_alloc<uint16_t>(rows * n_q_ * hd_);
    k16_ = dev_alloc<uint16_t>(rows * n_kv_ * hd_);
    v16_ = dev_alloc<uint16_t>(rows * n_kv_ * hd_);
    tok_ = dev_alloc<int32_t>(rows);
    pos_ = dev_alloc<int32_t>(rows);
    slots_ = dev_alloc<int32_t>(rows);
    greedy_ = dev_alloc<int32_t>(rows);
    // page table: slot s owns pages [s * max_pages_per_seq, (s + 1) * max_pages_per_seq) of every pool
    std::vector<int32_t> table(static_cast<size_t>(max_batch_) * max_pages_per_seq_);
    for (size_t i = 0; i < table.size(); ++i) table[i] = static_cast<int32_t>(i);
    table_ = dev_alloc<int32_t>(table.size());
    cuda_check(cudaMemcpy(table_, table.data(), table.size() * sizeof(int32_t), cudaMemcpyHostToDevice), "page table");
    // scratch: decode split-KV partials, or one prefill chunk's attention split and DeltaNet records
    rl_attn_decode_params dp;
    std::memset(&dp, 0, sizeof dp);
    dp.n_q = n_q_, dp.n_kv = n_kv_, dp.head_dim = hd_, dp.kv_dtype = RL_KV_F16, dp.batch = max_batch_;
    dp.page_tokens = 64, dp.n_pages = plan.n_pages, dp.max_pages_per_seq = max_pages_per_seq_, dp.max_seq_len = ctx_;
    ws_bytes_ = rl_attn_decode_workspace_bytes(&dp);
    rl_attn_prefill_params pp;
    std::memset(&pp, 0, sizeof pp);
    pp.n_q = n_q_, pp.n_kv = n_kv_, pp.head_dim = hd_, pp.seq = pf_cap_, pp.br = 128, pp.bc = 64;
    pp.pos0 = std::max(0, ctx_ - pf_cap_), pp.page_tokens = 64, pp.n_pages = plan.n_pages, pp.n_table = max_pages_per_seq_;
    ws_bytes_ = std::max(ws_bytes_, rl_attn_prefill_workspace_bytes(&pp));
    ws_bytes_ = std::max(ws_bytes_, rl_cache_delta_prefill_workspace_bytes(cache_, pf_cap_));
    ws_ = dev_alloc<unsigned char>(ws_bytes_ + 256);
    greedy_host_.assign(static_cast<size_t>(max_batch_), 0);
    pos_host_.assign(static_cast<size_t>(max_batch_), 0);
}

EngineB200::~EngineB200() {
    if (stream_) cudaStreamSynchronize(static_cast<cudaStream_t>(stream_));
    rl_cache_destroy(cache_);
    for (void* p : {static_cast<void*>(x_), static_cast<void*>(qg_), static_cast<void*>(k_), static_cast<void*>(v_),
                    static_cast<void*>(q_), static_cast<void*>(gate_), static_cast<void*>(o_), static_cast<void*>(qkv_),
                    static_cast<void*>(z_), static_cast<void*>(a_), static_cast<void*>(b_), static_cast<void*>(beta_),
                    static_cast<void*>(g_), static_cast<void*>(dy_), static_cast<void*>(logits_), q16_, k16_, v16_, ws_,
                    static_cast<void*>(tok_), static_cast<void*>(pos_), static_cast<void*>(slots_),
                    static_cast<void*>(greedy_), static_cast<void*>(table_)})
        if (p) cudaFree(p);
    if (stream_) cudaStreamDestroy(static_cast<cudaStream_t>(stream_));
}

// One decode step of B sequences: launch_decode_batch (cuda_engine.cu:18999-19106) over the rl_* operators.
void EngineB200::step(const int32_t* tokens, const int* poss, const int* slots, int B) {
    if (B < 1 || B > max_batch_) throw std::runtime_error("decode batch outside [1, max_batch]");
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    std::vector<int32_t> pos32(poss, poss + B), slot32(slots, slots + B);
    for (int b = 0; b < B; ++b)
        if (pos32[static_cast<size_t>(b)] < 0 || pos32[static_cast<size_t>(b)] >= ctx_) throw std::runtime_error("position outside the context");
    cuda_check(cudaMemcpyAsync(tok_, tokens, sizeof(int32_t) * B, cudaMemcpyHostToDevice, st), "tokens");
    cuda_check(cudaMemcpyAsync(pos_, pos32.data(), sizeof(int32_t) * B, cudaMemcpyHostToDevice, st), "positions");
    cuda_check(cudaMemcpyAsync(slots_, slot32.data(), sizeof(int32_t) * B, cudaMemcpyHostToDevice, st), "slots");
    // the page-table rows of the sequences in this batch, in batch order
    int32_t* rows = table_;                    // identity slots: rows are already in place
    bool identity = true;
    for (int b = 0; b < B; ++b) identity = identity && slots[b] == b;
    if (!identity) throw std::runtime_error("decode_tokens expects sequence b in cache slot b");
    dense_->embed(tok_, B, x_, stream_);
    for (int i = 0; i < m_->n_layers; ++i) {
        const DenseHooks::LayerSmall w = dense_->small(i);
        const int s = slot_of_layer_[static_cast<size_t>(i)];
        if (types_[static_cast<size_t>(i)] == RL_LAYER_FULL_ATTENTION) {
            dense_->attn_in(i, x_, B, qg_, k_, v_, stream_);
            rl_attn_qk_prepare_params qp;
            qp.n_q = n_q_, qp.n_kv = n_kv_, qp.head_dim = hd_, qp.rotary_dim = rotary_dim_, qp.rows = B, qp.pos0 = 0;
            qp.theta = m_->rope.theta, qp.eps = m_->rms_eps;
            check(rl_attn_qk_prepare(qg_, k_, w.q_norm, w.k_norm, pos_, q_, gate_, &qp, stream_), "rl_attn_qk_prepare");
            rl_kv_append_params ap;
            std::memset(&ap, 0, sizeof ap);
            ap.n_kv = n_kv_, ap.head_dim = hd_, ap.batch = B, ap.n_tok = 1, ap.page_tokens = 64;
            ap.n_pages = max_batch_ * max_pages_per_seq_, ap.max_pages_per_seq = max_pages_per_seq_;
            check(rl_kv_append(rl_cache_k_pool(cache_, s), rl_cache_v_pool(cache_, s), rows, pos_, k_, v_, &ap, stream_),
                  "rl_kv_append");
            rl_attn_decode_params dp;
            std::memset(&dp, 0, sizeof dp);
            dp.n_q = n_q_, dp.n_kv = n_kv_, dp.head_dim = hd_, dp.kv_dtype = RL_KV_F16, dp.batch = B, dp.page_tokens = 64;
            dp.n_pages = ap.n_pages, dp.max_pages_per_seq = max_pages_per_seq_, dp.max_seq_len = ctx_, dp.len_add = 1;
            check(rl_attn_decode(rl_cache_k_pool(cache_, s), rl_cache_v_pool(cache_, s), rows, pos_, q_, gate_, o_, ws_,
                                 ws_bytes_, &dp, stream_),
                  "rl_attn_decode");
            dense_->attn_out(i, o_, B, x_, stream_);
        } else {
            dense_->delta_in(i, x_, B, qkv_, z_, a_, b_, stream_);
            check(rl_delta_gates(a_, b_, w.A_log, w.dt_bias, beta_, g_, B, n_v_, stream_), "rl_delta_gates");
            rl_gdn_decode_params gp;
            gp.n_v = n_v_, gp.n_qk = n_k_, gp.dk = dk_, gp.dv = dv_, gp.conv_k = 4, gp.batch = B, gp.n_slots = max_batch_;
            gp.head_map = m_->gdn_v_tiled ? RL_HEADS_TILED : RL_HEADS_GROUPED;
            gp.eps_l2 = 1e-6f;
            check(rl_gdn_decode(rl_cache_state(cache_, s), rl_cache_conv(cache_, s), rl_cache_conv_phase(cache_, s), slots_,
                                qkv_, w.conv_w, beta_, g_, dy_, &gp, stream_),
                  "rl_gdn_decode");
            check(rl_gated_rmsnorm(dy_, z_, w.gnorm, dy_, B, n_v_, dv_, m_->rms_eps, stream_), "rl_gated_rmsnorm");
            dense_->delta_out(i, dy_, B, x_, stream_);
        }
    }
    // every DeltaNet layer has taken its token: move the conv rings on (phases of all layers are contiguous)
    int n_delta = 0;
    for (int t : types_) n_delta += t == RL_LAYER_LINEAR_ATTENTION;
    if (n_delta) check(rl_gdn_phase_advance(rl_cache_conv_phase(cache_, 0), slots_, n_delta, max_batch_, B, 1, stream_), "rl_gdn_phase_advance");
    dense_->logits(x_, B, logits_, greedy_, stream_);
    cuda_check(cudaMemcpyAsync(greedy_host_.data(), greedy_, sizeof(int32_t) * B, cudaMemcpyDeviceToHost, st), "greedy");
    cuda_check(cudaStreamSynchronize(st), "decode step");
    if (int code = rl_device_error(stream_)) throw std::runtime_error(std::string("device: ") + rl_device_error_string(code));
    for (int b = 0; b < B; ++b) pos_host_[static_cast<size_t>(b)] = poss[b] + 1;
    last_rows_ = B;
}

void EngineB200::decode_token(int32_t token) {
    const int p = pos_host_[0], s = 0;
    step(&token, &p, &s, 1);
}

void EngineB200::decode_tokens(const int32_t* tokens, const int* poss, int B) {
    std::vector<int> slots(static_cast<size_t>(B));
    for (int b = 0; b < B; ++b) slots[static_cast<size_t>(b)] = b;
    step(tokens, poss, slots.data(), B);
}

// One chunk of a prompt: launch_prefill_chunk (cuda_engine.cu:18338-18590) over the rl_* operators.
void EngineB200::chunk(const int32_t* ids, int T, int slot, int pos0) {
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    cuda_check(cudaMemcpyAsync(tok_, ids, sizeof(int32_t) * T, cudaMemcpyHostToDevice, st), "prompt tokens");
    const int32_t* row = table_ + static_cast<size_t>(slot) * max_pages_per_seq_;
    dense_->embed(tok_, T, x_, stream_);
    for (int i = 0; i < m_->n_layers; ++i) {
        const DenseHooks::LayerSmall w = dense_->small(i);
        const int s = slot_of_layer_[static_cast<size_t>(i)];
        if (types_[static_cast<size_t>(i)] == RL_LAYER_FULL_ATTENTION) {
            dense_->attn_in(i, x_, T, qg_, k_, v_, stream_);
            rl_attn_qk_prepare_params qp;
            qp.n_q = n_q_, qp.n_kv = n_kv_, qp.head_dim = hd_, qp.rotary_dim = rotary_dim_, qp.rows = T, qp.pos0 = pos0;
            qp.theta = m_->rope.theta, qp.eps = m_->rms_eps;
            check(rl_attn_qk_prepare(qg_, k_, w.q_norm, w.k_norm, nullptr, q_, gate_, &qp, stream_), "rl_attn_qk_prepare");
            check(rl_cast_f32_to_bf16(q_, q16_, static_cast<size_t>(T) * n_q_ * hd_, stream_), "cast q");
            check(rl_cast_f32_to_bf16(k_, k16_, static_cast<size_t>(T) * n_kv_ * hd_, stream_), "cast k");
            check(rl_cast_f32_to_bf16(v_, v16_, static_cast<size_t>(T) * n_kv_ * hd_, stream_), "cast v");
            rl_attn_prefill_params pp;
            std::memset(&pp, 0, sizeof pp);
            pp.n_q = n_q_, pp.n_kv = n_kv_, pp.head_dim = hd_, pp.seq = T, pp.br = 128, pp.bc = 64, pp.pos0 = pos0;
            pp.page_tokens = 64, pp.n_pages = max_batch_ * max_pages_per_seq_, pp.n_table = max_pages_per_seq_;
            check(rl_attn_prefill_ws(rl_cache_k_pool(cache_, s), rl_cache_v_pool(cache_, s), row, q16_, k16_, v16_, gate_, o_,
                                     ws_, ws_bytes_, &pp, stream_),
                  "rl_attn_prefill");
            dense_->attn_out(i, o_, T, x_, stream_);
        } else {
            dense_->delta_in(i, x_, T, qkv_, z_, a_, b_, stream_);
            check(rl_delta_gates(a_, b_, w.A_log, w.dt_bias, beta_, g_, T, n_v_, stream_), "rl_delta_gates");
            check(rl_cache_delta_prefill(cache_, s, slot, pos0, T, qkv_, w.conv_w, beta_, g_, dy_, ws_, ws_bytes_, stream_),
                  "rl_cache_delta_prefill");
            check(rl_gated_rmsnorm(dy_, z_, w.gnorm, dy_, T, n_v_, dv_, m_->rms_eps, stream_), "rl_gated_rmsnorm");
            dense_->delta_out(i, dy_, T, x_, stream_);
        }
    }
    last_rows_ = T;
}

void EngineB200::prefill_slot(const int32_t* ids, int n, int slot) {
    if (slot < 0 || slot >= max_batch_) throw std::runtime_error("prefill slot outside the cache");
    if (n < 1 || n > ctx_) throw std::runtime_error("prompt longer than the context");
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    for (int pos0 = 0; pos0 < n; pos0 += pf_cap_) chunk(ids + pos0, std::min(pf_cap_, n - pos0), slot, pos0);
    // logits of the last prompt token only (row T - 1 of the last chunk)
    const int T_last = last_rows_;
    dense_->logits(x_ + static_cast<size_t>(T_last - 1) * hidden_, 1, logits_ + static_cast<size_t>(slot) * vocab_,
                   greedy_ + slot, stream_);
    cuda_check(cudaMemcpyAsync(&greedy_host_[static_cast<size_t>(slot)], greedy_ + slot, sizeof(int32_t),
                               cudaMemcpyDeviceToHost, st), "greedy");
    cuda_check(cudaStreamSynchronize(st), "prefill");
    if (int code = rl_device_error(stream_)) throw std::runtime_error(std::string("device: ") + rl_device_error_string(code));
    pos_host_[static_cast<size_t>(slot)] = n;
}

void EngineB200::copy_logits_n(float* host, int B) const {
    cuda_check(cudaMemcpy(host, logits_, sizeof(float) * static_cast<size_t>(B) * vocab_, cudaMemcpyDeviceToHost), "logits");
}

void EngineB200::copy_greedy_n(int32_t* host, int B) {
    std::copy(greedy_host_.begin(), greedy_host_.begin() + B, host);
}

// DualCache::zero for the first n_slots sequences (the whole cache when that is all of them).
void EngineB200::zero_slots(int n_slots) {
    if (n_slots >= max_batch_) {
        check(rl_cache_zero(cache_, stream_), "rl_cache_zero");
    } else {
        int n_delta = 0;
        for (int t : types_) n_delta += t == RL_LAYER_LINEAR_ATTENTION;
        const size_t s_bytes = sizeof(float) * n_v_ * dk_ * dv_, c_bytes = sizeof(float) * conv_dim_ * 4;
        for (int d = 0; d < n_delta; ++d) {
            cuda_check(cudaMemsetAsync(rl_cache_state(cache_, d), 0, s_bytes * n_slots, static_cast<cudaStream_t>(stream_)), "zero S");
            cuda_check(cudaMemsetAsync(rl_cache_conv(cache_, d), 0, c_bytes * n_slots, static_cast<cudaStream_t>(stream_)), "zero conv");
            cuda_check(cudaMemsetAsync(rl_cache_conv_phase(cache_, d), 0, sizeof(int32_t) * n_slots, static_cast<cudaStream_t>(stream_)), "zero phase");
        }
    }
    std::fill(pos_host_.begin(), pos_host_.begin() + std::min(n_slots, max_batch_), 0);
}

// Copy sequence 0's KV pages, recurrent state and conv windows into slots 1 .. n_slots-1.
void EngineB200::replicate_slot0(int n_slots) {
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    n_slots = std::min(n_slots, max_batch_);
    int n_attn = 0, n_delta = 0;
    for (int t : types_) (t == RL_LAYER_FULL_ATTENTION ? n_attn : n_delta)++;
    const size_t seq_kv = sizeof(uint16_t) * static_cast<size_t>(max_pages_per_seq_) * n_kv_ * 64 * hd_;   // one slot's pages of one pool
    const size_t s_bytes = sizeof(float) * n_v_ * dk_ * dv_, c_bytes = sizeof(float) * conv_dim_ * 4;
    for (int s = 1; s < n_slots; ++s) {
        for (int a = 0; a < n_attn; ++a) {
            char* kp = static_cast<char*>(rl_cache_k_pool(cache_, a));
            char* vp = static_cast<char*>(rl_cache_v_pool(cache_, a));
            cuda_check(cudaMemcpyAsync(kp + s * seq_kv, kp, seq_kv, cudaMemcpyDeviceToDevice, st), "replicate K");
            cuda_check(cudaMemcpyAsync(vp + s * seq_kv, vp, seq_kv, cudaMemcpyDeviceToDevice, st), "replicate V");
        }
        for (int d = 0; d < n_delta; ++d) {
            char* S = reinterpret_cast<char*>(rl_cache_state(cache_, d));
            char* C = reinterpret_cast<char*>(rl_cache_conv(cache_, d));
            int32_t* ph = rl_cache_conv_phase(cache_, d);
            cuda_check(cudaMemcpyAsync(S + s * s_bytes, S, s_bytes, cudaMemcpyDeviceToDevice, st), "replicate S");
            cuda_check(cudaMemcpyAsync(C + s * c_bytes, C, c_bytes, cudaMemcpyDeviceToDevice, st), "replicate conv");
            cuda_check(cudaMemcpyAsync(ph + s, ph, sizeof(int32_t), cudaMemcpyDeviceToDevice, st), "replicate phase");
        }
        pos_host_[static_cast<size_t>(s)] = pos_host_[0];
        greedy_host_[static_cast<size_t>(s)] = greedy_host_[0];
    }
    cuda_check(cudaStreamSynchronize(st), "replicate_slot0");
}

// Engine::spec_verify (cuda_engine.h:72-82): consume the drafted tokens one step at a time and stop at the
// first one the model disagrees with -- the state then never holds a rejected token, so nothing has to be
// rolled back.  (The several-tokens-per-pass form with a state backup is rl_delta_recurrent_multi +
// rl_attn_prefill over the verify rows; the dense side must then run T rows per pass as well.)
int EngineB200::spec_verify(const int32_t* toks, int T, int32_t* preds) {
    if (T <= 0 || !toks) return 0;
    int n = 0;
    for (int i = 0; i < T; ++i) {
        decode_token(toks[i]);
        if (preds) preds[i] = greedy();
        ++n;
        if (i + 1 < T && greedy() != toks[i + 1]) break;
    }
    return n;
}

}  // namespace rapidllm::cuda_gen
