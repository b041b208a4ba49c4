// TEST INFRASTRUCTURE ONLY.  Nothing in the product path may link or load this.
//
// The reference states its compact KV cache (q8 K + TurboQuant-3 V) in CUDA only
// (src/kernels/cuda/cuda_engine.cu:199-299, 8224-8314, 8382-8454) and has no test vectors for
// it.  This shim compiles that translation unit where it lies (the Makefile passes its path as
// RL_REF_CUDA_TU and uses the reference's own compile flags) and adds C entry points that run the
// reference's own store / dequantise / decode kernels on host buffers, so that the tests can
// compare the library and the C restatement with the reference itself.
// Launch shapes are those of the reference's call sites (cuda_engine.cu:11702-11730, 18322-18336,
// 18967).  Nothing of the reference is copied: the kernels are reached through the include.
#include RL_REF_CUDA_TU

#include <cstdint>

namespace {

struct DevBuf {
    void* p = nullptr;
    cudaError_t err = cudaSuccess;
    DevBuf(size_t bytes, const void* host = nullptr) {
        err = cudaMalloc(&p, bytes ? bytes : 1);
        if (err == cudaSuccess && host) err = cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice);
    }
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    template <class T>
    T* as() const { return static_cast<T*>(p); }
};

int finish(cudaError_t e) {
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return static_cast<int>(e);
}

}  // namespace

using namespace rapidllm::cuda_gen;

extern "C" {

__attribute__((visibility("default"))) const char* rlref_cuda_error_string(int code) {
    return cudaGetErrorString(static_cast<cudaError_t>(code));
}

// store_k_q8_th_k + store_v_tq3_th_k over rows k, v fp32 [T][nkv][256] (host) ->
// kq int8 [T][nkv][256], ksc fp16 [T][nkv], vq u8 [T][nkv][2][48], vsc fp16 [T][nkv][2].
__attribute__((visibility("default"))) int rlref_cuda_compact_store(const float* k, const float* v, int T, int nkv,
                                                                    int8_t* kq, uint16_t* ksc, uint8_t* vq,
                                                                    uint16_t* vsc) {
    const int hd = 256, nblk = hd / kTqBlk;
    const size_t rows = size_t(T) * nkv;
    DevBuf dk(rows * hd * 4, k), dv(rows * hd * 4, v), dkq(rows * hd), dksc(rows * 2), dvq(rows * nblk * kTq3B),
        dvsc(rows * nblk * 2);
    for (const DevBuf* b : {&dk, &dv, &dkq, &dksc, &dvq, &dvsc})
        if (b->err != cudaSuccess) return static_cast<int>(b->err);
    store_k_q8_th_k<<<dim3(nkv, T), 256>>>(dkq.as<int8_t>(), dksc.as<__half>(), dk.as<float>(), 0, T, nkv, hd);
    store_v_tq3_th_k<<<dim3(nblk, nkv, T), 128, kTqBlk * sizeof(float)>>>(dvq.as<uint8_t>(), dvsc.as<__half>(),
                                                                          dv.as<float>(), 0, T, nkv, hd);
    if (int e = finish(cudaSuccess)) return e;
    cudaError_t e = cudaMemcpy(kq, dkq.p, rows * hd, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(ksc, dksc.p, rows * 2, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(vq, dvq.p, rows * nblk * kTq3B, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(vsc, dvsc.p, rows * nblk * 2, cudaMemcpyDeviceToHost);
    return static_cast<int>(e);
}

// dequant_k_q8_h_k + dequant_v_tq3_h_k: the rebuild of the F16 window -> k16, v16 fp16 [T][nkv][256].
__attribute__((visibility("default"))) int rlref_cuda_compact_dequant(const int8_t* kq, const uint16_t* ksc,
                                                                      const uint8_t* vq, const uint16_t* vsc, int T,
                                                                      int nkv, uint16_t* k16, uint16_t* v16) {
    const int hd = 256, nblk = hd / kTqBlk;
    const size_t rows = size_t(T) * nkv;
    DevBuf dkq(rows * hd, kq), dksc(rows * 2, ksc), dvq(rows * nblk * kTq3B, vq), dvsc(rows * nblk * 2, vsc),
        dk(rows * hd * 2), dv(rows * hd * 2);
    for (const DevBuf* b : {&dkq, &dksc, &dvq, &dvsc, &dk, &dv})
        if (b->err != cudaSuccess) return static_cast<int>(b->err);
    dequant_k_q8_h_k<<<dim3(nkv, T), 256>>>(dk.as<__half>(), dkq.as<int8_t>(), dksc.as<__half>(), 0, T, nkv, hd);
    dequant_v_tq3_h_k<<<dim3(nblk, nkv, T), 128, kTqBlk * sizeof(float)>>>(dv.as<__half>(), dvq.as<uint8_t>(),
                                                                           dvsc.as<__half>(), 0, T, nkv, hd);
    if (int e = finish(cudaSuccess)) return e;
    cudaError_t e = cudaMemcpy(k16, dk.p, rows * hd * 2, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(v16, dv.p, rows * hd * 2, cudaMemcpyDeviceToHost);
    return static_cast<int>(e);
}

// qk_attn_decode_tq_gqa_k: one sequence, tokens [0, pos] of the compact cache; q, o fp32 [n_q][256].
__attribute__((visibility("default"))) int rlref_cuda_attn_decode_tq(const float* q, int pos, int n_q, int n_kv,
                                                                     const int8_t* kq, const uint16_t* ksc,
                                                                     const uint8_t* vq, const uint16_t* vsc, int T,
                                                                     float* o) {
    const int hd = 256, nblk = hd / kTqBlk;
    if (pos < 0 || pos >= T) return static_cast<int>(cudaErrorInvalidValue);
    const size_t rows = size_t(T) * n_kv;
    DevBuf dq(size_t(n_q) * hd * 4, q), dor(size_t(n_q) * hd * 4), dpos(4, &pos), dkq(rows * hd, kq),
        dksc(rows * 2, ksc), dvq(rows * nblk * kTq3B, vq), dvsc(rows * nblk * 2, vsc);
    for (const DevBuf* b : {&dq, &dor, &dpos, &dkq, &dksc, &dvq, &dvsc})
        if (b->err != cudaSuccess) return static_cast<int>(b->err);
    qk_attn_decode_tq_gqa_k<<<n_kv, 256>>>(dq.as<float>(), dor.as<float>(), dpos.as<int>(), n_q, n_kv, hd,
                                           dkq.as<int8_t>(), dksc.as<__half>(), dvq.as<uint8_t>(),
                                           dvsc.as<__half>());
    if (int e = finish(cudaSuccess)) return e;
    return static_cast<int>(cudaMemcpy(o, dor.p, size_t(n_q) * hd * 4, cudaMemcpyDeviceToHost));
}

}  // extern "C"
