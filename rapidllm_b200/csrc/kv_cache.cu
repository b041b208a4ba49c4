// Paged F16 KV cache maintenance: append / bulk write of K,V rows and gather back.
//
// The reference appends rows into a contiguous [pos][n_kv][hd] cache
// (src/runtime/dual_cache.cpp:74-79; CUDA store_kv_batch_h_k,
// src/kernels/cuda/cuda_engine.cu:8216-8221, __float2half = round to nearest
// even).  Here token s of a sequence lives in page table[s / 64], row s % 64 of
// the (page, head) slice, in the swizzled tile format of kv_slice_offset().
#include "common.cuh"
#include "kernels.h"

namespace rl {

// grid (ceil(n_tok / blockDim.y), n_kv, batch), block (32, 1 or 8): one token row per warp, one
// 16-byte chunk (8 dims) per thread.
__device__ __forceinline__ void kv_write_rows(const KvWriteArgs& a) {
    const int t = blockIdx.x * blockDim.y + threadIdx.y, h = blockIdx.y, b = blockIdx.z;
    const int lane = threadIdx.x;
    if (t >= a.n_tok) return;
    const int pos = (a.pos ? a.pos[b] : a.pos0) + t;
    if (a.pos_limit > 0 && pos >= a.pos_limit) return;
    const int pi = pos / kPageTokens;
    if (pos < 0 || pi >= a.max_pages_per_seq) {
        if (lane == 0) set_err(a.err, DEV_ERR_BAD_LEN);
        return;
    }
    const int page = a.page_table[size_t(b) * a.max_pages_per_seq + pi];
    if (page < 0 || page >= a.n_pages) {
        if (lane == 0) set_err(a.err, DEV_ERR_BAD_PAGE);
        return;
    }
    const int row = pos % kPageTokens;
    const size_t src = ((size_t(b) * a.n_tok + t) * a.n_kv + h) * kHeadDim + lane * 8;
    const size_t dst = (size_t(page) * a.n_kv + h) * kv_slice_elems() + kv_slice_offset(row, lane * 8);
    uint4 kk, vv;
    if (a.rows_fp16 == 1) {
        kk = *reinterpret_cast<const uint4*>(static_cast<const __half*>(a.k_rows) + src);
        vv = *reinterpret_cast<const uint4*>(static_cast<const __half*>(a.v_rows) + src);
    } else if (a.rows_fp16 == 2) {
        const uint4 kb = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.k_rows) + src);
        const uint4 vb = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.v_rows) + src);
        const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kb);
        const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vb);
        uint32_t ko[4], vo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 kf = __bfloat1622float2(k2[e]), vf = __bfloat1622float2(v2[e]);
            ko[e] = pack_h2(kf.x, kf.y);
            vo[e] = pack_h2(vf.x, vf.y);
        }
        kk = make_uint4(ko[0], ko[1], ko[2], ko[3]);
        vv = make_uint4(vo[0], vo[1], vo[2], vo[3]);
    } else {
        const float* kf = static_cast<const float*>(a.k_rows) + src;
        const float* vf = static_cast<const float*>(a.v_rows) + src;
        const float4 k0 = *reinterpret_cast<const float4*>(kf), k1 = *reinterpret_cast<const float4*>(kf + 4);
        const float4 v0 = *reinterpret_cast<const float4*>(vf), v1 = *reinterpret_cast<const float4*>(vf + 4);
        kk = make_uint4(pack_h2(k0.x, k0.y), pack_h2(k0.z, k0.w), pack_h2(k1.x, k1.y), pack_h2(k1.z, k1.w));
        vv = make_uint4(pack_h2(v0.x, v0.y), pack_h2(v0.z, v0.w), pack_h2(v1.x, v1.y), pack_h2(v1.z, v1.w));
    }
    *reinterpret_cast<uint4*>(a.k_pool + dst) = kk;
    *reinterpret_cast<uint4*>(a.v_pool + dst) = vv;
}

__global__ void __launch_bounds__(256) kv_write_kernel(KvWriteArgs a) {
    griddep_launch();
    if (!a.early) griddep_wait();
    kv_write_rows(a);
    if (a.early) griddep_wait();      // still completes after the kernel in front, as every kernel of a step does
}

// grid (n_tok, n_kv), 32 threads.
__global__ void __launch_bounds__(32)
kv_gather_kernel(const __half* pool, const int32_t* table, __half* out, int n_tok, int n_kv,
                 int n_pages, int* err) {
    const int t = blockIdx.x, h = blockIdx.y, lane = threadIdx.x;
    const int page = table[t / kPageTokens];
    if (page < 0 || page >= n_pages) {
        if (lane == 0) set_err(err, DEV_ERR_BAD_PAGE);
        return;
    }
    const size_t src = (size_t(page) * n_kv + h) * kv_slice_elems() + kv_slice_offset(t % kPageTokens, lane * 8);
    *reinterpret_cast<uint4*>(out + (size_t(t) * n_kv + h) * kHeadDim + lane * 8) =
        *reinterpret_cast<const uint4*>(pool + src);
}

__global__ void kv_slot_rows_kernel(int32_t* rows, const int32_t* slot_ids, int pages_per_slot, int n_slots, int* err) {
    griddep_launch();
    griddep_wait();
    const int b = blockIdx.x;
    int slot = slot_ids ? slot_ids[b] : b;
    if (slot < 0 || slot >= n_slots) {
        if (threadIdx.x == 0) set_err(err, DEV_ERR_BAD_SLOT);
        slot = 0;
    }
    for (int j = threadIdx.x; j < pages_per_slot; j += blockDim.x)
        rows[size_t(b) * pages_per_slot + j] = slot * pages_per_slot + j;
}

}  // namespace rl
