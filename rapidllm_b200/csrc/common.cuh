// Device-side helpers shared by the sm_100a kernels: mbarrier + bulk-copy (TMA)
// wrappers with bounded waits, warp-level MMA wrappers, error reporting.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rl {

// Error word written by kernels instead of trapping.  0 = ok.
enum DevErr : int {
    DEV_OK = 0,
    DEV_ERR_BAD_PAGE = 1,      // page-table entry outside the pool
    DEV_ERR_WAIT_TIMEOUT = 2,  // a bounded mbarrier wait gave up
    DEV_ERR_WORKSPACE = 3,     // more split-KV chunks than the workspace holds
    DEV_ERR_BAD_SLOT = 4,      // state-cache slot outside the cache
    DEV_ERR_BAD_LEN = 5,       // sequence length outside the page table
};

__device__ __forceinline__ void set_err(int* err, int code) {
    if (err) atomicCAS(err, 0, code);
}

// Programmatic dependent launch: a kernel launched with the stream-serialisation attribute may
// become resident while the kernel before it in the stream is still running.  griddep_wait()
// blocks until every kernel before this one has completed and its writes are visible (a no-op in
// a plain launch); griddep_launch() lets the next kernel's CTAs be scheduled from here on.  Every
// kernel of the decode step waits before it reads or writes anything, so only launch latency and
// per-CTA set-up overlap the kernel in front.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -----------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after kWaitLimitNs of wall time (each poll may itself suspend
// for a hardware-defined time), so a lost arrival can never hang the GPU.
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > kWaitLimitNs) return false;
    }
}

// ---- TMA (untiled bulk copy global -> shared, completes on an mbarrier) ----
// dst, src 16-byte aligned; bytes a multiple of 16.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// ---- TMA bulk store shared -> global (completion tracked by bulk async-groups) ----
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src_smem)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's bulk groups still have to READ their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- shared-memory loads through 32-bit shared-space addresses (no generic-pointer arithmetic) ----
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// ---- warp MMA m16n8k16, fp16 inputs, fp32 accumulate ----------------------
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The five in-warp stages (distances 1, 2, 4, 8, 16) of an unnormalised Walsh-Hadamard transform
// over values held one per lane: at distance d the lane whose bit d is clear keeps the sum of the
// pair, its partner keeps (lower - upper).
__device__ __forceinline__ float wht32_in_warp(float x, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const float partner = __shfl_xor_sync(0xffffffffu, x, d);
        const bool upper = (lane & d) != 0;
        x = upper ? (partner - x) : (x + partner);
    }
    return x;
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- KV page geometry ------------------------------------------------------
// A page holds kPageTokens tokens of every KV head.  One (page, head) slice of
// K (or V) is kept in HBM already in the shared-memory tile format the tensor
// cores read: hd/64 sub-tiles, each [kPageTokens rows][128 bytes], with the
// 16-byte chunk index of a row XOR-ed by (row & 7) (the 128-byte swizzle).  A
// slice therefore moves to shared memory with linear bulk copies and is read
// there without bank conflicts.  Element (tok, d) of a slice lives at
// kv_slice_offset(tok, d) halves from the slice start.
constexpr int kPageTokens = 64;
constexpr int kHeadDim = 256;
__host__ __device__ __forceinline__ size_t kv_slice_elems() { return size_t(kPageTokens) * kHeadDim; }
__host__ __device__ __forceinline__ int kv_slice_offset(int tok, int d) {
    const int sub = d >> 6;
    const int chunk = ((d & 63) >> 3) ^ (tok & 7);
    return sub * (kPageTokens * 64) + tok * 64 + chunk * 8 + (d & 7);
}


// ---- compact KV records (q8 K + TQ3 V), one per (page, head, half page) -----------
constexpr int kCompactHalfTokens = 32;
constexpr int kCompactVOff = 8192;
constexpr int kCompactKScaleOff = 11264;
constexpr int kCompactVScaleOff = 11328;
constexpr int kCompactRecordBytes = 11456;
// Byte offset, inside a record, of the 6 bytes holding the codes of dims 64j + 8g .. +7 for
// the token pair that contains row `row` (0..31): V codes are grouped per 16-token block as
// [pair half AB = 0,1][g = 0..7][c = 0..3][24 B] so that the 16 lanes (g, c) of a half warp read
// 16 consecutive 24-byte groups (conflict-free 8-byte loads).
__host__ __device__ __forceinline__ int compact_v_offset(int row, int g, int j) {
    const int q = (row & 15) >> 1;
    return kCompactVOff + (row >> 4) * 1536 + (q >> 2) * 768 + g * 96 + (q & 3) * 24 + j * 6;
}

}  // namespace rl
