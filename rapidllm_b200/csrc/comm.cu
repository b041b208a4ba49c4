// Communicator of the GPUs of one node that share a decode step (rl_comm_* of the C ABI).
//
// The reference engine is single-GPU; dividing one batch over several B200 is new here.  The
// mixers shard without moving KV or state (KV heads / DeltaNet value heads / sequences / token
// ranges); the only exchange is an all-gather of the small per-layer outputs (head slices, or
// split-KV partials merged by lse_combine_kernel), issued from rl_stack_decode on a side stream
// so that it runs beside the following layers.  The collective is NCCL's ncclAllGather over
// NVLink / NVSwitch; the library binds NCCL at run time (dlopen of libnccl.so.2, so a process
// that already loaded NCCL -- a PyTorch host -- shares that copy) and has no link-time
// dependency on it.  No peer pointers and no multicast loads are used anywhere.
#include "comm.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdio>
#include <mutex>
#include <new>

static_assert(RL_COMM_ID_BYTES == sizeof(ncclUniqueId), "rl_comm id size must match ncclUniqueId");

namespace rl {

namespace {

struct NcclApi {
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclAllGather) AllGather = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
    bool ok = false;
    char why[160] = "";
};

NcclApi* nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            std::snprintf(api.why, sizeof api.why, "NCCL not found: %s", dlerror());
            return;
        }
        bool all = true;
        auto sym = [&](const char* name) {
            void* p = dlsym(h, name);
            if (!p) {
                all = false;
                std::snprintf(api.why, sizeof api.why, "NCCL lacks %s", name);
            }
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
        api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        api.ok = all;
    });
    return &api;
}

thread_local char g_comm_err[256] = "";

int nccl_fail(NcclApi* n, ncclResult_t r, const char* what) {
    std::snprintf(g_comm_err, sizeof g_comm_err, "%s: %s", what, n->GetErrorString ? n->GetErrorString(r) : "NCCL error");
    return 1;
}

}  // namespace

struct Comm {
    ncclComm_t comm = nullptr;
    int rank = 0, n_ranks = 1, device = 0;
};

const char* comm_last_error() { return g_comm_err; }

int comm_unique_id(void* id) {
    NcclApi* n = nccl_api();
    if (!n->ok) {
        std::snprintf(g_comm_err, sizeof g_comm_err, "%s", n->why);
        return 1;
    }
    ncclUniqueId uid;
    const ncclResult_t r = n->GetUniqueId(&uid);
    if (r != ncclSuccess) return nccl_fail(n, r, "ncclGetUniqueId");
    std::memcpy(id, &uid, sizeof uid);
    return 0;
}

int comm_create(const void* id, int rank, int n_ranks, Comm** out) {
    NcclApi* n = nccl_api();
    if (!n->ok) {
        std::snprintf(g_comm_err, sizeof g_comm_err, "%s", n->why);
        return 1;
    }
    Comm* c = new (std::nothrow) Comm();
    if (!c) {
        std::snprintf(g_comm_err, sizeof g_comm_err, "host allocation failed");
        return 1;
    }
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof uid);
    cudaGetDevice(&c->device);
    c->rank = rank;
    c->n_ranks = n_ranks;
    const ncclResult_t r = n->CommInitRank(&c->comm, n_ranks, uid, rank);
    if (r != ncclSuccess) {
        delete c;
        return nccl_fail(n, r, "ncclCommInitRank");
    }
    *out = c;
    return 0;
}

void comm_destroy(Comm* c) {
    if (!c) return;
    NcclApi* n = nccl_api();
    if (n->ok && c->comm) n->CommDestroy(c->comm);
    delete c;
}

int comm_rank(const Comm* c) { return c ? c->rank : 0; }
int comm_ranks(const Comm* c) { return c ? c->n_ranks : 1; }

int comm_group_start() {
    NcclApi* n = nccl_api();
    const ncclResult_t r = n->GroupStart();
    return r == ncclSuccess ? 0 : nccl_fail(n, r, "ncclGroupStart");
}

int comm_group_end() {
    NcclApi* n = nccl_api();
    const ncclResult_t r = n->GroupEnd();
    return r == ncclSuccess ? 0 : nccl_fail(n, r, "ncclGroupEnd");
}

int comm_all_gather_f32(Comm* c, const float* send, float* recv, size_t count, cudaStream_t st) {
    NcclApi* n = nccl_api();
    const ncclResult_t r = n->AllGather(send, recv, count, ncclFloat, c->comm, st);
    return r == ncclSuccess ? 0 : nccl_fail(n, r, "ncclAllGather");
}

}  // namespace rl
