// Thin run-time binding of NCCL used by the sharded decode step (comm.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include <cstring>

#include "../../include/rl_b200.h"

namespace rl {

struct Comm;

// All return 0 on success; on failure comm_last_error() has the message (per host thread).
const char* comm_last_error();
int comm_unique_id(void* id);                                   // RL_COMM_ID_BYTES bytes
int comm_create(const void* id, int rank, int n_ranks, Comm** out);   // on the current device
void comm_destroy(Comm* c);
int comm_rank(const Comm* c);
int comm_ranks(const Comm* c);
int comm_group_start();
int comm_group_end();
// recv [n_ranks][count], rank r's block = what rank r sent
int comm_all_gather_f32(Comm* c, const float* send, float* recv, size_t count, cudaStream_t st);

}  // namespace rl
