// Tensor-parallel communicator: NCCL resolved at run time with dlopen, so single-GPU use needs
// no NCCL at all.  Stands where rustgrad has CudaCollectiveGroup (src/collective.rs:322-345,441):
// sum all-reduce of f32 partials (the contracting-axis rule of src/sharding.rs:642-667) and an
// all-gather for the column-split vocabulary head.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace rg {

struct Comm {
  void *nccl_comm = nullptr;
  int rank = 0, world = 1;
};

// Fills 128 bytes with a fresh NCCL unique id (rank 0 calls it; the caller broadcasts it).
int32_t comm_unique_id(uint8_t out[128], std::string *err);
int32_t comm_init(Comm *c, const uint8_t id[128], int rank, int world, std::string *err);
void comm_destroy(Comm *c);
int32_t comm_allreduce_sum_f32(Comm *c, float *buf, size_t count, cudaStream_t stream, std::string *err);
// recv[r * count .. ] = send of rank r
int32_t comm_allgather_f32(Comm *c, const float *send, float *recv, size_t count, cudaStream_t stream, std::string *err);
int32_t comm_group_start(std::string *err);
int32_t comm_group_end(std::string *err);

}  // namespace rg
