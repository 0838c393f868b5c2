#include "comm.h"

#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <mutex>

#include "../../include/rg_b200.h"

namespace rg {
namespace {

struct Api {
  void *handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

Api *api(std::string *err) {
  static Api a;
  static std::once_flag once;
  static std::string load_error;
  std::call_once(once, [] {
    // A process that already loaded NCCL (for example through torch) gets that same copy back.
    a.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!a.handle) {
      load_error = std::string("dlopen libnccl.so.2: ") + dlerror();
      return;
    }
    auto sym = [&](const char *name) {
      void *p = dlsym(a.handle, name);
      if (!p && load_error.empty()) load_error = std::string("missing NCCL symbol ") + name;
      return p;
    };
    a.GetUniqueId = reinterpret_cast<decltype(a.GetUniqueId)>(sym("ncclGetUniqueId"));
    a.CommInitRank = reinterpret_cast<decltype(a.CommInitRank)>(sym("ncclCommInitRank"));
    a.CommDestroy = reinterpret_cast<decltype(a.CommDestroy)>(sym("ncclCommDestroy"));
    a.AllReduce = reinterpret_cast<decltype(a.AllReduce)>(sym("ncclAllReduce"));
    a.AllGather = reinterpret_cast<decltype(a.AllGather)>(sym("ncclAllGather"));
    a.GroupStart = reinterpret_cast<decltype(a.GroupStart)>(sym("ncclGroupStart"));
    a.GroupEnd = reinterpret_cast<decltype(a.GroupEnd)>(sym("ncclGroupEnd"));
    a.GetErrorString = reinterpret_cast<decltype(a.GetErrorString)>(sym("ncclGetErrorString"));
  });
  if (!load_error.empty()) {
    if (err) *err = load_error;
    return nullptr;
  }
  return &a;
}

int32_t check(Api *a, ncclResult_t r, const char *what, std::string *err) {
  if (r == ncclSuccess) return RG_OK;
  if (err) *err = std::string(what) + ": " + (a->GetErrorString ? a->GetErrorString(r) : "NCCL error");
  return RG_NCCL_ERROR;
}

}  // namespace

int32_t comm_unique_id(uint8_t out[128], std::string *err) {
  Api *a = api(err);
  if (!a) return RG_NCCL_ERROR;
  ncclUniqueId id;
  int32_t rc = check(a, a->GetUniqueId(&id), "ncclGetUniqueId", err);
  if (rc) return rc;
  memcpy(out, id.internal, 128);
  return RG_OK;
}

int32_t comm_init(Comm *c, const uint8_t idb[128], int rank, int world, std::string *err) {
  Api *a = api(err);
  if (!a) return RG_NCCL_ERROR;
  ncclUniqueId id;
  memcpy(id.internal, idb, 128);
  ncclComm_t comm;
  int32_t rc = check(a, a->CommInitRank(&comm, world, id, rank), "ncclCommInitRank", err);
  if (rc) return rc;
  c->nccl_comm = comm;
  c->rank = rank;
  c->world = world;
  return RG_OK;
}

void comm_destroy(Comm *c) {
  if (!c || !c->nccl_comm) return;
  Api *a = api(nullptr);
  if (a) a->CommDestroy(static_cast<ncclComm_t>(c->nccl_comm));
  c->nccl_comm = nullptr;
}

int32_t comm_allreduce_sum_f32(Comm *c, float *buf, size_t count, cudaStream_t stream, std::string *err) {
  Api *a = api(err);
  if (!a) return RG_NCCL_ERROR;
  return check(a, a->AllReduce(buf, buf, count, ncclFloat32, ncclSum, static_cast<ncclComm_t>(c->nccl_comm), stream),
               "ncclAllReduce", err);
}

int32_t comm_allgather_f32(Comm *c, const float *send, float *recv, size_t count, cudaStream_t stream, std::string *err) {
  Api *a = api(err);
  if (!a) return RG_NCCL_ERROR;
  return check(a, a->AllGather(send, recv, count, ncclFloat32, static_cast<ncclComm_t>(c->nccl_comm), stream), "ncclAllGather",
               err);
}

int32_t comm_group_start(std::string *err) {
  Api *a = api(err);
  if (!a) return RG_NCCL_ERROR;
  return check(a, a->GroupStart(), "ncclGroupStart", err);
}
int32_t comm_group_end(std::string *err) {
  Api *a = api(err);
  if (!a) return RG_NCCL_ERROR;
  return check(a, a->GroupEnd(), "ncclGroupEnd", err);
}

}  // namespace rg
