// Tensor-parallel plumbing: one context per GPU, one process (or thread) per rank.
// The collective after each row-split projection is an NCCL all-reduce over NVLink; NCCL is
// opened at run time (dlopen) so that single-GPU users do not need it.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include "qeng_internal.h"

namespace {

struct NcclApi {
  void* lib = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& api() {
  static NcclApi a;
  if (a.lib) return a;
  // a copy already loaded by the host program (same soname) is reused
  a.lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!a.lib) return a;
  a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(a.lib, "ncclGetUniqueId");
  a.CommInitRank = (decltype(a.CommInitRank))dlsym(a.lib, "ncclCommInitRank");
  a.AllReduce = (decltype(a.AllReduce))dlsym(a.lib, "ncclAllReduce");
  a.CommDestroy = (decltype(a.CommDestroy))dlsym(a.lib, "ncclCommDestroy");
  a.GetErrorString = (decltype(a.GetErrorString))dlsym(a.lib, "ncclGetErrorString");
  a.ok = a.GetUniqueId && a.CommInitRank && a.AllReduce && a.CommDestroy && a.GetErrorString;
  return a;
}

}  // namespace

int32_t qeng_tp_all_reduce_internal(qeng_ctx* ctx, float* buf, int64_t n, cudaStream_t stream) {
  if (ctx->tp_world <= 1) return QENG_OK;
  NcclApi& a = api();
  ncclResult_t r = a.AllReduce(buf, buf, (size_t)n, ncclFloat, ncclSum, (ncclComm_t)ctx->nccl_comm, stream);
  if (r != ncclSuccess) return qeng_fail(ctx, QENG_ERR_NCCL, "ncclAllReduce failed: %s", a.GetErrorString(r));
  return QENG_OK;
}

void qeng_tp_release(qeng_ctx* ctx) {
  if (ctx->nccl_comm) {
    api().CommDestroy((ncclComm_t)ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
  }
}

extern "C" {

int32_t qeng_tp_unique_id(uint8_t* out128) {
  if (!out128) return QENG_ERR_ARG;
  NcclApi& a = api();
  if (!a.ok) return QENG_ERR_NCCL;
  ncclUniqueId id;
  if (a.GetUniqueId(&id) != ncclSuccess) return QENG_ERR_NCCL;
  memcpy(out128, &id, 128);
  return QENG_OK;
}

int32_t qeng_tp_init(qeng_ctx* ctx, int32_t rank, int32_t world, const uint8_t* id128) {
  if (!ctx || !id128) return qeng_fail(ctx, QENG_ERR_ARG, "tp_init: null argument");
  if (world < 1 || rank < 0 || rank >= world) return qeng_fail(ctx, QENG_ERR_ARG, "tp_init: bad rank/world");
  if (ctx->nccl_comm) return qeng_fail(ctx, QENG_ERR_STATE, "tp_init: already initialised");
  NcclApi& a = api();
  if (!a.ok) return qeng_fail(ctx, QENG_ERR_NCCL, "tp_init: libnccl.so.2 could not be opened");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  ncclUniqueId id;
  memcpy(&id, id128, 128);
  ncclComm_t comm = nullptr;
  ncclResult_t r = a.CommInitRank(&comm, world, id, rank);
  if (r != ncclSuccess) return qeng_fail(ctx, QENG_ERR_NCCL, "ncclCommInitRank failed: %s", a.GetErrorString(r));
  ctx->nccl_comm = comm;
  ctx->tp_rank = rank;
  ctx->tp_world = world;
  return QENG_OK;
}

int32_t qeng_tp_all_reduce_f32(qeng_ctx* ctx, float* buf, int64_t n, void* stream) {
  if (!ctx || !buf || n <= 0) return qeng_fail(ctx, QENG_ERR_ARG, "tp_all_reduce_f32: bad argument");
  if (ctx->tp_world > 1 && !ctx->nccl_comm) return qeng_fail(ctx, QENG_ERR_STATE, "tp_all_reduce_f32: tp_init first");
  return qeng_tp_all_reduce_internal(ctx, buf, n, (cudaStream_t)stream);
}

}  // extern "C"
