// Tensor-parallel plumbing: one context per GPU, one process (or thread) per rank.
// The collective after each row-split projection is an NCCL all-reduce over NVLink; NCCL is
// opened at run time (dlopen) so that single-GPU users do not need it.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
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

// ---- one-shot all-reduce over peer memory ---------------------------------------------------
// For the small messages of decode (16 KB .. 256 KB) the cost of a collective is latency, not
// bandwidth.  Every rank owns an inbox [2 slots][world][kP2pMaxElems] of (value, tag) pairs in its
// own memory, mapped into every peer with CUDA IPC.  A call pushes the local partial sums, each
// paired with the call's sequence number in one 8-byte store, into the inbox of every rank (plain
// stores over NVLink, no multicast, no fences), then reads the `world` slices of its OWN inbox,
// waiting (bounded) until each pair carries this call's tag, and adds them in rank order, so all
// ranks get bit-identical sums.  Slots alternate per call (a rank can be at most one call ahead
// of a peer); a device-side call counter supplies the tag, so a captured graph can be replayed.
// The sum is added into `dst` (the residual stream): collective and residual add are one kernel.
constexpr int kP2pMaxElems = 16 * 4096;   // f32 elements per call (16 rows of d_model 4096)
constexpr int kP2pThreads = 256;
constexpr int kP2pSlice = kP2pThreads * 4;  // elements per CTA

struct P2pParams {
  uint2* inbox[8];     // inbox base of every rank (peer-mapped), [2][world][kP2pMaxElems]
  unsigned* counter;   // local: [0] completed calls, [1] CTAs done in the running call
  const float* src;    // local partial sums [n]
  float* dst;          // dst[i] += sum over ranks
  int n, rank, world;
  int32_t* status;
};

__global__ void __launch_bounds__(kP2pThreads) p2p_allreduce_add_kernel(const P2pParams p) {
  // the matmul that follows may start streaming its weights while this kernel waits for the peers
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  const int tid = threadIdx.x, cta = blockIdx.x;
  const unsigned seq = *p.counter + 1;  // read by every CTA before the last one to finish bumps it
  const int slot = seq & 1;
  const int i0 = cta * kP2pSlice + tid * 4;
  const bool active = i0 < p.n;  // n is a multiple of 4
  if (active) {
    const float4 v = *reinterpret_cast<const float4*>(p.src + i0);
    const uint32_t w[4] = {__float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w)};
    for (int r = 0; r < p.world; ++r) {
      const int peer = (p.rank + r) % p.world;  // spread the first stores over the links
      uint2* in = p.inbox[peer] + ((size_t)slot * p.world + p.rank) * kP2pMaxElems + i0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1,%2};\n" ::"l"(in + e), "r"(w[e]), "r"(seq) : "memory");
    }
    float4 acc = *reinterpret_cast<const float4*>(p.dst + i0);
    float* a = reinterpret_cast<float*>(&acc);
    bool failed = false;
    for (int r = 0; r < p.world && !failed; ++r) {
      const uint2* in = p.inbox[p.rank] + ((size_t)slot * p.world + r) * kP2pMaxElems + i0;
#pragma unroll
      for (int e = 0; e < 4 && !failed; ++e) {
        uint32_t val, tag;
        unsigned long long t0 = 0;
        for (int spin = 0;; ++spin) {
          asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];\n" : "=r"(val), "=r"(tag) : "l"(in + e) : "memory");
          if (tag == seq) break;
          if ((spin & 1023) == 1023) {  // bounded: two seconds, then report and leave
            unsigned long long t1;
            asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t1));
            if (t0 == 0) t0 = t1;
            if (t1 - t0 > 2000000000ull) {
              failed = true;
              atomicExch(p.status, 5);
              break;
            }
          }
        }
        if (!failed) a[e] += __uint_as_float(val);
      }
    }
    if (!failed) *reinterpret_cast<float4*>(p.dst + i0) = acc;
  }
  // the last CTA to finish advances the call counter (all CTAs have read it by then)
  __shared__ unsigned s_done;
  __syncthreads();
  if (tid == 0) s_done = atomicAdd(p.counter + 1, 1u);
  __syncthreads();
  if (s_done == gridDim.x - 1 && tid == 0) {
    p.counter[1] = 0;
    __threadfence();
    p.counter[0] = seq;
  }
}

// x += all-reduce(part) with the one-shot kernel when the peers are mapped and the message is small
bool qeng_tp_p2p_ready(const qeng_ctx* ctx, int64_t n) {
  return ctx->p2p_ready && n <= kP2pMaxElems && (n & 3) == 0;
}

int32_t qeng_tp_allreduce_add(qeng_ctx* ctx, float* dst, const float* part, int64_t n, cudaStream_t stream) {
  P2pParams p;
  for (int r = 0; r < 8; ++r) p.inbox[r] = r < ctx->tp_world ? reinterpret_cast<uint2*>(ctx->p2p_peer[r]) : nullptr;
  p.counter = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(ctx->p2p_local) + ctx->p2p_counter_off);
  p.src = part; p.dst = dst; p.n = (int)n; p.rank = ctx->tp_rank; p.world = ctx->tp_world; p.status = ctx->status;
  const int grid = (int)((n + kP2pSlice - 1) / kP2pSlice);
  p2p_allreduce_add_kernel<<<grid, kP2pThreads, 0, stream>>>(p);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_tp_all_reduce_internal(qeng_ctx* ctx, float* buf, int64_t n, cudaStream_t stream) {
  if (ctx->tp_world <= 1) return QENG_OK;
  NcclApi& a = api();
  ncclResult_t r = a.AllReduce(buf, buf, (size_t)n, ncclFloat, ncclSum, (ncclComm_t)ctx->nccl_comm, stream);
  if (r != ncclSuccess) return qeng_fail(ctx, QENG_ERR_NCCL, "ncclAllReduce failed: %s", a.GetErrorString(r));
  return QENG_OK;
}

void qeng_tp_release(qeng_ctx* ctx) {
  if (ctx->p2p_local) {
    for (int r = 0; r < ctx->tp_world; ++r)
      if (r != ctx->tp_rank && ctx->p2p_peer[r]) cudaIpcCloseMemHandle(ctx->p2p_peer[r]);
    cudaFree(ctx->p2p_local);
    ctx->p2p_local = nullptr;
    ctx->p2p_ready = false;
  }
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

int32_t qeng_tp_p2p_handle(qeng_ctx* ctx, uint8_t* out64) {
  if (!ctx || !out64) return qeng_fail(ctx, QENG_ERR_ARG, "tp_p2p_handle: null argument");
  if (ctx->tp_world < 2 || ctx->tp_world > 8) return qeng_fail(ctx, QENG_ERR_STATE, "tp_p2p_handle: needs 2..8 ranks (tp_init first)");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!ctx->p2p_local) {
    const size_t inbox = (size_t)2 * ctx->tp_world * kP2pMaxElems * sizeof(uint2);
    ctx->p2p_flag_off = inbox;
    ctx->p2p_counter_off = inbox;   // [0] calls completed, [1] CTAs done, [2] decode steps completed (tag base of the fused inbox)
    ctx->p2p_fuse_off = inbox + 256;
    const size_t total = inbox + 256 + qeng_tp_fuse_bytes(ctx->tp_world);
    QENG_CUDA(ctx, cudaMalloc(&ctx->p2p_local, total));
    QENG_CUDA(ctx, cudaMemset(ctx->p2p_local, 0, total));
  }
  cudaIpcMemHandle_t h;
  QENG_CUDA(ctx, cudaIpcGetMemHandle(&h, ctx->p2p_local));
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(out64, &h, 64);
  return QENG_OK;
}

int32_t qeng_tp_p2p_open(qeng_ctx* ctx, const uint8_t* handles) {
  if (!ctx || !handles) return qeng_fail(ctx, QENG_ERR_ARG, "tp_p2p_open: null argument");
  if (!ctx->p2p_local) return qeng_fail(ctx, QENG_ERR_STATE, "tp_p2p_open: call tp_p2p_handle first");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  for (int r = 0; r < ctx->tp_world; ++r) {
    if (r == ctx->tp_rank) {
      ctx->p2p_peer[r] = ctx->p2p_local;
      continue;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)r * 64, 64);
    void* ptr = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "tp_p2p_open: rank %d: %s", r, cudaGetErrorString(e));
    ctx->p2p_peer[r] = ptr;
  }
  ctx->p2p_ready = ctx->p2p_allowed;
  return QENG_OK;
}

int32_t qeng_tp_p2p_reset(qeng_ctx* ctx) {
  if (!ctx) return QENG_ERR_ARG;
  if (!ctx->p2p_local) return qeng_fail(ctx, QENG_ERR_STATE, "tp_p2p_reset: no inbox (tp_p2p_handle first)");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  QENG_CUDA(ctx, cudaDeviceSynchronize());
  const size_t inbox = (size_t)2 * ctx->tp_world * kP2pMaxElems * sizeof(uint2);
  QENG_CUDA(ctx, cudaMemset(ctx->p2p_local, 0, inbox + 256 + qeng_tp_fuse_bytes(ctx->tp_world)));  // tags and the counters start over
  QENG_CUDA(ctx, cudaMemset(ctx->status, 0, 4));
  return QENG_OK;
}

__global__ void tp_add_kernel(float* __restrict__ x, const float* __restrict__ p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += p[i];
}

int32_t qeng_tp_all_reduce_add_f32(qeng_ctx* ctx, float* dst, float* part, int64_t n, void* stream) {
  if (!ctx || !dst || !part || n <= 0) return qeng_fail(ctx, QENG_ERR_ARG, "tp_all_reduce_add_f32: bad argument");
  if (ctx->tp_world > 1 && !ctx->nccl_comm) return qeng_fail(ctx, QENG_ERR_STATE, "tp_all_reduce_add_f32: tp_init first");
  if (ctx->tp_world > 1 && qeng_tp_p2p_ready(ctx, n)) return qeng_tp_allreduce_add(ctx, dst, part, n, (cudaStream_t)stream);
  int32_t rc = qeng_tp_all_reduce_internal(ctx, part, n, (cudaStream_t)stream);
  if (rc != QENG_OK) return rc;
  tp_add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(dst, part, n);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_tp_all_reduce_f32(qeng_ctx* ctx, float* buf, int64_t n, void* stream) {
  if (!ctx || !buf || n <= 0) return qeng_fail(ctx, QENG_ERR_ARG, "tp_all_reduce_f32: bad argument");
  if (ctx->tp_world > 1 && !ctx->nccl_comm) return qeng_fail(ctx, QENG_ERR_STATE, "tp_all_reduce_f32: tp_init first");
  return qeng_tp_all_reduce_internal(ctx, buf, n, (cudaStream_t)stream);
}

}  // extern "C"

// ---- fused decode: what is left of the collective when the matmuls carry it ----------------------
#include "gemm_q4_s8.cuh"

// x[rows][dm] += sum over ranks of the parts of `kind` tagged for (step, layer): the one gather of a
// decode step that no matmul staging absorbs (after the last layer's down projection).
__global__ void __launch_bounds__(256) tp_fuse_gather_kernel(float* __restrict__ x, const uint2* __restrict__ inbox, int rows, int dm,
                                                             int world, const unsigned* __restrict__ seq, unsigned tags_per_step,
                                                             unsigned tag_off, int32_t* status) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;  // group of 8 values
  const int per_row = dm / 8;
  if (g >= rows * per_row) return;
  const int m = g / per_row, k0 = (g - m * per_row) * 8;
  const unsigned tag = *seq * tags_per_step + tag_off + 1u;
  q4s8::Waits W;
  float4* xp = reinterpret_cast<float4*>(x + (size_t)m * dm + k0);
  float4 a = xp[0], b = xp[1];
  for (int r = 0; r < world; ++r) {
    float part[8];
    q4s8::poll8(inbox + ((size_t)r * kTpFuseRows + m) * kTpFuseDm + k0, tag, part, W, status);
    a.x += part[0]; a.y += part[1]; a.z += part[2]; a.w += part[3];
    b.x += part[4]; b.y += part[5]; b.z += part[6]; b.w += part[7];
  }
  xp[0] = a;
  xp[1] = b;
}
__global__ void tp_fuse_advance_kernel(unsigned* seq) { *seq += 1u; }

bool qeng_tp_fuse_ready(const qeng_ctx* ctx, int64_t rows, int64_t dm) {
  return ctx->tp_world > 1 && ctx->p2p_ready && rows <= kTpFuseRows && dm <= kTpFuseDm && (dm & 7) == 0;
}
// inbox of `kind` as mapped on this rank for peer r (own rank included)
uint2* qeng_tp_fuse_inbox(const qeng_ctx* ctx, int r, int kind) {
  char* base = reinterpret_cast<char*>(ctx->p2p_peer[r]) + ctx->p2p_fuse_off;
  return reinterpret_cast<uint2*>(base) + (size_t)kind * ctx->tp_world * kTpFuseRows * kTpFuseDm;
}
const unsigned* qeng_tp_fuse_seq(const qeng_ctx* ctx) {
  return reinterpret_cast<const unsigned*>(reinterpret_cast<const char*>(ctx->p2p_local) + ctx->p2p_counter_off) + 2;
}
int32_t qeng_tp_fuse_gather(qeng_ctx* ctx, float* x, int64_t rows, int64_t dm, int kind, int layer, int layers, cudaStream_t stream) {
  const int groups = (int)(rows * dm / 8);
  tp_fuse_gather_kernel<<<(groups + 255) / 256, 256, 0, stream>>>(x, qeng_tp_fuse_inbox(ctx, ctx->tp_rank, kind), (int)rows, (int)dm,
                                                                   ctx->tp_world, qeng_tp_fuse_seq(ctx), 2u * (unsigned)layers,
                                                                   2u * (unsigned)layer + (unsigned)kind, ctx->status);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}
int32_t qeng_tp_fuse_advance(qeng_ctx* ctx, cudaStream_t stream) {
  tp_fuse_advance_kernel<<<1, 1, 0, stream>>>(const_cast<unsigned*>(qeng_tp_fuse_seq(ctx)));
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}
