// Context and error plumbing of libqeng.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>

#include "qeng_internal.h"

int32_t qeng_fail(qeng_ctx* ctx, int32_t code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx) ctx->err = buf;
  return code;
}

#ifdef QENG_TRACE
static const size_t kStatusBytes = 256 + 8 * (8 + 30000 * 8);
#else
static const size_t kStatusBytes = 256;
#endif

extern "C" {

int32_t qeng_version(void) { return 100; }

int32_t qeng_create(int32_t device, qeng_ctx** out) { return qeng_create_opts(device, nullptr, out); }

int32_t qeng_create_opts(int32_t device, const qeng_options* opts, qeng_ctx** out) {
  if (!out) return QENG_ERR_ARG;
  *out = nullptr;
  qeng_options o = {};
  if (opts) {  // an older caller's (shorter) struct leaves the newer fields at their defaults
    if (opts->struct_size < (int32_t)sizeof(int32_t) || opts->struct_size > 4096) return QENG_ERR_ARG;
    memcpy(&o, opts, (size_t)opts->struct_size < sizeof o ? (size_t)opts->struct_size : sizeof o);
  }
  if (o.attn_ctas_per_sm < 0 || o.attn_ctas_per_sm > 64) return QENG_ERR_ARG;
  if (o.stream_groups != 0 && o.stream_groups != 1 && o.stream_groups != 2 && o.stream_groups != 4) return QENG_ERR_ARG;
  if (o.stream_stage_chunks != 0 && (o.stream_stage_chunks < 4 || o.stream_stage_chunks > 64)) return QENG_ERR_ARG;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) return QENG_ERR_CUDA;  // no CPU fallback
  if (device < 0 || device >= count) return QENG_ERR_ARG;
  qeng_ctx* ctx = new qeng_ctx();
  ctx->device = device;
  cudaDeviceProp prop;
  if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    delete ctx;
    return QENG_ERR_CUDA;
  }
  if (prop.major != 10) {  // the kernels are built for sm_100a only
    delete ctx;
    return QENG_ERR_CUDA;
  }
  ctx->sm_count = prop.multiProcessorCount;
  ctx->pdl = !o.no_pdl;
  ctx->l2_prefetch = !o.no_l2_prefetch;
  ctx->p2p_allowed = !o.no_p2p_allreduce;
  ctx->attn_cluster = !o.no_attn_cluster;
  ctx->step_kernel = o.step_kernel != 0;
  ctx->attn_ctas_per_sm = o.attn_ctas_per_sm > 0 ? o.attn_ctas_per_sm : 3;
  ctx->stream_groups = o.stream_groups;
  ctx->stream_stage_chunks = o.stream_stage_chunks & ~1;  // a two-chunk work item never straddles stages
  if (cudaMalloc(&ctx->status, kStatusBytes) != cudaSuccess || cudaMemset(ctx->status, 0, kStatusBytes) != cudaSuccess) {
    delete ctx;
    return QENG_ERR_CUDA;
  }
  const size_t tail_slots = (size_t)ctx->sm_count * 4 * 4;  // CTAs x rows of the fused LM head
  if (cudaMalloc(&ctx->tail_val, tail_slots * 4) != cudaSuccess || cudaMalloc(&ctx->tail_idx, tail_slots * 4) != cudaSuccess ||
      cudaMalloc(&ctx->tail_cnt, 64) != cudaSuccess || cudaMemset(ctx->tail_cnt, 0, 64) != cudaSuccess) {
    qeng_destroy(ctx);
    return QENG_ERR_CUDA;
  }
  *out = ctx;
  return QENG_OK;
}

int32_t qeng_destroy(qeng_ctx* ctx) {
  if (!ctx) return QENG_ERR_ARG;
  cudaSetDevice(ctx->device);
  qeng_tp_release(ctx);
  if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
  if (ctx->status) cudaFree(ctx->status);
  if (ctx->xbf16) cudaFree(ctx->xbf16);
  if (ctx->ximage) cudaFree(ctx->ximage);
  if (ctx->tail_val) cudaFree(ctx->tail_val);
  if (ctx->tail_idx) cudaFree(ctx->tail_idx);
  if (ctx->tail_cnt) cudaFree(ctx->tail_cnt);
  delete ctx;
  return QENG_OK;
}

const char* qeng_last_error(const qeng_ctx* ctx) { return ctx ? ctx->err.c_str() : "null context"; }

int32_t qeng_device_status(qeng_ctx* ctx) {
  if (!ctx) return QENG_ERR_ARG;
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  QENG_CUDA(ctx, cudaDeviceSynchronize());
  int32_t status = 0;
  QENG_CUDA(ctx, cudaMemcpy(&status, ctx->status, 4, cudaMemcpyDeviceToHost));
  if (status == 0) return QENG_OK;
  QENG_CUDA(ctx, cudaMemset(ctx->status, 0, 4));
  QENG_CUDA(ctx, cudaMemset(ctx->tail_cnt, 0, 64));
  return qeng_fail(ctx, QENG_ERR_DEVICE_STATUS,
                   "a kernel reported status %d (1 = page id outside the pool, 2 = position outside the cache, "
                   "3 = token id outside the vocabulary, 4 = a bounded wait on a copy or MMA ran out, 5 = a peer never delivered its part of an all-reduce)", status);
}

int32_t qeng_sm_count(const qeng_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

#ifdef QENG_TRACE
// tuning builds only: the 256 bytes behind the status pointer (status word, timestamps, cycle counters);
// the counters are cleared after the read
int32_t qeng_debug_status_words(qeng_ctx* ctx, unsigned long long* out32) {
  cudaDeviceSynchronize();
  if (cudaMemcpy(out32, ctx->status, 256, cudaMemcpyDeviceToHost) != cudaSuccess) return -4;
  return cudaMemset(reinterpret_cast<char*>(ctx->status) + 64, 0, 192) == cudaSuccess ? 0 : -4;
}
// the launch log: records of 8 u64 (kind, stamps); cleared after the read
int32_t qeng_debug_trace(qeng_ctx* ctx, unsigned long long* out, int32_t max_records, int32_t* n) {
  cudaDeviceSynchronize();
  unsigned long long cnt = 0;
  char* base = reinterpret_cast<char*>(ctx->status) + 256;
  if (cudaMemcpy(&cnt, base, 8, cudaMemcpyDeviceToHost) != cudaSuccess) return -4;
  if (cnt > 30000) cnt = 30000;
  if (cnt > (unsigned long long)max_records) cnt = (unsigned long long)max_records;
  if (cnt && cudaMemcpy(out, base + 64, cnt * 64, cudaMemcpyDeviceToHost) != cudaSuccess) return -4;
  *n = (int32_t)cnt;
  return cudaMemset(base, 0, 64) == cudaSuccess ? 0 : -4;
}
#endif

}  // extern "C"
