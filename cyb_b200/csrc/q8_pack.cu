// 8-bit block weights (32-wide blocks, one f16 scale, signed bytes: w = q * s): import into the
// device layout, the device-side inverse (bit-exactness check), dequantisation and the import-time
// quantiser.  "tensor data (Q4/Q8/F16/F32)" is what a cyb model container holds
// (decide/pipeline.md:28); the model the reference ships by default was imported as q8
// (shell/src/worlds/models/mod.rs:68-73).
//
// Device layout: rows in tiles of 16, K in chunks of 64 (two 32-blocks) like the 4-bit layout; the
// weight plane holds per (tile, chunk, block, lane) one uint4.  With g = lane / 4, t = lane % 4 its
// words are the bytes of
//   x: row g,     k = 32 blk + 8 t + {0, 2, 4, 6}      y: row g + 8, the same k
//   z: row g,     k = 32 blk + 8 t + {1, 3, 5, 7}      w: row g + 8, the same k
// i.e. exactly the A registers of mma.sync.m16n8k32 in the k-slot order the staged activation bytes
// use (even k of the lane's 8 in slots 4t..4t+3, odd k in 16+4t..16+4t+3), so the decode matmul loads
// them and issues the MMA with no unpacking.  A row tile is contiguous (1024 B per chunk).  The scale
// plane is the 4-bit layout's.  1.0625 B/weight.
#include <stdlib.h>
#include <string.h>

#include <cuda_fp16.h>

#include "qeng_internal.h"

namespace {

// position of (row n, k) in the weight plane, in bytes
__host__ __device__ inline size_t q8_pos(int64_t n, int64_t k, int64_t nchunks) {
  const int64_t tile = n / 16, r = n % 16, g = r % 8, hi = r / 8;
  const int64_t blk = k / 32, kk = k % 32, t = kk / 8, j = kk % 8;
  const int64_t chunk = blk / 2, b1 = blk % 2;
  const int64_t word = (j & 1) * 2 + hi;  // x, y: even k; z, w: odd k
  return (size_t)(((tile * nchunks + chunk) * 2 + b1) * 32 + g * 4 + t) * 16 + (size_t)word * 4 + (size_t)(j >> 1);
}

__global__ void unpack_q8_kernel(const unsigned char* __restrict__ qs, const uint2* __restrict__ sc, int64_t N, int64_t K,
                                 int64_t nchunks, int8_t* __restrict__ q, uint16_t* __restrict__ s) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * K) return;
  const int64_t n = i / K, k = i % K;
  q[i] = (int8_t)qs[q8_pos(n, k, nchunks)];
  if (k % 32 == 0) {
    const int64_t tile = n / 16, r = n % 16, g = r % 8, hi = r / 8, blk = k / 32;
    const uint16_t* sp = reinterpret_cast<const uint16_t*>(sc + (tile * nchunks + blk / 2) * 8 + g);
    s[n * (K / 32) + blk] = sp[(blk % 2) * 2 + hi];
  }
}

__global__ void dequant_q8_kernel(const unsigned char* __restrict__ qs, const uint2* __restrict__ sc, int64_t N, int64_t K,
                                  int64_t nchunks, float* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * K) return;
  const int64_t n = i / K, k = i % K;
  const int64_t tile = n / 16, r = n % 16, g = r % 8, hi = r / 8, blk = k / 32;
  const __half* sp = reinterpret_cast<const __half*>(sc + (tile * nchunks + blk / 2) * 8 + g);
  out[i] = (float)(int8_t)qs[q8_pos(n, k, nchunks)] * __half2float(sp[(blk % 2) * 2 + hi]);
}

__device__ __forceinline__ float load_f32(const void* src, int dtype, int64_t i) {
  if (dtype == QENG_F32) return reinterpret_cast<const float*>(src)[i];
  if (dtype == QENG_F16) return __half2float(reinterpret_cast<const __half*>(src)[i]);
  return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(src)[i] << 16);
}

// Import-time quantiser, one thread per (row, 32-block): d = max|x| / 127 (f32), q = roundf(x * (1/d))
// (half away from zero), scale stored as f16(d) - the published Q8_0 rule.  Blocks of the padding
// chunk half (K not a multiple of 64) get scale 0 and zero bytes.
__global__ void quantize_q8_kernel(const void* __restrict__ src, int dtype, int64_t N, int64_t K, int64_t ld, int64_t nchunks,
                                   unsigned char* __restrict__ qs, uint2* __restrict__ sc) {
  const int64_t nblk2 = nchunks * 2;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * nblk2) return;
  const int64_t n = i / nblk2, blk = i % nblk2;
  const int64_t tile = n / 16, r = n % 16, g = r % 8, hi = r / 8;
  uint16_t* sp = reinterpret_cast<uint16_t*>(sc + (tile * nchunks + blk / 2) * 8 + g);
  if (blk * 32 >= K) {
    sp[(blk % 2) * 2 + hi] = 0;
    for (int k = 0; k < 32; ++k) qs[q8_pos(n, blk * 32 + k, nchunks)] = 0;
    return;
  }
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) {
    v[k] = load_f32(src, dtype, n * ld + blk * 32 + k);
    amax = fmaxf(amax, fabsf(v[k]));
  }
  const float d = __fdiv_rn(amax, 127.0f);
  const float id = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
  sp[(blk % 2) * 2 + hi] = __half_as_ushort(__float2half_rn(d));
#pragma unroll
  for (int k = 0; k < 32; ++k) qs[q8_pos(n, blk * 32 + k, nchunks)] = (unsigned char)(int8_t)(int)roundf(__fmul_rn(v[k], id));
}

int32_t alloc_q8(qeng_ctx* ctx, int64_t N, int64_t K, qeng_weight** out, const char* who) {
  *out = nullptr;
  if (N <= 0 || K <= 0 || K % 32 != 0 || N % 16 != 0)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "%s: need K %% 32 == 0 and N %% 16 == 0 (N=%lld K=%lld)", who, (long long)N, (long long)K);
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t nblk = K / 32, nchunks = (nblk + 1) / 2, ntiles = N / 16;
  const size_t qs_bytes = (size_t)ntiles * nchunks * 1024, sc_bytes = (size_t)ntiles * nchunks * 64;
  qeng_weight* w = new qeng_weight();
  w->fmt = QENG_FMT_Q8;
  w->N = N; w->K = K; w->ntiles = ntiles; w->nchunks = nchunks;
  w->qs = nullptr; w->sc = nullptr; w->bytes = (int64_t)(qs_bytes + sc_bytes);
  cudaError_t e = cudaMalloc(&w->qs, qs_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&w->sc, sc_bytes);
  if (e != cudaSuccess) {
    if (w->qs) cudaFree(w->qs);
    delete w;
    return qeng_fail(ctx, QENG_ERR_CUDA, "%s: allocation failed: %s", who, cudaGetErrorString(e));
  }
  *out = w;
  return QENG_OK;
}

}  // namespace

void qeng_weight_dequant_q8(const qeng_weight* w, float* out, cudaStream_t stream) {
  const int64_t total = w->N * w->K;
  dequant_q8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const unsigned char*>(w->qs), w->sc,
                                                                         w->N, w->K, w->nchunks, out);
}

extern "C" {

int32_t qeng_weight_pack_q8(qeng_ctx* ctx, const int8_t* q, const uint16_t* s, int64_t N, int64_t K, qeng_weight** out) {
  if (!ctx || !q || !s || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_pack_q8: null argument");
  qeng_weight* w = nullptr;
  int32_t rc = alloc_q8(ctx, N, K, &w, "weight_pack_q8");
  if (rc != QENG_OK) return rc;
  const int64_t nblk = K / 32, nchunks = w->nchunks, ntiles = w->ntiles;
  const size_t qs_bytes = (size_t)ntiles * nchunks * 1024, sc_bytes = (size_t)ntiles * nchunks * 64;
  unsigned char* hq = nullptr;
  uint16_t* hs = nullptr;
  if (cudaMallocHost(&hq, qs_bytes) != cudaSuccess || cudaMallocHost(&hs, sc_bytes) != cudaSuccess) {
    if (hq) cudaFreeHost(hq);
    qeng_weight_free(ctx, w);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_pack_q8: pinned allocation failed");
  }
  memset(hq, 0, qs_bytes);
  memset(hs, 0, sc_bytes);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const int64_t tile = n / 16, r = n % 16, g = r % 8, hi = r / 8;
    for (int64_t blk = 0; blk < nblk; blk++) {
      hs[((tile * nchunks + blk / 2) * 8 + g) * 4 + (blk % 2) * 2 + hi] = s[n * nblk + blk];
      for (int k = 0; k < 32; k++) hq[q8_pos(n, blk * 32 + k, nchunks)] = (unsigned char)q[n * K + blk * 32 + k];
    }
  }
  cudaError_t e = cudaMemcpy(w->qs, hq, qs_bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(w->sc, hs, sc_bytes, cudaMemcpyHostToDevice);
  cudaFreeHost(hq);
  cudaFreeHost(hs);
  if (e != cudaSuccess) {
    qeng_weight_free(ctx, w);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_pack_q8: upload failed: %s", cudaGetErrorString(e));
  }
  *out = w;
  return QENG_OK;
}

int32_t qeng_weight_unpack_q8(qeng_ctx* ctx, const qeng_weight* w, int8_t* q, uint16_t* s) {
  if (!ctx || !w || !q || !s) return qeng_fail(ctx, QENG_ERR_ARG, "weight_unpack_q8: null argument");
  if (w->fmt != QENG_FMT_Q8) return qeng_fail(ctx, QENG_ERR_ARG, "weight_unpack_q8: the weight holds 4-bit blocks");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  int8_t* dq = nullptr;
  uint16_t* ds = nullptr;
  const size_t nq = (size_t)w->N * w->K, ns = (size_t)w->N * (w->K / 32);
  QENG_CUDA(ctx, cudaMalloc(&dq, nq));
  if (cudaMalloc(&ds, ns * 2) != cudaSuccess) {
    cudaFree(dq);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_unpack_q8: allocation failed");
  }
  unpack_q8_kernel<<<(unsigned)((nq + 255) / 256), 256>>>(reinterpret_cast<const unsigned char*>(w->qs), w->sc, w->N, w->K,
                                                          w->nchunks, dq, ds);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpy(q, dq, nq, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(s, ds, ns * 2, cudaMemcpyDeviceToHost);
  cudaFree(dq);
  cudaFree(ds);
  if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "weight_unpack_q8: %s", cudaGetErrorString(e));
  return QENG_OK;
}

int32_t qeng_weight_quantize_q8(qeng_ctx* ctx, const void* w_dev, int32_t dtype, int64_t N, int64_t K, int64_t ld,
                                qeng_weight** out, void* stream) {
  if (!ctx || !w_dev || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_quantize_q8: null argument");
  if (dtype != QENG_F32 && dtype != QENG_F16 && dtype != QENG_BF16) return qeng_fail(ctx, QENG_ERR_ARG, "weight_quantize_q8: unknown dtype");
  if (ld < K) return qeng_fail(ctx, QENG_ERR_ARG, "weight_quantize_q8: leading dimension below K");
  qeng_weight* w = nullptr;
  int32_t rc = alloc_q8(ctx, N, K, &w, "weight_quantize_q8");
  if (rc != QENG_OK) return rc;
  const int64_t units = N * w->nchunks * 2;
  quantize_q8_kernel<<<(unsigned)((units + 127) / 128), 128, 0, (cudaStream_t)stream>>>(
      w_dev, dtype, N, K, ld, w->nchunks, reinterpret_cast<unsigned char*>(w->qs), w->sc);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    qeng_weight_free(ctx, w);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_quantize_q8: %s", cudaGetErrorString(e));
  }
  *out = w;
  return QENG_OK;
}

}  // extern "C"
