// Import of 4-bit block weights into the device layout, and the device-side
// inverse (bit-exactness check) and dequantisation.
#include <stdlib.h>
#include <string.h>

#include <cuda_fp16.h>

#include <vector>

#include "qeng_internal.h"

namespace {

// one 32-bit word = codes of k0..k0+7 of one row, nibble j = code[k0+j]
inline uint32_t pack8(const uint8_t* p) {
  uint32_t w = 0;
  for (int j = 0; j < 8; j++) w |= (uint32_t)(p[j] & 15u) << (4 * j);
  return w;
}

// Inverse of the tiling: every thread owns one (row, 8-code word).
__global__ void unpack_q4_kernel(const uint4* __restrict__ qs, const uint2* __restrict__ sc,
                                 int64_t N, int64_t K, int64_t nchunks, uint8_t* __restrict__ q,
                                 uint16_t* __restrict__ s) {
  int64_t words_per_row = K / 8;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * words_per_row) return;
  int64_t n = i / words_per_row, wk = i % words_per_row;  // word index along K
  int64_t blk = wk / 4;
  int t = (int)(wk % 4);
  int64_t tile = n / 16, chunk = blk / 2;
  int r = (int)(n % 16), g = r % 8, hi = r / 8, b1 = (int)(blk % 2);
  const uint32_t* lane = reinterpret_cast<const uint32_t*>(qs + (tile * nchunks + chunk) * 32 + g * 4 + t);
  uint32_t w = lane[b1 * 2 + hi];
  uint8_t* dst = q + n * K + wk * 8;
#pragma unroll
  for (int j = 0; j < 8; j++) dst[j] = (uint8_t)((w >> (4 * j)) & 15u);
  if (t == 0) {
    const uint16_t* sp = reinterpret_cast<const uint16_t*>(sc + (tile * nchunks + chunk) * 8 + g);
    s[n * (K / 32) + blk] = sp[b1 * 2 + hi];
  }
}

__global__ void dequant_q4_kernel(const uint4* __restrict__ qs, const uint2* __restrict__ sc,
                                  int64_t N, int64_t K, int64_t nchunks, float* __restrict__ out) {
  int64_t words_per_row = K / 8;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * words_per_row) return;
  int64_t n = i / words_per_row, wk = i % words_per_row;
  int64_t blk = wk / 4;
  int t = (int)(wk % 4);
  int64_t tile = n / 16, chunk = blk / 2;
  int r = (int)(n % 16), g = r % 8, hi = r / 8, b1 = (int)(blk % 2);
  const uint32_t* lane = reinterpret_cast<const uint32_t*>(qs + (tile * nchunks + chunk) * 32 + g * 4 + t);
  uint32_t w = lane[b1 * 2 + hi];
  const __half* sp = reinterpret_cast<const __half*>(sc + (tile * nchunks + chunk) * 8 + g);
  float scale = __half2float(sp[b1 * 2 + hi]);
  float* dst = out + n * K + wk * 8;
#pragma unroll
  for (int j = 0; j < 8; j++) dst[j] = (float)((int)((w >> (4 * j)) & 15u) - 8) * scale;
}

// Import-time quantiser: one warp per (row tile, 64-wide chunk) writes its 512 bytes of the nibble
// plane and its 64 bytes of the scale plane directly in the device layout.  Lane (g, t) owns rows g
// and g+8, both 32-blocks of the chunk, and the 8 codes at k = 32 blk + 8 t .. + 7 of each.
// Per block: the element of largest magnitude (the first on ties) / -8 is the scale d (stored as
// f16); code = min(15, trunc(x * (1/d) + 8.5)) with separately rounded f32 multiply and add.
__device__ __forceinline__ float load_as_f32(const void* src, int dtype, int64_t i) {
  if (dtype == QENG_F32) return reinterpret_cast<const float*>(src)[i];
  if (dtype == QENG_F16) return __half2float(reinterpret_cast<const __half*>(src)[i]);
  return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(src)[i] << 16);
}

__global__ void __launch_bounds__(256) quantize_q4_kernel(const void* __restrict__ src, int dtype, int64_t K, int64_t ld,
                                                          int64_t nchunks, int64_t nunits, uint4* __restrict__ qs,
                                                          uint2* __restrict__ sc) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (unit >= nunits) return;
  const int64_t tile = unit / nchunks, c = unit % nchunks;
  uint32_t words[4], sbits[4];
#pragma unroll
  for (int idx = 0; idx < 4; ++idx) {
    const int b1 = idx >> 1, hi = idx & 1;
    const int64_t n = tile * 16 + hi * 8 + g, k0 = (2 * c + b1) * 32;
    words[idx] = 0u;
    sbits[idx] = 0u;
    if (k0 >= K) continue;  // padding block of an odd block count: zero codes, zero scale (warp-uniform)
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = load_as_f32(src, dtype, n * ld + k0 + t * 8 + j);
    float amax = -1.f, mval = 0.f;
    int midx = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = fabsf(v[j]);
      if (a > amax) { amax = a; mval = v[j]; midx = t * 8 + j; }
    }
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
      const float oa = __shfl_xor_sync(0xffffffffu, amax, o);
      const float ov = __shfl_xor_sync(0xffffffffu, mval, o);
      const int oi = __shfl_xor_sync(0xffffffffu, midx, o);
      if (oa > amax || (oa == amax && oi < midx)) { amax = oa; mval = ov; midx = oi; }
    }
    const float d = mval * -0.125f;
    const float inv = d != 0.f ? __fdiv_rn(1.0f, d) : 0.f;
    uint32_t w = 0u;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int q = (int)__fadd_rn(__fmul_rn(v[j], inv), 8.5f);
      q = q > 15 ? 15 : (q < 0 ? 0 : q);
      w |= (uint32_t)q << (4 * j);
    }
    words[idx] = w;
    sbits[idx] = (uint32_t)__half_as_ushort(__float2half_rn(d));
  }
  qs[unit * 32 + lane] = make_uint4(words[0], words[1], words[2], words[3]);
  if (t == 0) sc[unit * 8 + g] = make_uint2(sbits[0] | (sbits[1] << 16), sbits[2] | (sbits[3] << 16));
}

}  // namespace

extern "C" {

int32_t qeng_weight_quantize_q4(qeng_ctx* ctx, const void* w_dev, int32_t dtype, int64_t N, int64_t K, int64_t ld,
                                qeng_weight** out, void* stream) {
  if (!ctx || !w_dev || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_quantize_q4: null argument");
  *out = nullptr;
  if (dtype != QENG_F32 && dtype != QENG_F16 && dtype != QENG_BF16)
    return qeng_fail(ctx, QENG_ERR_ARG, "weight_quantize_q4: dtype must be f32, f16 or bf16");
  if (N <= 0 || K <= 0 || K % 32 != 0 || N % 16 != 0 || ld < K)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "weight_quantize_q4: need K %% 32 == 0, N %% 16 == 0, ld >= K (N=%lld K=%lld ld=%lld)",
                     (long long)N, (long long)K, (long long)ld);
  QENG_ENTER(ctx);
  qeng_weight* w = new qeng_weight();
  w->N = N; w->K = K; w->ntiles = N / 16; w->nchunks = (K / 32 + 1) / 2;
  const size_t qs_bytes = (size_t)w->ntiles * w->nchunks * 32 * sizeof(uint4);
  const size_t sc_bytes = (size_t)w->ntiles * w->nchunks * 8 * sizeof(uint2);
  w->qs = nullptr; w->sc = nullptr; w->bytes = (int64_t)(qs_bytes + sc_bytes);
  cudaError_t e = cudaMalloc(&w->qs, qs_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&w->sc, sc_bytes);
  if (e != cudaSuccess) {
    if (w->qs) cudaFree(w->qs);
    delete w;
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_quantize_q4: allocation failed: %s", cudaGetErrorString(e));
  }
  const int64_t nunits = w->ntiles * w->nchunks;
  quantize_q4_kernel<<<(unsigned)((nunits + 7) / 8), 256, 0, (cudaStream_t)stream>>>(w_dev, dtype, K, ld, w->nchunks, nunits,
                                                                                     w->qs, w->sc);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    cudaFree(w->qs);
    cudaFree(w->sc);
    delete w;
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_quantize_q4: launch failed: %s", cudaGetErrorString(e));
  }
  *out = w;
  return QENG_OK;
}


int32_t qeng_weight_pack_q4(qeng_ctx* ctx, const uint8_t* q, const uint16_t* s, int64_t N, int64_t K,
                            qeng_weight** out) {
  if (!ctx || !q || !s || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_pack_q4: null argument");
  *out = nullptr;
  if (N <= 0 || K <= 0 || K % 32 != 0 || N % 16 != 0)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "weight_pack_q4: need K %% 32 == 0 and N %% 16 == 0 (N=%lld K=%lld)",
                     (long long)N, (long long)K);
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  int64_t nblk = K / 32, nchunks = (nblk + 1) / 2, ntiles = N / 16;
  size_t qs_bytes = (size_t)ntiles * nchunks * 32 * sizeof(uint4);
  size_t sc_bytes = (size_t)ntiles * nchunks * 8 * sizeof(uint2);
  uint4* hq = nullptr;
  uint2* hs = nullptr;
  QENG_CUDA(ctx, cudaMallocHost(&hq, qs_bytes));
  if (cudaMallocHost(&hs, sc_bytes) != cudaSuccess) {
    cudaFreeHost(hq);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_pack_q4: pinned allocation failed");
  }
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t tile = 0; tile < ntiles; tile++) {
    for (int64_t c = 0; c < nchunks; c++) {
      uint32_t* wq = reinterpret_cast<uint32_t*>(hq + (tile * nchunks + c) * 32);
      uint16_t* ws = reinterpret_cast<uint16_t*>(hs + (tile * nchunks + c) * 8);
      for (int b1 = 0; b1 < 2; b1++) {
        int64_t blk = 2 * c + b1;
        bool pad = blk >= nblk;
        for (int hi = 0; hi < 2; hi++)
          for (int g = 0; g < 8; g++) {
            int64_t n = tile * 16 + hi * 8 + g;
            ws[g * 4 + b1 * 2 + hi] = pad ? (uint16_t)0 : s[n * nblk + blk];
            for (int t = 0; t < 4; t++) {
              uint32_t w = 0;
              if (!pad) {
                const uint8_t* p = q + n * K + blk * 32 + t * 8;
                for (int j = 0; j < 8; j++) bad |= (p[j] > 15);
                w = pack8(p);
              }
              wq[(g * 4 + t) * 4 + b1 * 2 + hi] = w;
            }
          }
      }
    }
  }
  if (bad) {
    cudaFreeHost(hq);
    cudaFreeHost(hs);
    return qeng_fail(ctx, QENG_ERR_ARG, "weight_pack_q4: code outside 0..15");
  }
  qeng_weight* w = new qeng_weight();
  w->N = N; w->K = K; w->ntiles = ntiles; w->nchunks = nchunks;
  w->qs = nullptr; w->sc = nullptr; w->bytes = (int64_t)(qs_bytes + sc_bytes);
  cudaError_t e = cudaMalloc(&w->qs, qs_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&w->sc, sc_bytes);
  if (e == cudaSuccess) e = cudaMemcpy(w->qs, hq, qs_bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(w->sc, hs, sc_bytes, cudaMemcpyHostToDevice);
  cudaFreeHost(hq);
  cudaFreeHost(hs);
  if (e != cudaSuccess) {
    if (w->qs) cudaFree(w->qs);
    if (w->sc) cudaFree(w->sc);
    delete w;
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_pack_q4: upload failed: %s", cudaGetErrorString(e));
  }
  *out = w;
  return QENG_OK;
}

int32_t qeng_weight_unpack_q4(qeng_ctx* ctx, const qeng_weight* w, uint8_t* q, uint16_t* s) {
  if (!ctx || !w || !q || !s) return qeng_fail(ctx, QENG_ERR_ARG, "weight_unpack_q4: null argument");
  if (w->fmt != QENG_FMT_Q4) return qeng_fail(ctx, QENG_ERR_ARG, "weight_unpack_q4: the weight holds another block format");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  uint8_t* dq = nullptr;
  uint16_t* ds = nullptr;
  size_t nq = (size_t)w->N * w->K, ns = (size_t)w->N * (w->K / 32);
  QENG_CUDA(ctx, cudaMalloc(&dq, nq));
  if (cudaMalloc(&ds, ns * 2) != cudaSuccess) {
    cudaFree(dq);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_unpack_q4: allocation failed");
  }
  int64_t total = w->N * (w->K / 8);
  unpack_q4_kernel<<<(unsigned)((total + 255) / 256), 256>>>(w->qs, w->sc, w->N, w->K, w->nchunks, dq, ds);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpy(q, dq, nq, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(s, ds, ns * 2, cudaMemcpyDeviceToHost);
  cudaFree(dq);
  cudaFree(ds);
  if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "weight_unpack_q4: %s", cudaGetErrorString(e));
  return QENG_OK;
}

int32_t qeng_weight_dequant_f32(qeng_ctx* ctx, const qeng_weight* w, float* out, void* stream) {
  if (!ctx || !w || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_dequant_f32: null argument");
  if (w->fmt == QENG_FMT_K4) {
    qeng_weight_dequant_k4(w, out, (cudaStream_t)stream);
    QENG_LAUNCH_CHECK(ctx);
    return QENG_OK;
  }
  if (w->fmt == QENG_FMT_Q8) {
    qeng_weight_dequant_q8(w, out, (cudaStream_t)stream);
    QENG_LAUNCH_CHECK(ctx);
    return QENG_OK;
  }
  int64_t total = w->N * (w->K / 8);
  dequant_q4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(w->qs, w->sc, w->N, w->K,
                                                                                       w->nchunks, out);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_weight_set_next(qeng_ctx* ctx, qeng_weight* w, const qeng_weight* next) {
  if (!ctx || !w) return qeng_fail(ctx, QENG_ERR_ARG, "weight_set_next: null argument");
  w->next = next;
  return QENG_OK;
}

int32_t qeng_weight_free(qeng_ctx* ctx, qeng_weight* w) {
  if (!w) return QENG_OK;
  if (ctx) cudaSetDevice(ctx->device);
  if (w->qs) cudaFree(w->qs);
  if (w->sc) cudaFree(w->sc);
  delete w;
  return QENG_OK;
}

int64_t qeng_weight_rows(const qeng_weight* w) { return w ? w->N : 0; }
int64_t qeng_weight_cols(const qeng_weight* w) { return w ? w->K : 0; }
int32_t qeng_weight_format(const qeng_weight* w) { return !w ? 0 : (w->fmt == QENG_FMT_Q8 ? 8 : (w->fmt == QENG_FMT_K4 ? 14 : 4)); }
int64_t qeng_weight_device_bytes(const qeng_weight* w) { return w ? w->bytes : 0; }

}  // extern "C"
