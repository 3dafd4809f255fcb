// "K-quant" 4-bit weights (the published Q4_K super-block: 256 weights = 8 sub-blocks of 32, one f16
// scale d and one f16 minimum scale dmin per super-block, a 6-bit scale and a 6-bit minimum per
// sub-block, 4-bit codes): w = (d * sc_j) * code - (dmin * m_j).  The reference names "fused Q4_K
// matmul" as what its own runtime lacked for a catalog model (decide/model-lifecycle.md:175).
//
// Import expands a super-block into what the decode matmul consumes per 32-block: the codes in the
// 4-bit device layout (identical to the one of qeng_weight_pack_q4) and, per (row, 32-block), the
// f32 pair D = d * sc_j, M = dmin * m_j (both products are exact in f32: 11-bit x 6-bit).  Scale plane
// per (row tile, 64-wide chunk, lane group g): {De(g), De(g+8), Do(g), Do(g+8), Me(g), Me(g+8), Mo(g),
// Mo(g+8)} (e / o = the chunk's even / odd block): 256 B per chunk, 0.75 B per weight on the device.
#include <stdlib.h>
#include <string.h>

#include <cuda_fp16.h>

#include <vector>

#include "qeng_internal.h"

namespace {

inline float half_bits_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 31u, man = h & 1023u;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {  // subnormal
      int e = -1;
      uint32_t m = man;
      do { m <<= 1; ++e; } while ((m & 1024u) == 0);
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 1023u) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

inline uint32_t pack8(const uint8_t* p) {
  uint32_t w = 0;
  for (int j = 0; j < 8; j++) w |= (uint32_t)(p[j] & 15u) << (4 * j);
  return w;
}

__global__ void unpack_k4_kernel(const uint4* __restrict__ qs, const float* __restrict__ sc, int64_t N, int64_t K,
                                 int64_t nchunks, uint8_t* __restrict__ q, float* __restrict__ dm) {
  const int64_t words_per_row = K / 8;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * words_per_row) return;
  const int64_t n = i / words_per_row, wk = i % words_per_row;
  const int64_t blk = wk / 4;
  const int t = (int)(wk % 4);
  const int64_t tile = n / 16, chunk = blk / 2;
  const int r = (int)(n % 16), g = r % 8, hi = r / 8, b1 = (int)(blk % 2);
  const uint32_t* lane = reinterpret_cast<const uint32_t*>(qs + (tile * nchunks + chunk) * 32 + g * 4 + t);
  const uint32_t w = lane[b1 * 2 + hi];
  uint8_t* dst = q + n * K + wk * 8;
#pragma unroll
  for (int j = 0; j < 8; j++) dst[j] = (uint8_t)((w >> (4 * j)) & 15u);
  if (t == 0) {
    const float* sp = sc + ((tile * nchunks + chunk) * 8 + g) * 8;
    dm[(n * (K / 32) + blk) * 2] = sp[b1 * 2 + hi];
    dm[(n * (K / 32) + blk) * 2 + 1] = sp[4 + b1 * 2 + hi];
  }
}

__global__ void dequant_k4_kernel(const uint4* __restrict__ qs, const float* __restrict__ sc, int64_t N, int64_t K,
                                  int64_t nchunks, float* __restrict__ out) {
  const int64_t words_per_row = K / 8;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * words_per_row) return;
  const int64_t n = i / words_per_row, wk = i % words_per_row;
  const int64_t blk = wk / 4;
  const int t = (int)(wk % 4);
  const int64_t tile = n / 16, chunk = blk / 2;
  const int r = (int)(n % 16), g = r % 8, hi = r / 8, b1 = (int)(blk % 2);
  const uint32_t* lane = reinterpret_cast<const uint32_t*>(qs + (tile * nchunks + chunk) * 32 + g * 4 + t);
  const uint32_t w = lane[b1 * 2 + hi];
  const float* sp = sc + ((tile * nchunks + chunk) * 8 + g) * 8;
  const float D = sp[b1 * 2 + hi], M = sp[4 + b1 * 2 + hi];
  float* dst = out + n * K + wk * 8;
#pragma unroll
  for (int j = 0; j < 8; j++) dst[j] = __fsub_rn(__fmul_rn(D, (float)((w >> (4 * j)) & 15u)), M);
}

}  // namespace

void qeng_weight_dequant_k4(const qeng_weight* w, float* out, cudaStream_t stream) {
  const int64_t total = w->N * (w->K / 8);
  dequant_k4_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(w->qs, reinterpret_cast<const float*>(w->sc), w->N, w->K,
                                                                         w->nchunks, out);
}

// codes [N][K] (0..15) and (D, M) f32 pairs [N][K/32][2], HOST pointers
int32_t qeng_weight_pack_k4(qeng_ctx* ctx, const uint8_t* q, const float* dm, int64_t N, int64_t K, qeng_weight** out) {
  if (!ctx || !q || !dm || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_pack_k4: null argument");
  *out = nullptr;
  if (N <= 0 || K <= 0 || K % 32 != 0 || N % 16 != 0)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "weight_pack_k4: need K %% 32 == 0 and N %% 16 == 0 (N=%lld K=%lld)", (long long)N, (long long)K);
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t nblk = K / 32, nchunks = (nblk + 1) / 2, ntiles = N / 16;
  const size_t qs_bytes = (size_t)ntiles * nchunks * 512, sc_bytes = (size_t)ntiles * nchunks * 256;
  uint32_t* hq = nullptr;
  float* hs = nullptr;
  QENG_CUDA(ctx, cudaMallocHost(&hq, qs_bytes));
  if (cudaMallocHost(&hs, sc_bytes) != cudaSuccess) {
    cudaFreeHost(hq);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_pack_k4: pinned allocation failed");
  }
  memset(hq, 0, qs_bytes);
  memset(hs, 0, sc_bytes);
  int bad = 0;
#pragma omp parallel for schedule(static) reduction(| : bad)
  for (int64_t n = 0; n < N; n++) {
    const int64_t tile = n / 16, r = n % 16, g = r % 8, hi = r / 8;
    for (int64_t blk = 0; blk < nblk; blk++) {
      const int64_t chunk = blk / 2, b1 = blk % 2;
      float* sp = hs + ((tile * nchunks + chunk) * 8 + g) * 8;
      sp[b1 * 2 + hi] = dm[(n * nblk + blk) * 2];
      sp[4 + b1 * 2 + hi] = dm[(n * nblk + blk) * 2 + 1];
      for (int t = 0; t < 4; t++) {
        const uint8_t* p = q + n * K + blk * 32 + t * 8;
        for (int j = 0; j < 8; j++) bad |= (p[j] > 15);
        hq[(((tile * nchunks + chunk) * 32 + g * 4 + t) * 4) + b1 * 2 + hi] = pack8(p);
      }
    }
  }
  if (bad) {
    cudaFreeHost(hq);
    cudaFreeHost(hs);
    return qeng_fail(ctx, QENG_ERR_ARG, "weight_pack_k4: code outside 0..15");
  }
  qeng_weight* w = new qeng_weight();
  w->fmt = QENG_FMT_K4;
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
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_pack_k4: upload failed: %s", cudaGetErrorString(e));
  }
  *out = w;
  return QENG_OK;
}

// One row-major matrix of Q4_K super-blocks (144 bytes per 256 weights: f16 d, f16 dmin, 12 bytes of
// packed 6-bit scales and minima, 128 bytes of codes) -> codes and (D, M) pairs per 32-block.
int32_t qeng_q4k_expand(qeng_ctx* ctx, const uint8_t* blocks, int64_t N, int64_t K, std::vector<uint8_t>* q, std::vector<float>* dm) {
  if (K % 256 != 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "q4_k: K must be a multiple of 256 (K=%lld)", (long long)K);
  const int64_t nsb = K / 256;
  q->resize((size_t)N * K);
  dm->resize((size_t)N * (K / 32) * 2);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    for (int64_t sb = 0; sb < nsb; sb++) {
      const uint8_t* b = blocks + (n * nsb + sb) * 144;
      uint16_t hd, hm;
      memcpy(&hd, b, 2);
      memcpy(&hm, b + 2, 2);
      const float d = half_bits_to_float(hd), dmin = half_bits_to_float(hm);
      const uint8_t* sc = b + 4;
      const uint8_t* qs = b + 16;
      for (int j = 0; j < 8; j++) {
        int s6, m6;
        if (j < 4) {
          s6 = sc[j] & 63;
          m6 = sc[j + 4] & 63;
        } else {
          s6 = (sc[j + 4] & 15) | ((sc[j - 4] >> 6) << 4);
          m6 = (sc[j + 4] >> 4) | ((sc[j] >> 6) << 4);
        }
        float* o = dm->data() + ((size_t)(n * (K / 32) + sb * 8 + j)) * 2;
        o[0] = d * (float)s6;
        o[1] = dmin * (float)m6;
        // sub-blocks 2i and 2i+1 share 32 bytes: low nibbles = sub-block 2i, high nibbles = 2i+1
        const uint8_t* src = qs + (j / 2) * 32;
        uint8_t* dst = q->data() + (size_t)n * K + sb * 256 + j * 32;
        for (int k = 0; k < 32; k++) dst[k] = (j & 1) ? (uint8_t)(src[k] >> 4) : (uint8_t)(src[k] & 15);
      }
    }
  }
  return QENG_OK;
}

extern "C" {

int32_t qeng_weight_pack_q4k(qeng_ctx* ctx, const uint8_t* blocks, int64_t N, int64_t K, qeng_weight** out) {
  if (!ctx || !blocks || !out) return qeng_fail(ctx, QENG_ERR_ARG, "weight_pack_q4k: null argument");
  *out = nullptr;
  if (N <= 0 || N % 16 != 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "weight_pack_q4k: N must be a positive multiple of 16");
  std::vector<uint8_t> q;
  std::vector<float> dm;
  int32_t rc = qeng_q4k_expand(ctx, blocks, N, K, &q, &dm);
  if (rc != QENG_OK) return rc;
  return qeng_weight_pack_k4(ctx, q.data(), dm.data(), N, K, out);
}

int32_t qeng_weight_unpack_k4(qeng_ctx* ctx, const qeng_weight* w, uint8_t* q, float* dm) {
  if (!ctx || !w || !q || !dm) return qeng_fail(ctx, QENG_ERR_ARG, "weight_unpack_k4: null argument");
  if (w->fmt != QENG_FMT_K4) return qeng_fail(ctx, QENG_ERR_ARG, "weight_unpack_k4: the weight holds another block format");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  uint8_t* dq = nullptr;
  float* ds = nullptr;
  const size_t nq = (size_t)w->N * w->K, ns = (size_t)w->N * (w->K / 32) * 2;
  QENG_CUDA(ctx, cudaMalloc(&dq, nq));
  if (cudaMalloc(&ds, ns * 4) != cudaSuccess) {
    cudaFree(dq);
    return qeng_fail(ctx, QENG_ERR_CUDA, "weight_unpack_k4: allocation failed");
  }
  const int64_t total = w->N * (w->K / 8);
  unpack_k4_kernel<<<(unsigned)((total + 255) / 256), 256>>>(w->qs, reinterpret_cast<const float*>(w->sc), w->N, w->K, w->nchunks, dq, ds);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpy(q, dq, nq, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(dm, ds, ns * 4, cudaMemcpyDeviceToHost);
  cudaFree(dq);
  cudaFree(ds);
  if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "weight_unpack_k4: %s", cudaGetErrorString(e));
  return QENG_OK;
}

}  // extern "C"
