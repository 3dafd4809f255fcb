// Small operators of the decode loop: RMSNorm, RoPE, SwiGLU, residual add,
// embedding gather, bf16 LM head, greedy argmax.  All are HBM- or
// latency-bound elementwise / row-reduction kernels.
#include <math.h>

#include "qeng_internal.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < nw; ++w) tot += sh[w];
  return tot;
}

__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gamma, int D, float eps,
                               float* __restrict__ y) {
  __shared__ float sh[32];
  const float* xr = x + (size_t)blockIdx.x * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) ss += xr[i] * xr[i];
  const float r = rsqrtf(block_sum(ss, sh) / (float)D + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) y[(size_t)blockIdx.x * D + i] = xr[i] * r * gamma[i];
}

// standalone RoPE: angles in double so that no table is needed
__global__ void rope_kernel(float* x, const int32_t* pos, int H, int hd, float base) {
  const int m = blockIdx.x, half = hd / 2;
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx - h * half;
    const double ang = (double)pos[m] * pow((double)base, -2.0 * (double)i / (double)hd);
    double s, c;
    sincos(ang, &s, &c);
    float* p = x + ((size_t)m * H + h) * hd;
    const double a = p[i], b = p[i + half];
    p[i] = (float)(a * c - b * s);
    p[i + half] = (float)(b * c + a * s);
  }
}

__global__ void swiglu_kernel(const float* __restrict__ gate, const float* __restrict__ up, int64_t n,
                              float* __restrict__ y) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float g = gate[i];
    y[i] = g / (1.0f + expf(-g)) * up[i];
  }
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t n, float* __restrict__ y) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = a[i] + b[i];
}

__global__ void embed_kernel(const uint16_t* __restrict__ table, const int32_t* __restrict__ tokens, int D, int V,
                             float* __restrict__ x, int32_t* status) {
  const int m = blockIdx.x;
  int tok = tokens[m];
  if ((unsigned)tok >= (unsigned)V) {
    if (threadIdx.x == 0) atomicExch(status, 3);
    tok = 0;
  }
  for (int i = threadIdx.x; i < D; i += blockDim.x)
    x[(size_t)m * D + i] = __uint_as_float((uint32_t)table[(size_t)tok * D + i] << 16);
}

// LM head: one warp per vocabulary row, up to kLmM activation rows staged in shared memory
// (optionally RMS-normalised on the way in).  Each lane keeps 8 independent 128-bit weight loads
// in flight.  With finalisation, every CTA leaves its (max, lowest index) per row in a scratch
// slot and the CTA that arrives last (atomic counter, no waiting) picks the token, records it,
// advances the sequences and gathers the next embedding.
constexpr int kLmM = 4;
constexpr int kLmU = 8;

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); }

__global__ void __launch_bounds__(256) lm_head_kernel(const qeng_lm_tail t, float* part_val, int32_t* part_idx,
                                                      int32_t* counter, int32_t* status) {
  extern __shared__ __align__(16) float xs[];  // [M][D]
  __shared__ float sh[32];
  __shared__ float wv[8][kLmM];
  __shared__ int wi[8][kLmM];
  __shared__ int s_last;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int M = t.M, D = t.D, V = t.V;
  const int v0 = t.v0, Vtot = t.Vtot > 0 ? t.Vtot : V;
  const size_t ldl = t.Vtot > 0 ? (size_t)t.ldl : (size_t)V;
  for (int m = 0; m < M; ++m) {
    float rs = 1.f;
    if (t.gamma != nullptr) {
      float ss = 0.f;
      for (int i = tid; i < D; i += 256) {
        const float v = t.x[(size_t)m * D + i];
        ss += v * v;
      }
      rs = rsqrtf(block_sum(ss, sh) / (float)D + t.eps);
    }
    for (int i = tid; i < D; i += 256)
      xs[(size_t)m * D + i] = t.gamma != nullptr ? t.x[(size_t)m * D + i] * rs * t.gamma[i] : t.x[(size_t)m * D + i];
  }
  __syncthreads();

  float bestv[kLmM];
  int besti[kLmM];
#pragma unroll
  for (int m = 0; m < kLmM; ++m) { bestv[m] = -INFINITY; besti[m] = 0x7fffffff; }
  const int nwarps = gridDim.x * 8;
  const int nvec = D / 8;
  const uint4* table = reinterpret_cast<const uint4*>(t.table);
  for (int v = blockIdx.x * 8 + warp; v < V; v += nwarps) {
    const uint4* row = table + (size_t)v * nvec;
    float acc[kLmM];
#pragma unroll
    for (int m = 0; m < kLmM; ++m) acc[m] = 0.f;
    for (int c0 = lane; c0 < nvec; c0 += 32 * kLmU) {
      uint4 w[kLmU];
#pragma unroll
      for (int u = 0; u < kLmU; ++u) {
        const int c = c0 + 32 * u;
        w[u] = make_uint4(0u, 0u, 0u, 0u);
        if (c < nvec)
          asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                       : "=r"(w[u].x), "=r"(w[u].y), "=r"(w[u].z), "=r"(w[u].w)
                       : "l"(row + c));
      }
#pragma unroll
      for (int u = 0; u < kLmU; ++u) {
        const int c = c0 + 32 * u;
        if (c < nvec) {
          float wf[8];
          wf[0] = __uint_as_float(w[u].x << 16); wf[1] = __uint_as_float(w[u].x & 0xffff0000u);
          wf[2] = __uint_as_float(w[u].y << 16); wf[3] = __uint_as_float(w[u].y & 0xffff0000u);
          wf[4] = __uint_as_float(w[u].z << 16); wf[5] = __uint_as_float(w[u].z & 0xffff0000u);
          wf[6] = __uint_as_float(w[u].w << 16); wf[7] = __uint_as_float(w[u].w & 0xffff0000u);
#pragma unroll
          for (int m = 0; m < kLmM; ++m) {
            if (m < M) {
              const float4 x0 = *reinterpret_cast<const float4*>(xs + (size_t)m * D + c * 8);
              const float4 x1 = *reinterpret_cast<const float4*>(xs + (size_t)m * D + c * 8 + 4);
              acc[m] += wf[0] * x0.x + wf[1] * x0.y + wf[2] * x0.z + wf[3] * x0.w + wf[4] * x1.x + wf[5] * x1.y +
                        wf[6] * x1.z + wf[7] * x1.w;
            }
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kLmM; ++m) {
      if (m < M) {
        const float tot = warp_sum(acc[m]);
        if (lane == 0) t.logits[(size_t)m * ldl + v0 + v] = t.softcap > 0.f ? t.softcap * tanhf(tot / t.softcap) : tot;
        if (better(tot, v0 + v, bestv[m], besti[m])) { bestv[m] = tot; besti[m] = v0 + v; }
      }
    }
  }
  if (t.next == nullptr && t.pairs == nullptr) return;

  // ---- greedy finalisation ---------------------------------------------------------------
  if (lane == 0)
    for (int m = 0; m < M; ++m) { wv[warp][m] = bestv[m]; wi[warp][m] = besti[m]; }
  __syncthreads();
  if (tid < M) {
    float bv = wv[0][tid];
    int bi = wi[0][tid];
    for (int w = 1; w < 8; ++w)
      if (better(wv[w][tid], wi[w][tid], bv, bi)) { bv = wv[w][tid]; bi = wi[w][tid]; }
    __stcg(part_val + (size_t)blockIdx.x * kLmM + tid, bv);
    __stcg(part_idx + (size_t)blockIdx.x * kLmM + tid, bi);
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(counter, 1) == (int)gridDim.x - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  __shared__ int tok[kLmM];
  for (int m = 0; m < M; ++m) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = tid; c < (int)gridDim.x; c += 256) {
      const float v = __ldcg(part_val + (size_t)c * kLmM + m);
      const int i = __ldcg(part_idx + (size_t)c * kLmM + m);
      if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    __syncthreads();
    if (lane == 0) { wv[warp][0] = bv; wi[warp][0] = bi; }
    __syncthreads();
    if (tid == 0) {
      for (int w = 1; w < 8; ++w)
        if (better(wv[w][0], wi[w][0], bv, bi)) { bv = wv[w][0]; bi = wi[w][0]; }
      if (t.pairs != nullptr) {  // a vocabulary shard: the ranks' (max, index) pairs meet in a later kernel
        t.pairs[2 * (t.pair_slot + m)] = bv;
        t.pairs[2 * (t.pair_slot + m) + 1] = (float)bi;  // exact: sharded vocabularies stay below 2^24
        continue;
      }
      if ((unsigned)bi >= (unsigned)Vtot) { bi = 0; atomicExch(status, 3); }  // only if every logit was NaN
      tok[m] = bi;
      t.next[m] = bi;
      const int st = *t.step;
      t.out_tokens[(size_t)(st + 1) * M + m] = bi;
      t.pos[m] += 1;
      t.lens[m] += 1;
    }
  }
  __syncthreads();
  if (tid == 0) {
    if (t.pairs == nullptr) *t.step += 1;
    *counter = 0;  // ready for the next launch
  }
  if (t.pairs != nullptr) return;
  for (int m = 0; m < M; ++m)
    for (int i = tid; i < D; i += 256)
      t.xout[(size_t)m * D + i] = __uint_as_float((uint32_t)t.emb[(size_t)tok[m] * D + i] << 16);
}

__global__ void argmax_kernel(const float* __restrict__ logits, int V, int32_t* __restrict__ idx) {
  __shared__ float bv[32];
  __shared__ int bi[32];
  const float* row = logits + (size_t)blockIdx.x * V;
  float best = -INFINITY;
  int besti = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best || (v == best && i < besti)) { best = v; besti = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, besti, o);
    if (ov > best || (ov == best && oi < besti)) { best = ov; besti = oi; }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { bv[warp] = best; bi[warp] = besti; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (bv[w] > best || (bv[w] == best && bi[w] < besti)) { best = bv[w]; besti = bi[w]; }
    idx[blockIdx.x] = besti == 0x7fffffff ? 0 : besti;
  }
}

}  // namespace

int32_t qeng_lm_head_fused(qeng_ctx* ctx, const qeng_lm_tail& t, cudaStream_t stream) {
  if (t.M < 1 || t.M > kLmM) return qeng_fail(ctx, QENG_ERR_SHAPE, "lm_head: at most %d rows per launch", kLmM);
  if (t.V <= 0 || t.D <= 0 || t.D % 8 != 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "lm_head: D must be a positive multiple of 8");
  if ((size_t)t.M * t.D * 4 > 200 * 1024) return qeng_fail(ctx, QENG_ERR_SHAPE, "lm_head: D too large for the staging buffer");
  if ((reinterpret_cast<uintptr_t>(t.table) & 15) != 0) return qeng_fail(ctx, QENG_ERR_ALIGN, "lm_head: table must be 16-byte aligned");
  static bool configured_on[64] = {};  // the opt-in shared-memory size is set per device
  bool& configured = configured_on[ctx->device & 63];
  if (!configured) {
    QENG_CUDA(ctx, cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  const int grid = ctx->sm_count * 2;
  lm_head_kernel<<<grid, 256, (size_t)t.M * t.D * 4, stream>>>(t, ctx->tail_val, ctx->tail_idx, ctx->tail_cnt, ctx->status);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

extern "C" {

int32_t qeng_rmsnorm(qeng_ctx* ctx, const float* x, const float* gamma, int64_t M, int64_t D, float eps, float* y,
                     void* stream) {
  if (!ctx || !x || !gamma || !y) return qeng_fail(ctx, QENG_ERR_ARG, "rmsnorm: null argument");
  if (M <= 0 || D <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "rmsnorm: empty shape");
  QENG_ENTER(ctx);
  rmsnorm_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(x, gamma, (int)D, eps, y);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_rope(qeng_ctx* ctx, float* x, const int32_t* pos, int64_t M, int64_t H, int64_t hd, float base,
                  void* stream) {
  if (!ctx || !x || !pos) return qeng_fail(ctx, QENG_ERR_ARG, "rope: null argument");
  if (M <= 0 || H <= 0 || hd <= 0 || hd % 2) return qeng_fail(ctx, QENG_ERR_SHAPE, "rope: bad shape");
  QENG_ENTER(ctx);
  rope_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(x, pos, (int)H, (int)hd, base);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_swiglu(qeng_ctx* ctx, const float* gate, const float* up, int64_t n, float* y, void* stream) {
  if (!ctx || !gate || !up || !y) return qeng_fail(ctx, QENG_ERR_ARG, "swiglu: null argument");
  if (n <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "swiglu: empty shape");
  QENG_ENTER(ctx);
  swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gate, up, n, y);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_add(qeng_ctx* ctx, const float* a, const float* b, int64_t n, float* y, void* stream) {
  if (!ctx || !a || !b || !y) return qeng_fail(ctx, QENG_ERR_ARG, "add: null argument");
  if (n <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "add: empty shape");
  QENG_ENTER(ctx);
  add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, n, y);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_embed(qeng_ctx* ctx, const uint16_t* table_bf16, const int32_t* tokens, int64_t M, int64_t D, int64_t V,
                   float* x, void* stream) {
  if (!ctx || !table_bf16 || !tokens || !x) return qeng_fail(ctx, QENG_ERR_ARG, "embed: null argument");
  if (M <= 0 || D <= 0 || V <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "embed: empty shape");
  QENG_ENTER(ctx);
  embed_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(table_bf16, tokens, (int)D, (int)V, x, ctx->status);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_lm_head(qeng_ctx* ctx, const uint16_t* table_bf16, const float* x, int64_t M, int64_t D, int64_t V,
                                float* logits, void* stream) {
  if (!ctx || !table_bf16 || !x || !logits) return qeng_fail(ctx, QENG_ERR_ARG, "lm_head: null argument");
  if (M <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "lm_head: empty shape");
  QENG_ENTER(ctx);
  for (int64_t m0 = 0; m0 < M; m0 += kLmM) {
    qeng_lm_tail t;
    t.table = table_bf16; t.x = x + m0 * D; t.M = (int)(M - m0 < kLmM ? M - m0 : kLmM); t.D = (int)D; t.V = (int)V;
    t.logits = logits + m0 * V;
    int32_t rc = qeng_lm_head_fused(ctx, t, (cudaStream_t)stream);
    if (rc != QENG_OK) return rc;
  }
  return QENG_OK;
}

int32_t qeng_argmax(qeng_ctx* ctx, const float* logits, int64_t M, int64_t V, int32_t* idx, void* stream) {
  if (!ctx || !logits || !idx) return qeng_fail(ctx, QENG_ERR_ARG, "argmax: null argument");
  if (M <= 0 || V <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "argmax: empty shape");
  QENG_ENTER(ctx);
  argmax_kernel<<<(unsigned)M, 1024, 0, (cudaStream_t)stream>>>(logits, (int)V, idx);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

}  // extern "C"
