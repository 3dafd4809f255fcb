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

// LM head: one warp per vocabulary row, up to kLmM activation rows held in shared memory.
constexpr int kLmM = 4;
__global__ void __launch_bounds__(256) lm_head_kernel(const uint4* __restrict__ table, const float* __restrict__ x,
                                                      int M, int D, int V, float* __restrict__ logits) {
  extern __shared__ __align__(16) float xs[];  // [M][D]
  for (int i = threadIdx.x; i < M * D; i += blockDim.x) xs[i] = x[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int nwarps = gridDim.x * (blockDim.x >> 5);
  for (int v = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); v < V; v += nwarps) {
    const uint4* row = table + (size_t)v * (D / 8);
    float acc[kLmM];
#pragma unroll
    for (int m = 0; m < kLmM; ++m) acc[m] = 0.f;
    for (int c = lane; c < D / 8; c += 32) {
      uint4 w;
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                   : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                   : "l"(row + c));
      float wf[8];
      wf[0] = __uint_as_float(w.x << 16); wf[1] = __uint_as_float(w.x & 0xffff0000u);
      wf[2] = __uint_as_float(w.y << 16); wf[3] = __uint_as_float(w.y & 0xffff0000u);
      wf[4] = __uint_as_float(w.z << 16); wf[5] = __uint_as_float(w.z & 0xffff0000u);
      wf[6] = __uint_as_float(w.w << 16); wf[7] = __uint_as_float(w.w & 0xffff0000u);
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
#pragma unroll
    for (int m = 0; m < kLmM; ++m) {
      const float tot = warp_sum(acc[m]);
      if (m < M && lane == 0) logits[(size_t)m * V + v] = tot;
    }
  }
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

extern "C" {

int32_t qeng_rmsnorm(qeng_ctx* ctx, const float* x, const float* gamma, int64_t M, int64_t D, float eps, float* y,
                     void* stream) {
  if (!ctx || !x || !gamma || !y) return qeng_fail(ctx, QENG_ERR_ARG, "rmsnorm: null argument");
  if (M <= 0 || D <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "rmsnorm: empty shape");
  rmsnorm_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(x, gamma, (int)D, eps, y);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_rope(qeng_ctx* ctx, float* x, const int32_t* pos, int64_t M, int64_t H, int64_t hd, float base,
                  void* stream) {
  if (!ctx || !x || !pos) return qeng_fail(ctx, QENG_ERR_ARG, "rope: null argument");
  if (M <= 0 || H <= 0 || hd <= 0 || hd % 2) return qeng_fail(ctx, QENG_ERR_SHAPE, "rope: bad shape");
  rope_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(x, pos, (int)H, (int)hd, base);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_swiglu(qeng_ctx* ctx, const float* gate, const float* up, int64_t n, float* y, void* stream) {
  if (!ctx || !gate || !up || !y) return qeng_fail(ctx, QENG_ERR_ARG, "swiglu: null argument");
  if (n <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "swiglu: empty shape");
  swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(gate, up, n, y);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_add(qeng_ctx* ctx, const float* a, const float* b, int64_t n, float* y, void* stream) {
  if (!ctx || !a || !b || !y) return qeng_fail(ctx, QENG_ERR_ARG, "add: null argument");
  if (n <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "add: empty shape");
  add_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, n, y);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_embed(qeng_ctx* ctx, const uint16_t* table_bf16, const int32_t* tokens, int64_t M, int64_t D, int64_t V,
                   float* x, void* stream) {
  if (!ctx || !table_bf16 || !tokens || !x) return qeng_fail(ctx, QENG_ERR_ARG, "embed: null argument");
  if (M <= 0 || D <= 0 || V <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "embed: empty shape");
  embed_kernel<<<(unsigned)M, 256, 0, (cudaStream_t)stream>>>(table_bf16, tokens, (int)D, (int)V, x, ctx->status);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_lm_head(qeng_ctx* ctx, const uint16_t* table_bf16, const float* x, int64_t M, int64_t D, int64_t V,
                     float* logits, void* stream) {
  if (!ctx || !table_bf16 || !x || !logits) return qeng_fail(ctx, QENG_ERR_ARG, "lm_head: null argument");
  if (M <= 0 || V <= 0 || D <= 0 || D % 8 != 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "lm_head: D must be a positive multiple of 8");
  if ((size_t)kLmM * D * 4 > 200 * 1024) return qeng_fail(ctx, QENG_ERR_SHAPE, "lm_head: D too large for the staging buffer");
  if ((reinterpret_cast<uintptr_t>(table_bf16) & 15) != 0) return qeng_fail(ctx, QENG_ERR_ALIGN, "lm_head: table must be 16-byte aligned");
  static bool configured = false;
  if (!configured) {
    QENG_CUDA(ctx, cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  int grid = ctx->sm_count * 2;
  for (int64_t m0 = 0; m0 < M; m0 += kLmM) {
    int mm = (int)(M - m0 < kLmM ? M - m0 : kLmM);
    lm_head_kernel<<<grid, 256, (size_t)mm * D * 4, (cudaStream_t)stream>>>(
        reinterpret_cast<const uint4*>(table_bf16), x + m0 * D, mm, (int)D, (int)V, logits + m0 * V);
    QENG_LAUNCH_CHECK(ctx);
  }
  return QENG_OK;
}

int32_t qeng_argmax(qeng_ctx* ctx, const float* logits, int64_t M, int64_t V, int32_t* idx, void* stream) {
  if (!ctx || !logits || !idx) return qeng_fail(ctx, QENG_ERR_ARG, "argmax: null argument");
  if (M <= 0 || V <= 0) return qeng_fail(ctx, QENG_ERR_SHAPE, "argmax: empty shape");
  argmax_kernel<<<(unsigned)M, 1024, 0, (cudaStream_t)stream>>>(logits, (int)V, idx);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

}  // extern "C"
