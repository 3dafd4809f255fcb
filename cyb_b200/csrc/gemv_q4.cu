// Decode-side quantized matmul: y[M,N] = x[M,K] . dequant(W)^T for small M.
//
// The kernel is HBM-bound: it streams the packed 4-bit weights exactly once
// with warp-wide 128-bit loads (512 contiguous bytes per instruction), unpacks
// them in registers and contracts them on the tensor pipe with
// mma.sync.m16n8k16 (weights = A rows, activations = B columns), so the same
// code serves M = 1 .. 32 at no extra memory traffic.
//
// Arithmetic (exact up to f32 accumulation):
//  * a 4-bit code c is placed in the low bits of an f16, i.e. the subnormal
//    c * 2^-24: one AND per two codes, no int->float conversion;
//  * f32 activations are split x = hi + lo into two f16 terms that occupy two
//    B columns, so no activation precision is lost (bf16/f16 activations use
//    one column);
//  * the zero point is removed per 32-block from the activation block sums:
//    sum_k x_k (c_k - 8) = sum_k x_k c_k - 8 sum_k x_k;
//  * the f16 block scale is applied in f32 to the block result.
#include <mma.h>

#include "qeng_internal.h"

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

struct GemvParams {
  const uint4* qs;
  const uint2* sc;
  int ntiles, nchunks;
  int K;
  const void* x;
  int x_dtype;
  long long ldx;
  int M, cols, split;
  float* y;
  long long ldy;
  const float* gamma;
  float eps;
  int epilogue;
  const float* resid;
  int slice_chunks;  // chunks of 64 k staged in shared memory at once
};

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream(const uint2* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ float load_act(const void* x, int dtype, long long i) {
  if (dtype == QENG_F32) return reinterpret_cast<const float*>(x)[i];
  if (dtype == QENG_F16) return __half2float(reinterpret_cast<const __half*>(x)[i]);
  uint32_t u = (uint32_t)reinterpret_cast<const uint16_t*>(x)[i] << 16;
  return __uint_as_float(u);
}

// position of k (relative to the slice start) inside the staged f16 row: the
// eight values of one (block, t) group are stored in the order 0,4,1,5,2,6,3,7
// so that one 128-bit shared load yields the four B registers of both MMAs.
__device__ __forceinline__ int stage_pos(int kk) {
  int j = kk & 7;
  return (kk & ~7) + ((j & 3) << 1) + (j >> 2);
}

template <int NT, int U>
__global__ void __launch_bounds__(kThreads) gemv_q4_kernel(const GemvParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int slice_k = p.slice_chunks * 64;
  const int CS = slice_k + 32;  // column stride in halves (64-byte skew between columns)
  __half* xs_h = reinterpret_cast<__half*>(smem_raw);
  float* xsum = reinterpret_cast<float*>(smem_raw + (size_t)p.cols * CS * 2);
  float* red = xsum + p.slice_chunks * 2 * (8 * NT);
  float* rinv = red + kWarps * 16 * 8 * NT;  // [M] 1/rms when the norm is fused
  __shared__ float warp_part[kWarps];

  const int nslices = (p.nchunks + p.slice_chunks - 1) / p.slice_chunks;

  // fused RMSNorm: 1/rms of every activation row, computed once per CTA
  if (p.gamma != nullptr) {
    for (int m = 0; m < p.M; ++m) {
      float ss = 0.f;
      for (int k = tid; k < p.K; k += kThreads) {
        float v = load_act(p.x, p.x_dtype, (long long)m * p.ldx + k);
        ss += v * v;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) warp_part[warp] = ss;
      __syncthreads();
      if (tid == 0) {
        float tot = 0.f;
        for (int w = 0; w < kWarps; ++w) tot += warp_part[w];
        rinv[m] = rsqrtf(tot / (float)p.K + p.eps);
      }
      __syncthreads();
    }
  }

  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

    const uint4* qbase = p.qs + (size_t)tile * p.nchunks * 32 + lane;
    const uint2* sbase = p.sc + (size_t)tile * p.nchunks * 8 + g;

    for (int slice = 0; slice < nslices; ++slice) {
      const int c_begin = slice * p.slice_chunks;
      const int c_end = min(p.nchunks, c_begin + p.slice_chunks);
      uint4 wq[U];
      uint2 ws[U];
      // the first batch of weight loads does not depend on the activations:
      // issue it before the staging so both latencies overlap
      int c0 = c_begin + warp;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        int c = c0 + u * kWarps;
        if (c < c_end) {
          wq[u] = ldg_stream(qbase + (size_t)c * 32);
          ws[u] = ldg_stream(sbase + (size_t)c * 8);
        }
      }
      const bool restage = (nslices > 1) || (tile == (int)blockIdx.x);
      if (restage) {
        if (slice > 0 || tile != (int)blockIdx.x) __syncthreads();  // readers of the previous slice are done
        const int k0 = c_begin * 64;
        const int kn = (c_end - c_begin) * 64;
        for (int idx = tid; idx < p.M * kn; idx += kThreads) {
          int m = idx / kn, kk = idx - m * kn, k = k0 + kk;
          float v = 0.f;
          if (k < p.K) {
            v = load_act(p.x, p.x_dtype, (long long)m * p.ldx + k);
            if (p.gamma != nullptr) v = v * rinv[m] * p.gamma[k];
          }
          int pos = stage_pos(kk);
          if (p.split) {
            __half hi = __float2half_rn(v);
            __half lo = __float2half_rn(v - __half2float(hi));
            xs_h[(size_t)(2 * m) * CS + pos] = hi;
            xs_h[(size_t)(2 * m + 1) * CS + pos] = lo;
          } else {
            xs_h[(size_t)m * CS + pos] = __float2half_rn(v);
          }
        }
        __syncthreads();
        // block sums carry the zero point: -8 * 2^-24 * sum of the staged f16 values
        const int nblk = (c_end - c_begin) * 2;
        for (int idx = tid; idx < nblk * 8 * NT; idx += kThreads) {
          int col = idx / nblk, blk = idx - col * nblk;
          float sum = 0.f;
          if (col < p.cols) {
            const __half2* h2 = reinterpret_cast<const __half2*>(xs_h + (size_t)col * CS + blk * 32);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              float2 f = __half22float2(h2[i]);
              sum += f.x + f.y;
            }
          }
          xsum[blk * (8 * NT) + col] = sum * (-8.0f * 5.9604644775390625e-08f);
        }
        __syncthreads();
      }

      while (c0 < c_end) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          int c = c0 + u * kWarps;
          if (c < c_end) {
            const int cl = c - c_begin;
            const uint4 w = wq[u];
            const uint2 s2 = ws[u];
#pragma unroll
            for (int b1 = 0; b1 < 2; ++b1) {
              const uint32_t w0 = b1 ? w.z : w.x, w1 = b1 ? w.w : w.y;
              const uint32_t m4 = 0x000f000fu;
              const uint32_t a00 = w0 & m4, a01 = w1 & m4, a02 = (w0 >> 4) & m4, a03 = (w1 >> 4) & m4;
              const uint32_t a10 = (w0 >> 8) & m4, a11 = (w1 >> 8) & m4, a12 = (w0 >> 12) & m4,
                             a13 = (w1 >> 12) & m4;
              const uint32_t sbits = b1 ? s2.y : s2.x;
              const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sbits));
              const int blk = cl * 2 + b1;
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                uint4 xb = make_uint4(0u, 0u, 0u, 0u);
                if (nt * 8 + g < p.cols)
                  xb = *reinterpret_cast<const uint4*>(xs_h + (size_t)(nt * 8 + g) * CS + blk * 32 + t * 8);
                float d[4] = {0.f, 0.f, 0.f, 0.f};
                mma16816(d, a00, a01, a02, a03, xb.x, xb.y);
                mma16816(d, a10, a11, a12, a13, xb.z, xb.w);
                const float2 z = *reinterpret_cast<const float2*>(xsum + blk * (8 * NT) + nt * 8 + 2 * t);
                acc[nt][0] = fmaf(sf.x, d[0] + z.x, acc[nt][0]);
                acc[nt][1] = fmaf(sf.x, d[1] + z.y, acc[nt][1]);
                acc[nt][2] = fmaf(sf.y, d[2] + z.x, acc[nt][2]);
                acc[nt][3] = fmaf(sf.y, d[3] + z.y, acc[nt][3]);
              }
            }
          }
        }
        c0 += U * kWarps;
        if (c0 < c_end) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            int c = c0 + u * kWarps;
            if (c < c_end) {
              wq[u] = ldg_stream(qbase + (size_t)c * 32);
              ws[u] = ldg_stream(sbase + (size_t)c * 8);
            }
          }
        }
      }
    }

    // ---- cross-warp reduction and epilogue ---------------------------------
    // red[warp][act][row16]
    const int acts = p.split ? 4 * NT : 8 * NT;
    float* myred = red + warp * (16 * 8 * NT);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (p.split) {
        int a = nt * 4 + t;
        myred[a * 16 + g] = acc[nt][0] + acc[nt][1];
        myred[a * 16 + g + 8] = acc[nt][2] + acc[nt][3];
      } else {
        int a = nt * 8 + 2 * t;
        myred[a * 16 + g] = acc[nt][0];
        myred[(a + 1) * 16 + g] = acc[nt][1];
        myred[a * 16 + g + 8] = acc[nt][2];
        myred[(a + 1) * 16 + g + 8] = acc[nt][3];
      }
    }
    __syncthreads();
    if (p.epilogue == QENG_EPI_SWIGLU) {
      for (int e = tid; e < acts * 8; e += kThreads) {
        int a = e >> 3, r = e & 7;
        if (a < p.M) {
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            gate += red[w * (16 * 8 * NT) + a * 16 + r];
            up += red[w * (16 * 8 * NT) + a * 16 + r + 8];
          }
          gate *= 16777216.0f;
          up *= 16777216.0f;
          p.y[(size_t)a * p.ldy + (size_t)tile * 8 + r] = gate / (1.0f + __expf(-gate)) * up;
        }
      }
    } else
    for (int e = tid; e < acts * 16; e += kThreads) {
      int a = e >> 4, r = e & 15;
      if (a < p.M) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += red[w * (16 * 8 * NT) + e];
        v *= 16777216.0f;
        size_t o = (size_t)a * p.ldy + (size_t)tile * 16 + r;
        if (p.epilogue == QENG_EPI_ACCUM) v += p.y[o];
        else if (p.epilogue == QENG_EPI_RESID) v += p.resid[o];
        p.y[o] = v;
      }
    }
    // the next tile's staging/reduction reuse is protected by the barrier at its start
    if (nslices == 1 && tile + (int)gridDim.x < p.ntiles) __syncthreads();
  }
}

template <int NT, int U>
int32_t launch(qeng_ctx* ctx, const GemvParams& p, int grid, size_t smem, cudaStream_t stream) {
  static bool configured_on[64] = {};  // the opt-in shared-memory size is set per device
  bool& configured = configured_on[ctx->device & 63];
  if (!configured) {
    QENG_CUDA(ctx, cudaFuncSetAttribute(gemv_q4_kernel<NT, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = true;
  }
  gemv_q4_kernel<NT, U><<<grid, kThreads, smem, stream>>>(p);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

}  // namespace

int32_t qeng_gemm_q4_decode(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M,
                            int64_t ldx, float* y, int64_t ldy, bool split_f32, const qeng_gemm_fuse& fuse,
                            cudaStream_t stream) {
  {
    bool handled = false;
    int32_t rc = qeng_gemm_q4_stream(ctx, w, x, x_dtype, M, ldx, y, ldy, fuse, stream, &handled);
    if (handled || rc != QENG_OK) return rc;
  }
  if (w->fmt != QENG_FMT_Q4)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4: this shape (M=%lld, N=%lld, K=%lld) is outside what the streaming kernel takes for this block format",
                     (long long)M, (long long)w->N, (long long)w->K);
  const int split = (x_dtype == QENG_F32 && split_f32) ? 1 : 0;
  const int max_m = split ? 16 : 32;
  if (M < 1 || M > max_m) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4_decode: M=%lld outside 1..%d", (long long)M, max_m);
  GemvParams p;
  p.qs = w->qs; p.sc = w->sc;
  p.ntiles = (int)w->ntiles; p.nchunks = (int)w->nchunks; p.K = (int)w->K;
  p.x = x; p.x_dtype = x_dtype; p.ldx = ldx; p.M = (int)M;
  p.cols = split ? 2 * (int)M : (int)M; p.split = split;
  p.y = y; p.ldy = ldy;
  p.gamma = fuse.norm_gamma; p.eps = fuse.norm_eps;
  p.epilogue = fuse.epilogue; p.resid = fuse.resid;
  const int NT = p.cols <= 8 ? 1 : (p.cols <= 16 ? 2 : 4);
  // shared memory: staged activations + block sums + reduction buffer + 1/rms
  const size_t fixed = (size_t)kWarps * 16 * 8 * NT * 4 + 64 * 4;
  const size_t budget = 96 * 1024;
  auto need = [&](int sc) { return (size_t)p.cols * (sc * 64 + 32) * 2 + (size_t)sc * 2 * 8 * NT * 4 + fixed; };
  int sc = p.nchunks;
  if (need(sc) > budget) {
    sc = (int)((budget - fixed) / ((size_t)p.cols * 128 + 2 * 8 * NT * 4));
    sc = sc / kWarps * kWarps;
    if (sc < kWarps) sc = kWarps;
  }
  p.slice_chunks = sc;
  const size_t smem = need(sc);
  const int grid = p.ntiles;
  switch (NT) {
    case 1: return launch<1, 8>(ctx, p, grid, smem, stream);
    case 2: return launch<2, 4>(ctx, p, grid, smem, stream);
    default: return launch<4, 4>(ctx, p, grid, smem, stream);
  }
}

extern "C" {

int32_t qeng_gemm_q4(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M, int64_t ldx,
                     float* y, int64_t ldy, int32_t flags, void* stream) {
  if (!ctx || !w || !x || !y) return qeng_fail(ctx, QENG_ERR_ARG, "gemm_q4: null argument");
  if (x_dtype < QENG_F32 || x_dtype > QENG_BF16) return qeng_fail(ctx, QENG_ERR_ARG, "gemm_q4: bad x_dtype %d", x_dtype);
  if (M < 1) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4: M=%lld", (long long)M);
  if (ldx < w->K || ldy < w->N) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4: leading dimension smaller than the row");
  QENG_ENTER(ctx);
  if (M >= kPrefillRows && w->fmt == QENG_FMT_Q4)  // dense contraction: dequantise to bf16 in shared memory, tcgen05 MMA
    return qeng_gemm_q4_prefill(ctx, w, x, x_dtype, M, ldx, y, ldy, (flags & QENG_GEMM_ACCUMULATE) ? 1 : 0, (cudaStream_t)stream);
  qeng_gemm_fuse fuse;
  fuse.epilogue = (flags & QENG_GEMM_ACCUMULATE) ? QENG_EPI_ACCUM : QENG_EPI_STORE;
  fuse.two_limbs = (flags & QENG_GEMM_FAST_F16) != 0;
  const bool split = x_dtype == QENG_F32 && !(flags & QENG_GEMM_FAST_F16);
  const int64_t step = w->fmt == QENG_FMT_K4 ? 4 : 16;  // rows per pass over the weights
  const size_t esz = x_dtype == QENG_F32 ? 4 : 2;
  for (int64_t m0 = 0; m0 < M; m0 += step) {
    int64_t mm = M - m0 < step ? M - m0 : step;
    int32_t rc = qeng_gemm_q4_decode(ctx, w, reinterpret_cast<const char*>(x) + (size_t)m0 * ldx * esz, x_dtype, mm,
                                     ldx, y + m0 * ldy, ldy, split, fuse, (cudaStream_t)stream);
    if (rc != QENG_OK) return rc;
  }
  return QENG_OK;
}

int32_t qeng_gemv_q4(qeng_ctx* ctx, const qeng_weight* w, const float* x, float* y, void* stream) {
  if (!w) return qeng_fail(ctx, QENG_ERR_ARG, "gemv_q4: null weight");
  return qeng_gemm_q4(ctx, w, x, QENG_F32, 1, w->K, y, w->N, 0, stream);
}

}  // extern "C"
