// Prefill-side quantized matmul on the 5th-generation tensor cores:
//   y[M,N] (f32) = x[M,K] (bf16) . bf16(dequant(W))[N,K]^T, f32 accumulation in TMEM.
//
// One CTA computes a 256 x 128 or 256 x 256 output tile (128 rows when M is small).  Per 64-wide K stage:
//   * loader warps copy the 256 x 64 bf16 activation tile into shared memory with 16-byte
//     cp.async, placing every chunk where the 128-byte swizzled K-major layout wants it;
//   * dequant warps read the packed 4-bit tile (8 row tiles x one chunk: 4.6 KB), turn each
//     code into bf16((c-8)*s) and store the 128 x 64 tile in the same swizzled layout;
//   * one thread issues tcgen05.mma (M=128, N=128 or 256, K=16; two accumulators share the
//     weight tile, so the dequantisation is amortised over 256 rows); tcgen05.commit hands the stage
//     back to the producers.
// The epilogue reads the accumulators with tcgen05.ld and stores f32 rows.
// Tensor-bound: 2*M*N*K flop; packed weights are re-read M/256 times from L2, activations
// N/128 times.
//
// Every wait is bounded; on expiry the kernel records status 4, stops waiting and still frees
// its tensor memory before it returns.
#include <cuda_bf16.h>

#include "qeng_internal.h"

namespace {

constexpr int kBM = 256, kBK = 64;
constexpr int kATile = kBM * kBK * 2;  // 32 KB
constexpr int kLoaders = 128;
// Two tile widths: BN = 128 (4 stages of 48 KB, 256 TMEM columns) and BN = 256 (3 stages of 64 KB,
// all 512 TMEM columns), which halves the L2 reads of the activation tile per flop.
template <int BN> struct TcCfg {
  static constexpr int kBTile = BN * kBK * 2;
  static constexpr int kStage = kATile + kBTile;
  static constexpr int kStages = BN == 128 ? 4 : 3;
  static constexpr int kDequant = BN;                        // one thread per two packed lanes
  static constexpr int kThreads = 32 + kLoaders + kDequant;  // warp 0 issues MMAs
  static constexpr int kTmemCols = 2 * BN;                   // two 128 x BN f32 accumulators
};

struct TcParams {
  const uint4* qs;
  const uint2* sc;
  int nchunks, ntiles;  // packed layout: K chunks of 64, row tiles of 16
  const __nv_bfloat16* x;  // [M][ldx]
  long long ldx;
  int M, N, K;
  float* y;
  long long ldy;
  int accumulate;
  int accs;  // accumulators per CTA: the output tile is (128 * accs) x 128
  int32_t* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up (false) two seconds after the first failed attempt; a healthy wait ends
// in microseconds.  The clock is read once per 64 attempts.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t0));
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t1;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t1));
    if (t1 - t0 > 2000000000ull) return false;
  }
}

// 64-bit shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffff) >> 4);  // start address
  d |= (uint64_t)1 << 16;                   // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;         // stride byte offset
  d |= (uint64_t)1 << 46;                   // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                   // 128-byte swizzle
  return d;
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}

__device__ __forceinline__ uint32_t bf16x2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int kBN>
__global__ void __launch_bounds__(TcCfg<kBN>::kThreads, 1) gemm_q4_tc_kernel(const TcParams p) {
  constexpr int kStages = TcCfg<kBN>::kStages, kStage = TcCfg<kBN>::kStage, kDequant = TcCfg<kBN>::kDequant;
  constexpr int kTmemCols = TcCfg<kBN>::kTmemCols;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the swizzle pattern is a function of the address: the tiles must start on 1024-byte boundaries
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t bars[3 * 4 + 1];
  __shared__ uint32_t tmem_slot;
  uint64_t* full_a = bars;
  uint64_t* full_b = bars + kStages;
  uint64_t* empty = bars + 2 * kStages;
  uint64_t* acc_full = bars + 3 * kStages;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bm = 128 * p.accs;
  const int m_tiles = (p.M + bm - 1) / bm;
  const int mt = blockIdx.x % m_tiles, nt = blockIdx.x / m_tiles;  // M walks fastest: the weight tile stays in L2
  const int m0 = mt * bm, n0 = nt * kBN;
  const int nk = p.nchunks;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(full_a + s), kLoaders);
      mbar_init(smem_u32(full_b + s), kDequant);
      mbar_init(smem_u32(empty + s), 1);
    }
    mbar_init(smem_u32(acc_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 0) {  // tensor memory for the two accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_slot)), "n"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ===== MMA issuer =====================================================================
    if (lane == 0) {
      // instruction descriptor: f32 accumulate, bf16 x bf16, both K-major, N = 128, M = 128
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      bool failed = false;
      int s = 0;
      uint32_t ph = 0;
      for (int kt = 0; kt < nk; ++kt) {
        if (!failed && !(mbar_wait(smem_u32(full_a + s), ph) && mbar_wait(smem_u32(full_b + s), ph))) failed = true;
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t a_addr = smem_u32(smem + (size_t)s * kStage);
        const uint32_t b_addr = a_addr + kATile;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k) {
          const uint64_t bdesc = make_desc(b_addr + k * 32);
          const uint32_t acc = (kt > 0 || k > 0) ? 1u : 0u;
          umma_bf16(tmem_base, make_desc(a_addr + k * 32), bdesc, idesc, acc);
          if (p.accs > 1) umma_bf16(tmem_base + kBN, make_desc(a_addr + 128 * 128 + k * 32), bdesc, idesc, acc);
        }
        umma_commit(smem_u32(empty + s));  // the stage is free once these MMAs have read it
        if (++s == kStages) { s = 0; ph ^= 1u; }
      }
      umma_commit(smem_u32(acc_full));
      if (failed) atomicExch(p.status, 4);
    }
  } else if (warp <= kLoaders / 32) {
    // ===== activation loaders: 256 x 64 bf16 per stage, 16 chunks of 16 bytes per thread ========
    const int lt = tid - 32;
    bool failed = false;
    int s = 0;
    uint32_t ph = 0;
    for (int kt = 0; kt < nk + kStages - 1; ++kt) {
      if (kt < nk) {
        if (!failed && !mbar_wait(smem_u32(empty + s), ph ^ 1u)) failed = true;
        const uint32_t a_addr = smem_u32(smem + (size_t)s * kStage);
        const int k0 = kt * kBK;
#pragma unroll
        for (int i = 0; i < (kBM * 8) / kLoaders; ++i) {
          if (i * kLoaders >= bm * 8) break;  // a 128-row tile fills half of the stage
          const int c = lt + i * kLoaders;  // chunk id: row = c / 8, 16-byte chunk j = c % 8
          const int r = c >> 3, j = c & 7;
          const int gm = m0 + r, gk = k0 + j * 8;
          const bool ok = gm < p.M && gk < p.K;
          const __nv_bfloat16* src = p.x + (ok ? (size_t)gm * p.ldx + gk : 0);
          const uint32_t dst = a_addr + r * 128 + ((j ^ (r & 7)) << 4);
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0) : "memory");
        }
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
      // the stage issued kStages-1 iterations ago has landed: make it visible to the tensor core
      if (kt >= kStages - 1) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(kStages - 1) : "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        const int sd = (kt - (kStages - 1)) % kStages;
        mbar_arrive(smem_u32(full_a + sd));
      }
      if (kt < nk && ++s == kStages) { s = 0; ph ^= 1u; }
    }
    if (failed && lt == 0) atomicExch(p.status, 4);
  } else {
    // ===== dequant: 128 rows x 64 k per stage; thread = (row tile, lane of the packed layout) ====
    const int dt = tid - 32 - kLoaders;  // 0..kDequant-1
    bool failed = false;
    int s = 0;
    uint32_t ph = 0;
    // a thread handles packed lanes dt and dt+kDequant of the 2*kBN (kBN/16 row tiles x 32 lanes)
    uint4 wn[2];
    uint2 scn[2];
    auto fetch = [&](int kt) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int pl = dt + h * kDequant, tl = pl >> 5, ln = pl & 31;
        const int tile = (n0 >> 4) + tl;
        wn[h] = make_uint4(0u, 0u, 0u, 0u);
        scn[h] = make_uint2(0u, 0u);
        if (tile < p.ntiles && kt < nk) {
          wn[h] = __ldg(p.qs + ((size_t)tile * p.nchunks + kt) * 32 + ln);
          scn[h] = __ldg(p.sc + ((size_t)tile * p.nchunks + kt) * 8 + (ln >> 2));
        }
      }
    };
    fetch(0);
    for (int kt = 0; kt < nk; ++kt) {
      uint4 w[2] = {wn[0], wn[1]};
      uint2 sc2[2] = {scn[0], scn[1]};
      fetch(kt + 1);  // the next stage's packed words travel while this one is converted
      if (!failed && !mbar_wait(smem_u32(empty + s), ph ^ 1u)) failed = true;
      const uint32_t b_addr = smem_u32(smem + (size_t)s * kStage) + kATile;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int pl = dt + h * kDequant, tl = pl >> 5, ln = pl & 31, g = ln >> 2, t = ln & 3;
        const uint32_t words[4] = {w[h].x, w[h].y, w[h].z, w[h].w};
        const __half2 s01 = *reinterpret_cast<const __half2*>(&sc2[h].x);  // (row g, blk 0), (row g+8, blk 0)
        const __half2 s23 = *reinterpret_cast<const __half2*>(&sc2[h].y);  // (row g, blk 1), (row g+8, blk 1)
        const float sc[4] = {__low2float(s01), __high2float(s01), __low2float(s23), __high2float(s23)};
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // q = blk * 2 + (row g+8 ? 1 : 0)
          const int r = tl * 16 + g + (q & 1) * 8;  // row within the 128-row tile
          const int j = (q >> 1) * 4 + t;           // 16-byte chunk within the 128-byte row: k = 8j .. 8j+7
          const float scale = sc[q], off = -136.0f * scale;
          const uint32_t wv = words[q];
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // 0x4300 | c is the bf16 128 + c; shifted into an f32 it is exact
            const float f0 = __uint_as_float((0x4300u | ((wv >> (8 * e)) & 15u)) << 16);
            const float f1 = __uint_as_float((0x4300u | ((wv >> (8 * e + 4)) & 15u)) << 16);
            o[e] = bf16x2(fmaf(f0, scale, off), fmaf(f1, scale, off));
          }
          const uint32_t dst = b_addr + r * 128 + ((j ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(dst), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]) : "memory");
        }
      }
      asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
      mbar_arrive(smem_u32(full_b + s));
      if (++s == kStages) { s = 0; ph ^= 1u; }
    }
    if (failed && dt == 0) atomicExch(p.status, 4);
  }

  // ===== epilogue: warps 1..4 own the four 32-lane quadrants of tensor memory =================
  if (warp >= 1 && warp <= 4) {
    const bool ok = mbar_wait(smem_u32(acc_full), 0);
    if (!ok && lane == 0) atomicExch(p.status, 4);
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const int quad = warp & 3;  // a warp may touch lanes 32*(warp%4) .. +31
    if (ok) {
#pragma unroll 1
      for (int acc = 0; acc < p.accs; ++acc) {
        const int gm = m0 + acc * 128 + quad * 32 + lane;
#pragma unroll 1
        for (int c0 = 0; c0 < kBN; c0 += 32) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kBN + c0);
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
              "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
              "%28,%29,%30,%31}, [%32];\n"
              : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
              : "r"(taddr));
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (gm < p.M) {
            float* dst = p.y + (size_t)gm * p.ldy + n0 + c0;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (n0 + c0 + i < p.N) {
                float f = __uint_as_float(v[i]);
                if (p.accumulate) f += dst[i];
                dst[i] = f;
              }
            }
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "n"(kTmemCols));
  }
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ x, long long ldx, __nv_bfloat16* __restrict__ y, int M, int K) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < (long long)M * K) {
    const long long m = i / K, k = i - m * K;
    y[i] = __float2bfloat16_rn(x[m * ldx + k]);
  }
}

}  // namespace

// y[M,N] = x . bf16(dequant(W))^T for large M.  f32 / f16 activations are rounded to bf16 first
// (a scratch of M*K*2 bytes owned by the context; grown outside the steady state).
int32_t qeng_gemm_q4_prefill(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M, int64_t ldx,
                             float* y, int64_t ldy, int accumulate, cudaStream_t stream) {
  if (w && w->fmt != QENG_FMT_Q4) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4_prefill: 4-bit blocks only");
  if (x_dtype == QENG_F16) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4 (prefill): f16 activations are not supported, use f32 or bf16");
  const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
  long long ldb = ldx;
  if (x_dtype == QENG_F32) {
    const size_t need = (size_t)M * w->K * 2;
    if (need > ctx->xbf16_bytes) {
      QENG_CUDA(ctx, cudaSetDevice(ctx->device));
      QENG_CUDA(ctx, cudaDeviceSynchronize());
      if (ctx->xbf16) cudaFree(ctx->xbf16);
      ctx->xbf16 = nullptr;
      ctx->xbf16_bytes = 0;
      QENG_CUDA(ctx, cudaMalloc(&ctx->xbf16, need));
      ctx->xbf16_bytes = need;
    }
    const long long n = (long long)M * w->K;
    f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const float*>(x), ldx,
                                                                         reinterpret_cast<__nv_bfloat16*>(ctx->xbf16), (int)M, (int)w->K);
    QENG_LAUNCH_CHECK(ctx);
    xb = reinterpret_cast<const __nv_bfloat16*>(ctx->xbf16);
    ldb = w->K;
  }
  if ((reinterpret_cast<uintptr_t>(xb) & 15) != 0 || (ldb & 7) != 0)
    return qeng_fail(ctx, QENG_ERR_ALIGN, "gemm_q4 (prefill): activations must be 16-byte aligned with a leading dimension multiple of 8");
  TcParams p;
  p.qs = w->qs; p.sc = w->sc; p.nchunks = (int)w->nchunks; p.ntiles = (int)w->ntiles;
  p.x = xb; p.ldx = ldb; p.M = (int)M; p.N = (int)w->N; p.K = (int)w->K;
  p.y = y; p.ldy = ldy; p.accumulate = accumulate; p.status = ctx->status;
  // 256-wide tiles when they still give every SM at least two tiles, else 128-wide; 256-row tiles
  // amortise the dequantisation, 128-row tiles when those would leave SMs idle
  const int64_t mt256 = (M + kBM - 1) / kBM;
  const bool wide = mt256 * ((w->N + 255) / 256) >= 2 * (int64_t)ctx->sm_count;
  const int bn = wide ? 256 : 128;
  const int n_tiles = (int)((w->N + bn - 1) / bn);
  p.accs = mt256 * n_tiles >= ctx->sm_count ? 2 : 1;
  const int m_tiles = (int)((M + 128 * p.accs - 1) / (128 * p.accs));
  static bool configured_on[64] = {};  // the opt-in shared-memory size is set per device
  bool& configured = configured_on[ctx->device & 63];
  if (!configured) {
    QENG_CUDA(ctx, cudaFuncSetAttribute(gemm_q4_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        TcCfg<128>::kStages * TcCfg<128>::kStage + 1024));
    QENG_CUDA(ctx, cudaFuncSetAttribute(gemm_q4_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        TcCfg<256>::kStages * TcCfg<256>::kStage + 1024));
    configured = true;
  }
  if (wide)
    gemm_q4_tc_kernel<256><<<m_tiles * n_tiles, TcCfg<256>::kThreads, TcCfg<256>::kStages * TcCfg<256>::kStage + 1024, stream>>>(p);
  else
    gemm_q4_tc_kernel<128><<<m_tiles * n_tiles, TcCfg<128>::kThreads, TcCfg<128>::kStages * TcCfg<128>::kStage + 1024, stream>>>(p);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}
