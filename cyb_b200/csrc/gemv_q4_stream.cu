// Streaming decode GEMV/GEMM over 4-bit block weights: the bandwidth kernel.
//
// One persistent CTA per SM: a producer warp and 16 consumer warps around a
// ring of shared-memory stages.  The producer walks this CTA's row tiles
// (16 rows x K, contiguous in the packed layout) and copies them stage by
// stage (64 chunks: 32 KB of nibbles + 4 KB of scales) with bulk asynchronous
// copies (cp.async.bulk, completion counted on an mbarrier), so ~170 KB per SM
// are in flight without holding registers and independent of what the
// consumers are doing.  Consumers take the chunks of a stage round-robin, read
// them with conflict-free 128-bit shared loads, unpack in registers and
// contract on the tensor pipe (mma.sync.m16n8k16, weights = A, activations = B;
// arithmetic as in gemv_q4.cu).  At the end of a row tile the 16 partial
// accumulators meet in shared memory (one named barrier, double-buffered) and
// one warp applies the fused epilogue.
//
// HBM-bound: algorithmic bytes = N*K*0.5625 + activations + outputs.
#include <cstdlib>
#include "qeng_internal.h"

namespace {

constexpr int kSC = 64;                        // chunks (of 64 k) per stage
constexpr int kStageBytes = kSC * (512 + 64);  // nibbles then scales: 36864
constexpr int kCW = 16;                        // consumer warps
constexpr int kCT = kCW * 32;                  // consumer threads
constexpr int kThreadsS = kCT + 32;            // + producer warp
constexpr int kMaxStages = 12;
constexpr int kGroups = 3;                     // groups of 8 k one consumer thread stages: K <= 8 * kGroups * kCT

struct StreamParams {
  // the matrix multiplied next (may be null): its tiles are requested into L2 once this
  // CTA's own loads are all issued
  const uint4* pf_qs;
  const uint2* pf_sc;
  int pf_ntiles, pf_nchunks;
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
  int nstages;
  int32_t* status;
  qeng_qkv_epi qkv;
};

// d = a.b + c (m16n8k16, f16 operands, f32 accumulate)
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
// One attempt: the hardware may park the thread until the phase completes or the hinted time passes.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(1000u)
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
// 1-D bulk copy global -> shared, completion counted in bytes on the mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds64f(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];\n" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ void l2_prefetch(const void* gptr, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(gptr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kCT) : "memory"); }
// the warps of one tile group (named barriers 2, 3, ...)
template <int GW>
__device__ __forceinline__ void group_sync(int gi) { asm volatile("bar.sync %0, %1;\n" ::"r"(2 + gi), "n"(GW * 32) : "memory"); }

__device__ __forceinline__ float act_f32(const void* x, int dtype, long long i) {
  if (dtype == QENG_F32) return reinterpret_cast<const float*>(x)[i];
  if (dtype == QENG_F16) return __half2float(reinterpret_cast<const __half*>(x)[i]);
  return __uint_as_float((uint32_t)reinterpret_cast<const uint16_t*>(x)[i] << 16);
}

__device__ __forceinline__ uint32_t h2bits(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int NT, int kTG>
__global__ void __launch_bounds__(kThreadsS, 1) gemv_q4_stream_kernel(const StreamParams p) {
  constexpr int kGW = kCW / kTG;  // warps per tile group
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int Kp = p.nchunks * 64;
  const int CS = Kp + 32;  // halves per staged activation column (64-byte skew)
  const int nblk = p.nchunks * 2;
  const int NS = p.nstages;
  // carve: ring | barriers | activations | block sums | reduction buffers
  unsigned char* ring = smem;
  unsigned char* after_ring = smem + (size_t)NS * kStageBytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(after_ring);
  uint64_t* empty = full + kMaxStages;
  __half* xs_h = reinterpret_cast<__half*>(after_ring + 2 * kMaxStages * 8 + 64);
  float* xsum = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(xs_h) + (size_t)p.cols * CS * 2);
  float* red = xsum + (size_t)nblk * 8 * NT;  // [2][kCW][16 * 8 * NT]
  __shared__ float warp_part[4 * kCW], oscale[32];

  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");  // the next kernel may start its own weight stream
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(full + s), 1);
      mbar_init(smem_u32(empty + s), kGW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  const int stages_per_tile = (p.nchunks + kSC - 1) / kSC;

  if (warp == kCW) {
    // ===== producer: stream this CTA's row tiles through the ring ==================
    if (lane == 0) {
      bool failed = false;
      const int NSg = NS / kTG;  // ring slots per tile group; group g owns slots [g * NSg, (g + 1) * NSg)
      int tcount = 0;
      for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount) {
        const int grp = tcount % kTG;
        int use = (tcount / kTG) * stages_per_tile;  // stage uses of this group so far
        for (int st = 0; st < stages_per_tile; ++st, ++use) {
          const int s = grp * NSg + use % NSg;
          const uint32_t ph = (uint32_t)(use / NSg) & 1u;
          if (!failed && !mbar_wait(smem_u32(empty + s), ph ^ 1u)) failed = true;
          const int c0 = st * kSC;
          const int nc = min(kSC, p.nchunks - c0);
          const uint32_t bar = smem_u32(full + s);
          const uint32_t dst = smem_u32(ring + (size_t)s * kStageBytes);
          const size_t chunk = (size_t)tile * p.nchunks + c0;
          mbar_expect_tx(bar, (uint32_t)nc * 576u);
          bulk_g2s(dst, p.qs + chunk * 32, (uint32_t)nc * 512u, bar);
          bulk_g2s(dst + kSC * 512, p.sc + chunk * 8, (uint32_t)nc * 64u, bar);
        }
      }
      if (failed) atomicExch(p.status, 4);
    }
    __syncwarp();
    // Own loads are all in flight: ask L2 for this CTA's share of the next matrix, so that HBM
    // does not idle while the consumers drain the ring and the next kernel starts up.
    if (p.pf_qs != nullptr) {
      const uint32_t qb = (uint32_t)p.pf_nchunks * 512u, sb = (uint32_t)p.pf_nchunks * 64u;
      for (int tile = blockIdx.x + gridDim.x * lane; tile < p.pf_ntiles; tile += gridDim.x * 32) {
        const char* q = reinterpret_cast<const char*>(p.pf_qs) + (size_t)tile * qb;
        for (uint32_t o = 0; o < qb; o += 32768u) l2_prefetch(q + o, min(32768u, qb - o));
        l2_prefetch(reinterpret_cast<const char*>(p.pf_sc) + (size_t)tile * sb, sb);
      }
    }
    return;
  }

  // ===== consumers ====================================================================
  // The weights never change, so only the consumers wait for the kernel that produced the
  // activations (a no-op unless launched with programmatic stream serialization).
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  // ---- stage the activations as f16 (hi | lo columns), fused RMSNorm -----------------
  // Row m is scaled by a power of two 2^sh so that its largest magnitude lands in
  // [2^14, 2^15): the f16 split hi + lo then never touches the subnormal range for
  // values that matter, and the slots that meet a code pre-multiplied by 16 (see the
  // unpacking below) can hold x/16 exactly.  The epilogue multiplies by 2^-sh.
  // One thread owns up to kGroups groups of 8 consecutive k (loaded once, kept in
  // registers across the reduction); the 4 groups of a 32-block sit in one quad.
  const int ngroups = Kp / 8;
  const bool vec_ok = p.x_dtype == QENG_F32 && ((reinterpret_cast<uintptr_t>(p.x) | (uintptr_t)(p.ldx * 4)) & 15) == 0 &&
                      (p.gamma == nullptr || (reinterpret_cast<uintptr_t>(p.gamma) & 15) == 0) && (p.K & 7) == 0;
  // The raw values of row m + 1 are requested before row m is reduced and converted, so with
  // several activation rows only the first one waits for memory.
  auto load_row = [&](int m, float (&dst)[kGroups][8]) {
#pragma unroll
    for (int j = 0; j < kGroups; ++j) {
      const int k0 = (tid + j * kCT) * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) dst[j][i] = 0.f;
      if (k0 < p.K) {
        if (vec_ok) {
          const float4* xp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (long long)m * p.ldx + k0);
          const float4 a = xp[0], b = xp[1];
          dst[j][0] = a.x; dst[j][1] = a.y; dst[j][2] = a.z; dst[j][3] = a.w;
          dst[j][4] = b.x; dst[j][5] = b.y; dst[j][6] = b.z; dst[j][7] = b.w;
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (k0 + i < p.K) dst[j][i] = act_f32(p.x, p.x_dtype, (long long)m * p.ldx + k0 + i);
        }
      }
    }
  };
  float nv[kGroups][8];
  load_row(0, nv);
  for (int m = 0; m < p.M; ++m) {
    float v[kGroups][8];
#pragma unroll
    for (int j = 0; j < kGroups; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) v[j][i] = nv[j][i];
    if (m + 1 < p.M) load_row(m + 1, nv);
    float ss = 0.f, amax = 0.f;
#pragma unroll
    for (int j = 0; j < kGroups; ++j) {
      const int k0 = (tid + j * kCT) * 8;
      if (k0 < p.K) {
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[j][i], v[j][i], ss);
        if (p.gamma != nullptr) {
          if (vec_ok) {
            const float4* gp = reinterpret_cast<const float4*>(p.gamma + k0);
            const float4 a = gp[0], b = gp[1];
            v[j][0] *= a.x; v[j][1] *= a.y; v[j][2] *= a.z; v[j][3] *= a.w;
            v[j][4] *= b.x; v[j][5] *= b.y; v[j][6] *= b.z; v[j][7] *= b.w;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (k0 + i < p.K) v[j][i] *= p.gamma[k0 + i];
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    }
    float* wp = warp_part + (m & 1) * (2 * kCW);  // double-buffered: one barrier per row
    if (lane == 0) {
      wp[warp] = ss;
      wp[kCW + warp] = amax;
    }
    consumer_sync();
    float tot = 0.f, mx = 0.f;
#pragma unroll
    for (int w = 0; w < kCW; ++w) {
      tot += wp[w];
      mx = fmaxf(mx, wp[kCW + w]);
    }
    float rs = 1.f;
    if (p.gamma != nullptr) {
      rs = rsqrtf(tot / (float)p.K + p.eps);
      mx *= rs;
    }
    int sh = 0;
    if (mx > 0.f && mx < 3.0e38f) sh = 14 - (((int)(__float_as_uint(mx) >> 23) & 0xff) - 127);
    sh = max(-100, min(100, sh));
    const float mul = rs * __uint_as_float((uint32_t)(sh + 127) << 23);
    if (tid == 0) oscale[m] = __uint_as_float((uint32_t)(127 - sh) << 23);
    const int colh = p.split ? 2 * m : m;
#pragma unroll
    for (int j = 0; j < kGroups; ++j) {
      const int grp = tid + j * kCT;
      // whole warps take part (the block sums use shuffles); ngroups is a multiple of 8, so a quad
      // is either entirely valid or entirely past the end
      if ((grp & ~31) < ngroups) {
        const bool valid = grp < ngroups;
        const int k0 = grp * 8;
        float a[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float t0 = v[j][i] * mul;
          a[i] = (i & 1) ? t0 * 0.0625f : t0;  // odd k of the group meet codes pre-multiplied by 16
        }
        // order 0,4,1,5,2,6,3,7: one 128-bit shared load yields the B registers of both MMAs of a block
        uint4 hi;
        hi.x = h2bits(a[0], a[4]); hi.y = h2bits(a[1], a[5]); hi.z = h2bits(a[2], a[6]); hi.w = h2bits(a[3], a[7]);
        const __half2* hh = reinterpret_cast<const __half2*>(&hi);
        const float2 a0 = __half22float2(hh[0]), a1 = __half22float2(hh[1]), a2 = __half22float2(hh[2]),
                     a3 = __half22float2(hh[3]);
        // block sums carry the zero point: -8 * 2^-24 * sum of the values the MMA effectively sees
        float hsum = ((a0.x + a0.y) + (a2.x + a2.y)) + 16.f * ((a1.x + a1.y) + (a3.x + a3.y));
        float lsum = 0.f;
        if (valid) *reinterpret_cast<uint4*>(xs_h + (size_t)colh * CS + k0) = hi;
        if (p.split) {
          uint4 lo;
          lo.x = h2bits(a[0] - a0.x, a[4] - a0.y); lo.y = h2bits(a[1] - a1.x, a[5] - a1.y);
          lo.z = h2bits(a[2] - a2.x, a[6] - a2.y); lo.w = h2bits(a[3] - a3.x, a[7] - a3.y);
          const __half2* ll = reinterpret_cast<const __half2*>(&lo);
          const float2 b0 = __half22float2(ll[0]), b1 = __half22float2(ll[1]), b2 = __half22float2(ll[2]),
                       b3 = __half22float2(ll[3]);
          lsum = ((b0.x + b0.y) + (b2.x + b2.y)) + 16.f * ((b1.x + b1.y) + (b3.x + b3.y));
          if (valid) *reinterpret_cast<uint4*>(xs_h + (size_t)(colh + 1) * CS + k0) = lo;
        }
        hsum += __shfl_xor_sync(0xffffffffu, hsum, 1);
        hsum += __shfl_xor_sync(0xffffffffu, hsum, 2);
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
        lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
        if (valid && (lane & 3) == 0) {
          const int blk = grp >> 2;
          xsum[blk * (8 * NT) + colh] = hsum * (-8.0f * 5.9604644775390625e-08f);
          if (p.split) xsum[blk * (8 * NT) + colh + 1] = lsum * (-8.0f * 5.9604644775390625e-08f);
        }
      }
    }
  }
  consumer_sync();

  // ---- main loop over this CTA's row tiles -------------------------------------------
  // The consumer warps form kTG independent groups that take the CTA's tiles in turn: while one
  // group reduces a tile and waits for its next stage, the other keeps the pipes busy.
  const int gi = warp / kGW, wi = warp % kGW;
  // Lanes whose B column lies beyond the activations read an existing column instead:
  // every load stays in bounds and unpredicated, and their output columns are ignored.
  // All addresses are 32-bit shared-space byte addresses advanced by compile-time strides.
  uint32_t xcol[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
    xcol[nt] = smem_u32(xs_h) + (uint32_t)((min(nt * 8 + g, p.cols - 1) * CS + t * 8) * 2) + (uint32_t)wi * 128u;
  const uint32_t zcol = smem_u32(xsum) + (uint32_t)t * 8u + (uint32_t)wi * (2u * 32u * NT);
  const uint32_t ring_w = smem_u32(ring) + (uint32_t)wi * 512u + (uint32_t)lane * 16u;
  const uint32_t ring_s = smem_u32(ring) + kSC * 512u + (uint32_t)wi * 64u + (uint32_t)g * 8u;
  const int red_stride = 16 * 8 * NT;  // floats per warp per buffer
  bool failed = false;
  // Each group owns NS / kTG consecutive ring slots and is the only waiter on their barriers, so a
  // barrier's phases are seen strictly in order however far the groups drift apart.
  const int NSg = NS / kTG, s_first = gi * NSg, s_end = s_first + NSg;
  int s = s_first, buf = 0, tcount = 0;
  uint32_t ph = 0;
  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount) {
    if ((tcount % kTG) != gi) continue;  // another group's tile
    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    uint32_t xo = 0, zo = 0;  // byte offsets of the current stage along k
    for (int st = 0; st < stages_per_tile; ++st) {
      if (!failed && !mbar_wait(smem_u32(full + s), ph)) failed = true;
      const int nc = min(kSC, p.nchunks - st * kSC);
      const uint32_t wb = ring_w + (uint32_t)s * kStageBytes;
      const uint32_t sb = ring_s + (uint32_t)s * kStageBytes;
#pragma unroll
      for (int rep = 0; rep < kSC / kGW; ++rep) {
        if (wi + rep * kGW < nc) {
          const uint4 w = lds128(wb + rep * (kGW * 512));
          const uint2 s2 = lds64(sb + rep * (kGW * 64));
#pragma unroll
          for (int b1 = 0; b1 < 2; ++b1) {
            // A fragments: a 4-bit code c in the low mantissa bits of an f16 is the subnormal
            // c*2^-24; one nibble higher it is 16c*2^-24 (its activation slot holds x/16).
            const uint32_t w0 = b1 ? w.z : w.x, w1 = b1 ? w.w : w.y;
            const uint32_t v0 = w0 >> 8, v1 = w1 >> 8;
            const uint32_t mlo = 0x000f000fu, mhi = 0x00f000f0u;
            const uint32_t sbits = b1 ? s2.y : s2.x;
            const float2 sf = __half22float2(*reinterpret_cast<const __half2*>(&sbits));
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const uint4 xb = lds128(xcol[nt] + xo + (rep * kGW * 128 + b1 * 64));
              const float2 z = lds64f(zcol + zo + ((rep * kGW * 2 + b1) * 32 * NT + nt * 32));
              float d[4];
              mma16816(d, w0 & mlo, w1 & mlo, w0 & mhi, w1 & mhi, xb.x, xb.y, z.x, z.y, z.x, z.y);
              mma16816(d, v0 & mlo, v1 & mlo, v0 & mhi, v1 & mhi, xb.z, xb.w, d[0], d[1], d[2], d[3]);
              acc[nt][0] = fmaf(sf.x, d[0], acc[nt][0]);
              acc[nt][1] = fmaf(sf.x, d[1], acc[nt][1]);
              acc[nt][2] = fmaf(sf.y, d[2], acc[nt][2]);
              acc[nt][3] = fmaf(sf.y, d[3], acc[nt][3]);
            }
          }
        }
      }
      xo += kSC * 128;
      zo += kSC * 2 * 32 * NT;
      // this warp is done with the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(empty + s));
      if (++s == s_end) {
        s = s_first;
        ph ^= 1u;
      }
    }

    // ---- the 16 partial accumulators meet in shared memory --------------------------
    // red[buf][warp][act][row16]; the reader of buffer `buf` finishes before it arrives at
    // the next tile's barrier, and buffer `buf` is written again only after that barrier
    float* myred = red + (((size_t)gi * 2 + buf) * kGW + wi) * red_stride;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (p.split) {
        const int a = nt * 4 + t;
        myred[a * 16 + g] = acc[nt][0] + acc[nt][1];
        myred[a * 16 + g + 8] = acc[nt][2] + acc[nt][3];
      } else {
        const int a = nt * 8 + 2 * t;
        myred[a * 16 + g] = acc[nt][0];
        myred[(a + 1) * 16 + g] = acc[nt][1];
        myred[a * 16 + g + 8] = acc[nt][2];
        myred[(a + 1) * 16 + g + 8] = acc[nt][3];
      }
    }
    group_sync<kGW>(gi);
    if (wi == ((tcount / kTG) % kGW)) {
      const float* rb = red + ((size_t)gi * 2 + buf) * kGW * red_stride;
      if (p.epilogue == QENG_EPI_QKV) {
        const qeng_qkv_epi& E = p.qkv;
        const int head = tile >> 3, i = ((tile & 7) << 3);
        for (int e = lane; e < p.M * 8; e += 32) {
          const int a = e >> 3, r = e & 7;
          float lo = 0.f, hi = 0.f;  // dims i+r and i+r+64 of this head
#pragma unroll
          for (int w = 0; w < kGW; ++w) {
            lo += rb[w * red_stride + a * 16 + r];
            hi += rb[w * red_stride + a * 16 + r + 8];
          }
          const float os = oscale[a];
          lo = lo * 16777216.0f * os;
          hi = hi * 16777216.0f * os;
          const int ps = E.pos[a];
          if (ps < 0 || ps >= E.max_seq || (ps >> 4) >= E.max_pages) {
            atomicExch(p.status, 2);
            continue;
          }
          const int d = i + r;
          if (head < E.Hq + E.Hkv) {
            const float c = E.cs[(size_t)ps * 128 + d], sn = E.cs[(size_t)ps * 128 + 64 + d];
            const float a0 = lo * c - hi * sn, a1 = hi * c + lo * sn;
            lo = a0;
            hi = a1;
          }
          if (head < E.Hq) {
            __half* dst = E.q16 + ((size_t)a * E.Hq + head) * 128 + d;
            dst[0] = __float2half_rn(lo);
            dst[64] = __float2half_rn(hi);
          } else {
            const int pid = E.table[(size_t)a * E.max_pages + (ps >> 4)];
            if ((unsigned)pid >= (unsigned)E.pages) {
              atomicExch(p.status, 1);
              continue;
            }
            const int kh = head - E.Hq;
            const int isv = kh >= E.Hkv ? 1 : 0;
            __half* dst = E.pool + (((size_t)pid * E.Hkv + (kh - isv * E.Hkv)) * 2 + isv) * (16 * 128) + (ps & 15) * 128 + d;
            dst[0] = __float2half_rn(lo);
            dst[64] = __float2half_rn(hi);
          }
        }
      } else if (p.epilogue == QENG_EPI_SWIGLU) {
        for (int e = lane; e < p.M * 8; e += 32) {
          const int a = e >> 3, r = e & 7;
          float gate = 0.f, up = 0.f;
#pragma unroll
          for (int w = 0; w < kGW; ++w) {
            gate += rb[w * red_stride + a * 16 + r];
            up += rb[w * red_stride + a * 16 + r + 8];
          }
          const float os = oscale[a];
          gate = gate * 16777216.0f * os;
          up = up * 16777216.0f * os;
          p.y[(size_t)a * p.ldy + (size_t)tile * 8 + r] = gate / (1.0f + __expf(-gate)) * up;
        }
      } else {
        for (int e = lane; e < p.M * 16; e += 32) {
          const int a = e >> 4, r = e & 15;
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kGW; ++w) v += rb[w * red_stride + a * 16 + r];
          v = v * 16777216.0f * oscale[a];
          const size_t o = (size_t)a * p.ldy + (size_t)tile * 16 + r;
          if (p.epilogue == QENG_EPI_ACCUM) v += p.y[o];
          else if (p.epilogue == QENG_EPI_RESID) v += p.resid[o];
          p.y[o] = v;
        }
      }
    }
    buf ^= 1;
  }
  if (failed && lane == 0) atomicExch(p.status, 4);
}

template <int NT, int kTG>
int32_t launch_stream(qeng_ctx* ctx, const StreamParams& p, size_t smem, cudaStream_t stream) {
  static bool configured_on[64] = {};  // the opt-in shared-memory size is set per device
  bool& configured = configured_on[ctx->device & 63];
  if (!configured) {
    QENG_CUDA(ctx, cudaFuncSetAttribute(gemv_q4_stream_kernel<NT, kTG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    configured = true;
  }
  const int grid = p.ntiles < ctx->sm_count ? p.ntiles : ctx->sm_count;
  // programmatic stream serialization: this kernel may become resident while its predecessor is still
  // running; everything that depends on the predecessor sits behind griddepcontrol.wait
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kThreadsS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  QENG_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_q4_stream_kernel<NT, kTG>, p));
  return QENG_OK;
}

}  // namespace

namespace {
struct StreamFit {
  bool ok;
  int split, cols, NT, nstages;
  size_t smem;
};
StreamFit stream_fit(const qeng_weight* w, int x_dtype, int64_t M, bool split_f32) {
  StreamFit f = {};
  f.split = (x_dtype == QENG_F32 && split_f32) ? 1 : 0;
  f.cols = f.split ? 2 * (int)M : (int)M;
  if (M < 1 || f.cols > 32) return f;
  if (w->nchunks * 64 > 8 * kGroups * kCT) return f;  // staged through registers: K <= 12288
  f.NT = f.cols <= 8 ? 1 : (f.cols <= 16 ? 2 : 4);
  const int64_t Kp = w->nchunks * 64;
  const size_t fixed = (size_t)2 * kMaxStages * 8 + 64                  // barriers
                       + (size_t)f.cols * (Kp + 32) * 2                 // staged activations
                       + (size_t)w->nchunks * 2 * 8 * f.NT * 4          // block sums
                       + (size_t)2 * kCW * 16 * 8 * f.NT * 4;           // reduction buffers
  const size_t budget = 226 * 1024 - 512;
  if (fixed + (size_t)2 * kStageBytes > budget) return f;
  f.nstages = (int)((budget - fixed) / kStageBytes);
  if (f.nstages > kMaxStages) f.nstages = kMaxStages;
  f.smem = (size_t)f.nstages * kStageBytes + fixed;
  f.ok = true;
  return f;
}
}  // namespace

bool qeng_gemm_q4_stream_fits(const qeng_weight* w, int64_t M, bool split) {
  return stream_fit(w, QENG_F32, M, split).ok;
}

// *handled = false when the shape does not fit this kernel (activations too large to keep
// resident in shared memory); the caller then uses the register-streaming kernel.
int32_t qeng_gemm_q4_stream(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M,
                            int64_t ldx, float* y, int64_t ldy, bool split_f32, const qeng_gemm_fuse& fuse,
                            cudaStream_t stream, bool* handled) {
  *handled = false;
  const StreamFit f = stream_fit(w, x_dtype, M, split_f32);
  if (!f.ok) {
    if (fuse.epilogue == QENG_EPI_QKV) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4: the fused q|k|v epilogue needs the streaming kernel");
    return QENG_OK;
  }
  StreamParams p;
  p.qs = w->qs; p.sc = w->sc;
  p.ntiles = (int)w->ntiles; p.nchunks = (int)w->nchunks; p.K = (int)w->K;
  p.x = x; p.x_dtype = x_dtype; p.ldx = ldx; p.M = (int)M; p.cols = f.cols; p.split = f.split;
  p.y = y; p.ldy = ldy;
  p.gamma = fuse.norm_gamma; p.eps = fuse.norm_eps; p.epilogue = fuse.epilogue; p.resid = fuse.resid;
  p.nstages = f.nstages; p.status = ctx->status;
  const qeng_weight* nx = ctx->l2_prefetch ? w->next : nullptr;
  p.pf_qs = nx ? nx->qs : nullptr; p.pf_sc = nx ? nx->sc : nullptr;
  p.pf_ntiles = nx ? (int)nx->ntiles : 0; p.pf_nchunks = nx ? (int)nx->nchunks : 0;
  p.qkv = qeng_qkv_epi();
  if (fuse.epilogue == QENG_EPI_QKV) {
    if (!fuse.qkv) return qeng_fail(ctx, QENG_ERR_ARG, "gemm_q4: fused q|k|v epilogue without its arguments");
    p.qkv = *fuse.qkv;
  }
  *handled = true;
  // Tile groups: more groups hide more of the per-tile reduction, but a group with no tile idles,
  // so the split follows the number of tiles a CTA owns.
  const int grid = p.ntiles < ctx->sm_count ? p.ntiles : ctx->sm_count;
  const int per_cta = (p.ntiles + grid - 1) / grid;
  int tg = per_cta >= 8 ? 4 : (per_cta >= 2 ? 2 : 1);
  // every group keeps at least two ring slots, and no fewer than one row tile needs (K > 4096: a tile
  // spans several stages, and a group whose ring is shorter than its tile stalls the producer)
  const int spt = (p.nchunks + kSC - 1) / kSC;
  while (tg > 1 && f.nstages / tg < (spt > 2 ? spt : 2)) tg >>= 1;
  if (ctx->stream_groups == 1 || ctx->stream_groups == 2 || ctx->stream_groups == 4) tg = ctx->stream_groups;
#define QENG_STREAM_CASE(NT_)                                                   \
  (tg == 4 ? launch_stream<NT_, 4>(ctx, p, f.smem, stream)                      \
           : (tg == 2 ? launch_stream<NT_, 2>(ctx, p, f.smem, stream) : launch_stream<NT_, 1>(ctx, p, f.smem, stream)))
  switch (f.NT) {
    case 1: return QENG_STREAM_CASE(1);
    case 2: return QENG_STREAM_CASE(2);
    default: return QENG_STREAM_CASE(4);
  }
#undef QENG_STREAM_CASE
}
