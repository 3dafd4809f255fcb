// The fused decode step: every layer of one greedy step in ONE persistent kernel.
//
// A decode step at batch 1 is ~100 MB of 4-bit weights per layer against a few kilobytes of
// activations.  Launched operator by operator, each matmul pays launch latency, activation
// staging, the fill of its copy ring and the drain of its last tile before the next can start:
// several microseconds per launch against 1.5 .. 8 us of streaming.  Here one cooperative
// grid (one CTA per SM) runs the whole chain
//     q|k|v -> attention -> o -> gate|up -> down        (x number of layers)
// and the producer warp of every CTA never stops: it walks the weights of all matrices in loop
// order through the CTA's ring of bulk-copy stages, running ahead of the consumers across the
// operator boundaries (the weights do not depend on anything), so HBM keeps streaming while the
// consumers synchronise, stage the next activations or work on the attention.
//
// Synchronisation between operators:
//   * o and down produce partial sums of the residual update.  Their epilogue stores (value, tag)
//     pairs -- one 8-byte store each, the tag is the step's sequence number -- into an inbox in
//     global memory; every CTA's next staging polls the inbox until the tags are current, adds
//     the parts in rank order onto the residual stream it keeps in registers, normalises and
//     quantises.  No barrier, no atomics, and with tensor parallelism the same stores go to every
//     peer's inbox over NVLink (plain peer stores): the all-reduce costs no launch of its own.
//   * attention -> o and gate|up -> down hand their rows over the same way (tagged pairs in an
//     attention box / activation box); q|k|v -> attention is the one grid barrier per layer (one
//     atomic arrival per CTA, bounded wait): the attention reads the KV pages other CTAs appended.
// Every wait is bounded (two seconds); on expiry the kernel records a status and runs on to its
// end without waiting again.
#include <math.h>
#include <string.h>

#include <vector>

#include "gemm_q4_s8.cuh"

namespace {
using namespace q4s8;

constexpr int kTG = 4;               // tile groups
constexpr int kGW = kCW / kTG;       // warps per group
constexpr int kStageChunks = 32;     // chunks per ring slot (18 KB)
constexpr uint32_t kSlotBytes = kStageChunks * 576u;
constexpr int kMaxB = 2;             // activation rows the step kernel takes
constexpr int kHD = 128;
constexpr int kMaxSplit = 4;         // attention splits per (sequence, kv head)
constexpr int kAttRow = 136;         // pairs per (sequence, head, split) row of the attention box (64-byte multiple)
constexpr int kAttnBytes = kCW * 4 * kHD * 4 + kCW * 4 * 2 * 4 + 4 * kHD * 4;  // merge buffers + q

struct StepMat {
  const uint4* qs;
  const uint2* sc;
  int ntiles, nchunks, K, pad;
};
struct StepLayer {
  StepMat m[4];  // q|k|v, o, gate|up, down
  const float* norm1;
  const float* norm2;
  __half* pool;
};

struct StepParams {
  const StepLayer* layers;
  int nlayers;
  int dm, F, Hq, Hkv, grp, max_pages, pages, max_seq;
  float eps, scale_log2;
  float* x;             // [B][dm] in: embedding of the token to feed; out: the last layer's output
  const int32_t *pos, *lens, *table;
  const float* cs;      // rotary table [max_seq][64 cos | 64 sin]
  __half* q16;          // [B][Hq][128]
  uint2* att_box;       // [B][Hq][kMaxSplit][kAttRow] tagged pairs: 128 unnormalised outputs, then (max, sum)
  uint2* act_box;       // [B][F] tagged pairs: the SwiGLU output
  uint2* inbox[8];      // per rank: [2 kinds][world][kMaxB][dm] (value, tag) pairs
  int world, rank;
  unsigned* sync;       // [0] steps completed (the tag base), [1] grid-barrier arrivals
  int32_t* status;
  int nstages;          // ring slots
  uint32_t zero_bytes;  // bytes of the zero region at the head of the staging area
  unsigned long long* trace;  // [2 CTAs (first, last)][layers][16] %globaltimer stamps of the phases
};

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kCT) : "memory"); }
__device__ __forceinline__ void group_sync(int gi) { asm volatile("bar.sync %0, %1;\n" ::"r"(2 + gi), "n"(kGW * 32) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// All consumer warps of all CTAs.  `target` = arrivals that complete this barrier.
__device__ __forceinline__ void grid_barrier(unsigned* cnt, unsigned target, int tid, Waits& w, int32_t* status) {
  consumer_sync();
  if (tid == 0) {
    __threadfence();
    atomicAdd(cnt, 1u);
    if (!w.failed) {
      const unsigned long long t0 = globaltimer();
      while ((int)(ld_acquire(cnt) - target) < 0) {
        if (globaltimer() - t0 > 2000000000ull) {
          atomicExch(status, 6);
          w.failed = true;  // this CTA waits for nobody any more
          break;
        }
      }
    }
    __threadfence();
  }
  consumer_sync();
}

enum { kEpiQkv = 0, kEpiPush = 1, kEpiSwiglu = 2 };
enum { kM1L3 = 0, kM1L2 = 1, kM2L2 = 2 };

template <int B>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const StepParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int NS = p.nstages;
  unsigned char* ring = smem;
  unsigned char* xreg = smem + (size_t)NS * kSlotBytes;  // kSlotBytes is a multiple of 128
  const uint32_t xbase = smem_u32(xreg);
  __shared__ float red[kTG * 2 * kGW * B * 16];
  __shared__ __align__(8) uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ float warp_part[2 * kCW];
  constexpr int red_stride = B * 16;

  const unsigned seq = *reinterpret_cast<volatile unsigned*>(p.sync);  // steps completed before this one
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(full + s), 1);
      mbar_init(smem_u32(empty + s), kGW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  if (warp == kCW) {
    // ===== producer: every matrix of every layer, in loop order, through one ring ==============
    if (lane == 0) {
      bool failed = false;
      unsigned q = 0;  // stage sequence number: slot q % NS, phase (q / NS) & 1
      for (int l = 0; l < p.nlayers; ++l) {
        for (int mt = 0; mt < 4; ++mt) {
          const StepMat M = p.layers[l].m[mt];
          for (int tile = blockIdx.x; tile < M.ntiles; tile += gridDim.x) {
            for (int c0 = 0; c0 < M.nchunks; c0 += kStageChunks, ++q) {
              const int s = (int)(q % (unsigned)NS);
              const uint32_t ph = (q / (unsigned)NS) & 1u;
              if (!failed && !mbar_wait(smem_u32(empty + s), ph ^ 1u)) failed = true;
              const int nc = min(kStageChunks, M.nchunks - c0);
              const uint32_t bar = smem_u32(full + s);
              const uint32_t dst = smem_u32(ring) + (uint32_t)s * kSlotBytes;
              const size_t chunk = (size_t)tile * M.nchunks + c0;
              mbar_expect_tx(bar, (uint32_t)nc * 576u);
              bulk_g2s(dst, M.qs + chunk * 32, (uint32_t)nc * 512u, bar);
              bulk_g2s(dst + kStageChunks * 512u, M.sc + chunk * 8, (uint32_t)nc * 64u, bar);
            }
          }
        }
      }
      if (failed) atomicExch(p.status, 4);
    }
    return;
  }

  // ===== consumers ======================================================================
  Waits W;
  const int gi = warp / kGW, wi = warp % kGW;
  const unsigned nbar_step = (unsigned)p.nlayers;  // one grid barrier per layer (q|k|v -> attention)
  unsigned bar_target = seq * nbar_step * gridDim.x;  // arrivals before this step's first barrier
  unsigned q = 0;        // stage sequence number, in step with the producer
  int tcount = 0;        // tiles of this CTA so far (all operators): tile -> group tcount % kTG
  int buf = 0;
  bool ring_failed = false;

  // zero region of the staging area (the lanes of other blocks' columns read it)
  for (uint32_t o = (uint32_t)tid * 16u; o < p.zero_bytes; o += kCT * 16u)
    asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(xbase + 64u + o), "r"(0u) : "memory");

  // the residual stream: this thread owns k = 8 tid .. 8 tid + 7 of every row
  const int k0 = tid * 8;
  const bool own = k0 < p.dm;
  float xres[B][8];
#pragma unroll
  for (int b = 0; b < B; ++b) {
#pragma unroll
    for (int i = 0; i < 8; ++i) xres[b][i] = 0.f;
    if (own) {
      const float4* xp = reinterpret_cast<const float4*>(p.x + (size_t)b * p.dm + k0);
      const float4 a = xp[0], c = xp[1];
      xres[b][0] = a.x; xres[b][1] = a.y; xres[b][2] = a.z; xres[b][3] = a.w;
      xres[b][4] = c.x; xres[b][5] = c.y; xres[b][6] = c.z; xres[b][7] = c.w;
    }
  }
  const size_t inbox_kind = (size_t)p.world * kMaxB * p.dm;  // pairs per kind
  const uint2* my_inbox = p.inbox[p.rank];

  // x += sum over ranks of the parts tagged `tag` in inbox kind `kind`
  auto gather = [&](int kind, unsigned tag) {
    if (!own) return;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      for (int r = 0; r < p.world; ++r) {
        float part[8];
        poll8(my_inbox + (size_t)kind * inbox_kind + ((size_t)r * kMaxB + b) * p.dm + k0, tag, part, W, p.status);
#pragma unroll
        for (int i = 0; i < 8; ++i) xres[b][i] += part[i];
      }
    }
  };
  // RMSNorm of the residual rows with gain `gamma`, quantised into the staging area
  // a norm's gains for this thread's 8 values: requested one operator ahead of their use, so that
  // the (cold) load is not on the critical path between two operators
  auto load_gains = [&](const float* gamma, float (&gm)[8]) {
    if (own) {
      const float4* gp = reinterpret_cast<const float4*>(gamma + k0);
      const float4 a = __ldg(gp), c = __ldg(gp + 1);
      gm[0] = a.x; gm[1] = a.y; gm[2] = a.z; gm[3] = a.w; gm[4] = c.x; gm[5] = c.y; gm[6] = c.z; gm[7] = c.w;
    }
  };
  auto prefetch_gains = [&](const float* gamma) {
    if (own && (tid & 3) == 0) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(gamma + k0));  // one 128-byte line per 4 threads
  };
  auto stage_norm = [&](const float (&gm)[8], int mode, const XLayout& L) {
#pragma unroll
    for (int b = 0; b < B; ++b) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(xres[b][i], xres[b][i], ss);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      float* wp = warp_part + (b & 1) * kCW;
      if (lane == 0) wp[warp] = ss;
      consumer_sync();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; ++w) tot += wp[w];
      const float rs = rsqrtf(tot / (float)p.dm + p.eps);
      if ((k0 >> 3 & ~31) < L.nblk * 4) {  // whole warps take part in the block reductions
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = own ? xres[b][i] * rs * gm[i] : 0.f;
        const bool valid = (k0 >> 3) < L.nblk * 4;
        if (mode == kM1L3)
          quantise_group<3>(v, valid, xbase + L.xq, L.col_stride, xbase + L.zin, xbase + L.fex, L.zs, (tid >> 2) * 32, tid & 3);
        else
          quantise_group<2>(v, valid, xbase + L.xq + (uint32_t)(2 * b) * L.col_stride, L.col_stride,
                            xbase + L.zin + (uint32_t)(2 * b) * L.zs, xbase + L.fex + (uint32_t)(2 * b) * L.zs, L.zs,
                            (tid >> 2) * 32, tid & 3);
      }
    }
    consumer_sync();
  };
  // rows of K values from global memory (`src`, leading dimension ld), quantised in two limbs
  auto stage_plain = [&](auto&& load8, int K, const XLayout& L) {
    const int ngroups = L.nblk * 4;
#pragma unroll
    for (int b = 0; b < B; ++b) {
      for (int grp0 = 0; grp0 < ngroups; grp0 += kCT) {
        const int grp = grp0 + tid;
        if ((grp & ~31) < ngroups) {
          float v[8];
          load8(b, grp * 8, grp < ngroups && grp * 8 < K, v);
          quantise_group<2>(v, grp < ngroups, xbase + L.xq + (uint32_t)(2 * b) * L.col_stride, L.col_stride,
                            xbase + L.zin + (uint32_t)(2 * b) * L.zs, xbase + L.fex + (uint32_t)(2 * b) * L.zs, L.zs,
                            (grp >> 2) * 32, grp & 3);
        }
      }
    }
    consumer_sync();
  };

  // this CTA's row tiles of one matrix: contraction, cross-warp reduction, epilogue
  auto run_tiles = [&](const StepMat& M, int mode, const XLayout& L, int epi, int l, unsigned tag, int kind) {
    const int spt = (M.nchunks + kStageChunks - 1) / kStageChunks;
    int tg_count = 0;  // tiles this group has finished in this operator (rotates the epilogue warp)
    for (int tile = blockIdx.x; tile < M.ntiles; tile += gridDim.x, ++tcount) {
      if ((tcount % kTG) != gi) {
        q += (unsigned)spt;  // another group's tile
        continue;
      }
      float acc[2] = {0.f, 0.f};
      for (int c0 = 0; c0 < M.nchunks; c0 += kStageChunks, ++q) {
        const int s = (int)(q % (unsigned)NS);
        const uint32_t ph = (q / (unsigned)NS) & 1u;
        if (!ring_failed && !mbar_wait(smem_u32(full + s), ph)) ring_failed = true;
        const int nc = min(kStageChunks, M.nchunks - c0);
        const uint32_t wb = smem_u32(ring) + (uint32_t)s * kSlotBytes;
        const uint32_t sb = wb + kStageChunks * 512u;
        if (mode == kM1L3) consume_m1l3<kGW>(acc, wb, sb, nc, c0 * 2, L, xbase, wi, lane);
        else if (mode == kM1L2) consume_g4<kGW>(acc, wb, sb, nc, c0 * 2, L, xbase, wi, lane);
        else consume_g2<kGW>(acc, wb, sb, nc, c0 * 2, L, xbase, wi, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + s));
      }
      float* myred = red + (((size_t)gi * 2 + buf) * kGW + wi) * red_stride;
      if (B == 1) {
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 1);
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 2);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 2);
        if (t == 0) { myred[g] = acc[0]; myred[g + 8] = acc[1]; }
      } else {
        acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], 1);
        acc[1] += __shfl_xor_sync(0xffffffffu, acc[1], 1);
        if ((t & 1) == 0) { myred[(t >> 1) * 16 + g] = acc[0]; myred[(t >> 1) * 16 + g + 8] = acc[1]; }
      }
      group_sync(gi);
      if (wi == (tg_count % kGW)) {
        const float* rb = red + ((size_t)gi * 2 + buf) * kGW * red_stride;
        auto total = [&](int a, int r) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kGW; ++w) v += rb[w * red_stride + a * 16 + r];
          return v;
        };
        if (epi == kEpiQkv) {
          // rotary embedding, f16 rounding, q to its buffer, k and v into the page pool (the rows of a
          // head are stored permuted so that rows r and r + 8 of a tile are the rotary pair)
          const int head = tile >> 3, i0 = ((tile & 7) << 3);
          for (int e = lane; e < B * 8; e += 32) {
            const int a = e >> 3, r = e & 7;
            float lo = total(a, r), hi = total(a, r + 8);
            const int ps = p.pos[a];
            if (ps < 0 || ps >= p.max_seq || (ps >> 4) >= p.max_pages) {
              atomicExch(p.status, 2);
              continue;
            }
            const int d = i0 + r;
            if (head < p.Hq + p.Hkv) {
              const float c = p.cs[(size_t)ps * 128 + d], sn = p.cs[(size_t)ps * 128 + 64 + d];
              const float a0 = lo * c - hi * sn, a1 = hi * c + lo * sn;
              lo = a0;
              hi = a1;
            }
            if (head < p.Hq) {
              __half* dst = p.q16 + ((size_t)a * p.Hq + head) * 128 + d;
              dst[0] = __float2half_rn(lo);
              dst[64] = __float2half_rn(hi);
            } else {
              const int pid = p.table[(size_t)a * p.max_pages + (ps >> 4)];
              if ((unsigned)pid >= (unsigned)p.pages) {
                atomicExch(p.status, 1);
                continue;
              }
              const int kh = head - p.Hq;
              const int isv = kh >= p.Hkv ? 1 : 0;
              __half* dst = p.layers[l].pool + (((size_t)pid * p.Hkv + (kh - isv * p.Hkv)) * 2 + isv) * (16 * 128) + (ps & 15) * 128 + d;
              dst[0] = __float2half_rn(lo);
              dst[64] = __float2half_rn(hi);
            }
          }
        } else if (epi == kEpiSwiglu) {
          for (int e = lane; e < B * 8; e += 32) {
            const int a = e >> 3, r = e & 7;
            const float gate = total(a, r), up = total(a, r + 8);
            st_pair(p.act_box + (size_t)a * p.F + (size_t)tile * 8 + r, gate / (1.0f + __expf(-gate)) * up, tag);
          }
        } else {
          // this rank's part of the residual update, tagged, into every rank's inbox
          for (int e = lane; e < B * 16; e += 32) {
            const int a = e >> 4, r = e & 15;
            const float v = total(a, r);
            const size_t o = (size_t)kind * inbox_kind + ((size_t)p.rank * kMaxB + a) * p.dm + (size_t)tile * 16 + r;
            for (int rr = 0; rr < p.world; ++rr) st_pair(p.inbox[(p.rank + rr) % p.world] + o, v, tag);
          }
        }
      }
      ++tg_count;
      buf ^= 1;
    }
  };

  // phase stamps of the first and the last CTA (one thread each), for qeng_decoder_step_profile
  const int trace_sel = blockIdx.x == 0 ? 0 : (blockIdx.x == gridDim.x - 1 ? 1 : -1);
  auto stamp = [&](int l, int i) {
    if (trace_sel >= 0 && tid == 0) p.trace[((size_t)trace_sel * p.nlayers + l) * 16 + i] = globaltimer();
  };
  for (int l = 0; l < p.nlayers; ++l) {
    const StepLayer& Ly = p.layers[l];
    stamp(l, 0);
    const unsigned tag_o = (seq * (unsigned)p.nlayers + (unsigned)l) * 2u + 1u, tag_d = tag_o + 1u;
    // ---- q|k|v ---------------------------------------------------------------------------------
    float gain1[8];
    load_gains(Ly.norm1, gain1);  // in flight while the parts are polled
    if (l > 0) gather(1, tag_d - 2u);
    {
      const int mode = B == 1 ? kM1L3 : kM2L2;
      const XLayout L = x_layout(B == 1 ? 3 : 4, Ly.m[0].nchunks, true, p.zero_bytes);
      stamp(l, 1);
      stage_norm(gain1, mode, L);
      stamp(l, 2);
      run_tiles(Ly.m[0], mode, L, kEpiQkv, l, 0u, 0);
    }
    stamp(l, 3);
    bar_target += gridDim.x;
    grid_barrier(p.sync + 1, bar_target, tid, W, p.status);
    stamp(l, 4);

    // ---- attention: CTA u < B * Hkv * kMaxSplit takes (sequence, kv head, split) ---------------
    {
      const int u = blockIdx.x;
      const int b = u / (p.Hkv * kMaxSplit), h = (u / kMaxSplit) % p.Hkv, s = u % kMaxSplit;
      if (b < B) {
        const int len = p.lens[b];
        const int npages = min((len + 15) >> 4, p.max_pages);
        const int S = max(1, min(kMaxSplit, (npages + kCW - 1) / kCW));
        if (s < S) {
          // staging area (behind the zero region): q as f32 [grp][128], then the warps' partials
          float* qsm = reinterpret_cast<float*>(xreg + 64 + ((p.zero_bytes + 127) & ~127u));
          float* sm_o = qsm + 4 * kHD;                     // [kCW][4][128]
          float* sm_ml = sm_o + kCW * 4 * kHD;             // [kCW][4][2]
          for (int i = tid; i < p.grp * kHD; i += kCT)
            qsm[i] = __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(p.q16) + ((size_t)b * p.Hq + (size_t)h * p.grp) * kHD + i)));
          consumer_sync();
          const int tk = lane >> 1, hf = lane & 1;
          float m_run[4], l_run[4], o[4][4];
#pragma unroll
          for (int hh = 0; hh < 4; ++hh) {
            m_run[hh] = -INFINITY;
            l_run[hh] = 0.f;
            o[hh][0] = o[hh][1] = o[hh][2] = o[hh][3] = 0.f;
          }
          const __half* pool = Ly.pool;
          for (int pg = s + S * warp; pg < npages; pg += S * kCW) {
            const int pid = p.table[(size_t)b * p.max_pages + pg];
            if ((unsigned)pid >= (unsigned)p.pages) {
              if (lane == 0) atomicExch(p.status, 1);
              continue;
            }
            const __half* kt = pool + ((size_t)pid * p.Hkv + h) * (2 * 16 * kHD);
            const __half* vt = kt + 16 * kHD;
            // scores of token tk: this lane's half of the 128 dims
            uint4 kq[8];
            const uint4* kp = reinterpret_cast<const uint4*>(kt + tk * kHD + hf * 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) kq[i] = __ldcg(kp + i);  // rows written by other CTAs in this launch: L2, not L1
            float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const __half2* h2 = reinterpret_cast<const __half2*>(&kq[i]);
              const float2 k01 = __half22float2(h2[0]), k23 = __half22float2(h2[1]), k45 = __half22float2(h2[2]),
                           k67 = __half22float2(h2[3]);
#pragma unroll
              for (int hh = 0; hh < 4; ++hh) {
                if (hh < p.grp) {
                  const float4 qa = *reinterpret_cast<const float4*>(qsm + hh * kHD + hf * 64 + i * 8);
                  const float4 qb = *reinterpret_cast<const float4*>(qsm + hh * kHD + hf * 64 + i * 8 + 4);
                  sc[hh] += k01.x * qa.x + k01.y * qa.y + k23.x * qa.z + k23.y * qa.w + k45.x * qb.x + k45.y * qb.y +
                            k67.x * qb.z + k67.y * qb.w;
                }
              }
            }
            const int tok = pg * 16 + tk;
            float pr[4];
#pragma unroll
            for (int hh = 0; hh < 4; ++hh) {
              float sv = sc[hh] + __shfl_xor_sync(0xffffffffu, sc[hh], 1);
              sv = tok < len ? sv * p.scale_log2 : -INFINITY;
              float tmax = sv;
#pragma unroll
              for (int off = 2; off < 32; off <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, off));
              const float m_new = fmaxf(m_run[hh], tmax);  // finite: token 0 of a listed page is valid
              const float alpha = exp2f(m_run[hh] - m_new);
              pr[hh] = exp2f(sv - m_new);
              l_run[hh] = l_run[hh] * alpha + (hf == 0 ? pr[hh] : 0.f);
              m_run[hh] = m_new;
              o[hh][0] *= alpha; o[hh][1] *= alpha; o[hh][2] *= alpha; o[hh][3] *= alpha;
            }
            // o += P V: this lane owns dims 4 lane .. 4 lane + 3
            uint2 vv[16];
            const uint2* vp = reinterpret_cast<const uint2*>(vt + lane * 4);
#pragma unroll
            for (int j = 0; j < 16; ++j) vv[j] = __ldcg(vp + j * (kHD / 4));
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const __half2* h2 = reinterpret_cast<const __half2*>(&vv[j]);
              float2 v01 = __half22float2(h2[0]), v23 = __half22float2(h2[1]);
              if (pg * 16 + j >= len) v01 = v23 = make_float2(0.f, 0.f);  // probability 0, but the row may hold anything
#pragma unroll
              for (int hh = 0; hh < 4; ++hh) {
                const float pj = __shfl_sync(0xffffffffu, pr[hh], 2 * j);
                o[hh][0] = fmaf(pj, v01.x, o[hh][0]);
                o[hh][1] = fmaf(pj, v01.y, o[hh][1]);
                o[hh][2] = fmaf(pj, v23.x, o[hh][2]);
                o[hh][3] = fmaf(pj, v23.y, o[hh][3]);
              }
            }
          }
#pragma unroll
          for (int hh = 0; hh < 4; ++hh) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], off);
            *reinterpret_cast<float4*>(sm_o + ((size_t)warp * 4 + hh) * kHD + lane * 4) = make_float4(o[hh][0], o[hh][1], o[hh][2], o[hh][3]);
            if (lane == 0) {
              sm_ml[(warp * 4 + hh) * 2] = m_run[hh];
              sm_ml[(warp * 4 + hh) * 2 + 1] = l_run[hh];
            }
          }
          consumer_sync();
          if (tid < p.grp * kHD) {
            const int hh = tid >> 7, d = tid & 127;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < kCW; ++w) M = fmaxf(M, sm_ml[(w * 4 + hh) * 2]);
            float Lsum = 0.f, O = 0.f;
#pragma unroll
            for (int w = 0; w < kCW; ++w) {
              const float mw = sm_ml[(w * 4 + hh) * 2];
              const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);  // a warp without pages
              Lsum = fmaf(sm_ml[(w * 4 + hh) * 2 + 1], f, Lsum);
              O = fmaf(sm_o[((size_t)w * 4 + hh) * kHD + d], f, O);
            }
            uint2* row = p.att_box + (((size_t)b * p.Hq + (size_t)h * p.grp + hh) * kMaxSplit + s) * kAttRow;
            st_pair(row + d, O, tag_o);
            if (d == 0) {
              st_pair(row + kHD, M, tag_o);
              st_pair(row + kHD + 1, Lsum, tag_o);
            }
          }
        }
      }
    }
    stamp(l, 5);
    stamp(l, 6);

    // ---- o: merge the attention splits while staging, parts of the residual update to the inbox --
    {
      const int mode = B == 1 ? kM1L2 : kM2L2;
      const int K = p.Hq * kHD;
      const XLayout L = x_layout(2 * B, B == 1 ? (Ly.m[1].nchunks + 1) & ~1 : Ly.m[1].nchunks, true, p.zero_bytes);
      stage_plain(
          [&](int b, int kk, bool valid, float(&v)[8]) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            if (!valid) return;
            const int len = p.lens[b];
            const int npages = min((len + 15) >> 4, p.max_pages);
            const int S = max(1, min(kMaxSplit, (npages + kCW - 1) / kCW));
            const int qh = kk >> 7, d = kk & 127;
            const uint2* row = p.att_box + ((size_t)b * p.Hq + qh) * kMaxSplit * kAttRow;
            float M = -INFINITY, Lsum = 0.f;
            for (int s = 0; s < S; ++s) {  // running merge: (max, sum, out) of the splits seen so far
              float os[8], ml[2];
              poll8(row + (size_t)s * kAttRow + d, tag_o, os, W, p.status);
              poll2(row + (size_t)s * kAttRow + kHD, tag_o, ml, W, p.status);
              const float Mn = fmaxf(M, ml[0]);
              const float fo = M == -INFINITY ? 0.f : exp2f(M - Mn), fn = ml[0] == -INFINITY ? 0.f : exp2f(ml[0] - Mn);
              Lsum = Lsum * fo + ml[1] * fn;
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = v[i] * fo + os[i] * fn;
              M = Mn;
            }
            const float inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] *= inv;
          },
          K, L);
      stamp(l, 7);
      prefetch_gains(Ly.norm2);
      run_tiles(Ly.m[1], mode, L, kEpiPush, l, tag_o, 0);
    }
    stamp(l, 8);
    // ---- gate|up: x += o's update, norm, SwiGLU in the epilogue ------------------------------------
    float gain2[8];
    load_gains(Ly.norm2, gain2);
    gather(0, tag_o);
    stamp(l, 9);
    {
      const int mode = B == 1 ? kM1L2 : kM2L2;
      const XLayout L = x_layout(2 * B, B == 1 ? (Ly.m[2].nchunks + 1) & ~1 : Ly.m[2].nchunks, true, p.zero_bytes);
      stage_norm(gain2, mode, L);
      stamp(l, 10);
      run_tiles(Ly.m[2], mode, L, kEpiSwiglu, l, tag_o, 0);
    }
    stamp(l, 11);
    stamp(l, 12);
    // ---- down ------------------------------------------------------------------------------------------
    {
      const int mode = B == 1 ? kM1L2 : kM2L2;
      const XLayout L = x_layout(2 * B, B == 1 ? (Ly.m[3].nchunks + 1) & ~1 : Ly.m[3].nchunks, true, p.zero_bytes);
      stage_plain(
          [&](int b, int kk, bool valid, float(&v)[8]) {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = 0.f;
            if (!valid) return;
            poll8(p.act_box + (size_t)b * p.F + kk, tag_o, v, W, p.status);
          },
          p.F, L);
      stamp(l, 13);
      if (l + 1 < p.nlayers) prefetch_gains(p.layers[l + 1].norm1);
      run_tiles(Ly.m[3], mode, L, kEpiPush, l, tag_d, 1);
    }
    stamp(l, 14);
  }
  // ---- the step's output: CTA 0 completes the residual stream and leaves it for the LM head ----
  if (blockIdx.x == 0) {
    const unsigned tag_last = (seq * (unsigned)p.nlayers + (unsigned)(p.nlayers - 1)) * 2u + 2u;
    gather(1, tag_last);
    if (own) {
#pragma unroll
      for (int b = 0; b < B; ++b) {
        float4* xp = reinterpret_cast<float4*>(p.x + (size_t)b * p.dm + k0);
        xp[0] = make_float4(xres[b][0], xres[b][1], xres[b][2], xres[b][3]);
        xp[1] = make_float4(xres[b][4], xres[b][5], xres[b][6], xres[b][7]);
      }
    }
    consumer_sync();
    if (tid == 0) {
      __threadfence();
      *reinterpret_cast<volatile unsigned*>(p.sync) = seq + 1u;
    }
  }
  if ((ring_failed) && lane == 0) atomicExch(p.status, 4);
}

}  // namespace

// ---- host side ----------------------------------------------------------------------------------
struct qeng_step {
  StepParams p;
  StepLayer* dev_layers = nullptr;
  uint2 *att_box = nullptr, *act_box = nullptr;
  unsigned* sync = nullptr;
  unsigned long long* trace = nullptr;
  uint2* own_inbox = nullptr;  // single-rank: the inbox is plain device memory owned here
  size_t smem = 0;
  int grid = 0;
};

size_t qeng_step_inbox_bytes(int world, int dm) { return (size_t)2 * world * kMaxB * dm * sizeof(uint2); }

void qeng_step_free(qeng_step* s) {
  if (!s) return;
  if (s->dev_layers) cudaFree(s->dev_layers);
  if (s->att_box) cudaFree(s->att_box);
  if (s->act_box) cudaFree(s->act_box);
  if (s->sync) cudaFree(s->sync);
  if (s->trace) cudaFree(s->trace);
  if (s->own_inbox) cudaFree(s->own_inbox);
  delete s;
}

// Plans the fused step for a decoder, or leaves *out null when the shapes are outside what the
// kernel takes (the caller then runs the operator-by-operator chain).
int32_t qeng_step_create(qeng_ctx* ctx, const qeng_step_desc& d, qeng_step** out) {
  *out = nullptr;
  if (!ctx->step_kernel) return QENG_OK;
  const int grp = d.Hq / d.Hkv;
  if (d.dm % 128 != 0 || d.dm > 8 * kCT || grp < 1 || grp > 4 || d.F % 8 != 0) return QENG_OK;
  if (kMaxB * d.Hkv * kMaxSplit > ctx->sm_count) return QENG_OK;
  if (d.world > 1 && !d.peer_inbox[0]) return QENG_OK;
  // staging area: zero region + the widest operand (down: K = F, or q|k|v in three limbs), or the attention buffers
  int max_chunks = 0;
  for (const auto& L : d.layers)
    for (int i = 0; i < 4; ++i) {
      if (!L.w[i]) return qeng_fail(ctx, QENG_ERR_STATE, "decode step: a layer matrix is missing");
      max_chunks = (int)L.w[i]->nchunks > max_chunks ? (int)L.w[i]->nchunks : max_chunks;
    }
  const int alloc = (max_chunks + 1) & ~1;
  const uint32_t zero_bytes = x_zero_bytes(x_layout(2, alloc, true));
  size_t xbytes = 0;
  for (int cols : {3, 4}) {
    const XLayout L = x_layout(cols, alloc, true, zero_bytes);
    xbytes = L.bytes > xbytes ? L.bytes : xbytes;
  }
  const size_t attn = 64 + ((zero_bytes + 127) & ~127u) + kAttnBytes + 256;
  if (attn > xbytes) xbytes = attn;
  xbytes = (xbytes + 127) & ~(size_t)127;
  const size_t budget = 226 * 1024 - 6 * 1024;  // static shared memory of the kernel comes on top
  if (xbytes + 4 * kSlotBytes > budget) return QENG_OK;
  int ns = (int)((budget - xbytes) / kSlotBytes);
  if (ns > kMaxStages) ns = kMaxStages;
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  qeng_step* s = new qeng_step();
  StepParams& p = s->p;
  memset(&p, 0, sizeof p);
  std::vector<StepLayer> hl(d.layers.size());
  for (size_t l = 0; l < d.layers.size(); ++l) {
    for (int i = 0; i < 4; ++i) {
      const qeng_weight* w = d.layers[l].w[i];
      hl[l].m[i] = StepMat{w->qs, w->sc, (int)w->ntiles, (int)w->nchunks, (int)w->K, 0};
    }
    hl[l].norm1 = d.layers[l].norm1;
    hl[l].norm2 = d.layers[l].norm2;
    hl[l].pool = d.layers[l].pool;
  }
  cudaError_t e = cudaMalloc(&s->dev_layers, hl.size() * sizeof(StepLayer));
  if (e == cudaSuccess) e = cudaMemcpy(s->dev_layers, hl.data(), hl.size() * sizeof(StepLayer), cudaMemcpyHostToDevice);
  const size_t att_bytes = (size_t)kMaxB * d.Hq * kMaxSplit * kAttRow * sizeof(uint2);
  const size_t act_bytes = (size_t)kMaxB * d.F * sizeof(uint2);
  if (e == cudaSuccess) e = cudaMalloc(&s->att_box, att_bytes);
  if (e == cudaSuccess) e = cudaMemset(s->att_box, 0, att_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&s->act_box, act_bytes);
  if (e == cudaSuccess) e = cudaMemset(s->act_box, 0, act_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&s->sync, 64);
  if (e == cudaSuccess) e = cudaMemset(s->sync, 0, 64);
  if (e == cudaSuccess) e = cudaMalloc(&s->trace, (size_t)2 * hl.size() * 16 * 8);
  if (e == cudaSuccess) e = cudaMemset(s->trace, 0, (size_t)2 * hl.size() * 16 * 8);
  if (e == cudaSuccess && d.world == 1) {
    e = cudaMalloc(&s->own_inbox, qeng_step_inbox_bytes(1, d.dm));
    if (e == cudaSuccess) e = cudaMemset(s->own_inbox, 0, qeng_step_inbox_bytes(1, d.dm));
  }
  if (e != cudaSuccess) {
    qeng_step_free(s);
    return qeng_fail(ctx, QENG_ERR_CUDA, "decode step: %s", cudaGetErrorString(e));
  }
  p.layers = s->dev_layers; p.nlayers = (int)d.layers.size();
  p.dm = d.dm; p.F = d.F; p.Hq = d.Hq; p.Hkv = d.Hkv; p.grp = grp; p.max_pages = d.max_pages; p.pages = d.pages; p.max_seq = d.max_seq;
  p.eps = d.eps; p.scale_log2 = 1.4426950408889634f / sqrtf((float)kHD);
  p.x = d.x; p.pos = d.pos; p.lens = d.lens; p.table = d.table; p.cs = d.cs; p.q16 = d.q16;
  p.att_box = s->att_box; p.act_box = s->act_box;
  p.world = d.world; p.rank = d.rank;
  for (int r = 0; r < 8; ++r) p.inbox[r] = d.world == 1 ? (r == 0 ? s->own_inbox : nullptr) : reinterpret_cast<uint2*>(d.peer_inbox[r]);
  p.sync = s->sync; p.status = ctx->status;
  p.nstages = ns; p.zero_bytes = zero_bytes; p.trace = s->trace;
  s->smem = (size_t)ns * kSlotBytes + xbytes;
  s->grid = ctx->sm_count;
  // opt-in dynamic shared memory: the kernel's static arrays come on top, so ask for what is used
  e = cudaFuncSetAttribute(decode_step_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s->smem);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(decode_step_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s->smem);
  if (e != cudaSuccess) {
    qeng_step_free(s);
    return qeng_fail(ctx, QENG_ERR_CUDA, "decode step: %s", cudaGetErrorString(e));
  }
  // all CTAs must be resident together (they wait for one another): check before the first launch
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<1>, kThreads, s->smem);
  if (e != cudaSuccess || per_sm < 1) {
    qeng_step_free(s);
    return QENG_OK;
  }
  *out = s;
  return QENG_OK;
}

bool qeng_step_takes(const qeng_step* s, int B) { return s != nullptr && B >= 1 && B <= kMaxB; }

// One decode step over all layers for B rows: reads and rewrites d.x.  Cooperative launch: the
// runtime refuses it if the grid could not be co-resident.
int32_t qeng_step_launch(qeng_ctx* ctx, qeng_step* s, int B, cudaStream_t stream) {
  void* args[] = {&s->p};
  cudaError_t e;
  if (B == 1) e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_step_kernel<1>), dim3(s->grid), dim3(kThreads), args, s->smem, stream);
  else e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_step_kernel<2>), dim3(s->grid), dim3(kThreads), args, s->smem, stream);
  if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "decode step launch: %s", cudaGetErrorString(e));
  return QENG_OK;
}

// Device timestamps (ns, %globaltimer) of the last fused step: [2 CTAs: first, last][layers][16 stamps].
int32_t qeng_step_profile(qeng_ctx* ctx, qeng_step* s, uint64_t* out, int32_t capacity, int32_t* n) {
  const int32_t total = 2 * s->p.nlayers * 16;
  *n = total < capacity ? total : capacity;
  QENG_CUDA(ctx, cudaDeviceSynchronize());
  QENG_CUDA(ctx, cudaMemcpy(out, s->trace, (size_t)*n * 8, cudaMemcpyDeviceToHost));
  return QENG_OK;
}
