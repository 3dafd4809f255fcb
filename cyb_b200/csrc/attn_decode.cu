// Decode attention (GQA) over a paged f16 KV cache, split over the KV length.
//
// Pool layout: f16 [page][kv head][K|V][16 tokens][128], so the K tile and the
// V tile of one (page, kv head) are 8 KB contiguous.  One CTA serves one
// (sequence, kv head, split).  A producer warp looks up the page ids and brings
// the CTA's page tiles into a ring of 8 KB shared-memory slots with bulk
// asynchronous copies (cp.async.bulk, completion counted on an mbarrier), so the
// bytes in flight per SM (two CTAs x 80 KB) do not depend on registers.  Four
// consumer warps take the slots round-robin, read the K and V tiles into MMA
// fragments with 128-bit shared loads (the contraction index of an MMA may be
// permuted freely as long as both operands agree, which lets every lane read
// contiguous 16-byte pieces), and keep an online softmax (max, sum, out) per
// query head of the group.  Warps are merged in shared memory.  Splits: the eight CTAs of a thread-block cluster take the pages of a
// sequence round-robin and merge through distributed shared memory (no scratch,
// no atomics); caches beyond 16K tokens fall back to fixed page ranges merged
// through a scratch buffer by the CTA that arrives last.
//
// HBM-bound: algorithmic bytes = sum_b len_b * kv_heads * 2 * 128 * 2.
#include <math.h>
#include <stdlib.h>

#include "qeng_internal.h"

namespace {

constexpr int kAW = 4;  // consumer warps per CTA (one more warp produces)
constexpr int kAT = (kAW + 1) * 32;  // threads per CTA
constexpr int kRing = 8;             // ring slots of one page tile (K and V of 16 tokens: 8 KB)
// A slot must always be consumed by the same warp (page i goes to warp i % kAW and slot i % kRing):
// a warp that consumed round r of a slot cannot then wait for round r + 2 before round r + 1 has
// landed, which a parity wait could not tell from round r + 2 being there.
static_assert(kRing % kAW == 0, "every ring slot belongs to one consumer warp");
constexpr int kSlotBytes = 2 * 16 * 128 * 2;
constexpr int kHD = 128;
constexpr int kCS = 8;  // largest cluster: CTAs (splits) per sequence and kv head; the launch picks 1, 2, 4 or 8

__device__ __forceinline__ uint32_t cluster_map(const void* smem_ptr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(smem_ptr)), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ float ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
// hardware barrier over all threads of the cluster (every thread of every CTA executes it)
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}

struct AttnParams {
  const __half* pool;
  const __half* q;
  const int32_t* table;
  const int32_t* lens;
  float* part_o;   // [B][Hq][S][128]
  float* part_ml;  // [B][Hq][S][2]
  float* out;      // [B][Hq][128]
  int32_t* status;
  int* counters;   // [B][Hkv] arrivals per (sequence, kv head); null = merge in a second kernel
  int pages, Hkv, Hq, grp, max_pages, pps, S;
  float scale_log2;
  float scale, softcap;  // softcap > 0: logits = softcap * tanh(q.k * scale / softcap) (Gemma family)
  int window;            // > 0: only the last `window` tokens of a sequence are attended (sliding window)
};

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
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(1000u)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up (false) two seconds after the first failed attempt.
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
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  return *reinterpret_cast<const uint4*>(__cvta_shared_to_generic((size_t)addr));
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_nc(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <bool kCl>
__device__ __forceinline__ void attn_decode_body(const AttnParams& p) {
  // the output projection that follows may start streaming its weights as CTAs of this kernel retire
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  extern __shared__ __align__(128) unsigned char ring[];  // kRing slots of one page tile (K then V)
  __shared__ __align__(8) uint64_t full[kRing], empty[kRing];
  __shared__ int slot_ok[kRing];
  const int s = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  // Without a window the first 32 page-table entries of this CTA do not depend on the sequence
  // length: the producer asks for them together with the length instead of after it (one memory
  // round trip less on the way to the first page).  Entries past the sequence are read (the table
  // row is max_pages long) and never used.
  int pid_spec = -1;
  if (warp == kAW && p.window == 0) {
    const int idx = kCl ? s + lane * p.S : s * p.pps + lane;
    if (idx < p.max_pages && (kCl || lane < p.pps)) pid_spec = p.table[(size_t)b * p.max_pages + idx];
  }
  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(smem_u32(full + i), 1);
      mbar_init(smem_u32(empty + i), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();
  // Pages of this CTA, in order: in a cluster the CTAs interleave the pages of the sequence (page =
  // first + cs * i), otherwise a CTA owns the pages [first, first + pps).  With a sliding window the
  // pages that lie entirely before the window are not visited at all.
  const int cs = p.S;  // cluster path: CTAs in the cluster (= gridDim.x)
  const int len = p.lens[b];
  const int npages = min((len + 15) >> 4, p.max_pages);
  const int win0 = p.window > 0 ? max(0, len - p.window) : 0;  // first token inside the window
  const int pg_first = win0 >> 4;
  const int first = kCl ? pg_first + s : pg_first + s * p.pps;
  const int pstep = kCl ? cs : 1;
  const int pend = kCl ? npages : min(npages, pg_first + s * p.pps + p.pps);
  const int n_mine = first < pend ? (pend - first + pstep - 1) / pstep : 0;
  if (!kCl && n_mine == 0) {
    if (p.counters != nullptr && s == 0 && tid < kHD)  // empty sequence: nobody else writes its output
      for (int hh = 0; hh < p.grp; ++hh) p.out[((size_t)b * p.Hq + (size_t)h * p.grp + hh) * kHD + tid] = 0.f;
    return;
  }

  // merge buffers: they live in the ring, which is free once every page of this CTA is consumed
  float (*sm_o)[8][kHD] = reinterpret_cast<float (*)[8][kHD]>(ring);                                   // [kAW][8][kHD]
  float (*c_o)[kHD] = reinterpret_cast<float (*)[kHD]>(ring + sizeof(float) * kAW * 8 * kHD);           // [8][kHD]
  float (*sm_m)[8] = reinterpret_cast<float (*)[8]>(ring + sizeof(float) * (kAW + 1) * 8 * kHD);        // [kAW][8]
  float (*sm_l)[8] = sm_m + kAW;                                                                        // [kAW][8]
  float* c_m = &sm_l[kAW][0];                                                                           // [8]
  float* c_l = c_m + 8;                                                                                 // [8]

  float m_run = -INFINITY, l_run = 0.f;
  float o[16][4];
#pragma unroll
  for (int j = 0; j < 16; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[j][i] = 0.f;

  if (warp == kAW) {
    // ===== producer: page ids 32 at a time, one 8 KB bulk copy per page ==========================
    bool failed = false;
    for (int base = 0; base < n_mine; base += 32) {
      const int i = base + lane;
      int pid = -1;
      if (i < n_mine) pid = (base == 0 && p.window == 0) ? pid_spec : p.table[(size_t)b * p.max_pages + first + i * pstep];
      const int cnt = min(32, n_mine - base);
      for (int j = 0; j < cnt; ++j) {
        const int pj = __shfl_sync(0xffffffffu, pid, j);
        if (lane == 0) {
          const int it = base + j, slot = it % kRing;
          if (!failed && !mbar_wait(smem_u32(empty + slot), ((uint32_t)(it / kRing) & 1u) ^ 1u)) failed = true;
          const uint32_t bar = smem_u32(full + slot);
          if ((unsigned)pj >= (unsigned)p.pages) {  // malformed page table: record, hand over an empty slot
            atomicExch(p.status, 1);
            slot_ok[slot] = 0;
            mbar_arrive(bar);
          } else {
            slot_ok[slot] = 1;
            mbar_expect_tx(bar, kSlotBytes);
            bulk_g2s(smem_u32(ring) + (uint32_t)slot * kSlotBytes, p.pool + ((size_t)pj * p.Hkv + h) * (2 * 16 * kHD), kSlotBytes, bar);
          }
        }
      }
    }
    if (failed && lane == 0) atomicExch(p.status, 4);
  } else {
    // ===== consumers =================================================================================
    // Q fragments: row g of the A operand = query head h*grp+g (rows >= grp are zero)
    uint4 qa[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) qa[i] = make_uint4(0u, 0u, 0u, 0u);
    if (g < p.grp) {
      const uint4* qp = reinterpret_cast<const uint4*>(p.q + ((size_t)b * p.Hq + (size_t)h * p.grp + g) * kHD);
#pragma unroll
      for (int i = 0; i < 4; ++i) qa[i] = qp[i * 4 + t];
    }
    auto compute_tile = [&](int pg, uint32_t kt, uint32_t vt) {
      // K rows of tokens g and g+8: the 16 bytes at d = 32i + 8t .. +7.  V is fetched only after the
      // scores are done, so that the K and V fragments never hold registers at the same time.
      uint4 kq[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) kq[nt][i] = lds128(kt + (uint32_t)(((nt * 8 + g) * 16 + i * 4 + t) * 16));
      // S = Q K^T for 16 tokens: two n-tiles of 8 tokens
      float sacc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mma16816(sacc[nt], qa[i].x, 0u, qa[i].y, 0u, kq[nt][i].x, kq[nt][i].y);
          mma16816(sacc[nt], qa[i].z, 0u, qa[i].w, 0u, kq[nt][i].z, kq[nt][i].w);
        }
      }
      // scale (optionally soft-capped), log2 domain, mask the tail of the last page and what lies before the window
      const int tok0 = pg * 16;
      float sv[4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int tok = tok0 + nt * 8 + 2 * t + c;
          float x = sacc[nt][c] * p.scale;
          if (p.softcap > 0.f) x = p.softcap * tanhf(x / p.softcap);
          sv[nt * 2 + c] = (tok < len && tok >= win0) ? x * 1.4426950408889634f : -INFINITY;
        }
      float tmax = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      const float m_new = fmaxf(m_run, tmax);  // finite: a listed page holds at least one attended token
      const float alpha = exp2f(m_run - m_new);
      float pr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pr[i] = exp2f(sv[i] - m_new);
      l_run = l_run * alpha + (pr[0] + pr[1] + pr[2] + pr[3]);
      m_run = m_new;
      if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          o[j][0] *= alpha;
          o[j][1] *= alpha;
        }
      }
      // P as A operand, split into two f16 terms so no probability precision is lost
      const uint32_t ph0 = pack_h2(pr[0], pr[1]), ph1 = pack_h2(pr[2], pr[3]);
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&ph0));
      const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&ph1));
      const uint32_t pl0 = pack_h2(pr[0] - f0.x, pr[1] - f0.y), pl1 = pack_h2(pr[2] - f1.x, pr[3] - f1.y);
      // V rows of tokens 2t, 2t+1, 2t+8, 2t+9: d = 8g..8g+7 and 64+8g..64+8g+7
      uint4 vv[4][2];
#pragma unroll
      for (int x = 0; x < 4; ++x) {
        const int tk = 2 * t + (x & 1) + ((x >> 1) << 3);
#pragma unroll
        for (int r = 0; r < 2; ++r) vv[x][r] = lds128(vt + (uint32_t)((tk * 16 + r * 8 + g) * 16));
      }
      // zero V rows that are not attended (their probability is 0, but 0 * garbage may be NaN)
      if (tok0 + 16 > len || tok0 < win0) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int tok = tok0 + 2 * t + (x & 1) + ((x >> 1) << 3);
          if (tok >= len || tok < win0) vv[x][0] = vv[x][1] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // O += P V : n-tile j covers d = 8n + (j&7) + 64*(j>>3), n = column of the tile
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int r = j >> 3, jj = j & 7;
        const uint32_t* va = reinterpret_cast<const uint32_t*>(&vv[0][r]);
        const uint32_t* vb = reinterpret_cast<const uint32_t*>(&vv[1][r]);
        const uint32_t* vc = reinterpret_cast<const uint32_t*>(&vv[2][r]);
        const uint32_t* vd = reinterpret_cast<const uint32_t*>(&vv[3][r]);
        const uint32_t sel = (jj & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(va[jj >> 1], vb[jj >> 1], sel);
        const uint32_t b1 = __byte_perm(vc[jj >> 1], vd[jj >> 1], sel);
        mma16816(o[j], ph0, 0u, ph1, 0u, b0, b1);
        mma16816(o[j], pl0, 0u, pl1, 0u, b0, b1);
      }
    };
    bool failed = false;
    for (int it = warp; it < n_mine; it += kAW) {
      const int slot = it % kRing;
      if (!failed && !mbar_wait(smem_u32(full + slot), (uint32_t)(it / kRing) & 1u)) failed = true;
      if (slot_ok[slot]) {
        const uint32_t kt = smem_u32(ring) + (uint32_t)slot * kSlotBytes, vt = kt + 16 * kHD * 2;
        compute_tile(first + it * pstep, kt, vt);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(empty + slot));  // the slot may be refilled
    }
    if (failed && lane == 0) atomicExch(p.status, 4);
  }

  // ---- merge the warps of this CTA ------------------------------------------
  __syncthreads();  // every warp is done with the ring: it becomes the merge buffers
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (warp < kAW && g < p.grp) {
    if (t == 0) {
      sm_m[warp][g] = m_run;
      sm_l[warp][g] = l_run;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int dbase = (j & 7) + 64 * (j >> 3);
      sm_o[warp][g][8 * (2 * t) + dbase] = o[j][0];
      sm_o[warp][g][8 * (2 * t + 1) + dbase] = o[j][1];
    }
  }
  __syncthreads();
  const int ns = kCl ? cs : (npages - pg_first + p.pps - 1) / p.pps;  // splits that hold pages
  const bool direct = !kCl && p.counters != nullptr && ns == 1;  // a single split: no partials needed
  for (int hh = 0; hh < p.grp && tid < kHD; ++hh) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAW; ++w) M = fmaxf(M, sm_m[w][hh]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < kAW; ++w) {
      const float f = sm_m[w][hh] == -INFINITY ? 0.f : exp2f(sm_m[w][hh] - M);  // a warp without pages
      L += sm_l[w][hh] * f;
      O += sm_o[w][hh][tid] * f;
    }
    if (kCl) {
      c_o[hh][tid] = O;
      if (tid == 0) {
        c_m[hh] = M;
        c_l[hh] = L;
      }
    } else if (direct) {
      p.out[((size_t)b * p.Hq + (size_t)h * p.grp + hh) * kHD + tid] = O / L;
    } else {
      const size_t row = ((size_t)b * p.Hq + (size_t)h * p.grp + hh) * p.S + s;
      __stcg(p.part_o + row * kHD + tid, O);
      if (tid == 0) {
        __stcg(p.part_ml + row * 2, M);
        __stcg(p.part_ml + row * 2 + 1, L);
      }
    }
  }
  if (kCl) {
    // ---- cluster merge: CTA `s` owns 128 / cs dims of every query head and reads the partials of
    // all CTAs of the cluster through distributed shared memory
    if (cs > 1) cluster_sync();
    else __syncthreads();
    const int dper = kHD / cs;
    for (int e = tid; e < p.grp * dper; e += kAT) {
      const int hh = e / dper, d = s * dper + e % dper;
      float mr[kCS], lr[kCS], orr[kCS];
#pragma unroll
      for (int r = 0; r < kCS; ++r) {
        mr[r] = -INFINITY;
        lr[r] = orr[r] = 0.f;
        if (r < cs) {
          mr[r] = ld_cluster(cluster_map(&c_m[hh], r));
          lr[r] = ld_cluster(cluster_map(&c_l[hh], r));
          orr[r] = ld_cluster(cluster_map(&c_o[hh][d], r));
        }
      }
      float M = -INFINITY;
#pragma unroll
      for (int r = 0; r < kCS; ++r) M = fmaxf(M, mr[r]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int r = 0; r < kCS; ++r) {
        const float f = mr[r] == -INFINITY ? 0.f : exp2f(mr[r] - M);  // a CTA without pages
        L = fmaf(lr[r], f, L);
        O = fmaf(orr[r], f, O);
      }
      p.out[((size_t)b * p.Hq + (size_t)h * p.grp + hh) * kHD + d] = L > 0.f ? O / L : 0.f;
    }
    if (cs > 1) cluster_sync();  // nobody leaves while a peer may still read its shared memory
    return;
  }
  if (p.counters == nullptr || direct) return;
  // ---- the CTA that completes this (sequence, kv head) merges its splits (no waiting) ----
  __shared__ int s_last;
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(p.counters + b * p.Hkv + h, 1) == ns - 1;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // one warp per query head; lanes first share the (max, sum) pairs of the splits, then each lane
  // merges 4 of the 128 output dims with independent (pipelined) loads
  for (int hh = warp; hh < p.grp && warp < kAW; hh += kAW) {
    const size_t row0 = ((size_t)b * p.Hq + (size_t)h * p.grp + hh) * p.S;
    float M = -INFINITY;
    for (int s2 = lane; s2 < ns; s2 += 32) M = fmaxf(M, __ldcg(p.part_ml + (row0 + s2) * 2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    for (int s2 = lane; s2 < ns; s2 += 32) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (row0 + s2) * 2));
      L += ml.y * exp2f(ml.x - M);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int s2 = 0; s2 < ns; ++s2) {
      const float f = exp2f(__ldcg(p.part_ml + (row0 + s2) * 2) - M);
      const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + (row0 + s2) * kHD) + lane);
      O.x = fmaf(v.x, f, O.x); O.y = fmaf(v.y, f, O.y); O.z = fmaf(v.z, f, O.z); O.w = fmaf(v.w, f, O.w);
    }
    const float inv = 1.f / L;
    reinterpret_cast<float4*>(p.out + ((size_t)b * p.Hq + (size_t)h * p.grp + hh) * kHD)[lane] =
        make_float4(O.x * inv, O.y * inv, O.z * inv, O.w * inv);
  }
  __syncthreads();
  if (tid == 0) p.counters[b * p.Hkv + h] = 0;  // ready for the next call
}

// three CTAs per SM (<= 136 registers): this path is chosen when there are many pages per SM to cover
__global__ void __launch_bounds__(kAT, 3) attn_decode_kernel(const AttnParams p) { attn_decode_body<false>(p); }

// launched with a cluster dimension of (p.S, 1, 1) = (gridDim.x, 1, 1)
__global__ void __launch_bounds__(kAT) attn_decode_cluster_kernel(const AttnParams p) {
#ifdef QENG_TRACE
  unsigned long long* rec = nullptr;
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) rec = qeng_trace_open(p.status, 2);
#endif
  attn_decode_body<true>(p);
#ifdef QENG_TRACE
  if (rec) rec[4] = qeng_trace_now();
#endif
}

__global__ void __launch_bounds__(kHD) attn_combine_kernel(const AttnParams p) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int len = p.lens[b];
  const int npages = min((len + 15) >> 4, p.max_pages);
  const int pg_first = p.window > 0 ? max(0, len - p.window) >> 4 : 0;
  const int ns = (npages - pg_first + p.pps - 1) / p.pps;
  const size_t row0 = ((size_t)b * p.Hq + head) * p.S;
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, p.part_ml[(row0 + s) * 2]);
  float L = 0.f, O = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float f = exp2f(p.part_ml[(row0 + s) * 2] - M);
    L += p.part_ml[(row0 + s) * 2 + 1] * f;
    O += p.part_o[(row0 + s) * kHD + d] * f;
  }
  p.out[((size_t)b * p.Hq + head) * kHD + d] = ns > 0 ? O / L : 0.f;
}

__global__ void kv_append_kernel(__half* pool, const float* k, const float* v, const int32_t* table,
                                 const int32_t* pos, int B, int Hkv, int pages, int max_pages, int32_t* status) {
  const int b = blockIdx.y, h = blockIdx.x, d = threadIdx.x;
  const int ps = pos[b];
  const int pg = ps >> 4;
  if (pg >= max_pages) {
    if (d == 0) atomicExch(status, 2);
    return;
  }
  const int pid = table[(size_t)b * max_pages + pg];
  if ((unsigned)pid >= (unsigned)pages) {
    if (d == 0) atomicExch(status, 1);
    return;
  }
  __half* base = pool + ((size_t)pid * Hkv + h) * (2 * 16 * kHD) + (ps & 15) * kHD + d;
  base[0] = __float2half_rn(k[((size_t)b * Hkv + h) * kHD + d]);
  base[16 * kHD] = __float2half_rn(v[((size_t)b * Hkv + h) * kHD + d]);
}

}  // namespace

// ---- scratch for the entry point that allocates nothing ---------------------------------
// Some hosts may not allocate device memory once they are running: a runtime that hands the
// engine a fixed memory budget at start-up, or a caller inside a region where the CUDA
// allocator must not be entered (a latency-critical token loop, a process that shares the GPU
// under a hard memory cap).  For them the split partials live in this file-scope array, which
// every GPU that loads the library holds from load to exit.  4 MiB covers
// B * Hq * splits * 130 <= 1048576 floats, e.g. 16 sequences x 32 heads x 15 splits.
constexpr size_t kStaticScratchFloats = (size_t)1 << 20;
static __device__ __align__(256) float g_attn_static_scratch[kStaticScratchFloats];
// In host code the array's name is only a handle: the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
constexpr int kMaxDevices = 64;
static float* g_attn_static_addr[kMaxDevices] = {};

constexpr int kMaxAttnCounters = 1 << 16;  // (sequence, kv head) pairs per call

// Splits: enough CTAs to fill the machine several times over, at least one page per warp.
static int pages_per_split(const qeng_ctx* ctx, int64_t B, int64_t Hkv, int64_t max_pages) {
  // the fixed-split kernel keeps three CTAs per SM resident: one full wave of them is the target
  int64_t target = (int64_t)ctx->sm_count * (ctx->attn_ctas_per_sm > 0 ? ctx->attn_ctas_per_sm : 3);
  // splits per (sequence, kv head) that fill the wave, then equal page ranges for the longest sequence
  int64_t S = (target + B * Hkv - 1) / (B * Hkv);
  if (S < 1) S = 1;
  int64_t pps = (max_pages + S - 1) / S;
  pps = (pps + kAW - 1) / kAW * kAW;
  if (pps < kAW) pps = kAW;
  if (pps > 128) pps = 128;
  return (int)pps;
}

// Grow the split scratch of the context to what a call of this shape needs.
// The steady state never allocates; a growing call drains the device first.
int32_t qeng_attn_reserve(qeng_ctx* ctx, int64_t B, int64_t Hq, int64_t Hkv, int64_t max_pages) {
  const int pps = pages_per_split(ctx, B, Hkv, max_pages);
  const int64_t S = (max_pages + pps - 1) / pps;
  if (B * Hkv > kMaxAttnCounters)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "attn: B * kv_heads = %lld exceeds %d", (long long)(B * Hkv), kMaxAttnCounters);
  // arrival counters first (fixed place for every shape), partials behind them
  size_t need = (size_t)kMaxAttnCounters * sizeof(int) + (size_t)B * Hq * S * (kHD + 2) * sizeof(float);
  if (need <= ctx->attn_scratch_bytes) return QENG_OK;
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  QENG_CUDA(ctx, cudaDeviceSynchronize());
  if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
  ctx->attn_scratch = nullptr;
  ctx->attn_scratch_bytes = 0;
  ctx->scratch_gen++;
  QENG_CUDA(ctx, cudaMalloc(&ctx->attn_scratch, need));
  QENG_CUDA(ctx, cudaMemset(ctx->attn_scratch, 0, need));  // the arrival counters start at zero and return to it
  ctx->attn_scratch_bytes = need;
  return QENG_OK;
}

extern "C" {

int32_t qeng_kv_pool_create(qeng_ctx* ctx, int64_t pages, int64_t kv_heads, int64_t hd, qeng_kv_pool** out) {
  if (!ctx || !out) return qeng_fail(ctx, QENG_ERR_ARG, "kv_pool_create: null argument");
  *out = nullptr;
  if (hd != kHD) return qeng_fail(ctx, QENG_ERR_SHAPE, "kv_pool_create: head_dim must be 128 (got %lld)", (long long)hd);
  if (pages <= 0 || kv_heads <= 0) return qeng_fail(ctx, QENG_ERR_ARG, "kv_pool_create: pages and kv_heads must be positive");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  qeng_kv_pool* p = new qeng_kv_pool();
  p->pages = pages; p->kv_heads = kv_heads; p->hd = hd; p->data = nullptr;
  size_t bytes = (size_t)pages * kv_heads * 2 * 16 * hd * sizeof(__half);
  cudaError_t e = cudaMalloc(&p->data, bytes);
  if (e == cudaSuccess) e = cudaMemset(p->data, 0, bytes);
  if (e != cudaSuccess) {
    if (p->data) cudaFree(p->data);
    delete p;
    return qeng_fail(ctx, QENG_ERR_CUDA, "kv_pool_create: %s", cudaGetErrorString(e));
  }
  *out = p;
  return QENG_OK;
}

int32_t qeng_kv_pool_free(qeng_ctx* ctx, qeng_kv_pool* pool) {
  if (!pool) return QENG_OK;
  if (ctx) cudaSetDevice(ctx->device);
  if (pool->data) cudaFree(pool->data);
  delete pool;
  return QENG_OK;
}

void* qeng_kv_pool_data(const qeng_kv_pool* pool) { return pool ? pool->data : nullptr; }
int64_t qeng_kv_pool_pages(const qeng_kv_pool* pool) { return pool ? pool->pages : 0; }

int32_t qeng_kv_append(qeng_ctx* ctx, qeng_kv_pool* pool, const float* k, const float* v, const int32_t* page_table,
                       int64_t max_pages, const int32_t* pos, int64_t B, void* stream) {
  if (!ctx || !pool || !k || !v || !page_table || !pos) return qeng_fail(ctx, QENG_ERR_ARG, "kv_append: null argument");
  if (B <= 0 || max_pages <= 0) return qeng_fail(ctx, QENG_ERR_ARG, "kv_append: B and max_pages must be positive");
  QENG_ENTER(ctx);
  dim3 grid((unsigned)pool->kv_heads, (unsigned)B);
  kv_append_kernel<<<grid, kHD, 0, (cudaStream_t)stream>>>(pool->data, k, v, page_table, pos, (int)B,
                                                           (int)pool->kv_heads, (int)pool->pages, (int)max_pages,
                                                           ctx->status);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

// opt-in shared memory of the two attention kernels (the page-tile ring), once per device
static int32_t attn_configure(qeng_ctx* ctx) {
  static bool configured_on[64] = {};
  bool& configured = configured_on[ctx->device & 63];
  if (configured) return QENG_OK;
  QENG_CUDA(ctx, cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing * kSlotBytes));
  QENG_CUDA(ctx, cudaFuncSetAttribute(attn_decode_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kRing * kSlotBytes));
  configured = true;
  return QENG_OK;
}

int32_t qeng_attn_decode(qeng_ctx* ctx, const qeng_kv_pool* pool, const uint16_t* q_f16, const int32_t* page_table,
                         int64_t max_pages, const int32_t* lens, int64_t B, int64_t Hq, float scale, float* out,
                         void* stream) {
  return qeng_attn_decode_ex(ctx, pool, q_f16, page_table, max_pages, lens, B, Hq, scale, 0.f, 0, out, stream);
}

int32_t qeng_attn_decode_ex(qeng_ctx* ctx, const qeng_kv_pool* pool, const uint16_t* q_f16, const int32_t* page_table,
                            int64_t max_pages, const int32_t* lens, int64_t B, int64_t Hq, float scale, float softcap,
                            int32_t window, float* out, void* stream) {
  if (!ctx || !pool || !q_f16 || !page_table || !lens || !out) return qeng_fail(ctx, QENG_ERR_ARG, "attn_decode: null argument");
  if (B <= 0 || max_pages <= 0 || Hq <= 0) return qeng_fail(ctx, QENG_ERR_ARG, "attn_decode: B, Hq, max_pages must be positive");
  if (softcap < 0.f || window < 0) return qeng_fail(ctx, QENG_ERR_ARG, "attn_decode: softcap and window must not be negative");
  if (Hq % pool->kv_heads != 0 || Hq / pool->kv_heads > 8)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "attn_decode: query heads per kv head must divide evenly and be <= 8");
  if (((reinterpret_cast<uintptr_t>(q_f16) | reinterpret_cast<uintptr_t>(out)) & 15) != 0)
    return qeng_fail(ctx, QENG_ERR_ALIGN, "attn_decode: q and out must be 16-byte aligned");
  QENG_ENTER(ctx);
  int32_t rc0 = attn_configure(ctx);
  if (rc0 != QENG_OK) return rc0;
  AttnParams p;
  p.pool = pool->data; p.q = reinterpret_cast<const __half*>(q_f16);
  p.table = page_table; p.lens = lens; p.out = out; p.status = ctx->status;
  p.pages = (int)pool->pages; p.Hkv = (int)pool->kv_heads; p.Hq = (int)Hq; p.grp = (int)(Hq / pool->kv_heads);
  p.max_pages = (int)max_pages;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.scale = scale; p.softcap = softcap; p.window = window;
  const bool no_cluster = !ctx->attn_cluster;
  // Cluster path: 1, 2, 4 or 8 CTAs per (sequence, kv head), as many as keep the grid within about one
  // wave (two CTAs per SM), merged through distributed shared memory; caches beyond 16K tokens and
  // long caches at large batch (bandwidth-bound, a little faster there) take the fixed splits below.
  int cs = kCS;
  while (cs > 1 && B * pool->kv_heads * cs > 2 * (int64_t)ctx->sm_count) cs >>= 1;
  if (!no_cluster && max_pages <= 1024 && B * pool->kv_heads * max_pages <= 16384) {
    p.pps = 0; p.S = cs; p.counters = nullptr; p.part_o = nullptr; p.part_ml = nullptr;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cs, (unsigned)p.Hkv, (unsigned)B);
    cfg.blockDim = dim3(kAT);
    cfg.dynamicSmemBytes = kRing * kSlotBytes;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QENG_CUDA(ctx, cudaLaunchKernelEx(&cfg, attn_decode_cluster_kernel, p));
    return QENG_OK;
  }
  p.pps = pages_per_split(ctx, B, pool->kv_heads, max_pages);
  p.S = (int)((max_pages + p.pps - 1) / p.pps);
  int32_t rc = qeng_attn_reserve(ctx, B, Hq, pool->kv_heads, max_pages);
  if (rc != QENG_OK) return rc;
  p.counters = reinterpret_cast<int*>(ctx->attn_scratch);
  p.part_o = ctx->attn_scratch + kMaxAttnCounters;
  p.part_ml = p.part_o + (size_t)B * Hq * p.S * kHD;
  dim3 grid((unsigned)p.S, (unsigned)p.Hkv, (unsigned)B);
  attn_decode_kernel<<<grid, kAT, kRing * kSlotBytes, (cudaStream_t)stream>>>(p);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

int32_t qeng_attn_decode_noalloc(qeng_ctx* ctx, const qeng_kv_pool* pool, const uint16_t* q_f16,
                                 const int32_t* page_table, int64_t max_pages, const int32_t* lens, int64_t B,
                                 int64_t Hq, float scale, float* out, void* stream) {
  if (!ctx || !pool || !q_f16 || !page_table || !lens || !out)
    return qeng_fail(ctx, QENG_ERR_ARG, "attn_decode_noalloc: null argument");
  if (B <= 0 || max_pages <= 0 || Hq <= 0)
    return qeng_fail(ctx, QENG_ERR_ARG, "attn_decode_noalloc: B, Hq, max_pages must be positive");
  if (Hq % pool->kv_heads != 0 || Hq / pool->kv_heads > 8)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "attn_decode_noalloc: query heads per kv head must divide evenly and be <= 8");
  if ((reinterpret_cast<uintptr_t>(q_f16) & 15) != 0)
    return qeng_fail(ctx, QENG_ERR_ALIGN, "attn_decode_noalloc: q must be 16-byte aligned");
  if (ctx->device < 0 || ctx->device >= kMaxDevices)
    return qeng_fail(ctx, QENG_ERR_ARG, "attn_decode_noalloc: device index %d outside 0..%d", ctx->device, kMaxDevices - 1);
  QENG_ENTER(ctx);
  AttnParams p;
  p.pps = pages_per_split(ctx, B, pool->kv_heads, max_pages);
  p.S = (int)((max_pages + p.pps - 1) / p.pps);
  const size_t need = (size_t)B * Hq * p.S * (kHD + 2);
  if (need > kStaticScratchFloats)
    return qeng_fail(ctx, QENG_ERR_SHAPE,
                     "attn_decode_noalloc: B*Hq*splits*130 = %zu floats exceeds the built-in scratch of %zu floats "
                     "(B=%lld Hq=%lld splits=%d); use qeng_attn_decode",
                     need, kStaticScratchFloats, (long long)B, (long long)Hq, p.S);
  // set-up, once per device: resolve the array's device address with that device current
  if (!g_attn_static_addr[ctx->device]) {
    QENG_CUDA(ctx, cudaSetDevice(ctx->device));
    float* addr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&addr), g_attn_static_scratch);
    if (e != cudaSuccess || !addr)
      return qeng_fail(ctx, QENG_ERR_CUDA, "attn_decode_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
    g_attn_static_addr[ctx->device] = addr;
  }
  float* scratch = g_attn_static_addr[ctx->device];
  p.pool = pool->data; p.q = reinterpret_cast<const __half*>(q_f16);
  p.table = page_table; p.lens = lens; p.out = out; p.status = ctx->status;
  p.pages = (int)pool->pages; p.Hkv = (int)pool->kv_heads; p.Hq = (int)Hq; p.grp = (int)(Hq / pool->kv_heads);
  p.max_pages = (int)max_pages;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.scale = scale; p.softcap = 0.f; p.window = 0;
  {
    int32_t rc0 = attn_configure(ctx);
    if (rc0 != QENG_OK) return rc0;
  }
  // every partial that the merge reads is written by this call first: nothing has to start at zero
  p.counters = nullptr;  // merge in a second kernel
  p.part_o = scratch;
  p.part_ml = scratch + (size_t)B * Hq * p.S * kHD;
  dim3 grid((unsigned)p.S, (unsigned)p.Hkv, (unsigned)B);
  attn_decode_kernel<<<grid, kAT, kRing * kSlotBytes, (cudaStream_t)stream>>>(p);
  QENG_LAUNCH_CHECK(ctx);
  dim3 grid2((unsigned)Hq, (unsigned)B);
  attn_combine_kernel<<<grid2, kHD, 0, (cudaStream_t)stream>>>(p);
  QENG_LAUNCH_CHECK(ctx);
  return QENG_OK;
}

}  // extern "C"
