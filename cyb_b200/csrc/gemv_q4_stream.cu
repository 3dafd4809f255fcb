// Streaming decode GEMV/GEMM over block-quantised weights: the bandwidth kernel.
//
// One persistent CTA per SM: 16 consumer warps and one producer warp per tile group around a ring
// of shared-memory stages.  A producer walks its row tiles (16 rows x K, contiguous in the packed
// layout) and copies them stage by stage (up to 64 chunks of 64 k: a whole row tile of K = 4096,
// 36 KB for 4-bit blocks) with bulk asynchronous copies (cp.async.bulk, completion counted on an
// mbarrier), so ~200 KB per SM are in flight without holding registers and independent of what the
// consumers are doing.  Consumers take the chunks of a stage round-robin, read them with
// conflict-free 128-bit shared loads and contract on the tensor pipe with integer MMAs against the
// activations quantised to block fixed point (gemm_q4_s8.cuh has the arithmetic).
//
// One or two activation rows: all 16 warps work on every tile, park their partial sums of a tile in
// shared memory and move on; the CTA meets once per 16 tiles, sums the partials and runs the fused
// epilogues of those tiles in parallel (kTG = 0).  Three to 16 rows: the warps form 1, 2 or 4 tile
// groups, each with its own ring and producer warp, and reduce per tile over one named barrier.
//
// Up to 4 activation rows keep the whole K range staged; more rows (up to 16 per launch) arrive as
// quantised images per K slice (quantise_rows_kernel), the weights of a slice are streamed for all
// of the CTA's tiles and the partial sums kept in shared memory between slices, so the weights
// still cross HBM once per launch.
//
// Weight formats: 4-bit blocks (nibbles unpacked in registers, zero point 8), 8-bit blocks (the
// bytes are the MMA operand as stored), 4-bit K-quant blocks (f32 scale and minimum per block, up to
// 4 rows).  HBM-bound: algorithmic bytes = N*K*{0.5625, 1.0625, 0.75} + activations + outputs.
#include <cstdlib>
#include "gemm_q4_s8.cuh"

namespace {
using namespace q4s8;

constexpr int kStageChunks = 64;  // 64-wide K chunks per ring stage (36 KB: a whole row tile of K = 4096)
constexpr int kDeferTiles = 16;   // tiles whose partial sums a CTA parks before it meets to reduce them
constexpr int kGroups = 3;  // groups of 8 k one consumer thread stages in the single-slice mode: K <= 8 * kGroups * kCT

struct StreamParams {
  // the matrix multiplied next (may be null): its tiles are requested into L2 once this
  // CTA's own loads are all issued
  const uint4* pf_qs;
  const uint2* pf_sc;
  int pf_ntiles, pf_nchunks, pf_wchunk, pf_schunk;
  const uint4* qs;
  const uint2* sc;
  int ntiles, nchunks;
  int K;
  const void* x;
  int x_dtype;
  long long ldx;
  int M, cols;
  float* y;
  long long ldy;
  const float* gamma;
  float eps;
  int epilogue;
  const float* resid;
  int nstages;        // ring slots
  int stage_chunks;   // chunks per ring slot
  int slice_chunks;   // chunks of K staged at once (= all of them in single-slice mode)
  int nslices;
  int32_t* status;
  qeng_qkv_epi qkv;
  // more than 4 rows: the activations arrive quantised, as one ready-made image of the staging area
  // per K slice (written by quantise_rows_kernel), and are brought in with one bulk copy per slice
  const unsigned char* ximage;
  uint32_t ximage_slice_bytes;
  // tensor parallelism carried by the matmuls (qeng_gemm_fuse::tp_push_kind / tp_gather_kind)
  uint2* push_inbox[8];        // every rank's inbox of the push kind, as mapped here
  int push_world, push_rank;   // push_world = 0: the epilogue writes y as usual
  const uint2* gather_inbox;   // this rank's inbox of the gather kind
  int gather_world;            // 0: x is used as it is
  float* x_writeback;          // the gathered rows, written by CTA 0 (the residual stream itself)
  const unsigned* tp_seq;      // decode steps completed: the tag base
  unsigned tp_tags_per_step, push_tag_off, gather_tag_off;
};

// Quantises the activation rows once per matmul (instead of once per CTA) into the exact bytes the
// streaming kernel keeps in shared memory for a K slice: columns, accumulator start values and
// block factors at the offsets of x_layout().  Grid (slices, rows).
__global__ void __launch_bounds__(512) quantise_rows_kernel(const void* __restrict__ x, int x_dtype, long long ldx, int M, int K,
                                                            const float* __restrict__ gamma, float eps, int slice_chunks,
                                                            unsigned char* __restrict__ image, uint32_t slice_bytes,
                                                            const uint2* __restrict__ gather_inbox, int gather_world,
                                                            const unsigned* __restrict__ tp_seq, unsigned tags_per_step,
                                                            unsigned gather_tag_off, float* __restrict__ x_writeback,
                                                            int32_t* status) {
  extern __shared__ __align__(16) unsigned char qsm[];
  __shared__ float part[16];
  const int sl = blockIdx.x, m = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const XLayout L = x_layout(2 * M, slice_chunks, false);
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  // With a gather, the row (f32) is first completed in shared memory: x + the ranks' tagged parts, in
  // rank order; the CTA of slice 0 writes it back as the new residual row.
  float* xrow = nullptr;
  if (gather_world > 0) {
    xrow = reinterpret_cast<float*>(qsm + 2u * L.col_stride + 4u * L.zs);
    const unsigned tag = *tp_seq * tags_per_step + gather_tag_off + 1u;
    Waits W;
    for (int k0 = tid * 8; k0 < K; k0 += 512 * 8) {
      const float4* xp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(x) + (long long)m * ldx + k0);
      float4 a = xp[0], b = xp[1];
      for (int r = 0; r < gather_world; ++r) {
        float pt[8];
        poll8(gather_inbox + ((size_t)r * kTpFuseRows + m) * kTpFuseDm + k0, tag, pt, W, status);
        a.x += pt[0]; a.y += pt[1]; a.z += pt[2]; a.w += pt[3];
        b.x += pt[4]; b.y += pt[5]; b.z += pt[6]; b.w += pt[7];
      }
      *reinterpret_cast<float4*>(xrow + k0) = a;
      *reinterpret_cast<float4*>(xrow + k0 + 4) = b;
      if (sl == 0) {
        float4* wp = reinterpret_cast<float4*>(x_writeback + (long long)m * ldx + k0);
        wp[0] = a;
        wp[1] = b;
      }
    }
    __syncthreads();
  }
  auto xval = [&](int k) { return xrow ? xrow[k] : act_f32(x, x_dtype, (long long)m * ldx + k); };
  float rs = 1.f;
  if (gamma != nullptr) {
    float ss = 0.f;
    for (int k = tid; k < K; k += 512) {
      const float v = xval(k);
      ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) part[warp] = ss;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 16; ++w) tot += part[w];
    rs = rsqrtf(tot / (float)K + eps);
  }
  // local copy of this row's two columns and its z / f entries
  const uint32_t sx = smem_u32(qsm), sz = sx + 2u * L.col_stride, sf = sz + 2u * L.zs;
  const int ngroups = L.nblk * 4;
  for (int grp0 = 0; grp0 < ngroups; grp0 += 512) {
    const int grp = grp0 + tid;
    if ((grp & ~31) < ngroups) {
      float v[8];
      const int k0 = sl * slice_chunks * 64 + grp * 8;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[i] = 0.f;
        if (grp < ngroups && k0 + i < K) {
          v[i] = xval(k0 + i);
          if (gamma != nullptr) v[i] *= gamma[k0 + i] * rs;
        }
      }
      quantise_group<2>(v, grp < ngroups, sx, L.col_stride, sz, sf, L.zs, (grp >> 2) * 32, grp & 3);
    }
  }
  __syncthreads();
  unsigned char* img = image + (size_t)sl * slice_bytes;
  const uint4* src = reinterpret_cast<const uint4*>(qsm);
  uint4* dx = reinterpret_cast<uint4*>(img + L.xq + (size_t)(2 * m) * L.col_stride);
  for (uint32_t i = tid; i < 2u * L.col_stride / 16u; i += 512) dx[i] = src[i];
  uint4* dz = reinterpret_cast<uint4*>(img + L.zin + (size_t)(2 * m) * L.zs);
  const uint4* srz = reinterpret_cast<const uint4*>(qsm + 2u * L.col_stride);
  for (uint32_t i = tid; i < 2u * L.zs / 16u; i += 512) dz[i] = srz[i];
  uint4* df = reinterpret_cast<uint4*>(img + L.fex + (size_t)(2 * m) * L.zs);
  const uint4* srf = reinterpret_cast<const uint4*>(qsm + 2u * L.col_stride + 2u * L.zs);
  for (uint32_t i = tid; i < 2u * L.zs / 16u; i += 512) df[i] = srf[i];
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;\n" ::"n"(kCT) : "memory"); }
// the warps of one tile group (named barriers 2, 3, ...)
template <int GW>
__device__ __forceinline__ void group_sync(int gi) { asm volatile("bar.sync %0, %1;\n" ::"r"(2 + gi), "n"(GW * 32) : "memory"); }

// MODE: how the 8 MMA columns are used (gemm_q4_s8.cuh)
//   kM1L3: one activation row in three limbs (22 bits), two blocks per accumulator fragment
//   kM1L2: one row in two limbs (15 bits), four blocks per fragment
//   kM2L2: two rows in two limbs, two blocks per fragment
//   kMN  : NT tiles of four rows in two limbs, one block per fragment
enum { kM1L3 = 0, kM1L2 = 1, kM2L2 = 2, kMN = 3 };
template <int MODE, int NT, int kTG, bool Q8 = false, bool KQ = false>
__global__ void __launch_bounds__(kCT + 32 * (kTG == 0 ? 1 : kTG), 1) gemv_q4_stream_kernel(const StreamParams p) {
  constexpr uint32_t kWChunk = Q8 ? 1024u : 512u;  // bytes of the weight plane per 64-wide chunk of a row tile
  constexpr uint32_t kSChunk = KQ ? 256u : 64u;    // bytes of the scale plane per chunk (f16 scales, or f32 scale + minimum)
  // kTG = 0: all 16 warps work on every tile and the per-tile reduction is deferred: each warp parks its
  // partial sums of a tile in shared memory and moves on; the CTA meets once at the end (or every
  // kDeferTiles tiles), where the warps sum the partials and run the epilogues of the tiles in parallel
  constexpr bool kDefer = kTG == 0;
  constexpr int kTGe = kDefer ? 1 : kTG;  // tile groups (rings, producer warps)
  constexpr int kGW = kCW / kTGe;         // warps per tile group
  constexpr int kMR = MODE == kMN ? 4 * NT : (MODE == kM2L2 ? 2 : 1);  // activation rows the fragment layout holds
  constexpr int kLimbs = MODE == kM1L3 ? 3 : 2;
  constexpr bool kZeroed = MODE != kMN;
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int NS = p.nstages;
  const uint32_t stage_bytes = (uint32_t)p.stage_chunks * (kWChunk + kSChunk);
  const int sl_alloc = MODE == kM1L2 ? (p.slice_chunks + 1) & ~1 : p.slice_chunks;
  const XLayout L = x_layout(p.cols, sl_alloc, kZeroed, 0, KQ);
  // carve: ring | activations (128-byte aligned) | reduction buffers | slice accumulators | barriers
  unsigned char* ring = smem;
  unsigned char* xreg = smem + (((size_t)NS * stage_bytes + 127) & ~(size_t)127);
  const bool two_areas = MODE == kMN && p.ximage != nullptr;
  float* red = reinterpret_cast<float*>(xreg + (two_areas ? 2u * ((L.bytes + 127u) & ~127u) : L.bytes));  // [kTG][2][kGW][kMR * 16], deferred: [kDeferTiles][kCW][kMR * 16]
  constexpr int red_stride = kMR * 16;
  float* accsm = red + (kDefer ? kDeferTiles * kCW : kTGe * 2 * kGW) * red_stride;                 // [tiles of this CTA][kMR * 16] (several slices only)
  const int my_tiles = p.ntiles > (int)blockIdx.x ? (p.ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
  const int max_tiles = (p.ntiles + (int)gridDim.x - 1) / (int)gridDim.x;
  uint64_t* full = reinterpret_cast<uint64_t*>(accsm + (p.nslices > 1 ? (size_t)max_tiles * red_stride : 0));
  uint64_t* empty = full + kMaxStages;
  __shared__ __align__(8) uint64_t xbar[2];  // arrival of a slice image (two staging areas, used in turn)
  const bool imaged = MODE == kMN && p.ximage != nullptr;
  const uint32_t ximg_stride = (L.bytes + 127u) & ~127u;  // second staging area right behind the first
  __shared__ float warp_part[2 * kCW], rinv[16];
  const uint32_t xbase = smem_u32(xreg);
  (void)my_tiles;

#ifdef QENG_TRACE
  unsigned long long* trace = reinterpret_cast<unsigned long long*>(p.status) + 1;  // 7 stamps behind the status word
#define QENG_STAMP(i) do { if (blockIdx.x == 0 && tid == 0) trace[i] = globaltimer(); } while (0)
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // cycle counters kept in registers, written once at the end
#define QENG_TICK(v) const long long v = clock64()
#define QENG_TOCK(v, i, cond) do { tacc[(i) - 8] += clock64() - v; } while (0)
#define QENG_COUNT(i, cond) do { tacc[(i) - 8] += 1; } while (0)
#define QENG_FLUSH(i, cond) do { if (blockIdx.x == 0 && lane == 0 && (cond)) trace[i] += (unsigned long long)tacc[(i) - 8]; } while (0)
#else
#define QENG_STAMP(i) do { } while (0)
#define QENG_TICK(v) do { } while (0)
#define QENG_TOCK(v, i, cond) do { } while (0)
#define QENG_COUNT(i, cond) do { } while (0)
#define QENG_FLUSH(i, cond) do { } while (0)
#endif
  QENG_STAMP(0);
#ifdef QENG_TRACE
  unsigned long long* rec = nullptr;
  if (blockIdx.x == 0 && tid == 0) { rec = qeng_trace_open(p.status, 1000000ull * (unsigned)MODE + 1000ull * (unsigned)p.M + (unsigned)(p.ntiles / 16) + ((unsigned long long)p.nchunks << 32)); }
#define QENG_REC(i) do { if (rec) rec[i] = qeng_trace_now(); } while (0)
#else
#define QENG_REC(i) do { } while (0)
#endif
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");  // the next kernel may start its own weight stream
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(full + s), 1);
      mbar_init(smem_u32(empty + s), kGW);
    }
    mbar_init(smem_u32(xbar), 1);
    mbar_init(smem_u32(xbar + 1), 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  const int NSg = NS / kTGe;  // ring slots per tile group; group gi owns slots [gi * NSg, (gi + 1) * NSg)

  if (warp >= kCW) {
    // ===== producers: stream this CTA's row tiles through the ring, slice by slice ==========
    // One producer warp per tile group (a wait on a group's barrier suspends only that group's
    // feeder): each ring fills as its own consumers free slots, however far the groups drift apart.
    const int pg = warp - kCW;
    if (lane == 0) {
      bool failed = false;
      int tcount = 0, use = 0;
      for (int sl = 0; sl < p.nslices; ++sl) {
        const int cs0 = sl * p.slice_chunks, cs1 = min(p.nchunks, cs0 + p.slice_chunks);
        for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount) {
          if (tcount % kTGe != pg) continue;
          for (int c0 = cs0; c0 < cs1; c0 += p.stage_chunks, ++use) {
            const int s = pg * NSg + use % NSg;
            const uint32_t ph = (uint32_t)(use / NSg) & 1u;
            QENG_TICK(tp0);
            if (!failed && !mbar_wait(smem_u32(empty + s), ph ^ 1u)) failed = true;
            QENG_TOCK(tp0, 12, pg == 0);
            const int nc = min(p.stage_chunks, cs1 - c0);
            const uint32_t bar = smem_u32(full + s);
            const uint32_t dst = smem_u32(ring) + (uint32_t)s * stage_bytes;
            const size_t chunk = (size_t)tile * p.nchunks + c0;
            mbar_expect_tx(bar, (uint32_t)nc * (kWChunk + kSChunk));
            bulk_g2s(dst, reinterpret_cast<const char*>(p.qs) + chunk * kWChunk, (uint32_t)nc * kWChunk, bar);
            bulk_g2s(dst + (uint32_t)p.stage_chunks * kWChunk, reinterpret_cast<const char*>(p.sc) + chunk * kSChunk,
                     (uint32_t)nc * kSChunk, bar);
          }
        }
      }
      if (failed) atomicExch(p.status, 4);
      QENG_FLUSH(12, pg == 0);
    }
    __syncwarp();
    // Own loads are all in flight: ask L2 for this CTA's share of the next matrix, so that HBM
    // does not idle while the consumers drain the ring and the next kernel starts up.
    if (pg == 0 && p.pf_qs != nullptr) {
      const uint32_t qb = (uint32_t)p.pf_nchunks * (uint32_t)p.pf_wchunk, sb = (uint32_t)p.pf_nchunks * (uint32_t)p.pf_schunk;
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
  QENG_STAMP(1);
  const XLayout& Lz = L;
  // Work that does not depend on the kernel before: the zero region other blocks' lanes read (several
  // blocks per fragment), and the norm gains of this thread's groups, requested into L1 so that the
  // loads behind the reduction below find them there.
  if (kZeroed)
    for (uint32_t o = (uint32_t)tid * 16u; o < x_zero_bytes(Lz); o += kCT * 16u)
      asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};\n" ::"r"(xbase + Lz.zero + o), "r"(0u) : "memory");
  if (p.gamma != nullptr && p.ximage == nullptr)
    for (int k0 = tid * 8; k0 < p.K; k0 += kCT * 8) asm volatile("prefetch.global.L1 [%0];\n" ::"l"(p.gamma + k0));
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
  QENG_STAMP(2);
  QENG_REC(2);
  // tags of this call's pushes and gathers (the step counter is only stable behind the wait above)
  const unsigned tp_step = p.tp_seq != nullptr ? *p.tp_seq : 0u;
  const unsigned tag_push = tp_step * p.tp_tags_per_step + p.push_tag_off + 1u;
  const unsigned tag_gather = tp_step * p.tp_tags_per_step + p.gather_tag_off + 1u;
  Waits TW;
  (void)tag_gather;
  const bool vec_ok = p.x_dtype == QENG_F32 && ((reinterpret_cast<uintptr_t>(p.x) | (uintptr_t)(p.ldx * 4)) & 15) == 0 &&
                      (p.gamma == nullptr || (reinterpret_cast<uintptr_t>(p.gamma) & 15) == 0) && (p.K & 7) == 0;
  // eight consecutive activations of row m starting at k0 (zero beyond K)
  auto load8 = [&](int m, int k0, float (&dst)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) dst[i] = 0.f;
    if (k0 < p.K) {
      if (vec_ok) {
        const float4* xp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.x) + (long long)m * p.ldx + k0);
        const float4 a = xp[0], b = xp[1];
        dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
        dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (k0 + i < p.K) dst[i] = act_f32(p.x, p.x_dtype, (long long)m * p.ldx + k0 + i);
      }
    }
  };
  auto gamma8 = [&](int k0, float mul, float (&v)[8]) {
    if (p.gamma == nullptr || k0 >= p.K) return;
    if (vec_ok) {
      const float4* gp = reinterpret_cast<const float4*>(p.gamma + k0);
      const float4 a = gp[0], b = gp[1];
      v[0] *= a.x * mul; v[1] *= a.y * mul; v[2] *= a.z * mul; v[3] *= a.w * mul;
      v[4] *= b.x * mul; v[5] *= b.y * mul; v[6] *= b.z * mul; v[7] *= b.w * mul;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (k0 + i < p.K) v[i] *= p.gamma[k0 + i] * mul;
    }
  };
  // quantise the group at slice-local group index `grp` (block grp / 4, quad lane grp % 4) of row m
  auto put = [&](int m, int grp, const float (&v)[8], bool valid) {
    const uint32_t c0 = (uint32_t)(kLimbs * m);
    quantise_group<kLimbs>(v, valid, xbase + L.xq + c0 * L.col_stride, L.col_stride, xbase + L.zin + c0 * L.zs,
                           xbase + L.fex + c0 * L.zs, L.zs, (grp >> 2) * 32, grp & 3, KQ ? xbase + L.fsx + c0 * L.zs : 0u);
  };
  const int ngroups = L.nblk * 4;  // (block, quad lane) groups of the staged slice, padding included

  if (imaged) {
    // the first slice's image is requested now; later ones one slice ahead (see the main loop)
    if (tid == 0) {
      mbar_expect_tx(smem_u32(xbar), L.bytes);
      bulk_g2s(xbase, p.ximage, L.bytes, smem_u32(xbar));
    }
  } else if (p.nslices == 1) {
    // ---- whole K staged once; a thread keeps its groups in registers across the norm's reduction.
    // The raw values of row m + 1 are requested before row m is reduced and converted, so with
    // several activation rows only the first one waits for memory.
    float nv[kGroups][8];
    QENG_TICK(ts0);
#pragma unroll
    for (int j = 0; j < kGroups; ++j) load8(0, (tid + j * kCT) * 8, nv[j]);
#ifdef QENG_TRACE
    { float probe = nv[0][0]; asm volatile("" ::"f"(probe)); }  // the first value has arrived
    QENG_TOCK(ts0, 13, warp == 0);
#endif
    QENG_TICK(ts1);
    for (int m = 0; m < p.M; ++m) {
      float v[kGroups][8];
#pragma unroll
      for (int j = 0; j < kGroups; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j][i] = nv[j][i];
      if (m + 1 < p.M) {
#pragma unroll
        for (int j = 0; j < kGroups; ++j) load8(m + 1, (tid + j * kCT) * 8, nv[j]);
      }
      if (p.gather_world > 0) {
        // the ranks' parts of the residual update, added in rank order (the same bits on every rank)
#pragma unroll
        for (int j = 0; j < kGroups; ++j) {
          const int kk = (tid + j * kCT) * 8;
          if (kk < p.K) {
            for (int r = 0; r < p.gather_world; ++r) {
              float pt[8];
              poll8(p.gather_inbox + ((size_t)r * kTpFuseRows + m) * kTpFuseDm + kk, tag_gather, pt, TW, p.status);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[j][i] += pt[i];
            }
            if (blockIdx.x == 0) {
              float4* wp = reinterpret_cast<float4*>(p.x_writeback + (long long)m * p.ldx + kk);
              wp[0] = make_float4(v[j][0], v[j][1], v[j][2], v[j][3]);
              wp[1] = make_float4(v[j][4], v[j][5], v[j][6], v[j][7]);
            }
          }
        }
      }
      float rs = 1.f;
      if (p.gamma != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < kGroups; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) ss = fmaf(v[j][i], v[j][i], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float* wp = warp_part + (m & 1) * kCW;  // double-buffered: one barrier per row
        if (lane == 0) wp[warp] = ss;
        consumer_sync();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kCW; ++w) tot += wp[w];
        rs = rsqrtf(tot / (float)p.K + p.eps);
      }
      QENG_TOCK(ts1, 14, warp == 0);
      QENG_TICK(ts2);
#pragma unroll
      for (int j = 0; j < kGroups; ++j) {
        const int grp = tid + j * kCT;
        if ((grp & ~31) < ngroups) {  // whole warps take part (shuffles); ngroups is a multiple of 8
          gamma8(grp * 8, rs, v[j]);
          put(m, grp, v[j], grp < ngroups);
        }
      }
      QENG_TOCK(ts2, 15, warp == 0);
    }
  } else if (p.gamma != nullptr) {
    // ---- several slices: 1/rms of every row first (the slices are quantised as they come)
    for (int m = 0; m < p.M; ++m) {
      float ss = 0.f;
      for (int k0 = tid * 8; k0 < p.K; k0 += kCT * 8) {
        float v[8];
        load8(m, k0, v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      float* wp = warp_part + (m & 1) * kCW;
      if (lane == 0) wp[warp] = ss;
      consumer_sync();
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kCW; ++w) tot += wp[w];
      if (tid == 0) rinv[m] = rsqrtf(tot / (float)p.K + p.eps);
    }
  }
  consumer_sync();
  QENG_STAMP(3);
  QENG_REC(3);

  // ---- main loop: slices x this CTA's row tiles --------------------------------------------
  // The consumer warps form kTG independent groups that take the CTA's tiles in turn: while one
  // group reduces a tile and waits for its next stage, the other keeps the pipes busy.  Each group
  // owns NS / kTG consecutive ring slots and is the only waiter on their barriers, so a barrier's
  // phases are seen strictly in order however far the groups drift apart.
  const int gi = warp / kGW, wi = warp % kGW;
  bool failed = false;
  int tcount = 0, buf = 0, use = 0;

  // the fused epilogue of one row tile, run by one warp; total(a, r) = the finished sum for activation
  // row a and weight row r of the tile
  auto finish = [&](int tile, auto total) {
    if (p.epilogue == QENG_EPI_QKV) {
      const qeng_qkv_epi& E = p.qkv;
      const int head = tile >> 3, i = ((tile & 7) << 3);
      for (int e = lane; e < p.M * 8; e += 32) {
        const int a = e >> 3, r = e & 7;
        float lo = total(a, r), hi = total(a, r + 8);  // dims i+r and i+r+64 of this head
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
        const float gate = total(a, r), up = total(a, r + 8);
        p.y[(size_t)a * p.ldy + (size_t)tile * 8 + r] = gate / (1.0f + __expf(-gate)) * up;
      }
    } else if (p.push_world > 0) {
      // this rank's part of the residual update, tagged, into every rank's inbox (own included)
      for (int e = lane; e < p.M * 16; e += 32) {
        const int a = e >> 4, r = e & 15;
        const float v = total(a, r);
        const size_t o = ((size_t)p.push_rank * kTpFuseRows + a) * kTpFuseDm + (size_t)tile * 16 + r;
        for (int rr = 0; rr < p.push_world; ++rr) st_pair(p.push_inbox[(p.push_rank + rr) % p.push_world] + o, v, tag_push);
      }
    } else {
      for (int e = lane; e < p.M * 16; e += 32) {
        const int a = e >> 4, r = e & 15;
        float v = total(a, r);
        const size_t o = (size_t)a * p.ldy + (size_t)tile * 16 + r;
        if (p.epilogue == QENG_EPI_ACCUM) v += p.y[o];
        else if (p.epilogue == QENG_EPI_RESID) v += p.resid[o];
        p.y[o] = v;
      }
    }
  };
  // this lane's partial accumulators of a tile -> `dst` ([row a][16]) (one or two activation rows)
  auto park = [&](float* dst, float (&acc1)[2]) {
    if (MODE == kM1L3 || MODE == kM1L2) {
      acc1[0] += __shfl_xor_sync(0xffffffffu, acc1[0], 1);
      acc1[1] += __shfl_xor_sync(0xffffffffu, acc1[1], 1);
      acc1[0] += __shfl_xor_sync(0xffffffffu, acc1[0], 2);
      acc1[1] += __shfl_xor_sync(0xffffffffu, acc1[1], 2);
      if (t == 0) { dst[g] = acc1[0]; dst[g + 8] = acc1[1]; }
    } else {
      acc1[0] += __shfl_xor_sync(0xffffffffu, acc1[0], 1);
      acc1[1] += __shfl_xor_sync(0xffffffffu, acc1[1], 1);
      if ((t & 1) == 0) { dst[(t >> 1) * 16 + g] = acc1[0]; dst[(t >> 1) * 16 + g + 8] = acc1[1]; }
    }
  };

  if constexpr (kDefer) {
    // ---- one activation slice, up to two rows: no per-tile meeting -------------------------------
    int tl = 0, rot = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tl) {
      float acc1[2] = {0.f, 0.f};
      for (int c0 = 0; c0 < p.nchunks; c0 += p.stage_chunks, ++use) {
        const int s = use % NS;
        const uint32_t ph = (uint32_t)(use / NS) & 1u;
        QENG_TICK(tc0);
        if (!failed && !mbar_wait(smem_u32(full + s), ph)) failed = true;
        QENG_TOCK(tc0, 8, warp == 0);
        QENG_TICK(tc1);
        const int nc = min(p.stage_chunks, p.nchunks - c0);
        const uint32_t wb = smem_u32(ring) + (uint32_t)s * stage_bytes;
        const uint32_t sb = wb + (uint32_t)p.stage_chunks * kWChunk;
        const int blk0 = c0 * 2;
        // the warp that takes a stage's first item rotates, so that stages whose item count is not a
        // multiple of 16 load the warps evenly over a tile
        const int wr = (warp + kCW - rot) & (kCW - 1);
        if (MODE == kM1L3) consume_m1l3<kCW, Q8, KQ>(acc1, wb, sb, nc, blk0, L, xbase, wr, lane);
        else if (MODE == kM1L2) consume_g4<kCW, Q8, KQ>(acc1, wb, sb, nc, blk0, L, xbase, wr, lane);
        else consume_g2<kCW, Q8, KQ>(acc1, wb, sb, nc, blk0, L, xbase, wr, lane);
        rot = (rot + (MODE == kM1L2 ? (nc + 1) >> 1 : nc)) & (kCW - 1);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + s));
        QENG_TOCK(tc1, 9, warp == 0);
        QENG_COUNT(11, warp == 0);
      }
      QENG_TICK(tc2);
      const int slot = tl % kDeferTiles;
      park(red + ((size_t)slot * kCW + warp) * red_stride, acc1);
      const bool last_tile = tile + (int)gridDim.x >= p.ntiles;
      if (slot == kDeferTiles - 1 || last_tile) {
        consumer_sync();
        if (tl < kDeferTiles) QENG_STAMP(4);
        for (int j = warp; j <= slot; j += kCW) {
          const float* rb = red + (size_t)j * kCW * red_stride;
          finish(tile - (slot - j) * (int)gridDim.x, [&](int a, int r) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kCW; ++w) v += rb[w * red_stride + a * 16 + r];
            return v;
          });
        }
        if (!last_tile) consumer_sync();  // the parking area is free again
      }
      QENG_TOCK(tc2, 10, warp == 0);
    }
  } else {
  for (int sl = 0; sl < p.nslices; ++sl) {
    const int cs0 = sl * p.slice_chunks, cs1 = min(p.nchunks, cs0 + p.slice_chunks);
    uint32_t xb = xbase;  // this slice's staging area
    if (imaged) {
      if (sl > 0) consumer_sync();  // every warp is done with the slice before: its area may be refilled
      if (tid == 0 && sl + 1 < p.nslices) {
        const int nb = (sl + 1) & 1;
        mbar_expect_tx(smem_u32(xbar + nb), L.bytes);
        bulk_g2s(xbase + (uint32_t)nb * ximg_stride, p.ximage + (size_t)(sl + 1) * p.ximage_slice_bytes, L.bytes, smem_u32(xbar + nb));
      }
      xb = xbase + (uint32_t)(sl & 1) * ximg_stride;
      if (!failed && !mbar_wait(smem_u32(xbar + (sl & 1)), (uint32_t)(sl >> 1) & 1u)) failed = true;
    } else if (p.nslices > 1) {
      if (sl > 0) consumer_sync();  // every warp is done with the previous slice's activations
      for (int m = 0; m < p.M; ++m) {
        const float rs = p.gamma != nullptr ? rinv[m] : 1.f;
        for (int grp0 = 0; grp0 < ngroups; grp0 += kCT) {
          const int grp = grp0 + tid;
          if ((grp & ~31) < ngroups) {
            float v[8];
            const int k0 = cs0 * 64 + grp * 8;
            load8(m, grp < ngroups ? k0 : p.K, v);
            gamma8(k0, rs, v);
            put(m, grp, v, grp < ngroups);
          }
        }
      }
      consumer_sync();
    }
    int tl = 0;  // index of the tile among this CTA's tiles
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, ++tcount, ++tl) {
      if ((tcount % kTGe) != gi) continue;  // another group's tile
      float acc1[2] = {0.f, 0.f};
      float accn[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) accn[nt][0] = accn[nt][1] = 0.f;
      for (int c0 = cs0; c0 < cs1; c0 += p.stage_chunks, ++use) {
        const int s = gi * NSg + use % NSg;
        const uint32_t ph = (uint32_t)(use / NSg) & 1u;
        QENG_TICK(tc0);
        if (!failed && !mbar_wait(smem_u32(full + s), ph)) failed = true;
        QENG_TOCK(tc0, 8, warp == 0);
        QENG_TICK(tc1);
        const int nc = min(p.stage_chunks, cs1 - c0);
        const uint32_t wb = smem_u32(ring) + (uint32_t)s * stage_bytes;
        const uint32_t sb = wb + (uint32_t)p.stage_chunks * kWChunk;
        const int blk0 = (c0 - cs0) * 2;
        if (MODE == kM1L3) consume_m1l3<kGW, Q8, KQ>(acc1, wb, sb, nc, blk0, L, xb, wi, lane);
        else if (MODE == kM1L2) consume_g4<kGW, Q8, KQ>(acc1, wb, sb, nc, blk0, L, xb, wi, lane);
        else if (MODE == kM2L2) consume_g2<kGW, Q8, KQ>(acc1, wb, sb, nc, blk0, L, xb, wi, lane);
        else consume_g1<kGW, NT, Q8, KQ>(accn, wb, sb, nc, blk0, L, xb, p.cols, wi, lane);
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(empty + s));  // this warp is done with the stage
        QENG_TOCK(tc1, 9, warp == 0);
        QENG_COUNT(11, warp == 0);
      }
      QENG_TICK(tc2);

      // ---- the partial accumulators of the group's warps meet in shared memory ------------------
      // red[group][buf][warp][row m][16]; the reader of buffer `buf` finishes before it arrives at
      // the next tile's barrier, and buffer `buf` is written again only after that barrier
      float* myred = red + (((size_t)gi * 2 + buf) * kGW + wi) * red_stride;
      if (MODE != kMN) {
        park(myred, acc1);
      } else {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          myred[(nt * 4 + t) * 16 + g] = accn[nt][0];
          myred[(nt * 4 + t) * 16 + g + 8] = accn[nt][1];
        }
      }
      group_sync<kGW>(gi);
      if (tcount == 0) QENG_STAMP(4);
      if (wi == ((tcount / kTGe) % kGW)) {
        const float* rb = red + ((size_t)gi * 2 + buf) * kGW * red_stride;
        float* at = accsm + (size_t)tl * red_stride;
        const bool first = sl == 0, last = sl + 1 == p.nslices;
        // sum of the group's warps for activation row a, weight row r of the tile (plus earlier slices)
        auto total = [&](int a, int r) {
          float v = 0.f;
#pragma unroll
          for (int w = 0; w < kGW; ++w) v += rb[w * red_stride + a * 16 + r];
          if (!first) v += at[a * 16 + r];
          return v;
        };
        if (!last) {
          for (int e = lane; e < p.M * 16; e += 32) at[e] = total(e >> 4, e & 15);
        } else {
          finish(tile, total);
        }
      }
      buf ^= 1;
      QENG_TOCK(tc2, 10, warp == 0);
    }
  }
  }
  QENG_STAMP(5);
  QENG_REC(4);
#ifdef QENG_TRACE
  if (rec) { rec[5] = (unsigned long long)tacc[5]; rec[6] = (unsigned long long)tacc[6]; rec[7] = (unsigned long long)tacc[7]; }
#endif
  QENG_FLUSH(13, warp == 0); QENG_FLUSH(14, warp == 0); QENG_FLUSH(15, warp == 0);
  QENG_FLUSH(8, warp == 0); QENG_FLUSH(9, warp == 0); QENG_FLUSH(10, warp == 0); QENG_FLUSH(11, warp == 0);
  if (failed && lane == 0) atomicExch(p.status, 4);
}

template <int MODE, int NT, int kTG, bool Q8 = false, bool KQ = false>
int32_t launch_stream(qeng_ctx* ctx, const StreamParams& p, size_t smem, cudaStream_t stream) {
  static bool configured_on[64] = {};  // the opt-in shared-memory size is set per device
  bool& configured = configured_on[ctx->device & 63];
  if (!configured) {
    QENG_CUDA(ctx, cudaFuncSetAttribute(gemv_q4_stream_kernel<MODE, NT, kTG, Q8, KQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024));
    configured = true;
  }
  const int grid = p.ntiles < ctx->sm_count ? p.ntiles : ctx->sm_count;
  // programmatic stream serialization: this kernel may become resident while its predecessor is still
  // running; everything that depends on the predecessor sits behind griddepcontrol.wait
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(kCT + 32 * (kTG == 0 ? 1 : kTG));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = ctx->pdl ? 1 : 0;
  QENG_CUDA(ctx, cudaLaunchKernelEx(&cfg, gemv_q4_stream_kernel<MODE, NT, kTG, Q8, KQ>, p));
  return QENG_OK;
}

struct StreamFit {
  bool ok;
  int mode, NT, cols, nstages, stage_chunks, slice_chunks, nslices;
  bool imaged;
  bool defer;  // all 16 warps on every tile, the per-tile reduction deferred (kTG = 0)
  uint32_t image_slice_bytes;
  size_t smem;
};

// Shared-memory plan for a shape: the staged activations (whole K for up to 4 rows, else the
// largest K slice that leaves the ring at least ~100 KB), reduction buffers, then as many ring
// slots as fit.
StreamFit stream_fit(const qeng_ctx* ctx, const qeng_weight* w, int64_t M, bool two_limbs) {
  StreamFit f = {};
  if (M < 1 || M > 16) return f;
  const bool kq = w->fmt == QENG_FMT_K4;
  if (kq && M > 4) return f;  // 4-bit blocks with minima: up to 4 rows per pass (no activation images)
  f.mode = M == 1 ? (two_limbs ? kM1L2 : kM1L3) : (M == 2 ? kM2L2 : kMN);
  f.cols = f.mode == kM1L3 ? 3 : 2 * (int)M;
  f.NT = f.mode == kMN ? (int)((M + 3) / 4) : 1;
  const int kMR = f.mode == kMN ? 4 * f.NT : (f.mode == kM2L2 ? 2 : 1);
  const int nch = (int)w->nchunks;
  const int sms = ctx->sm_count > 0 ? ctx->sm_count : 148;
  const int grid = w->ntiles < sms ? (int)w->ntiles : sms;
  const int tiles_per_cta = (int)((w->ntiles + grid - 1) / grid);
  const size_t budget = 226 * 1024 - 1024;
  const size_t bars = 2 * kMaxStages * 8;
  f.imaged = M > 4;  // quantised once by a small kernel, copied in per slice
  auto plan = [&](int slice) -> bool {
    const int nsl = (nch + slice - 1) / slice;
    if (!f.imaged && nsl == 1 && nch * 64 > 8 * kGroups * kCT) return false;  // single-slice staging goes through registers: K <= 12288
    const int alloc = f.mode == kM1L2 ? (slice + 1) & ~1 : slice;
    const XLayout L = x_layout(f.cols, alloc, f.mode != kMN, 0, kq);
    f.defer = f.mode != kMN && nsl == 1 && (ctx->stream_groups == 0 || w->fmt != QENG_FMT_Q4);
    const size_t red = (size_t)(f.defer ? kDeferTiles : 2) * kCW * kMR * 16 * 4;  // grouped: the same for every number of groups
    const size_t accs = nsl > 1 ? (size_t)tiles_per_cta * kMR * 16 * 4 : 0;
    const size_t xarea = f.imaged ? 2 * (((size_t)L.bytes + 127) & ~(size_t)127) : L.bytes;
    const size_t fixed = xarea + red + accs + bars + 256;
    f.image_slice_bytes = (L.bytes + 127u) & ~127u;
    const int cap = ctx->stream_stage_chunks > 0 ? ctx->stream_stage_chunks : kStageChunks;
    const int sc = slice < cap ? slice : cap;
    const size_t slot = (size_t)sc * (w->fmt == QENG_FMT_Q8 ? 1088 : (kq ? 768 : 576));
    if (fixed + 2 * slot > budget) return false;
    int ns = (int)((budget - fixed) / slot);
    if (ns > kMaxStages) ns = kMaxStages;
    if ((size_t)ns * slot < (size_t)96 * 1024 && slice > 8) return false;  // too little in flight: stage a smaller K slice
    f.nstages = ns; f.stage_chunks = sc; f.slice_chunks = slice; f.nslices = nsl;
    f.smem = (((size_t)ns * slot + 127) & ~(size_t)127) + fixed;
    return true;
  };
  if (plan(nch)) { f.ok = true; return f; }  // the whole K range staged once
  for (int slice = 64; slice >= 8; slice >>= 1)
    if (slice < nch && plan(slice)) { f.ok = true; return f; }
  return f;
}
}  // namespace

bool qeng_gemm_q4_stream_fits(const qeng_ctx* ctx, const qeng_weight* w, int64_t M) { return stream_fit(ctx, w, M, false).ok; }

// Grow the context's activation-image scratch to what a matmul of M rows over `w` needs (never
// inside a stream capture: the decoder calls this before it captures a step).
int32_t qeng_gemm_q4_stream_reserve(qeng_ctx* ctx, const qeng_weight* w, int64_t M) {
  const StreamFit f = stream_fit(ctx, w, M, false);
  if (!f.ok || !f.imaged) return QENG_OK;
  const size_t need = (size_t)f.nslices * f.image_slice_bytes;
  if (need <= ctx->ximage_bytes) return QENG_OK;
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  QENG_CUDA(ctx, cudaDeviceSynchronize());
  if (ctx->ximage) cudaFree(ctx->ximage);
  ctx->ximage = nullptr;
  ctx->ximage_bytes = 0;
  QENG_CUDA(ctx, cudaMalloc(&ctx->ximage, need));
  ctx->ximage_bytes = need;
  ctx->scratch_gen++;
  return QENG_OK;
}

// *handled = false when the shape does not fit this kernel; the caller then uses the
// register-streaming kernel.
int32_t qeng_gemm_q4_stream(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M,
                            int64_t ldx, float* y, int64_t ldy, const qeng_gemm_fuse& fuse, cudaStream_t stream,
                            bool* handled) {
  *handled = false;
  const StreamFit f = stream_fit(ctx, w, M, fuse.two_limbs);
  if (!f.ok) {
    if (fuse.epilogue == QENG_EPI_QKV) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4: the fused q|k|v epilogue needs the streaming kernel");
    return QENG_OK;
  }
  StreamParams p;
  p.qs = w->qs; p.sc = w->sc;
  p.ntiles = (int)w->ntiles; p.nchunks = (int)w->nchunks; p.K = (int)w->K;
  p.x = x; p.x_dtype = x_dtype; p.ldx = ldx; p.M = (int)M; p.cols = f.cols;
  p.y = y; p.ldy = ldy;
  p.gamma = fuse.norm_gamma; p.eps = fuse.norm_eps; p.epilogue = fuse.epilogue; p.resid = fuse.resid;
  p.nstages = f.nstages; p.stage_chunks = f.stage_chunks; p.slice_chunks = f.slice_chunks; p.nslices = f.nslices;
  p.status = ctx->status;
  const qeng_weight* nx = ctx->l2_prefetch ? w->next : nullptr;
  p.pf_qs = nx ? nx->qs : nullptr; p.pf_sc = nx ? nx->sc : nullptr;
  p.pf_ntiles = nx ? (int)nx->ntiles : 0; p.pf_nchunks = nx ? (int)nx->nchunks : 0;
  p.pf_wchunk = nx && nx->fmt == QENG_FMT_Q8 ? 1024 : 512;
  p.pf_schunk = nx && nx->fmt == QENG_FMT_K4 ? 256 : 64;
  p.qkv = qeng_qkv_epi();
  if (fuse.epilogue == QENG_EPI_QKV) {
    if (!fuse.qkv) return qeng_fail(ctx, QENG_ERR_ARG, "gemm_q4: fused q|k|v epilogue without its arguments");
    p.qkv = *fuse.qkv;
  }
  p.push_world = 0; p.gather_world = 0; p.gather_inbox = nullptr; p.x_writeback = nullptr; p.tp_seq = nullptr;
  p.push_rank = ctx->tp_rank; p.tp_tags_per_step = 2u * (unsigned)fuse.tp_layers; p.push_tag_off = 0; p.gather_tag_off = 0;
  for (int r = 0; r < 8; ++r) p.push_inbox[r] = nullptr;
  if (fuse.tp_push_kind >= 0 || fuse.tp_gather_kind >= 0) {
    if (!qeng_tp_fuse_ready(ctx, M, fuse.tp_push_kind >= 0 ? w->N : w->K) || x_dtype != QENG_F32 || (ldx & 3) != 0)
      return qeng_fail(ctx, QENG_ERR_STATE, "gemm_q4: the fused tensor-parallel forms need mapped peers, f32 rows and at most %d rows", kTpFuseRows);
    p.tp_seq = qeng_tp_fuse_seq(ctx);
    if (fuse.tp_push_kind >= 0) {
      p.push_world = ctx->tp_world;
      for (int r = 0; r < ctx->tp_world; ++r) p.push_inbox[r] = qeng_tp_fuse_inbox(ctx, r, fuse.tp_push_kind);
      p.push_tag_off = 2u * (unsigned)fuse.tp_layer + (unsigned)fuse.tp_push_kind;
    }
    if (fuse.tp_gather_kind >= 0) {
      p.gather_world = ctx->tp_world;
      p.gather_inbox = qeng_tp_fuse_inbox(ctx, ctx->tp_rank, fuse.tp_gather_kind);
      p.gather_tag_off = 2u * (unsigned)fuse.tp_gather_layer + (unsigned)fuse.tp_gather_kind;
      if (!fuse.tp_writeback || fuse.tp_writeback == x) return qeng_fail(ctx, QENG_ERR_ARG, "gemm_q4: a gather needs a write-back buffer other than x");
      p.x_writeback = fuse.tp_writeback;
    }
  }
  p.ximage = nullptr; p.ximage_slice_bytes = f.image_slice_bytes;
  if (f.imaged) {
    int32_t rr = qeng_gemm_q4_stream_reserve(ctx, w, M);  // grows outside the steady state only
    if (rr != QENG_OK) return rr;
    const XLayout L = x_layout(f.cols, f.slice_chunks, false);
    const size_t qsmem = 2 * (size_t)L.col_stride + 4 * (size_t)L.zs + (p.gather_world > 0 ? (size_t)w->K * 4 : 0);
    static bool qconf[64] = {};
    if (!qconf[ctx->device & 63]) {
      QENG_CUDA(ctx, cudaFuncSetAttribute(quantise_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
      qconf[ctx->device & 63] = true;
    }
    if (qsmem > 64 * 1024) return qeng_fail(ctx, QENG_ERR_SHAPE, "gemm_q4: K slice too wide for the activation quantiser");
    cudaLaunchConfig_t qc = {};
    qc.gridDim = dim3((unsigned)f.nslices, (unsigned)M);
    qc.blockDim = dim3(512);
    qc.dynamicSmemBytes = qsmem;
    qc.stream = stream;
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    qa[0].val.programmaticStreamSerializationAllowed = 1;
    qc.attrs = qa;
    qc.numAttrs = ctx->pdl ? 1 : 0;
    QENG_CUDA(ctx, cudaLaunchKernelEx(&qc, quantise_rows_kernel, x, (int)x_dtype, (long long)ldx, (int)M, (int)w->K, fuse.norm_gamma,
                                      fuse.norm_eps, f.slice_chunks, reinterpret_cast<unsigned char*>(ctx->ximage), f.image_slice_bytes,
                                      p.gather_inbox, p.gather_world, p.tp_seq, p.tp_tags_per_step, p.gather_tag_off, p.x_writeback,
                                      ctx->status));
    // the main kernel then sees completed activations: its own staging gathers nothing
    p.gather_world = 0;
    p.ximage = reinterpret_cast<const unsigned char*>(ctx->ximage);
  }
  *handled = true;
  // Tile groups: more groups hide more of the per-tile reduction, but a group with no tile idles,
  // so the split follows the number of tiles a CTA owns.
  const int grid = p.ntiles < ctx->sm_count ? p.ntiles : ctx->sm_count;
  const int per_cta = (p.ntiles + grid - 1) / grid;
  // (a tile worked on by 4 warps takes ~1.8 us, by 8 warps ~0.9: with only two tiles per CTA two groups of
  // 8 warps finish sooner than two of four groups of 4)
  int tg = per_cta >= 3 ? 4 : (per_cta == 2 ? 2 : 1);
  // a group needs a ring of its own at least as long as one row tile
  const int spt = (f.slice_chunks + f.stage_chunks - 1) / f.stage_chunks;
  while (tg > 1 && f.nstages / tg < spt) tg >>= 1;
  if (ctx->stream_groups == 1 || ctx->stream_groups == 2 || ctx->stream_groups == 4) tg = ctx->stream_groups;
  while (tg > 1 && f.nstages / tg < 1) tg >>= 1;
#define QENG_STREAM_CASE(MODE_, NT_)                                                   \
  (tg == 4 ? launch_stream<MODE_, NT_, 4>(ctx, p, f.smem, stream)                      \
           : (tg == 2 ? launch_stream<MODE_, NT_, 2>(ctx, p, f.smem, stream) : launch_stream<MODE_, NT_, 1>(ctx, p, f.smem, stream)))
  if (w->fmt == QENG_FMT_K4) {  // 4-bit blocks with per-block scale and minimum: the deferred forms, or one tile group
    if (f.defer) {
      if (f.mode == kM1L3) return launch_stream<kM1L3, 1, 0, false, true>(ctx, p, f.smem, stream);
      if (f.mode == kM1L2) return launch_stream<kM1L2, 1, 0, false, true>(ctx, p, f.smem, stream);
      return launch_stream<kM2L2, 1, 0, false, true>(ctx, p, f.smem, stream);
    }
    if (f.mode == kM1L3) return launch_stream<kM1L3, 1, 1, false, true>(ctx, p, f.smem, stream);
    if (f.mode == kM1L2) return launch_stream<kM1L2, 1, 1, false, true>(ctx, p, f.smem, stream);
    if (f.mode == kM2L2) return launch_stream<kM2L2, 1, 1, false, true>(ctx, p, f.smem, stream);
    return launch_stream<kMN, 1, 1, false, true>(ctx, p, f.smem, stream);  // 3 or 4 rows
  }
  if (w->fmt == QENG_FMT_Q8) {  // 8-bit blocks: the deferred forms, or one tile group
    if (f.defer) {
      if (f.mode == kM1L3) return launch_stream<kM1L3, 1, 0, true>(ctx, p, f.smem, stream);
      if (f.mode == kM1L2) return launch_stream<kM1L2, 1, 0, true>(ctx, p, f.smem, stream);
      return launch_stream<kM2L2, 1, 0, true>(ctx, p, f.smem, stream);
    }
    if (f.mode == kM1L3) return launch_stream<kM1L3, 1, 1, true>(ctx, p, f.smem, stream);
    if (f.mode == kM1L2) return launch_stream<kM1L2, 1, 1, true>(ctx, p, f.smem, stream);
    if (f.mode == kM2L2) return launch_stream<kM2L2, 1, 1, true>(ctx, p, f.smem, stream);
    switch (f.NT) {
      case 1: return launch_stream<kMN, 1, 1, true>(ctx, p, f.smem, stream);
      case 2: return launch_stream<kMN, 2, 1, true>(ctx, p, f.smem, stream);
      case 3: return launch_stream<kMN, 3, 1, true>(ctx, p, f.smem, stream);
      default: return launch_stream<kMN, 4, 1, true>(ctx, p, f.smem, stream);
    }
  }
  if (f.defer) {
    if (f.mode == kM1L3) return launch_stream<kM1L3, 1, 0>(ctx, p, f.smem, stream);
    if (f.mode == kM1L2) return launch_stream<kM1L2, 1, 0>(ctx, p, f.smem, stream);
    return launch_stream<kM2L2, 1, 0>(ctx, p, f.smem, stream);
  }
  if (f.mode == kM1L3) return QENG_STREAM_CASE(kM1L3, 1);
  if (f.mode == kM1L2) return QENG_STREAM_CASE(kM1L2, 1);
  if (f.mode == kM2L2) return QENG_STREAM_CASE(kM2L2, 1);
  switch (f.NT) {
    case 1: return QENG_STREAM_CASE(kMN, 1);
    case 2: return QENG_STREAM_CASE(kMN, 2);
    case 3: return QENG_STREAM_CASE(kMN, 3);
    default: return QENG_STREAM_CASE(kMN, 4);
  }
#undef QENG_STREAM_CASE
}
