// The layer executor: runs the decode loop
//   embed -> per layer: norm, QKV, RoPE, KV append, attention, O proj (+residual),
//            norm, gate/up (+SwiGLU), down (+residual) -> norm -> LM head -> greedy sample
// over the kernels of this library.  One decode step is captured once into a
// CUDA graph and replayed; positions, lengths and the sampled tokens live on the
// device so that no host work sits between two steps.
//
// Fusions: RMSNorm into the activation staging of the following matmul, the
// residual add and SwiGLU into the matmul epilogues, RoPE + f16 rounding + KV
// append + q conversion into one small kernel.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "qeng_internal.h"

namespace {

constexpr int kHD = 128;
constexpr int kPage = 16;

struct HostMat {
  int fmt = QENG_FMT_Q4;
  int su = 1;  // 16-bit words of scale data per 32-block: 1 (an f16 scale) or 4 (f32 scale and minimum)
  std::vector<uint8_t> q;
  std::vector<uint16_t> s;
  int64_t N = 0, K = 0;
};

struct Layer {
  qeng_weight* wqkv = nullptr;
  qeng_weight* wo = nullptr;
  qeng_weight* wgu = nullptr;  // gate/up rows interleaved 8/8 per 16-row tile
  qeng_weight* wdown = nullptr;
  float* norm1 = nullptr;
  float* norm2 = nullptr;
  float *qnorm = nullptr, *knorm = nullptr;  // optional per-head gains [128] (QK-norm)
  HostMat pend[7];  // host shards waiting for their fusion partners
};

// rows of q|k|v (f32, straight from the QKV matmul) -> rotated q as f16, rotated k and v
// as f16 into the page pool at token index pos[row].  One warp per head; with per-head gains
// (qg, kg: the "QK-norm" of the Qwen3 family, decide/model-lifecycle.md:173-176) every q and k
// head is RMS-normalised over its 128 dims before the rotation.
__global__ void __launch_bounds__(256) rope_append_kernel(const float* __restrict__ qkv, const float* __restrict__ cs,
                                                          const int32_t* __restrict__ pos,
                                                          const int32_t* __restrict__ table, int max_pages, int pages,
                                                          int Hq, int Hkv, int max_seq, __half* __restrict__ q16,
                                                          __half* __restrict__ pool, int32_t* status,
                                                          const float* __restrict__ qg, const float* __restrict__ kg,
                                                          float eps) {
  const int row = blockIdx.x;
  const int ps = pos[row];
  if (ps < 0 || ps >= max_seq || (ps >> 4) >= max_pages) {
    if (threadIdx.x == 0) atomicExch(status, 2);
    return;
  }
  const int pid = table[(size_t)row * max_pages + (ps >> 4)];
  if ((unsigned)pid >= (unsigned)pages) {
    if (threadIdx.x == 0) atomicExch(status, 1);
    return;
  }
  const int nq = Hq * kHD, nkv = Hkv * kHD;
  const float* src = qkv + (size_t)row * (nq + 2 * nkv);
  const float* cosr = cs + (size_t)ps * kHD;  // [64 cos | 64 sin]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // rotated heads: Hq query heads then Hkv key heads; a lane owns the pairs (i, i+64), i = lane, lane+32
  for (int h = warp; h < Hq + Hkv; h += 8) {
    const float* gain = h < Hq ? qg : kg;
    float a[2], b[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = lane + 32 * u;
      // the q|k|v rows of a head are stored permuted: dim i sits at 16*((i&63)>>3) + (i&7) + 8*(i>>6)
      const int pi = ((i >> 3) << 4) + (i & 7);
      a[u] = src[h * kHD + pi];
      b[u] = src[h * kHD + pi + 8];
    }
    if (gain != nullptr) {
      float ss = a[0] * a[0] + b[0] * b[0] + a[1] * a[1] + b[1] * b[1];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float r = rsqrtf(ss / (float)kHD + eps);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = lane + 32 * u;
        a[u] = a[u] * r * gain[i];
        b[u] = b[u] * r * gain[i + 64];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = lane + 32 * u;
      const float c = cosr[i], s = cosr[64 + i];
      const __half lo = __float2half_rn(a[u] * c - b[u] * s), hi = __float2half_rn(b[u] * c + a[u] * s);
      if (h < Hq) {
        q16[(size_t)row * nq + h * kHD + i] = lo;
        q16[(size_t)row * nq + h * kHD + i + 64] = hi;
      } else {
        __half* kd = pool + ((size_t)pid * Hkv + (h - Hq)) * (2 * kPage * kHD) + (ps & 15) * kHD;
        kd[i] = lo;
        kd[i + 64] = hi;
      }
    }
  }
  for (int idx = threadIdx.x; idx < nkv; idx += blockDim.x) {
    const int h = idx >> 7, i = idx & 127;
    const int pi = (((i & 63) >> 3) << 4) + (i & 7) + ((i >> 6) << 3);
    pool[((size_t)pid * Hkv + h) * (2 * kPage * kHD) + kPage * kHD + (ps & 15) * kHD + i] =
        __float2half_rn(src[nq + nkv + h * kHD + pi]);
  }
}

// Unfused end of a decode step (batches the fused LM head does not take): record the sampled
// tokens as entry step+1, move every sequence one token on.
__global__ void advance_kernel(const int32_t* __restrict__ next, int32_t* pos, int32_t* lens, int32_t* out_tokens,
                               int32_t* step, int B) {
  const int b = threadIdx.x;
  const int st = *step;
  __syncthreads();
  if (b < B) {
    out_tokens[(size_t)(st + 1) * B + b] = next[b];
    pos[b] += 1;
    lens[b] += 1;
  }
  if (b == 0) *step = st + 1;
}

// Start of a decode call: the token sampled from the logits already present is entry 0.
__global__ void record_first_kernel(const int32_t* __restrict__ next, int32_t* out_tokens, int B) {
  if ((int)threadIdx.x < B) out_tokens[threadIdx.x] = next[threadIdx.x];
}

// Sharded LM head, last step: gathered[r][m] = (max logit, its global index) of rank r.  Pick the
// token (largest value, lowest index on ties, as the unsharded argmax does), record it, advance
// the sequences, gather the next embedding, and clear the gather buffer for the next step.
__global__ void __launch_bounds__(256) tp_pick_kernel(float* gathered, int world, int B, int V, int D,
                                                      const uint16_t* __restrict__ emb, float* __restrict__ xout,
                                                      int32_t* next, int32_t* pos, int32_t* lens, int32_t* out_tokens,
                                                      int32_t* step, int32_t* status) {
  __shared__ int tok[16];
  const int tid = threadIdx.x;
  if (tid < B) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < world; ++r) {
      const float v = gathered[2 * (r * B + tid)];
      const float fi = gathered[2 * (r * B + tid) + 1];
      const int i = fi >= 0.f && fi < 16777216.f ? (int)fi : 0x7fffffff;
      if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    if ((unsigned)bi >= (unsigned)V) { bi = 0; atomicExch(status, 3); }  // only if every logit was NaN
    tok[tid] = bi;
    next[tid] = bi;
    out_tokens[(size_t)(*step + 1) * B + tid] = bi;
    pos[tid] += 1;
    lens[tid] += 1;
  }
  __syncthreads();
  if (tid == 0) *step += 1;
  for (int i = tid; i < 2 * world * B; i += 256) gathered[i] = 0.f;
  for (int m = 0; m < B; ++m)
    for (int i = tid; i < D; i += 256)
      xout[(size_t)m * D + i] = __uint_as_float((uint32_t)emb[(size_t)tok[m] * D + i] << 16);
}

}  // namespace

struct qeng_decoder {
  qeng_model_cfg cfg;
  int Hq = 0, Hkv = 0, F = 0;  // local (per rank) head counts and FFN width
  int nqkv = 0;
  int max_pages = 0;           // pages per sequence
  int64_t pages = 0;           // pages per layer pool
  std::vector<Layer> layers;
  uint16_t* emb = nullptr;
  uint16_t* lm_head = nullptr;
  float* final_norm = nullptr;
  float* rope_cs = nullptr;    // [max_seq][64 cos | 64 sin]
  __half* pool = nullptr;      // [layers][pages][Hkv][2][16][128]
  qeng_kv_pool view;           // per-layer view handed to the attention entry point
  // activations (rows = batch in decode, batch*T in prefill)
  int64_t rows_cap = 0;
  float *x = nullptr, *qkv = nullptr, *att = nullptr, *act = nullptr, *part = nullptr;
  float* xalt = nullptr;  // second residual buffer: a fused tensor-parallel gather reads one and writes the other
  float *xnr = nullptr, *gu = nullptr;  // prefill only: normalised rows, gate|up before SwiGLU
  __half* q16 = nullptr;
  int32_t *pos = nullptr, *lens = nullptr, *table = nullptr, *tok = nullptr;  // per row
  // decode state
  float *xn = nullptr, *xlast = nullptr, *logits = nullptr;
  int32_t *next = nullptr, *out_tokens = nullptr, *step = nullptr, *dec_table = nullptr;
  int max_steps = 0;
  int32_t* h_out = nullptr;  // pinned: the tokens of a decode call, then the status word (one synchronisation per call)
  int batch = 0;
  std::vector<int32_t> len;  // host copy of sequence lengths
  bool have_logits = false;
  // tensor parallelism: the LM head is split by vocabulary rows [v0, v0 + vloc); every rank's
  // (max, index) pair per sequence is summed into `tp_gath` (the other ranks' slots of `tp_pairs`
  // stay zero, so the sum is a gather) and one small kernel picks the token
  bool vsplit = false;
  int v0 = 0, vloc = 0;
  float *tp_pairs = nullptr, *tp_gath = nullptr;  // [world][max_batch][2]
  bool next_ready = false;      // the last operation was a decode step: `next` holds the sampled token, `x` its embedding
  bool logits_partial = false;  // after a sharded decode step only columns [v0, v0 + vloc) are current
  cudaStream_t stream = nullptr;
  cudaStream_t own_stream = nullptr;
  cudaGraphExec_t graph = nullptr;
  int graph_batch = 0;
  uint64_t graph_scratch_gen = 0;  // ctx->scratch_gen at capture time
  // the fused decode step (all layers in one persistent kernel), planned lazily; dropped whenever a
  // buffer or weight it points at is replaced
  qeng_step* fused = nullptr;
  bool step_planned = false;
  int launches = 0;
};

namespace {

// Prompt rows go through the decode attention kernel one "sequence" per row, at most this many
// per launch (bounds its grid, its arrival counters and its split scratch).
constexpr int64_t kAttnRowsPerCall = 2048;

// Grow the per-row buffers.  A captured decode step holds their addresses, so it is dropped here
// and captured again by the next decode call.
int32_t ensure_rows(qeng_ctx* ctx, qeng_decoder* d, int64_t rows) {
  if (rows <= d->rows_cap) return QENG_OK;
  QENG_CUDA(ctx, cudaDeviceSynchronize());
  if (d->graph) { cudaGraphExecDestroy(d->graph); d->graph = nullptr; }
  qeng_step_free(d->fused); d->fused = nullptr; d->step_planned = false;
  float** fb[] = {&d->x, &d->xalt, &d->qkv, &d->att, &d->act, &d->part, &d->xnr, &d->gu};
  for (auto p : fb)
    if (*p) { cudaFree(*p); *p = nullptr; }
  if (d->q16) { cudaFree(d->q16); d->q16 = nullptr; }
  int32_t** ib[] = {&d->pos, &d->lens, &d->table, &d->tok};
  for (auto p : ib)
    if (*p) { cudaFree(*p); *p = nullptr; }
  d->rows_cap = 0;
  const int64_t dm = d->cfg.d_model;
  QENG_CUDA(ctx, cudaMalloc(&d->x, rows * dm * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->xalt, rows * dm * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->qkv, rows * d->nqkv * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->att, rows * d->Hq * kHD * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->act, rows * d->F * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->part, rows * dm * 4));
  if (rows >= kPrefillRows) {
    QENG_CUDA(ctx, cudaMalloc(&d->xnr, rows * dm * 4));
    QENG_CUDA(ctx, cudaMalloc(&d->gu, rows * 2 * d->F * 4));
  }
  QENG_CUDA(ctx, cudaMalloc(&d->q16, rows * d->Hq * kHD * 2));
  QENG_CUDA(ctx, cudaMalloc(&d->pos, rows * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->lens, rows * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->table, rows * d->max_pages * 4));
  QENG_CUDA(ctx, cudaMalloc(&d->tok, rows * 4));
  d->rows_cap = rows;
  return qeng_attn_reserve(ctx, rows < kAttnRowsPerCall ? rows : kAttnRowsPerCall, d->Hq, d->Hkv, d->max_pages);
}

// matmul over `rows` activation rows in chunks the decode kernels accept: the largest row count
// whose staged activations still fit the streaming kernel's shared memory (the weights are
// streamed once per chunk), else 16 rows on the register-streaming kernel
int32_t mm(qeng_ctx* ctx, qeng_decoder* d, const qeng_weight* w, const float* x, int64_t ldx, int64_t rows, float* y,
           int64_t ldy, const qeng_gemm_fuse& fuse, cudaStream_t st) {
  int64_t chunk = 16;
  for (int64_t c = 16; c >= 1; c >>= 1)
    if (qeng_gemm_q4_stream_fits(ctx, w, c)) { chunk = c; break; }
  for (int64_t m0 = 0; m0 < rows; m0 += chunk) {
    const int64_t mm_ = rows - m0 < chunk ? rows - m0 : chunk;
    qeng_gemm_fuse f = fuse;
    if (f.resid) f.resid = fuse.resid + m0 * ldy;
    qeng_qkv_epi E;
    if (f.qkv) {  // the fused q|k|v epilogue addresses its outputs by activation row
      E = *fuse.qkv;
      E.pos += m0;
      E.table += m0 * E.max_pages;
      E.q16 += m0 * E.Hq * kHD;
      f.qkv = &E;
    }
    int32_t rc = qeng_gemm_q4_decode(ctx, w, x + m0 * ldx, QENG_F32, mm_, ldx, y + m0 * ldy, ldy, true, f, st);
    if (rc != QENG_OK) return rc;
    d->launches++;
  }
  return QENG_OK;
}

// Row-split projection: x += in . W^T summed over the ranks.  One rank: the residual add is the
// matmul's epilogue.  Several ranks: partial sums, all-reduce over NVLink, then the add.
__global__ void add_inplace_kernel(float* __restrict__ x, const float* __restrict__ p, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += p[i];
}

int32_t row_split(qeng_ctx* ctx, qeng_decoder* d, const qeng_weight* w, const float* in, int64_t ldin, int64_t rows,
                  cudaStream_t st) {
  const int64_t dm = d->cfg.d_model;
  qeng_gemm_fuse f;
  f.two_limbs = true;  // 15-bit activations: only the q|k|v projection, which feeds the softmax, keeps 22
  if (d->cfg.tp_world == 1) {
    f.epilogue = QENG_EPI_ACCUM;
    return mm(ctx, d, w, in, ldin, rows, d->x, dm, f, st);
  }
  f.epilogue = QENG_EPI_STORE;
  int32_t rc = mm(ctx, d, w, in, ldin, rows, d->part, dm, f, st);
  if (rc != QENG_OK) return rc;
  const int64_t n = rows * dm;
  if (qeng_tp_p2p_ready(ctx, n)) {  // push, wait, sum and residual add in one kernel
    d->launches += 1;
    return qeng_tp_allreduce_add(ctx, d->x, d->part, n, st);
  }
  rc = qeng_tp_all_reduce_internal(ctx, d->part, n, st);
  if (rc != QENG_OK) return rc;
  add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(d->x, d->part, n);
  QENG_LAUNCH_CHECK(ctx);
  d->launches += 2;
  return QENG_OK;
}

// gate|up rows are interleaved 8/8 per 16-row tile: act[m][8j + r] = silu(gu[m][16j + r]) * gu[m][16j + r + 8]
__global__ void swiglu_interleaved_kernel(const float* __restrict__ gu, int64_t rows, int F, float* __restrict__ act) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * F) return;
  const int64_t m = i / F;
  const int c = (int)(i - m * F);
  const float* src = gu + m * 2 * F + (c >> 3) * 16 + (c & 7);
  const float g = src[0];
  act[i] = g / (1.0f + __expf(-g)) * src[8];
}

// The same layer for many rows (prompt phase): unfused small operators around the tensor-core matmul.
int32_t run_layer_prefill(qeng_ctx* ctx, qeng_decoder* d, int l, int64_t rows, const int32_t* table, cudaStream_t st) {
  Layer& L = d->layers[l];
  const int64_t dm = d->cfg.d_model, nq = (int64_t)d->Hq * kHD;
  const bool tp = d->cfg.tp_world > 1;
  __half* pool = d->pool + (size_t)l * d->pages * d->Hkv * 2 * kPage * kHD;
  int32_t rc = qeng_rmsnorm(ctx, d->x, L.norm1, rows, dm, d->cfg.rms_eps, d->xnr, st);
  if (rc == QENG_OK) rc = qeng_gemm_q4_prefill(ctx, L.wqkv, d->xnr, QENG_F32, rows, dm, d->qkv, d->nqkv, 0, st);
  if (rc != QENG_OK) return rc;
  rope_append_kernel<<<(unsigned)rows, 256, 0, st>>>(d->qkv, d->rope_cs, d->pos, table, d->max_pages, (int)d->pages,
                                                     d->Hq, d->Hkv, d->cfg.max_seq, d->q16, pool, ctx->status, L.qnorm, L.knorm, d->cfg.rms_eps);
  QENG_LAUNCH_CHECK(ctx);
  d->view.pages = d->pages; d->view.kv_heads = d->Hkv; d->view.hd = kHD; d->view.data = pool;
  for (int64_t r0 = 0; r0 < rows; r0 += kAttnRowsPerCall) {
    const int64_t nr = rows - r0 < kAttnRowsPerCall ? rows - r0 : kAttnRowsPerCall;
    rc = qeng_attn_decode_ex(ctx, &d->view, reinterpret_cast<const uint16_t*>(d->q16 + r0 * nq), table + r0 * d->max_pages,
                             d->max_pages, d->lens + r0, nr, d->Hq, 1.0f / sqrtf((float)kHD), d->cfg.attn_softcap,
                             d->cfg.sliding_window, d->att + r0 * nq, st);
    if (rc != QENG_OK) return rc;
  }
  const int64_t n = rows * dm;
  auto row_split_tc = [&](const qeng_weight* w, const float* in, int64_t ldin) -> int32_t {
    if (!tp) return qeng_gemm_q4_prefill(ctx, w, in, QENG_F32, rows, ldin, d->x, dm, 1, st);
    int32_t r = qeng_gemm_q4_prefill(ctx, w, in, QENG_F32, rows, ldin, d->part, dm, 0, st);
    if (r == QENG_OK) r = qeng_tp_all_reduce_internal(ctx, d->part, n, st);
    if (r != QENG_OK) return r;
    add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(d->x, d->part, n);
    return QENG_OK;
  };
  rc = row_split_tc(L.wo, d->att, nq);
  if (rc == QENG_OK) rc = qeng_rmsnorm(ctx, d->x, L.norm2, rows, dm, d->cfg.rms_eps, d->xnr, st);
  if (rc == QENG_OK) rc = qeng_gemm_q4_prefill(ctx, L.wgu, d->xnr, QENG_F32, rows, dm, d->gu, 2 * d->F, 0, st);
  if (rc != QENG_OK) return rc;
  const int64_t na = rows * d->F;
  swiglu_interleaved_kernel<<<(unsigned)((na + 255) / 256), 256, 0, st>>>(d->gu, rows, d->F, d->act);
  QENG_LAUNCH_CHECK(ctx);
  return row_split_tc(L.wdown, d->act, d->F);
}

// One layer over `rows` rows whose positions / lengths / page-table rows are on the device.
// `px`, when given (decode steps with mapped peers), selects the fused tensor-parallel form: o and
// down send their partial sums from the epilogue to every rank's inbox, the next matmul's staging
// adds the parts onto the residual rows of *px and leaves the result in the other residual buffer,
// to which *px then points.  No collective kernel runs.
int32_t run_layer(qeng_ctx* ctx, qeng_decoder* d, int l, int64_t rows, const int32_t* table, cudaStream_t st, float** px = nullptr) {
  Layer& L = d->layers[l];
  if (!L.wqkv || !L.wo || !L.wgu || !L.wdown || !L.norm1 || !L.norm2)
    return qeng_fail(ctx, QENG_ERR_STATE, "decoder: layer %d is not fully loaded", l);
  // the tensor-core prompt path dequantises 4-bit blocks; a layer with 8-bit blocks takes its prompt rows
  // through the decode kernels in passes of 16
  const bool all_q4 = L.wqkv->fmt == QENG_FMT_Q4 && L.wo->fmt == QENG_FMT_Q4 && L.wgu->fmt == QENG_FMT_Q4 && L.wdown->fmt == QENG_FMT_Q4;
  if (rows >= kPrefillRows && all_q4) return run_layer_prefill(ctx, d, l, rows, table, st);
  const int64_t dm = d->cfg.d_model;
  const bool fused = px != nullptr;
  float* x = fused ? *px : d->x;
  auto other = [&](float* cur) { return cur == d->x ? d->xalt : d->x; };
  __half* pool = d->pool + (size_t)l * d->pages * d->Hkv * 2 * kPage * kHD;
  qeng_gemm_fuse f;
  f.norm_gamma = L.norm1; f.norm_eps = d->cfg.rms_eps; f.epilogue = QENG_EPI_STORE;
  f.tp_layers = d->cfg.layers;
  if (fused && l > 0) {  // the parts of the previous layer's down projection
    f.tp_gather_kind = 1; f.tp_gather_layer = l - 1; f.tp_writeback = other(x);
  }
  int32_t rc;
  if ((L.qnorm == nullptr) != (L.knorm == nullptr))
    return qeng_fail(ctx, QENG_ERR_STATE, "decoder: layer %d has only one of the q / k head gains", l);
  if (L.qnorm == nullptr && qeng_gemm_q4_stream_fits(ctx, L.wqkv, 1)) {
    // q|k|v projection with rotary embedding, f16 rounding and KV append in its epilogue
    qeng_qkv_epi E;
    E.pos = d->pos; E.table = table; E.cs = d->rope_cs; E.q16 = d->q16; E.pool = pool;
    E.max_pages = d->max_pages; E.pages = (int)d->pages; E.Hq = d->Hq; E.Hkv = d->Hkv; E.max_seq = d->cfg.max_seq;
    f.epilogue = QENG_EPI_QKV; f.qkv = &E;
    rc = mm(ctx, d, L.wqkv, x, dm, rows, d->qkv, d->nqkv, f, st);
    if (rc != QENG_OK) return rc;
  } else {
    rc = mm(ctx, d, L.wqkv, x, dm, rows, d->qkv, d->nqkv, f, st);
    if (rc != QENG_OK) return rc;
    rope_append_kernel<<<(unsigned)rows, 256, 0, st>>>(d->qkv, d->rope_cs, d->pos, table, d->max_pages, (int)d->pages,
                                                       d->Hq, d->Hkv, d->cfg.max_seq, d->q16, pool, ctx->status, L.qnorm, L.knorm, d->cfg.rms_eps);
    QENG_LAUNCH_CHECK(ctx);
    d->launches++;
  }
  if (f.tp_gather_kind >= 0) x = other(x);  // the gathered rows are the residual stream from here on
  d->view.pages = d->pages; d->view.kv_heads = d->Hkv; d->view.hd = kHD; d->view.data = pool;
  rc = qeng_attn_decode_ex(ctx, &d->view, reinterpret_cast<const uint16_t*>(d->q16), table, d->max_pages, d->lens, rows,
                           d->Hq, 1.0f / sqrtf((float)kHD), d->cfg.attn_softcap, d->cfg.sliding_window, d->att, st);
  if (rc != QENG_OK) return rc;
  d->launches += 1;
  qeng_gemm_fuse fg;
  fg.norm_gamma = L.norm2; fg.norm_eps = d->cfg.rms_eps; fg.epilogue = QENG_EPI_SWIGLU; fg.two_limbs = true;
  fg.tp_layers = d->cfg.layers;
  if (!fused) {
    rc = row_split(ctx, d, L.wo, d->att, (int64_t)d->Hq * kHD, rows, st);
    if (rc != QENG_OK) return rc;
    rc = mm(ctx, d, L.wgu, d->x, dm, rows, d->act, d->F, fg, st);
    if (rc != QENG_OK) return rc;
    return row_split(ctx, d, L.wdown, d->act, d->F, rows, st);
  }
  qeng_gemm_fuse fp;
  fp.epilogue = QENG_EPI_STORE; fp.two_limbs = true; fp.tp_layers = d->cfg.layers; fp.tp_layer = l;
  fp.tp_push_kind = 0;
  rc = mm(ctx, d, L.wo, d->att, (int64_t)d->Hq * kHD, rows, d->part, dm, fp, st);
  if (rc != QENG_OK) return rc;
  fg.tp_gather_kind = 0; fg.tp_gather_layer = l; fg.tp_writeback = other(x);
  rc = mm(ctx, d, L.wgu, x, dm, rows, d->act, d->F, fg, st);
  if (rc != QENG_OK) return rc;
  x = other(x);
  fp.tp_push_kind = 1;
  rc = mm(ctx, d, L.wdown, d->act, d->F, rows, d->part, dm, fp, st);
  *px = x;
  return rc;
}

// sharded LM head: every rank fills its vocabulary columns of the logits, in chunks of up to 4 rows
int32_t tail_sharded(qeng_ctx* ctx, qeng_decoder* d, const float* x_last, int B, bool finalize, cudaStream_t st) {
  const int dm = d->cfg.d_model, V = d->cfg.vocab, W = d->cfg.tp_world, R = d->cfg.tp_rank;
  if (!finalize)  // the other ranks' columns must be zero for the sum below
    QENG_CUDA(ctx, cudaMemsetAsync(d->logits, 0, (size_t)B * V * 4, st));
  for (int m0 = 0; m0 < B; m0 += 4) {
    qeng_lm_tail t;
    t.table = d->lm_head; t.x = x_last + (size_t)m0 * dm; t.M = B - m0 < 4 ? B - m0 : 4; t.D = dm; t.V = d->vloc;
    t.logits = d->logits + (size_t)m0 * V; t.v0 = d->v0; t.Vtot = V; t.ldl = V;
    t.gamma = d->final_norm; t.eps = d->cfg.rms_eps; t.softcap = d->cfg.final_softcap;
    if (finalize) { t.pairs = d->tp_pairs; t.pair_slot = R * B + m0; }
    d->launches += 1;
    int32_t rc = qeng_lm_head_fused(ctx, t, st);
    if (rc != QENG_OK) return rc;
  }
  if (!finalize) {  // prompt end: every rank needs the full logits (zero + x = x, so the sum is exact)
    d->logits_partial = false;
    return qeng_tp_all_reduce_internal(ctx, d->logits, (int64_t)B * V, st);
  }
  const int64_t n = (int64_t)2 * W * B;  // a multiple of 4: W is even
  int32_t rc;
  if (qeng_tp_p2p_ready(ctx, n)) {
    rc = qeng_tp_allreduce_add(ctx, d->tp_gath, d->tp_pairs, n, st);  // tp_gath is zero on entry
  } else {
    QENG_CUDA(ctx, cudaMemcpyAsync(d->tp_gath, d->tp_pairs, n * 4, cudaMemcpyDeviceToDevice, st));
    rc = qeng_tp_all_reduce_internal(ctx, d->tp_gath, n, st);
    d->launches += 1;
  }
  if (rc != QENG_OK) return rc;
  tp_pick_kernel<<<1, 256, 0, st>>>(d->tp_gath, W, B, V, dm, d->emb, d->x, d->next, d->pos, d->lens, d->out_tokens,
                                    d->step, ctx->status);
  QENG_LAUNCH_CHECK(ctx);
  d->launches += 2;
  return QENG_OK;
}

// final norm + LM head (+ greedy finalisation: sample, record, advance, embed the next token)
int32_t tail(qeng_ctx* ctx, qeng_decoder* d, const float* x_last, int B, bool finalize, cudaStream_t st) {
  if (d->vsplit) return tail_sharded(ctx, d, x_last, B, finalize, st);
  if (B <= 4) {
    qeng_lm_tail t;
    t.table = d->lm_head; t.x = x_last; t.M = B; t.D = d->cfg.d_model; t.V = d->cfg.vocab; t.logits = d->logits;
    t.gamma = d->final_norm; t.eps = d->cfg.rms_eps; t.softcap = d->cfg.final_softcap;
    if (finalize) {
      t.next = d->next; t.emb = d->emb; t.xout = d->x; t.pos = d->pos; t.lens = d->lens;
      t.out_tokens = d->out_tokens; t.step = d->step;
    }
    d->launches += 1;
    return qeng_lm_head_fused(ctx, t, st);
  }
  int32_t rc = qeng_rmsnorm(ctx, x_last, d->final_norm, B, d->cfg.d_model, d->cfg.rms_eps, d->xn, st);
  if (rc != QENG_OK) return rc;
  for (int m0 = 0; m0 < B; m0 += 4) {  // the LM head takes 4 rows per launch
    qeng_lm_tail t;
    t.table = d->lm_head; t.x = d->xn + (size_t)m0 * d->cfg.d_model; t.M = B - m0 < 4 ? B - m0 : 4;
    t.D = d->cfg.d_model; t.V = d->cfg.vocab; t.logits = d->logits + (size_t)m0 * d->cfg.vocab;
    t.softcap = d->cfg.final_softcap;
    rc = qeng_lm_head_fused(ctx, t, st);
    if (rc != QENG_OK) return rc;
  }
  d->launches += 1 + (B + 3) / 4;
  if (!finalize) return QENG_OK;
  rc = qeng_argmax(ctx, d->logits, B, d->cfg.vocab, d->next, st);
  if (rc != QENG_OK) return rc;
  advance_kernel<<<1, 32 * ((B + 31) / 32), 0, st>>>(d->next, d->pos, d->lens, d->out_tokens, d->step, B);
  QENG_LAUNCH_CHECK(ctx);
  rc = qeng_embed(ctx, d->emb, d->next, B, d->cfg.d_model, d->cfg.vocab, d->x, st);
  d->launches += 3;
  return rc;
}

// Plan the fused step kernel for this decoder (once per set of weights and buffers).  Leaves
// d->fused null when the model is outside what the kernel takes: per-head q/k gains, more than one
// rank (the sharded step still runs operator by operator), unusual widths.
int32_t plan_step(qeng_ctx* ctx, qeng_decoder* d) {
  d->step_planned = true;
  if (d->cfg.tp_world != 1 || d->cfg.attn_softcap > 0.f || d->cfg.sliding_window > 0) return QENG_OK;
  qeng_step_desc desc;
  for (int l = 0; l < d->cfg.layers; ++l) {
    Layer& L = d->layers[l];
    if (!L.wqkv || !L.wo || !L.wgu || !L.wdown || !L.norm1 || !L.norm2 || L.qnorm || L.knorm) return QENG_OK;
    if (L.wqkv->fmt != QENG_FMT_Q4 || L.wo->fmt != QENG_FMT_Q4 || L.wgu->fmt != QENG_FMT_Q4 || L.wdown->fmt != QENG_FMT_Q4) return QENG_OK;
    qeng_step_layer_desc ld;
    ld.w[0] = L.wqkv; ld.w[1] = L.wo; ld.w[2] = L.wgu; ld.w[3] = L.wdown;
    ld.norm1 = L.norm1; ld.norm2 = L.norm2;
    ld.pool = d->pool + (size_t)l * d->pages * d->Hkv * 2 * kPage * kHD;
    desc.layers.push_back(ld);
  }
  desc.dm = d->cfg.d_model; desc.F = d->F; desc.Hq = d->Hq; desc.Hkv = d->Hkv;
  desc.max_pages = d->max_pages; desc.pages = (int)d->pages; desc.max_seq = d->cfg.max_seq; desc.eps = d->cfg.rms_eps;
  desc.x = d->x; desc.pos = d->pos; desc.lens = d->lens; desc.table = d->dec_table; desc.cs = d->rope_cs;
  desc.q16 = d->q16; desc.act = d->act;
  desc.world = 1; desc.rank = 0;
  return qeng_step_create(ctx, desc, &d->fused);
}

// one decode step, all state on the device: x holds the embedding of the token to feed
int32_t decode_step(qeng_ctx* ctx, qeng_decoder* d, cudaStream_t st) {
  const int B = d->batch;
  bool fused = d->cfg.tp_world > 1 && qeng_tp_fuse_ready(ctx, B, d->cfg.d_model);
  // the exchange through the matmul epilogues addresses inbox rows by the row index inside one
  // pass: every matrix must take the whole batch in one pass
  for (int l = 0; fused && l < d->cfg.layers; ++l) {
    const Layer& L = d->layers[l];
    fused = L.wqkv && L.wo && L.wgu && L.wdown && qeng_gemm_q4_stream_fits(ctx, L.wqkv, B) && qeng_gemm_q4_stream_fits(ctx, L.wo, B) &&
            qeng_gemm_q4_stream_fits(ctx, L.wgu, B) && qeng_gemm_q4_stream_fits(ctx, L.wdown, B);
  }
  float* x = d->x;
  for (int l = 0; l < d->cfg.layers; ++l) {
    int32_t rc = run_layer(ctx, d, l, B, d->dec_table, st, fused ? &x : nullptr);
    if (rc != QENG_OK) return rc;
  }
  if (fused) {
    // the one gather no matmul absorbs: the parts of the last down projection, added in place
    int32_t rc = qeng_tp_fuse_gather(ctx, x, B, d->cfg.d_model, 1, d->cfg.layers - 1, d->cfg.layers, st);
    if (rc != QENG_OK) return rc;
    d->launches += 2;
  }
  int32_t rc = tail(ctx, d, x, B, true, st);  // leaves the next token's embedding in d->x
  if (rc == QENG_OK && fused) rc = qeng_tp_fuse_advance(ctx, st);
  return rc;
}

// shard of a full host matrix: rows [r0,r1) x columns [k0,k1)
void take_shard(const uint8_t* q, const uint16_t* s, int su, int64_t K, int64_t r0, int64_t r1, int64_t k0, int64_t k1,
                HostMat& out) {
  out.N = r1 - r0; out.K = k1 - k0; out.su = su;
  out.q.resize((size_t)out.N * out.K);
  out.s.resize((size_t)out.N * out.K / 32 * su);
  for (int64_t r = r0; r < r1; ++r) {
    memcpy(&out.q[(size_t)(r - r0) * out.K], q + r * K + k0, (size_t)out.K);
    memcpy(&out.s[(size_t)(r - r0) * (out.K / 32) * su], s + (r * (K / 32) + k0 / 32) * su, (size_t)(out.K / 32) * 2 * su);
  }
}

}  // namespace

extern "C" {

int32_t qeng_decoder_create(qeng_ctx* ctx, const qeng_model_cfg* cfg, qeng_decoder** out) {
  if (!ctx || !cfg || !out) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_create: null argument");
  *out = nullptr;
  const int t = cfg->tp_world;
  if (t < 1 || cfg->tp_rank < 0 || cfg->tp_rank >= t) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_create: bad tp rank/world");
  if (cfg->head_dim != kHD) return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_create: head_dim must be 128");
  if (cfg->layers < 1 || cfg->heads < 1 || cfg->kv_heads < 1 || cfg->heads % cfg->kv_heads != 0 ||
      cfg->heads / cfg->kv_heads > 8)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_create: bad head counts");
  if (cfg->kv_heads % t != 0 || cfg->ffn % (16 * t) != 0 || cfg->d_model % 32 != 0 || (cfg->ffn / t) % 32 != 0 ||
      (cfg->heads * kHD / t) % 32 != 0)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_create: shapes do not shard evenly over %d ranks", t);
  if (cfg->attn_softcap < 0.f || cfg->sliding_window < 0 || cfg->final_softcap < 0.f)
    return qeng_fail(ctx, QENG_ERR_ARG, "decoder_create: attn_softcap, final_softcap and sliding_window must not be negative");
  if (cfg->max_batch < 1 || cfg->max_batch > 16 || cfg->max_seq < 1)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_create: max_batch must be 1..16 and max_seq positive");
  if (t > 1 && (ctx->tp_world != t || ctx->tp_rank != cfg->tp_rank))
    return qeng_fail(ctx, QENG_ERR_STATE, "decoder_create: call qeng_tp_init(rank %d, world %d) on this context first", cfg->tp_rank, t);
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  qeng_decoder* d = new qeng_decoder();
  d->cfg = *cfg;
  d->Hq = cfg->heads / t; d->Hkv = cfg->kv_heads / t; d->F = cfg->ffn / t;
  d->nqkv = (d->Hq + 2 * d->Hkv) * kHD;
  d->max_pages = (cfg->max_seq + kPage - 1) / kPage;
  d->pages = (int64_t)d->max_pages * cfg->max_batch;
  d->layers.resize(cfg->layers);
  d->max_steps = cfg->max_seq;
  d->vsplit = t > 1 && cfg->vocab % t == 0 && cfg->vocab <= (1 << 24);
  d->vloc = d->vsplit ? cfg->vocab / t : cfg->vocab;
  d->v0 = d->vsplit ? cfg->tp_rank * d->vloc : 0;
  const int64_t dm = cfg->d_model;
  const size_t pool_bytes = (size_t)cfg->layers * d->pages * d->Hkv * 2 * kPage * kHD * 2;
  cudaError_t e = cudaMalloc(&d->pool, pool_bytes);
  if (e == cudaSuccess) e = cudaMemset(d->pool, 0, pool_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&d->rope_cs, (size_t)cfg->max_seq * kHD * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d->xn, (size_t)cfg->max_batch * dm * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d->xlast, (size_t)cfg->max_batch * dm * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d->logits, (size_t)cfg->max_batch * cfg->vocab * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d->next, 64 * 4);
  if (e == cudaSuccess && d->vsplit) {
    const size_t pb = (size_t)2 * t * cfg->max_batch * 4;
    e = cudaMalloc(&d->tp_pairs, pb);
    if (e == cudaSuccess) e = cudaMemset(d->tp_pairs, 0, pb);
    if (e == cudaSuccess) e = cudaMalloc(&d->tp_gath, pb);
    if (e == cudaSuccess) e = cudaMemset(d->tp_gath, 0, pb);
  }
  if (e == cudaSuccess) e = cudaMalloc(&d->step, 4);
  if (e == cudaSuccess) e = cudaMalloc(&d->out_tokens, (size_t)(d->max_steps + 1) * cfg->max_batch * 4);
  if (e == cudaSuccess) e = cudaMallocHost(&d->h_out, ((size_t)d->max_steps * cfg->max_batch + 1) * 4);
  if (e == cudaSuccess) e = cudaMalloc(&d->dec_table, (size_t)cfg->max_batch * d->max_pages * 4);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&d->own_stream, cudaStreamNonBlocking);
  d->stream = d->own_stream;
  if (e != cudaSuccess) {
    qeng_decoder_free(ctx, d);
    return qeng_fail(ctx, QENG_ERR_CUDA, "decoder_create: %s", cudaGetErrorString(e));
  }
  // rotary table in double, stored as f32: [pos][cos 0..63 | sin 0..63]
  std::vector<float> cs((size_t)cfg->max_seq * kHD);
  for (int p = 0; p < cfg->max_seq; ++p)
    for (int i = 0; i < 64; ++i) {
      const double ang = (double)p * pow((double)cfg->rope_base, -2.0 * i / (double)kHD);
      cs[(size_t)p * kHD + i] = (float)cos(ang);
      cs[(size_t)p * kHD + 64 + i] = (float)sin(ang);
    }
  e = cudaMemcpy(d->rope_cs, cs.data(), cs.size() * 4, cudaMemcpyHostToDevice);
  // page table: sequence b owns pages p*max_batch + b (interleaved, so the
  // indirection is exercised)
  std::vector<int32_t> tb((size_t)cfg->max_batch * d->max_pages);
  for (int b = 0; b < cfg->max_batch; ++b)
    for (int p = 0; p < d->max_pages; ++p) tb[(size_t)b * d->max_pages + p] = p * cfg->max_batch + b;
  if (e == cudaSuccess) e = cudaMemcpy(d->dec_table, tb.data(), tb.size() * 4, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    qeng_decoder_free(ctx, d);
    return qeng_fail(ctx, QENG_ERR_CUDA, "decoder_create: %s", cudaGetErrorString(e));
  }
  int32_t rc = ensure_rows(ctx, d, cfg->max_batch);
  if (rc != QENG_OK) {
    qeng_decoder_free(ctx, d);
    return rc;
  }
  *out = d;
  return QENG_OK;
}

int32_t qeng_decoder_free(qeng_ctx* ctx, qeng_decoder* d) {
  if (!d) return QENG_OK;
  if (ctx) cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  if (d->graph) cudaGraphExecDestroy(d->graph);
  qeng_step_free(d->fused);
  for (auto& L : d->layers) {
    qeng_weight_free(ctx, L.wqkv); qeng_weight_free(ctx, L.wo); qeng_weight_free(ctx, L.wgu); qeng_weight_free(ctx, L.wdown);
    if (L.norm1) cudaFree(L.norm1);
    if (L.norm2) cudaFree(L.norm2);
    if (L.qnorm) cudaFree(L.qnorm);
    if (L.knorm) cudaFree(L.knorm);
  }
  void* bufs[] = {d->emb, d->lm_head, d->final_norm, d->rope_cs, d->pool, d->x, d->xalt, d->qkv, d->att, d->act, d->part, d->xnr, d->gu, d->q16,
                  d->pos, d->lens, d->table, d->tok, d->xn, d->xlast, d->logits, d->next, d->out_tokens, d->step, d->dec_table, d->tp_pairs, d->tp_gath};
  for (void* p : bufs)
    if (p) cudaFree(p);
  if (d->own_stream) cudaStreamDestroy(d->own_stream);
  if (d->h_out) cudaFreeHost(d->h_out);
  delete d;
  return QENG_OK;
}

// The order of the decode loop is fixed, so every fused matrix knows its successor: the
// streaming matmul uses it to keep HBM busy across kernel boundaries.
static void link_weights(qeng_decoder* d) {
  qeng_weight* prev = nullptr;
  for (auto& L : d->layers) {
    qeng_weight* seq[4] = {L.wqkv, L.wo, L.wgu, L.wdown};
    for (qeng_weight* w : seq) {
      if (!w) continue;
      w->next = nullptr;
      if (prev) prev->next = w;
      prev = w;
    }
  }
}

static int32_t pack_fmt(qeng_ctx* ctx, int fmt, const uint8_t* q, const uint16_t* s, int64_t N, int64_t K, qeng_weight** out) {
  if (fmt == QENG_FMT_Q8) return qeng_weight_pack_q8(ctx, reinterpret_cast<const int8_t*>(q), s, N, K, out);
  if (fmt == QENG_FMT_K4) return qeng_weight_pack_k4(ctx, q, reinterpret_cast<const float*>(s), N, K, out);
  return qeng_weight_pack_q4(ctx, q, s, N, K, out);
}

// one matrix of a layer in either block format: q holds one code (4-bit: 0..15) or one signed byte
// (8-bit) per weight; sharding, the rotary row order and the q|k|v / gate|up fusion work on bytes
static int32_t load_matrix_fmt(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, int32_t which, int fmt, const uint8_t* q,
                               const uint16_t* s, int64_t N, int64_t K) {
  if (!ctx || !d || !q || !s) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_matrix: null argument");
  if (layer < 0 || layer >= d->cfg.layers || which < 0 || which > QENG_W_DOWN)
    return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_matrix: bad layer/which");
  const qeng_model_cfg& c = d->cfg;
  const int t = c.tp_world, r = c.tp_rank;
  const int64_t dm = c.d_model, nq = (int64_t)c.heads * kHD, nkv = (int64_t)c.kv_heads * kHD;
  int64_t eN = 0, eK = 0;
  switch (which) {
    case QENG_W_Q: eN = nq; eK = dm; break;
    case QENG_W_K: case QENG_W_V: eN = nkv; eK = dm; break;
    case QENG_W_O: eN = dm; eK = nq; break;
    case QENG_W_GATE: case QENG_W_UP: eN = c.ffn; eK = dm; break;
    default: eN = dm; eK = c.ffn; break;
  }
  if (N != eN || K != eK)
    return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_load_matrix: matrix %d must be [%lld,%lld], got [%lld,%lld]", which,
                     (long long)eN, (long long)eK, (long long)N, (long long)K);
  Layer& L = d->layers[layer];
  HostMat& hm = L.pend[which];
  // the matrices fused into one (q|k|v, gate|up) must come in one format
  const int lo = which <= QENG_W_V ? QENG_W_Q : QENG_W_GATE, hi = which <= QENG_W_V ? QENG_W_V : QENG_W_UP;
  if (which <= QENG_W_V || which == QENG_W_GATE || which == QENG_W_UP)
    for (int i = lo; i <= hi; ++i)
      if (i != which && L.pend[i].N && L.pend[i].fmt != fmt)
        return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_matrix: layer %d mixes 4-bit and 8-bit blocks inside a fused matrix", layer);
  const bool row_split = which == QENG_W_O || which == QENG_W_DOWN;  // split along K, partial sums
  const int su = fmt == QENG_FMT_K4 ? 4 : 1;
  if (row_split) take_shard(q, s, su, K, 0, N, K / t * r, K / t * (r + 1), hm);
  else take_shard(q, s, su, K, N / t * r, N / t * (r + 1), 0, K, hm);
  hm.fmt = fmt;
  if (which <= QENG_W_V) {  // rotary pairs (i, i+64) of every head become MMA rows g / g+8 of one tile
    HostMat pm;
    pm.N = hm.N; pm.K = hm.K; pm.fmt = fmt; pm.su = su;
    pm.q.resize(hm.q.size());
    pm.s.resize(hm.s.size());
    for (int64_t row = 0; row < hm.N; ++row) {
      const int64_t head = row / kHD, i = row % kHD;
      const int64_t prow = head * kHD + (((i & 63) >> 3) << 4) + (i & 7) + ((i >> 6) << 3);
      memcpy(&pm.q[(size_t)prow * hm.K], &hm.q[(size_t)row * hm.K], (size_t)hm.K);
      memcpy(&pm.s[(size_t)prow * (hm.K / 32) * su], &hm.s[(size_t)row * (hm.K / 32) * su], (size_t)(hm.K / 32) * 2 * su);
    }
    hm = pm;
  }
  int32_t rc = QENG_OK;
  if (row_split) {
    qeng_weight** dst = which == QENG_W_O ? &L.wo : &L.wdown;
    qeng_weight_free(ctx, *dst); *dst = nullptr;
    rc = pack_fmt(ctx, fmt, hm.q.data(), hm.s.data(), hm.N, hm.K, dst);
    hm = HostMat();
  } else if (which <= QENG_W_V) {
    if (L.pend[QENG_W_Q].N && L.pend[QENG_W_K].N && L.pend[QENG_W_V].N) {
      HostMat f;
      f.K = dm; f.su = su; f.fmt = fmt;
      for (int i = QENG_W_Q; i <= QENG_W_V; ++i) {
        f.q.insert(f.q.end(), L.pend[i].q.begin(), L.pend[i].q.end());
        f.s.insert(f.s.end(), L.pend[i].s.begin(), L.pend[i].s.end());
        f.N += L.pend[i].N;
        L.pend[i] = HostMat();
      }
      qeng_weight_free(ctx, L.wqkv); L.wqkv = nullptr;
      rc = pack_fmt(ctx, fmt, f.q.data(), f.s.data(), f.N, f.K, &L.wqkv);
    }
  } else {
    if (L.pend[QENG_W_GATE].N && L.pend[QENG_W_UP].N) {
      // interleave: fused row 16*j + r = gate row 8*j + r (r < 8), up row 8*j + r - 8 (r >= 8)
      const HostMat& G = L.pend[QENG_W_GATE];
      const HostMat& U = L.pend[QENG_W_UP];
      HostMat f;
      f.N = 2 * G.N; f.K = dm; f.su = su; f.fmt = fmt;
      f.q.resize((size_t)f.N * f.K);
      f.s.resize((size_t)f.N * f.K / 32 * su);
      for (int64_t i = 0; i < G.N; ++i) {
        const int64_t rg = (i / 8) * 16 + i % 8, ru = rg + 8;
        memcpy(&f.q[(size_t)rg * dm], &G.q[(size_t)i * dm], (size_t)dm);
        memcpy(&f.q[(size_t)ru * dm], &U.q[(size_t)i * dm], (size_t)dm);
        memcpy(&f.s[(size_t)rg * (dm / 32) * su], &G.s[(size_t)i * (dm / 32) * su], (size_t)(dm / 32) * 2 * su);
        memcpy(&f.s[(size_t)ru * (dm / 32) * su], &U.s[(size_t)i * (dm / 32) * su], (size_t)(dm / 32) * 2 * su);
      }
      L.pend[QENG_W_GATE] = HostMat();
      L.pend[QENG_W_UP] = HostMat();
      qeng_weight_free(ctx, L.wgu); L.wgu = nullptr;
      rc = pack_fmt(ctx, fmt, f.q.data(), f.s.data(), f.N, f.K, &L.wgu);
    }
  }
  link_weights(d);
  if (d->graph) { cudaGraphExecDestroy(d->graph); d->graph = nullptr; }
  qeng_step_free(d->fused); d->fused = nullptr; d->step_planned = false;
  return rc;
}

int32_t qeng_decoder_load_matrix(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, int32_t which, const uint8_t* q,
                                 const uint16_t* s, int64_t N, int64_t K) {
  return load_matrix_fmt(ctx, d, layer, which, QENG_FMT_Q4, q, s, N, K);
}

int32_t qeng_decoder_load_matrix_q8(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, int32_t which, const int8_t* q,
                                    const uint16_t* s, int64_t N, int64_t K) {
  return load_matrix_fmt(ctx, d, layer, which, QENG_FMT_Q8, reinterpret_cast<const uint8_t*>(q), s, N, K);
}

int32_t qeng_decoder_load_matrix_q4k(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, int32_t which, const uint8_t* blocks,
                                     int64_t N, int64_t K) {
  if (!ctx || !d || !blocks) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_matrix_q4k: null argument");
  std::vector<uint8_t> q;
  std::vector<float> dm;
  int32_t rc = qeng_q4k_expand(ctx, blocks, N, K, &q, &dm);
  if (rc != QENG_OK) return rc;
  return load_matrix_fmt(ctx, d, layer, which, QENG_FMT_K4, q.data(), reinterpret_cast<const uint16_t*>(dm.data()), N, K);
}

int32_t qeng_decoder_load_norm(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, int32_t which, const float* gamma) {
  if (!ctx || !d || !gamma) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_norm: null argument");
  if (layer < 0 || layer >= d->cfg.layers || which < 0 || which > 3) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_norm: bad layer/which");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  Layer& L = d->layers[layer];
  float** dst = which == 0 ? &L.norm1 : which == 1 ? &L.norm2 : which == 2 ? &L.qnorm : &L.knorm;
  const size_t n = which < 2 ? (size_t)d->cfg.d_model : (size_t)kHD;  // 2, 3: per-head gains of q and k
  if (!*dst) QENG_CUDA(ctx, cudaMalloc(dst, n * 4));
  QENG_CUDA(ctx, cudaMemcpy(*dst, gamma, n * 4, cudaMemcpyHostToDevice));
  if (which >= 2 && d->graph) { cudaGraphExecDestroy(d->graph); d->graph = nullptr; }  // the step takes another path
  qeng_step_free(d->fused); d->fused = nullptr; d->step_planned = false;
  return QENG_OK;
}

int32_t qeng_decoder_load_head(qeng_ctx* ctx, qeng_decoder* d, const uint16_t* emb, const uint16_t* lm_head,
                               const float* final_gamma) {
  if (!ctx || !d || !emb || !lm_head || !final_gamma) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_load_head: null argument");
  const size_t n = (size_t)d->cfg.vocab * d->cfg.d_model;
  const size_t nloc = (size_t)d->vloc * d->cfg.d_model;  // this rank's vocabulary rows of the head
  lm_head += (size_t)d->v0 * d->cfg.d_model;
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  if (!d->emb) QENG_CUDA(ctx, cudaMalloc(&d->emb, n * 2));
  if (!d->lm_head) QENG_CUDA(ctx, cudaMalloc(&d->lm_head, nloc * 2));
  if (!d->final_norm) QENG_CUDA(ctx, cudaMalloc(&d->final_norm, (size_t)d->cfg.d_model * 4));
  QENG_CUDA(ctx, cudaMemcpy(d->emb, emb, n * 2, cudaMemcpyHostToDevice));
  QENG_CUDA(ctx, cudaMemcpy(d->lm_head, lm_head, nloc * 2, cudaMemcpyHostToDevice));
  QENG_CUDA(ctx, cudaMemcpy(d->final_norm, final_gamma, (size_t)d->cfg.d_model * 4, cudaMemcpyHostToDevice));
  return QENG_OK;
}

int32_t qeng_decoder_reset(qeng_ctx* ctx, qeng_decoder* d, int32_t batch) {
  if (!ctx || !d) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_reset: null argument");
  if (batch < 1 || batch > d->cfg.max_batch) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_reset: batch outside 1..max_batch");
  if (d->tp_pairs && batch != d->batch) {
    // the slot of a rank's (max, index) pair depends on the batch (rank * batch + sequence): pairs left
    // from another batch size would be added to another rank's slot
    QENG_CUDA(ctx, cudaSetDevice(ctx->device));
    const size_t pb = (size_t)2 * d->cfg.tp_world * d->cfg.max_batch * sizeof(float);
    QENG_CUDA(ctx, cudaStreamSynchronize(d->stream));
    QENG_CUDA(ctx, cudaMemsetAsync(d->tp_pairs, 0, pb, d->stream));
    QENG_CUDA(ctx, cudaMemsetAsync(d->tp_gath, 0, pb, d->stream));
  }
  d->batch = batch;
  d->len.assign(batch, 0);
  d->have_logits = false;
  d->logits_partial = false;
  d->next_ready = false;
  return QENG_OK;
}

int32_t qeng_decoder_prefill(qeng_ctx* ctx, qeng_decoder* d, const int32_t* tokens, int32_t batch, int32_t T) {
  if (!ctx || !d || !tokens) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_prefill: null argument");
  if (batch != d->batch) return qeng_fail(ctx, QENG_ERR_STATE, "decoder_prefill: batch differs from the last reset");
  if (T < 1) return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_prefill: empty prompt");
  for (int b = 0; b < batch; ++b)
    if (d->len[b] + T > d->cfg.max_seq) return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_prefill: prompt exceeds max_seq");
  if (!d->emb) return qeng_fail(ctx, QENG_ERR_STATE, "decoder_prefill: embeddings not loaded");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  const int64_t rows = (int64_t)batch * T;
  int32_t rc = ensure_rows(ctx, d, rows);
  if (rc != QENG_OK) return rc;
  cudaStream_t st = d->stream;
  std::vector<int32_t> pos(rows), lens(rows), table((size_t)rows * d->max_pages);
  for (int b = 0; b < batch; ++b)
    for (int tt = 0; tt < T; ++tt) {
      const int64_t r = (int64_t)b * T + tt;
      pos[r] = d->len[b] + tt;
      lens[r] = pos[r] + 1;
      for (int p = 0; p < d->max_pages; ++p) table[(size_t)r * d->max_pages + p] = p * d->cfg.max_batch + b;
    }
  int32_t* dtok = d->tok;
  cudaMemcpyAsync(dtok, tokens, rows * 4, cudaMemcpyHostToDevice, st);
  cudaMemcpyAsync(d->pos, pos.data(), rows * 4, cudaMemcpyHostToDevice, st);
  cudaMemcpyAsync(d->lens, lens.data(), rows * 4, cudaMemcpyHostToDevice, st);
  cudaMemcpyAsync(d->table, table.data(), table.size() * 4, cudaMemcpyHostToDevice, st);
  rc = qeng_embed(ctx, d->emb, dtok, rows, d->cfg.d_model, d->cfg.vocab, d->x, st);
  for (int l = 0; rc == QENG_OK && l < d->cfg.layers; ++l) rc = run_layer(ctx, d, l, rows, d->table, st);
  if (rc == QENG_OK) {
    // hidden state of the last prompt position of every sequence, gathered for the LM head
    for (int b = 0; b < batch; ++b)
      cudaMemcpyAsync(d->xlast + (size_t)b * d->cfg.d_model, d->x + ((size_t)b * T + T - 1) * d->cfg.d_model,
                      (size_t)d->cfg.d_model * 4, cudaMemcpyDeviceToDevice, st);
    rc = tail(ctx, d, d->xlast, batch, false, st);
  }
  cudaError_t e = cudaStreamSynchronize(st);
  if (rc != QENG_OK) return rc;
  if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "decoder_prefill: %s", cudaGetErrorString(e));
  for (int b = 0; b < batch; ++b) d->len[b] += T;
  d->have_logits = true;
  d->next_ready = false;
  return QENG_OK;
}

int32_t qeng_decoder_decode(qeng_ctx* ctx, qeng_decoder* d, int32_t steps, int32_t* out_tokens) {
  if (!ctx || !d || !out_tokens) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_decode: null argument");
  if (!d->have_logits) return qeng_fail(ctx, QENG_ERR_STATE, "decoder_decode: no logits yet (prefill first)");
  if (steps < 1 || steps > d->max_steps) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_decode: bad step count");
  const int B = d->batch;
  for (int b = 0; b < B; ++b)
    if (d->len[b] + steps > d->cfg.max_seq) return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_decode: would exceed max_seq");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaStream_t st = d->stream;
  {
    int32_t rc = qeng_attn_reserve(ctx, B, d->Hq, d->Hkv, d->max_pages);  // never allocate inside the capture
    const Layer& L0 = d->layers[0];
    const qeng_weight* ws[4] = {L0.wqkv, L0.wo, L0.wgu, L0.wdown};
    for (int i = 0; rc == QENG_OK && i < 4; ++i)
      if (ws[i]) rc = qeng_gemm_q4_stream_reserve(ctx, ws[i], B < 16 ? B : 16);
    if (rc != QENG_OK) return rc;
  }
  std::vector<int32_t> pos(B), lens(B);
  for (int b = 0; b < B; ++b) { pos[b] = d->len[b]; lens[b] = d->len[b] + 1; }
  if (!d->next_ready) {  // right after a decode step the device copies are already one token on
    QENG_CUDA(ctx, cudaMemcpyAsync(d->pos, pos.data(), B * 4, cudaMemcpyHostToDevice, st));
    QENG_CUDA(ctx, cudaMemcpyAsync(d->lens, lens.data(), B * 4, cudaMemcpyHostToDevice, st));
  }
  QENG_CUDA(ctx, cudaMemsetAsync(d->step, 0, 4, st));
  {  // the token sampled from the logits at hand is fed first; right after a decode step it has
     // been picked and embedded already by that step's last kernel
    int32_t rc = QENG_OK;
    if (!d->next_ready) {
      rc = qeng_argmax(ctx, d->logits, B, d->cfg.vocab, d->next, st);
      if (rc == QENG_OK) rc = qeng_embed(ctx, d->emb, d->next, B, d->cfg.d_model, d->cfg.vocab, d->x, st);
    }
    if (rc != QENG_OK) return rc;
    record_first_kernel<<<1, 32, 0, st>>>(d->next, d->out_tokens, B);
    QENG_LAUNCH_CHECK(ctx);
  }
  d->next_ready = false;  // until this call's steps have run to the end
  if (!d->step_planned) {
    int32_t rc = plan_step(ctx, d);
    if (rc != QENG_OK) return rc;
  }
  if (qeng_step_takes(d->fused, B)) {
    // all layers in one persistent kernel, then the LM head (norm, head, sample, advance, embed)
    for (int s = 0; s < steps; ++s) {
      d->launches = 1;
      int32_t rc = qeng_step_launch(ctx, d->fused, B, st);
      if (rc == QENG_OK) rc = tail(ctx, d, d->x, B, true, st);
      if (rc != QENG_OK) return rc;
    }
  } else {
    if (!d->graph || d->graph_batch != B || d->graph_scratch_gen != ctx->scratch_gen) {
      QENG_CUDA(ctx, cudaStreamSynchronize(st));
      if (d->graph) { cudaGraphExecDestroy(d->graph); d->graph = nullptr; }
      cudaGraph_t g = nullptr;
      QENG_CUDA(ctx, cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
      d->launches = 0;
      int32_t rc = decode_step(ctx, d, st);
      cudaError_t e = cudaStreamEndCapture(st, &g);
      if (rc != QENG_OK) { if (g) cudaGraphDestroy(g); return rc; }
      if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "decoder_decode: capture failed: %s", cudaGetErrorString(e));
      e = cudaGraphInstantiate(&d->graph, g, 0);
      cudaGraphDestroy(g);
      if (e != cudaSuccess) return qeng_fail(ctx, QENG_ERR_CUDA, "decoder_decode: instantiate failed: %s", cudaGetErrorString(e));
      d->graph_batch = B;
      d->graph_scratch_gen = ctx->scratch_gen;
    }
    for (int s = 0; s < steps; ++s) QENG_CUDA(ctx, cudaGraphLaunch(d->graph, st));
  }
  // tokens and status word through pinned memory: both copies are queued behind the steps and the
  // call synchronises once
  const size_t ntok = (size_t)steps * B;
  QENG_CUDA(ctx, cudaMemcpyAsync(d->h_out, d->out_tokens, ntok * 4, cudaMemcpyDeviceToHost, st));
  QENG_CUDA(ctx, cudaMemcpyAsync(d->h_out + ntok, ctx->status, 4, cudaMemcpyDeviceToHost, st));
  QENG_CUDA(ctx, cudaStreamSynchronize(st));
  const int32_t status = d->h_out[ntok];
  for (int b = 0; b < B; ++b) d->len[b] += steps;
  if (d->vsplit) d->logits_partial = true;
  d->next_ready = status == 0;
  if (status != 0) {
    cudaMemset(ctx->status, 0, 4);
    return qeng_fail(ctx, QENG_ERR_DEVICE_STATUS, "decoder_decode: a kernel reported status %d (1 = page id outside the pool, 2 = position outside the cache, 3 = token id outside the vocabulary)", status);
  }
  // device order is [step][batch]; the caller gets [batch][steps]
  for (int s = 0; s < steps; ++s)
    for (int b = 0; b < B; ++b) out_tokens[(size_t)b * steps + s] = d->h_out[(size_t)s * B + b];
  return QENG_OK;
}

int32_t qeng_decoder_logits(qeng_ctx* ctx, qeng_decoder* d, float* out) {
  if (!ctx || !d || !out) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_logits: null argument");
  if (!d->have_logits) return qeng_fail(ctx, QENG_ERR_STATE, "decoder_logits: no logits yet");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  if (d->logits_partial) {
    // sharded LM head: zero the other ranks' columns and sum over the ranks (every rank must make
    // this call); the bootstrap of the next decode call keeps using the token already picked
    const int V = d->cfg.vocab, B = d->batch;
    if (d->v0 > 0) QENG_CUDA(ctx, cudaMemset2DAsync(d->logits, (size_t)V * 4, 0, (size_t)d->v0 * 4, B, d->stream));
    if (d->v0 + d->vloc < V)
      QENG_CUDA(ctx, cudaMemset2DAsync(d->logits + d->v0 + d->vloc, (size_t)V * 4, 0, (size_t)(V - d->v0 - d->vloc) * 4, B, d->stream));
    int32_t rc = qeng_tp_all_reduce_internal(ctx, d->logits, (int64_t)B * V, d->stream);
    if (rc != QENG_OK) return rc;
    d->logits_partial = false;
  }
  QENG_CUDA(ctx, cudaStreamSynchronize(d->stream));
  QENG_CUDA(ctx, cudaMemcpy(out, d->logits, (size_t)d->batch * d->cfg.vocab * 4, cudaMemcpyDeviceToHost));
  return QENG_OK;
}

int32_t qeng_decoder_layer(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, const float* x_in, const int32_t* pos,
                           int32_t rows, float* x_out, void* stream) {
  if (!ctx || !d || !x_in || !pos || !x_out) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_layer: null argument");
  if (layer < 0 || layer >= d->cfg.layers) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_layer: bad layer");
  if (rows < 1 || rows > d->cfg.max_seq) return qeng_fail(ctx, QENG_ERR_SHAPE, "decoder_layer: bad row count");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  int32_t rc = ensure_rows(ctx, d, rows);
  if (rc != QENG_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  // all rows belong to sequence 0 (a prompt chunk or a single step)
  std::vector<int32_t> lens(rows), table((size_t)rows * d->max_pages);
  for (int r = 0; r < rows; ++r) {
    if (pos[r] < 0 || pos[r] >= d->cfg.max_seq) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_layer: position outside the cache");
    lens[r] = pos[r] + 1;
    for (int p = 0; p < d->max_pages; ++p) table[(size_t)r * d->max_pages + p] = p * d->cfg.max_batch;
  }
  QENG_CUDA(ctx, cudaMemcpyAsync(d->pos, pos, rows * 4, cudaMemcpyHostToDevice, st));
  QENG_CUDA(ctx, cudaMemcpyAsync(d->lens, lens.data(), rows * 4, cudaMemcpyHostToDevice, st));
  QENG_CUDA(ctx, cudaMemcpyAsync(d->table, table.data(), table.size() * 4, cudaMemcpyHostToDevice, st));
  d->next_ready = false;  // the activation buffer is reused
  QENG_CUDA(ctx, cudaMemcpyAsync(d->x, x_in, (size_t)rows * d->cfg.d_model * 4, cudaMemcpyDeviceToDevice, st));
  rc = run_layer(ctx, d, layer, rows, d->table, st);
  if (rc != QENG_OK) return rc;
  QENG_CUDA(ctx, cudaMemcpyAsync(x_out, d->x, (size_t)rows * d->cfg.d_model * 4, cudaMemcpyDeviceToDevice, st));
  QENG_CUDA(ctx, cudaStreamSynchronize(st));  // host staging buffers go out of scope
  return QENG_OK;
}

int32_t qeng_decoder_set_stream(qeng_ctx* ctx, qeng_decoder* d, void* stream) {
  if (!ctx || !d) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_set_stream: null argument");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  QENG_CUDA(ctx, cudaStreamSynchronize(d->stream));
  d->stream = stream ? (cudaStream_t)stream : d->own_stream;
  return QENG_OK;
}

int32_t qeng_decoder_weight(qeng_ctx* ctx, qeng_decoder* d, int32_t layer, int32_t fused_index,
                            const qeng_weight** out) {
  if (!ctx || !d || !out) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_weight: null argument");
  if (layer < 0 || layer >= d->cfg.layers || fused_index < 0 || fused_index > 3)
    return qeng_fail(ctx, QENG_ERR_ARG, "decoder_weight: bad layer/index");
  const Layer& L = d->layers[layer];
  const qeng_weight* w = fused_index == 0 ? L.wqkv : fused_index == 1 ? L.wo : fused_index == 2 ? L.wgu : L.wdown;
  if (!w) return qeng_fail(ctx, QENG_ERR_STATE, "decoder_weight: matrix not loaded yet");
  *out = w;
  return QENG_OK;
}

int32_t qeng_decoder_launches_per_step(const qeng_decoder* d) { return d ? d->launches : 0; }

int32_t qeng_decoder_config(qeng_ctx* ctx, const qeng_decoder* d, qeng_model_cfg* out) {
  if (!d || !out) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_config: null argument");
  *out = d->cfg;
  return QENG_OK;
}

int32_t qeng_decoder_step_profile(qeng_ctx* ctx, qeng_decoder* d, uint64_t* out_ns, int32_t capacity, int32_t* n_written) {
  if (!ctx || !d || !out_ns || !n_written) return qeng_fail(ctx, QENG_ERR_ARG, "decoder_step_profile: null argument");
  *n_written = 0;
  if (!d->fused) return qeng_fail(ctx, QENG_ERR_STATE, "decoder_step_profile: the fused step kernel is not in use for this decoder");
  QENG_CUDA(ctx, cudaSetDevice(ctx->device));
  return qeng_step_profile(ctx, d->fused, out_ns, capacity, n_written);
}

}  // extern "C"
