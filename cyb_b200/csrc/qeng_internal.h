// Internal declarations shared by the translation units of libqeng.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>
#include <vector>

#include "../../include/qeng.h"

// Device layout of a 4-bit block weight W[N,K] ("tile16"):
//  * rows are grouped in tiles of 16, K in chunks of 64 (two 32-blocks);
//    Kp = K rounded up to 64, the padding block has code 0 and scale 0;
//  * nibble plane: [tile][chunk][lane 0..31] one uint4 per lane; with
//    g = lane/4, t = lane%4 the four words are
//       .x = row g   , block 2c      .y = row g+8 , block 2c
//       .z = row g   , block 2c+1    .w = row g+8 , block 2c+1
//    and each word holds the codes of k = 32*block + 8*t + j in nibble j
//    (bits 4j..4j+3).  One warp-wide 128-bit load therefore fetches 512
//    contiguous bytes and every lane receives exactly the A-fragment words of
//    an m16n8k16 MMA over that chunk;
//  * scale plane: [tile][chunk][g 0..7] one uint2 = four f16:
//       (row g, blk 2c), (row g+8, blk 2c), (row g, blk 2c+1), (row g+8, blk 2c+1).
enum { QENG_FMT_Q4 = 0, QENG_FMT_Q8 = 1, QENG_FMT_K4 = 2 };

struct qeng_weight {
  int fmt = QENG_FMT_Q4;  // Q4: 4-bit codes, w = (c - 8) s; Q8: signed bytes, w = q s (both: one f16 s per 32-block);
                          // K4: 4-bit codes with f32 scale and minimum per 32-block, w = D c - M (the K-quant super-blocks, expanded)
  int64_t N, K;        // logical shape
  int64_t ntiles;      // N / 16
  int64_t nchunks;     // Kp / 64
  uint4* qs;           // weight plane: Q4 ntiles*nchunks*32 uint4 (nibbles), Q8 ntiles*nchunks*64 uint4 (bytes)
  uint2* sc;           // scale plane,  ntiles*nchunks*8 uint2 (K4: ntiles*nchunks*256 bytes)
  int64_t bytes;       // device bytes held
  const qeng_weight* next = nullptr;  // matrix the caller multiplies by after this one (L2 prefetch hint)
};

struct qeng_kv_pool {
  int64_t pages, kv_heads, hd;
  __half* data;        // [pages][kv_heads][2][16][hd]
};

struct qeng_ctx {
  int device = 0;
  int sm_count = 0;
  std::string err;
  // scratch for split-KV attention partials and device status words
  float* attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  int32_t* status = nullptr;  // device status word (0 = ok)
  // bf16 copy of f32 activations for the tensor-core prefill matmul
  void* xbf16 = nullptr;
  size_t xbf16_bytes = 0;
  // activations quantised once per decode-batch matmul (more than 4 rows), one image per K slice
  void* ximage = nullptr;
  size_t ximage_bytes = 0;
  // tensor parallelism (tp.cu)
  void* nccl_comm = nullptr;
  int tp_rank = 0, tp_world = 1;
  // peer-mapped inboxes of the one-shot all-reduce
  void* p2p_local = nullptr;
  void* p2p_peer[8] = {};
  size_t p2p_flag_off = 0, p2p_counter_off = 0;
  size_t p2p_fuse_off = 0;    // fused-decode inbox region inside the peer-mapped buffer
  bool p2p_ready = false;
  bool l2_prefetch = true;    // the streaming matmul requests the hinted next matrix into L2
  bool pdl = true;            // launch the streaming matmul with programmatic stream serialization
  // remaining switches of qeng_options
  bool p2p_allowed = true, attn_cluster = true, step_kernel = false;
  int attn_ctas_per_sm = 3, stream_groups = 0, stream_stage_chunks = 0;
  // bumped whenever attn_scratch moves: a captured graph that holds the old address is stale
  uint64_t scratch_gen = 0;
  // per-CTA argmax partials and the arrival counter of the fused LM head
  float* tail_val = nullptr;
  int32_t* tail_idx = nullptr;
  int32_t* tail_cnt = nullptr;
};

int32_t qeng_fail(qeng_ctx* ctx, int32_t code, const char* fmt, ...);

#define QENG_CUDA(ctx, expr)                                                              \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess)                                                               \
      return qeng_fail(ctx, QENG_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                       cudaGetErrorString(e__), __FILE__, __LINE__);                      \
  } while (0)

// Entry points make the context's device current (cheap when it already is).
#define QENG_ENTER(ctx)                                                                   \
  do {                                                                                    \
    int dev__ = -1;                                                                       \
    if (cudaGetDevice(&dev__) != cudaSuccess || dev__ != (ctx)->device) QENG_CUDA(ctx, cudaSetDevice((ctx)->device)); \
  } while (0)

#define QENG_LAUNCH_CHECK(ctx)                                                            \
  do {                                                                                    \
    cudaError_t e__ = cudaGetLastError();                                                 \
    if (e__ != cudaSuccess)                                                               \
      return qeng_fail(ctx, QENG_ERR_CUDA, "kernel launch failed: %s (%s:%d)",            \
                       cudaGetErrorString(e__), __FILE__, __LINE__);                      \
  } while (0)

// ---- fused entry used by the executor (gemv_q4.cu) -------------------------
// Epilogue of the fused q|k|v projection: rotary embedding, f16 rounding, q to its buffer and
// k, v straight into the page pool.  The rows of every 128-row head are stored permuted so that
// MMA rows g / g+8 of one tile are the rotary pair (i, i+64): tile j of a head holds dims
// 8j..8j+7 then 64+8j..64+8j+7.
struct qeng_qkv_epi {
  const int32_t* pos;      // [M] token position of each activation row
  const int32_t* table;    // [M][max_pages]
  const float* cs;         // [max_seq][64 cos | 64 sin]
  __half* q16;             // [M][Hq][128]
  __half* pool;            // [pages][Hkv][2][16][128]
  int max_pages, pages, Hq, Hkv, max_seq;
};

struct qeng_gemm_fuse {
  const float* norm_gamma = nullptr;  // if set: x is RMS-normalised (gain gamma) while it is staged
  float norm_eps = 0.f;
  int epilogue = 0;                   // see QENG_EPI_*
  const float* resid = nullptr;       // QENG_EPI_RESID: y = resid + x.W^T
  const qeng_qkv_epi* qkv = nullptr;  // QENG_EPI_QKV (streaming kernel only)
  bool two_limbs = false;             // a single activation row in 15 instead of 22 bits (QENG_GEMM_FAST_F16)
  // Tensor parallelism without a collective of its own (decode steps of up to kTpFuseRows rows):
  //   tp_push_kind >= 0: the epilogue sends this rank's partial sums, tagged, to every rank's inbox
  //                      of that kind (0: after o, 1: after down) instead of writing y;
  //   tp_gather_kind >= 0: the staging first adds all ranks' parts of that kind (tag of tp_gather_layer)
  //                      onto x, in rank order, and CTA 0 writes the updated rows back to x.
  int tp_push_kind = -1, tp_gather_kind = -1, tp_layer = 0, tp_gather_layer = 0, tp_layers = 1;
  float* tp_writeback = nullptr;      // where CTA 0 leaves the gathered rows: NOT x itself (other CTAs still read x)
};
constexpr int kTpFuseRows = 16;      // activation rows an inbox holds
constexpr int kTpFuseDm = 8192;      // widest residual stream an inbox holds
// bytes of the fused-decode inbox region: [2 kinds][world][kTpFuseRows][kTpFuseDm] (value, tag) pairs
inline size_t qeng_tp_fuse_bytes(int world) { return (size_t)2 * world * kTpFuseRows * kTpFuseDm * 8; }
// SWIGLU: rows g (gate) and g+8 (up) of every 16-row tile are combined into one
// output y[8*tile + g] = silu(gate) * up, so y has N/2 columns.
enum { QENG_EPI_STORE = 0, QENG_EPI_ACCUM = 1, QENG_EPI_RESID = 2, QENG_EPI_SWIGLU = 3, QENG_EPI_QKV = 4 };

int32_t qeng_gemm_q4_decode(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype,
                            int64_t M, int64_t ldx, float* y, int64_t ldy, bool split_f32,
                            const qeng_gemm_fuse& fuse, cudaStream_t stream);

// attn_decode.cu: size the context's split scratch for a shape (may allocate; never call while capturing)
int32_t qeng_attn_reserve(qeng_ctx* ctx, int64_t B, int64_t Hq, int64_t Hkv, int64_t max_pages);

// gemv_q4_stream.cu: the persistent bulk-copy kernel; *handled = false when the shape does not fit it
int32_t qeng_gemm_q4_stream(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M,
                            int64_t ldx, float* y, int64_t ldy, const qeng_gemm_fuse& fuse, cudaStream_t stream,
                            bool* handled);
// true when the streaming kernel takes this shape (its fused-only epilogues may then be used)
bool qeng_gemm_q4_stream_fits(const qeng_ctx* ctx, const qeng_weight* w, int64_t M);
int32_t qeng_gemm_q4_stream_reserve(qeng_ctx* ctx, const qeng_weight* w, int64_t M);

// ops.cu: LM head with optional fused RMSNorm and optional greedy finalisation (argmax over the
// vocabulary, record the token, advance the sequences, gather the next embedding) in one launch.
struct qeng_lm_tail {
  const uint16_t* table = nullptr;  // bf16 [V][D]
  const float* x = nullptr;         // [M][D]
  int M = 0, D = 0, V = 0;
  float* logits = nullptr;          // [M][V]
  const float* gamma = nullptr;     // fused RMSNorm gain (null = x is used as is)
  float eps = 0.f;
  int32_t* next = nullptr;          // [M] sampled token (null = no finalisation)
  const uint16_t* emb = nullptr;    // bf16 [V][D]
  float* xout = nullptr;            // [M][D] embedding of the sampled token
  int32_t* pos = nullptr;           // [M] += 1
  int32_t* lens = nullptr;          // [M] += 1
  int32_t* out_tokens = nullptr;    // out_tokens[(*step + 1) * M + m] = token
  int32_t* step = nullptr;          // += 1
  // vocabulary shard (tensor parallelism): `table` holds rows [v0, v0 + V) of a Vtot-row head;
  // logits row m starts at logits + m * ldl and this launch fills columns [v0, v0 + V)
  int v0 = 0, Vtot = 0, ldl = 0;    // Vtot = 0 means unsharded (Vtot = ldl = V)
  float* pairs = nullptr;           // instead of finalising: pairs[2 * (pair_slot + m)] = (max, index as f32)
  int pair_slot = 0;
  float softcap = 0.f;              // > 0: the logits written are softcap * tanh(logit / softcap); the
                                    // sampling compares the raw values (the map is monotonic)
};
int32_t qeng_lm_head_fused(qeng_ctx* ctx, const qeng_lm_tail& t, cudaStream_t stream);

// decode_step.cu: all layers of one decode step (1 or 2 rows) in one persistent cooperative kernel
struct qeng_step;
struct qeng_step_layer_desc {
  const qeng_weight* w[4];  // q|k|v, o, gate|up (interleaved), down
  const float *norm1, *norm2;
  __half* pool;             // this layer's KV pages
};
struct qeng_step_desc {
  std::vector<qeng_step_layer_desc> layers;
  int dm = 0, F = 0, Hq = 0, Hkv = 0, max_pages = 0, pages = 0, max_seq = 0;
  float eps = 0.f;
  float* x = nullptr;                 // [rows][dm] residual stream, read and rewritten by a step
  const int32_t *pos = nullptr, *lens = nullptr, *table = nullptr;
  const float* cs = nullptr;
  __half* q16 = nullptr;
  float* act = nullptr;
  int world = 1, rank = 0;
  void* peer_inbox[8] = {};           // world > 1: every rank's inbox as mapped here (own included)
};
// *out stays null when the shapes are outside what the kernel takes, or the context disabled it
int32_t qeng_step_create(qeng_ctx* ctx, const qeng_step_desc& d, qeng_step** out);
void qeng_step_free(qeng_step* s);
bool qeng_step_takes(const qeng_step* s, int B);
int32_t qeng_step_launch(qeng_ctx* ctx, qeng_step* s, int B, cudaStream_t stream);
size_t qeng_step_inbox_bytes(int world, int dm);
int32_t qeng_step_profile(qeng_ctx* ctx, qeng_step* s, uint64_t* out, int32_t capacity, int32_t* n);

// tp.cu
int32_t qeng_tp_all_reduce_internal(qeng_ctx* ctx, float* buf, int64_t n, cudaStream_t stream);
void qeng_tp_release(qeng_ctx* ctx);
bool qeng_tp_p2p_ready(const qeng_ctx* ctx, int64_t n);
int32_t qeng_tp_allreduce_add(qeng_ctx* ctx, float* dst, const float* part, int64_t n, cudaStream_t stream);
// fused decode (the matmuls carry the collective): see qeng_gemm_fuse::tp_push_kind
bool qeng_tp_fuse_ready(const qeng_ctx* ctx, int64_t rows, int64_t dm);
uint2* qeng_tp_fuse_inbox(const qeng_ctx* ctx, int r, int kind);
const unsigned* qeng_tp_fuse_seq(const qeng_ctx* ctx);
int32_t qeng_tp_fuse_gather(qeng_ctx* ctx, float* x, int64_t rows, int64_t dm, int kind, int layer, int layers, cudaStream_t stream);
int32_t qeng_tp_fuse_advance(qeng_ctx* ctx, cudaStream_t stream);

// gemm_q4_tc.cu: tcgen05 prefill matmul (bf16 operands, f32 accumulation in tensor memory)
int32_t qeng_gemm_q4_prefill(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype, int64_t M, int64_t ldx,
                             float* y, int64_t ldy, int accumulate, cudaStream_t stream);
constexpr int64_t kPrefillRows = 256;  // from this many rows on, matmuls take the tensor-core path

void qeng_weight_dequant_q8(const qeng_weight* w, float* out, cudaStream_t stream);
void qeng_weight_dequant_k4(const qeng_weight* w, float* out, cudaStream_t stream);
// 4-bit codes [N][K] and f32 (scale, minimum) pairs [N][K/32][2] (HOST) -> device weight; and the
// expansion of Q4_K super-blocks into that form
int32_t qeng_weight_pack_k4(qeng_ctx* ctx, const uint8_t* q, const float* dm, int64_t N, int64_t K, qeng_weight** out);
int32_t qeng_q4k_expand(qeng_ctx* ctx, const uint8_t* blocks, int64_t N, int64_t K, std::vector<uint8_t>* q, std::vector<float>* dm);

#if defined(QENG_TRACE) && defined(__CUDACC__)
// tuning builds only: a launch log behind the status word (status + 256 bytes: a counter, then records
// of 8 u64: kind, then %globaltimer stamps)
__device__ __forceinline__ unsigned long long qeng_trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned long long* qeng_trace_open(int32_t* status, unsigned long long kind) {
  unsigned long long* log = reinterpret_cast<unsigned long long*>(status) + 32;
  const unsigned long long idx = atomicAdd(log, 1ull);
  if (idx >= 30000ull) return log + 8;  // overflow: everything lands in record 0
  unsigned long long* rec = log + 8 + idx * 8;
  rec[0] = kind;
  rec[1] = qeng_trace_now();
  return rec;
}
#endif

