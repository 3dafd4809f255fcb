/* qeng — C ABI of the B200 (sm_100a) engine for cyb's local-LLM hot path.
 *
 * This is the surface a Rust host binds with `extern "C"`.  cyb reaches its
 * model runtime through soma-kernel -> glia `run` (shell/Cargo.toml:34,
 * Cargo.lock:8444-8462, 9091-9101); `run`'s per-backend operator set executes
 * the loop "embed -> per layer: norm, QKV, RoPE, KV cache, attention, O proj,
 * norm, FFN -> LM head -> sample" (decide/pipeline.md:51).  Each entry point
 * below replaces one operator of that loop (or the whole loop) on a B200.
 *
 * Conventions
 *  - every call returns an int32 status (QENG_OK = 0, negative = error) and
 *    never throws or aborts; qeng_last_error() gives the text of the last
 *    failure on that context;
 *  - a context is bound to one CUDA device and is used by one host thread at a
 *    time; one context per GPU for tensor parallelism;
 *  - activation / output pointers are DEVICE pointers owned by the caller;
 *    packed weights, KV pools and decoders are opaque handles owned by the
 *    engine; `stream` is a cudaStream_t passed as void* (NULL = default
 *    stream); work is asynchronous on that stream unless stated otherwise;
 *  - there is no CPU fallback: an unsupported shape is an error.
 */
#ifndef QENG_H_
#define QENG_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  QENG_OK = 0,
  QENG_ERR_ARG = -1,     /* null pointer, bad enum, value out of range */
  QENG_ERR_SHAPE = -2,   /* shape the kernels do not support */
  QENG_ERR_ALIGN = -3,   /* pointer or leading dimension not aligned */
  QENG_ERR_CUDA = -4,    /* a CUDA runtime call failed */
  QENG_ERR_NCCL = -5,    /* an NCCL call failed */
  QENG_ERR_TIMEOUT = -6, /* a bounded device-side wait ran out */
  QENG_ERR_DEVICE_STATUS = -7, /* a kernel reported an error through its status word */
  QENG_ERR_STATE = -8    /* call not valid in the object's current state */
};

/* element types of activation buffers */
enum { QENG_F32 = 0, QENG_F16 = 1, QENG_BF16 = 2 };

/* flags of qeng_gemm_q4 */
enum {
  QENG_GEMM_ACCUMULATE = 1, /* y += x.W^T instead of y = x.W^T (fused residual add) */
  QENG_GEMM_FAST_F16 = 2    /* a single activation row is quantised to 15 bits per 32-block
                               instead of 22 (a little faster; costs ~6e-5 of the error
                               budget instead of ~5e-7); no effect for 2 or more rows, which
                               always use 15 bits */
};

typedef struct qeng_ctx qeng_ctx;
typedef struct qeng_weight qeng_weight;
typedef struct qeng_kv_pool qeng_kv_pool;
typedef struct qeng_decoder qeng_decoder;

/* ---- context (replaces the backend object glia `run` creates per device;
 *      named "cpu . wgpu . honeycrisp" in decide/model-lifecycle.md:25) ------- */
int32_t qeng_version(void);
int32_t qeng_create(int32_t device, qeng_ctx** out);
/* Tuning switches of a context: a plain struct, fixed at creation (the library reads no
 * environment variable).  Zero-initialise, set struct_size = sizeof(qeng_options), then change
 * what you need; a field left at 0 keeps its default.  Results never depend on any of them
 * beyond f32 summation order. */
typedef struct qeng_options {
  int32_t struct_size;       /* sizeof(qeng_options) of the caller's header */
  int32_t no_pdl;            /* 1: launch the decode matmuls without programmatic dependent launch */
  int32_t no_l2_prefetch;    /* 1: ignore qeng_weight_set_next hints */
  int32_t no_p2p_allreduce;  /* 1: small all-reduces go through NCCL instead of the peer-store kernel */
  int32_t no_attn_cluster;   /* 1: decode attention always uses fixed splits + scratch */
  int32_t attn_ctas_per_sm;  /* CTAs per SM the split-KV attention aims for (default 3: one resident wave) */
  int32_t stream_groups;     /* tile groups of the streaming matmul: 1, 2 or 4 (default: by shape) */
  int32_t step_kernel;       /* 1: decode steps of 1 or 2 sequences run all layers in one persistent cooperative
                                kernel (tagged data flow between the operators) instead of one kernel per operator */
  int32_t stream_stage_chunks; /* 64-wide K chunks per shared-memory ring stage of the streaming matmul: 4..64
                                  (default 16) */
} qeng_options;
int32_t qeng_create_opts(int32_t device, const qeng_options* opts, qeng_ctx** out);
int32_t qeng_destroy(qeng_ctx* ctx);
const char* qeng_last_error(const qeng_ctx* ctx);
/* Drain the device, read and clear the status word kernels write when they meet a
 * malformed input (page id outside the pool, position outside the cache, token
 * outside the vocabulary): QENG_OK or QENG_ERR_DEVICE_STATUS. */
int32_t qeng_device_status(qeng_ctx* ctx);
/* SM count of the context's device (grid sizing, reporting). */
int32_t qeng_sm_count(const qeng_ctx* ctx);

/* ---- tensor parallelism (not in the reference: its runtime is single-device; the
 *      sharding is BASELINE's: column-split q/k/v/gate/up, row-split o/down, one sum
 *      after each row-split projection) ----------------------------------------------
 * One context per GPU and rank.  Rank 0 makes an id, the host program hands the 128
 * bytes to every rank (any channel), every rank calls qeng_tp_init (collective). */
int32_t qeng_tp_unique_id(uint8_t* out128);
int32_t qeng_tp_init(qeng_ctx* ctx, int32_t rank, int32_t world, const uint8_t* id128);
/* Optional, after qeng_tp_init: map every rank's inbox into every peer (CUDA IPC) so that the
 * small all-reduces of decode run as one low-latency push kernel over NVLink instead of NCCL.
 * Each rank exports 64 bytes with qeng_tp_p2p_handle; the host program gathers the world*64
 * bytes (rank order) and gives them to qeng_tp_p2p_open on every rank. */
int32_t qeng_tp_p2p_handle(qeng_ctx* ctx, uint8_t* out64);
int32_t qeng_tp_p2p_open(qeng_ctx* ctx, const uint8_t* handles);
/* Recovery after a peer failed to join (device status 5): the ranks' call counters no longer
 * agree.  With no collective in flight anywhere, every surviving rank calls this (it clears its
 * own inbox, call counter and status word), the host program makes sure all have returned (a
 * barrier on its own channel), and the one-shot all-reduce works again. */
int32_t qeng_tp_p2p_reset(qeng_ctx* ctx);
/* dst[n] += sum over ranks of part[n] (f32, device): the collective after a row-split projection
 * fused with the residual add.  Uses the one-shot peer-memory kernel when the peers are mapped
 * and n <= 65536 (n % 4 == 0), else NCCL followed by an add. */
int32_t qeng_tp_all_reduce_add_f32(qeng_ctx* ctx, float* dst, float* part, int64_t n, void* stream);
/* In-place sum of buf[n] (f32, device) over the ranks, on `stream` (NCCL over NVLink). */
int32_t qeng_tp_all_reduce_f32(qeng_ctx* ctx, float* buf, int64_t n, void* stream);

/* ---- 4-bit block weights ("Q4_0 ... for all backends", decide/pipeline.md:38,59;
 *      "tensor data (Q4/Q8/F16/F32)", decide/pipeline.md:28) --------------------
 * Import: q[N*K] holds one code 0..15 per byte (row-major, K contiguous),
 * s[N*K/32] one IEEE f16 bit pattern per 32 consecutive K.  Both are HOST
 * pointers; the call validates the codes, re-tiles them into the device layout
 * and uploads (synchronous).  K % 32 == 0, N % 16 == 0. */
int32_t qeng_weight_pack_q4(qeng_ctx* ctx, const uint8_t* q, const uint16_t* s,
                            int64_t N, int64_t K, qeng_weight** out);
/* Inverse, computed ON THE DEVICE from the packed layout (the bit-exactness
 * check): writes N*K codes and N*K/32 scales to HOST buffers (synchronous). */
int32_t qeng_weight_unpack_q4(qeng_ctx* ctx, const qeng_weight* w, uint8_t* q, uint16_t* s);
/* Device-side dequantisation to f32 [N,K] (device pointer), w = (q-8)*s. */
int32_t qeng_weight_dequant_f32(qeng_ctx* ctx, const qeng_weight* w, float* out, void* stream);
/* Import-time quantiser on the device ("Q4 (4-bit, 3.5x compression)" at import,
 * decide/pipeline.md:38-40,59): w_dev is a DEVICE matrix [N,K] of x_dtype (QENG_F32 / F16 / BF16)
 * with leading dimension ld.  Per 32-block the element of largest magnitude (first on ties) / -8
 * becomes the f16 scale d, and code = min(15, trunc(x / d + 8.5)) computed as x * (1/d) in f32.
 * The result is written directly in the device layout, asynchronously on `stream`; w_dev may be
 * released once the stream has passed this call.  K % 32 == 0, N % 16 == 0. */
int32_t qeng_weight_quantize_q4(qeng_ctx* ctx, const void* w_dev, int32_t x_dtype, int64_t N, int64_t K, int64_t ld,
                                qeng_weight** out, void* stream);
/* ---- 8-bit block weights ("tensor data (Q4/Q8/F16/F32)", decide/pipeline.md:28; the default
 *      model of the reference's catalog was imported as q8, shell/src/worlds/models/mod.rs:68-73)
 * w = q * s with q a signed byte and one f16 scale per 32 consecutive K (the published Q8_0 block).
 * A weight handle of this format is taken by qeng_gemm_q4 / qeng_gemv_q4 (any M: rows in passes of
 * 16 through the decode kernel; the tensor-core prefill kernel is for 4-bit blocks only),
 * qeng_weight_dequant_f32, qeng_weight_set_next and the getters.  Same shape rules as the 4-bit calls. */
int32_t qeng_weight_pack_q8(qeng_ctx* ctx, const int8_t* q, const uint16_t* s, int64_t N, int64_t K, qeng_weight** out);
/* Inverse, computed ON THE DEVICE from the packed layout: N*K bytes and N*K/32 scales to HOST buffers. */
int32_t qeng_weight_unpack_q8(qeng_ctx* ctx, const qeng_weight* w, int8_t* q, uint16_t* s);
/* Import-time quantiser on the device: per 32-block d = max|x| / 127 in f32 (stored as f16),
 * q = round-half-away(x * (1/d)).  Asynchronous on `stream`. */
int32_t qeng_weight_quantize_q8(qeng_ctx* ctx, const void* w_dev, int32_t x_dtype, int64_t N, int64_t K, int64_t ld,
                                qeng_weight** out, void* stream);
/* ---- "K-quant" 4-bit weights ("needs fused Q4_K matmul": what kept a catalog model from loading,
 *      decide/model-lifecycle.md:175).  blocks: HOST, row-major [N][K/256] super-blocks of 144 bytes in
 * the published Q4_K layout (f16 d, f16 dmin, 12 bytes holding eight 6-bit scales and eight 6-bit
 * minima, 128 bytes of codes: of every 32 bytes the low nibbles are sub-block 2i, the high nibbles
 * sub-block 2i+1); w = (d * sc_j) * code - (dmin * m_j).  K % 256 == 0, N % 16 == 0.  The weight is
 * expanded to per-32-block f32 (scale, minimum) pairs on the device (0.75 B per weight) and taken by
 * qeng_gemm_q4 / qeng_gemv_q4 (decode kernel, 4 rows per pass), qeng_weight_dequant_f32, the getters. */
int32_t qeng_weight_pack_q4k(qeng_ctx* ctx, const uint8_t* blocks, int64_t N, int64_t K, qeng_weight** out);
/* Inverse of the device layout (the bit-exactness check): codes [N][K] (0..15) and f32 pairs
 * (scale, minimum) [N][K/32][2] to HOST buffers. */
int32_t qeng_weight_unpack_k4(qeng_ctx* ctx, const qeng_weight* w, uint8_t* q, float* scale_min);
int32_t qeng_weight_free(qeng_ctx* ctx, qeng_weight* w);
int64_t qeng_weight_rows(const qeng_weight* w);
int64_t qeng_weight_cols(const qeng_weight* w);
int64_t qeng_weight_device_bytes(const qeng_weight* w);
/* The block format held: 4 (4-bit blocks, f16 scale), 8 (8-bit blocks), 14 (4-bit K-quant blocks with
 * scale and minimum). */
int32_t qeng_weight_format(const qeng_weight* w);
/* Hint: the matmul the caller runs after one over `w` is over `next` (NULL clears the hint).
 * The decode kernel then asks L2 for `next` while it finishes `w`, so that HBM keeps
 * streaming across the kernel boundary.  Results never depend on the hint.  `next` must stay
 * alive while the hint is set.  The reference has no counterpart: its loop order
 * (decide/pipeline.md:51) is what makes the next matrix known. */
int32_t qeng_weight_set_next(qeng_ctx* ctx, qeng_weight* w, const qeng_weight* next);

/* ---- quantized matmul (the "QKV / O proj / FFN" steps of decide/pipeline.md:51)
 * y[M,N] (f32, leading dimension ldy) = x[M,K] (x_dtype, leading dimension ldx)
 * . dequant(W)^T, f32 accumulation.  M < 256 runs the decode kernels (weights unpacked in
 * registers, activations in block fixed point: 22 bits for one row, 15 bits per row otherwise,
 * integer tensor-core contraction, per-block f32 scaling); M >= 256 the tensor-core prefill kernel, which rounds
 * activations and dequantised weights to bf16 (tolerance 5e-3 instead of 2e-3). */
int32_t qeng_gemm_q4(qeng_ctx* ctx, const qeng_weight* w, const void* x, int32_t x_dtype,
                     int64_t M, int64_t ldx, float* y, int64_t ldy, int32_t flags, void* stream);
/* M = 1, f32 activations: the decode GEMV. */
int32_t qeng_gemv_q4(qeng_ctx* ctx, const qeng_weight* w, const float* x, float* y, void* stream);

/* ---- small operators of the loop ------------------------------------------- */
/* y = x * gamma / sqrt(mean(x^2) + eps), rows of length D
 * ("norm = rms", decide/compile.md:95). */
int32_t qeng_rmsnorm(qeng_ctx* ctx, const float* x, const float* gamma, int64_t M, int64_t D,
                     float eps, float* y, void* stream);
/* In-place rotary embedding of x[M,H,hd] at integer positions pos[M]; pairs
 * (i, i+hd/2), angle pos*base^(-2i/hd) ("RoPE", decide/pipeline.md:51). */
int32_t qeng_rope(qeng_ctx* ctx, float* x, const int32_t* pos, int64_t M, int64_t H, int64_t hd,
                  float base, void* stream);
/* y = silu(gate) * up  ("ffn = swiglu", decide/compile.md:97). */
int32_t qeng_swiglu(qeng_ctx* ctx, const float* gate, const float* up, int64_t n, float* y, void* stream);
/* y = a + b (residual). */
int32_t qeng_add(qeng_ctx* ctx, const float* a, const float* b, int64_t n, float* y, void* stream);
/* x[M,D] f32 = table[tokens[m], :] for a bf16 table [V,D] ("embed"). */
int32_t qeng_embed(qeng_ctx* ctx, const uint16_t* table_bf16, const int32_t* tokens, int64_t M,
                   int64_t D, int64_t V, float* x, void* stream);
/* logits[M,V] f32 = x[M,D] f32 . table[V,D]^T, bf16 table ("LM head"). */
int32_t qeng_lm_head(qeng_ctx* ctx, const uint16_t* table_bf16, const float* x, int64_t M,
                     int64_t D, int64_t V, float* logits, void* stream);
/* idx[m] = lowest index of the maximum of row m ("sample", greedy). */
int32_t qeng_argmax(qeng_ctx* ctx, const float* logits, int64_t M, int64_t V, int32_t* idx, void* stream);

/* ---- KV cache and decode attention ("KV cache", "attention" of
 *      decide/pipeline.md:51; f16 KV, decide/runtime.md:35; GQA,
 *      decide/compile.md:96) ---------------------------------------------------
 * The pool is f16 [pages][kv_heads][2 (K,V)][16 tokens][hd]; a page table row
 * lists the pages of one sequence in order. hd must be 128. */
int32_t qeng_kv_pool_create(qeng_ctx* ctx, int64_t pages, int64_t kv_heads, int64_t hd, qeng_kv_pool** out);
int32_t qeng_kv_pool_free(qeng_ctx* ctx, qeng_kv_pool* pool);
/* device pointer of the pool's storage (tests upload prepared caches through it) */
void* qeng_kv_pool_data(const qeng_kv_pool* pool);
int64_t qeng_kv_pool_pages(const qeng_kv_pool* pool);
/* Append one token per sequence: k,v f32 [B,kv_heads,hd] rounded to f16 and
 * written at token index pos[b] of sequence b. */
int32_t qeng_kv_append(qeng_ctx* ctx, qeng_kv_pool* pool, const float* k, const float* v,
                       const int32_t* page_table, int64_t max_pages, const int32_t* pos, int64_t B,
                       void* stream);
/* out[B,Hq,hd] f32 = softmax(q K^T * scale) V per sequence over its first
 * lens[b] cached tokens; q f16 [B,Hq,hd]; split over the KV length with a
 * merge of the partial (max, sum, out) triples.  Uses scratch owned by ctx. */
int32_t qeng_attn_decode(qeng_ctx* ctx, const qeng_kv_pool* pool, const uint16_t* q_f16,
                         const int32_t* page_table, int64_t max_pages, const int32_t* lens,
                         int64_t B, int64_t Hq, float scale, float* out, void* stream);

/* The same with the two attention deltas of the Gemma family, which the reference lists among
 * what stopped its own catalog models ("Gemma extensions absent (softcapping, sliding window)",
 * decide/model-lifecycle.md:175-176): softcap > 0 replaces the logits q.k*scale by
 * softcap * tanh(q.k*scale / softcap); window > 0 attends only the last `window` cached tokens of
 * every sequence (pages wholly before the window are not read).  0 switches either off. */
int32_t qeng_attn_decode_ex(qeng_ctx* ctx, const qeng_kv_pool* pool, const uint16_t* q_f16,
                            const int32_t* page_table, int64_t max_pages, const int32_t* lens,
                            int64_t B, int64_t Hq, float scale, float softcap, int32_t window,
                            float* out, void* stream);

/* Same result as qeng_attn_decode, for callers that cannot allocate device memory
 * while they run: hosts that give the engine a fixed memory budget at start-up and
 * forbid later growth, or token loops that must never enter the CUDA allocator.
 * (No counterpart in the reference: its runtime owns all memory itself.)
 * The split partials go to a 4 MiB array built into the library (held on every GPU
 * that loads it, until exit) instead of context-owned scratch; the call makes no
 * cudaMalloc/cudaFree and calls no allocating library routine.  Limit:
 * B * Hq * splits * 130 <= 1048576 floats, where splits = ceil(max_pages /
 * pages_per_split) as the engine chooses it (e.g. 16 sequences x 32 heads x 15
 * splits); larger shapes return QENG_ERR_SHAPE with the sizes in the error text.
 * The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress), so make that first call outside any stream capture.
 * All calls on a device share the array: two calls whose kernels overlap on the GPU
 * (different streams, or different contexts on one device) race; calls on one
 * stream are ordered and safe.  Nothing in the array has to start at zero. */
int32_t qeng_attn_decode_noalloc(qeng_ctx* ctx, const qeng_kv_pool* pool, const uint16_t* q_f16,
                                 const int32_t* page_table, int64_t max_pages, const int32_t* lens,
                                 int64_t B, int64_t Hq, float scale, float* out, void* stream);

/* ---- the layer executor (the whole loop of decide/pipeline.md:51; what
 *      soma-kernel drives between SomaEvent::Prefill and SomaEvent::Answer,
 *      shell/src/worlds/soma_bridge.rs:244-277) -------------------------------- */
typedef struct qeng_model_cfg {
  int32_t layers, d_model, ffn, heads, kv_heads, head_dim, vocab;
  float rms_eps, rope_base;
  int32_t max_batch; /* sequences decoded together */
  int32_t max_seq;   /* tokens per sequence the KV pool is sized for */
  int32_t tp_rank, tp_world; /* tensor-parallel position of this context */
  float attn_softcap;        /* > 0: attention logits are soft-capped, softcap * tanh(logit / softcap) */
  int32_t sliding_window;    /* > 0: every layer attends only the last `sliding_window` tokens */
  float final_softcap;       /* > 0: the logits returned are final_softcap * tanh(logit / final_softcap) (Gemma);
                                greedy sampling is unchanged (the map is monotonic) */
} qeng_model_cfg;

/* matrices of one layer, in the order of the decode loop */
enum { QENG_W_Q = 0, QENG_W_K = 1, QENG_W_V = 2, QENG_W_O = 3, QENG_W_GATE = 4, QENG_W_UP = 5, QENG_W_DOWN = 6 };

int32_t qeng_decoder_create(qeng_ctx* ctx, const qeng_model_cfg* cfg, qeng_decoder** out);
int32_t qeng_decoder_free(qeng_ctx* ctx, qeng_decoder* dec);
/* Load one linear weight of one layer from HOST codes/scales of the FULL
 * (unsharded) matrix [N,K]; the decoder keeps this rank's shard only. */
int32_t qeng_decoder_load_matrix(qeng_ctx* ctx, qeng_decoder* dec, int32_t layer, int32_t which,
                                 const uint8_t* q, const uint16_t* s, int64_t N, int64_t K);
/* The same for 8-bit blocks (q: one signed byte per weight).  The matrices that the executor fuses
 * (q, k, v of a layer; gate, up of a layer) must come in one format; prompts of layers with 8-bit
 * blocks run through the decode kernels in passes of 16 rows. */
int32_t qeng_decoder_load_matrix_q8(qeng_ctx* ctx, qeng_decoder* dec, int32_t layer, int32_t which,
                                    const int8_t* q, const uint16_t* s, int64_t N, int64_t K);
/* The same for Q4_K super-blocks (see qeng_weight_pack_q4k); decode steps of up to 4 sequences take
 * such layers in one pass, larger batches and prompts in passes of 4 rows. */
int32_t qeng_decoder_load_matrix_q4k(qeng_ctx* ctx, qeng_decoder* dec, int32_t layer, int32_t which,
                                     const uint8_t* blocks, int64_t N, int64_t K);
/* RMSNorm gains of a layer (which = 0: before attention, 1: before FFN), HOST f32[d_model].
 * which = 2 / 3: optional per-head gains of q / k, HOST f32[head_dim] ("QK-norm", named as a
 * blocker for the catalog's Qwen3 models in decide/model-lifecycle.md:173-176): every q and k head
 * is RMS-normalised over its head_dim values before the rotary embedding; load both or neither. */
int32_t qeng_decoder_load_norm(qeng_ctx* ctx, qeng_decoder* dec, int32_t layer, int32_t which, const float* gamma);
/* Embedding table, LM head (bf16 bit patterns, HOST, [vocab,d_model]) and final norm gain.
 * With tensor parallelism pass the FULL head: a rank keeps vocabulary rows
 * [rank*vocab/world, (rank+1)*vocab/world) when vocab divides evenly (else the whole head), and
 * a decode step exchanges one (max, index) pair per sequence and rank to pick the token. */
int32_t qeng_decoder_load_head(qeng_ctx* ctx, qeng_decoder* dec, const uint16_t* emb, const uint16_t* lm_head,
                               const float* final_gamma);
/* The configuration a decoder was created with. */
int32_t qeng_decoder_config(qeng_ctx* ctx, const qeng_decoder* dec, qeng_model_cfg* out);
/* ---- `.model` containers (".cyb -> graph IR ... tensor index, tensor data (Q4/Q8/F16/F32)",
 *      decide/pipeline.md:28-30; container rules reference/format.md:16-18,110-117; the reference
 *      maps its model files, shell/src/lib.rs:31-33).  The tensor-index schema is this engine's own
 *      (the `cyb-model` page is not in the reference checkout): sections `config` (TOML keys
 *      hidden_size, intermediate_size, num_hidden_layers, num_attention_heads, num_key_value_heads,
 *      head_dim, vocab_size, rms_norm_eps, rope_theta, optional attn_logit_softcapping,
 *      sliding_window, final_logit_softcapping), `tensors` ([[tensor]] tables: name, dtype
 *      "Q4" | "Q8" | "F32" | "F16" | "BF16", shape, offset, size) and `weights` (binary).
 * Read a container's `config` into a qeng_model_cfg (max_batch = 1, max_seq = 0, tp = 1/0: the
 * caller sets those before qeng_decoder_create) and count its tensors.  ctx may be NULL. */
int32_t qeng_model_file_config(qeng_ctx* ctx, const char* path, qeng_model_cfg* out, int64_t* n_tensors);
/* Load every layer matrix, norm gain, embedding and LM head of a container into a decoder whose
 * configuration matches the file's (with tensor parallelism every rank reads the same file and
 * keeps its shard).  Q4 tensors are re-tiled from the mapped file; F32 / F16 / BF16 linear weights
 * are quantised on the device first; `lm_head.weight` may be absent (tied to the embedding);
 * `self_attn.q_norm / k_norm` are optional.  Synchronous. */
int32_t qeng_decoder_load_file(qeng_ctx* ctx, qeng_decoder* dec, const char* path);
/* Forget all sequences (KV lengths to zero). */
int32_t qeng_decoder_reset(qeng_ctx* ctx, qeng_decoder* dec, int32_t batch);
/* Prompt phase: tokens HOST int32 [batch, T]; fills the KV cache and leaves the
 * logits of the last prompt position.  Synchronous.  batch * T rows are processed at once (buffers
 * grow to that size on first use: about 150 KB per row at the 7B shape); from 256 rows on, layers of
 * 4-bit blocks take the tensor-core matmul.  Attention runs the decode kernel over the prompt rows in
 * launches of 2048 rows, so its KV traffic grows with T^2; feed long prompts in chunks (successive
 * calls append) to bound memory and to report progress. */
int32_t qeng_decoder_prefill(qeng_ctx* ctx, qeng_decoder* dec, const int32_t* tokens, int32_t batch, int32_t T);
/* Greedy decode: runs `steps` steps; each step samples from the current logits,
 * feeds the sampled token and computes the next logits.  Writes the sampled
 * tokens to HOST out_tokens [batch, steps].  Synchronous. */
int32_t qeng_decoder_decode(qeng_ctx* ctx, qeng_decoder* dec, int32_t steps, int32_t* out_tokens);
/* Copy the current logits [batch, vocab] (f32) to a HOST buffer.  With a vocabulary-sharded LM
 * head this is a collective call after a decode step (the columns are summed over the ranks):
 * every rank must make it. */
int32_t qeng_decoder_logits(qeng_ctx* ctx, qeng_decoder* dec, float* out);
/* Teacher-forced single layer for parity checks: x_in DEVICE f32 [batch,d_model]
 * at positions pos (HOST int32[batch]) -> x_out DEVICE f32 [batch,d_model];
 * appends to the KV cache of that layer. */
int32_t qeng_decoder_layer(qeng_ctx* ctx, qeng_decoder* dec, int32_t layer, const float* x_in,
                           const int32_t* pos, int32_t batch, float* x_out, void* stream);
/* Run prefill/decode on the caller's stream (NULL = the decoder's own stream), so
 * that the caller's events bracket the work. */
int32_t qeng_decoder_set_stream(qeng_ctx* ctx, qeng_decoder* dec, void* stream);
/* The packed weights the executor holds for one layer, as fused for the kernels:
 * 0 = q|k|v rows concatenated, 1 = o, 2 = gate/up interleaved 8/8 per 16 rows,
 * 3 = down.  Borrowed handle (valid until the matrix is reloaded or the decoder freed). */
int32_t qeng_decoder_weight(qeng_ctx* ctx, qeng_decoder* dec, int32_t layer, int32_t fused_index,
                            const qeng_weight** out);
/* Kernel launches issued per decode step (for reporting). */
int32_t qeng_decoder_launches_per_step(const qeng_decoder* dec);
/* Where the last fused decode step spent its time: device timestamps in nanoseconds, laid out
 * [2 CTAs: the grid's first and last][layers][16 stamps].  Stamps of a layer: 0 start, 1 residual
 * gathered, 2 q|k|v staged, 3 q|k|v done, 4 barrier passed, 5 attention done, 6 barrier passed,
 * 7 o staged, 8 o done, 9 residual gathered, 10 gate|up staged, 11 gate|up done, 12 barrier
 * passed, 13 down staged, 14 down done.  Synchronises the device.  QENG_ERR_STATE when the decoder
 * runs its steps operator by operator (no counterpart in the reference). */
int32_t qeng_decoder_step_profile(qeng_ctx* ctx, qeng_decoder* dec, uint64_t* out_ns, int32_t capacity,
                                  int32_t* n_written);

#ifdef __cplusplus
}
#endif
#endif /* QENG_H_ */
