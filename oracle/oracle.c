/* CPU oracle in C (OpenMP) for the block-quantized LLM hot path.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA path and the timed CPU
 * baseline.  The shipped library never links or calls this file.
 *
 * PARITY UNPINNED: the arithmetic restated here lives in the crate `run` 0.1.0
 * (glia), a path dependency absent from the cyb checkout (Cargo.lock:8444-8462),
 * and cyb holds no test or golden vector for it.  What cyb does pin:
 *   block format "Q4_0, 4-bit"                      decide/pipeline.md:38,59
 *   decode loop order                               decide/pipeline.md:51
 *   RMSNorm, GQA, SwiGLU, pre-norm                  decide/compile.md:95-99
 *   f16 KV cache                                    decide/runtime.md:35
 * The choices cyb leaves open are the ones oracle/ref.py documents; this file
 * follows them and is itself checked against ref.py by the CPU tests.
 *
 * CPU block layout (what a CPU runtime would stream): 18-byte blocks
 * {f16 scale; 16 bytes of nibbles}, byte j = code[2j] | code[2j+1] << 4.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

typedef struct __attribute__((packed)) { f16 s; uint8_t qs[16]; } orc_block;

int orc_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* q[N,K] codes 0..15 + s[N,K/32] f16 -> blocks[N*K/32] */
void orc_pack_q4(const uint8_t* q, const uint16_t* s, int64_t N, int64_t K, void* out) {
  orc_block* b = (orc_block*)out;
  int64_t nb = K / 32;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++)
    for (int64_t j = 0; j < nb; j++) {
      orc_block* o = &b[n * nb + j];
      memcpy(&o->s, &s[n * nb + j], 2);
      const uint8_t* src = q + n * K + j * 32;
      for (int i = 0; i < 16; i++) o->qs[i] = (uint8_t)(src[2 * i] | (src[2 * i + 1] << 4));
    }
}

#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
/* 32 codes of one block against 32 activations, 8 lanes at a time */
static inline float block_dot(const orc_block* b, const float* x) {
  const __m128i raw = _mm_loadu_si128((const __m128i*)b->qs);
  const __m128i m4 = _mm_set1_epi8(15);
  const __m128i lo = _mm_and_si128(raw, m4);                      /* codes 0,2,4,.. */
  const __m128i hi = _mm_and_si128(_mm_srli_epi16(raw, 4), m4);   /* codes 1,3,5,.. */
  const __m128i c0 = _mm_unpacklo_epi8(lo, hi);                   /* codes 0..15 */
  const __m128i c1 = _mm_unpackhi_epi8(lo, hi);                   /* codes 16..31 */
  const __m256i eight = _mm256_set1_epi32(8);
  __m256 acc = _mm256_setzero_ps();
  acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(c0), eight)), _mm256_loadu_ps(x), acc);
  acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(c0, 8)), eight)),
                        _mm256_loadu_ps(x + 8), acc);
  acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(c1), eight)), _mm256_loadu_ps(x + 16), acc);
  acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_sub_epi32(_mm256_cvtepu8_epi32(_mm_srli_si128(c1, 8)), eight)),
                        _mm256_loadu_ps(x + 24), acc);
  __m128 r = _mm_add_ps(_mm256_castps256_ps128(acc), _mm256_extractf128_ps(acc, 1));
  r = _mm_add_ps(r, _mm_movehl_ps(r, r));
  r = _mm_add_ss(r, _mm_shuffle_ps(r, r, 1));
  return _mm_cvtss_f32(r) * (float)b->s;
}
#else
static inline float block_dot(const orc_block* b, const float* x) {
  float w[32];
  for (int i = 0; i < 16; i++) {
    w[2 * i] = (float)((int)(b->qs[i] & 15) - 8);
    w[2 * i + 1] = (float)((int)(b->qs[i] >> 4) - 8);
  }
  float acc = 0.f;
#pragma omp simd reduction(+ : acc)
  for (int i = 0; i < 32; i++) acc += x[i] * w[i];
  return acc * (float)b->s;
}
#endif

/* y[M,N] = x[M,K] . dequant(W)^T ; f32 block sums, f64 across blocks */
void orc_gemm_q4(const float* x, const void* blocks, int64_t M, int64_t N, int64_t K, float* y) {
  const orc_block* W = (const orc_block*)blocks;
  int64_t nb = K / 32;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const orc_block* row = W + n * nb;
    for (int64_t m = 0; m < M; m++) {
      const float* xr = x + m * K;
      double acc = 0.0;
      for (int64_t j = 0; j < nb; j++) acc += (double)block_dot(row + j, xr + 32 * j);
      y[m * N + n] = (float)acc;
    }
  }
}

/* y[M,N] = x[M,K] . W^T for bf16 W (bit patterns) */
void orc_gemm_bf16(const float* x, const uint16_t* W, int64_t M, int64_t N, int64_t K, float* y) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; n++) {
    const uint16_t* row = W + n * K;
    for (int64_t m = 0; m < M; m++) {
      const float* xr = x + m * K;
      double acc = 0.0;
      for (int64_t k0 = 0; k0 < K; k0 += 64) {
        float part = 0.f;
        int64_t k1 = k0 + 64 < K ? k0 + 64 : K;
        for (int64_t k = k0; k < k1; k++) {
          uint32_t u = (uint32_t)row[k] << 16;
          float w;
          memcpy(&w, &u, 4);
          part += xr[k] * w;
        }
        acc += part;
      }
      y[m * N + n] = (float)acc;
    }
  }
}

void orc_rmsnorm(const float* x, const float* gamma, int64_t M, int64_t D, float eps, float* y) {
#pragma omp parallel for schedule(static) if (M > 1)
  for (int64_t m = 0; m < M; m++) {
    double ss = 0.0;
    for (int64_t i = 0; i < D; i++) ss += (double)x[m * D + i] * x[m * D + i];
    double r = 1.0 / sqrt(ss / (double)D + (double)eps);
    for (int64_t i = 0; i < D; i++) y[m * D + i] = (float)(x[m * D + i] * r * gamma[i]);
  }
}

/* in place, x[M,H,hd], half-split pairs (i, i+hd/2), angle = pos*base^(-2i/hd) */
void orc_rope(float* x, const int32_t* pos, int64_t M, int64_t H, int64_t hd, float base) {
  int64_t half = hd / 2;
  for (int64_t m = 0; m < M; m++)
    for (int64_t i = 0; i < half; i++) {
      double ang = (double)pos[m] * pow((double)base, -2.0 * (double)i / (double)hd);
      double c = cos(ang), s = sin(ang);
      for (int64_t h = 0; h < H; h++) {
        float* p = x + (m * H + h) * hd;
        double a = p[i], b = p[i + half];
        p[i] = (float)(a * c - b * s);
        p[i + half] = (float)(b * c + a * s);
      }
    }
}

void orc_swiglu(const float* gate, const float* up, int64_t n, float* y) {
#pragma omp parallel for schedule(static) if (n > 65536)
  for (int64_t i = 0; i < n; i++) {
    double g = gate[i];
    y[i] = (float)(g / (1.0 + exp(-g)) * (double)up[i]);
  }
}

/* Decode attention over a paged f16 pool laid out [page][kv head][K|V][tok][hd].
 * q f16 [B,Hq,hd], lens[B], table[B,max_pages]; out f32 [B,Hq,hd]. */
void orc_attn_decode(const uint16_t* q_, const uint16_t* pool_, const int32_t* table,
                     const int32_t* lens, int64_t B, int64_t Hq, int64_t Hkv, int64_t hd,
                     int64_t page, int64_t max_pages, float scale, float* out) {
  const f16* q = (const f16*)q_;
  const f16* pool = (const f16*)pool_;
  int64_t grp = Hq / Hkv;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
  for (int64_t b = 0; b < B; b++)
    for (int64_t h = 0; h < Hq; h++) {
      int64_t L = lens[b], kvh = h / grp;
      const f16* qv = q + (b * Hq + h) * hd;
      double* lg = (double*)malloc(sizeof(double) * (size_t)(L > 0 ? L : 1));
      double mx = -INFINITY;
      for (int64_t t = 0; t < L; t++) {
        int64_t pid = table[b * max_pages + t / page];
        const f16* kr = pool + (((pid * Hkv + kvh) * 2 + 0) * page + t % page) * hd;
        float acc = 0.f;
        for (int64_t i = 0; i < hd; i++) acc += (float)qv[i] * (float)kr[i];
        lg[t] = (double)acc * scale;
        if (lg[t] > mx) mx = lg[t];
      }
      double den = 0.0;
      double o[512];
      for (int64_t i = 0; i < hd; i++) o[i] = 0.0;
      for (int64_t t = 0; t < L; t++) {
        double p = exp(lg[t] - mx);
        den += p;
        int64_t pid = table[b * max_pages + t / page];
        const f16* vr = pool + (((pid * Hkv + kvh) * 2 + 1) * page + t % page) * hd;
        for (int64_t i = 0; i < hd; i++) o[i] += p * (double)(float)vr[i];
      }
      for (int64_t i = 0; i < hd; i++) out[(b * Hq + h) * hd + i] = L > 0 ? (float)(o[i] / den) : 0.f;
      free(lg);
    }
}

/* ---------------- CPU decoder (one decode step), used as the timed baseline -- */
typedef struct {
  int32_t layers, d, ffn, heads, kv_heads, hd, vocab;
  float eps, rope_base;
} orc_cfg;

typedef struct {
  orc_cfg c;
  void** w;           /* per layer 7 block matrices: q,k,v,o,gate,up,down */
  float** norms;      /* per layer 2 gains */
  const uint16_t* emb;     /* bf16 [vocab,d] */
  const uint16_t* lm_head; /* bf16 [vocab,d] */
  const float* final_norm;
  f16* pool;          /* [layers][page][kvh][2][16][hd] */
  int64_t pages_per_layer;
} orc_decoder;

void* orc_decoder_new(const orc_cfg* c, int64_t pages_per_layer) {
  orc_decoder* D = (orc_decoder*)calloc(1, sizeof(orc_decoder));
  D->c = *c;
  D->w = (void**)calloc((size_t)c->layers * 7, sizeof(void*));
  D->norms = (float**)calloc((size_t)c->layers * 2, sizeof(float*));
  D->pages_per_layer = pages_per_layer;
  size_t n = (size_t)c->layers * (size_t)pages_per_layer * c->kv_heads * 2 * 16 * c->hd;
  D->pool = (f16*)calloc(n, sizeof(f16));
  return D;
}
void orc_decoder_set_matrix(void* d, int layer, int which, void* blocks) { ((orc_decoder*)d)->w[layer * 7 + which] = blocks; }
void orc_decoder_set_norm(void* d, int layer, int which, float* g) { ((orc_decoder*)d)->norms[layer * 2 + which] = g; }
void orc_decoder_set_head(void* d, const uint16_t* emb, const uint16_t* lm, const float* fn) {
  orc_decoder* D = (orc_decoder*)d;
  D->emb = emb; D->lm_head = lm; D->final_norm = fn;
}
uint16_t* orc_decoder_pool(void* d) { return (uint16_t*)((orc_decoder*)d)->pool; }
void orc_decoder_free(void* d) {
  orc_decoder* D = (orc_decoder*)d;
  free(D->w); free(D->norms); free(D->pool); free(D);
}

/* One decode step for B sequences: tokens[B] at positions pos[B] (= current
 * length of each sequence); page tables as in orc_attn_decode.  Writes logits
 * [B,vocab] and next[B] (greedy, lowest index on ties). */
void orc_decoder_step(void* d, const int32_t* tokens, const int32_t* pos, const int32_t* table,
                      int64_t max_pages, int64_t B, float* logits, int32_t* next) {
  orc_decoder* D = (orc_decoder*)d;
  const orc_cfg* c = &D->c;
  int64_t dm = c->d, F = c->ffn, Hq = c->heads, Hkv = c->kv_heads, hd = c->hd;
  int64_t nq = Hq * hd, nkv = Hkv * hd;
  float* x = (float*)malloc(sizeof(float) * B * dm);
  float* xn = (float*)malloc(sizeof(float) * B * dm);
  float* qb = (float*)malloc(sizeof(float) * B * nq);
  float* kb = (float*)malloc(sizeof(float) * B * nkv);
  float* vb = (float*)malloc(sizeof(float) * B * nkv);
  uint16_t* q16 = (uint16_t*)malloc(2 * B * nq);
  float* att = (float*)malloc(sizeof(float) * B * nq);
  float* t0 = (float*)malloc(sizeof(float) * B * dm);
  float* g = (float*)malloc(sizeof(float) * B * F);
  float* u = (float*)malloc(sizeof(float) * B * F);
  int32_t* lens = (int32_t*)malloc(4 * B);
  for (int64_t b = 0; b < B; b++) {
    for (int64_t i = 0; i < dm; i++) {
      uint32_t w = (uint32_t)D->emb[(int64_t)tokens[b] * dm + i] << 16;
      memcpy(&x[b * dm + i], &w, 4);
    }
    lens[b] = pos[b] + 1;
  }
  for (int l = 0; l < c->layers; l++) {
    f16* pool = D->pool + (size_t)l * D->pages_per_layer * Hkv * 2 * 16 * hd;
    orc_rmsnorm(x, D->norms[l * 2], B, dm, c->eps, xn);
    orc_gemm_q4(xn, D->w[l * 7 + 0], B, nq, dm, qb);
    orc_gemm_q4(xn, D->w[l * 7 + 1], B, nkv, dm, kb);
    orc_gemm_q4(xn, D->w[l * 7 + 2], B, nkv, dm, vb);
    orc_rope(qb, pos, B, Hq, hd, c->rope_base);
    orc_rope(kb, pos, B, Hkv, hd, c->rope_base);
    for (int64_t b = 0; b < B; b++) {
      int64_t pid = table[b * max_pages + pos[b] / 16], slot = pos[b] % 16;
      for (int64_t h = 0; h < Hkv; h++)
        for (int64_t i = 0; i < hd; i++) {
          pool[(((pid * Hkv + h) * 2 + 0) * 16 + slot) * hd + i] = (f16)kb[(b * Hkv + h) * hd + i];
          pool[(((pid * Hkv + h) * 2 + 1) * 16 + slot) * hd + i] = (f16)vb[(b * Hkv + h) * hd + i];
        }
      for (int64_t i = 0; i < nq; i++) {
        f16 v = (f16)qb[b * nq + i];
        memcpy(&q16[b * nq + i], &v, 2);
      }
    }
    orc_attn_decode(q16, (const uint16_t*)pool, table, lens, B, Hq, Hkv, hd, 16, max_pages,
                    1.0f / sqrtf((float)hd), att);
    orc_gemm_q4(att, D->w[l * 7 + 3], B, dm, nq, t0);
    for (int64_t i = 0; i < B * dm; i++) x[i] += t0[i];
    orc_rmsnorm(x, D->norms[l * 2 + 1], B, dm, c->eps, xn);
    orc_gemm_q4(xn, D->w[l * 7 + 4], B, F, dm, g);
    orc_gemm_q4(xn, D->w[l * 7 + 5], B, F, dm, u);
    orc_swiglu(g, u, B * F, g);
    orc_gemm_q4(g, D->w[l * 7 + 6], B, dm, F, t0);
    for (int64_t i = 0; i < B * dm; i++) x[i] += t0[i];
  }
  orc_rmsnorm(x, D->final_norm, B, dm, c->eps, xn);
  orc_gemm_bf16(xn, D->lm_head, B, c->vocab, dm, logits);
  for (int64_t b = 0; b < B; b++) {
    int32_t best = 0;
    for (int32_t i = 1; i < c->vocab; i++)
      if (logits[b * c->vocab + i] > logits[b * c->vocab + best]) best = i;
    next[b] = best;
  }
  free(x); free(xn); free(qb); free(kb); free(vb); free(q16); free(att); free(t0); free(g); free(u); free(lens);
}
