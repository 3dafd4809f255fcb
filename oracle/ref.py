"""CPU oracle (NumPy, float64) for the block-quantized LLM hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the product path may import this file;
only the tests, the smoke check and the CPU-baseline legs of the benchmark do.

PARITY UNPINNED.  The arithmetic of this path lives in the crate ``run`` 0.1.0
(glia), reached through ``soma-kernel`` 0.1.0 — both are path dependencies
that are not part of the cyb checkout (Cargo.lock:8444-8462, 9091-9101;
shell/Cargo.toml:34) and no test or golden vector in cyb touches them.  This
file therefore restates the published arithmetic, constrained by the lines of
cyb that describe the runtime:

* block format "Q4_0 … 4-bit, 3.5x compression"   decide/pipeline.md:38,59
* op order of the decode loop                      decide/pipeline.md:51
* RMSNorm / GQA / SwiGLU / pre-norm                decide/compile.md:95-99
* KV cache held as f16                             decide/runtime.md:35
* head_dim = 128                                   decide/hardware.md:34

Choices that cyb does not pin are defined HERE and the CUDA path must match:

* dequant: ``w[n,k] = (q[n,k] - 8) * f32(s[n, k//32])``, q in 0..15.
* matmul:  ``y[m,n] = sum_b s[n,b] * sum_{k in b} x[m,k] * (q[n,k]-8)``.
* RoPE: half-split pairing (i, i+hd/2), angle = pos * base**(-2i/hd).
* q (after RoPE), K (after RoPE) and V are rounded to f16 (RNE) before the
  attention; softmax and the weighted sum are exact (f64 here).
* residual stream, norms, SwiGLU: full precision.
* greedy sampling: lowest index among equal maxima.
"""
from __future__ import annotations

import numpy as np

BLOCK = 32
ZERO_POINT = 8


# --------------------------------------------------------------------------
# seeded input generators (identical bits for CPU and GPU: always made on host)
# --------------------------------------------------------------------------
def rng_of(seed):
    return np.random.Generator(np.random.PCG64(seed))


def make_q4(rng, n, k):
    """4-bit codes uniform in 0..15 and one f16 scale ~U(0.002,0.02) per block."""
    q = rng.integers(0, 16, (n, k), dtype=np.uint8)
    s = rng.uniform(0.002, 0.02, (n, k // BLOCK)).astype(np.float16)
    return q, s


def to_bf16(x):
    """Round f32 -> bf16 (nearest even); returned as f32 holding bf16 values."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(x))


def bf16_bits(x):
    """f32 array holding bf16 values -> uint16 bit patterns."""
    return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)


def config1(seed=0, n=4096, k=4096):
    """Single GEMV: draw order x, q, s."""
    rng = rng_of(seed)
    x = rng.standard_normal((1, k), dtype=np.float32)
    q, s = make_q4(rng, n, k)
    return x, q, s


def config2(index, m, n, k):
    """Decode-batch GEMM: same draws, activations rounded to bf16; seed 1+index."""
    rng = rng_of(1 + index)
    x = to_bf16(rng.standard_normal((m, k), dtype=np.float32))
    q, s = make_q4(rng, n, k)
    return x, q, s


# --------------------------------------------------------------------------
# block format
# --------------------------------------------------------------------------
def centred(q):
    """The integer a weight stands for: code - 8 for 4-bit blocks (uint8 codes), the byte itself for
    8-bit blocks (int8)."""
    q = np.asarray(q)
    return q.astype(np.int32) if q.dtype == np.int8 else q.astype(np.int32) - ZERO_POINT


def dequant(q, s, dtype=np.float64):
    """w = (q-8)*s for 4-bit codes (uint8), w = q*s for 8-bit blocks (int8); exact in f32 and f64.
    K-quant weights come as codes (uint8) with s = f32 pairs [N, K/32, 2] (scale D, minimum M):
    w = D*q - M (a product and a difference, each rounded when dtype is float32)."""
    s = np.asarray(s)
    if s.ndim == 3:
        D = np.repeat(s[..., 0].astype(dtype), BLOCK, axis=1)
        M = np.repeat(s[..., 1].astype(dtype), BLOCK, axis=1)
        return (D * np.asarray(q).astype(dtype)).astype(dtype) - M
    return centred(q).astype(dtype) * np.repeat(s.astype(dtype), BLOCK, axis=1)


# ---- "K-quant" 4-bit super-blocks (the published Q4_K layout; "needs fused Q4_K matmul",
# decide/model-lifecycle.md:175) -------------------------------------------------------------
Q4K_BYTES = 144  # per 256 weights: f16 d, f16 dmin, 12 bytes of 6-bit scales / minima, 128 bytes of codes


def q4k_pack(d, dmin, sc, mn, codes):
    """Build super-blocks from their fields: d, dmin float16 [N, S]; sc, mn uint8 [N, S, 8] (0..63);
    codes uint8 [N, S*256] (0..15).  Returns uint8 [N, S, 144]."""
    n, S = d.shape
    out = np.zeros((n, S, Q4K_BYTES), np.uint8)
    out[..., 0:2] = np.ascontiguousarray(d, np.float16).reshape(n, S, 1).view(np.uint8)
    out[..., 2:4] = np.ascontiguousarray(dmin, np.float16).reshape(n, S, 1).view(np.uint8)
    sc, mn = sc.astype(np.uint8), mn.astype(np.uint8)
    p = out[..., 4:16]
    for j in range(4):
        p[..., j] = (sc[..., j] & 63) | ((sc[..., j + 4] >> 4) << 6)
        p[..., j + 4] = (mn[..., j] & 63) | ((mn[..., j + 4] >> 4) << 6)
        p[..., j + 8] = (sc[..., j + 4] & 15) | ((mn[..., j + 4] & 15) << 4)
    c = codes.reshape(n, S, 4, 2, 32)  # pairs of sub-blocks share 32 bytes: low nibbles 2i, high nibbles 2i+1
    out[..., 16:] = (c[:, :, :, 0, :] | (c[:, :, :, 1, :] << 4)).reshape(n, S, 128)
    return out


def q4k_unpack(blocks, n, k):
    """Super-blocks -> (codes uint8 [n, k], pairs float32 [n, k/32, 2] = (d*sc_j, dmin*m_j))."""
    b = np.ascontiguousarray(blocks, np.uint8).reshape(n, k // 256, Q4K_BYTES)
    d = b[..., 0:2].copy().view(np.float16)[..., 0].astype(np.float32)
    dmin = b[..., 2:4].copy().view(np.float16)[..., 0].astype(np.float32)
    p = b[..., 4:16]
    sc = np.empty(b.shape[:2] + (8,), np.uint8)
    mn = np.empty_like(sc)
    for j in range(4):
        sc[..., j] = p[..., j] & 63
        mn[..., j] = p[..., j + 4] & 63
        sc[..., j + 4] = (p[..., j + 8] & 15) | ((p[..., j] >> 6) << 4)
        mn[..., j + 4] = (p[..., j + 8] >> 4) | ((p[..., j + 4] >> 6) << 4)
    qs = b[..., 16:].reshape(n, k // 256, 4, 32)
    codes = np.stack([qs & 15, qs >> 4], axis=3).reshape(n, k)
    dm = np.stack([d[..., None] * sc.astype(np.float32), dmin[..., None] * mn.astype(np.float32)], axis=-1)
    return codes.astype(np.uint8), dm.reshape(n, k // 32, 2).astype(np.float32)


def make_q4k(rng, n, k, wild=False):
    """Synthetic Q4_K matrix: (codes, pairs, blocks).  Default: magnitudes like make_q4's and minima
    near 8 scales, i.e. roughly zero-mean weights as a quantiser of real tensors produces; wild = True
    draws scales and minima independently (weights with large per-block offsets)."""
    S = k // 256
    d = (rng.uniform(0.002, 0.02, (n, S)) / 32.0).astype(np.float16)
    sc = rng.integers(1, 64, (n, S, 8)).astype(np.uint8)
    if wild:
        dmin = (rng.uniform(0.002, 0.02, (n, S)) / 4.0).astype(np.float16)
        mn = rng.integers(0, 64, (n, S, 8)).astype(np.uint8)
    else:
        dmin = (d.astype(np.float32) * 8.0).astype(np.float16)
        mn = np.clip(np.rint(sc * rng.uniform(0.8, 1.2, sc.shape)), 0, 63).astype(np.uint8)
    codes = rng.integers(0, 16, (n, k), dtype=np.uint8)
    blocks = q4k_pack(d, dmin, sc, mn, codes)
    q, dm = q4k_unpack(blocks, n, k)
    assert np.array_equal(q, codes)
    return q, dm, blocks


def quantize_q8(w):
    """Import-time quantiser to 8-bit blocks ("tensor data (Q4/Q8/F16/F32)", decide/pipeline.md:28), the
    published Q8_0 rule, all in float32: per 32-block d = max|x| / 127, scale = f16(d),
    q = round-half-away-from-zero(x * (1/d)) (1/d = 0 when d = 0).  Integer outputs: the device
    quantiser must match bit for bit."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % BLOCK == 0
    b = w.reshape(n, k // BLOCK, BLOCK)
    d = (np.abs(b).max(axis=2) / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    v = (b * inv[..., None]).astype(np.float32)
    t = np.trunc(v)
    q = t + np.where(np.abs(v - t) >= np.float32(0.5), np.sign(v), np.float32(0.0))  # roundf
    return q.astype(np.int8).reshape(n, k), d.astype(np.float16)


def make_q8(rng, n, k):
    """Synthetic 8-bit block weights: bytes uniform in -127..127, scales like make_q4's / 16 (so that
    the dequantised magnitudes match the 4-bit matrices')."""
    q = rng.integers(-127, 128, (n, k), dtype=np.int8)
    s = (rng.uniform(0.002, 0.02, (n, k // BLOCK)) / 16.0).astype(np.float16)
    return q, s


def quantize_q4(w):
    """Import-time quantiser, F32/F16/BF16 matrix -> codes + f16 scales ("Q4 (4-bit, 3.5x
    compression)", decide/pipeline.md:38-40,59).  Per 32-block, the published Q4_0 rule: take
    the element of largest magnitude (the first one on ties), d = that element / -8, the
    scale is f16(d), and code = min(15, trunc(x * (1/d) + 8.5)), all in float32 (1/d = 0 when
    d = 0).  Integer outputs: the device quantiser must match bit for bit."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    assert k % BLOCK == 0
    b = w.reshape(n, k // BLOCK, BLOCK)
    idx = np.argmax(np.abs(b), axis=2)  # first occurrence of the maximum
    mx = np.take_along_axis(b, idx[..., None], axis=2)[..., 0]
    d = (mx / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d != 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    y = (b * inv[..., None]).astype(np.float32) + np.float32(8.5)
    q = np.minimum(15, y.astype(np.float32).astype(np.int32)).astype(np.uint8)
    return q.reshape(n, k), d.astype(np.float16)


def dequant_bf16(q, s):
    """Dequantize, then round each weight to bf16 (what the prefill path feeds
    its tensor-core contraction)."""
    return to_bf16(dequant(q, s, np.float32)).astype(np.float64)


def gemm_q4(x, q, s):
    """y[m,n] = sum_b s[n,b] * sum_{k in b} x[m,k]*(q[n,k]-8), float64."""
    if np.asarray(s).ndim == 3:  # K-quant pairs: scale and minimum per block
        return gemm_q4_fast(x, q, s)
    m, k = x.shape
    n = q.shape[0]
    nb = k // BLOCK
    xi = x.astype(np.float64).reshape(m, nb, BLOCK)
    qi = centred(q).astype(np.float64).reshape(n, nb, BLOCK)
    # block partial sums then scale; chunk n to bound memory
    y = np.empty((m, n), np.float64)
    step = max(1, (1 << 24) // (nb * BLOCK * max(m, 1)))
    s64 = s.astype(np.float64)
    for n0 in range(0, n, step):
        part = np.einsum("mbk,nbk->mnb", xi, qi[n0:n0 + step], optimize=True)
        y[:, n0:n0 + step] = (part * s64[None, n0:n0 + step]).sum(-1)
    return y


def gemm_q4_fast(x, q, s):
    """Same value as gemm_q4 up to f64 rounding, via one BLAS call."""
    return x.astype(np.float64) @ dequant(q, s).T


def gemm_q4_bf16w(x, q, s):
    """Prefill variant: weights rounded to bf16 before the contraction."""
    return x.astype(np.float64) @ dequant_bf16(q, s).T


# --------------------------------------------------------------------------
# small ops
# --------------------------------------------------------------------------
def rmsnorm(x, gamma, eps=1e-5):
    x = x.astype(np.float64)
    r = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return x * r * gamma.astype(np.float64)


def rope_tables(max_pos, hd=128, base=10000.0):
    """cos/sin[pos, i] for i < hd/2, float64."""
    i = np.arange(hd // 2, dtype=np.float64)
    theta = base ** (-2.0 * i / hd)
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * theta[None, :]
    return np.cos(ang), np.sin(ang)


def rope(x, pos, hd=128, base=10000.0):
    """x[..., heads, hd] rotated at integer positions pos[...] (half-split pairs)."""
    x = x.astype(np.float64)
    half = hd // 2
    i = np.arange(half, dtype=np.float64)
    theta = base ** (-2.0 * i / hd)
    ang = np.asarray(pos, dtype=np.float64)[..., None, None] * theta
    c, s_ = np.cos(ang), np.sin(ang)
    a, b = x[..., :half], x[..., half:]
    return np.concatenate([a * c - b * s_, b * c + a * s_], axis=-1)


def silu(x):
    return x / (1.0 + np.exp(-x))


def swiglu(gate, up):
    return silu(gate.astype(np.float64)) * up.astype(np.float64)


def f16_round(x):
    return np.asarray(x).astype(np.float16).astype(np.float64)


# --------------------------------------------------------------------------
# decode attention (GQA) over per-sequence K/V
# --------------------------------------------------------------------------
def attn_decode(q, ks, vs, scale=None, softcap=0.0, window=0):
    """q [B,Hq,hd]; ks/vs: list of [len_b,Hkv,hd].  Returns [B,Hq,hd] float64.
    softcap > 0: logits = softcap * tanh(q.k * scale / softcap); window > 0: only the last `window`
    cached tokens are attended (the two attention deltas of the Gemma family that the reference
    lists as missing from its runtime, decide/model-lifecycle.md:175-176)."""
    B, Hq, hd = q.shape
    scale = 1.0 / np.sqrt(hd) if scale is None else scale
    out = np.zeros((B, Hq, hd), np.float64)
    for b in range(B):
        k = ks[b].astype(np.float64)
        v = vs[b].astype(np.float64)
        if window > 0:
            k, v = k[-window:], v[-window:]
        if k.shape[0] == 0:
            continue
        Hkv = k.shape[1]
        grp = Hq // Hkv
        for h in range(Hq):
            kh = k[:, h // grp]
            logit = (kh @ q[b, h].astype(np.float64)) * scale
            if softcap > 0:
                logit = softcap * np.tanh(logit / softcap)
            logit -= logit.max()
            p = np.exp(logit)
            p /= p.sum()
            out[b, h] = p @ v[:, h // grp]
    return out


def paged_kv(rng, lens, Hkv=8, hd=128, page=16, shuffle=True):
    """Config-4 style KV: per sequence K,V f16 ~N(0,1), scattered into a page pool
    laid out [page][kv head][K|V][token in page][hd] in shuffled page order.
    Returns (ks, vs, pool f16, page_table int32 [B,max_pages])."""
    B = len(lens)
    npages = [(int(l) + page - 1) // page for l in lens]
    total = int(sum(npages))
    order = rng.permutation(total) if shuffle else np.arange(total)
    pool = np.zeros((total, Hkv, 2, page, hd), np.float16)
    table = np.full((B, max(npages)), -1, np.int32)
    ks, vs = [], []
    nxt = 0
    for b in range(B):
        L = int(lens[b])
        k = rng.standard_normal((L, Hkv, hd), dtype=np.float32).astype(np.float16)
        v = rng.standard_normal((L, Hkv, hd), dtype=np.float32).astype(np.float16)
        ks.append(k)
        vs.append(v)
        for p in range(npages[b]):
            pid = int(order[nxt]); nxt += 1
            table[b, p] = pid
            t0, t1 = p * page, min(L, (p + 1) * page)
            pool[pid, :, 0, : t1 - t0] = k[t0:t1].transpose(1, 0, 2)
            pool[pid, :, 1, : t1 - t0] = v[t0:t1].transpose(1, 0, 2)
    return ks, vs, pool, table


def config4(seed=4, B=16, Hq=32, Hkv=8, hd=128, lo=512, hi=4096, page=16):
    rng = rng_of(seed)
    lens = rng.integers(lo, hi + 1, B).astype(np.int32)
    q = rng.standard_normal((B, Hq, hd), dtype=np.float32).astype(np.float16)
    ks, vs, pool, table = paged_kv(rng, lens, Hkv, hd, page)
    return lens, q, ks, vs, pool, table


# --------------------------------------------------------------------------
# Llama-style decoder
# --------------------------------------------------------------------------
class DecoderConfig:
    def __init__(self, layers=32, d=4096, ffn=11008, heads=32, kv_heads=8, hd=128,
                 vocab=32000, eps=1e-5, rope_base=10000.0, attn_softcap=0.0, sliding_window=0, final_softcap=0.0):
        self.layers, self.d, self.ffn = layers, d, ffn
        self.heads, self.kv_heads, self.hd = heads, kv_heads, hd
        self.vocab, self.eps, self.rope_base = vocab, eps, rope_base
        self.attn_softcap, self.sliding_window, self.final_softcap = attn_softcap, sliding_window, final_softcap

    @property
    def qkv_rows(self):
        return (self.heads + 2 * self.kv_heads) * self.hd


def make_decoder_weights(cfg, seed=5, fmt="q4"):
    """All linear weights as 4-bit blocks (or 8-bit blocks with fmt="q8"; independent streams per
    matrix); embeddings and lm_head bf16 ~N(0,0.02); RMSNorm gains 1."""
    ss = np.random.SeedSequence(seed)
    kids = ss.spawn(2 + 7 * cfg.layers)
    g = lambda i: np.random.Generator(np.random.PCG64(kids[i]))
    W = {"emb": to_bf16(g(0).standard_normal((cfg.vocab, cfg.d), dtype=np.float32) * 0.02),
         "lm_head": to_bf16(g(1).standard_normal((cfg.vocab, cfg.d), dtype=np.float32) * 0.02),
         "final_norm": np.ones(cfg.d, np.float32), "layers": []}
    shapes = [("wq", cfg.heads * cfg.hd, cfg.d), ("wk", cfg.kv_heads * cfg.hd, cfg.d),
              ("wv", cfg.kv_heads * cfg.hd, cfg.d), ("wo", cfg.d, cfg.heads * cfg.hd),
              ("wgate", cfg.ffn, cfg.d), ("wup", cfg.ffn, cfg.d), ("wdown", cfg.d, cfg.ffn)]
    for l in range(cfg.layers):
        lw = {"norm1": np.ones(cfg.d, np.float32), "norm2": np.ones(cfg.d, np.float32)}
        for j, (name, n, k) in enumerate(shapes):
            if fmt == "q4k":
                q, dm, blocks = make_q4k(g(2 + 7 * l + j), n, k)
                lw[name] = (q, dm)
                lw[name + "_q4k"] = blocks
            else:
                lw[name] = (make_q8 if fmt == "q8" else make_q4)(g(2 + 7 * l + j), n, k)
        W["layers"].append(lw)
    return W


class Decoder:
    """Teacher of the executor: float64 forward with the f16 roundings of the
    spec.  KV is kept per sequence as python lists (no paging: paging is a
    storage detail of the device path)."""

    def __init__(self, cfg, W, mm=gemm_q4_fast):
        self.cfg, self.W, self.mm = cfg, W, mm
        self.k = None
        self.v = None

    def reset(self, batch):
        L = self.cfg.layers
        self.k = [[np.zeros((0, self.cfg.kv_heads, self.cfg.hd)) for _ in range(batch)] for _ in range(L)]
        self.v = [[np.zeros((0, self.cfg.kv_heads, self.cfg.hd)) for _ in range(batch)] for _ in range(L)]

    def layer(self, l, x, pos, trace=None):
        """x [B,T,d] at positions pos [B,T]; appends T tokens to each sequence."""
        cfg, lw = self.cfg, self.W["layers"][l]
        B, T, d = x.shape
        n1 = rmsnorm(x, lw["norm1"], cfg.eps).reshape(B * T, d)
        qp = self.mm(n1, *lw["wq"]).reshape(B, T, cfg.heads, cfg.hd)
        kp = self.mm(n1, *lw["wk"]).reshape(B, T, cfg.kv_heads, cfg.hd)
        vp = self.mm(n1, *lw["wv"]).reshape(B, T, cfg.kv_heads, cfg.hd)
        if "qnorm" in lw:  # per-head RMS norm of q and k before the rotation (Qwen3 family)
            qp = rmsnorm(qp, lw["qnorm"], cfg.eps)
            kp = rmsnorm(kp, lw["knorm"], cfg.eps)
        qr = f16_round(rope(qp, pos, cfg.hd, cfg.rope_base))
        kr = f16_round(rope(kp, pos, cfg.hd, cfg.rope_base))
        vr = f16_round(vp)
        att = np.zeros((B, T, cfg.heads, cfg.hd))
        for b in range(B):
            base = self.k[l][b].shape[0]
            self.k[l][b] = np.concatenate([self.k[l][b], kr[b]], 0)
            self.v[l][b] = np.concatenate([self.v[l][b], vr[b]], 0)
            for t in range(T):
                n = base + t + 1
                att[b, t] = attn_decode(qr[b, t][None], [self.k[l][b][:n]], [self.v[l][b][:n]],
                                        softcap=cfg.attn_softcap, window=cfg.sliding_window)[0]
        h = x + self.mm(att.reshape(B * T, -1), *lw["wo"]).reshape(B, T, d)
        n2 = rmsnorm(h, lw["norm2"], cfg.eps).reshape(B * T, d)
        act = swiglu(self.mm(n2, *lw["wgate"]), self.mm(n2, *lw["wup"]))
        out = h + self.mm(act, *lw["wdown"]).reshape(B, T, d)
        if trace is not None:
            trace.append(dict(q=qr, k=kr, v=vr, att=att, h=h, act=act, out=out))
        return out

    def forward(self, tokens, pos, trace=None):
        """tokens [B,T] -> logits of the LAST position [B,vocab] (float64)."""
        x = self.W["emb"][tokens].astype(np.float64)
        for l in range(self.cfg.layers):
            x = self.layer(l, x, pos, trace)
        xn = rmsnorm(x[:, -1], self.W["final_norm"], self.cfg.eps)
        logits = xn @ self.W["lm_head"].astype(np.float64).T
        if self.cfg.final_softcap > 0:
            logits = self.cfg.final_softcap * np.tanh(logits / self.cfg.final_softcap)
        return logits

    def generate(self, prompt, steps):
        """prompt [B,P] -> (tokens [B,steps], logits per step list)."""
        B, P = prompt.shape
        self.reset(B)
        pos = np.tile(np.arange(P), (B, 1))
        logits = self.forward(prompt, pos)
        outs, logs = [], []
        for s in range(steps):
            nxt = logits.argmax(-1)
            outs.append(nxt)
            logs.append(logits)
            if s + 1 == steps:
                break
            logits = self.forward(nxt[:, None], np.full((B, 1), P + s))
        return np.stack(outs, 1), logs


def err_inf(y, ref):
    """The gate metric: max|y-ref| / max|ref|."""
    ref = np.asarray(ref, np.float64)
    return float(np.abs(np.asarray(y, np.float64) - ref).max() / max(np.abs(ref).max(), 1e-300))
