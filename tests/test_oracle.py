"""CPU tests of the oracle itself: known answers derived from the block format,
agreement of the C restatement with the float64 NumPy one, and the committed
golden fixtures.  (The reference holds no vectors for this path: parity with
it is unpinned; these tests pin the oracle against itself.)"""
import os

import numpy as np
import pytest

from oracle import ref

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def test_all_codes_eight_gives_zero():
    x = ref.rng_of(1).standard_normal((2, 64), dtype=np.float32)
    q = np.full((16, 64), 8, np.uint8)
    s = np.full((16, 2), 0.01, np.float16)
    assert np.all(ref.gemm_q4(x, q, s) == 0.0)


def test_one_hot_selects_a_column():
    rng = ref.rng_of(2)
    q, s = ref.make_q4(rng, 32, 96)
    w = ref.dequant(q, s)
    for k in (0, 31, 32, 95):
        x = np.zeros((1, 96), np.float32)
        x[0, k] = 1.0
        assert np.array_equal(ref.gemm_q4(x, q, s)[0], w[:, k])


def test_dequant_is_exact_in_f32():
    q, s = ref.make_q4(ref.rng_of(3), 16, 64)
    assert np.array_equal(ref.dequant(q, s, np.float32).astype(np.float64), ref.dequant(q, s, np.float64))


def test_scale_extremes():
    q = np.tile(np.arange(16, dtype=np.uint8), (16, 2))
    for sv in (np.float16(6.1e-5), np.float16(65504.0)):
        s = np.full((16, 1), sv, np.float16)
        x = np.ones((1, 32), np.float32)
        y = ref.gemm_q4(x, q, s)
        assert np.allclose(y, float(sv) * (np.arange(16).sum() * 2 - 8 * 32))


def test_blockwise_and_blas_forms_agree():
    x, q, s = ref.config1(0, 128, 256)
    assert ref.err_inf(ref.gemm_q4_fast(x, q, s), ref.gemm_q4(x, q, s)) < 1e-13


def test_bf16_rounding_helper():
    x = np.array([1.0, 1.00390625, 1.01171875, -3.1415927, 65280.0, 1e-40], np.float32)
    r = ref.to_bf16(x)
    assert np.all((r.view(np.uint32) & 0xFFFF) == 0)
    assert r[1] == 1.0 and r[2] == np.float32(1.015625)  # ties to even, then up


def test_attention_known_answers():
    rng = ref.rng_of(4)
    q = rng.standard_normal((1, 4, 128), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((1, 1, 128), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((1, 1, 128), dtype=np.float32).astype(np.float16)
    out = ref.attn_decode(q, [k], [v])
    assert np.allclose(out[0], v[0, 0].astype(np.float64))  # len 1 -> V[0]
    k5 = np.repeat(k, 5, 0)
    v5 = rng.standard_normal((5, 1, 128), dtype=np.float32).astype(np.float16)
    out = ref.attn_decode(q, [k5], [v5])
    assert np.allclose(out[0, 0], v5[:, 0].astype(np.float64).mean(0))  # equal keys -> mean of V
    qs = np.repeat(q[:, :1], 4, 1)
    out = ref.attn_decode(qs, [k5], [v5])
    assert np.array_equal(out[0, 0], out[0, 3])  # same q in a group -> same output


def test_rope_and_norm_known_answers():
    x = ref.rng_of(5).standard_normal((2, 3, 128), dtype=np.float32)
    assert np.array_equal(ref.rope(x, np.zeros(2, np.int32)), x.astype(np.float64))  # pos 0 = identity
    r = ref.rope(x, np.array([7, 9]))
    assert np.allclose((r ** 2).sum(-1), (x.astype(np.float64) ** 2).sum(-1))  # rotation keeps the norm
    c = np.full((1, 64), 3.0, np.float32)
    assert np.allclose(ref.rmsnorm(c, np.ones(64, np.float32), 0.0), 1.0)


def test_c_port_matches_numpy_oracle(oracle_c):
    x, q, s = ref.config1(7, 64, 160)
    y = ref.gemm_q4(x, q, s)
    yc = oracle_c.gemm_q4(x, oracle_c.pack_q4(q, s), 64, 160)
    assert ref.err_inf(yc, y) < 1e-6
    lens, qq, ks, vs, pool, table = ref.config4(4, B=4, lo=1, hi=80)
    assert ref.err_inf(oracle_c.attn_decode(qq, pool, table, lens), ref.attn_decode(qq, ks, vs)) < 1e-5
    g = GOLD
    assert ref.err_inf(oracle_c.rmsnorm(g["rms_x"], g["rms_g"], 1e-5), g["rms_y"]) < 1e-6
    assert ref.err_inf(oracle_c.rope(g["rope_x"], g["rope_pos"], 10000.0), g["rope_y"]) < 1e-6
    assert ref.err_inf(oracle_c.swiglu(g["swiglu_g"], g["swiglu_u"]), g["swiglu_y"]) < 1e-6


def test_golden_fixtures_reproduce():
    g = GOLD
    for name in ("gemv_64x96", "gemm_5x48x160", "gemm_16x32x64", "enum"):
        y = ref.gemm_q4(g[name + "_x"], g[name + "_q"], g[name + "_s"])
        assert ref.err_inf(y, g[name + "_y"]) < 1e-14
    assert ref.err_inf(ref.rmsnorm(g["rms_x"], g["rms_g"], 1e-5), g["rms_y"]) < 1e-14
    assert ref.err_inf(ref.rope(g["rope_x"], g["rope_pos"]), g["rope_y"]) < 1e-14
    q, s = ref.quantize_q4(g["quant_x"])
    assert np.array_equal(q, g["quant_q"]) and np.array_equal(s.view(np.uint16), g["quant_s"].view(np.uint16))


def test_c_decoder_matches_numpy_decoder(oracle_c):
    """The CPU decode loop (timed baseline) against the float64 teacher on the tiny golden decoder."""
    g = GOLD
    cfg = ref.DecoderConfig(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)
    W = ref.make_decoder_weights(cfg, seed=5)
    prompt = g["dec_prompt"]
    B, P = prompt.shape
    max_pages = 2
    dec = oracle_c.CpuDecoder(cfg, W, pages_per_layer=B * max_pages)
    table = np.arange(B * max_pages, dtype=np.int32).reshape(B, max_pages)
    logits = None
    for t in range(P):
        logits, nxt = dec.step(prompt[:, t], np.full(B, t, np.int32), table)
    assert ref.err_inf(logits, g["dec_logits"][0]) < 2e-3
    toks = []
    for s in range(3):
        toks.append(nxt.copy())
        logits, nxt = dec.step(nxt, np.full(B, P + s, np.int32), table)
    assert np.array_equal(np.stack(toks, 1), g["dec_tokens"][:, :3])
    dec.close()


def _quantizer_cases():
    rng = ref.rng_of(31)
    x = (rng.standard_normal((48, 160)) * rng.uniform(1e-3, 3.0, (48, 1))).astype(np.float32)
    x[0, :32] = 0.0                     # an all-zero block: scale 0, every code 8
    x[1, 5], x[1, 9] = -7.5, 7.5        # a tie in magnitude: the first element decides the sign of d
    x[2, 32:64] = np.arange(-16, 16)    # the largest magnitude is negative: code 15 is reached
    return x


def test_quantizer_known_answers():
    x = _quantizer_cases()
    q, s = ref.quantize_q4(x)
    assert q.dtype == np.uint8 and q.max() <= 15 and s.dtype == np.float16
    assert np.all(q[0, :32] == 8) and s[0, 0] == 0
    assert s[1, 0] == np.float16(7.5 / 8) and q[1, 5] == 0 and q[1, 9] == 15  # d = -7.5 / -8 > 0
    assert s[2, 1] == np.float16(2.0) and q[2, 32] == 0 and q[2, 63] == 15
    # the reconstruction error stays within half a step of the block's scale (one step at the clamped end)
    err = np.abs(ref.dequant(q, s, np.float32) - x)
    step = np.repeat(np.abs(s.astype(np.float32)), 32, axis=1)
    assert np.all(err <= step * 1.001 + 1e-6)


def test_quantizer_matches_the_gguf_package_if_present():
    """Independent pin: the third-party `gguf` package implements the same published rule for the
    type it calls Q4_0 (18-byte blocks: f16 scale, then low nibbles = elements 0..15, high nibbles
    = elements 16..31).  Codes and scale bits must agree exactly; nibble ORDER is a layout matter."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    x = _quantizer_cases()
    q, s = ref.quantize_q4(x)
    n, k = x.shape
    b = quants.quantize(x, gguf.GGMLQuantizationType.Q4_0).reshape(n, k // 32, 18)
    d = b[..., :2].copy().view(np.float16)[..., 0]
    codes = np.concatenate([b[..., 2:] & 15, b[..., 2:] >> 4], axis=-1).reshape(n, k)
    assert np.array_equal(d.view(np.uint16), s.view(np.uint16))
    assert np.array_equal(codes, q)
    assert np.allclose(quants.dequantize(b.reshape(n, -1), gguf.GGMLQuantizationType.Q4_0), ref.dequant(q, s, np.float32))


def test_q8_quantizer_known_answers_and_gguf_pin():
    """8-bit blocks: d = max|x| / 127, q = round-half-away(x / d); w = q * s.  Where the third-party
    `gguf` package is present its Q8_0 (34-byte blocks: f16 scale, 32 signed bytes) must give the same
    bytes and scale bits."""
    x = _quantizer_cases()
    q, s = ref.quantize_q8(x)
    assert q.dtype == np.int8 and q.min() >= -127 and q.max() <= 127
    b = x.reshape(x.shape[0], -1, 32)
    amax = np.abs(b).max(2)
    assert np.array_equal(np.abs(q.reshape(b.shape)).max(2)[amax > 0], np.full((amax > 0).sum(), 127))
    assert np.all(q.reshape(b.shape)[amax == 0] == 0) and np.all(s[amax == 0] == 0)
    w = ref.dequant(q, s, np.float32)
    assert np.all(np.abs(w - x).reshape(b.shape) <= (amax / 127 * 0.51 + np.abs(amax) * 2e-3)[..., None])
    assert np.array_equal(ref.gemm_q4(x[:2], q, s), ref.gemm_q4(x[:2], q, s))
    assert np.allclose(ref.gemm_q4(x[:3], q, s), ref.gemm_q4_fast(x[:3], q, s), rtol=1e-12, atol=1e-9)
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    g = quants.quantize(x, gguf.GGMLQuantizationType.Q8_0).reshape(x.shape[0], -1, 34)
    assert np.array_equal(g[..., :2].copy().view(np.uint16)[..., 0], s.view(np.uint16))
    assert np.array_equal(g[..., 2:].copy().view(np.int8).reshape(q.shape), q)


def test_q4k_fields_round_trip_and_gguf_pin():
    """K-quant super-blocks: the 6-bit scale / minimum packing and the nibble order round-trip, and
    where the third-party `gguf` package is present its Q4_K dequantizer gives the same f32 weights
    from the same bytes (random field values included)."""
    rng = ref.rng_of(41)
    n, k = 48, 768
    S = k // 256
    d = rng.uniform(1e-4, 1e-2, (n, S)).astype(np.float16)
    dmin = rng.uniform(1e-4, 1e-2, (n, S)).astype(np.float16)
    sc = rng.integers(0, 64, (n, S, 8)).astype(np.uint8)
    mn = rng.integers(0, 64, (n, S, 8)).astype(np.uint8)
    codes = rng.integers(0, 16, (n, k), dtype=np.uint8)
    blocks = ref.q4k_pack(d, dmin, sc, mn, codes)
    q, dm = ref.q4k_unpack(blocks, n, k)
    assert np.array_equal(q, codes)
    assert np.array_equal(dm[..., 0].reshape(n, S, 8), d.astype(np.float32)[..., None] * sc)
    assert np.array_equal(dm[..., 1].reshape(n, S, 8), dmin.astype(np.float32)[..., None] * mn)
    w = ref.dequant(q, dm, np.float32)
    assert np.array_equal(w[0, :32], (dm[0, 0, 0] * codes[0, :32].astype(np.float32)).astype(np.float32) - dm[0, 0, 1])
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    raw = rng.integers(0, 256, blocks.shape, dtype=np.uint8)
    raw[..., 0:4] = blocks[..., 0:4]  # keep finite f16 d / dmin
    for b in (blocks, raw):
        qq, dd = ref.q4k_unpack(b, n, k)
        assert np.array_equal(quants.dequantize(b.reshape(n, -1), gguf.GGMLQuantizationType.Q4_K), ref.dequant(qq, dd, np.float32))

