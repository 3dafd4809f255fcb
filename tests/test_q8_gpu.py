"""8-bit block weights through the C ABI: layout round trip, device quantiser, the decode matmul and
the executor against the oracle ("tensor data (Q4/Q8/F16/F32)", decide/pipeline.md:28)."""
import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
TOL = 2e-3      # the gate
TIGHT = 2e-4    # what the 15-bit activation forms reach


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_pack_unpack_is_bit_exact(ctx):
    rng = ref.rng_of(80)
    for n, k in ((16, 32), (48, 96), (64, 4096)):  # 96: half a padding chunk
        q, s = ref.make_q8(rng, n, k)
        q[0, :4] = (-128, -127, 127, 0)
        w = ctx.pack_q8(q, s)
        assert w.q8 and (w.rows, w.cols) == (n, k)
        q2, s2 = w.unpack()
        assert np.array_equal(q2, q) and np.array_equal(s2.view(np.uint16), s.view(np.uint16))
        assert np.array_equal(w.dequant().cpu().numpy(), ref.dequant(q, s, np.float32))
        w.free()


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
def test_device_quantizer_matches_the_oracle(ctx, dtype):
    import torch
    rng = ref.rng_of(81)
    x = (rng.standard_normal((64, 224)) * rng.uniform(1e-3, 3.0, (64, 1))).astype(np.float32)
    x[0, :32] = 0.0
    x[1, 32:64] = np.arange(-16, 16) / 4.0
    xt = _t(x).to(getattr(torch, dtype))
    w = ctx.quantize_q8(xt)
    q, s = w.unpack()
    qo, so = ref.quantize_q8(xt.float().cpu().numpy())
    assert np.array_equal(q, qo) and np.array_equal(s.view(np.uint16), so.view(np.uint16))
    w.free()


@pytest.mark.parametrize("n,k", [(256, 512), (1024, 4096), (512, 11008), (48, 96)])
def test_decode_matmul_parity(ctx, n, k):
    from cyb_b200 import qeng
    rng = ref.rng_of(82 + n + k)
    q, s = ref.make_q8(rng, n, k)
    w = ctx.pack_q8(q, s)
    for m in (1, 2, 3, 8, 16, 20):
        x = rng.standard_normal((m, k), dtype=np.float32)
        want = ref.gemm_q4_fast(x, q, s)
        y = ctx.gemm_q4(w, _t(x)).cpu().numpy()
        e = ref.err_inf(y, want)
        assert e < TOL, (m, e)
        assert e < (2e-6 if m == 1 else TIGHT), (m, e)
        if m == 1:
            e15 = ref.err_inf(ctx.gemm_q4(w, _t(x), flags=qeng.GEMM_FAST_F16).cpu().numpy(), want)
            assert e15 < TIGHT, e15
    # exact cases: a one-hot activation picks a column of the dequantised matrix
    x = np.zeros((1, k), np.float32)
    x[0, 37 % k] = 1.0
    assert np.array_equal(ctx.gemm_q4(w, _t(x)).cpu().numpy()[0], ref.dequant(q, s, np.float32)[:, 37 % k])
    w.free()


CFG = dict(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)


def test_decoder_with_8bit_blocks_matches_the_teacher(ctx):
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=9, fmt="q8")
    dec = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                      vocab=cfg.vocab, max_batch=5, max_seq=96)
    qeng.load_decoder_weights(dec, W, cfg)
    for bn, t in ((1, 40), (5, 11)):
        prompt = ref.rng_of(90 + bn).integers(0, cfg.vocab, (bn, t)).astype(np.int32)
        want, logs = ref.Decoder(cfg, W).generate(prompt, 6)
        dec.reset(bn)
        dec.prefill(prompt)
        assert ref.err_inf(dec.logits(), logs[0]) < TOL
        assert np.array_equal(dec.decode(6), want)
    # a prompt long enough for the tensor-core path of 4-bit layers (>= 256 rows) stays on the decode kernels
    prompt = ref.rng_of(95).integers(0, cfg.vocab, (4, 70)).astype(np.int32)
    dec2 = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                       vocab=cfg.vocab, max_batch=4, max_seq=96)
    qeng.load_decoder_weights(dec2, W, cfg)
    want, logs = ref.Decoder(cfg, W).generate(prompt, 3)
    dec2.reset(4)
    dec2.prefill(prompt)
    assert ref.err_inf(dec2.logits(), logs[0]) < TOL
    assert np.array_equal(dec2.decode(3), want)
    ctx.device_status()
    # mixing the formats inside a fused matrix is refused
    q4 = ref.make_q4(ref.rng_of(1), cfg.heads * cfg.hd, cfg.d)
    with pytest.raises(qeng.QengError):
        dec2.load_matrix(0, 0, *q4)
        dec2.load_matrix(0, 1, *W["layers"][0]["wk"])
    dec.free()
    dec2.free()
