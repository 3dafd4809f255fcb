"""K-quant 4-bit super-blocks (Q4_K) through the C ABI: expansion round trip, the decode matmul and
the executor against the oracle ("needs fused Q4_K matmul", decide/model-lifecycle.md:175)."""
import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
TOL = 2e-3
TIGHT = 2e-4


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_expansion_is_bit_exact(ctx):
    rng = ref.rng_of(60)
    for n, k in ((16, 256), (48, 768), (64, 4096)):
        q, dm, blocks = ref.make_q4k(rng, n, k)
        w = ctx.pack_q4k(blocks, n, k)
        assert w.fmt == 14 and (w.rows, w.cols) == (n, k)
        q2, dm2 = w.unpack()
        assert np.array_equal(q2, q) and np.array_equal(dm2.view(np.uint32), dm.view(np.uint32))
        assert np.array_equal(w.dequant().cpu().numpy(), ref.dequant(q, dm, np.float32))
        w.free()


@pytest.mark.parametrize("n,k", [(256, 512), (1024, 4096), (512, 11008)])
def test_decode_matmul_parity(ctx, n, k):
    from cyb_b200 import qeng
    rng = ref.rng_of(61 + n + k)
    q, dm, blocks = ref.make_q4k(rng, n, k, wild=(n == 256))  # one shape with independent scales and minima
    w = ctx.pack_q4k(blocks, n, k)
    for m in (1, 2, 3, 4, 7):
        x = rng.standard_normal((m, k), dtype=np.float32)
        want = ref.gemm_q4_fast(x, q, dm)
        e = ref.err_inf(ctx.gemm_q4(w, _t(x)).cpu().numpy(), want)
        assert e < TOL, (m, e)
        assert e < (2e-6 if m == 1 else TIGHT), (m, e)
        if m == 1:
            e15 = ref.err_inf(ctx.gemm_q4(w, _t(x), flags=qeng.GEMM_FAST_F16).cpu().numpy(), want)
            assert e15 < TIGHT, e15
    # a constant activation block isolates the minimum term: y = sum_j (D_j sum(q) - 32 M_j)
    x = np.ones((1, k), np.float32)
    want = ref.gemm_q4_fast(x, q, dm)
    assert ref.err_inf(ctx.gemm_q4(w, _t(x)).cpu().numpy(), want) < 2e-6
    w.free()


CFG = dict(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)


def test_decoder_with_kquant_blocks_matches_the_teacher(ctx):
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=11, fmt="q4k")
    dec = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                      vocab=cfg.vocab, max_batch=5, max_seq=96)
    qeng.load_decoder_weights(dec, W, cfg)
    for bn, t in ((1, 23), (5, 9)):  # 5 sequences: passes of 4 rows
        prompt = ref.rng_of(70 + bn).integers(0, cfg.vocab, (bn, t)).astype(np.int32)
        want, logs = ref.Decoder(cfg, W).generate(prompt, 6)
        dec.reset(bn)
        dec.prefill(prompt)
        assert ref.err_inf(dec.logits(), logs[0]) < TOL
        assert np.array_equal(dec.decode(6), want)
    ctx.device_status()
    dec.free()
