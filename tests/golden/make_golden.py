"""Writes the small golden fixtures of tests/golden/ from the float64 oracle.

    python tests/golden/make_golden.py

The reference holds no golden vector, known-answer test or fixture for this
path (its runtime crates are absent from the checkout), so these vectors are
self-derived: they pin the oracle against accidental change and give the CUDA
path fixed inputs/outputs that do not depend on the oracle code being present.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref  # noqa: E402


def main():
    out = {}
    # GEMV / GEMM, ragged K (odd number of 32-blocks) and several M
    for name, (m, n, k, seed) in {"gemv_64x96": (1, 64, 96, 11), "gemm_5x48x160": (5, 48, 160, 12),
                                   "gemm_16x32x64": (16, 32, 64, 13)}.items():
        rng = ref.rng_of(seed)
        x = rng.standard_normal((m, k), dtype=np.float32)
        q, s = ref.make_q4(rng, n, k)
        out[name + "_x"], out[name + "_q"], out[name + "_s"] = x, q, s
        out[name + "_y"] = ref.gemm_q4(x, q, s)
    # one block enumerating all codes, scale 1
    q = np.arange(32, dtype=np.uint8).reshape(1, 32) % 16
    q = np.repeat(q, 16, 0)
    out["enum_q"], out["enum_s"] = q, np.ones((16, 1), np.float16)
    out["enum_x"] = np.linspace(-1, 1, 32, dtype=np.float32).reshape(1, 32)
    out["enum_y"] = ref.gemm_q4(out["enum_x"], q, out["enum_s"])
    # attention: page edges 1, 15, 16, 17 and a longer ragged one
    lens = np.array([1, 15, 16, 17, 70], np.int32)
    rng = ref.rng_of(14)
    qq = rng.standard_normal((5, 8, 128), dtype=np.float32).astype(np.float16)
    ks, vs, pool, table = ref.paged_kv(rng, lens, Hkv=2)
    out["attn_lens"], out["attn_q"], out["attn_pool"], out["attn_table"] = lens, qq, pool, table
    out["attn_out"] = ref.attn_decode(qq, ks, vs)
    # small ops
    rng = ref.rng_of(15)
    x = rng.standard_normal((3, 256), dtype=np.float32) * 5
    g = rng.uniform(0.5, 1.5, 256).astype(np.float32)
    out["rms_x"], out["rms_g"], out["rms_y"] = x, g, ref.rmsnorm(x, g, 1e-5)
    xr = rng.standard_normal((4, 3, 128), dtype=np.float32)
    pos = np.array([0, 1, 511, 4095], np.int32)
    out["rope_x"], out["rope_pos"], out["rope_y"] = xr, pos, ref.rope(xr, pos)
    a, b = rng.standard_normal((2, 500), dtype=np.float32) * 4
    out["swiglu_g"], out["swiglu_u"], out["swiglu_y"] = a, b, ref.swiglu(a, b)
    # a tiny decoder: 2 layers, d 256, ffn 512, 4/2 heads, vocab 320; prompt 9, 6 steps, batch 2
    cfg = ref.DecoderConfig(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)
    W = ref.make_decoder_weights(cfg, seed=5)
    dec = ref.Decoder(cfg, W)
    prompt = ref.rng_of(16).integers(0, cfg.vocab, (2, 9)).astype(np.int32)
    toks, logs = dec.generate(prompt, 6)
    out["dec_prompt"], out["dec_tokens"] = prompt, toks.astype(np.int32)
    out["dec_logits"] = np.stack(logs, 0)  # [steps, batch, vocab]
    # import-time quantiser: zero block, a tie in magnitude, a negative extreme, ragged scales
    rng = ref.rng_of(17)
    xq = (rng.standard_normal((32, 96)) * rng.uniform(1e-3, 3.0, (32, 1))).astype(np.float32)
    xq[0, :32] = 0.0
    xq[1, 5], xq[1, 9] = -7.5, 7.5
    xq[2, 32:64] = np.arange(-16, 16)
    out["quant_x"] = xq
    out["quant_q"], out["quant_s"] = ref.quantize_q4(xq)
    # the same tiny decoder with per-head q / k gains (QK-norm): greedy tokens and first logits
    rng = ref.rng_of(18)
    gains = rng.uniform(0.5, 1.5, (cfg.layers, 2, cfg.hd)).astype(np.float32)
    Wn = ref.make_decoder_weights(cfg, seed=5)
    for l, lw in enumerate(Wn["layers"]):
        lw["qnorm"], lw["knorm"] = gains[l, 0], gains[l, 1]
    toks_n, logs_n = ref.Decoder(cfg, Wn).generate(prompt, 6)
    out["qkn_gains"], out["qkn_tokens"], out["qkn_logits0"] = gains, toks_n.astype(np.int32), logs_n[0]
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **out)
    print("wrote", os.path.join(HERE, "golden.npz"), sum(v.nbytes for v in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
