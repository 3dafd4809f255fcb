"""The layer executor against the float64 teacher: teacher-forced layers, then
free-running greedy decode on the tiny golden decoder."""
import os

import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
CFG = dict(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)


def _make(ctx, max_batch=2, max_seq=64):
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=5)
    dec = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                      vocab=cfg.vocab, max_batch=max_batch, max_seq=max_seq)
    qeng.load_decoder_weights(dec, W, cfg)
    return cfg, W, dec


def test_teacher_forced_layers(ctx):
    import torch
    cfg, W, dec = _make(ctx)
    teacher = ref.Decoder(cfg, W)
    teacher.reset(1)
    rng = ref.rng_of(40)
    T = 19
    x = rng.standard_normal((1, T, cfg.d), dtype=np.float32) * 3
    pos = np.arange(T)
    for l in range(cfg.layers):
        want = teacher.layer(l, x.astype(np.float64), pos[None])
        got = dec.layer(l, torch.from_numpy(x[0]).cuda(), pos).cpu().numpy()
        assert ref.err_inf(got, want[0]) < 2e-3
        assert ref.err_inf(got, want[0]) < 5e-4
        # one decode step on top of the cached prompt
        x1 = rng.standard_normal((1, 1, cfg.d), dtype=np.float32)
        want1 = teacher.layer(l, x1.astype(np.float64), np.array([[T]]))
        got1 = dec.layer(l, torch.from_numpy(x1[0]).cuda(), np.array([T])).cpu().numpy()
        assert ref.err_inf(got1, want1[0]) < 5e-4
    dec.free()


def test_greedy_decode_matches_golden(ctx):
    g = GOLD
    cfg, W, dec = _make(ctx)
    prompt = g["dec_prompt"]
    steps = g["dec_tokens"].shape[1]
    dec.reset(prompt.shape[0])
    dec.prefill(prompt)
    assert ref.err_inf(dec.logits(), g["dec_logits"][0]) < 2e-3
    toks = dec.decode(steps)
    assert np.array_equal(toks, g["dec_tokens"])
    # a second call continues the same sequences (graph replay path)
    more = dec.decode(2)
    teacher = ref.Decoder(cfg, W)
    want, _ = teacher.generate(prompt, steps + 2)
    assert np.array_equal(np.concatenate([toks, more], 1), want)
    dec.free()


def test_state_errors(ctx):
    from cyb_b200 import qeng
    cfg, W, dec = _make(ctx, max_batch=1, max_seq=32)
    dec.reset(1)
    with pytest.raises(qeng.QengError) as e:
        dec.decode(1)  # no logits yet
    assert e.value.code == -8
    with pytest.raises(qeng.QengError) as e:
        dec.prefill(np.zeros((1, 33), np.int32))  # longer than the cache
    assert e.value.code == -2
    dec.free()


def test_teacher_forced_layer_on_the_tensor_core_path(ctx):
    """256 rows or more take the tcgen05 matmul (bf16 operands): gate 5e-3 per layer against the
    unrounded float64 teacher; the decode step on top of that cache is back on the exact path."""
    import torch
    cfg, W, dec = _make(ctx, max_batch=1, max_seq=320)
    teacher = ref.Decoder(cfg, W)
    teacher.reset(1)
    rng = ref.rng_of(41)
    T = 272
    x = rng.standard_normal((1, T, cfg.d), dtype=np.float32)
    pos = np.arange(T)
    want = teacher.layer(0, x.astype(np.float64), pos[None])
    got = dec.layer(0, torch.from_numpy(x[0]).cuda(), pos).cpu().numpy()
    ctx.device_status()
    e = ref.err_inf(got, want[0])
    assert e < 5e-3, e
    dec.free()


def test_full_size_layer_teacher_forced(ctx):
    """One layer at BASELINE's full widths (d 4096, FFN 11008, 32/8 heads): 6 prompt rows then one
    decode row, teacher-forced against the float64 oracle (gate 2e-3 on the layer output; measured
    ~1e-3: the 15-bit block fixed point of the activations entering o / gate|up / down, whose
    per-matmul error of ~6e-5 is amplified by the heavy-tailed SwiGLU output of these synthetic
    weights)."""
    import torch
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(layers=1, d=4096, ffn=11008, heads=32, kv_heads=8, vocab=256)
    W = ref.make_decoder_weights(cfg, seed=77)
    dec = ctx.decoder(layers=1, d_model=4096, ffn=11008, heads=32, kv_heads=8, vocab=256, max_batch=1, max_seq=32)
    qeng.load_decoder_weights(dec, W, cfg)
    teacher = ref.Decoder(cfg, W)
    teacher.reset(1)
    rng = ref.rng_of(78)
    T = 6
    x = rng.standard_normal((1, T, cfg.d), dtype=np.float32) * 2
    want = teacher.layer(0, x.astype(np.float64), np.arange(T)[None])
    got = dec.layer(0, torch.from_numpy(x[0]).cuda(), np.arange(T)).cpu().numpy()
    e = ref.err_inf(got, want[0])
    assert e < 2e-3, e
    x1 = rng.standard_normal((1, 1, cfg.d), dtype=np.float32) * 2
    want1 = teacher.layer(0, x1.astype(np.float64), np.array([[T]]))
    got1 = dec.layer(0, torch.from_numpy(x1[0]).cuda(), np.array([T])).cpu().numpy()
    e1 = ref.err_inf(got1, want1[0])
    assert e1 < 2e-3, e1
    ctx.device_status()
    dec.free()


def test_qk_norm_layers_and_greedy_decode(ctx):
    """Per-head RMS norm of q and k before the rotation (the Qwen3-family delta): teacher-forced
    layers and free-running greedy tokens against the float64 teacher with the same gains."""
    import torch
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=5)
    rng = ref.rng_of(91)
    for lw in W["layers"]:
        lw["qnorm"] = rng.uniform(0.5, 1.5, cfg.hd).astype(np.float32)
        lw["knorm"] = rng.uniform(0.5, 1.5, cfg.hd).astype(np.float32)
    dec = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                      vocab=cfg.vocab, max_batch=2, max_seq=64)
    qeng.load_decoder_weights(dec, W, cfg)
    teacher = ref.Decoder(cfg, W)
    teacher.reset(1)
    T = 9
    x = rng.standard_normal((1, T, cfg.d), dtype=np.float32) * 3
    for l in range(cfg.layers):
        want = teacher.layer(l, x.astype(np.float64), np.arange(T)[None])
        got = dec.layer(l, torch.from_numpy(x[0]).cuda(), np.arange(T)).cpu().numpy()
        assert ref.err_inf(got, want[0]) < 5e-4
    # the gains matter: without them the same input gives another result
    plain = ref.Decoder(cfg, {**W, "layers": [{k: v for k, v in lw.items() if k not in ("qnorm", "knorm")} for lw in W["layers"]]})
    plain.reset(1)
    assert ref.err_inf(plain.layer(0, x.astype(np.float64), np.arange(T)[None])[0], teacher_layer0(cfg, W, x, T)) > 1e-3
    prompt = GOLD["dec_prompt"]
    dec.reset(prompt.shape[0])
    dec.prefill(prompt)
    toks = dec.decode(6)
    want, logs = ref.Decoder(cfg, W).generate(prompt, 6)
    assert np.array_equal(toks, want)
    # only one of the two gains is a state error
    dec2 = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                       vocab=cfg.vocab, max_batch=1, max_seq=64)
    W2 = ref.make_decoder_weights(cfg, seed=5)
    qeng.load_decoder_weights(dec2, W2, cfg)
    dec2.load_norm(0, 2, np.ones(cfg.hd, np.float32))
    with pytest.raises(qeng.QengError) as e:
        dec2.layer(0, torch.zeros(1, cfg.d, device="cuda"), np.array([0]))
    assert e.value.code == -8
    dec.free()
    dec2.free()


def teacher_layer0(cfg, W, x, T):
    t = ref.Decoder(cfg, W)
    t.reset(1)
    return t.layer(0, x.astype(np.float64), np.arange(T)[None])[0]


def test_qk_norm_decode_matches_the_golden_fixture(ctx):
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=5)
    for l, lw in enumerate(W["layers"]):
        lw["qnorm"], lw["knorm"] = GOLD["qkn_gains"][l, 0], GOLD["qkn_gains"][l, 1]
    dec = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                      vocab=cfg.vocab, max_batch=2, max_seq=64)
    qeng.load_decoder_weights(dec, W, cfg)
    prompt = GOLD["dec_prompt"]
    dec.reset(prompt.shape[0])
    dec.prefill(prompt)
    assert ref.err_inf(dec.logits(), GOLD["qkn_logits0"]) < 2e-3
    assert np.array_equal(dec.decode(GOLD["qkn_tokens"].shape[1]), GOLD["qkn_tokens"])
    dec.free()


@pytest.mark.parametrize("batch", [5, 16])
def test_greedy_decode_at_larger_batches(ctx, batch):
    """Batches above 4 leave the fused LM head (separate norm, head, argmax, advance, embed) and run
    the matmuls in row chunks: logits after the prompt and greedy tokens against the float64 teacher."""
    cfg, W, dec = _make(ctx, max_batch=batch, max_seq=48)
    teacher = ref.Decoder(cfg, W)
    prompt = ref.rng_of(300 + batch).integers(0, cfg.vocab, (batch, 7)).astype(np.int32)
    steps = 6
    want, logs = teacher.generate(prompt, steps)
    dec.reset(batch)
    dec.prefill(prompt)
    assert ref.err_inf(dec.logits(), logs[0]) < 2e-3
    toks = dec.decode(steps)
    ctx.device_status()
    # a greedy token may only differ where the teacher's two best logits are closer than the error gate
    for b in range(batch):
        for s in range(steps):
            if toks[b, s] != want[b, s]:
                top = np.sort(logs[s][b])[-2:]
                assert top[1] - top[0] < 2e-3 * np.abs(logs[s][b]).max(), (b, s)
                break  # the sequences differ from here on
    assert (toks == want).mean() > 0.9
    dec.free()


def test_decode_after_the_buffers_grew(ctx):
    """prefill(short) -> decode -> reset -> prefill(longer) -> decode on ONE decoder: the second
    decode must not replay a step captured over buffers that were reallocated in between."""
    cfg, W, dec = _make(ctx, max_batch=1, max_seq=400)
    teacher = ref.Decoder(cfg, W)
    rng = ref.rng_of(55)
    for plen in (8, 200, 300, 12):   # 300 rows also crosses into the tensor-core prompt path
        prompt = rng.integers(0, cfg.vocab, (1, plen)).astype(np.int32)
        dec.reset(1)
        dec.prefill(prompt)
        got = dec.decode(4)
        ctx.device_status()
        if plen < 256:
            want, _ = teacher.generate(prompt, 4)
            assert np.array_equal(got, want), plen
        else:  # bf16 prompt path: compare with a fresh decoder instead of the exact teacher
            cfg2, W2, fresh = _make(ctx, max_batch=1, max_seq=400)
            fresh.reset(1)
            fresh.prefill(prompt)
            assert np.array_equal(got, fresh.decode(4)), plen
            fresh.free()
    dec.free()


def test_full_size_prompt_of_512_rows_then_a_decode_row(ctx):
    """One layer at the full widths over a 512-row prompt (the tensor-core path), teacher-forced
    against the float64 teacher that applies the same two roundings (activations and dequantised
    weights to bf16) — gate 5e-3; then one decode row on top of that cache, on the exact path,
    against the teacher with unrounded matmuls over the cache it built — gate 2e-3.  At these
    widths the attention logits have a spread of ~10, so a teacher that skipped the bf16 roundings
    would measure the softmax's sensitivity to them, not the kernels."""
    import torch
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(layers=1, d=4096, ffn=11008, heads=32, kv_heads=8, vocab=256)
    W = ref.make_decoder_weights(cfg, seed=79)
    dec = ctx.decoder(layers=1, d_model=4096, ffn=11008, heads=32, kv_heads=8, vocab=256, max_batch=1, max_seq=544)
    qeng.load_decoder_weights(dec, W, cfg)
    teacher = ref.Decoder(cfg, W, mm=lambda x, q, s: ref.gemm_q4_bf16w(ref.to_bf16(x), q, s))
    teacher.reset(1)
    rng = ref.rng_of(80)
    T = 512
    x = rng.standard_normal((1, T, cfg.d), dtype=np.float32)
    want = teacher.layer(0, x.astype(np.float64), np.arange(T)[None])
    got = dec.layer(0, torch.from_numpy(x[0]).cuda(), np.arange(T)).cpu().numpy()
    ctx.device_status()
    e = ref.err_inf(got, want[0])
    assert e < 5e-3, e
    teacher.mm = ref.gemm_q4_fast
    x1 = rng.standard_normal((1, 1, cfg.d), dtype=np.float32)
    want1 = teacher.layer(0, x1.astype(np.float64), np.array([[T]]))
    got1 = dec.layer(0, torch.from_numpy(x1[0]).cuda(), np.array([T])).cpu().numpy()
    e1 = ref.err_inf(got1, want1[0])
    assert e1 < 2e-3, e1
    ctx.device_status()
    dec.free()


@pytest.mark.parametrize("batch", [1, 2])
def test_fused_step_kernel_matches_the_teacher(built_lib, batch):
    """The opt-in fused decode step (all layers in one persistent cooperative kernel, operators
    linked by tagged stores and one grid barrier per layer): greedy tokens and logits against the
    float64 teacher, decode calls of several lengths, a reset in between, and the phase profile."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from cyb_b200 import qeng
    c = qeng.Context(0, step_kernel=1)
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=5)
    dec = c.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                    vocab=cfg.vocab, max_batch=2, max_seq=96)
    qeng.load_decoder_weights(dec, W, cfg)
    teacher = ref.Decoder(cfg, W)
    for plen in (5, 37):   # 37 tokens: three pages, the newest token mid-page
        prompt = ref.rng_of(900 + plen + batch).integers(0, cfg.vocab, (batch, plen)).astype(np.int32)
        want, logs = teacher.generate(prompt, 9)
        dec.reset(batch)
        dec.prefill(prompt)
        got = np.concatenate([dec.decode(1), dec.decode(5), dec.decode(3)], 1)
        assert dec.launches_per_step == 2  # the step kernel and the LM head
        c.device_status()
        assert np.array_equal(got, want), (plen, got, want)
        assert ref.err_inf(dec.logits(), teacher.forward(want[:, -1:], np.full((batch, 1), plen + 8))) < 2e-3
    prof = dec.step_profile()
    assert prof.shape == (2, cfg.layers, 16) and (np.diff(prof[0, :, :15].astype(np.int64), axis=1) >= 0).all()
    dec.free()
    c.close()


def test_softcap_and_sliding_window_decoder(ctx):
    """A decoder with soft-capped attention logits, a sliding window of 8 tokens and soft-capped final
    logits (the Gemma-family deltas): prompt logits and greedy tokens against the float64 teacher with
    the same switches."""
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG, attn_softcap=20.0, sliding_window=8, final_softcap=3.0)
    W = ref.make_decoder_weights(cfg, seed=5)
    dec = ctx.decoder(layers=cfg.layers, d_model=cfg.d, ffn=cfg.ffn, heads=cfg.heads, kv_heads=cfg.kv_heads,
                      vocab=cfg.vocab, max_batch=2, max_seq=64, attn_softcap=20.0, sliding_window=8, final_softcap=3.0)
    qeng.load_decoder_weights(dec, W, cfg)
    prompt = ref.rng_of(77).integers(0, cfg.vocab, (2, 21)).astype(np.int32)
    want, logs = ref.Decoder(cfg, W).generate(prompt, 8)
    dec.reset(2)
    dec.prefill(prompt)
    assert ref.err_inf(dec.logits(), logs[0]) < 2e-3
    assert np.abs(dec.logits()).max() <= 3.0
    assert np.array_equal(dec.decode(8), want)
    plain, _ = ref.Decoder(ref.DecoderConfig(**CFG), W).generate(prompt, 8)
    assert not np.array_equal(plain, want)  # the switches change the continuation on this input
    ctx.device_status()
    dec.free()
