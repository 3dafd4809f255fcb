"""The `.model` container reader: parsing rules on the CPU (no device needed), and on the GPU that
a decoder loaded from a file behaves exactly like one loaded from arrays."""
import os

import numpy as np
import pytest

from oracle import ref

import model_file_writer as mfw

CFG = dict(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)


def _sample(tmp_path, **kw):
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=5)
    path = os.path.join(tmp_path, "toy.model")
    n = mfw.write_model(path, cfg, W, **kw)
    return cfg, W, path, n


def test_container_config_is_parsed_without_a_device(built_lib, tmp_path):
    from cyb_b200 import qeng
    cfg, W, path, n = _sample(tmp_path)
    mc, nt = qeng.model_file_config(path)
    assert (mc.layers, mc.d_model, mc.ffn, mc.heads, mc.kv_heads, mc.head_dim, mc.vocab) == (2, 256, 512, 4, 2, 128, 320)
    assert abs(mc.rms_eps - 1e-5) < 1e-12 and mc.rope_base == 10000.0 and nt == n
    head = open(path, "rb").read(4096).decode("utf-8", "replace")
    assert head.startswith("[cyb]") and "~~~config\n" in head  # `head -50` tells what is inside (format.md)


def test_malformed_containers_are_rejected(built_lib, tmp_path):
    from cyb_b200 import qeng
    cfg, W, path, n = _sample(tmp_path)
    raw = open(path, "rb").read()

    def bad(data, name):
        p = os.path.join(tmp_path, name)
        open(p, "wb").write(data)
        with pytest.raises(qeng.QengError):
            qeng.model_file_config(p)
    bad(raw.replace(b"~~~", b"---"), "nodelim.model")                    # rule 1: no ~~~ at all
    bad(raw.replace(b"~~~tensors\n", b"~~~tensorz\n"), "order.model")     # rule 2: names follow the [[files]] order
    bad(raw[: len(raw) - 100], "short.model")                             # rule 3: `size` runs past the end
    bad(raw.replace(b"hidden_size", b"hidden_sz"), "cfg.model")           # config key missing
    bad(raw.replace(b'dtype = "Q4"', b'dtype = "Q5"', 1), "dtype.model")  # unknown tensor type
    bad(raw.replace(b"~~~config\n", b"~~~config\r\n"), "crlf.model")      # CRLF is not a delimiter
    with pytest.raises(qeng.QengError):
        qeng.model_file_config(os.path.join(tmp_path, "absent.model"))


@pytest.mark.gpu
@pytest.mark.parametrize("linear_dtype,tie", [("Q4", False), ("F32", False), ("F16", True), ("Q8", False), ("Q4_K", False), ("Q4_0", False)])
def test_decoder_loaded_from_a_file_equals_one_loaded_from_arrays(ctx, tmp_path, linear_dtype, tie):
    from cyb_b200 import qeng
    cfg = ref.DecoderConfig(**CFG)
    W = ref.make_decoder_weights(cfg, seed=5, fmt={"Q8": "q8", "Q4_K": "q4k"}.get(linear_dtype, "q4"))
    if tie:
        W["lm_head"] = W["emb"]
    path = os.path.join(tmp_path, "toy.model")
    mfw.write_model(path, cfg, W, linear_dtype=linear_dtype, tie_head=tie)
    if linear_dtype not in ("Q4", "Q8", "Q4_K", "Q4_0"):
        # float weights are quantised at load: what the decoder must then hold is the oracle's
        # quantisation of the stored (rounded) matrix, not the codes the file was made from
        W = dict(W, layers=[dict(lw) for lw in W["layers"]])
        for lw in W["layers"]:
            for key in mfw.HF:
                w = ref.dequant(*lw[key], np.float32)
                if linear_dtype == "F16":
                    w = w.astype(np.float16).astype(np.float32)
                lw[key] = ref.quantize_q4(w)
        for lw in W["layers"]:
            lw["norm2"] = np.asarray(lw["norm2"], np.float16).astype(np.float32)
    mc, _ = qeng.model_file_config(path, ctx)
    kw = dict(layers=mc.layers, d_model=mc.d_model, ffn=mc.ffn, heads=mc.heads, kv_heads=mc.kv_heads, vocab=mc.vocab,
              head_dim=mc.head_dim, rms_eps=mc.rms_eps, rope_base=mc.rope_base, max_batch=2, max_seq=64)
    a, b = ctx.decoder(**kw), ctx.decoder(**kw)
    a.load_file(path)
    qeng.load_decoder_weights(b, W, cfg)
    prompt = ref.rng_of(3).integers(0, cfg.vocab, (2, 9)).astype(np.int32)
    outs = []
    for dec in (a, b):
        dec.reset(2)
        dec.prefill(prompt)
        outs.append((dec.logits(), dec.decode(6)))
    assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
    want, _ = ref.Decoder(cfg, W).generate(prompt, 6)
    assert np.array_equal(outs[0][1], want)
    # the packed weights are bit-identical too
    for l in range(cfg.layers):
        for i in range(4):
            qa, sa = a.weight(l, i).unpack()
            qb, sb = b.weight(l, i).unpack()
            assert np.array_equal(qa, qb) and np.array_equal(sa.view(np.uint8), sb.view(np.uint8))
    # a decoder of another shape refuses the file
    c = ctx.decoder(**{**kw, "ffn": 1024})
    with pytest.raises(qeng.QengError) as e:
        c.load_file(path)
    assert e.value.code == -2
    for d in (a, b, c):
        d.free()


def test_block_byte_orders_match_the_gguf_package():
    """The "Q4_0" and "Q8" tensor encodings of the container are byte for byte what the third-party
    `gguf` package writes for its Q4_0 / Q8_0 types (so tensor data of that origin loads as it is)."""
    gguf = pytest.importorskip("gguf")
    from gguf import quants
    x = ref.rng_of(2).standard_normal((16, 96)).astype(np.float32)
    q, s = ref.quantize_q4(x)
    assert np.array_equal(np.frombuffer(mfw.q4_0_blocks(q, s), np.uint8),
                          quants.quantize(x, gguf.GGMLQuantizationType.Q4_0).reshape(-1))
    q8, s8 = ref.quantize_q8(x)
    assert np.array_equal(np.frombuffer(mfw.q8_blocks(q8, s8), np.uint8),
                          quants.quantize(x, gguf.GGMLQuantizationType.Q8_0).reshape(-1))
