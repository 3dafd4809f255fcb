"""Writes a `.model` container (a `.cyb` file: TOML frontmatter, `~~~name` sections, sized binary)
from a weight dict of the oracle's layout, with the tensor-index schema the engine reads
(sections `config`, `tensors`, `weights`; one [[tensor]] table per tensor with name, dtype, shape,
offset, size).  Test infrastructure: the sample files of the loader tests come from here."""
from __future__ import annotations

import numpy as np

HF = {"wq": "self_attn.q_proj", "wk": "self_attn.k_proj", "wv": "self_attn.v_proj", "wo": "self_attn.o_proj",
      "wgate": "mlp.gate_proj", "wup": "mlp.up_proj", "wdown": "mlp.down_proj"}


def q4_blocks(q, s):
    """codes [N,K] + f16 scales [N,K/32] -> row-major 18-byte blocks (scale, then k = 2i | k = 2i+1 << 4)."""
    n, k = q.shape
    out = np.empty((n * k // 32, 18), np.uint8)
    out[:, :2] = np.ascontiguousarray(s, np.float16).reshape(-1, 1).view(np.uint8)
    b = q.reshape(-1, 16, 2)
    out[:, 2:] = (b[:, :, 0] | (b[:, :, 1] << 4)).astype(np.uint8)
    return out.tobytes()


def q4_0_blocks(q, s):
    """The same 18-byte block in the nibble order of the published Q4_0: byte i = k = i | (k = i + 16) << 4."""
    n, k = q.shape
    out = np.empty((n * k // 32, 18), np.uint8)
    out[:, :2] = np.ascontiguousarray(s, np.float16).reshape(-1, 1).view(np.uint8)
    b = q.reshape(-1, 32)
    out[:, 2:] = (b[:, :16] | (b[:, 16:] << 4)).astype(np.uint8)
    return out.tobytes()


def q8_blocks(q, s):
    """bytes [N,K] int8 + f16 scales [N,K/32] -> row-major 34-byte blocks (scale, then the 32 bytes)."""
    n, k = q.shape
    out = np.empty((n * k // 32, 34), np.uint8)
    out[:, :2] = np.ascontiguousarray(s, np.float16).reshape(-1, 1).view(np.uint8)
    out[:, 2:] = np.ascontiguousarray(q, np.int8).reshape(-1, 32).view(np.uint8)
    return out.tobytes()


def bf16_bits(x):
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def write_model(path, cfg, W, linear_dtype="Q4", tie_head=False, name="sample"):
    """linear_dtype: "Q4" stores the codes as they are; "F16" / "F32" / "BF16" stores the dequantised
    matrix (the loader quantises it again on the device: exact for F32, and for F16/BF16 whenever
    (q-8)*s is representable)."""
    from oracle import ref
    tensors, blobs, off = [], [], 0

    def add(tname, dtype, shape, data):
        nonlocal off
        tensors.append((tname, dtype, shape, off, len(data)))
        blobs.append(data)
        off += len(data)

    def linear(tname, q, s):
        if np.asarray(q).dtype == np.int8:  # 8-bit blocks are stored as they are
            add(tname, "Q8", list(q.shape), q8_blocks(q, s))
        elif linear_dtype == "Q4":
            add(tname, "Q4", list(q.shape), q4_blocks(q, s))
        elif linear_dtype == "Q4_0":
            add(tname, "Q4_0", list(q.shape), q4_0_blocks(q, s))
        else:
            w = ref.dequant(q, s, np.float32)
            if linear_dtype == "F32":
                add(tname, "F32", list(q.shape), w.tobytes())
            elif linear_dtype == "F16":
                add(tname, "F16", list(q.shape), w.astype(np.float16).tobytes())
            else:
                add(tname, "BF16", list(q.shape), bf16_bits(w).tobytes())

    add("model.embed_tokens.weight", "BF16", [cfg.vocab, cfg.d], bf16_bits(W["emb"]).tobytes())
    for l, lw in enumerate(W["layers"]):
        pre = "model.layers.%d." % l
        for key, hf in HF.items():
            if key + "_q4k" in lw:  # K-quant super-blocks are stored as they are
                add(pre + hf + ".weight", "Q4_K", list(lw[key][0].shape), np.ascontiguousarray(lw[key + "_q4k"], np.uint8).tobytes())
            else:
                linear(pre + hf + ".weight", *lw[key])
        add(pre + "input_layernorm.weight", "F32", [cfg.d], np.asarray(lw["norm1"], np.float32).tobytes())
        add(pre + "post_attention_layernorm.weight", "F16", [cfg.d], np.asarray(lw["norm2"], np.float16).tobytes())
        if "qnorm" in lw:
            add(pre + "self_attn.q_norm.weight", "F32", [cfg.hd], np.asarray(lw["qnorm"], np.float32).tobytes())
            add(pre + "self_attn.k_norm.weight", "F32", [cfg.hd], np.asarray(lw["knorm"], np.float32).tobytes())
    add("model.norm.weight", "F32", [cfg.d], np.asarray(W["final_norm"], np.float32).tobytes())
    if not tie_head:
        add("lm_head.weight", "BF16", [cfg.vocab, cfg.d], bf16_bits(W["lm_head"]).tobytes())
    weights = b"".join(blobs)
    front = ('[cyb]\ntypes = ["model"]\nname = "%s"\n\n[[files]]\nname = "config"\nformat = "toml"\n\n'
             '[[files]]\nname = "tensors"\nformat = "toml"\n\n[[files]]\nname = "weights"\nformat = "raw"\nsize = %d\n'
             % (name, len(weights)))
    config = ('architecture = "LlamaStyle"  # the family name cyb uses for its catalog models\n'
              "hidden_size = %d\nintermediate_size = %d\nnum_hidden_layers = %d\nnum_attention_heads = %d\n"
              "num_key_value_heads = %d\nhead_dim = %d\nvocab_size = %d\nrms_norm_eps = %r\nrope_theta = %r\n"
              % (cfg.d, cfg.ffn, cfg.layers, cfg.heads, cfg.kv_heads, cfg.hd, cfg.vocab, cfg.eps, cfg.rope_base))
    index = "".join('[[tensor]]\nname = "%s"\ndtype = "%s"\nshape = %s\noffset = %d\nsize = %d\n\n' % t for t in tensors)
    with open(path, "wb") as f:
        f.write(front.encode())
        f.write(b"~~~config\n" + config.encode())
        f.write(b"~~~tensors\n" + index.encode())
        f.write(b"~~~weights\n" + weights)
    return len(tensors)
