"""The tensor-parallel path on CPU: two gloo ranks shard one decoder layer by the engine's rules
(tests/tp_rules.py), compute their parts with the oracle, sum the row-split partials with an
all-reduce, and must reproduce the unsharded layer."""
import os
import socket

import numpy as np
import pytest

from oracle import ref


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out):
    import torch
    import torch.distributed as dist
    import tp_rules as tp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = ref.DecoderConfig(layers=1, d=256, ffn=512, heads=4, kv_heads=2, vocab=64)
    W = ref.make_decoder_weights(cfg, seed=9)
    lw = W["layers"][0]
    x = ref.rng_of(3).standard_normal((1, 5, cfg.d), dtype=np.float32).astype(np.float64)
    pos = np.arange(5)[None]
    sh = {nm: tp.shard_matrix(nm, *lw[nm], rank, world) for nm in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown")}

    def allreduce(a):
        t = torch.from_numpy(np.ascontiguousarray(a))
        dist.all_reduce(t)
        return t.numpy()

    hq, hkv = cfg.heads // world, cfg.kv_heads // world
    n1 = ref.rmsnorm(x, lw["norm1"], cfg.eps).reshape(5, cfg.d)
    q = ref.f16_round(ref.rope(ref.gemm_q4(n1, *sh["wq"]).reshape(1, 5, hq, 128), pos))
    k = ref.f16_round(ref.rope(ref.gemm_q4(n1, *sh["wk"]).reshape(1, 5, hkv, 128), pos))
    v = ref.f16_round(ref.gemm_q4(n1, *sh["wv"]).reshape(1, 5, hkv, 128))
    att = np.zeros((5, hq, 128))
    for t in range(5):
        att[t] = ref.attn_decode(q[0, t][None], [k[0, :t + 1]], [v[0, :t + 1]])[0]
    h = x[0] + allreduce(ref.gemm_q4(att.reshape(5, -1), *sh["wo"]))
    n2 = ref.rmsnorm(h, lw["norm2"], cfg.eps)
    act = ref.swiglu(ref.gemm_q4(n2, *sh["wgate"]), ref.gemm_q4(n2, *sh["wup"]))
    y = h + allreduce(ref.gemm_q4(act, *sh["wdown"]))
    # LM head split by vocabulary rows: every rank contributes its (max, global index) pair in its own
    # slot of a zeroed vector; the all-reduce (a sum with zeros) is the gather; every rank picks the token
    v0, v1 = tp.vocab_shard(cfg.vocab, rank, world)
    xn = ref.rmsnorm(y[-1:], W["final_norm"], cfg.eps)
    logits = xn @ W["lm_head"][v0:v1].astype(np.float64).T
    pairs = np.zeros((world, 1, 2), np.float32)
    pairs[rank, 0] = (np.float32(logits[0].max()), np.float32(v0 + int(logits[0].argmax())))
    token = tp.pick_token(allreduce(pairs))[0]
    if rank == 0:
        teacher = ref.Decoder(cfg, W)
        teacher.reset(1)
        want = teacher.layer(0, x, pos)[0]
        full = ref.rmsnorm(want[-1:], W["final_norm"], cfg.eps) @ W["lm_head"].astype(np.float64).T
        assert token == int(full[0].argmax()), (token, int(full[0].argmax()))
        out.put(float(np.abs(y - want).max() / np.abs(want).max()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_layer_matches_unsharded():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    err = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err < 1e-12, err


def test_shard_bounds_cover_and_reject():
    import tp_rules as tp
    for world in (1, 2, 4, 8):
        rows = [tp.shard_bounds("wgate", 11008, 4096, r, world) for r in range(world)]
        assert rows[0][0] == 0 and rows[-1][1] == 11008 and all(a[1] == b[0] for a, b in zip(rows, rows[1:]))
        cols = [tp.shard_bounds("wdown", 4096, 11008, r, world) for r in range(world)]
        assert cols[0][2] == 0 and cols[-1][3] == 11008 and all(c[2] % 32 == 0 for c in cols)
    with pytest.raises(ValueError):
        tp.shard_bounds("wdown", 4096, 11008, 0, 16)  # 688 is not a whole number of 32-blocks


def test_vocab_shard_and_token_pick():
    import tp_rules as tp
    for world in (2, 4, 8):
        b = [tp.vocab_shard(32000, r, world) for r in range(world)]
        assert b[0][0] == 0 and b[-1][1] == 32000 and all(x[1] == y[0] for x, y in zip(b, b[1:]))
    assert tp.vocab_shard(32001, 1, 2) == (0, 32001)   # does not divide: replicated
    assert tp.vocab_shard(32000, 0, 1) == (0, 32000)
    # ties go to the lowest global index, whichever rank holds it
    pairs = np.array([[[1.5, 7.0]], [[2.5, 16003.0]], [[2.5, 9001.0]], [[-1.0, 30000.0]]], np.float32)
    assert tp.pick_token(pairs) == [9001]
