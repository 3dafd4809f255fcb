"""Tensor parallelism on real GPUs (needs >= 2): two ranks, NCCL all-reduce after the row-split
projections; tokens and logits must match the unsharded oracle decoder."""
import os
import socket

import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cyb_b200 import qeng
    ctx = qeng.Context(rank)

    def exchange(b):
        obj = [b]
        dist.broadcast_object_list(obj, src=0)
        return obj[0]
    def allgather(b):
        outl = [None] * world
        dist.all_gather_object(outl, b)
        return outl
    ctx.tp_init(rank, world, exchange, allgather)
    t = torch.full((1000,), float(rank + 1), device="cuda")
    ctx.all_reduce_(t)
    torch.cuda.synchronize()
    assert float(t[0]) == sum(range(1, world + 1))
    cfg = ref.DecoderConfig(layers=2, d=256, ffn=512, heads=4, kv_heads=2, vocab=320)
    W = ref.make_decoder_weights(cfg, seed=5)
    dec = ctx.decoder(layers=2, d_model=256, ffn=512, heads=4, kv_heads=2, vocab=320, max_batch=2, max_seq=64,
                      tp_rank=rank, tp_world=world)
    qeng.load_decoder_weights(dec, W, cfg)
    prompt = GOLD["dec_prompt"]
    dec.reset(prompt.shape[0])
    dec.prefill(prompt)
    e = ref.err_inf(dec.logits(), GOLD["dec_logits"][0])
    toks = dec.decode(GOLD["dec_tokens"].shape[1])
    ctx.device_status()
    out.put((rank, e, toks.tolist()))
    dist.barrier()
    dec.free()
    dist.destroy_process_group()


def test_two_rank_decoder_matches_golden(built_lib):
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = [out.get(timeout=300) for _ in range(2)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, e, toks in res:
        assert e < 2e-3, (rank, e)
        assert toks == GOLD["dec_tokens"].tolist(), rank


def _lonely_rank_main(rank, world, port, out):
    """Rank 0 starts an all-reduce that rank 1 never joins: the bounded wait must run out, the
    status word must say so, and the context must stay usable.  Rank 1 is idle the whole time."""
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cyb_b200 import qeng
    ctx = qeng.Context(rank)

    def exchange(b):
        obj = [b]
        dist.broadcast_object_list(obj, src=0)
        return obj[0]

    def allgather(b):
        outl = [None] * world
        dist.all_gather_object(outl, b)
        return outl
    ctx.tp_init(rank, world, exchange, allgather)
    res = None
    if rank == 0:
        dst = torch.zeros(4096, device="cuda")
        part = torch.ones(4096, device="cuda")
        ctx.all_reduce_add_(dst, part)  # nobody answers
        try:
            ctx.device_status()
            res = "no error"
        except qeng.QengError as e:
            res = (e.code, "peer" in str(e))
        # the context still computes
        rng = ref.rng_of(1)
        q, s = ref.make_q4(rng, 32, 64)
        x = rng.standard_normal((1, 64), dtype=np.float32)
        w = ctx.pack_q4(q, s)
        y = ctx.gemm_q4(w, torch.from_numpy(x).cuda()).cpu().numpy()
        res = res + (ref.err_inf(y, ref.gemm_q4(x, q, s)) < 2e-6,) if isinstance(res, tuple) else res
    dist.barrier()  # rank 0 is done, nothing is in flight
    # recovery: the call counters disagree now; both ranks clear their inboxes, meet on the host,
    # and the next all-reduce (joined by both) must work
    ctx.tp_p2p_reset()
    dist.barrier()
    dst = torch.full((4096,), 10.0, device="cuda")
    part = torch.full((4096,), float(rank + 1), device="cuda")
    ctx.all_reduce_add_(dst, part)
    torch.cuda.synchronize()
    ctx.device_status()
    ok = bool((dst == 13.0).all())
    if rank == 0:
        res = res + (ok,) if isinstance(res, tuple) else res
    dist.barrier()  # nobody leaves with a collective in flight
    out.put((rank, res))
    dist.destroy_process_group()


def test_missing_peer_is_reported_not_hung(built_lib):
    import torch
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_lonely_rank_main, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(out.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res[0] == (-7, True, True, True), res
