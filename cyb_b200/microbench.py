"""Kernel microbenchmarks over the C ABI (device-resident inputs, CUDA events).

    python -m cyb_b200.microbench gemv --n 4096 --k 4096 [--m 1] [--dtype f32|bf16] [--pool 24] [--iters 20]
    python -m cyb_b200.microbench attn [--batch 16] [--lo 512] [--hi 4096]
    python -m cyb_b200.microbench lmhead [--m 1]
    python -m cyb_b200.microbench prefill [--m 2048] [--n 11008] [--k 4096]
    python -m torch.distributed.run --nproc-per-node 2 -m cyb_b200.microbench allreduce [--elems 4096]

`gemv` rotates through a pool of distinct packed weights larger than the 126 MB
L2, so every launch streams its weights from HBM; the figure printed is
algorithmic bytes / time.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np


def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def gemv(args):
    import torch
    from cyb_b200 import qeng
    opts = {k: v for k, v in (("stream_groups", args.groups), ("stream_stage_chunks", args.stage_chunks)) if v}
    ctx = qeng.Context(0, **opts)
    n, k, m = args.n, args.k, args.m
    wbytes = n * k * (1.0625 if args.q8 else 0.5625)
    pool = args.pool or max(2, int(160e6 // wbytes) + 1)
    quant = ctx.quantize_q8 if args.q8 else ctx.quantize_q4
    ws = [quant(torch.randn(n, k, device="cuda") * 0.05) for _ in range(pool)]  # timing only: any weights do
    dt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[args.dtype]
    x = torch.randn(m, k, device="cuda").to(dt)
    y = torch.empty(m, n, device="cuda")
    algo = wbytes + m * k * x.element_size() + m * n * 4
    # the launches are replayed from a CUDA graph so that the host launch rate does not bound the figure
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(2 * pool):
            ctx.gemm_q4(ws[i % pool], x, out=y, flags=args.flags)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for w in ws:
            ctx.gemm_q4(w, x, out=y, flags=args.flags)
    graph.replay()
    e0, e1 = _events(torch)
    torch.cuda.synchronize()
    e0.record()
    for it in range(args.iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.iters * pool)
    ctx.device_status()
    print(json.dumps({"kernel": "gemm_q4", "n": n, "k": k, "m": m, "dtype": args.dtype, "pool": pool,
                      "us_per_launch": us, "algo_bytes": algo, "gbs": algo / us / 1e3}))


def attn(args):
    import torch
    from cyb_b200 import qeng
    ctx = qeng.Context(0)
    rng = np.random.Generator(np.random.PCG64(4))
    B, Hq, Hkv = args.batch, 32, 8
    lens = rng.integers(args.lo, args.hi + 1, B).astype(np.int32)
    npages = (lens + 15) // 16
    total = int(npages.sum())
    pools = []
    for _ in range(args.pool):
        p = ctx.kv_pool(total, Hkv)
        p.tensor().normal_()
        pools.append(p)
    order = rng.permutation(total).astype(np.int32)
    table = np.zeros((B, int(npages.max())), np.int32)
    off = 0
    for b in range(B):
        table[b, :npages[b]] = order[off:off + npages[b]]
        off += npages[b]
    q = torch.randn(B, Hq, 128, device="cuda").half()
    tb, ln = torch.from_numpy(table).cuda(), torch.from_numpy(lens).cuda()
    algo = float(lens.sum()) * Hkv * 2 * 128 * 2 + 2 * B * Hq * 128 * 2
    # replayed from a CUDA graph (8 calls per pool entry) so that the host launch rate does not bound
    # the figure of small cases
    reps = 8
    out = torch.empty(B, Hq, 128, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(3):
            ctx.attn_decode(pools[i % args.pool], q, tb, ln, out=out)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(reps):
            for p in pools:
                ctx.attn_decode(p, q, tb, ln, out=out)
    graph.replay()
    e0, e1 = _events(torch)
    torch.cuda.synchronize()
    e0.record()
    for it in range(args.iters):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.iters * args.pool * reps)
    ctx.device_status()
    print(json.dumps({"kernel": "attn_decode", "batch": B, "tokens": int(lens.sum()), "us_per_call": us,
                      "algo_bytes": algo, "gbs": algo / us / 1e3}))


def lmhead(args):
    import torch
    from cyb_b200 import qeng
    ctx = qeng.Context(0)
    V, D = 32000, 4096
    tb = (torch.randn(V, D, device="cuda") * 0.02).bfloat16().view(torch.int16)
    x = torch.randn(args.m, D, device="cuda")
    for _ in range(3):
        ctx.lm_head(tb, x)
    e0, e1 = _events(torch)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    tot = 0.0
    for it in range(args.iters):
        flush.zero_()
        e0.record()
        ctx.lm_head(tb, x)
        e1.record()
        torch.cuda.synchronize()
        tot += e0.elapsed_time(e1)
    us = tot * 1e3 / args.iters
    algo = V * D * 2 + args.m * (D + V) * 4
    print(json.dumps({"kernel": "lm_head", "m": args.m, "us_per_call": us, "algo_bytes": algo, "gbs": algo / us / 1e3}))


def prefill(args):
    import torch
    from cyb_b200 import qeng
    ctx = qeng.Context(0)
    n, k, m = args.n, args.k, args.m
    rng = np.random.Generator(np.random.PCG64(0))
    q = rng.integers(0, 16, (n, k), dtype=np.uint8)
    s = rng.uniform(0.002, 0.02, (n, k // 32)).astype(np.float16)
    w = ctx.pack_q4(q, s)
    x = torch.randn(m, k, device="cuda").bfloat16()
    y = torch.empty(m, n, device="cuda")
    for _ in range(3):
        ctx.gemm_q4(w, x, out=y)
    e0, e1 = _events(torch)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.iters):
        ctx.gemm_q4(w, x, out=y)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    ctx.device_status()
    print(json.dumps({"kernel": "gemm_q4 (tcgen05 prefill)", "m": m, "n": n, "k": k, "ms": ms,
                      "tflops": 2.0 * m * n * k / ms / 1e9}))


def allreduce(args):
    """Run under torch.distributed.run, one rank per GPU: latency of dst += allreduce(part)."""
    import os
    import torch
    import torch.distributed as dist
    from cyb_b200 import qeng
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo")
    ctx = qeng.Context(rank)

    def bc(b):
        o = [b]
        dist.broadcast_object_list(o, src=0)
        return o[0]

    def ag(b):
        o = [None] * world
        dist.all_gather_object(o, b)
        return o
    ctx.tp_init(rank, world, bc, ag)
    part = torch.ones(args.elems, device="cuda")
    dst = torch.zeros(args.elems, device="cuda")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(4):
            ctx.all_reduce_add_(dst, part)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(50):
            ctx.all_reduce_add_(dst, part)
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = _events(torch)
    e0.record()
    for _ in range(args.iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (args.iters * 50)
    ctx.device_status()
    expect = world * (4 + 50 * (args.iters + 1))
    if rank == 0:
        print(json.dumps({"kernel": "all_reduce_add", "world": world, "n": args.elems, "us_per_call": us,
                          "correct": bool(float(dst[0]) == expect and float(dst[-1]) == expect)}))
    dist.barrier()
    dist.destroy_process_group()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="cyb_b200.microbench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("gemv")
    g.add_argument("--n", type=int, default=4096)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--m", type=int, default=1)
    g.add_argument("--dtype", default="f32")
    g.add_argument("--pool", type=int, default=0)
    g.add_argument("--iters", type=int, default=20)
    g.add_argument("--flags", type=int, default=0)
    g.add_argument("--groups", type=int, default=0, help="tile groups of the streaming kernel (1, 2, 4; 0 = by shape)")
    g.add_argument("--q8", action="store_true", help="8-bit blocks instead of 4-bit")
    g.add_argument("--stage-chunks", type=int, default=0, help="K chunks per ring stage (0 = default)")
    a = sub.add_parser("attn")
    a.add_argument("--batch", type=int, default=16)
    a.add_argument("--lo", type=int, default=512)
    a.add_argument("--hi", type=int, default=4096)
    a.add_argument("--pool", type=int, default=2)
    a.add_argument("--iters", type=int, default=20)
    l = sub.add_parser("lmhead")
    l.add_argument("--m", type=int, default=1)
    l.add_argument("--iters", type=int, default=10)
    pf = sub.add_parser("prefill")
    pf.add_argument("--m", type=int, default=2048)
    pf.add_argument("--n", type=int, default=11008)
    pf.add_argument("--k", type=int, default=4096)
    pf.add_argument("--iters", type=int, default=10)
    ar = sub.add_parser("allreduce")
    ar.add_argument("--elems", type=int, default=4096)
    ar.add_argument("--iters", type=int, default=20)
    args = ap.parse_args(argv)
    {"allreduce": allreduce, "gemv": gemv, "attn": attn, "lmhead": lmhead, "prefill": prefill}[args.cmd](args)


if __name__ == "__main__":
    main()
