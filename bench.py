#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s of a 7B-shaped 4-bit Llama-style
decoder (32 layers, d 4096, FFN 11008, 32/8 heads, vocab 32000) on N B200s,
the HBM roofline of its dominant kernel, and the kernel-level figures of the
other configurations (single GEMV, decode-batch GEMM sweep, prefill GEMM,
decode attention, LM head, batch-16 decode).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

A step is one decode step (one new token per sequence) at context >= 512.
Prints ONE JSON line (rank 0).  Inputs are synthetic: seeded random 4-bit
weights, bf16 embeddings / LM head ~N(0, 0.02), a random 512-token prompt.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL = dict(layers=32, d=4096, ffn=11008, heads=32, kv_heads=8, hd=128, vocab=32000)
PROMPT = 512
METRIC = "decode tokens/s (7B 4-bit, 1/2/4/8 B200); quant GEMV HBM GB/s vs peak"
# DRAM bytes (read + written) per algorithmic byte of the decode matmul, from one ncu capture of
# the gate|up shape (50.80 MB read + 9.5 KB written against 50.83 MB algorithmic); the traffic
# grows in proportion to N*K, so the bench line scales this constant instead of measuring it.
NCU_TRAFFIC_PER_ALGO_BYTE = 0.9996
GOLDEN = os.path.join(ROOT, "tests", "golden")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["layers"], help="for quick checks only; the bench config is 32")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the kernel-level legs")
    ap.add_argument("--save-tokens", default=None, help="write the generated tokens (JSON) to this path")
    return ap.parse_args()


# --------------------------------------------------------------------------
# synthetic weights: per-matrix independent streams, made on the host
# --------------------------------------------------------------------------
def layer_shapes(m):
    nq, nkv = m["heads"] * m["hd"], m["kv_heads"] * m["hd"]
    return [("wq", nq, m["d"]), ("wk", nkv, m["d"]), ("wv", nkv, m["d"]), ("wo", m["d"], nq),
            ("wgate", m["ffn"], m["d"]), ("wup", m["ffn"], m["d"]), ("wdown", m["d"], m["ffn"])]


def gen_matrix(seed, n, k):
    rng = np.random.Generator(np.random.PCG64(seed))
    q = rng.integers(0, 16, (n, k), dtype=np.uint8)
    s = rng.uniform(0.002, 0.02, (n, k // 32)).astype(np.float16)
    return q, s


def gen_table(seed, v, d):
    rng = np.random.Generator(np.random.PCG64(seed))
    x = rng.standard_normal((v, d), dtype=np.float32) * np.float32(0.02)
    u = x.view(np.uint32).astype(np.uint64)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def algo_bytes_per_step(m, batch, ctx_len, tp=1):
    """Algorithmic HBM bytes of one decode step per GPU: packed weights once,
    bf16 LM head once, KV read once."""
    lin = sum(n * k for _, n, k in layer_shapes(m)) * m["layers"]
    kv = batch * ctx_len * m["kv_heads"] * 2 * m["hd"] * 2 * m["layers"]
    return (lin * 0.5625 + m["vocab"] * m["d"] * 2 + kv) / tp


# --------------------------------------------------------------------------
# clocks: read-only NVML polling from a thread, fast enough to land samples inside a timed
# region of a few tens of milliseconds (nvidia-smi's own loop is too slow to start for that)
# --------------------------------------------------------------------------
class ClockSampler:
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, index=0, period_s=0.002):
        self.index, self.period, self.rows, self.marks = index, period_s, [], []
        self.stop = threading.Event()
        self.h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            dev = self._physical(index)
            self.h = pynvml.nvmlDeviceGetHandleByIndex(dev) if isinstance(dev, int) else pynvml.nvmlDeviceGetHandleByUUID(dev)
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.h = None

    @staticmethod
    def _physical(index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",") if v.strip() != ""]
            if index < len(ids):
                return int(ids[index]) if ids[index].isdigit() else ids[index]
        return index

    def _run(self):
        nv = self.nv
        while not self.stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                except Exception:
                    rs = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
                self.rows.append((time.perf_counter(), sm, rs))
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.h is not None:
            self.t = threading.Thread(target=self._run, daemon=True)
            self.t.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        if self.h is not None:
            self.t.join(timeout=1)

    def region(self):
        """Context manager marking a timed region: only samples taken inside regions count."""
        sampler = self

        class _R:
            def __enter__(self):
                self.t0 = time.perf_counter()

            def __exit__(self, *a):
                sampler.marks.append((self.t0, time.perf_counter()))
        return _R()

    def summary(self):
        inside = [r for r in self.rows if any(a <= r[0] <= b for a, b in self.marks)]
        sm = [r[1] for r in inside]
        bits = 0
        for r in inside:
            bits |= r[2]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": getattr(self, "max_sm", None),
                "reasons": [n for n, b in self.REASONS.items() if bits & b], "samples": len(sm),
                "how": "NVML polled every %.0f ms from a thread; samples inside the timed regions only" % (self.period * 1e3)}


# --------------------------------------------------------------------------
# CPU baseline (the oracle's C port on the host cores) — rank 0 only
# --------------------------------------------------------------------------
def _host_cores():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def _cpu_env():
    """All host cores, threads pinned: must run before the oracle's OpenMP runtime loads
    (torch.distributed.run exports OMP_NUM_THREADS=1 to its workers)."""
    os.environ["OMP_NUM_THREADS"] = str(_host_cores())
    os.environ.setdefault("OMP_PROC_BIND", "close")
    os.environ.setdefault("OMP_PLACES", "cores")


def cpu_decode_rate(m, batch, ctx_len, budget_s=None, steps=None, warmup=3):
    """Times CPU decode steps on a bounded sample: `sample_layers` of the model's
    layers (per-layer cost is identical; the LM head is timed in full) with a
    synthetic KV cache of ctx_len tokens.  Returns a dict: tokens/s extrapolated to
    the full depth (from the median step), its min/max over the timed steps, cores, description."""
    from oracle import cport, ref
    cores = cport.threads()
    sample_layers = min(m["layers"], 2)
    cfg = ref.DecoderConfig(layers=sample_layers, d=m["d"], ffn=m["ffn"], heads=m["heads"], kv_heads=m["kv_heads"],
                            hd=m["hd"], vocab=m["vocab"])
    W = {"layers": [], "final_norm": np.ones(m["d"], np.float32)}
    for l in range(sample_layers):
        lw = {"norm1": np.ones(m["d"], np.float32), "norm2": np.ones(m["d"], np.float32)}
        for j, (nm, n, k) in enumerate(layer_shapes(m)):
            lw[nm] = gen_matrix(1000 + 7 * l + j, n, k)
        W["layers"].append(lw)
    tb = gen_table(1, m["vocab"], m["d"])
    f32 = lambda bits: (bits.astype(np.uint32) << 16).view(np.float32)
    W["emb"], W["lm_head"] = f32(tb), f32(gen_table(2, m["vocab"], m["d"]))
    max_pages = (ctx_len + 64 + 15) // 16
    dec = cport.CpuDecoder(cfg, W, pages_per_layer=batch * max_pages)
    pool = dec.pool()
    rng = np.random.Generator(np.random.PCG64(3))
    pool[:] = rng.standard_normal(pool.shape[0], dtype=np.float32).astype(np.float16)
    table = np.arange(batch * max_pages, dtype=np.int32).reshape(batch, max_pages)
    toks = rng.integers(0, m["vocab"], batch).astype(np.int32)
    # layers and head are timed separately: the slice's step holds the whole head
    x = rng.standard_normal((batch, m["d"]), dtype=np.float32)
    for _ in range(warmup):
        cport.gemm_bf16(x, dec.lm)
    th = []
    for _ in range(7):
        t0 = time.perf_counter()
        cport.gemm_bf16(x, dec.lm)
        th.append(time.perf_counter() - t0)
    t_head = statistics.median(th)
    for i in range(warmup):
        dec.step(toks, np.full(batch, ctx_len + i, np.int32), table)
    times = []
    t_start = time.perf_counter()
    n = 0
    while True:
        t0 = time.perf_counter()
        dec.step(toks, np.full(batch, ctx_len + 1 + n % 32, np.int32), table)
        times.append(time.perf_counter() - t0)
        n += 1
        if steps is not None:
            if n >= steps:
                break
        elif time.perf_counter() - t_start > budget_s or n >= 256:
            break
    dec.close()

    def full(t_step):
        th_ = min(t_head, 0.9 * t_step)  # never extrapolate a negative layer time
        return (t_step - th_) / sample_layers * m["layers"] + th_
    per_full = full(statistics.median(times))
    desc = ("%d decode steps (after %d warm-up) of a %d-layer slice (+ full LM head) at context %d, batch %d, "
            "extrapolated x%d/%d layers; median step" % (n, warmup, sample_layers, ctx_len, batch, m["layers"], sample_layers))
    return {"value": batch / per_full, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc,
            "min": batch / full(max(times)), "max": batch / full(min(times)), "s_per_step": per_full}


def run_reference(args):
    """The reference arm: the CPU restatement of the path (the reference's own
    runtime crates are absent from its checkout) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    _cpu_env()
    m = dict(MODEL)
    t0 = time.perf_counter()
    r = cpu_decode_rate(m, args.batch, PROMPT, steps=max(args.steps, 1), warmup=max(args.warmup, 3))
    line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": r["s_per_step"] * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "configs[4]: 32-layer d4096 ffn11008 32/8-head 4-bit decoder, greedy decode at context %d, batch %d" % (PROMPT, args.batch)},
            "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "min", "max")},
            "e2e": {"value": r["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line))


# --------------------------------------------------------------------------
# kernel-level legs (1 GPU): device-resident inputs, graph replay over a pool of distinct
# buffers larger than L2, CUDA events on the replaying stream
# --------------------------------------------------------------------------
def _time_graph(torch, calls, iters=10):
    """calls: list of zero-argument launchers.  Returns microseconds per call."""
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for c in calls:
            c()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for c in calls:
            c()
    for _ in range(3):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * len(calls))


def kernel_legs(ctx, torch, peaks):
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf = float(peaks.get("bf16_tflops", 1590.0))
    out = []
    L2 = 160e6  # a pool at least this large never fits the 126 MB L2

    def wpool(n, k, count, q8=False):
        quant = ctx.quantize_q8 if q8 else ctx.quantize_q4
        return [quant(torch.randn(n, k, device="cuda") * 0.05) for _ in range(count)]

    def gemm_leg(name, m, n, k, dt, q8=False):
        wb = n * k * (1.0625 if q8 else 0.5625)
        ws = wpool(n, k, max(2, int(L2 // wb) + 1), q8)
        x = torch.randn(m, k, device="cuda").to(dt)
        y = torch.empty(m, n, device="cuda")
        us = _time_graph(torch, [lambda w=w: ctx.gemm_q4(w, x, out=y) for w in ws])
        algo = wb + m * k * x.element_size() + m * n * 4
        out.append({"name": name, "m": m, "n": n, "k": k, "x": str(dt).split(".")[-1], "algo_bytes": algo, "us": us,
                    "achieved": algo / us / 1e3, "unit": "GB/s", "frac": algo / us / 1e3 / hbm,
                    "l2_policy": "pool of %d distinct weights (%.0f MB) replayed from a graph" % (len(ws), len(ws) * wb / 1e6)})
        for w in ws:
            w.free()

    gemm_leg("configs[0] gemv", 1, 4096, 4096, torch.float32)
    for (n, k) in [(4096, 4096), (11008, 4096), (4096, 11008)]:
        for m in (1, 8, 32):
            gemm_leg("configs[1] decode-batch gemm", m, n, k, torch.bfloat16)
    # 8-bit blocks ("tensor data (Q4/Q8/F16/F32)"): the same kernel on signed bytes, 1.0625 B per weight
    for (n, k) in [(4096, 4096), (11008, 4096)]:
        gemm_leg("8-bit blocks, decode gemv", 1, n, k, torch.float32, q8=True)
    # prefill: tensor-bound
    for (n, k) in [(11008, 4096), (4096, 11008)]:
        w0 = wpool(n, k, 1)[0]
        for m in (512, 2048, 8192):
            per = n * k * 0.5625 + m * k * 2 + m * n * 4
            cnt = max(1, int(L2 // per) + 1)
            xs = [torch.randn(m, k, device="cuda").bfloat16() for _ in range(cnt)]
            ys = [torch.empty(m, n, device="cuda") for _ in range(cnt)]
            ws = [w0] + (wpool(n, k, cnt - 1) if cnt > 1 else [])
            us = _time_graph(torch, [lambda i=i: ctx.gemm_q4(ws[i], xs[i], out=ys[i]) for i in range(cnt)], iters=5)
            fl = 2.0 * m * n * k
            out.append({"name": "configs[2] prefill gemm", "m": m, "n": n, "k": k, "flops": fl, "us": us,
                        "achieved": fl / us / 1e6, "unit": "TFLOP/s", "frac": fl / us / 1e6 / tf,
                        "l2_policy": "%d distinct (weight, activation, output) sets, %.0f MB per call" % (cnt, per / 1e6)})
            for w in ws[1:]:
                w.free()
            del xs, ys
        w0.free()
    # decode attention, configs[3]
    rng = np.random.Generator(np.random.PCG64(4))
    B, Hq, Hkv = 16, 32, 8
    lens = rng.integers(512, 4097, B).astype(np.int32)
    npages = (lens + 15) // 16
    total = int(npages.sum())
    pools = []
    for _ in range(2):
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
    o = torch.empty(B, Hq, 128, device="cuda")
    us = _time_graph(torch, [lambda p=p: ctx.attn_decode(p, q, tb, ln, out=o) for p in pools] * 4)
    algo = float(lens.sum()) * Hkv * 2 * 128 * 2 + 2 * B * Hq * 128 * 2
    out.append({"name": "configs[3] decode attention", "batch": B, "tokens": int(lens.sum()), "algo_bytes": algo, "us": us,
                "achieved": algo / us / 1e3, "unit": "GB/s", "frac": algo / us / 1e3 / hbm,
                "l2_policy": "2 distinct KV pools (%.0f MB) replayed from a graph" % (2 * algo / 1e6)})
    for p in pools:
        p.free()
    # LM head (bf16 [32000, 4096]), M = 1
    V, D = MODEL["vocab"], MODEL["d"]
    tbs = [(torch.randn(V, D, device="cuda") * 0.02).bfloat16().view(torch.int16) for _ in range(2)]
    x = torch.randn(1, D, device="cuda")
    lo = torch.empty(1, V, device="cuda")

    us = _time_graph(torch, [lambda t=t: ctx.lm_head(t, x, out=lo) for t in tbs] * 2)
    algo = V * D * 2 + (D + V) * 4
    out.append({"name": "lm head", "m": 1, "algo_bytes": algo, "us": us, "achieved": algo / us / 1e3, "unit": "GB/s",
                "frac": algo / us / 1e3 / hbm, "l2_policy": "2 distinct tables (524 MB) replayed from a graph"})
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("bench.py: --gpus %d but WORLD_SIZE %d (launch with torch.distributed.run for N>1)" % (args.gpus, world))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    # the weight import (re-tiling on the host) is OpenMP-parallel; torch.distributed.run pins
    # OMP_NUM_THREADS to 1, so give every rank its share of the cores before the library loads
    if world == 1:
        _cpu_env()  # also the CPU-baseline leg's settings: OpenMP reads them once, when it loads
    else:
        os.environ["OMP_NUM_THREADS"] = str(max(1, _host_cores() // world))
    from cyb_b200 import qeng
    m = dict(MODEL)
    m["layers"] = args.layers
    B, K, Wm = args.batch, args.steps, max(args.warmup, 3)
    B16 = 16  # the second half of configs[4]
    ctx = qeng.Context(local)
    if world > 1:
        def exchange(b):
            obj = [b]
            dist.broadcast_object_list(obj, src=0)
            return obj[0]
        def allgather(b):
            out = [None] * world
            dist.all_gather_object(out, b)
            return out
        ctx.tp_init(rank, world, exchange, allgather)
    max_seq = PROMPT + Wm + 2 * K + 64
    dec = ctx.decoder(layers=m["layers"], d_model=m["d"], ffn=m["ffn"], heads=m["heads"], kv_heads=m["kv_heads"],
                      vocab=m["vocab"], max_batch=max(B, B16), max_seq=max_seq, tp_rank=rank, tp_world=world)
    t_load = time.perf_counter()
    for l in range(m["layers"]):
        for j, (nm, n, k) in enumerate(layer_shapes(m)):
            dec.load_matrix(l, j, *gen_matrix(1000 + 7 * l + j, n, k))
        dec.load_norm(l, 0, np.ones(m["d"], np.float32))
        dec.load_norm(l, 1, np.ones(m["d"], np.float32))
    dec.load_head(gen_table(1, m["vocab"], m["d"]), gen_table(2, m["vocab"], m["d"]), np.ones(m["d"], np.float32))
    t_load = time.perf_counter() - t_load

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def maxr(v):
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dec.use_current_stream()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    teacher, decode_errs = None, []
    tpath = os.path.join(GOLDEN, "config5_teacher.npz")
    if B == 1 and m["layers"] == MODEL["layers"] and os.path.exists(tpath):
        teacher = dict(np.load(tpath))

    def run_batch(Bn, Kn, clk=None):
        """prompt of PROMPT tokens then Wm warm-up and Kn timed decode steps at batch Bn."""
        prompt = np.random.Generator(np.random.PCG64(7)).integers(0, m["vocab"], (Bn, PROMPT)).astype(np.int32)
        dec.reset(Bn)
        dec.prefill(prompt)  # first call: buffers grow, kernels load
        dec.reset(Bn)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        dec.prefill(prompt)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        logits0 = dec.logits()
        if teacher is not None and Bn == 1:
            # teacher-forced while the tokens agree: logits of the first decode steps against the fixture
            n = min(8, Wm)
            got, errs = [], []
            for s_ in range(n):
                got.append(dec.decode(1))
                lg = dec.logits()
                if s_ + 1 < len(teacher["tokens"]) and all(int(g_[0, 0]) == int(teacher["tokens"][i]) for i, g_ in enumerate(got)):
                    li = teacher["top_idx"][s_ + 1]
                    errs.append(float(np.abs(lg[0, li] - teacher["top_val"][s_ + 1]).max() / teacher["absmax"][s_ + 1]))
            decode_errs.extend(errs)
            warm = np.concatenate(got + ([dec.decode(Wm - n)] if Wm > n else []), 1)
        else:
            warm = dec.decode(Wm)
        barrier()
        if clk is not None:
            with clk.region():
                ev0.record()
                toks = dec.decode(Kn)
                ev1.record()
                barrier()
        else:
            ev0.record()
            toks = dec.decode(Kn)
            ev1.record()
            barrier()
        ms = maxr(ev0.elapsed_time(ev1))
        return ms, t_prefill, np.concatenate([warm, toks], 1), logits0

    with ClockSampler(local) as clk:
        ms, t_prefill, tokens, logits0 = run_batch(B, K, clk)
        value = B * K / (ms * 1e-3)
        launches = dec.launches_per_step * K
        ctx_mid = PROMPT + Wm + K // 2
        # ---- end to end: one call per token, every token read back to the host ---
        barrier()
        with clk.region():
            t0 = time.perf_counter()
            for _ in range(K):
                dec.decode(1)
            torch.cuda.synchronize()
            e2e_s = time.perf_counter() - t0
        e2e = B * K / maxr(e2e_s)

    # ---- what was computed: tokens against the float64 teacher and against the 1-GPU run ------
    check = {"tokens_crc32": "%08x" % zlib.crc32(np.ascontiguousarray(tokens, np.int32).tobytes()), "tokens_checked": 0}
    if B == 1 and m["layers"] == MODEL["layers"]:
        seq = tokens[0]
        if teacher is not None:
            t = teacher
            n = min(len(seq), len(t["tokens"]))
            agree = 0
            while agree < n and seq[agree] == t["tokens"][agree]:
                agree += 1
            li = t["top_idx"][0]
            check.update({"teacher_tokens": n, "teacher_prefix": agree,
                          "teacher_logits_err_step0": float(np.abs(logits0[0, li] - t["top_val"][0]).max() / t["absmax"][0]),
                          "teacher_logits_err_decode_steps": decode_errs,
                          "teacher": "float64 oracle, free-running greedy decode of the same seeded model (fixture); errors are max|logit - teacher| over the teacher's 8 best, / max|logit|"})
        ppath = os.path.join(GOLDEN, "bench_tokens_tp1.json")
        if os.path.exists(ppath):
            ref1 = json.load(open(ppath))["tokens"]
            n = min(len(seq), len(ref1))
            agree = 0
            while agree < n and int(seq[agree]) == ref1[agree]:
                agree += 1
            check.update({"tokens_checked": n, "tokens_match_tp1": agree == n, "tokens_common_prefix_tp1": agree})
    if args.save_tokens and rank == 0:
        json.dump({"tokens": [int(v) for v in tokens[0]], "batch": B, "warmup": Wm, "steps": K, "world": world},
                  open(args.save_tokens, "w"))

    # ---- roofline of the dominant kernel: the 4-bit GEMV over this decoder's own
    # weights (32 layers x 4 fused matrices = distinct buffers >> L2), timed with events
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    ws = [dec.weight(l, i) for l in range(m["layers"]) for i in range(4)]
    xs = {k: torch.randn(1, k, device="cuda") for k in {w.cols for w in ws}}
    ys = {w.rows: torch.empty(1, w.rows, device="cuda") for w in ws}
    algo = sum(w.rows * w.cols * 0.5625 + w.cols * 4 + w.rows * 4 for w in ws)
    # the activation precision each matrix gets inside the decoder: 22 bits for q|k|v, 15 for the rest
    flag = [0, qeng.GEMM_FAST_F16, qeng.GEMM_FAST_F16, qeng.GEMM_FAST_F16]
    per_launch_us = _time_graph(torch, [lambda w=w, i=i: ctx.gemm_q4(w, xs[w.cols], out=ys[w.rows], flags=flag[i % 4])
                                        for i, w in enumerate(ws)])
    achieved = algo / len(ws) / per_launch_us / 1e3
    roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "traffic": NCU_TRAFFIC_PER_ALGO_BYTE * algo / len(ws),
            "traffic_how": "one ncu capture of the gate|up shape (DRAM bytes = 0.9996 x algorithmic), scaled by N*K; not measured in this run",
            "kernel": "gemv_q4_stream_kernel (M=1, f32 activations), the decoder's own 4 x %d layer matrices in loop order, each at the precision the decoder uses" % m["layers"],
            "bytes_per_launch": algo / len(ws), "us_per_launch": per_launch_us,
            "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback",
            "frac_of_nominal_8tbs": achieved / 8000.0,
            "step_frac": algo_bytes_per_step(m, B, ctx_mid, world) / (ms * 1e-3 / K) / 1e9 / peak}

    # ---- batch 16 (the other half of configs[4]) and the kernel-level legs -----------------
    kernels = []
    b16 = None
    if not args.no_kernels and B != B16:
        K16 = min(K, 32)
        ms16, tp16, _, _ = run_batch(B16, K16)
        ctx16 = PROMPT + Wm + K16 // 2
        b16 = {"name": "configs[4] batch 16 decode", "value": B16 * K16 / (ms16 * 1e-3), "unit": "tokens/s",
               "ms_per_step": ms16 / K16, "steps": K16,
               "step_frac": algo_bytes_per_step(m, B16, ctx16, world) / (ms16 * 1e-3 / K16) / 1e9 / peak,
               "prefill_tokens_per_s": B16 * PROMPT / tp16}
    ctx.device_status()
    dec.free()
    if not args.no_kernels and world == 1:
        kernels = kernel_legs(ctx, torch, peaks)
        ctx.device_status()

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": Wm,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "s8 x u4 integer tensor-core contraction per 32-block (activations in 15/22-bit block fixed point), f32 accumulate",
                "data": "synthetic",
                "config": {"workload": "configs[4]: 32-layer d4096 ffn11008 32/8-head vocab-32000 4-bit decoder, prompt %d then greedy decode, batch %d" % (PROMPT, B),
                           "layers": m["layers"], "batch": B, "context_at_start": PROMPT + Wm, "parallelism": "tp%d" % world,
                           "l2_policy": "inputs larger than L2 (3.4 GB of weights streamed per step)"},
                "clocks": clk.summary(), "gpu_launches": launches,
                "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 4 * B + 4,
                        "how": "one qeng_decoder_decode(1) call per token, sampled token copied to the host every step"},
                "roofline": roof, "check": check, "prefill_s": t_prefill, "prefill_tokens_per_s": B * PROMPT / t_prefill,
                "load_s": t_load}
        if b16 is not None:
            line["batch16"] = b16
        if kernels:
            line["kernels"] = kernels
        if not args.no_cpu_baseline and world == 1:
            r = cpu_decode_rate(m, B, PROMPT, budget_s=12.0)
            line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample", "min", "max")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
