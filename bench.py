#!/usr/bin/env python
"""Headline benchmark: greedy decode tokens/s of a 7B-shaped 4-bit Llama-style
decoder (32 layers, d 4096, FFN 11008, 32/8 heads, vocab 32000) on N B200s,
and the HBM roofline of its dominant kernel, the 4-bit decode GEMV.

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

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL = dict(layers=32, d=4096, ffn=11008, heads=32, kv_heads=8, hd=128, vocab=32000)
PROMPT = 512
METRIC = "decode tokens/s (7B 4-bit, 1/2/4/8 B200); quant GEMV HBM GB/s vs peak"
# (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes of one launch of the decode
# matmul, from the ncu capture summarised in profiles/gemv_q4_stream_22016x4096_m1.md
# (50.80 MB read + 9.5 KB written against 50.83 MB algorithmic); traffic grows with N*K.
NCU_TRAFFIC_PER_ALGO_BYTE = 0.9996


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=MODEL["layers"], help="for quick checks only; the bench config is 32")
    ap.add_argument("--no-cpu-baseline", action="store_true")
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
# clocks
# --------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 9 and r[5 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# --------------------------------------------------------------------------
# CPU baseline (the oracle's C port on the host cores) — rank 0 only
# --------------------------------------------------------------------------
def cpu_decode_rate(m, batch, ctx_len, budget_s, steps=None):
    """Times CPU decode steps on a bounded sample: `sample_layers` of the model's
    layers (per-layer cost is identical; the LM head is timed in full) with a
    synthetic KV cache of ctx_len tokens.  Returns (tokens/s extrapolated to
    the full depth, cores, description, seconds per full step)."""
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
    # time layers and head separately: t_layers from the 2-layer model minus head, head from a direct call
    x = rng.standard_normal((batch, m["d"]), dtype=np.float32)
    cport.gemm_bf16(x, dec.lm)  # warm (first touch of the table)
    th = []
    for _ in range(3):
        t0 = time.perf_counter()
        cport.gemm_bf16(x, dec.lm)
        th.append(time.perf_counter() - t0)
    t_head = statistics.median(th)
    dec.step(toks, np.full(batch, ctx_len, np.int32), table)  # warm
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
        elif time.perf_counter() - t_start > budget_s or n >= 64:
            break
    t_step = statistics.median(times)
    t_head = min(t_head, 0.9 * t_step)  # the slice's step contains the head: never extrapolate a negative layer time
    per_full = (t_step - t_head) / sample_layers * m["layers"] + t_head
    dec.close()
    desc = ("%d decode steps of a %d-layer slice (+ full LM head) at context %d, batch %d, extrapolated x%d/%d layers"
            % (n, sample_layers, ctx_len, batch, m["layers"], sample_layers))
    return batch / per_full, cores, desc, per_full


def run_reference(args):
    """The reference arm: the CPU restatement of the path (the reference's own
    runtime crates are absent from its checkout) on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m = dict(MODEL)
    total = args.warmup + args.steps
    t0 = time.perf_counter()
    rate, cores, desc, per_full = cpu_decode_rate(m, args.batch, PROMPT, budget_s=None, steps=max(total, 1))
    line = {"impl": "reference", "metric": METRIC, "value": rate, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_full * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "configs[4]: 32-layer d4096 ffn11008 32/8-head 4-bit decoder, greedy decode at context %d, batch %d" % (PROMPT, args.batch)},
            "cpu_baseline": {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc},
            "e2e": {"value": rate, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "wall_s": time.perf_counter() - t0}
    print(json.dumps(line))


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
    os.environ["OMP_NUM_THREADS"] = str(max(1, (os.cpu_count() or 1) // max(world, 1)))
    from cyb_b200 import qeng
    m = dict(MODEL)
    m["layers"] = args.layers
    B, K, Wm = args.batch, args.steps, max(args.warmup, 3)
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
                      vocab=m["vocab"], max_batch=B, max_seq=max_seq, tp_rank=rank, tp_world=world)
    t_load = time.perf_counter()
    for l in range(m["layers"]):
        for j, (nm, n, k) in enumerate(layer_shapes(m)):
            dec.load_matrix(l, j, *gen_matrix(1000 + 7 * l + j, n, k))
        dec.load_norm(l, 0, np.ones(m["d"], np.float32))
        dec.load_norm(l, 1, np.ones(m["d"], np.float32))
    dec.load_head(gen_table(1, m["vocab"], m["d"]), gen_table(2, m["vocab"], m["d"]), np.ones(m["d"], np.float32))
    t_load = time.perf_counter() - t_load

    prompt = np.random.Generator(np.random.PCG64(7)).integers(0, m["vocab"], (B, PROMPT)).astype(np.int32)
    dec.use_current_stream()
    dec.reset(B)
    dec.prefill(prompt)  # first call: buffers grow, kernels load
    dec.reset(B)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    dec.prefill(prompt)
    torch.cuda.synchronize()
    t_prefill = time.perf_counter() - t0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed decode: K steps replayed from the captured graph ------
    dec.decode(Wm)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        barrier()
        ev0.record()
        dec.decode(K)
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1)
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = B * K / (ms * 1e-3)
    launches = dec.launches_per_step * K
    ctx_mid = PROMPT + Wm + K // 2

    # ---- end to end: one call per token, every token read back to the host ---
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        dec.decode(1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e = B * K / float(t.item())

    # ---- roofline of the dominant kernel: the 4-bit GEMV over this decoder's own
    # weights (32 layers x 4 fused matrices = distinct buffers >> L2), timed with events
    roof = None
    if True:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        ws = [dec.weight(l, i) for l in range(m["layers"]) for i in range(4)]
        xs = {k: torch.randn(k, device="cuda") for k in {w.cols for w in ws}}
        ys = {w.rows: torch.empty(w.rows, device="cuda") for w in ws}
        algo = sum(w.rows * w.cols * 0.5625 + w.cols * 4 + w.rows * 4 for w in ws)
        # replayed from a CUDA graph so that the host launch rate does not bound the figure
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for w in ws:
                ctx.gemv_q4(w, xs[w.cols], out=ys[w.rows])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for w in ws:
                ctx.gemv_q4(w, xs[w.cols], out=ys[w.rows])
        for _ in range(3):
            graph.replay()
        reps = 10
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(reps):
            graph.replay()
        ev1.record()
        torch.cuda.synchronize()
        per_launch_s = ev0.elapsed_time(ev1) * 1e-3 / (reps * len(ws))
        achieved = algo / len(ws) / per_launch_s / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "traffic": (NCU_TRAFFIC_PER_ALGO_BYTE * algo / len(ws)) if NCU_TRAFFIC_PER_ALGO_BYTE else None,
                "kernel": "gemv_q4_stream_kernel<NT=1,TG> (M=1, f32 activations)", "bytes_per_launch": algo / len(ws),
                "us_per_launch": per_launch_s * 1e6,
                "peak_source": "measured (MEASURED_PEAKS.json hbm_gbs)" if "hbm_gbs" in peaks else "fallback",
                "step_frac": algo_bytes_per_step(m, B, ctx_mid, world) / (ms * 1e-3 / K) / 1e9 / peak}
    ctx.device_status()

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": Wm,
                "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32 accumulate over 4-bit weights (f16 tensor-core operands, exact split activations)",
                "data": "synthetic",
                "config": {"workload": "configs[4]: 32-layer d4096 ffn11008 32/8-head vocab-32000 4-bit decoder, prompt %d then greedy decode, batch %d" % (PROMPT, B),
                           "layers": m["layers"], "batch": B, "context_at_start": PROMPT + Wm, "parallelism": "tp%d" % world,
                           "l2_policy": "inputs larger than L2 (3.4 GB of weights streamed per step)"},
                "clocks": clk.summary(), "gpu_launches": launches,
                "e2e": {"value": e2e, "unit": "tokens/s", "h2d_bytes_per_step": 8 * B, "d2h_bytes_per_step": 4 * B + 4,
                        "how": "one qeng_decoder_decode(1) call per token, sampled token copied to the host every step"},
                "roofline": roof, "prefill_s": t_prefill, "prefill_tokens_per_s": B * PROMPT / t_prefill,
                "load_s": t_load}
        if not args.no_cpu_baseline and world == 1:
            rate, cores, desc, _ = cpu_decode_rate(m, B, PROMPT, budget_s=15.0)
            line["cpu_baseline"] = {"value": rate, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line))
    dec.free()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
