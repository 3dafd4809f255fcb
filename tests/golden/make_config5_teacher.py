"""Writes tests/golden/config5_teacher.npz: the float64 teacher's free-running greedy decode of
the benchmark's own model (configs[4]: 32 layers, d 4096, FFN 11008, 32/8 heads, vocab 32000,
the seeded weights, tables and 512-token prompt of bench.py) — the tokens of the first steps
and, per step, the teacher's best logits (indices and values) and the largest |logit|.

    python tests/golden/make_config5_teacher.py [--steps 32]

Takes about half an hour of CPU time and ~10 GB of memory.  The prompt (512 rows, the
tensor-core path on the device) is computed with activations and dequantised weights rounded
to bf16, as the device does from 256 rows on; the decode steps use unrounded matmuls.
"""
import argparse
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
import bench  # noqa: E402  (definitions only: the seeded generators of the benchmark)
from oracle import ref  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--layers", type=int, default=bench.MODEL["layers"])
    ap.add_argument("--out", default=os.path.join(HERE, "config5_teacher.npz"))
    args = ap.parse_args()
    m = dict(bench.MODEL)
    m["layers"] = args.layers
    cfg = ref.DecoderConfig(layers=m["layers"], d=m["d"], ffn=m["ffn"], heads=m["heads"], kv_heads=m["kv_heads"],
                            hd=m["hd"], vocab=m["vocab"])
    names = ["wq", "wk", "wv", "wo", "wgate", "wup", "wdown"]
    W = {"layers": [], "final_norm": np.ones(m["d"], np.float32)}
    for l in range(m["layers"]):
        lw = {"norm1": np.ones(m["d"], np.float32), "norm2": np.ones(m["d"], np.float32)}
        for j, (nm, n, k) in enumerate(bench.layer_shapes(m)):
            lw[names[j]] = bench.gen_matrix(1000 + 7 * l + j, n, k)
        W["layers"].append(lw)
    f32 = lambda bits: (bits.astype(np.uint32) << 16).view(np.float32)
    W["emb"], W["lm_head"] = f32(bench.gen_table(1, m["vocab"], m["d"])), f32(bench.gen_table(2, m["vocab"], m["d"]))
    prompt = np.random.Generator(np.random.PCG64(7)).integers(0, m["vocab"], (1, bench.PROMPT)).astype(np.int32)
    teacher = ref.Decoder(cfg, W, mm=lambda x, q, s: ref.gemm_q4_bf16w(ref.to_bf16(x), q, s))
    teacher.reset(1)
    t0 = time.time()
    logits = teacher.forward(prompt, np.arange(bench.PROMPT)[None])
    print("prompt done in %.0f s" % (time.time() - t0), flush=True)
    teacher.mm = ref.gemm_q4_fast
    toks, top_i, top_v, amax = [], [], [], []
    for s in range(args.steps):
        order = np.argsort(-logits[0])[:8]
        toks.append(int(order[0]))
        top_i.append(order.astype(np.int32))
        top_v.append(logits[0, order])
        amax.append(float(np.abs(logits[0]).max()))
        print("step %d token %d gap %.3g of %.3g (%.0f s)" % (s, order[0], logits[0, order[0]] - logits[0, order[1]],
                                                             amax[-1], time.time() - t0), flush=True)
        if s + 1 < args.steps:
            logits = teacher.forward(np.array([[order[0]]]), np.array([[bench.PROMPT + s]]))
        np.savez(args.out, tokens=np.array(toks, np.int32), top_idx=np.array(top_i), top_val=np.array(top_v),
                 absmax=np.array(amax), prompt_len=bench.PROMPT, layers=m["layers"])


if __name__ == "__main__":
    main()
