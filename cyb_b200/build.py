"""Build libqeng.so (CUDA, sm_100a only) in-tree with nvcc.

    python -m cyb_b200.build            # build if sources are newer than the library
    python -m cyb_b200.build --force

The library lands in cyb_b200/_lib/ so that it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "_lib")
LIB = os.path.join(OUT_DIR, "libqeng.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-O3", "-lineinfo", "-std=c++17", "--use_fast_math=false",
                     "-Xcompiler", "-fPIC,-fopenmp,-O3", "-Xptxas", "-v"]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _deps():
    inc = os.path.join(HERE, "..", "include", "qeng.h")
    return sources() + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".h")] + [inc]


def up_to_date():
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(p) <= t for p in _deps())


def build(force=False, verbose=False, extra_flags=(), out_dir=None):
    """Compile every .cu and link libqeng.so.  `extra_flags` (e.g. -D tuning macros) and
    `out_dir` build a variant beside the default library (load it with QENG_LIB=path)."""
    global_default = out_dir is None and not extra_flags
    if global_default and not force and up_to_date():
        return LIB
    OUT_DIR_ = out_dir or OUT_DIR
    LIB_ = os.path.join(OUT_DIR_, "libqeng.so")
    os.makedirs(OUT_DIR_, exist_ok=True)
    nvcc = _nvcc()
    flags = [f for f in NVCC_FLAGS if f != "--use_fast_math=false"] + list(extra_flags)

    def compile_one(src):
        obj = os.path.join(OUT_DIR_, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc] + flags + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed for %s:\n%s\n%s" % (src, r.stdout, r.stderr))
        return obj, r.stderr

    with ThreadPoolExecutor(max_workers=min(8, len(sources()))) as ex:
        results = list(ex.map(compile_one, sources()))
    log = "\n".join(err for _, err in results)
    with open(os.path.join(OUT_DIR_, "ptxas.log"), "w") as f:
        f.write(log)
    if verbose:
        print(log)
    objs = [o for o, _ in results]
    cmd = [nvcc] + ARCH + ["-shared", "-o", LIB_] + objs + ["-Xcompiler", "-fopenmp", "-lgomp"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n%s\n%s" % (r.stdout, r.stderr))
    return LIB_


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
