"""ctypes access to the C restatement (oracle/oracle.c): the checker's fast leg
and the timed CPU baseline.  TEST INFRASTRUCTURE ONLY — the product never
imports this module."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(_HERE, "_build", "liboracle.so")


def build(force=False):
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE] + (["-B"] if force else []), check=True, capture_output=True)
    return LIB


_lib = None
_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class Cfg(C.Structure):
    _fields_ = [("layers", _i32), ("d", _i32), ("ffn", _i32), ("heads", _i32), ("kv_heads", _i32), ("hd", _i32),
                ("vocab", _i32), ("eps", _f32), ("rope_base", _f32)]


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        _lib = C.CDLL(LIB)
        _lib.orc_threads.restype = _i32
        _lib.orc_decoder_new.restype = _vp
        _lib.orc_decoder_new.argtypes = [C.POINTER(Cfg), _i64]
        _lib.orc_decoder_pool.restype = _vp
        _lib.orc_decoder_pool.argtypes = [_vp]
        for name, args in {
            "orc_pack_q4": [_vp, _vp, _i64, _i64, _vp],
            "orc_gemm_q4": [_vp, _vp, _i64, _i64, _i64, _vp],
            "orc_gemm_bf16": [_vp, _vp, _i64, _i64, _i64, _vp],
            "orc_rmsnorm": [_vp, _vp, _i64, _i64, _f32, _vp],
            "orc_rope": [_vp, _vp, _i64, _i64, _i64, _f32],
            "orc_swiglu": [_vp, _vp, _i64, _vp],
            "orc_attn_decode": [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _f32, _vp],
            "orc_decoder_set_matrix": [_vp, _i32, _i32, _vp],
            "orc_decoder_set_norm": [_vp, _i32, _i32, _vp],
            "orc_decoder_set_head": [_vp, _vp, _vp, _vp],
            "orc_decoder_free": [_vp],
            "orc_decoder_step": [_vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp],
        }.items():
            getattr(_lib, name).argtypes = args
            getattr(_lib, name).restype = None
    return _lib


def _p(a):
    return a.ctypes.data_as(_vp)


def threads():
    return lib().orc_threads()


def pack_q4(q, s):
    q = np.ascontiguousarray(q, np.uint8)
    s = np.ascontiguousarray(s, np.float16)
    n, k = q.shape
    out = np.empty(n * (k // 32) * 18, np.uint8)
    lib().orc_pack_q4(_p(q), _p(s), n, k, _p(out))
    return out


def gemm_q4(x, blocks, n, k):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty((x.shape[0], n), np.float32)
    lib().orc_gemm_q4(_p(x), _p(blocks), x.shape[0], n, k, _p(y))
    return y


def gemm_bf16(x, w_bits):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w_bits, np.uint16)
    y = np.empty((x.shape[0], w.shape[0]), np.float32)
    lib().orc_gemm_bf16(_p(x), _p(w), x.shape[0], w.shape[0], w.shape[1], _p(y))
    return y


def rmsnorm(x, gamma, eps):
    x = np.ascontiguousarray(x, np.float32)
    g = np.ascontiguousarray(gamma, np.float32)
    y = np.empty_like(x)
    lib().orc_rmsnorm(_p(x), _p(g), x.shape[0], x.shape[1], eps, _p(y))
    return y


def rope(x, pos, base):
    x = np.array(x, np.float32, order="C")
    p = np.ascontiguousarray(pos, np.int32)
    m, h, hd = x.shape
    lib().orc_rope(_p(x), _p(p), m, h, hd, base)
    return x


def swiglu(g, u):
    g = np.ascontiguousarray(g, np.float32)
    u = np.ascontiguousarray(u, np.float32)
    y = np.empty_like(g)
    lib().orc_swiglu(_p(g), _p(u), g.size, _p(y))
    return y


def attn_decode(q16, pool16, table, lens, scale=None):
    q = np.ascontiguousarray(q16, np.float16)
    pool = np.ascontiguousarray(pool16, np.float16)
    table = np.ascontiguousarray(table, np.int32)
    lens = np.ascontiguousarray(lens, np.int32)
    b, hq, hd = q.shape
    hkv, page = pool.shape[1], pool.shape[3]
    out = np.empty((b, hq, hd), np.float32)
    scale = float(hd) ** -0.5 if scale is None else scale
    lib().orc_attn_decode(_p(q), _p(pool), _p(table), _p(lens), b, hq, hkv, hd, page, table.shape[1], scale, _p(out))
    return out


class CpuDecoder:
    """The CPU decode loop over 18-byte blocks (timed baseline)."""

    def __init__(self, cfg, W, pages_per_layer):
        self.cfg = cfg
        self.c = Cfg(cfg.layers, cfg.d, cfg.ffn, cfg.heads, cfg.kv_heads, cfg.hd, cfg.vocab, cfg.eps, cfg.rope_base)
        self.h = lib().orc_decoder_new(C.byref(self.c), pages_per_layer)
        self.keep = []
        names = ["wq", "wk", "wv", "wo", "wgate", "wup", "wdown"]
        for l, lw in enumerate(W["layers"]):
            for i, nm in enumerate(names):
                blk = pack_q4(*lw[nm])
                self.keep.append(blk)
                lib().orc_decoder_set_matrix(self.h, l, i, _p(blk))
            for i, nm in enumerate(["norm1", "norm2"]):
                g = np.ascontiguousarray(lw[nm], np.float32)
                self.keep.append(g)
                lib().orc_decoder_set_norm(self.h, l, i, _p(g))
        bits = lambda x: (np.ascontiguousarray(x, np.float32).view(np.uint32) >> 16).astype(np.uint16)
        self.emb, self.lm = bits(W["emb"]), bits(W["lm_head"])
        self.fn = np.ascontiguousarray(W["final_norm"], np.float32)
        lib().orc_decoder_set_head(self.h, _p(self.emb), _p(self.lm), _p(self.fn))
        self.pages_per_layer = pages_per_layer

    def pool(self):
        n = self.cfg.layers * self.pages_per_layer * self.cfg.kv_heads * 2 * 16 * self.cfg.hd
        ptr = lib().orc_decoder_pool(self.h)
        return np.ctypeslib.as_array((C.c_uint16 * n).from_address(ptr)).view(np.float16)

    def step(self, tokens, pos, table):
        tokens = np.ascontiguousarray(tokens, np.int32)
        pos = np.ascontiguousarray(pos, np.int32)
        table = np.ascontiguousarray(table, np.int32)
        b = tokens.size
        logits = np.empty((b, self.cfg.vocab), np.float32)
        nxt = np.empty(b, np.int32)
        lib().orc_decoder_step(self.h, _p(tokens), _p(pos), _p(table), table.shape[1], b, _p(logits), _p(nxt))
        return logits, nxt

    def close(self):
        if self.h:
            lib().orc_decoder_free(self.h)
            self.h = None
