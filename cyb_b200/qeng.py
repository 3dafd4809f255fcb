"""ctypes binding of libqeng (include/qeng.h) — the same entry points a Rust
host would bind with ``extern "C"``.  PyTorch is used only to own device memory
and streams; every computation goes through the C ABI into the CUDA library.

There is no CPU fallback: if the library is missing, importing this module
raises; if no B200 is visible, ``Context()`` raises.
"""
from __future__ import annotations

import ctypes as C
import os
import re

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("QENG_LIB") or os.path.join(_HERE, "_lib", "libqeng.so")
HEADER_PATH = os.path.join(_HERE, "..", "include", "qeng.h")

F32, F16, BF16 = 0, 1, 2
GEMM_ACCUMULATE, GEMM_FAST_F16 = 1, 2
W_Q, W_K, W_V, W_O, W_GATE, W_UP, W_DOWN = range(7)

ERRORS = {0: "OK", -1: "ERR_ARG", -2: "ERR_SHAPE", -3: "ERR_ALIGN", -4: "ERR_CUDA", -5: "ERR_NCCL",
          -6: "ERR_TIMEOUT", -7: "ERR_DEVICE_STATUS", -8: "ERR_STATE"}


class QengError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("qeng %s (%d): %s" % (ERRORS.get(code, "?"), code, msg))
        self.code = code


def declared_symbols(header=HEADER_PATH):
    """Names of all functions include/qeng.h declares."""
    text = open(header).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qeng_[a-z0-9_]+)\s*\(", text)))


def load_library(path=LIB_PATH):
    if not os.path.exists(path):
        raise ImportError("libqeng.so is not built (%s): run `python -m cyb_b200.build`; there is no CPU fallback" % path)
    return C.CDLL(path)


_lib = load_library()

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class Options(C.Structure):
    """qeng_options: tuning switches fixed when a context is created (0 keeps the default)."""
    _fields_ = [("struct_size", C.c_int32), ("no_pdl", C.c_int32), ("no_l2_prefetch", C.c_int32),
                ("no_p2p_allreduce", C.c_int32), ("no_attn_cluster", C.c_int32), ("attn_ctas_per_sm", C.c_int32),
                ("stream_groups", C.c_int32), ("step_kernel", C.c_int32), ("stream_stage_chunks", C.c_int32)]


class ModelCfg(C.Structure):
    _fields_ = [("layers", _i32), ("d_model", _i32), ("ffn", _i32), ("heads", _i32), ("kv_heads", _i32),
                ("head_dim", _i32), ("vocab", _i32), ("rms_eps", _f32), ("rope_base", _f32),
                ("max_batch", _i32), ("max_seq", _i32), ("tp_rank", _i32), ("tp_world", _i32),
                ("attn_softcap", _f32), ("sliding_window", _i32), ("final_softcap", _f32)]


def _sig(name, res, *args):
    f = getattr(_lib, name)
    f.restype = res
    f.argtypes = list(args)
    return f


_sig("qeng_version", _i32)
_sig("qeng_create", _i32, _i32, C.POINTER(_vp))
_sig("qeng_create_opts", _i32, _i32, C.POINTER(Options), C.POINTER(_vp))
_sig("qeng_destroy", _i32, _vp)
_sig("qeng_last_error", C.c_char_p, _vp)
_sig("qeng_device_status", _i32, _vp)
_sig("qeng_sm_count", _i32, _vp)
_sig("qeng_tp_unique_id", _i32, _vp)
_sig("qeng_tp_init", _i32, _vp, _i32, _i32, _vp)
_sig("qeng_tp_p2p_handle", _i32, _vp, _vp)
_sig("qeng_tp_p2p_open", _i32, _vp, _vp)
_sig("qeng_tp_p2p_reset", _i32, _vp)
_sig("qeng_tp_all_reduce_add_f32", _i32, _vp, _vp, _vp, _i64, _vp)
_sig("qeng_tp_all_reduce_f32", _i32, _vp, _vp, _i64, _vp)
_sig("qeng_weight_pack_q4", _i32, _vp, _vp, _vp, _i64, _i64, C.POINTER(_vp))
_sig("qeng_weight_unpack_q4", _i32, _vp, _vp, _vp, _vp)
_sig("qeng_weight_dequant_f32", _i32, _vp, _vp, _vp, _vp)
_sig("qeng_weight_quantize_q4", _i32, _vp, _vp, _i32, _i64, _i64, _i64, C.POINTER(_vp), _vp)
_sig("qeng_weight_pack_q4k", _i32, _vp, _vp, _i64, _i64, C.POINTER(_vp))
_sig("qeng_weight_unpack_k4", _i32, _vp, _vp, _vp, _vp)
_sig("qeng_weight_pack_q8", _i32, _vp, _vp, _vp, _i64, _i64, C.POINTER(_vp))
_sig("qeng_weight_unpack_q8", _i32, _vp, _vp, _vp, _vp)
_sig("qeng_weight_quantize_q8", _i32, _vp, _vp, _i32, _i64, _i64, _i64, C.POINTER(_vp), _vp)
_sig("qeng_weight_free", _i32, _vp, _vp)
_sig("qeng_weight_set_next", _i32, _vp, _vp, _vp)
_sig("qeng_weight_rows", _i64, _vp)
_sig("qeng_weight_cols", _i64, _vp)
_sig("qeng_weight_device_bytes", _i64, _vp)
_sig("qeng_weight_format", _i32, _vp)
_sig("qeng_gemm_q4", _i32, _vp, _vp, _vp, _i32, _i64, _i64, _vp, _i64, _i32, _vp)
_sig("qeng_gemv_q4", _i32, _vp, _vp, _vp, _vp, _vp)
_sig("qeng_rmsnorm", _i32, _vp, _vp, _vp, _i64, _i64, _f32, _vp, _vp)
_sig("qeng_rope", _i32, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _vp)
_sig("qeng_swiglu", _i32, _vp, _vp, _vp, _i64, _vp, _vp)
_sig("qeng_add", _i32, _vp, _vp, _vp, _i64, _vp, _vp)
_sig("qeng_embed", _i32, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp)
_sig("qeng_lm_head", _i32, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp)
_sig("qeng_argmax", _i32, _vp, _vp, _i64, _i64, _vp, _vp)
_sig("qeng_kv_pool_create", _i32, _vp, _i64, _i64, _i64, C.POINTER(_vp))
_sig("qeng_kv_pool_free", _i32, _vp, _vp)
_sig("qeng_kv_pool_data", _vp, _vp)
_sig("qeng_kv_pool_pages", _i64, _vp)
_sig("qeng_kv_append", _i32, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _vp)
_sig("qeng_attn_decode", _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _f32, _vp, _vp)
_sig("qeng_attn_decode_ex", _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _f32, _f32, _i32, _vp, _vp)
_sig("qeng_attn_decode_noalloc", _i32, _vp, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _f32, _vp, _vp)
_sig("qeng_decoder_create", _i32, _vp, C.POINTER(ModelCfg), C.POINTER(_vp))
_sig("qeng_decoder_free", _i32, _vp, _vp)
_sig("qeng_decoder_load_matrix", _i32, _vp, _vp, _i32, _i32, _vp, _vp, _i64, _i64)
_sig("qeng_decoder_load_matrix_q8", _i32, _vp, _vp, _i32, _i32, _vp, _vp, _i64, _i64)
_sig("qeng_decoder_load_matrix_q4k", _i32, _vp, _vp, _i32, _i32, _vp, _i64, _i64)
_sig("qeng_decoder_load_norm", _i32, _vp, _vp, _i32, _i32, _vp)
_sig("qeng_decoder_load_head", _i32, _vp, _vp, _vp, _vp, _vp)
_sig("qeng_decoder_reset", _i32, _vp, _vp, _i32)
_sig("qeng_decoder_prefill", _i32, _vp, _vp, _vp, _i32, _i32)
_sig("qeng_decoder_decode", _i32, _vp, _vp, _i32, _vp)
_sig("qeng_decoder_logits", _i32, _vp, _vp, _vp)
_sig("qeng_decoder_layer", _i32, _vp, _vp, _i32, _vp, _vp, _i32, _vp, _vp)
_sig("qeng_decoder_set_stream", _i32, _vp, _vp, _vp)
_sig("qeng_decoder_weight", _i32, _vp, _vp, _i32, _i32, C.POINTER(_vp))
_sig("qeng_decoder_launches_per_step", _i32, _vp)
_sig("qeng_decoder_config", _i32, _vp, _vp, C.POINTER(ModelCfg))
_sig("qeng_model_file_config", _i32, _vp, C.c_char_p, C.POINTER(ModelCfg), C.POINTER(_i64))
_sig("qeng_decoder_load_file", _i32, _vp, _vp, C.c_char_p)
_sig("qeng_decoder_step_profile", _i32, _vp, _vp, _vp, _i32, C.POINTER(_i32))


def _np_ptr(a):
    return a.ctypes.data_as(_vp)


def _dev_ptr(t):
    return _vp(t.data_ptr())


def _cur_stream():
    import torch
    return _vp(torch.cuda.current_stream().cuda_stream)


class Context:
    """One engine context on one CUDA device."""

    def __init__(self, device=0, **options):
        """`options`: fields of qeng_options (no_pdl, no_l2_prefetch, no_p2p_allreduce, no_attn_cluster,
        attn_ctas_per_sm, stream_groups, step_kernel, stream_stage_chunks)."""
        h = _vp()
        if options:
            o = Options(struct_size=C.sizeof(Options), **{k: int(v) for k, v in options.items()})
            rc = _lib.qeng_create_opts(device, C.byref(o), C.byref(h))
        else:
            rc = _lib.qeng_create(device, C.byref(h))
        if rc != 0:
            raise QengError(rc, "qeng_create failed (no B200 visible, or device index out of range)")
        self.h = h
        self.device = device

    def close(self):
        if self.h:
            _lib.qeng_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc):
        if rc != 0:
            raise QengError(rc, _lib.qeng_last_error(self.h).decode())

    @property
    def sm_count(self):
        return _lib.qeng_sm_count(self.h)

    # ---- tensor parallelism ---------------------------------------------------
    def tp_init(self, rank, world, exchange, allgather=None):
        """Collective.  `exchange(bytes_or_None) -> bytes` must broadcast rank 0's 128-byte id
        to every rank over any host channel (e.g. torch.distributed.broadcast_object_list).
        `allgather(bytes) -> [bytes per rank]`, if given, also maps the peers' inboxes for the
        one-shot all-reduce of decode."""
        buf = (C.c_uint8 * 128)()
        if rank == 0:
            rc = _lib.qeng_tp_unique_id(buf)
            if rc != 0:
                raise QengError(rc, "qeng_tp_unique_id failed (libnccl.so.2 not loadable?)")
        ident = exchange(bytes(buf) if rank == 0 else None)
        arr = (C.c_uint8 * 128).from_buffer_copy(ident)
        self.check(_lib.qeng_tp_init(self.h, rank, world, arr))
        if allgather is not None and 2 <= world <= 8:
            hb = (C.c_uint8 * 64)()
            self.check(_lib.qeng_tp_p2p_handle(self.h, hb))
            parts = allgather(bytes(hb))
            allb = (C.c_uint8 * (64 * world)).from_buffer_copy(b"".join(parts))
            self.check(_lib.qeng_tp_p2p_open(self.h, allb))

    def tp_p2p_reset(self):
        """After a failed collective: clear this rank's inbox, call counter and status (all ranks, then a host barrier)."""
        self.check(_lib.qeng_tp_p2p_reset(self.h))

    def all_reduce_add_(self, dst, part):
        self.check(_lib.qeng_tp_all_reduce_add_f32(self.h, _dev_ptr(dst), _dev_ptr(part), part.numel(), _cur_stream()))
        return dst

    def all_reduce_(self, t):
        self.check(_lib.qeng_tp_all_reduce_f32(self.h, _dev_ptr(t), t.numel(), _cur_stream()))
        return t

    def device_status(self):
        self.check(_lib.qeng_device_status(self.h))

    # ---- weights ----------------------------------------------------------
    def pack_q4(self, q, s):
        """q uint8 [N,K] codes 0..15, s float16 [N,K/32] (host numpy)."""
        q = np.ascontiguousarray(q, dtype=np.uint8)
        s = np.ascontiguousarray(s, dtype=np.float16)
        n, k = q.shape
        if s.shape != (n, k // 32):
            raise QengError(-2, "scale shape %s does not match codes %s" % (s.shape, q.shape))
        h = _vp()
        self.check(_lib.qeng_weight_pack_q4(self.h, _np_ptr(q), _np_ptr(s), n, k, C.byref(h)))
        return Weight(self, h)

    def pack_q4k(self, blocks, n, k):
        """blocks: uint8 array of n * k / 256 Q4_K super-blocks of 144 bytes (row-major)."""
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        if blocks.size != n * (k // 256) * 144:
            raise QengError(-2, "Q4_K data of %d bytes does not match [%d, %d]" % (blocks.size, n, k))
        h = _vp()
        self.check(_lib.qeng_weight_pack_q4k(self.h, _np_ptr(blocks), n, k, C.byref(h)))
        return Weight(self, h)

    def pack_q8(self, q, s):
        """q int8 [N,K] signed bytes, s float16 [N,K/32] (host numpy): w = q * s."""
        q = np.ascontiguousarray(q, dtype=np.int8)
        s = np.ascontiguousarray(s, dtype=np.float16)
        n, k = q.shape
        if s.shape != (n, k // 32):
            raise QengError(-2, "scale shape %s does not match bytes %s" % (s.shape, q.shape))
        h = _vp()
        self.check(_lib.qeng_weight_pack_q8(self.h, _np_ptr(q), _np_ptr(s), n, k, C.byref(h)))
        return Weight(self, h, q8=True)

    def quantize_q8(self, w):
        """Quantise a CUDA matrix [N,K] (float32 / float16 / bfloat16) into packed 8-bit blocks on the device."""
        import torch
        dt = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[w.dtype]
        assert w.is_cuda and w.dim() == 2 and w.stride(1) == 1
        h = _vp()
        self.check(_lib.qeng_weight_quantize_q8(self.h, _dev_ptr(w), dt, w.shape[0], w.shape[1], w.stride(0),
                                                C.byref(h), _cur_stream()))
        return Weight(self, h, q8=True)

    def quantize_q4(self, w):
        """Quantise a CUDA matrix [N,K] (float32 / float16 / bfloat16) into a packed weight on the device."""
        import torch
        dt = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[w.dtype]
        assert w.is_cuda and w.dim() == 2 and w.stride(1) == 1
        h = _vp()
        self.check(_lib.qeng_weight_quantize_q4(self.h, _dev_ptr(w), dt, w.shape[0], w.shape[1], w.stride(0),
                                                C.byref(h), _cur_stream()))
        return Weight(self, h)

    # ---- ops (torch CUDA tensors in, torch CUDA tensors out) ---------------
    def gemm_q4(self, w, x, out=None, flags=0):
        import torch
        dt = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16}[x.dtype]
        assert x.is_cuda and x.dim() == 2 and x.stride(1) == 1
        m = x.shape[0]
        if out is None:
            out = torch.empty((m, w.rows), dtype=torch.float32, device=x.device)
        self.check(_lib.qeng_gemm_q4(self.h, w.h, _dev_ptr(x), dt, m, x.stride(0), _dev_ptr(out), out.stride(0), flags,
                                     _cur_stream()))
        return out

    def gemv_q4(self, w, x, out=None):
        import torch
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        if out is None:
            out = torch.empty((w.rows,), dtype=torch.float32, device=x.device)
        self.check(_lib.qeng_gemv_q4(self.h, w.h, _dev_ptr(x), _dev_ptr(out), _cur_stream()))
        return out

    def rmsnorm(self, x, gamma, eps):
        import torch
        y = torch.empty_like(x)
        self.check(_lib.qeng_rmsnorm(self.h, _dev_ptr(x), _dev_ptr(gamma), x.shape[0], x.shape[1], eps, _dev_ptr(y),
                                     _cur_stream()))
        return y

    def rope_(self, x, pos, base):
        m, h, hd = x.shape
        self.check(_lib.qeng_rope(self.h, _dev_ptr(x), _dev_ptr(pos), m, h, hd, base, _cur_stream()))
        return x

    def swiglu(self, gate, up):
        import torch
        y = torch.empty_like(gate)
        self.check(_lib.qeng_swiglu(self.h, _dev_ptr(gate), _dev_ptr(up), gate.numel(), _dev_ptr(y), _cur_stream()))
        return y

    def add(self, a, b):
        import torch
        y = torch.empty_like(a)
        self.check(_lib.qeng_add(self.h, _dev_ptr(a), _dev_ptr(b), a.numel(), _dev_ptr(y), _cur_stream()))
        return y

    def embed(self, table_bf16, tokens):
        import torch
        v, d = table_bf16.shape
        x = torch.empty((tokens.numel(), d), dtype=torch.float32, device=tokens.device)
        self.check(_lib.qeng_embed(self.h, _dev_ptr(table_bf16), _dev_ptr(tokens), tokens.numel(), d, v, _dev_ptr(x),
                                   _cur_stream()))
        return x

    def lm_head(self, table_bf16, x, out=None):
        import torch
        v, d = table_bf16.shape
        if out is None:
            out = torch.empty((x.shape[0], v), dtype=torch.float32, device=x.device)
        self.check(_lib.qeng_lm_head(self.h, _dev_ptr(table_bf16), _dev_ptr(x), x.shape[0], d, v, _dev_ptr(out),
                                     _cur_stream()))
        return out

    def argmax(self, logits):
        import torch
        idx = torch.empty((logits.shape[0],), dtype=torch.int32, device=logits.device)
        self.check(_lib.qeng_argmax(self.h, _dev_ptr(logits), logits.shape[0], logits.shape[1], _dev_ptr(idx),
                                    _cur_stream()))
        return idx

    # ---- KV cache ----------------------------------------------------------
    def kv_pool(self, pages, kv_heads, hd=128):
        h = _vp()
        self.check(_lib.qeng_kv_pool_create(self.h, pages, kv_heads, hd, C.byref(h)))
        return KVPool(self, h, pages, kv_heads, hd)

    def kv_append(self, pool, k, v, table, pos):
        self.check(_lib.qeng_kv_append(self.h, pool.h, _dev_ptr(k), _dev_ptr(v), _dev_ptr(table), table.shape[1],
                                       _dev_ptr(pos), pos.numel(), _cur_stream()))

    def attn_decode(self, pool, q, table, lens, scale=None, out=None, softcap=0.0, window=0):
        import torch
        b, hq, hd = q.shape
        assert q.dtype == torch.float16 and q.is_contiguous()
        if out is None:
            out = torch.empty((b, hq, hd), dtype=torch.float32, device=q.device)
        scale = float(hd) ** -0.5 if scale is None else scale
        if softcap or window:
            self.check(_lib.qeng_attn_decode_ex(self.h, pool.h, _dev_ptr(q), _dev_ptr(table), table.shape[1], _dev_ptr(lens),
                                                b, hq, scale, float(softcap), int(window), _dev_ptr(out), _cur_stream()))
        else:
            self.check(_lib.qeng_attn_decode(self.h, pool.h, _dev_ptr(q), _dev_ptr(table), table.shape[1], _dev_ptr(lens),
                                             b, hq, scale, _dev_ptr(out), _cur_stream()))
        return out

    def attn_decode_noalloc(self, pool, q, table, lens, scale=None, out=None):
        """qeng_attn_decode_noalloc: the split scratch is the library's built-in array, nothing is
        allocated by the engine (pass `out` to keep the caller side allocation-free as well)."""
        import torch
        b, hq, hd = q.shape
        assert q.dtype == torch.float16 and q.is_contiguous()
        if out is None:
            out = torch.empty((b, hq, hd), dtype=torch.float32, device=q.device)
        scale = float(hd) ** -0.5 if scale is None else scale
        self.check(_lib.qeng_attn_decode_noalloc(self.h, pool.h, _dev_ptr(q), _dev_ptr(table), table.shape[1],
                                                 _dev_ptr(lens), b, hq, scale, _dev_ptr(out), _cur_stream()))
        return out

    def decoder(self, **kw):
        return Decoder(self, **kw)


class Weight:
    def __init__(self, ctx, h, q8=None):
        self.ctx, self.h = ctx, h
        self.fmt = _lib.qeng_weight_format(h)
        self.q8 = self.fmt == 8
        self.rows = _lib.qeng_weight_rows(h)
        self.cols = _lib.qeng_weight_cols(h)
        self.device_bytes = _lib.qeng_weight_device_bytes(h)

    def unpack(self):
        if self.fmt == 14:  # K-quant: codes and f32 (scale, minimum) pairs
            q = np.empty((self.rows, self.cols), np.uint8)
            dm = np.empty((self.rows, self.cols // 32, 2), np.float32)
            self.ctx.check(_lib.qeng_weight_unpack_k4(self.ctx.h, self.h, _np_ptr(q), _np_ptr(dm)))
            return q, dm
        q = np.empty((self.rows, self.cols), np.int8 if self.q8 else np.uint8)
        s = np.empty((self.rows, self.cols // 32), np.float16)
        fn = _lib.qeng_weight_unpack_q8 if self.q8 else _lib.qeng_weight_unpack_q4
        self.ctx.check(fn(self.ctx.h, self.h, _np_ptr(q), _np_ptr(s)))
        return q, s

    def dequant(self):
        import torch
        out = torch.empty((self.rows, self.cols), dtype=torch.float32, device="cuda:%d" % self.ctx.device)
        self.ctx.check(_lib.qeng_weight_dequant_f32(self.ctx.h, self.h, _dev_ptr(out), _cur_stream()))
        return out

    def set_next(self, nxt):
        """Hint that the matmul after one over this matrix is over `nxt` (None clears it)."""
        self._next = nxt  # keep it alive while the hint is set
        self.ctx.check(_lib.qeng_weight_set_next(self.ctx.h, self.h, nxt.h if nxt is not None else None))

    def free(self):
        if self.h:
            _lib.qeng_weight_free(self.ctx.h, self.h)
            self.h = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.free()
        except Exception:
            pass


class KVPool:
    def __init__(self, ctx, h, pages, kv_heads, hd):
        self.ctx, self.h, self.pages, self.kv_heads, self.hd = ctx, h, pages, kv_heads, hd

    def tensor(self):
        """The pool's storage as a torch f16 view [pages, kv_heads, 2, 16, hd]."""
        import torch
        n = self.pages * self.kv_heads * 2 * 16 * self.hd
        ptr = _lib.qeng_kv_pool_data(self.h)
        iface = {"shape": (n,), "typestr": "<f2", "data": (ptr, False), "version": 2}

        class _Holder:
            __cuda_array_interface__ = iface
        return torch.as_tensor(_Holder(), device="cuda:%d" % self.ctx.device).view(self.pages, self.kv_heads, 2, 16, self.hd)

    def free(self):
        if self.h:
            _lib.qeng_kv_pool_free(self.ctx.h, self.h)
            self.h = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.free()
        except Exception:
            pass


class Decoder:
    """The layer executor behind the C ABI (qeng_decoder_*)."""

    def __init__(self, ctx, layers, d_model, ffn, heads, kv_heads, vocab, head_dim=128, rms_eps=1e-5,
                 rope_base=10000.0, max_batch=1, max_seq=1024, tp_rank=0, tp_world=1, attn_softcap=0.0, sliding_window=0,
                 final_softcap=0.0):
        self.ctx = ctx
        self.cfg = ModelCfg(layers, d_model, ffn, heads, kv_heads, head_dim, vocab, rms_eps, rope_base, max_batch,
                            max_seq, tp_rank, tp_world, attn_softcap, sliding_window, final_softcap)
        h = _vp()
        ctx.check(_lib.qeng_decoder_create(ctx.h, C.byref(self.cfg), C.byref(h)))
        self.h = h
        self.batch = 0

    def load_matrix_q4k(self, layer, which, blocks, n, k):
        """blocks: the matrix as Q4_K super-blocks (uint8, n * k / 256 * 144 bytes)."""
        blocks = np.ascontiguousarray(blocks, dtype=np.uint8).reshape(-1)
        self.ctx.check(_lib.qeng_decoder_load_matrix_q4k(self.ctx.h, self.h, layer, which, _np_ptr(blocks), n, k))

    def load_matrix(self, layer, which, q, s):
        """q uint8 codes 0..15 (4-bit blocks) or int8 bytes (8-bit blocks), s float16 scales."""
        q8 = np.asarray(q).dtype == np.int8
        q = np.ascontiguousarray(q, dtype=np.int8 if q8 else np.uint8)
        s = np.ascontiguousarray(s, dtype=np.float16)
        fn = _lib.qeng_decoder_load_matrix_q8 if q8 else _lib.qeng_decoder_load_matrix
        self.ctx.check(fn(self.ctx.h, self.h, layer, which, _np_ptr(q), _np_ptr(s), q.shape[0], q.shape[1]))

    def load_file(self, path):
        """Load all weights from a `.model` container (qeng_decoder_load_file)."""
        self.ctx.check(_lib.qeng_decoder_load_file(self.ctx.h, self.h, str(path).encode()))

    def load_norm(self, layer, which, gamma):
        g = np.ascontiguousarray(gamma, dtype=np.float32)
        self.ctx.check(_lib.qeng_decoder_load_norm(self.ctx.h, self.h, layer, which, _np_ptr(g)))

    def load_head(self, emb_bits, lm_bits, final_gamma):
        e = np.ascontiguousarray(emb_bits, dtype=np.uint16)
        l = np.ascontiguousarray(lm_bits, dtype=np.uint16)
        g = np.ascontiguousarray(final_gamma, dtype=np.float32)
        self.ctx.check(_lib.qeng_decoder_load_head(self.ctx.h, self.h, _np_ptr(e), _np_ptr(l), _np_ptr(g)))

    def reset(self, batch):
        self.ctx.check(_lib.qeng_decoder_reset(self.ctx.h, self.h, batch))
        self.batch = batch

    def prefill(self, tokens):
        t = np.ascontiguousarray(tokens, dtype=np.int32)
        self.ctx.check(_lib.qeng_decoder_prefill(self.ctx.h, self.h, _np_ptr(t), t.shape[0], t.shape[1]))

    def decode(self, steps):
        out = np.empty((self.batch, steps), np.int32)
        self.ctx.check(_lib.qeng_decoder_decode(self.ctx.h, self.h, steps, _np_ptr(out)))
        return out

    def logits(self):
        out = np.empty((self.batch, self.cfg.vocab), np.float32)
        self.ctx.check(_lib.qeng_decoder_logits(self.ctx.h, self.h, _np_ptr(out)))
        return out

    def layer(self, layer, x, pos):
        import torch
        out = torch.empty_like(x)
        p = np.ascontiguousarray(pos, dtype=np.int32)
        self.ctx.check(_lib.qeng_decoder_layer(self.ctx.h, self.h, layer, _dev_ptr(x), _np_ptr(p), x.shape[0],
                                               _dev_ptr(out), _cur_stream()))
        return out

    def weight(self, layer, fused_index):
        """Borrowed handle of a fused layer weight (0 qkv, 1 o, 2 gate/up, 3 down)."""
        h = _vp()
        self.ctx.check(_lib.qeng_decoder_weight(self.ctx.h, self.h, layer, fused_index, C.byref(h)))
        w = Weight.__new__(Weight)
        w.ctx, w.h = self.ctx, h
        w.rows, w.cols = _lib.qeng_weight_rows(h), _lib.qeng_weight_cols(h)
        w.device_bytes = _lib.qeng_weight_device_bytes(h)
        w.fmt = _lib.qeng_weight_format(h)
        w.q8 = w.fmt == 8
        w.free = lambda: None  # borrowed
        return w

    def use_current_stream(self):
        self.ctx.check(_lib.qeng_decoder_set_stream(self.ctx.h, self.h, _cur_stream()))

    def step_profile(self):
        """Phase timestamps (ns) of the last fused decode step: array [2 CTAs, layers, 16]."""
        out = np.zeros(2 * self.cfg.layers * 16, np.uint64)
        n = _i32(0)
        self.ctx.check(_lib.qeng_decoder_step_profile(self.ctx.h, self.h, _np_ptr(out), out.size, C.byref(n)))
        return out[:n.value].reshape(2, self.cfg.layers, 16)

    @property
    def launches_per_step(self):
        return _lib.qeng_decoder_launches_per_step(self.h)

    def free(self):
        if self.h:
            _lib.qeng_decoder_free(self.ctx.h, self.h)
            self.h = None

    def __del__(self):
        try:
            if self.ctx.h:
                self.free()
        except Exception:
            pass


def model_file_config(path, ctx=None):
    """(ModelCfg, number of tensors) of a `.model` container; raises QengError on a malformed file."""
    cfg = ModelCfg()
    n = _i64(0)
    rc = _lib.qeng_model_file_config(ctx.h if ctx is not None else None, str(path).encode(), C.byref(cfg), C.byref(n))
    if rc != 0:
        raise QengError(rc, _lib.qeng_last_error(ctx.h).decode() if ctx is not None else "malformed model file")
    return cfg, n.value


def load_decoder_weights(dec, W, cfg):
    """Feed a weight dict into a Decoder: W["layers"][l][name] = (codes, scales)
    for name in wq wk wv wo wgate wup wdown, norm1/norm2 gains, and bf16-valued
    f32 tables W["emb"], W["lm_head"], gain W["final_norm"]."""
    names = ["wq", "wk", "wv", "wo", "wgate", "wup", "wdown"]
    for l, lw in enumerate(W["layers"]):
        for i, nm in enumerate(names):
            if nm + "_q4k" in lw:  # the matrix as Q4_K super-blocks (lw[nm] then holds its expansion)
                dec.load_matrix_q4k(l, i, lw[nm + "_q4k"], *lw[nm][0].shape)
            else:
                dec.load_matrix(l, i, *lw[nm])
        dec.load_norm(l, 0, lw["norm1"])
        dec.load_norm(l, 1, lw["norm2"])
        if "qnorm" in lw:  # optional per-head gains of q and k
            dec.load_norm(l, 2, lw["qnorm"])
            dec.load_norm(l, 3, lw["knorm"])

    def bits(x):
        return (np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) >> 16).astype(np.uint16)
    dec.load_head(bits(W["emb"]), bits(W["lm_head"]), W["final_norm"])
