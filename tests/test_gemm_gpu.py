"""Parity of the CUDA quantized matmul (through the C ABI) with the oracle.
Gate: unpacked codes/scales bit-exact; outputs max|y-ref|/max|ref| <= 2e-3
(f64 oracle)."""
import os

import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
TOL = 2e-3
# What the decode kernels actually reach, asserted beside the gate: activations are quantised to
# 15 bits relative to the largest magnitude of their 32-block (two signed bytes per value for the
# integer tensor-core contraction); everything after that is exact up to f32 accumulation.
# Measured 2e-5 .. 6e-5 of max|y| on Gaussian activations.
TIGHT = 2e-4
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def _t(a, dtype=None):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


@pytest.mark.parametrize("n,k", [(16, 32), (16, 96), (48, 160), (256, 512), (4096, 4096), (1376, 4096), (4096, 1376)])
def test_pack_unpack_bit_exact(ctx, n, k):
    q, s = ref.make_q4(ref.rng_of(n * 7 + k), n, k)
    w = ctx.pack_q4(q, s)
    q2, s2 = w.unpack()
    assert np.array_equal(q, q2)
    assert np.array_equal(s.view(np.uint16), s2.view(np.uint16))
    assert np.array_equal(w.dequant().cpu().numpy(), ref.dequant(q, s, np.float32))
    w.free()


def test_pack_rejects_bad_input(ctx):
    from cyb_b200 import qeng
    q, s = ref.make_q4(ref.rng_of(1), 16, 64)
    bad = q.copy()
    bad[3, 5] = 16
    with pytest.raises(qeng.QengError) as e:
        ctx.pack_q4(bad, s)
    assert e.value.code == -1
    with pytest.raises(qeng.QengError) as e:
        ctx.pack_q4(q[:8], s[:8])  # N % 16 != 0
    assert e.value.code == -2


def test_config1_gemv(ctx):
    x, q, s = ref.config1(0)
    w = ctx.pack_q4(q, s)
    y = ctx.gemv_q4(w, _t(x[0])).cpu().numpy()
    yref = ref.gemm_q4_fast(x, q, s)[0]
    e = ref.err_inf(y, yref)
    assert e < TOL, e
    assert e < 2e-6, e   # a single activation row is carried in 22 bits: f32-accurate
    yf = ctx.gemm_q4(w, _t(x), flags=2).cpu().numpy()  # QENG_GEMM_FAST_F16: 15 bits
    assert ref.err_inf(yf, yref) < TIGHT
    w.free()


@pytest.mark.parametrize("name", ["gemv_64x96", "gemm_5x48x160", "gemm_16x32x64", "enum"])
def test_golden_vectors(ctx, name):
    g = GOLD
    w = ctx.pack_q4(g[name + "_q"], g[name + "_s"])
    y = ctx.gemm_q4(w, _t(g[name + "_x"])).cpu().numpy()
    assert ref.err_inf(y, g[name + "_y"]) < TIGHT
    w.free()


def test_known_answers(ctx):
    import torch
    # all codes 8 -> exactly zero: the zero point is removed in integer arithmetic
    q = np.full((16, 64), 8, np.uint8)
    s = np.full((16, 2), 0.01, np.float16)
    w = ctx.pack_q4(q, s)
    x = ref.rng_of(3).standard_normal((3, 64), dtype=np.float32)
    assert float(ctx.gemm_q4(w, _t(x)).abs().max()) == 0.0
    w.free()
    # one-hot activations select a column of dequant(W) exactly
    q, s = ref.make_q4(ref.rng_of(4), 32, 96)
    wd = ref.dequant(q, s, np.float32)
    w = ctx.pack_q4(q, s)
    for k in (0, 7, 31, 32, 95):
        x = np.zeros((1, 96), np.float32)
        x[0, k] = 1.0
        assert np.array_equal(ctx.gemm_q4(w, _t(x)).cpu().numpy()[0], wd[:, k])
    # identical rows give identical outputs whatever M is
    x1 = ref.rng_of(5).standard_normal((1, 96), dtype=np.float32)
    y1 = ctx.gemm_q4(w, _t(x1)).cpu().numpy()
    y8 = ctx.gemm_q4(w, _t(np.repeat(x1, 8, 0))).cpu().numpy()
    assert all(np.array_equal(y8[i], y8[0]) for i in range(8))  # bit-identical among themselves
    # one row is quantised to 22 bits, eight rows to 15 bits each: equal within the tighter of the two bounds
    assert ref.err_inf(y8[0], y1[0]) < TIGHT
    w.free()


@pytest.mark.parametrize("idx,m,n,k", [(i, m, n, k) for i, (n, k) in enumerate([(4096, 4096), (11008, 4096), (4096, 11008)])
                                       for m in (1, 8, 32)])
def test_config2_sweep(ctx, idx, m, n, k):
    import torch
    x, q, s = ref.config2(idx, m, n, k)
    w = ctx.pack_q4(q, s)
    xb = _t(x).to(torch.bfloat16)
    y = ctx.gemm_q4(w, xb).cpu().numpy()
    e = ref.err_inf(y, ref.gemm_q4_fast(x, q, s))
    assert e < TOL, e
    w.free()


@pytest.mark.parametrize("m", [1, 2, 3, 7, 16, 17, 40])
def test_ragged_m_f32_and_accumulate(ctx, m):
    from cyb_b200 import qeng
    rng = ref.rng_of(100 + m)
    x = rng.standard_normal((m, 160), dtype=np.float32)
    q, s = ref.make_q4(rng, 48, 160)
    w = ctx.pack_q4(q, s)
    yref = ref.gemm_q4(x, q, s)
    y = ctx.gemm_q4(w, _t(x))
    assert ref.err_inf(y.cpu().numpy(), yref) < TIGHT
    y2 = ctx.gemm_q4(w, _t(x), out=y.clone(), flags=qeng.GEMM_ACCUMULATE)
    assert ref.err_inf(y2.cpu().numpy(), 2 * yref) < TIGHT
    yf = ctx.gemm_q4(w, _t(x), flags=qeng.GEMM_FAST_F16)
    assert ref.err_inf(yf.cpu().numpy(), yref) < TOL
    yh = ctx.gemm_q4(w, _t(x).half())
    assert ref.err_inf(yh.cpu().numpy(), ref.gemm_q4(x.astype(np.float16).astype(np.float32), q, s)) < TIGHT
    w.free()


def test_linearity_at_full_size(ctx):
    """Size-independent property at a BASELINE shape: W(a x1 + b x2) = a W x1 + b W x2."""
    rng = ref.rng_of(9)
    q, s = ref.make_q4(rng, 11008, 4096)
    w = ctx.pack_q4(q, s)
    x1 = rng.standard_normal((1, 4096), dtype=np.float32)
    x2 = rng.standard_normal((1, 4096), dtype=np.float32)
    y1, y2 = ctx.gemm_q4(w, _t(x1)), ctx.gemm_q4(w, _t(x2))
    y3 = ctx.gemm_q4(w, _t(2 * x1 - 3 * x2))
    lin = (2 * y1 - 3 * y2)
    assert float((y3 - lin).abs().max() / lin.abs().max()) < 2 * TIGHT
    w.free()


@pytest.mark.parametrize("m,n,k", [(256, 128, 64), (300, 144, 96), (512, 1376, 4096), (512, 11008, 4096), (512, 4096, 11008)])
def test_prefill_tensor_core_path(ctx, m, n, k):
    """M >= 256 takes the tcgen05 kernel: activations and dequantised weights are rounded to bf16
    (tolerance 5e-3 against the unrounded oracle; ~1e-5 against the oracle with the same roundings)."""
    import torch
    rng = ref.rng_of(1000 + m + n + k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    q, s = ref.make_q4(rng, n, k)
    w = ctx.pack_q4(q, s)
    y = ctx.gemm_q4(w, _t(x)).cpu().numpy()
    ctx.device_status()
    xb = ref.to_bf16(x)
    same = ref.gemm_q4_bf16w(xb, q, s)
    assert ref.err_inf(y, same) < 2e-5, ref.err_inf(y, same)
    assert ref.err_inf(y, ref.gemm_q4_fast(x, q, s)) < 5e-3
    # bf16 activations go in directly; accumulate adds to what is there
    yb = ctx.gemm_q4(w, _t(xb).to(torch.bfloat16), out=_t(y.copy()), flags=1).cpu().numpy()
    assert ref.err_inf(yb, 2 * same) < 2e-5
    w.free()


def _sample_rows(m):
    """Rows that hit every position of a 256-row tile and both ends of the matrix."""
    r = np.concatenate([np.arange(0, m, 13), [0, 127, 128, 255, 256, 257, m - 258, m - 257, m - 129, m - 2, m - 1]])
    return np.unique(r[(r >= 0) & (r < m)])


@pytest.mark.parametrize("m,n,k", [(2048, 11008, 4096), (8192, 11008, 4096), (8192, 4096, 11008), (2049, 11024, 4096)])
def test_prefill_wide_tile_kernel(ctx, m, n, k):
    """The M = 2048 and 8192 cases of the prefill sweep select the 256-wide output tile (all 512
    tensor-memory columns); (2049, 11024) adds a partial last row tile and a partial last column
    tile.  The device computes every row; the oracle checks a sample of rows that covers every
    position inside a tile (the float64 product of the full matrix would take minutes)."""
    import torch
    rng = ref.rng_of(2000 + m + n + k)
    x = rng.standard_normal((m, k), dtype=np.float32)
    q, s = ref.make_q4(rng, n, k)
    w = ctx.pack_q4(q, s)
    y = ctx.gemm_q4(w, _t(x))
    ctx.device_status()
    rows = _sample_rows(m)
    ys = y[torch.from_numpy(rows).cuda()].cpu().numpy()
    xb = ref.to_bf16(x[rows])
    same = xb.astype(np.float64) @ ref.dequant_bf16(q, s).T
    assert ref.err_inf(ys, same) < 2e-5, ref.err_inf(ys, same)
    assert ref.err_inf(ys, x[rows].astype(np.float64) @ ref.dequant(q, s).T) < 5e-3
    # every row, through a size-independent property: the column sums of y equal (sum of rows of bf16(x)) . W^T
    colsum = y.double().sum(0).cpu().numpy()
    want = ref.to_bf16(x).astype(np.float64).sum(0)[None] @ ref.dequant_bf16(q, s).T
    assert ref.err_inf(colsum, want[0]) < 1e-4
    # accumulate form on bf16 activations
    y2 = ctx.gemm_q4(w, _t(ref.to_bf16(x)).to(torch.bfloat16), out=y.clone(), flags=1)
    assert float((y2 - 2 * y).abs().max()) <= 1e-5 * float(y.abs().max())
    w.free()


@pytest.mark.parametrize("n,k", [(768, 4096), (4096, 512), (2752, 4096), (4096, 1376), (1536, 4096), (4096, 2752)])
def test_tensor_parallel_shard_shapes(ctx, n, k):
    """The per-rank matrices of the 2/4/8-way sharded decoder (K = 1376 has an odd number of
    32-blocks, K = 512 fills a quarter of a copy stage): GEMV with the fused epilogues' plain form."""
    rng = ref.rng_of(n + 3 * k)
    x = rng.standard_normal((1, k), dtype=np.float32)
    q, s = ref.make_q4(rng, n, k)
    w = ctx.pack_q4(q, s)
    y = ctx.gemm_q4(w, _t(x)).cpu().numpy()
    assert ref.err_inf(y, ref.gemm_q4_fast(x, q, s)) < TIGHT
    x4 = rng.standard_normal((4, k), dtype=np.float32)
    y4 = ctx.gemm_q4(w, _t(x4)).cpu().numpy()
    assert ref.err_inf(y4, ref.gemm_q4_fast(x4, q, s)) < TIGHT
    w.free()


@pytest.mark.parametrize("dtype", ["float32", "float16", "bfloat16"])
@pytest.mark.parametrize("n,k", [(16, 32), (48, 160), (4096, 4096), (1376, 4096)])
def test_device_quantizer_bit_exact(ctx, n, k, dtype):
    """Import-time quantiser on the device against the oracle's: codes and scale bits identical, for
    every input type, a padded (odd) block count included; then the weight is usable as any other."""
    import torch
    rng = ref.rng_of(n + k)
    x = (rng.standard_normal((n, k)) * rng.uniform(1e-3, 3.0, (n, 1))).astype(np.float32)
    x[0, :32] = 0.0
    x[1, 5], x[1, 9] = -7.5, 7.5
    xt = _t(x).to(getattr(torch, dtype))
    want_q, want_s = ref.quantize_q4(xt.float().cpu().numpy())
    w = ctx.quantize_q4(xt)
    q, s = w.unpack()
    assert np.array_equal(q, want_q)
    assert np.array_equal(s.view(np.uint16), want_s.view(np.uint16))
    a = ref.rng_of(5).standard_normal((1, k), dtype=np.float32)
    y = ctx.gemm_q4(w, _t(a)).cpu().numpy()
    assert ref.err_inf(y, ref.gemm_q4(a, want_q, want_s)) < TOL
    w.free()


def test_device_quantizer_strided_input_and_errors(ctx):
    import torch
    from cyb_b200 import qeng
    x = torch.randn(32, 200, device="cuda")
    view = x[:, :160]  # leading dimension 200
    w = ctx.quantize_q4(view)
    q, s = w.unpack()
    want_q, want_s = ref.quantize_q4(view.cpu().numpy())
    assert np.array_equal(q, want_q) and np.array_equal(s.view(np.uint16), want_s.view(np.uint16))
    with pytest.raises(qeng.QengError) as e:
        ctx.quantize_q4(x[:, :100])  # K % 32 != 0
    assert e.value.code == -2


def test_next_matrix_hint_never_changes_results(ctx):
    """qeng_weight_set_next is a pure performance hint (an L2 prefetch of the matrix used next):
    outputs are bit-identical with, without, and after clearing it."""
    rng = ref.rng_of(77)
    q1, s1 = ref.make_q4(rng, 4096, 4096)
    q2, s2 = ref.make_q4(rng, 1376, 4096)
    w1, w2 = ctx.pack_q4(q1, s1), ctx.pack_q4(q2, s2)
    x = _t(rng.standard_normal((1, 4096), dtype=np.float32))
    base1, base2 = ctx.gemm_q4(w1, x).clone(), ctx.gemm_q4(w2, x).clone()
    w1.set_next(w2)
    w2.set_next(w1)
    for _ in range(3):
        assert bool((ctx.gemm_q4(w1, x) == base1).all())
        assert bool((ctx.gemm_q4(w2, x) == base2).all())
    w1.set_next(None)
    w2.set_next(None)
    assert bool((ctx.gemm_q4(w1, x) == base1).all())
    ctx.device_status()
    w1.free()
    w2.free()


def test_device_quantizer_matches_the_golden_fixture(ctx):
    w = ctx.quantize_q4(_t(GOLD["quant_x"]))
    q, s = w.unpack()
    assert np.array_equal(q, GOLD["quant_q"])
    assert np.array_equal(s.view(np.uint16), GOLD["quant_s"].view(np.uint16))
    w.free()
