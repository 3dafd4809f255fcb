"""The allocation-free attention entry point (qeng_attn_decode_noalloc) against the
regular one.  It exists for hosts that must not allocate device memory while they
run (a fixed memory budget handed over at start-up, or a token loop that may never
enter the CUDA allocator): its split scratch is an array built into the library.
The file name keeps it last in collection order, so a run that stops at the first
failure has already run every other test; it also passes alone in a fresh process."""
import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_noalloc_matches_regular_entry_point_twice(ctx):
    import torch
    lens, q, ks, vs, pool_np, table = ref.config4(seed=41, B=5, lo=1, hi=700)
    pool = ctx.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool.tensor().copy_(_t(pool_np))
    qd, td, ld = _t(q), _t(table), _t(lens)
    want = ctx.attn_decode(pool, qd, td, ld)
    assert ref.err_inf(want.cpu().numpy(), ref.attn_decode(q, ks, vs)) < 1e-4
    out = torch.empty_like(want)
    for call in range(2):  # the array keeps the previous call's contents: the second call must not care
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        # free bytes as the driver sees them: this also counts a cudaMalloc made inside the library,
        # which torch's own allocator statistics would never show.  The first call may load the
        # kernels' module, so the comparison is made on the second one.
        before = torch.cuda.mem_get_info()[0]
        ctx.attn_decode_noalloc(pool, qd, td, ld, out=out)
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == before
        assert float((out - want).abs().max()) <= 1e-6 * float(want.abs().max()), call
    # a different shape right after, then the first one again
    lens2, q2, ks2, vs2, pool2_np, table2 = ref.config4(seed=42, B=2, lo=30, hi=90)
    pool2 = ctx.kv_pool(pool2_np.shape[0], pool2_np.shape[1])
    pool2.tensor().copy_(_t(pool2_np))
    got2 = ctx.attn_decode_noalloc(pool2, _t(q2), _t(table2), _t(lens2)).cpu().numpy()
    assert ref.err_inf(got2, ref.attn_decode(q2, ks2, vs2)) < 1e-4
    ctx.attn_decode_noalloc(pool, qd, td, ld, out=out)
    assert float((out - want).abs().max()) <= 1e-6 * float(want.abs().max())
    pool.free()
    pool2.free()


def test_noalloc_at_the_documented_limit_shape(ctx):
    """16 sequences x 32 heads with caches of 512..4096 tokens (15 splits): the example the header
    gives for what the built-in array holds.  Checked against the regular entry point and the oracle."""
    import torch
    lens, q, ks, vs, pool_np, table = ref.config4(seed=4)
    pool = ctx.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool.tensor().copy_(_t(pool_np))
    qd, td, ld = _t(q), _t(table), _t(lens)
    want = ctx.attn_decode(pool, qd, td, ld)
    out = torch.empty_like(want)
    for call in range(2):
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]
        ctx.attn_decode_noalloc(pool, qd, td, ld, out=out)
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info()[0] == before
        assert float((out - want).abs().max()) <= 1e-6 * float(want.abs().max()), call
    assert ref.err_inf(out.cpu().numpy(), ref.attn_decode(q, ks, vs)) < 1e-4
    pool.free()


def test_noalloc_rejects_shapes_beyond_the_built_in_scratch(ctx):
    import torch
    from cyb_b200 import qeng
    B, Hq, Hkv, max_pages = 64, 64, 8, 4096  # far more partials than 4 MiB holds
    pool = ctx.kv_pool(4, Hkv)
    q = torch.zeros((B, Hq, 128), dtype=torch.float16, device="cuda")
    table = torch.zeros((B, max_pages), dtype=torch.int32, device="cuda")
    lens = torch.zeros((B,), dtype=torch.int32, device="cuda")
    with pytest.raises(qeng.QengError) as e:
        ctx.attn_decode_noalloc(pool, q, table, lens)
    assert e.value.code == -2 and "exceeds the built-in scratch" in str(e.value)
    pool.free()
