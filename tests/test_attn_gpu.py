"""Parity of the decode attention and the KV append (through the C ABI) with the oracle."""
import os

import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
TOL = 2e-3
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run(ctx, q, pool_np, table, lens):
    pool = ctx.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool.tensor().copy_(_t(pool_np))
    out = ctx.attn_decode(pool, _t(q), _t(table), _t(lens)).cpu().numpy()
    pool.free()
    return out


def test_golden_page_edges(ctx):
    g = GOLD
    out = _run(ctx, g["attn_q"], g["attn_pool"], g["attn_table"], g["attn_lens"])
    assert ref.err_inf(out, g["attn_out"]) < 1e-4


def test_config4(ctx):
    lens, q, ks, vs, pool, table = ref.config4()
    out = _run(ctx, q, pool, table, lens)
    e = ref.err_inf(out, ref.attn_decode(q, ks, vs))
    assert e < TOL, e
    assert e < 1e-4, e


def test_config4_repeated_with_a_cold_cache(ctx):
    """The same call several times, the cache overwritten in between (page copies then land out of
    order): every repetition must give the same, correct result."""
    import torch
    lens, q, ks, vs, pool_np, table = ref.config4()
    want = ref.attn_decode(q, ks, vs)
    pool = ctx.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool.tensor().copy_(_t(pool_np))
    tq, tt, tl = _t(q), _t(table), _t(lens)
    for rep in range(12):
        if rep % 3 == 0:
            torch.empty(1 << 28, dtype=torch.uint8, device="cuda").random_()
        out = ctx.attn_decode(pool, tq, tt, tl).cpu().numpy()
        assert ref.err_inf(out, want) < 1e-4, rep
    pool.free()


def test_known_answers(ctx):
    rng = ref.rng_of(21)
    # len 1 -> V[0]; empty sequence -> zeros
    lens = np.array([1, 0, 5], np.int32)
    q = rng.standard_normal((3, 8, 128), dtype=np.float32).astype(np.float16)
    ks, vs, pool, table = ref.paged_kv(rng, np.array([1, 1, 5]), Hkv=2)
    ks[2][:] = ks[2][0]  # all keys equal -> mean of V
    # rebuild the pool with the modified keys
    ks2, vs2 = ks, vs
    pool[:] = 0
    nxt = {0: table[0, 0], 1: table[1, 0], 2: table[2, 0]}
    for b in (0, 2):
        L = ks2[b].shape[0]
        pool[nxt[b], :, 0, :L] = ks2[b].transpose(1, 0, 2)
        pool[nxt[b], :, 1, :L] = vs2[b].transpose(1, 0, 2)
    out = _run(ctx, q, pool, table, lens)
    assert np.allclose(out[0], np.repeat(vs[0][0].astype(np.float32), 4, 0), atol=1e-6)
    assert np.all(out[1] == 0)
    assert np.allclose(out[2], np.repeat(vs[2].astype(np.float32).mean(0), 4, 0), atol=2e-3)


def test_group_shares_kv(ctx):
    rng = ref.rng_of(22)
    lens = np.array([100], np.int32)
    q1 = rng.standard_normal((1, 1, 128), dtype=np.float32).astype(np.float16)
    q = np.repeat(q1, 8, 1)
    ks, vs, pool, table = ref.paged_kv(rng, lens, Hkv=2)
    out = _run(ctx, q, pool, table, lens)
    for h in (1, 2, 3):
        assert np.array_equal(out[0, 0], out[0, h])
    for h in (5, 6, 7):
        assert np.array_equal(out[0, 4], out[0, h])


def test_garbage_beyond_length_is_ignored(ctx):
    rng = ref.rng_of(23)
    lens = np.array([17, 33], np.int32)
    q = rng.standard_normal((2, 4, 128), dtype=np.float32).astype(np.float16)
    ks, vs, pool, table = ref.paged_kv(rng, lens, Hkv=1)
    ref_out = ref.attn_decode(q, ks, vs)
    for b in range(2):  # poison the unused slots of each last page with NaN/Inf
        last = table[b, (lens[b] - 1) // 16]
        pool[last, :, :, lens[b] % 16:, :] = np.float16(np.nan) if b == 0 else np.float16(np.inf)
    out = _run(ctx, q, pool, table, lens)
    assert np.isfinite(out).all()
    assert ref.err_inf(out, ref_out) < 1e-4


def test_bad_page_id_is_reported_not_dereferenced(ctx):
    from cyb_b200 import qeng
    rng = ref.rng_of(24)
    lens = np.array([40], np.int32)
    q = rng.standard_normal((1, 4, 128), dtype=np.float32).astype(np.float16)
    ks, vs, pool, table = ref.paged_kv(rng, lens, Hkv=1)
    table = table.copy()
    table[0, 1] = 10 ** 6
    _run(ctx, q, pool, table, lens)
    with pytest.raises(qeng.QengError) as e:
        ctx.device_status()
    assert e.value.code == -7
    ctx.device_status()  # cleared


def test_kv_append_round_trip(ctx):
    import torch
    rng = ref.rng_of(25)
    B, Hkv = 3, 2
    pool = ctx.kv_pool(12, Hkv)
    table = np.array([[3, 7, 1, 0], [2, 9, 4, 5], [11, 10, 8, 6]], np.int32)
    pos = np.array([0, 15, 16], np.int32)
    k = rng.standard_normal((B, Hkv, 128), dtype=np.float32)
    v = rng.standard_normal((B, Hkv, 128), dtype=np.float32)
    ctx.kv_append(pool, _t(k), _t(v), _t(table), _t(pos))
    p = pool.tensor().cpu().numpy()
    for b in range(B):
        pid, slot = table[b, pos[b] // 16], pos[b] % 16
        assert np.array_equal(p[pid, :, 0, slot], k[b].astype(np.float16))
        assert np.array_equal(p[pid, :, 1, slot], v[b].astype(np.float16))
    assert np.count_nonzero(p) == B * Hkv * 2 * 128
    pool.free()


@pytest.mark.parametrize("softcap,window", [(50.0, 0), (0.0, 40), (30.0, 100), (0.0, 16), (0.0, 1)])
def test_softcap_and_sliding_window(ctx, softcap, window):
    """The attention deltas of the Gemma family (qeng_attn_decode_ex): soft-capped logits and a sliding
    window over the last tokens, ragged lengths around page and window edges, against the oracle."""
    lens, q, ks, vs, pool_np, table = ref.config4(seed=60 + window, B=6, lo=1, hi=300)
    lens[:3] = [window if window else 5, 17, max(window - 1, 1)]
    # rebuild K/V for the changed lengths
    rng = ref.rng_of(61 + window)
    ks, vs, pool_np, table = ref.paged_kv(rng, lens, 8, 128, 16)
    q = (q.astype(np.float32) * 3).astype(np.float16)  # larger logits, so that the cap bites
    pool = ctx.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool.tensor().copy_(_t(pool_np))
    out = ctx.attn_decode(pool, _t(q), _t(table), _t(lens), softcap=softcap, window=window).cpu().numpy()
    want = ref.attn_decode(q, ks, vs, softcap=softcap, window=window)
    assert ref.err_inf(out, want) < 1e-4
    if softcap or window:
        assert ref.err_inf(ref.attn_decode(q, ks, vs), want) > 1e-3  # the switches matter on this input
    ctx.device_status()
    pool.free()


def test_long_cache_on_the_fixed_split_path_with_a_window(ctx):
    lens = np.array([4096, 3000, 513, 2049], np.int32)
    rng = ref.rng_of(70)
    q = rng.standard_normal((4, 32, 128), dtype=np.float32).astype(np.float16)
    ks, vs, pool_np, table = ref.paged_kv(rng, lens, 8, 128, 16)
    pool = ctx.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool.tensor().copy_(_t(pool_np))
    from cyb_b200 import qeng
    c2 = qeng.Context(0, no_attn_cluster=1)  # force the fixed splits + last-arriver merge
    pool2 = c2.kv_pool(pool_np.shape[0], pool_np.shape[1])
    pool2.tensor().copy_(_t(pool_np))
    for window in (0, 1000):
        want = ref.attn_decode(q, ks, vs, window=window)
        for c, pl in ((ctx, pool), (c2, pool2)):
            out = c.attn_decode(pl, _t(q), _t(table), _t(lens), window=window).cpu().numpy()
            assert ref.err_inf(out, want) < 1e-4, window
            c.device_status()
    pool.free()
    pool2.free()
    c2.close()
