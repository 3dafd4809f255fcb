"""Parity of the small operators (through the C ABI) with the oracle."""
import os

import numpy as np
import pytest

from oracle import ref

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def _t(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_rmsnorm(ctx):
    g = GOLD
    y = ctx.rmsnorm(_t(g["rms_x"]), _t(g["rms_g"]), 1e-5).cpu().numpy()
    assert ref.err_inf(y, g["rms_y"]) < 2e-6


def test_rope(ctx):
    g = GOLD
    y = ctx.rope_(_t(g["rope_x"]), _t(g["rope_pos"]), 10000.0).cpu().numpy()
    assert ref.err_inf(y, g["rope_y"]) < 2e-6
    x = g["rope_x"][:1]
    assert np.array_equal(ctx.rope_(_t(x), _t(np.zeros(1, np.int32)), 10000.0).cpu().numpy(), x)


def test_swiglu_add(ctx):
    g = GOLD
    y = ctx.swiglu(_t(g["swiglu_g"]), _t(g["swiglu_u"])).cpu().numpy()
    assert ref.err_inf(y, g["swiglu_y"]) < 2e-6
    a, b = g["swiglu_g"], g["swiglu_u"]
    assert np.array_equal(ctx.add(_t(a), _t(b)).cpu().numpy(), a + b)


@pytest.mark.parametrize("m", [1, 3, 5, 16])
def test_embed_lm_head_argmax(ctx, m):
    import torch
    rng = ref.rng_of(30 + m)
    V, D = 1000, 256
    table = ref.to_bf16(rng.standard_normal((V, D), dtype=np.float32) * 0.02)
    tb = _t(ref.bf16_bits(table)).view(torch.int16)
    toks = rng.integers(0, V, m).astype(np.int32)
    x = ctx.embed(tb, _t(toks)).cpu().numpy()
    assert np.array_equal(x, table[toks])
    h = rng.standard_normal((m, D), dtype=np.float32)
    logits = ctx.lm_head(tb, _t(h))
    lref = h.astype(np.float64) @ table.astype(np.float64).T
    assert ref.err_inf(logits.cpu().numpy(), lref) < 2e-6
    idx = ctx.argmax(logits).cpu().numpy()
    assert np.array_equal(idx, logits.cpu().numpy().argmax(-1))
    # ties resolve to the lowest index
    tie = torch.zeros((2, 700), device="cuda")
    tie[0, 5] = tie[0, 300] = 3.0
    tie[1, 699] = 1.0
    assert ctx.argmax(tie).cpu().tolist() == [5, 699]


def test_embed_rejects_bad_token(ctx):
    import torch
    from cyb_b200 import qeng
    tb = torch.zeros((10, 64), dtype=torch.int16, device="cuda")
    ctx.embed(tb, _t(np.array([3, 11], np.int32)))
    with pytest.raises(qeng.QengError):
        ctx.device_status()
