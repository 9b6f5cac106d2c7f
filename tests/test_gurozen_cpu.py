"""Gurozen without a GPU: configuration checks, the order of layer runs, the registry entry, weight names, the frequency table, and
closed-form self-checks of the plain oracle."""
import json
import math

import numpy as np
import pytest

from tests import oracle_gurozen as O


def _cfg(layers, loop=None):
    raw = {"architecture": "Gurozen", "vocab": 11, "width": 8, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "logit_scale": 2.0, "layers": layers}
    if loop:
        raw["loop"] = dict(zip(("start", "stop", "times"), loop))
    return raw


def _attn(**kw):
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "conv": 2, "scale": 0.5, "softcap": 10.0, "rot": {"base": 100.0, "dims": 2}}
    m.update(kw)
    return {"type": "attention", "mixer": m, "mlp": None}


def _delta(**kw):
    m = {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 3, "conv": 3}
    m.update(kw)
    return {"type": "channel_delta", "mixer": m, "mlp": None}


def test_config_checks_and_layer_runs():
    from krasis_b200.gurozen import GurozenConfig
    cfg = GurozenConfig.from_dict(_cfg([_attn(), _delta(), _attn(), _delta()], loop=(1, 3, 3)))
    assert cfg.runs() == [(0, False), (1, True), (2, False), (1, True), (2, False), (1, True), (2, False), (3, False)]
    assert cfg.runs() == O.layer_runs(cfg.raw)
    assert GurozenConfig.from_dict(_cfg([_attn(), _delta()])).runs() == [(0, False), (1, False)]
    assert GurozenConfig.from_dict(_cfg([_attn(), _delta()], loop=(0, 2, 1))).runs() == [(0, True), (1, False)]
    assert GurozenConfig.from_dict(_cfg([_attn(), _delta()], loop=(1, 1, 5))).runs() == [(0, False), (1, False)]
    for bad in (_cfg([{"type": "latent", "mixer": _attn()["mixer"], "mlp": None}]), _cfg([_attn(heads=3, kv_heads=2)]),
                _cfg([dict(_attn(), mlp={"kind": "conv"})]), _cfg([_attn()], loop=(0, 2, 2)), _cfg([_attn()], loop=(1, 0, 2))):
        with pytest.raises(ValueError):
            GurozenConfig.from_dict(bad)


def test_registry_knows_the_design(tmp_path):
    from krasis_b200.registry import architecture_of
    (tmp_path / "config.json").write_text(json.dumps(_cfg([])))
    assert architecture_of(str(tmp_path)) == "Gurozen"


def test_random_weights_have_the_designs_names():
    from krasis_b200.gurozen import GurozenConfig, random_weights
    mlp = {"kind": "moe", "expert": {"ff": 5}, "router": {"experts": 4, "top": 2, "scale": 1.5, "groups": {"count": 2, "keep": 1}}, "shared": {"ff": 7}}
    cfg = GurozenConfig.from_dict(_cfg([dict(_attn(), mlp={"kind": "dense", "ff": 9}), dict(_delta(), mlp=mlp)], loop=(0, 1, 2)))
    w = random_weights(cfg, 0)
    assert w["loop.in"].shape == (8, 16) and w["embed.norm"].shape == (8,) and "head" not in w
    assert w["l0.mix.q"].shape == (8, 8) and w["l0.mix.k.b"].shape == (4,) and w["l0.mix.q.norm"].shape == (8,) and w["l0.mix.v.conv"].shape == (6, 2)
    assert w["l1.mix.dt_bias"].shape == (8,) and w["l1.mix.A_log"].shape == (2,) and w["l1.mix.a2"].shape[0] == 8 and w["l1.mix.g2"].shape[0] == 6
    assert w["l1.mlp.router"].shape == (4, 8) and w["l1.mlp.e3.up"].shape == (5, 8) and "l1.mlp.e0.gate" not in w
    assert w["l1.mlp.shared.sg"].shape == (1, 8) and w["l0.mlp.down"].shape == (8, 9) and "l1.mix.q.b" not in w


def test_frequency_table_against_the_oracle():
    from krasis_b200.mixers import llama3_table
    for sc in (None, {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}, {"factor": 2.0, "low": 2.0, "high": 2.0, "original": 30}):
        rot = {"base": 3000.0, "dims": 16}
        if sc:
            rot["scaling"] = sc
        assert np.allclose(llama3_table(16, 3000.0, sc).numpy(), O.rot_frequencies(rot), rtol=1e-14, atol=0)
    f = O.rot_frequencies({"base": 3000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}})
    plain = O.rot_frequencies({"base": 3000.0, "dims": 16})
    assert f[0] == plain[0] and math.isclose(f[-1], plain[-1] / 4.0) and np.all(f <= plain) and np.all(f >= plain / 4.0 * (1 - 1e-12))


def test_oracle_convolution_and_rotation():
    u = np.arange(12, dtype=np.float64).reshape(6, 2)
    taps = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = O.causal_conv(u, taps)
    assert np.array_equal(y[:, 1], u[:, 1])                                   # the last column is the current token's
    assert y[0, 0] == 0.0 and y[1, 0] == 100 * 2 + 10 * 0 and y[3, 0] == 100 * 6 + 10 * 4 + 2
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = 1.0                                                          # dimension 0 turns with dimension 2 (dims 4)
    r = O.rotate_half(x, [0, 1, 2], {"base": 1.0, "dims": 4})
    assert np.allclose(r[:, 0, 0], np.cos([0, 1, 2])) and np.allclose(r[:, 0, 2], np.sin([0, 1, 2])) and np.all(r[:, 0, [1, 3, 4, 5]] == 0)


def test_oracle_delta_rule_closed_forms():
    """One head, one token: S = k u^T with u = beta v, o = (k . q) beta v.  Two equal keys: the second write replaces what the decay
    left of the first."""
    W = 4
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "conv": 1}
    eye = np.eye(W)
    w = {"q": eye[:2], "k": eye[:2], "v": eye[2:], "q.conv": np.ones((2, 1)), "k.conv": np.ones((2, 1)), "v.conv": np.ones((2, 1)),
         "b": np.zeros((1, W)), "a1": np.zeros((1, W)), "a2": np.zeros((2, 1)), "g1": np.zeros((1, W)), "g2": np.zeros((2, 1)),
         "A_log": np.zeros(1), "dt_bias": np.array([0.0, 50.0]), "norm": np.ones(2), "o": np.eye(4)[:, :2]}
    h = np.array([[1.0, 0.0, 2.0, -1.0]])
    _, S = O.channel_delta(h, w, m, 0.0, return_state=True)
    kq = O.silu(1.0) / math.sqrt(O.silu(1.0) ** 2 + 1e-6)
    v = O.silu(np.array([2.0, -1.0]))
    assert np.allclose(S[0], np.outer([kq, 0.0], 0.5 * v))
    _, S2 = O.channel_delta(np.concatenate([h, h]), w, m, 0.0, return_state=True)
    g0 = math.exp(-math.log(2.0))                                             # softplus(0) = ln 2 on channel 0, exp(-50) ~ 0 on channel 1
    first = g0 * 0.5 * v * kq
    assert np.allclose(S2[0][0], first + kq * 0.5 * (v - kq * first))


def test_oracle_router_groups():
    h = np.eye(6)[:1]
    router = np.zeros((6, 6))
    router[:, 0] = [3.0, -3.0, 2.0, 2.0, 1.0, -9.0]                          # scores .95 .05 | .88 .88 | .73 ~0: best pair is the middle group
    ids, wt = O.route(h, router, {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}})
    assert ids[0].tolist() == [2, 3] and np.allclose(wt[0], [1.5, 1.5])
    ids, wt = O.route(h, router, {"experts": 6, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 2}})
    assert ids[0].tolist() == [0, 2] and math.isclose(wt[0].sum(), 1.0)
