"""Zaronex without a GPU: configuration checks, the registry entry, weight names, and closed-form self-checks of the plain oracle
(windows and pooled blocks, the sink, the turning of values, both recurrences, the depth average)."""
import json
import math

import numpy as np
import pytest

from tests import oracle_zaronex as O


def _cfg(layers):
    return {"architecture": "Zaronex", "vocab": 11, "width": 8, "norm": {"eps": 1e-5}, "layers": layers}


def _latent(**kw):
    m = {"heads": 2, "dim": 4, "rot_dim": 2, "vdim": 6, "kv_rank": 5, "q_rank": 3, "scale": 0.5, "mask": {"size": 4}, "rot": {"base": 100.0, "dims": 2}}
    m.update(kw)
    return {"type": "latent_attention", "mixer": m, "mlp": None}


def _left(**kw):
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 0.5, "mask": {"size": 3, "pool": 2}, "rot": {"base": 100.0, "dims": 2}}
    m.update(kw)
    return m


def _par(**kw):
    return {"type": "parallel", "mixer": {"left": _left(**kw), "right": {"heads": 2, "dim": 3, "vdim": 4, "tau": 2.0}}, "mlp": {"kind": "dense", "ff": 9}}


def _par2(**kw):
    return {"type": "parallel_2", "mixer": {"left": _left(**kw), "right": {"inner": 6, "state": 3, "dt_rank": 2, "conv": 3}}, "mlp": None}


def test_config_checks():
    from krasis_b200.zaronex import ZaronexConfig
    cfg = ZaronexConfig.from_dict(_cfg([_latent(), _par(), _par2()]))
    assert cfg.vocab == 11 and cfg.width == 8 and cfg.eps == 1e-5 and len(cfg.layers) == 3
    for bad in (_cfg([{"type": "attention", "mixer": {}, "mlp": None}]), _cfg([_par(heads=3, kv_heads=2)]),
                _cfg([dict(_latent(), mlp={"kind": "moe"})])):
        with pytest.raises(ValueError):
            ZaronexConfig.from_dict(bad)


def test_registry_knows_the_design(tmp_path):
    from krasis_b200.registry import architecture_of
    (tmp_path / "config.json").write_text(json.dumps(_cfg([])))
    assert architecture_of(str(tmp_path)) == "Zaronex"


def test_random_weights_have_the_designs_names():
    from krasis_b200.zaronex import ZaronexConfig, random_weights
    w = random_weights(ZaronexConfig.from_dict(_cfg([_latent(), _par(), _par2()])), 0)
    assert w["embed"].shape == (11, 8) and w["head"].shape == (11, 8) and w["final.norm"].shape == (8,)
    assert w["l0.mix.dq"].shape == (3, 8) and w["l0.mix.uq"].shape == (12, 3) and w["l0.mix.dkv"].shape == (7, 8) and w["l0.mix.dkv.norm"].shape == (5,)
    assert w["l0.mix.uk"].shape == (8, 5) and w["l0.mix.uv"].shape == (12, 5) and w["l0.mix.g"].shape == (12, 8) and "l0.norm2" not in w
    assert w["l1.mix.left.q.b"].shape == (8,) and w["l1.mix.left.sink"].shape == (2,) and w["l1.mix.left.g"].shape == (12, 8)
    assert w["l1.mix.right.a2"].shape[0] == 6 and w["l1.mix.right.a2.b"].shape == (6,) and w["l1.mix.right.norm"].shape == (4,)
    assert w["l1.mix.left.out"].shape == (8,) and w["l1.mlp.down"].shape == (8, 9)
    assert w["l2.mix.left.q.norm"].shape == (8,) and w["l2.mix.left.k.norm"].shape == (4,) and "l2.mix.left.sink" not in w and "l2.mix.left.q.b" not in w
    assert w["l2.mix.right.in"].shape == (12, 8) and w["l2.mix.right.conv"].shape == (6, 3) and w["l2.mix.right.x"].shape == (8, 6)
    assert w["l2.mix.right.dt"].shape == (6, 2) and w["l2.mix.right.A_log"].shape == (6, 3)
    assert [w[f"l{i}.dwa"].numel() for i in range(3)] == [2, 3, 4]


def test_frequency_table_against_the_oracle():
    from krasis_b200.mixers import rotary_table
    for dims, base, factor in ((16, 3000.0, 1.0), (6, 20000.0, 8.0), (2, 7.0, 2.5)):
        assert np.allclose(rotary_table(dims, base, factor).numpy(), O.pair_frequencies(dims, base, factor), rtol=1e-14, atol=0)


def test_oracle_windows_and_pooled_blocks():
    assert O.window_keys(10, 4) == [7, 8, 9, 10] and O.window_keys(2, 4) == [0, 1, 2] and O.window_keys(5, 1) == [5]
    # position 10, window 4: positions 7 .. 10 are seen one by one; blocks of 3 end at 2, 5, 8: those ending at or before 6 are seen
    assert O.pooled_blocks(10, 4, 3) == [0, 1]
    assert O.pooled_blocks(9, 4, 3) == [0, 1] and O.pooled_blocks(8, 4, 3) == [0] and O.pooled_blocks(5, 4, 3) == [] and O.pooled_blocks(6, 4, 3) == [0]
    assert O.pooled_blocks(3, 1, 1) == [0, 1, 2]


def test_oracle_sink_takes_weight_without_a_value():
    keys, vals = np.zeros((2, 3)), np.array([[1.0, 0.0], [0.0, 1.0]])
    assert np.allclose(O.visible_softmax(np.ones(3), keys, vals, 1.0), [0.5, 0.5])
    assert np.allclose(O.visible_softmax(np.ones(3), keys, vals, 1.0, sink=0.0), [1 / 3, 1 / 3])
    assert np.allclose(O.visible_softmax(np.ones(3), keys, vals, 1.0, sink=math.log(2.0)), [0.25, 0.25])


def test_oracle_turns():
    x = np.zeros((3, 1, 6))
    x[:, 0, 0] = 1.0
    r = O.turn(x, 1.0, [0, 1, 2], np.array([1.0, 0.5]), True)                 # halves: dimension 0 turns with dimension 2
    assert np.allclose(r[:, 0, 0], np.cos([0, 1, 2])) and np.allclose(r[:, 0, 2], np.sin([0, 1, 2])) and np.all(r[:, 0, [1, 3, 4, 5]] == 0)
    r = O.turn(x, 1.0, [0, 1, 2], np.array([1.0, 0.5]), False)                # interleaved: dimension 0 turns with dimension 1
    assert np.allclose(r[:, 0, 1], np.sin([0, 1, 2])) and np.all(r[:, 0, 2:] == 0)
    y = np.random.default_rng(0).normal(size=(4, 2, 6))
    back = O.turn(O.turn(y, 1.0, [3, 5, 8, 13], O.pair_frequencies(6, 50.0), False), -1.0, [3, 5, 8, 13], O.pair_frequencies(6, 50.0), False)
    assert np.allclose(back, y)


def test_oracle_gated_linear_attention_closed_form():
    """One head, two tokens: S_2 = diag(alpha_2) k_1 v_1^T + k_2 v_2^T and o_2 = S_2^T q_2."""
    W, m = 4, {"heads": 1, "dim": 2, "vdim": 2, "tau": 2.0}
    eye = np.eye(W)
    w = {"q": eye[:2], "k": eye[:2], "v": eye[2:], "g": np.zeros((2, W)), "a1": np.zeros((1, W)), "a2": np.zeros((2, 1)),
         "a2.b": np.array([0.0, 40.0]), "norm": np.ones(2), "o": np.eye(2)}
    h = np.array([[1.0, 2.0, 3.0, -1.0], [0.5, -1.0, 2.0, 2.0]])
    S = np.zeros((1, 2, 2))
    O.gated_linear_attention(h, w, m, 0.0, state=S)
    alpha = np.array([0.5 ** 0.5, 1.0])                                       # sigmoid(0)^(1/2), sigmoid(40)^(1/2)
    want = alpha[:, None] * np.outer(h[0, :2], h[0, 2:]) + np.outer(h[1, :2], h[1, 2:])
    assert np.allclose(S[0], want)


def test_oracle_selective_scan_closed_form():
    """One channel, one state, no convolution memory: S_t = exp(dt A) S_(t-1) + dt x B, y = S C + D x."""
    m = {"inner": 1, "state": 1, "dt_rank": 1, "conv": 1}
    w = {"in": np.array([[1.0, 0.0], [0.0, 1.0]]), "conv": np.ones((1, 1)), "conv.b": np.zeros(1), "x": np.array([[0.0], [1.0], [2.0]]),
         "dt": np.zeros((1, 1)), "dt.b": np.array([math.log(math.e - 1.0)]), "A_log": np.zeros((1, 1)), "D": np.array([0.5]), "o": np.ones((1, 1))}
    h = np.array([[1.0, 0.3], [2.0, -0.4]])
    x = O.silu(h[:, 0])                                                       # dt = softplus(ln(e - 1)) = 1, A = -1, B = x, C = 2 x
    s1 = x[0] * x[0]
    s2 = math.exp(-1.0) * s1 + x[1] * x[1]
    y = np.array([s1 * 2 * x[0] + 0.5 * x[0], s2 * 2 * x[1] + 0.5 * x[1]]) * O.silu(h[:, 1])
    assert np.allclose(O.selective_scan(h, w, m)[:, 0], y)


def test_oracle_depth_average_uses_every_earlier_result():
    from krasis_b200.zaronex import ZaronexConfig, random_weights
    raw = _cfg([_latent(), _par(), _par2()])
    w = {k: v.numpy().astype(np.float64) for k, v in random_weights(ZaronexConfig.from_dict(raw), 3).items()}
    tk = [1, 5, 2, 7, 7, 3, 0, 9, 4]
    base = O.forward(raw, w, tk)
    w2 = dict(w)
    w2["l2.dwa"] = w["l2.dwa"].copy()
    w2["l2.dwa"][0] += 0.5                                                    # more of the embedding output in the last average
    x0 = w["embed"][np.asarray(tk)]
    trace, trace2 = [], []
    O.forward(raw, w, tk, trace)
    moved = O.forward(raw, w2, tk, trace2)
    assert np.allclose(trace2[2] - trace[2], 0.5 * x0) and np.allclose(trace2[1], trace[1]) and not np.allclose(moved, base)
