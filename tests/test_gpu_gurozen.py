"""Gurozen on the GPU against the plain float64 oracle (tests/oracle_gurozen.py): each mechanism alone, then the whole model through
the scheduler — prefill against decoding, portions down to two tokens, unequal batches, reuse of pages and slots, far keys and page
borders with peaked scores, the looped span, long decoding of the recurrence, odd sizes, and greedy generation through the generation
entry point.  Small random configurations made here; none of them is a shipped model's."""
import json
import struct

import numpy as np
import pytest
import torch

from tests import oracle_gurozen as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def seq():
    from krasis_b200.build import build_seq
    build_seq()
    from krasis_b200 import seqops
    seqops.load()
    return seqops


def attn(heads=6, kv_heads=3, dim=16, vdim=20, conv=3, rot_dims=12, base=5000.0, scaling="default", scale=None, softcap=5.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale if scale is not None else dim ** -0.5,
         "softcap": softcap}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if scaling == "default":
            scaling = {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 40}
        if scaling:
            m["rot"]["scaling"] = scaling
    return m


def delta(heads=4, kv_heads=2, dim=16, vdim=24, conv=4):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def dense(ff=56):
    return {"kind": "dense", "ff": ff}


def moe(experts=16, top=3, groups=4, keep=2, ff=24, shared=40, scale=1.5):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def A(mixer=None, mlp=None):
    return {"type": "attention", "mixer": mixer or attn(), "mlp": mlp}


def D(mixer=None, mlp=None):
    return {"type": "channel_delta", "mixer": mixer or delta(), "mlp": mlp}


def model_cfg(layers, width=48, vocab=50, loop=(1, 3, 2), mult=0.7, logit_scale=0.25, eps=1e-5):
    raw = {"architecture": "Gurozen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "logit_scale": logit_scale,
           "layers": layers}
    if loop:
        raw["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return raw


def default_layers():
    return [A(attn(), dense()), D(delta(), moe()), A(attn(heads=2, kv_heads=1, dim=24, vdim=40, conv=2, rot_dims=24, scaling=None, softcap=0.0), moe(experts=5, top=2, groups=1, keep=1, shared=0)),
            D(delta(heads=3, kv_heads=3, dim=32, vdim=32, conv=2), dense(ff=33)), A(attn(heads=4, kv_heads=4, dim=8, vdim=8, rot_dims=4, conv=4))]


def build(raw, dtype=torch.float32, seed=0, page_size=None, tweak=None):
    from krasis_b200.gurozen import GurozenConfig, GurozenModel, random_weights
    cfg = GurozenConfig.from_dict(raw)
    w = random_weights(cfg, seed)
    if tweak:
        tweak(w)
    model = GurozenModel(cfg, w, dtype=dtype)
    if page_size:
        model.page_size = page_size
    return model, {k: v.numpy().astype(np.float64) for k, v in w.items()}


def sched(model, max_tokens=512, max_requests=4, **kw):
    from krasis_b200.scheduler import Scheduler
    return Scheduler(model, max_tokens=max_tokens, max_requests=max_requests, **kw)


def toks(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def close(got, want, rel, what=""):
    got = np.asarray(got, dtype=np.float64)
    err = np.abs(got - want).max() / max(np.abs(want).max(), 1e-9)
    assert err <= rel, f"{what}: relative error {err:.3e} > {rel:.1e}"


def run_portions(model, tokens, cuts, s=None, rid="a", finish=True):
    """Feed `tokens` in portions of the given sizes (the rest one by one); logits of every position."""
    s = s or sched(model)
    out, at = [], 0
    for n in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        out.append(s.step([(rid, tokens[at:at + n], list(range(n)))]).cpu().numpy())
        at += n
    if finish:
        s.finish(rid)
    return np.concatenate(out, 0)


def rnd(*shape, seed=0, sd=1.0):
    return (torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * sd).to(torch.bfloat16).float()


def f64(d):
    return {k: v.numpy().astype(np.float64) for k, v in d.items()}


def under(d):
    return {k.replace(".", "_"): v for k, v in d.items()}


# ------------------------------------------------------------------------------------------------ mechanisms alone

def attn_weights(m, W, seed):
    H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    w = {"o": rnd(W, H * dv, seed=seed, sd=0.1)}
    for i, (n, rows) in enumerate((("q", H * d), ("k", G * d), ("v", G * dv))):
        w[n] = rnd(rows, W, seed=seed + 1 + i, sd=W ** -0.5 * 2)
        w[n + ".b"] = rnd(rows, seed=seed + 4 + i, sd=0.3)
        if K:
            w[n + ".conv"] = rnd(rows, K, seed=seed + 7 + i, sd=0.6)
        if n != "v":
            w[n + ".norm"] = 1 + rnd(rows, seed=seed + 10 + i, sd=0.3)
    return w


def make_attention(m, w, dtype=torch.float32):
    from krasis_b200.mixers import MultiMapAttention, llama3_table
    rot = m.get("rot") or {}
    dims = rot.get("dims", 0)
    freq = llama3_table(dims, rot["base"], rot.get("scaling")) if dims else None
    return MultiMapAttention(under(w), m["heads"], m["kv_heads"], 1, m["dim"], m["vdim"], m["scale"], 1e-5, dtype, torch.device(DEV),
                             rot_dims=dims, rot_freq=freq, rot_half=True, norm_whole=True, conv_taps=m["conv"], softcap=m["softcap"])


def run_attention(seq, mixer, h, cuts, page_size=4, slot=1):
    from krasis_b200.attention import HeadKVCache, RecurrentStatePool, SequenceKVState
    T = h.shape[0]
    kv = HeadKVCache([mixer.cache_dims()], DEV, max_pages=(T + page_size - 1) // page_size + 2, dtype=mixer.dtype, page_size=page_size)
    pool = RecurrentStatePool(3, DEV)
    tail = mixer.register_state(pool)
    st = SequenceKVState(kv)
    kc, vc = kv.get_layer_caches(0)
    out, at = [], 0
    for n in list(cuts) + [1] * (T - sum(cuts)):
        st.ensure_capacity(n)
        tb = seq.StepTables([([0] * n, st.seq_len, slot, st.pages)], torch.device(DEV))
        out.append(mixer.forward(h[at:at + n].to(DEV, mixer.dtype).contiguous(), tb, kc, vc, page_size, tail=tail).cpu().numpy())
        st.advance(n)
        at += n
    return np.concatenate(out, 0)


@pytest.mark.parametrize("m", [attn(), attn(heads=2, kv_heads=2, dim=32, vdim=8, conv=1, rot_dims=32, scaling=None),
                               attn(heads=8, kv_heads=1, dim=6, vdim=70, conv=5, rot_dims=2, softcap=0.0),
                               attn(heads=3, kv_heads=3, dim=10, vdim=33, conv=0, rot_dims=0, scale=0.7, softcap=1.5),
                               attn(heads=4, kv_heads=2, dim=16, vdim=16, conv=2, rot_dims=16, base=50.0, scaling={"factor": 3.0, "low": 2.0, "high": 2.0, "original": 12})])
def test_attention_alone(seq, m):
    W, T = 48, 41
    w = attn_weights(m, W, seed=3)
    h = rnd(T, W, seed=1)
    want = O.attention(h.numpy().astype(np.float64), f64(w), m, 1e-5)
    mixer = make_attention(m, w)
    for cuts in ([T], [], [2, 2, 5, 17], [30, 2]):
        close(run_attention(seq, mixer, h, cuts), want, 3e-5, f"portions {cuts}")


def test_frequency_table_has_all_three_regimes():
    from krasis_b200.mixers import llama3_table
    rot = {"base": 5000.0, "dims": 24, "scaling": {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 40}}
    want = O.rot_frequencies(rot)
    plain = O.rot_frequencies({"base": 5000.0, "dims": 24})
    kinds = {"kept": (want == plain).sum(), "slowed": np.isclose(want, plain / 8.0).sum()}
    assert kinds["kept"] >= 2 and kinds["slowed"] >= 2 and kinds["kept"] + kinds["slowed"] < 12      # and blended ones in between
    got = llama3_table(24, 5000.0, rot["scaling"]).numpy()
    assert np.allclose(got, want, rtol=1e-14, atol=0)


def test_softcap_and_far_key_in_decode_grid(seq):
    """One decoded token over hundreds of keys runs as several blocks per token whose pieces are merged.  Scores are large enough for the
    cap to bite (the oracle without the cap differs by far more than the tolerance)."""
    m = attn(heads=4, kv_heads=2, dim=16, vdim=32, rot_dims=16, scale=2.0, softcap=3.0)
    W, T = 32, 300
    w = attn_weights(m, W, seed=9)
    h = rnd(T, W, seed=4)
    want = O.attention(h.numpy().astype(np.float64), f64(w), m, 1e-5)
    nocap = O.attention(h.numpy().astype(np.float64), f64(w), dict(m, softcap=0.0), 1e-5)
    assert np.abs(nocap - want).max() > 0.05 * np.abs(want).max()
    close(run_attention(seq, make_attention(m, w), h, [T - 3], page_size=64), want, 3e-5, "fp32, cut key range")
    close(run_attention(seq, make_attention(m, w, torch.bfloat16), h, [T - 3], page_size=64), want, 3e-2, "bf16, cut key range")


def delta_weights(m, W, seed, rank=5, slow=False):
    H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    w = {"o": rnd(W, H * dv, seed=seed, sd=0.1), "b": rnd(H, W, seed=seed + 1, sd=W ** -0.5 * 2), "a1": rnd(rank, W, seed=seed + 2, sd=W ** -0.5),
         "a2": rnd(H * d, rank, seed=seed + 3, sd=1.0), "g1": rnd(rank + 2, W, seed=seed + 4, sd=W ** -0.5), "g2": rnd(H * dv, rank + 2, seed=seed + 5, sd=1.0),
         "A_log": rnd(H, seed=seed + 6, sd=0.5) - (5.0 if slow else 1.0), "dt_bias": rnd(H * d, seed=seed + 7, sd=0.7), "norm": 1 + rnd(dv, seed=seed + 8, sd=0.2)}
    for i, (n, rows) in enumerate((("q", G * d), ("k", G * d), ("v", H * dv))):
        w[n] = rnd(rows, W, seed=seed + 10 + i, sd=W ** -0.5 * 2)
        w[n + ".conv"] = rnd(rows, K, seed=seed + 13 + i, sd=0.6)
    return w


def run_delta(seq, mixer, h, cuts, slot=2):
    from krasis_b200.attention import RecurrentStatePool
    pool = RecurrentStatePool(3, DEV)
    tail, state = mixer.register_state(pool)
    out, at, T = [], 0, h.shape[0]
    for n in list(cuts) + [1] * (T - sum(cuts)):
        tb = seq.StepTables([([0] * n, at, slot, [0])], torch.device(DEV))
        out.append(mixer.forward(h[at:at + n].to(DEV, mixer.dtype).contiguous(), tb, tail, state).cpu().numpy())
        at += n
    return np.concatenate(out, 0), state[slot].cpu().numpy()


@pytest.mark.parametrize("m", [delta(), delta(heads=3, kv_heads=3, dim=32, vdim=32, conv=2), delta(heads=4, kv_heads=1, dim=64, vdim=64, conv=3),
                               delta(heads=2, kv_heads=1, dim=128, vdim=32, conv=4), delta(heads=1, kv_heads=1, dim=5, vdim=3, conv=1),
                               delta(heads=6, kv_heads=2, dim=20, vdim=70, conv=6), delta(heads=2, kv_heads=1, dim=256, vdim=250, conv=2)])
def test_channel_delta_alone(seq, m):
    from krasis_b200.mixers import ChannelDeltaMixer
    W, T = 40, 37
    w = delta_weights(m, W, seed=5)
    h = rnd(T, W, seed=2)
    want, want_state = O.channel_delta(h.numpy().astype(np.float64), f64(w), m, 1e-5, return_state=True)
    dec = np.exp(-np.exp(f64(w)["A_log"])[:, None] * O.softplus(f64(w)["dt_bias"]).reshape(m["heads"], m["dim"]))
    assert dec.std() > 0.02, "the decays of a head's channels must differ for the test to see them"
    mixer = ChannelDeltaMixer(under(w), m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], 1e-5, torch.float32, torch.device(DEV))
    for cuts in ([T], [], [2, 2, 9, 17], [31, 2]):
        got, state = run_delta(seq, mixer, h, cuts)
        close(got, want, 3e-5, f"portions {cuts}")
        close(state, want_state, 3e-5, f"state after portions {cuts}")


def test_squared_relu_and_silu_units(seq):
    from krasis_b200.mixers import GatedMLP
    W, F, T = 40, 72, 19
    w = {"gate": rnd(F, W, seed=1, sd=0.5), "up": rnd(F, W, seed=2, sd=0.5), "down": rnd(W, F, seed=3, sd=0.2)}
    h = rnd(T, W, seed=4)
    hw, hh = f64(w), h.numpy().astype(np.float64)
    close(GatedMLP(w, torch.float32, DEV, act="silu").forward(h.cuda()).cpu().numpy(), O.dense_ff(hh, hw), 2e-5, "silu")
    un = {"up": w["up"], "down": w["down"]}
    close(GatedMLP(un, torch.float32, DEV, act="relu2", gated=False).forward(h.cuda()).cpu().numpy(),
          O.squared_relu_expert(hh, hw["up"], hw["down"]), 2e-5, "squared relu")
    got = GatedMLP(un, torch.bfloat16, DEV, act="relu2", gated=False).forward(h.cuda().bfloat16()).cpu().numpy()
    close(got, O.squared_relu_expert(hh, hw["up"], hw["down"]), 3e-2, "squared relu, bf16")


@pytest.mark.parametrize("E,top,groups,keep", [(12, 3, 4, 2), (15, 2, 3, 1), (7, 7, 1, 1), (64, 5, 8, 3), (9, 1, 9, 4), (6, 2, 3, 3)])
def test_router_groups_by_their_two_best(seq, E, top, groups, keep):
    T, W = 33, 24
    h, rw = rnd(T, W, seed=E), rnd(E, W, seed=E + 1, sd=0.6)
    rt = {"experts": E, "top": top, "scale": 1.7, "groups": {"count": groups, "keep": keep}}
    want_ids, want_w = O.route(h.numpy().astype(np.float64), rw.numpy().astype(np.float64), rt)
    if groups > 1 and keep < groups and E // groups > 1:                 # the rule differs from "best single member" on these inputs
        s = O.sigmoid(h.numpy().astype(np.float64) @ rw.numpy().astype(np.float64).T).reshape(T, groups, -1)
        assert (s.max(-1).argmax(-1) != np.sort(s, -1)[..., -2:].sum(-1).argmax(-1)).any()
    z = seq.gemm(h.cuda(), rw.cuda())
    ids, wt = seq.route(z, None, top, groups, keep, "sigmoid", True, 1.7, "top2")
    assert (ids.cpu().numpy() == want_ids).all()
    close(wt.cpu().numpy(), want_w, 1e-5, "router weights")


@pytest.mark.parametrize("T", [1, 5, 70, 200])
def test_routed_experts_with_gated_shared_expert(seq, T):
    from krasis_b200.mixers import RoutedExperts
    W, E, F = 32, 10, 24
    mlp = moe(experts=E, top=3, groups=5, keep=3, ff=F, shared=40, scale=2.5)
    w = {"router": rnd(E, W, seed=1, sd=0.5), "shared.up": rnd(40, W, seed=2, sd=0.3), "shared.down": rnd(W, 40, seed=3, sd=0.2),
         "shared.sg": rnd(1, W, seed=4, sd=0.5)}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = rnd(F, W, seed=10 + e, sd=0.3), rnd(W, F, seed=30 + e, sd=0.2)
    h = rnd(T, W, seed=5)
    want = O.moe_ff(h.numpy().astype(np.float64), f64(w), mlp)
    gate = O.sigmoid(h.numpy().astype(np.float64) @ f64(w)["shared.sg"].T)
    assert T == 1 or gate.std() > 0.02
    rx = RoutedExperts(under(w), E, 0, 3, torch.float32, DEV, groups=5, keep=3, score="sigmoid", renorm=True, out_scale=2.5, gated=False,
                       act="relu2", group_score="top2")
    got = rx.forward(h.cuda()).cpu().numpy()
    close(got, want, 3e-5, f"{T} tokens")
    if T > 1:                                      # a row alone equals the row in the batch
        close(rx.forward(h[3:4].cuda()).cpu().numpy(), got[3:4].astype(np.float64), 1e-5, "row alone")


def test_norm_around_zero_and_residual_multiplier(seq):
    T, W = 7, 50
    x, y, wn = rnd(T, W, seed=1), rnd(T, W, seed=2), rnd(W, seed=3, sd=0.2)
    xg = x.cuda().clone()
    h = seq.residual_scale_rms(xg, y.cuda(), 0.3, norm=wn.cuda(), w_shift=1.0, eps=1e-3)
    xs = x.numpy().astype(np.float64) + 0.3 * y.numpy().astype(np.float64)
    close(xg.cpu().numpy(), xs, 1e-6, "residual sum")
    close(h.cpu().numpy(), O.norm_around_zero(xs, wn.numpy().astype(np.float64), 1e-3), 1e-6, "norm")
    seq.residual_scale_rms(xg, norm=wn.cuda(), w_shift=1.0, eps=1e-3, in_place=True)
    close(xg.cpu().numpy(), O.norm_around_zero(xs, wn.numpy().astype(np.float64), 1e-3), 1e-6, "norm in place")


# ------------------------------------------------------------------------------------------------ the whole model

def test_layer_trace_matches_oracle(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=1, page_size=4)
    tk = toks(29, raw["vocab"], 5)
    col = []
    want = O.forward(raw, w, tk, col)
    model.layer_trace = []
    got = run_portions(model, tk, [29])
    trace, model.layer_trace = model.layer_trace, None
    assert len(trace) == len(col) == 7                    # layers 1 and 2 run twice
    for i, (a, b) in enumerate(zip(trace, col)):
        close(a.cpu().numpy(), b, 2e-5, f"residual stream after layer run {i}")
    close(got, want, 4e-5, "logits")


def test_prefill_vs_decode_vs_portions(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=2, page_size=4)
    tk = toks(61, raw["vocab"], 9)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [61]), want, 4e-5, "whole prompt")
    close(run_portions(model, tk, []), want, 4e-5, "token by token")
    for cuts in ([2, 2, 2, 2], [3, 5, 7, 11, 13], [1, 4, 4, 4, 30], [59, 2], [31], [8, 8, 8], [7, 2, 7, 2]):
        close(run_portions(model, tk, cuts), want, 4e-5, f"portions {cuts}")


@pytest.mark.parametrize("loop", [None, (0, 5, 1), (0, 2, 3), (3, 5, 2), (2, 2, 4)])
def test_loop_spans(seq, loop):
    raw = model_cfg(default_layers(), loop=loop)
    model, w = build(raw, seed=21, page_size=4)
    tk = toks(33, raw["vocab"], 2)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [33]), want, 4e-5, "whole")
    close(run_portions(model, tk, [9, 2, 14]), want, 4e-5, "portions")


def test_unequal_batch_equals_each_alone(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=3, page_size=4)
    reqs = {"a": toks(37, 50, 1), "b": toks(5, 50, 2), "c": toks(22, 50, 3), "d": toks(1, 50, 4)}
    want = {k: O.forward(raw, w, v) for k, v in reqs.items()}
    s = sched(model, max_tokens=256)
    plan = [[("a", 9), ("b", 2), ("c", 22)], [("a", 1), ("b", 1), ("d", 1)], [("a", 20), ("b", 2)], [("a", 7)]]
    at, got = {k: 0 for k in reqs}, {k: [] for k in reqs}
    for step in plan:
        lg = s.step([(k, reqs[k][at[k]:at[k] + n], list(range(n))) for k, n in step]).cpu().numpy()
        o = 0
        for k, n in step:
            got[k].append(lg[o:o + n])
            o += n
            at[k] += n
    for k in reqs:
        assert at[k] == len(reqs[k])
        close(np.concatenate(got[k], 0), want[k], 4e-5, f"request {k} in a mixed batch")


def test_pages_and_slots_are_reused(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=4, page_size=4)
    s = sched(model, max_tokens=48, max_requests=2)             # 12 pages, 2 slots: every later request runs on used ones
    free0 = s.kv_cache.free_page_count
    for i in range(5):
        a, b = toks(23 + i, 50, 10 + i), toks(9 + 2 * i, 50, 20 + i)
        la = s.step([("a", a[:10], list(range(10))), ("b", b, list(range(len(b))))]).cpu().numpy()
        s.finish("b")
        lb = s.step([("a", a[10:], list(range(len(a) - 10)))]).cpu().numpy()
        s.finish("a")
        close(np.concatenate([la[:10], lb], 0), O.forward(raw, w, a), 4e-5, f"pass {i}, request a")
        close(la[10:], O.forward(raw, w, b), 4e-5, f"pass {i}, request b")
        assert s.kv_cache.free_page_count == free0 and s.state_pool.free_slot_count == 2
    with pytest.raises(RuntimeError):
        s.step([("x", toks(60, 50, 1), [])])                    # more pages than the pool has


def test_far_key_and_page_borders_with_peaked_scores(seq):
    """One attention layer whose keys use head 0's query projection, whose query and key convolutions keep the current token only and
    whose scores are scaled up: a token that appears once, far back, and again near the end meets its own key there across 300 positions
    and shares the softmax with it (its value differs: the value convolution mixes in the neighbours).  The oracle is checked to move by
    far more than the tolerance when that far token is replaced.  Pages of 64 and of 4 put the far key and the portion edges at
    different places in a page."""
    raw = model_cfg([A(attn(heads=2, kv_heads=1, dim=32, vdim=24, rot_dims=0, conv=3, scale=1.5, softcap=40.0), dense(ff=32))], vocab=40, loop=None)

    def tweak(w):
        w["l0.mix.k"], w["l0.mix.k.b"] = w["l0.mix.q"][:32].clone(), w["l0.mix.q.b"][:32].clone()
        w["l0.mix.q.conv"][:, :-1] = 0
        w["l0.mix.k.conv"], w["l0.mix.k.norm"] = w["l0.mix.q.conv"][:32].clone(), w["l0.mix.q.norm"][:32].clone()
    tk = toks(330, 39, 4)
    marks = (-12, -7, -1)
    tk[5] = 39
    for i in marks:
        tk[i] = 39
    for page in (64, 4):
        model, w = build(raw, seed=8, page_size=page, tweak=tweak)
        want = O.forward(raw, w, tk)
        gone = list(tk)
        gone[5] = 0
        moved = np.abs(O.forward(raw, w, gone) - want).max(-1) / np.abs(want).max()
        assert all(moved[i] > 1e-2 for i in marks), moved[list(marks)]
        close(run_portions(model, tk, [330], s=sched(model, 1024)), want, 5e-5, "whole prompt")
        close(run_portions(model, tk, [300], s=sched(model, 1024)), want, 5e-5, "decoded over a far key")
        close(run_portions(model, tk, [128, 2, 100, 64], s=sched(model, 1024)), want, 5e-5, "portions")


def test_recurrence_carries_the_first_token_through_long_decoding(seq):
    """Slow decays: token 0 still moves the last logits after 200 tokens, most of them decoded one by one."""
    raw = model_cfg([D(delta(heads=2, kv_heads=1, dim=32, vdim=32, conv=3), dense(ff=40)), D(delta(heads=2, kv_heads=2, dim=16, vdim=8, conv=2))], loop=(0, 1, 2))

    def tweak(w):
        for k in w:
            if k.endswith("A_log"):
                w[k] = w[k] - 4.0
    model, w = build(raw, seed=12, page_size=8, tweak=tweak)
    tk = toks(200, 50, 6)
    want = O.forward(raw, w, tk)
    other = [(tk[0] + 1) % 50] + tk[1:]
    assert np.abs(O.forward(raw, w, other)[-1] - want[-1]).max() > 1e-3 * np.abs(want).max()
    close(run_portions(model, tk, [5]), want, 5e-5, "195 decoded tokens")
    close(run_portions(model, tk, [64, 64, 64]), want, 5e-5, "portions, then decoded")


def test_first_tokens_and_single_token_requests(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=11, page_size=4)
    for n in (1, 2, 3):
        tk = toks(n, 50, n)
        close(run_portions(model, tk, [n]), O.forward(raw, w, tk), 4e-5, f"{n}-token request")
    s = sched(model)
    lg = s.step([("p", [7], [0]), ("q", [7], [0]), ("r", [3, 7], [1])]).cpu().numpy()
    close(lg[0], O.forward(raw, w, [7])[0], 4e-5, "one token")
    assert np.allclose(lg[0], lg[1], rtol=0, atol=1e-6)
    close(lg[2], O.forward(raw, w, [3, 7])[1], 4e-5, "second token")


@pytest.mark.parametrize("layers,loop", [
    ([A(attn(heads=1, kv_heads=1, dim=2, vdim=1, conv=1, rot_dims=2, softcap=0.0)), D(delta(heads=1, kv_heads=1, dim=1, vdim=1, conv=1), moe(experts=1, top=1, groups=1, keep=1, ff=3, shared=0))], (0, 2, 1)),
    ([D(delta(heads=5, kv_heads=5, dim=20, vdim=20, conv=2), moe(experts=8, top=4, groups=4, keep=3, ff=8, shared=8, scale=1.0)),
      A(attn(heads=10, kv_heads=5, dim=20, vdim=20, rot_dims=4, conv=7), moe(experts=9, top=2, groups=9, keep=2, ff=130, shared=0)),
      A(attn(heads=2, kv_heads=2, dim=34, vdim=130, rot_dims=6, base=10.0), dense(ff=7))], (1, 2, 3)),
])
def test_other_sizes_and_degenerate_values(seq, layers, loop):
    raw = model_cfg(layers, width=36, vocab=23, loop=loop, mult=1.0, logit_scale=1.0, eps=1e-3)
    model, w = build(raw, seed=13, page_size=2)
    tk = toks(27, 23, 8)
    want = O.forward(raw, w, tk)
    close(run_portions(model, tk, [27]), want, 5e-5, "whole")
    close(run_portions(model, tk, [4, 2, 9]), want, 5e-5, "portions")


def test_bfloat16_serving_close_to_oracle(seq):
    """bfloat16 weights, GEMM inputs and cache.  With dense feed-forwards every position is bounded.  With routed experts a choice
    between two experts whose scores differ by less than the rounding of bfloat16 may fall the other way; that moves the position a lot
    and, through the keys and the recurrent state, the ones after it, so there the bound is on the median position."""
    tk = toks(40, 50, 2)
    dense_layers = [dict(L, mlp=dense(ff=40) if L["mlp"] else None) for L in default_layers()]
    for layers, stat, what in ((dense_layers, np.max, "dense"), (default_layers(), np.median, "experts")):
        raw = model_cfg(layers)
        model, w = build(raw, dtype=torch.bfloat16, seed=14, page_size=4)
        want = O.forward(raw, w, tk)
        a, b = run_portions(model, tk, [40]), run_portions(model, tk, [9, 2, 13])

        def bound(got, ref, rel, name):
            err = stat(np.abs(got.astype(np.float64) - ref).max(-1)) / np.abs(ref).max()
            assert err <= rel, f"{what}, {name}: {err:.3e}"
        bound(a, want, 6e-2, "bf16 whole")
        bound(b, want, 6e-2, "bf16 portions")
        bound(b, a.astype(np.float64), 6e-2, "bf16: portions against whole")


def test_tensor_core_prefill_of_capped_attention_and_experts(seq):
    """bfloat16 with 128 query / key dims and 128 or 256 value dims: portions of 128 tokens or more run the tcgen05 attention core (the cap
    applied to its scores), long steps run the routed experts as grouped tcgen05 GEMMs.  Against the oracle and against the plain
    kernels on the same bf16 cache, with scores large enough for the cap to bite."""
    from krasis_b200.build import build as build_core
    build_core()
    for vdim, heads, kv_heads, cap in ((128, 2, 1, 4.0), (256, 4, 2, 2.5), (128, 2, 2, 0.0)):
        layers = [A(attn(heads=heads, kv_heads=kv_heads, dim=128, vdim=vdim, rot_dims=64, conv=3, scale=0.6, softcap=cap), dense(ff=64)),
                  D(delta(heads=2, kv_heads=1, dim=64, vdim=64), moe(experts=8, top=2, groups=4, keep=2, ff=64, shared=64))]
        raw = model_cfg(layers, width=64, loop=(0, 1, 2))
        model, w = build(raw, dtype=torch.bfloat16, seed=31)
        mixer, rx = model.layers[0]["mixer"], model.layers[1]["mlp"]
        assert mixer.tc_shape
        tk = toks(700, raw["vocab"], 16)
        want = O.forward(raw, w, tk)
        if cap:                                     # the cap must move the logits by far more than the tolerances below
            loose = json.loads(json.dumps(raw))
            loose["layers"][0]["mixer"]["softcap"] = 0.0
            assert np.abs(O.forward(loose, w, tk) - want).max() > 0.15 * np.abs(want).max()

        def most(got, ref, rel, what):              # a router choice may fall the other way in bfloat16: four positions out of five
            err = np.abs(got.astype(np.float64) - ref).max(-1) / np.abs(ref).max()
            assert np.quantile(err, 0.8) <= rel, f"{what}: {np.quantile(err, 0.8):.3e}"
        fast_whole = run_portions(model, tk, [700], s=sched(model, 1024))
        fast_parts = run_portions(model, tk, [130, 257, 128, 150], s=sched(model, 1024))          # then 35 single tokens through the plain kernels
        mixer.tc_min_portion, rx.tc_min_rows_per_expert = 1 << 30, 1 << 30
        plain = run_portions(model, tk, [700], s=sched(model, 1024))
        mixer.tc_min_portion, rx.tc_min_rows_per_expert = 128, 16
        most(plain, want, 5e-2, f"cap {cap}: plain kernels against the oracle")
        most(fast_whole, want, 5e-2, f"cap {cap}: tensor-core prefill against the oracle")
        most(fast_whole, plain.astype(np.float64), 3e-2, f"cap {cap}: tensor-core prefill against the plain kernels")
        most(fast_parts, plain.astype(np.float64), 3e-2, f"cap {cap}: tensor-core portions against the plain kernels")


def test_greedy_generation_through_the_entry_point(seq):
    """Scheduler.generate (admission, portions under a token budget, decode beside prefill, slot and page reuse) against greedy
    decoding with the oracle.  Steps whose two best logits are closer than the comparison tolerance end the comparison of a prompt."""
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=9, page_size=4)
    prompts = [toks(n, 50, 50 + n) for n in (19, 3, 33, 8, 1, 12)]
    s = sched(model, max_tokens=160, max_requests=3)
    outs = s.generate(prompts, max_new_tokens=12, step_tokens=16)
    assert s.kv_cache.free_page_count == 40 and s.state_pool.free_slot_count == 3 and not s.live
    checked = 0
    for p, out in zip(prompts, outs):
        assert len(out) == 12
        seqn = list(p)
        for tok in out:
            lg = O.forward(raw, w, seqn)[-1]
            top = np.sort(lg)[-2:]
            if top[1] - top[0] < 1e-3 * np.abs(lg).max():
                break
            assert tok == int(np.argmax(lg))
            seqn.append(tok)
            checked += 1
    assert checked >= 40


def test_decode_steps_replayed_from_cuda_graphs_equal_eager_steps(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=17, page_size=4)
    a, b = toks(70, 50, 1), toks(60, 50, 2)
    outs = []
    for graphs in (False, True):
        s = sched(model, max_tokens=512, max_requests=3, cuda_graphs=graphs)
        got = [s.step([("a", a[:20], [19]), ("b", b[:5], [4])])]
        for i in range(40):
            got.append(s.step([("a", [a[20 + i]], [0]), ("b", [b[5 + i]], [0])]))
        s.finish("b")
        for i in range(8):
            got.append(s.step([("a", [a[60 + i]], [0])]))
        outs.append([g.clone() for g in got])
        if graphs:
            assert sum(1 for v in s._graphs.values() if v) >= 2
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    close(outs[1][-1][0].cpu().numpy(), O.forward(raw, w, a[:68])[67], 5e-5, "last decoded token of request a")


def test_registry_loads_a_checkpoint_directory_and_the_trace_runner_replays_it(seq, tmp_path, monkeypatch, capsys):
    import io
    import sys
    from krasis_b200 import trace_runner
    from krasis_b200.gurozen import GurozenConfig, random_weights
    from krasis_b200.registry import architecture_of, load_model
    raw = model_cfg(default_layers())
    w = random_weights(GurozenConfig.from_dict(raw), 10)
    header, blobs, off = {}, [], 0
    for k, v in w.items():
        b = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert architecture_of(str(tmp_path)) == "Gurozen"
    tk = toks(25, 50, 14)
    want = O.forward(raw, {k: v.numpy().astype(np.float64) for k, v in w.items()}, tk)
    close(run_portions(load_model(str(tmp_path), dtype=torch.float32), tk, [25]), want, 4e-5, "loaded checkpoint")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tk[:10], "want": [0, 9]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": tk[10:12], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": tk[12:], "want": [12]}, {"id": "y", "tokens": tk[:3], "want": [2]}], "end": ["x", "y"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out = tmp_path / "out"
    assert trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), want[[0, 9]], 4e-5, "step 0")
    close(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1), want[[24, 2]], 4e-5, "step 2")
