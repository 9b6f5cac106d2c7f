"""Zaronex on the GPU against the plain float64 oracle (tests/oracle_zaronex.py): each mechanism alone, then the whole model through
the scheduler — prefill against decoding, portions down to two tokens, unequal batches, reuse of pages and slots, far keys, page
borders and the edges of windows and pooled blocks with peaked scores, the first tokens of a sequence, long decoding of the
recurrences, odd sizes, and greedy generation through the generation entry point.  Small random configurations made here; none of
them is a shipped model's."""
import json
import struct

import numpy as np
import pytest
import torch

from tests import oracle_zaronex as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EPS = 1e-5


@pytest.fixture(scope="module")
def seq():
    from krasis_b200.build import build_seq
    build_seq()
    from krasis_b200 import seqops
    seqops.load()
    return seqops


# ------------------------------------------------------------------------------------------------ configurations
def latent(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=12, q_rank=9, size=7, base=300.0, scale=0.3, factor=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
         "mask": {"size": size}, "rot": {"base": base, "dims": rot_dim}}
    if factor:
        m["rot"]["scaling"] = {"factor": factor}
    return m


def left(heads=4, kv_heads=2, dim=12, vdim=10, size=9, pool=None, rot_dims=8, base=500.0, scale=0.4, factor=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}}
    if pool:
        m["mask"]["pool"] = pool
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
        if factor:
            m["rot"]["scaling"] = {"factor": factor}
    return m


def gla(heads=3, dim=6, vdim=10, tau=4.0):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}


def scan(inner=20, state=5, dt_rank=3, conv=4):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def LA(m=None, mlp="dense"):
    return {"type": "latent_attention", "mixer": m or latent(), "mlp": dense() if mlp == "dense" else mlp}


def P1(l=None, r=None, mlp="dense"):
    return {"type": "parallel", "mixer": {"left": l or left(pool=4), "right": r or gla()}, "mlp": dense() if mlp == "dense" else mlp}


def P2(l=None, r=None, mlp="dense"):
    return {"type": "parallel_2", "mixer": {"left": l or left(kv_heads=4, rot_dims=6, factor=3.0, size=11), "right": r or scan()},
            "mlp": dense() if mlp == "dense" else mlp}


def model_cfg(layers, width=40, vocab=50, eps=EPS):
    return {"architecture": "Zaronex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def default_layers():
    return [P1(), LA(), P2(mlp=None), LA(latent(heads=2, dim=4, rot_dim=8, vdim=6, kv_rank=5, q_rank=16, size=30, factor=2.0), mlp=None),
            P1(left(heads=2, kv_heads=1, dim=16, vdim=24, size=5, pool=7, rot_dims=16), gla(heads=1, dim=40, vdim=36, tau=1.0), dense(ff=17)),
            P2(left(heads=6, kv_heads=3, dim=8, vdim=4, size=64, rot_dims=0), scan(inner=33, state=40, dt_rank=1, conv=1))]


def build(raw, dtype=torch.float32, seed=0, page_size=None, tweak=None):
    from krasis_b200.zaronex import ZaronexConfig, ZaronexModel, random_weights
    cfg = ZaronexConfig.from_dict(raw)
    w = random_weights(cfg, seed)
    if tweak:
        tweak(w)
    model = ZaronexModel(cfg, w, dtype=dtype)
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
def left_weights(m, W, seed, kind):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"o": rnd(W, H * dv, seed=seed, sd=0.2)}
    for i, (n, rows) in enumerate((("q", H * d), ("k", G * d), ("v", G * dv))):
        w[n] = rnd(rows, W, seed=seed + 1 + i, sd=W ** -0.5 * 2)
        if kind == "parallel":
            w[n + ".b"] = rnd(rows, seed=seed + 4 + i, sd=0.3)
        elif n != "v":
            w[n + ".norm"] = 1 + rnd(rows, seed=seed + 10 + i, sd=0.3)
    if kind == "parallel":
        w["sink"] = rnd(H, seed=seed + 20, sd=1.5)
        w["g"] = rnd(H * dv, W, seed=seed + 21, sd=W ** -0.5 * 2)
    return w


def make_left(m, w, kind, dtype=torch.float32):
    from krasis_b200.mixers import MultiMapAttention
    halves, rot_values = (True, False) if kind == "parallel" else (False, True)
    dims, base, factor = O.rot_of(m)
    return MultiMapAttention(under(w), m["heads"], m["kv_heads"], 1, m["dim"], m["vdim"], m["scale"], EPS, dtype, torch.device(DEV),
                             window=m["mask"]["size"], rot_dims=dims, rot_base=base, rot_factor=factor, rot_half=halves,
                             norm_whole="q.norm" in w, pool=m["mask"].get("pool") or 0, rot_values=rot_values, gate_per_element=True)


class OneSequence:
    """A cache, a state pool and the tables of one sequence fed in portions, for a mixer on its own."""

    def __init__(self, seq, dims, page_size, tokens, dtype=torch.float32, register=None, slot=1):
        from krasis_b200.attention import HeadKVCache, RecurrentStatePool, SequenceKVState
        self.seq, self.page_size, self.slot = seq, page_size, slot
        self.kv = HeadKVCache([dims], DEV, max_pages=(tokens + page_size - 1) // page_size + 2, dtype=dtype, page_size=page_size)
        self.pool = RecurrentStatePool(3, DEV)
        self.state = register(self.pool) if register else None
        self.st = SequenceKVState(self.kv)

    def portions(self, T, cuts):
        at = 0
        for n in list(cuts) + [1] * (T - sum(cuts)):
            self.st.ensure_capacity(n)
            yield at, n, self.seq.StepTables([([0] * n, self.st.seq_len, self.slot, self.st.pages)], torch.device(DEV))
            self.st.advance(n)
            at += n


def run_left(seq, mixer, h, cuts, page_size=4):
    one = OneSequence(seq, mixer.cache_dims(), page_size, h.shape[0], mixer.dtype)
    kc, vc = one.kv.get_layer_caches(0)
    out = []
    for at, n, tb in one.portions(h.shape[0], cuts):
        out.append(mixer.forward(h[at:at + n].to(DEV, mixer.dtype).contiguous(), tb, kc, vc, page_size,
                                 pooled=one.kv.get_pooled_caches(0)).cpu().numpy())
    return np.concatenate(out, 0)


CUTS = ([41], [], [2, 2, 5, 17], [30, 2], [3, 1, 1, 9, 2])


@pytest.mark.parametrize("m", [left(pool=4), left(heads=2, kv_heads=2, dim=32, vdim=8, size=5, pool=7, rot_dims=32),
                               left(heads=8, kv_heads=1, dim=6, vdim=70, size=12, pool=3, rot_dims=2),
                               left(heads=3, kv_heads=3, dim=10, vdim=33, size=100, pool=2, rot_dims=0, scale=0.7),
                               left(heads=4, kv_heads=2, dim=16, vdim=16, size=1, pool=1, rot_dims=16, base=50.0, factor=3.0),
                               left(heads=2, kv_heads=1, dim=8, vdim=8, size=6, pool=None)])
def test_window_attention_with_pooled_blocks_sink_and_gate(seq, m):
    W, T = 48, 41
    w = left_weights(m, W, seed=3, kind="parallel")
    h = rnd(T, W, seed=1)
    want = O.grouped_window_attention(h.numpy().astype(np.float64), f64(w), dict(m, halves=True), EPS, list(range(T)))
    mixer = make_left(m, w, "parallel")
    for cuts in CUTS:
        close(run_left(seq, mixer, h, cuts), want, 3e-5, f"portions {cuts}")
    loose = dict(f64(w))
    del loose["sink"]                                  # the sink must matter by far more than the tolerance
    other = O.grouped_window_attention(h.numpy().astype(np.float64), loose, dict(m, halves=True), EPS, list(range(T)))
    assert np.abs(other - want).max() > 1e-2 * np.abs(want).max()


@pytest.mark.parametrize("m", [left(kv_heads=4, rot_dims=6, factor=3.0, size=11), left(heads=2, kv_heads=1, dim=16, vdim=34, size=4, rot_dims=16),
                               left(heads=6, kv_heads=3, dim=8, vdim=4, size=64, rot_dims=0),
                               left(heads=1, kv_heads=1, dim=4, vdim=2, size=3, rot_dims=4, base=7.0, factor=8.0)])
def test_window_attention_with_whole_norms_and_rotated_values(seq, m):
    W, T = 48, 41
    w = left_weights(m, W, seed=5, kind="parallel_2")
    h = rnd(T, W, seed=2)
    want = O.grouped_window_attention(h.numpy().astype(np.float64), f64(w), dict(m, halves=False), EPS, list(range(T)), value_turn=True)
    mixer = make_left(m, w, "parallel_2")
    for cuts in CUTS:
        close(run_left(seq, mixer, h, cuts), want, 3e-5, f"portions {cuts}")
    plain = O.grouped_window_attention(h.numpy().astype(np.float64), f64(w), dict(m, halves=False), EPS, list(range(T)), value_turn=False)
    assert np.abs(plain - want).max() > 1e-2 * np.abs(want).max()          # the turning of the values shows


def peaked_inputs(T, W, d, marks, seed=0):
    """Hidden states for identity-like q / k projections such that the query at the last position scores the marked positions far above
    all others: h[j] = a_j u for marked j (u the last token's direction), small noise elsewhere.  Returns (h, |u|^2)."""
    h = rnd(T, W, seed=seed, sd=0.05)
    u = torch.zeros(W)
    u[:d] = rnd(d, seed=seed + 1).abs() + 0.5
    h[T - 1] = u
    for j, a in marks.items():
        h[j] = (a * u + rnd(W, seed=seed + 2 + j, sd=0.05)).to(torch.bfloat16).float()
    return h, float((u * u).sum())


@pytest.mark.parametrize("size,pool,page", [(9, 4, 4), (6, 5, 8), (16, 3, 4), (8, 8, 8)])
def test_edges_of_the_window_and_of_pooled_blocks_with_peaked_scores(seq, size, pool, page):
    """The last token's query is made to score a few positions far above the rest: the first and last position inside the window, the
    last position that has left it, one position of the newest block that is seen, one of the block that is not seen yet, and a
    far block.  A window or block rule that is off by one moves the output by much more than the tolerance — in a prompt and when the
    last token is decoded alone."""
    W, d, dv, T = 32, 8, 6, 61
    m = left(heads=2, kv_heads=1, dim=d, vdim=dv, size=size, pool=pool, rot_dims=0, scale=1.0)
    i = T - 1
    seen = O.pooled_blocks(i, size, pool)
    newest, unseen = seen[-1], seen[-1] + 1
    # block members are scaled by the block length so that the block's mean key scores like a single marked position
    marks = {1: 0.7 * pool, newest * pool: 0.6 * pool, newest * pool + pool - 1: 0.9 * pool, i - 1: 1.2, i - size + 1: 1.5, i - size: 1.7}
    if unseen * pool + pool - 1 < i - size + 1:            # a block between the seen ones and the window
        marks[unseen * pool] = 1.6 * pool
    w = left_weights(m, W, seed=11, kind="parallel")
    eye = torch.zeros(2 * d, W)
    eye[:d, :d] = torch.eye(d)
    eye[d:, :d] = torch.eye(d)
    w["q"], w["k"] = eye.clone(), eye[:d].clone()
    w["q.b"], w["k.b"] = torch.zeros(2 * d), torch.zeros(d)
    w["sink"] = torch.tensor([2.0, -1.0])
    h, uu = peaked_inputs(T, W, d, marks, seed=4)
    m["scale"] = 3.0 / uu                                   # a mark a scores about 3 a, everything else about 0
    h64 = h.numpy().astype(np.float64)
    want = O.grouped_window_attention(h64, f64(w), dict(m, halves=True), EPS, list(range(T)))
    for wrong in (dict(m, mask={"size": size + 1, "pool": pool}), dict(m, mask={"size": size - 1, "pool": pool}) if size > 1 else None,
                  dict(m, mask={"size": size})):
        if wrong:
            off = O.grouped_window_attention(h64, f64(w), dict(wrong, halves=True), EPS, list(range(T)))
            assert np.abs(off[i] - want[i]).max() > 3e-2 * np.abs(want[i]).max()
    mixer = make_left(m, w, "parallel")
    for cuts in ([T], [T - 1], [T - 3, 2], [5, 2, 2, 40]):
        close(run_left(seq, mixer, h, cuts, page_size=page)[i], want[i], 3e-5, f"portions {cuts}")


def latent_weights(m, W, seed):
    H, dn, dr, dv, r, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    return {"dq": rnd(rq, W, seed=seed, sd=W ** -0.5 * 2), "dq.norm": 1 + rnd(rq, seed=seed + 1, sd=0.3), "uq": rnd(H * (dn + dr), rq, seed=seed + 2, sd=rq ** -0.5 * 2),
            "dkv": rnd(r + dr, W, seed=seed + 3, sd=W ** -0.5 * 2), "dkv.norm": 1 + rnd(r, seed=seed + 4, sd=0.3),
            "uk": rnd(H * dn, r, seed=seed + 5, sd=r ** -0.5 * 2), "uv": rnd(H * dv, r, seed=seed + 6, sd=r ** -0.5),
            "g": rnd(H * dv, W, seed=seed + 7, sd=W ** -0.5 * 2), "o": rnd(W, H * dv, seed=seed + 8, sd=0.2)}


@pytest.mark.parametrize("m", [latent(), latent(heads=2, dim=4, rot_dim=8, vdim=6, kv_rank=5, q_rank=16, size=30, factor=2.0),
                               latent(heads=9, dim=16, rot_dim=2, vdim=40, kv_rank=24, q_rank=3, size=1),
                               latent(heads=1, dim=1, rot_dim=4, vdim=8, kv_rank=8, q_rank=8, size=100)])
def test_latent_attention_with_query_latent_window_and_gate(seq, m):
    from krasis_b200.mixers import WindowLatentAttention, rotary_table
    W, T = 48, 41
    w = latent_weights(m, W, seed=7)
    h = rnd(T, W, seed=3)
    want = O.latent_attention(h.numpy().astype(np.float64), f64(w), m, EPS, list(range(T)))
    dims, base, factor = O.rot_of(m)
    mixer = WindowLatentAttention(under(w), m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["scale"], m["mask"]["size"], dims,
                                  base, None, EPS, torch.float32, torch.device(DEV), rot_freq=rotary_table(dims, base, factor))
    for cuts in CUTS:
        one = OneSequence(seq, mixer.cache_dims(), 4, T)
        ckv, kr = one.kv.get_layer_caches(0)
        got = np.concatenate([mixer.forward(h[at:at + n].to(DEV).contiguous(), tb, ckv, kr, 4).cpu().numpy() for at, n, tb in one.portions(T, cuts)], 0)
        close(got, want, 3e-5, f"portions {cuts}")


def gla_weights(m, W, seed, rank=5):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    return {"q": rnd(H * dk, W, seed=seed, sd=W ** -0.5 * 2), "k": rnd(H * dk, W, seed=seed + 1, sd=W ** -0.5 * 2),
            "v": rnd(H * dv, W, seed=seed + 2, sd=W ** -0.5 * 2), "g": rnd(H * dv, W, seed=seed + 3, sd=W ** -0.5 * 2),
            "a1": rnd(rank, W, seed=seed + 4, sd=W ** -0.5 * 2), "a2": rnd(H * dk, rank, seed=seed + 5), "a2.b": rnd(H * dk, seed=seed + 6) + 2.0,
            "norm": 1 + rnd(dv, seed=seed + 7, sd=0.3), "o": rnd(W, H * dv, seed=seed + 8, sd=0.2)}


@pytest.mark.parametrize("m", [gla(), gla(heads=1, dim=40, vdim=36, tau=1.0), gla(heads=2, dim=128, vdim=32, tau=16.0),
                               gla(heads=5, dim=1, vdim=3, tau=2.5), gla(heads=2, dim=70, vdim=130, tau=8.0),
                               gla(heads=3, dim=32, vdim=96, tau=2.0), gla(heads=2, dim=64, vdim=64, tau=16.0), gla(heads=1, dim=256, vdim=32, tau=5.0)])
def test_gated_linear_attention_alone(seq, m):
    from krasis_b200.mixers import GatedLinearAttention
    W, T = 48, 41
    w = gla_weights(m, W, seed=13)
    h = rnd(T, W, seed=5)
    want = O.gated_linear_attention(h.numpy().astype(np.float64), f64(w), m, EPS)
    mixer = GatedLinearAttention(under(w), m["heads"], m["dim"], m["vdim"], m["tau"], EPS, torch.float32, torch.device(DEV))
    assert mixer.register_state_kernel == (m["dim"] in (32, 64, 128, 256) and m["vdim"] % 32 == 0)      # both forms of the kernel are covered
    for cuts in CUTS:
        one = OneSequence(seq, (1, 1), 4, T, register=mixer.register_state)
        got = np.concatenate([mixer.forward(h[at:at + n].to(DEV).contiguous(), tb, one.state).cpu().numpy() for at, n, tb in one.portions(T, cuts)], 0)
        close(got, want, 3e-5, f"portions {cuts}")


def scan_weights(m, W, seed):
    C, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
    return {"in": rnd(2 * C, W, seed=seed, sd=W ** -0.5 * 2), "conv": rnd(C, K, seed=seed + 1, sd=0.6), "conv.b": rnd(C, seed=seed + 2, sd=0.3),
            "x": rnd(R + 2 * N, C, seed=seed + 3, sd=C ** -0.5 * 2), "dt": rnd(C, R, seed=seed + 4), "dt.b": rnd(C, seed=seed + 5) - 1.0,
            "A_log": rnd(C, N, seed=seed + 6, sd=0.7), "D": rnd(C, seed=seed + 7), "o": rnd(W, C, seed=seed + 8, sd=0.2)}


@pytest.mark.parametrize("m", [scan(), scan(inner=33, state=40, dt_rank=1, conv=1), scan(inner=64, state=16, dt_rank=4, conv=2),
                               scan(inner=7, state=1, dt_rank=2, conv=9), scan(inner=12, state=130, dt_rank=5, conv=3)])
def test_selective_scan_alone(seq, m):
    from krasis_b200.mixers import SelectiveScan
    W, T = 48, 41
    w = scan_weights(m, W, seed=17)
    h = rnd(T, W, seed=6)
    want = O.selective_scan(h.numpy().astype(np.float64), f64(w), m)
    mixer = SelectiveScan(under(w), m["inner"], m["state"], m["dt_rank"], m["conv"], torch.float32, torch.device(DEV))
    for cuts in CUTS:
        one = OneSequence(seq, (1, 1), 4, T, register=mixer.register_state)
        got = np.concatenate([mixer.forward(h[at:at + n].to(DEV).contiguous(), tb, *one.state).cpu().numpy() for at, n, tb in one.portions(T, cuts)], 0)
        close(got, want, 3e-5, f"portions {cuts}")


def test_side_by_side_merge_and_depth_average(seq):
    T, W = 9, 37
    a, b, wa, wb = rnd(T, W, seed=1), rnd(T, W, seed=2, sd=3.0), 1 + rnd(W, seed=3, sd=0.3), 1 + rnd(W, seed=4, sd=0.3)
    got = seq.branch_merge(a.to(DEV), b.to(DEV), wa.to(DEV), wb.to(DEV), EPS, 0.5).cpu().numpy()
    close(got, O.side_by_side(a.numpy().astype(np.float64), b.numpy().astype(np.float64), {"left.out": wa.numpy(), "right.out": wb.numpy()}, EPS), 1e-6)
    n = 5
    stack = rnd(n, T, W, seed=5).to(DEV)
    keep = stack.clone()
    x, y, coef, nw = rnd(T, W, seed=6), rnd(T, W, seed=7), rnd(n, seed=8), 1 + rnd(W, seed=9, sd=0.3)
    xd = x.to(DEV).clone()
    h = seq.depth_mix(stack, n, coef.to(DEV), xd, y.to(DEV), norm=nw.to(DEV), out_dtype=torch.float32, eps=EPS)
    newest = (x + y).numpy().astype(np.float64)
    want = sum(coef[j].item() * keep[j].cpu().numpy().astype(np.float64) for j in range(n - 1)) + coef[n - 1].item() * newest
    close(stack[n - 1].cpu().numpy(), newest, 1e-7, "the newest result joins the stack")
    assert torch.equal(stack[:n - 1], keep[:n - 1])
    close(xd.cpu().numpy(), want, 1e-6, "weighted sum")
    close(h.cpu().numpy(), O.rms_norm(want, nw.numpy().astype(np.float64), EPS), 1e-6, "its norm")


# ------------------------------------------------------------------------------------------------ the model through the scheduler
def test_prefill_against_the_oracle_layer_by_layer(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=1, page_size=4)
    tk = toks(75, raw["vocab"], 3)
    trace = []
    want = O.forward(raw, w, tk, trace)
    model.layer_trace = []
    got = run_portions(model, tk, [75])
    for i, (a, b) in enumerate(zip(model.layer_trace, trace)):
        close(a.cpu().numpy(), b, 3e-5, f"stream after layer {i} ({raw['layers'][i]['type']})")
    model.layer_trace = None
    close(got, want, 5e-5, "logits")


def test_decoding_and_portions_equal_prefill(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=2, page_size=4)
    tk = toks(70, raw["vocab"], 4)
    want = O.forward(raw, w, tk)
    for cuts in ([], [2] * 35, [2, 3, 4, 5, 6, 7, 8, 9], [33, 2, 2, 31], [69]):
        close(run_portions(model, tk, cuts), want, 5e-5, f"portions {cuts}")


def test_first_tokens_of_a_sequence(seq):
    """One, two and three tokens: windows, blocks and recurrences that have nothing behind them yet."""
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=3, page_size=4)
    for n in (1, 2, 3):
        tk = toks(n, raw["vocab"], 20 + n)
        want = O.forward(raw, w, tk)
        close(run_portions(model, tk, [n]), want, 5e-5, f"{n} tokens at once")
        close(run_portions(model, tk, []), want, 5e-5, f"{n} tokens one by one")


def test_unequal_requests_in_one_batch_equal_each_alone(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=4, page_size=4)
    a, b, c = toks(50, 50, 5), toks(23, 50, 6), toks(9, 50, 7)
    want = {k: O.forward(raw, w, v) for k, v in (("a", a), ("b", b), ("c", c))}
    s = sched(model, max_tokens=256)
    got = {"a": [], "b": [], "c": []}

    def step(*parts):
        out = s.step([(rid, t, list(range(len(t)))) for rid, t in parts]).cpu().numpy()
        at = 0
        for rid, t in parts:
            got[rid].append(out[at:at + len(t)])
            at += len(t)
    step(("a", a[:30]), ("b", b[:2]))
    step(("b", b[2:4]), ("a", a[30:31]), ("c", c[:7]))
    step(("c", c[7:8]), ("a", a[31:32]), ("b", b[4:21]))
    step(("a", a[32:]), ("c", c[8:]))
    step(("b", b[21:]),)
    for k in got:
        close(np.concatenate(got[k], 0), want[k], 5e-5, f"request {k}")


def test_pages_and_slots_are_reused(seq):
    """A pool of a few pages and two slots serves five requests one after another and two at a time; what a finished request left in its
    pages, pooled rows and state slots must not reach the next one."""
    raw = model_cfg(default_layers())
    model, w = build(raw, seed=5, page_size=4)
    s = sched(model, max_tokens=64, max_requests=2)
    reqs = [toks(n, 50, 30 + n) for n in (29, 31, 14, 30, 7)]
    for i, tk in enumerate(reqs):
        close(run_portions(model, tk, [len(tk) // 2, 2], s=s, rid=i), O.forward(raw, w, tk), 5e-5, f"request {i}")
        assert s.kv_cache.free_page_count == 16 and s.state_pool.free_slot_count == 2
    x, y = reqs[2], reqs[4]
    out = s.step([("x", x, [len(x) - 1]), ("y", y, [len(y) - 1])]).cpu().numpy()
    close(out[0], O.forward(raw, w, x)[-1], 5e-5, "two at a time, first")
    close(out[1], O.forward(raw, w, y)[-1], 5e-5, "two at a time, second")


def test_long_decoding_of_the_recurrences_and_windows(seq):
    raw = model_cfg([P1(left(size=20, pool=6)), P2(), LA()])
    model, w = build(raw, seed=6)
    tk = toks(330, raw["vocab"], 8)
    want = O.forward(raw, w, tk)
    got = run_portions(model, tk, [10])                     # 320 tokens decoded one by one, across five pages of 64
    close(got, want, 1e-4, "330 tokens")
    close(got[-1], want[-1], 1e-4, "the last token")


def test_bfloat16_serving_stays_near_the_oracle(seq):
    raw = model_cfg(default_layers())
    model, w = build(raw, dtype=torch.bfloat16, seed=7, page_size=8)
    tk = toks(90, raw["vocab"], 9)
    want = O.forward(raw, w, tk)
    whole = run_portions(model, tk, [90])
    parts = run_portions(model, tk, [40, 2, 17])
    for got, what in ((whole, "prefill"), (parts, "portions and decoding")):
        err = np.abs(got.astype(np.float64) - want).max(-1) / np.abs(want).max()
        assert np.quantile(err, 0.9) <= 4e-2, f"{what}: {np.quantile(err, 0.9):.3e}"


def test_other_sizes_than_any_shipped_model(seq):
    """Every size that tends to coincide in shipped configurations is made different here, or 1: heads equal to key/value heads, one
    head, a latent larger than the width, more pooled rows than a page has tokens, a window of one, no feed-forward at all."""
    layers = [LA(latent(heads=1, dim=2, rot_dim=2, vdim=2, kv_rank=30, q_rank=1, size=1), mlp=None),
              P1(left(heads=1, kv_heads=1, dim=2, vdim=2, size=1, pool=1, rot_dims=2), gla(heads=1, dim=1, vdim=1, tau=0.5), mlp=None),
              P2(left(heads=5, kv_heads=5, dim=6, vdim=6, size=2, rot_dims=6, factor=1.5), scan(inner=3, state=3, dt_rank=3, conv=2), dense(ff=1)),
              P1(left(heads=6, kv_heads=2, dim=4, vdim=8, size=3, pool=9, rot_dims=4), gla(heads=4, dim=9, vdim=5, tau=3.0))]
    raw = model_cfg(layers, width=22, vocab=13)
    model, w = build(raw, seed=8, page_size=4)
    tk = toks(45, 13, 10)
    want = O.forward(raw, w, tk)
    for cuts in ([45], [], [7, 2, 2]):
        close(run_portions(model, tk, cuts), want, 5e-5, f"portions {cuts}")


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
    from krasis_b200.registry import architecture_of, load_model
    from krasis_b200.zaronex import ZaronexConfig, random_weights
    raw = model_cfg(default_layers())
    w = random_weights(ZaronexConfig.from_dict(raw), 10)
    header, blobs, off = {}, [], 0
    for k, v in w.items():
        b = v.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(v.shape), "data_offsets": [off, off + len(b)]}
        blobs.append(b)
        off += len(b)
    hj = json.dumps(header).encode()
    (tmp_path / "model.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (tmp_path / "config.json").write_text(json.dumps(raw))
    assert architecture_of(str(tmp_path)) == "Zaronex"
    tk = toks(25, 50, 14)
    want = O.forward(raw, {k: v.numpy().astype(np.float64) for k, v in w.items()}, tk)
    close(run_portions(load_model(str(tmp_path), dtype=torch.float32), tk, [25]), want, 5e-5, "loaded checkpoint")
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": tk[:10], "want": [0, 9]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": tk[10:12], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": tk[12:], "want": [12]}, {"id": "y", "tokens": tk[:3], "want": [2]}], "end": ["x", "y"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    out = tmp_path / "out"
    assert trace_runner.main(["--model", str(tmp_path), "--dtype", "float32", "--out", str(out), "--max-tokens", "128"]) == 0
    assert [ln for ln in capsys.readouterr().out.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "1.f32").exists()
    close(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1), want[[0, 9]], 5e-5, "step 0")
    close(np.fromfile(out / "2.f32", dtype="<f4").reshape(2, -1), want[[24, 2]], 5e-5, "step 2")


def test_tensor_core_prefill_with_sink_pooled_blocks_and_rotated_values(seq):
    """bfloat16 with 128 query / key dims and 128 or 256 value dims: portions of 128 tokens or more run the tcgen05 attention core — the
    sink inside it, the pooled blocks as a second pass joined by the two log-sum-exps, the values rotated before the cache and turned
    back after the core.  Against the oracle and against the plain kernels on the same bf16 cache."""
    from krasis_b200.build import build as build_core
    build_core()
    # (a) one mixer with peaked scores: the last token scores members of the newest seen block, of a far block and of its window far above
    # the rest, so that a lost or mis-weighted block moves the output by far more than the bf16 tolerance
    W = d = 128
    T, size, pool = 400, 100, 32
    m = left(heads=2, kv_heads=1, dim=d, vdim=128, size=size, pool=pool, rot_dims=0, scale=1.0)
    i = T - 1
    newest = O.pooled_blocks(i, size, pool)[-1]
    marks = {3: 0.7 * pool, newest * pool + 5: 0.6 * pool, newest * pool + pool - 1: 0.9 * pool, i - 1: 1.2, i - size + 1: 1.5, i - size: 1.7}
    w = left_weights(m, W, seed=21, kind="parallel")
    w["q"], w["k"] = torch.cat([torch.eye(d), torch.eye(d)], 0), torch.eye(d)
    w["q.b"], w["k.b"] = torch.zeros(2 * d), torch.zeros(d)
    w["sink"] = torch.tensor([7.0, 0.5])
    h, uu = peaked_inputs(T, W, d, marks, seed=6)
    m["scale"] = 5.0 / uu                                   # a mark a scores about 5 a: the marked keys outweigh the hundred plain ones
    h64 = h.numpy().astype(np.float64)
    want = O.grouped_window_attention(h64, f64(w), dict(m, halves=True), EPS, list(range(T)))
    for wrong in (dict(m, mask={"size": size}), dict(m, mask={"size": size + 1, "pool": pool})):
        off = O.grouped_window_attention(h64, f64(w), dict(wrong, halves=True), EPS, list(range(T)))
        assert np.abs(off[i] - want[i]).max() > 0.1 * np.abs(want[i]).max()
    nosink = dict(f64(w))
    del nosink["sink"]
    assert np.abs(O.grouped_window_attention(h64, nosink, dict(m, halves=True), EPS, list(range(T)))[i] - want[i]).max() > 0.1 * np.abs(want[i]).max()
    mixer = make_left(m, w, "parallel", dtype=torch.bfloat16)
    assert mixer.tc_shape
    fast = run_left(seq, mixer, h, [T], page_size=8)
    parts = run_left(seq, mixer, h, [130, 2, T - 132], page_size=8)
    mixer.tc_min_portion = 1 << 30
    plain = run_left(seq, mixer, h, [T], page_size=8)
    scale_ = np.abs(want).max()
    for got, what in ((plain, "plain kernels"), (fast, "tensor-core prefill"), (parts, "tensor-core portions")):
        err = np.abs(got.astype(np.float64) - want).max(-1) / scale_
        assert err[i] <= 3e-2 and np.quantile(err, 0.9) <= 3e-2, f"{what}: last token {err[i]:.3e}, 90th percentile {np.quantile(err, 0.9):.3e}"
    # (b) the whole model
    layers = [P1(left(heads=2, kv_heads=1, dim=128, vdim=128, size=200, pool=48, rot_dims=64), gla(heads=2, dim=64, vdim=64)),
              P2(left(heads=4, kv_heads=2, dim=128, vdim=256, size=300, rot_dims=32, factor=2.0), scan(inner=64, state=16, dt_rank=8, conv=4)),
              LA(latent(heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=64, q_rank=64, size=250, scale=0.07))]
    raw = model_cfg(layers, width=64)
    model, wm = build(raw, dtype=torch.bfloat16, seed=31)
    assert all(model.layers[k]["mixer"].left.tc_shape for k in (0, 1)) and model.layers[2]["mixer"].tc_shape
    tk = toks(600, raw["vocab"], 16)
    want = O.forward(raw, wm, tk)

    def most(got, ref, rel, what):
        err = np.abs(got.astype(np.float64) - ref).max(-1) / np.abs(ref).max()
        assert np.quantile(err, 0.9) <= rel, f"{what}: {np.quantile(err, 0.9):.3e}"
    fast_whole = run_portions(model, tk, [600], s=sched(model, 1024))
    fast_parts = run_portions(model, tk, [130, 257, 128, 60], s=sched(model, 1024))
    for k in (0, 1):
        model.layers[k]["mixer"].left.tc_min_portion = 1 << 30
    model.layers[2]["mixer"].tc_min_portion = 1 << 30
    plain = run_portions(model, tk, [600], s=sched(model, 1024))
    most(plain, want, 5e-2, "plain kernels against the oracle")
    most(fast_whole, want, 5e-2, "tensor-core prefill against the oracle")
    most(fast_whole, plain.astype(np.float64), 3e-2, "tensor-core prefill against the plain kernels")
    most(fast_parts, plain.astype(np.float64), 3e-2, "tensor-core portions against the plain kernels")
