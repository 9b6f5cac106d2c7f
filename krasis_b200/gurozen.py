"""Gurozen: a decoder-only design of pre-normed layers, x <- x + m mixer(norm1(x)), x <- x + m ff(norm2(x)) with one residual multiplier
m and RMS norms whose weight tensors hold the offset from one (x / rms(x) * (1 + w)).  The embedding output is normed; the output head is the
embedding table again, times a logit scale.

Mixers:
  "attention"      grouped-query softmax attention, causal over the whole sequence: biased q / k / v projections, a short causal
                   convolution over time on every projected channel, one RMS norm over the whole of q and one over the whole of k,
                   rotary positions on the first rot.dims dimensions of each head (dimension i with i + dims / 2) with frequencies
                   rescaled by wavelength, scores scaled and soft-capped by tanh
  "channel_delta"  gated delta rule with one decay per head and key channel (krasis_b200.mixers.ChannelDeltaMixer)
Feed-forwards: dense SiLU-gated, or a mixture of ungated squared-relu experts (sigmoid router scores, expert groups scored by their
two best members, weights renormalised and scaled) plus a shared expert with a per-token sigmoid gate.
A span of layers runs several times in a row with the same weights; each pass has caches and states of its own and starts with
x <- W_in [x; x0], x0 being the embedding output.

config.json keys: architecture, vocab, width, norm.eps, residual_mult, logit_scale, loop {start, stop, times},
layers [{type, mixer: {heads, kv_heads, dim, vdim, conv, scale, softcap, rot {base, dims, scaling {factor, low, high, original}}},
         mlp: null | {kind: "dense", ff} | {kind: "moe", expert.ff, router {experts, top, scale, groups {count, keep}}, shared.ff}}].
Tensor names: embed, embed.norm, loop.in, final.norm, l<i>.norm1, l<i>.norm2,
attention: l<i>.mix.{q, k, v}[.b | .conv], l<i>.mix.{q, k}.norm, l<i>.mix.o;
channel_delta: l<i>.mix.{q, k, v}[.conv], l<i>.mix.{b, a1, a2, g1, g2, A_log, dt_bias, norm, o};
l<i>.mlp.{gate, up, down} | l<i>.mlp.{router, e<j>.{up, down}, shared.{up, down, sg}}.

The model exposes the step interface of `krasis_b200.scheduler`: `make_caches`, `forward_step(tables, want_rows)`.
The residual stream, every norm and everything that feeds a recurrence are fp32; `dtype` (bfloat16 or float32) is the type of weights,
GEMM inputs and the key / value cache.
"""
import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import seqops as ops
from .attention import HeadKVCache, RecurrentStatePool
from .mixers import ChannelDeltaMixer, GatedMLP, MultiMapAttention, RoutedExperts, lin, llama3_table

NORM_SHIFT = 1.0          # a norm's weight tensor holds the offset from one
GROUP_MEMBERS = "top2"    # an expert group competes with its best two members added up


@dataclass
class GurozenConfig:
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_scale: float
    layers: List[dict]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0
    raw: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "GurozenConfig":
        loop = raw.get("loop") or {}
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), eps=float(raw["norm"]["eps"]),
                  residual_mult=float(raw.get("residual_mult", 1.0)), logit_scale=float(raw.get("logit_scale", 1.0)),
                  layers=list(raw["layers"]), loop_start=int(loop.get("start", 0)), loop_stop=int(loop.get("stop", 0)),
                  loop_times=int(loop.get("times", 0)), raw=raw)
        for i, L in enumerate(cfg.layers):
            if L["type"] not in ("attention", "channel_delta"):
                raise ValueError(f"unknown mixer type {L['type']!r}")
            m = L["mixer"]
            if m["heads"] % m["kv_heads"]:
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            mlp = L.get("mlp")
            if mlp and mlp.get("kind", "dense") not in ("dense", "moe"):
                raise ValueError(f"unknown feed-forward kind {mlp.get('kind')!r}")
        if not (0 <= cfg.loop_start <= cfg.loop_stop <= len(cfg.layers)) or cfg.loop_times < 0:
            raise ValueError("loop span outside the layer list")
        return cfg

    @property
    def has_loop(self) -> bool:
        return self.loop_times >= 1 and self.loop_stop > self.loop_start

    def runs(self):
        """[(layer index, True if a pass of the looped span starts with this run)] in execution order."""
        n = len(self.layers)
        if not self.has_loop:
            return [(i, False) for i in range(n)]
        out = [(i, False) for i in range(self.loop_start)]
        for _ in range(self.loop_times):
            out += [(i, i == self.loop_start) for i in range(self.loop_start, self.loop_stop)]
        return out + [(i, False) for i in range(self.loop_stop, n)]


def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):].replace(".", "_"): v for k, v in weights.items() if k.startswith(prefix)}


def random_weights(cfg: GurozenConfig, seed: int = 0) -> dict:
    """Random tensors of the design's names and shapes (bf16-representable fp32 on the CPU): tests and benchmarks."""
    g = torch.Generator().manual_seed(seed)
    W = cfg.width
    r = lambda *s, sd=1.0: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16).float()
    nw = lambda n: (0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    w = {"embed": r(cfg.vocab, W), "embed.norm": nw(W), "final.norm": nw(W)}
    if cfg.has_loop:
        w["loop.in"] = r(W, 2 * W, sd=(2 * W) ** -0.5)
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L["mixer"]
        H, G, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
        w[p + "norm1"] = nw(W)
        if L["type"] == "attention":
            for nm, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[p + "mix." + nm] = r(rows, W, sd=W ** -0.5)
                w[p + f"mix.{nm}.b"] = r(rows, sd=0.1)
                w[p + f"mix.{nm}.conv"] = r(rows, K, sd=0.5)
                if nm != "v":
                    w[p + f"mix.{nm}.norm"] = (1.0 + 0.1 * torch.randn(rows, generator=g)).to(torch.bfloat16).float()
        else:
            for nm, rows in (("q", G * d), ("k", G * d), ("v", H * dv)):
                w[p + "mix." + nm] = r(rows, W, sd=W ** -0.5 * 2)
                w[p + f"mix.{nm}.conv"] = r(rows, K, sd=0.5)
            rk = max(1, min(W, 16))
            w.update({p + "mix.b": r(H, W, sd=W ** -0.5), p + "mix.a1": r(rk, W, sd=W ** -0.5), p + "mix.a2": r(H * d, rk, sd=rk ** -0.5),
                      p + "mix.g1": r(rk, W, sd=W ** -0.5), p + "mix.g2": r(H * dv, rk, sd=rk ** -0.5), p + "mix.A_log": (r(H, sd=0.5) - 2.0).to(torch.bfloat16).float(),
                      p + "mix.dt_bias": r(H * d, sd=0.5), p + "mix.norm": (1.0 + 0.1 * torch.randn(dv, generator=g)).to(torch.bfloat16).float()})
        w[p + "mix.o"] = r(W, H * dv, sd=(H * dv) ** -0.5)
        mlp = L.get("mlp")
        if not mlp:
            continue
        w[p + "norm2"] = nw(W)
        if mlp.get("kind", "dense") == "dense":
            F = mlp["ff"]
            w.update({p + "mlp.gate": r(F, W, sd=W ** -0.5), p + "mlp.up": r(F, W, sd=W ** -0.5), p + "mlp.down": r(W, F, sd=F ** -0.5)})
        else:
            rt, F = mlp["router"], mlp["expert"]["ff"]
            w[p + "mlp.router"] = r(rt["experts"], W, sd=W ** -0.5 * 2)
            for e in range(rt["experts"]):
                w.update({p + f"mlp.e{e}.up": r(F, W, sd=W ** -0.5), p + f"mlp.e{e}.down": r(W, F, sd=F ** -0.5)})
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                w.update({p + "mlp.shared.up": r(Fs, W, sd=W ** -0.5), p + "mlp.shared.down": r(W, Fs, sd=Fs ** -0.5),
                          p + "mlp.shared.sg": r(1, W, sd=W ** -0.5)})
    return w


class GurozenModel:
    """Weights on the device plus the step function; caches and state slots are made by `make_caches` for a serving session."""

    architecture = "Gurozen"
    page_size = 64

    def __init__(self, cfg: GurozenConfig, weights: dict, dtype=torch.bfloat16, device=0):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype: bfloat16 or float32")
        if not torch.cuda.is_available():
            raise RuntimeError("GurozenModel needs a CUDA device (krasis_b200 has no CPU path)")
        ops.load()
        self.cfg, self.dtype = cfg, dtype
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        dev, eps = self.device, cfg.eps
        d = lambda t: t.to(device=dev, dtype=dtype).contiguous()
        f = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()
        self.embed = d(weights["embed"])                  # also the output head
        self.embed_norm, self.final_norm = f(weights["embed.norm"]), f(weights["final.norm"])
        self.loop_in = d(weights["loop.in"]) if cfg.has_loop else None
        self.layers = []
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L["mixer"]
            mw = _sub(weights, p + "mix.")
            lay = {"type": L["type"], "norm1": f(weights[p + "norm1"])}
            if L["type"] == "attention":
                rot = m.get("rot") or {}
                dims = int(rot.get("dims", 0))
                freq = llama3_table(dims, rot.get("base", 10000.0), rot.get("scaling")) if dims else None
                lay["mixer"] = MultiMapAttention(mw, m["heads"], m["kv_heads"], 1, m["dim"], m["vdim"], m["scale"], eps, dtype, dev,
                                                 rot_dims=dims, rot_freq=freq, rot_half=True, norm_whole=True, conv_taps=m.get("conv", 0),
                                                 softcap=m.get("softcap") or 0.0)
            else:
                lay["mixer"] = ChannelDeltaMixer(mw, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], eps, dtype, dev)
            mlp = L.get("mlp")
            if not mlp:
                lay["mlp"] = None
            else:
                lay["norm2"] = f(weights[p + "norm2"])
                fw = _sub(weights, p + "mlp.")
                if mlp.get("kind", "dense") == "dense":
                    lay["mlp"] = GatedMLP(fw, dtype, dev, act="silu")
                else:
                    rt = mlp["router"]
                    grp = rt.get("groups") or {}
                    lay["mlp"] = RoutedExperts(fw, rt["experts"], 0, rt["top"], dtype, dev, groups=grp.get("count", 1), keep=grp.get("keep", 1),
                                               score="sigmoid", renorm=True, out_scale=rt.get("scale", 1.0), gated=False, act="relu2",
                                               group_score=GROUP_MEMBERS)
            self.layers.append(lay)
        self.runs = cfg.runs()

    # ------------------------------------------------------------------------------------------- construction
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype=torch.bfloat16, device=0, **_):
        from . import loader
        cfg = GurozenConfig.from_dict(json.load(open(os.path.join(model_dir, "config.json"))))
        return cls(cfg, loader.read_named_tensors(model_dir), dtype=dtype, device=device)

    @classmethod
    def random(cls, cfg: GurozenConfig, seed: int = 0, dtype=torch.bfloat16, device=0):
        return cls(cfg, random_weights(cfg, seed), dtype=dtype, device=device)

    # ------------------------------------------------------------------------------------------- serving interface
    def make_caches(self, max_tokens: int, max_requests: int):
        """(paged cache, state pool) for a session that holds at most max_tokens tokens (each request rounded up to whole pages) in at
        most max_requests live requests.  Every run of a layer gets its own key / value pools, convolution tail and recurrent state."""
        pages = (max_tokens + self.page_size - 1) // self.page_size
        dims, self._run_cache, self._run_state = [], {}, {}
        pool = RecurrentStatePool(max_requests, self.device)
        for ri, (li, _) in enumerate(self.runs):
            mixer = self.layers[li]["mixer"]
            if isinstance(mixer, MultiMapAttention):
                self._run_cache[ri] = len(dims)
                dims.append(mixer.cache_dims())
            self._run_state[ri] = mixer.register_state(pool)
        self.kv_cache = HeadKVCache(dims, self.device, max_pages=max(pages, 1), dtype=self.dtype, page_size=self.page_size)
        self.state_pool = pool
        return self.kv_cache, pool

    def forward_step(self, tb: ops.StepTables, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every layer run; returns fp32 logits [len(want_rows), vocab] (None if nothing is wanted)."""
        cfg, eps, dt, m = self.cfg, self.cfg.eps, self.dtype, self.cfg.residual_mult
        x = ops.embed(self.embed, tb.tokens, 1.0)
        ops.residual_scale_rms(x, norm=self.embed_norm, w_shift=NORM_SHIFT, eps=eps, in_place=True)
        x0 = x.clone() if cfg.has_loop else None
        y = None                                       # sublayer output not yet added to x: the add rides on the next norm
        for ri, (li, starts_pass) in enumerate(self.runs):
            lay = self.layers[li]
            if starts_pass:
                if y is not None:
                    ops.residual_scale_rms(x, y, m, eps=eps)
                    y = None
                x = lin(torch.cat([x, x0], 1).to(dt), self.loop_in, torch.float32)
            h = ops.residual_scale_rms(x, y, m, norm=lay["norm1"], w_shift=NORM_SHIFT, out_dtype=dt, eps=eps)
            if lay["type"] == "attention":
                kc, vc = self.kv_cache.get_layer_caches(self._run_cache[ri])
                y = lay["mixer"].forward(h, tb, kc, vc, self.kv_cache.page_size, tail=self._run_state[ri])
            else:
                tail, state = self._run_state[ri]
                y = lay["mixer"].forward(h, tb, tail, state)
            if lay["mlp"] is not None:
                h = ops.residual_scale_rms(x, y, m, norm=lay["norm2"], w_shift=NORM_SHIFT, out_dtype=dt, eps=eps)
                y = lay["mlp"].forward(h)
            if self.layer_trace is not None:
                ops.residual_scale_rms(x, y, m, eps=eps)
                y = None
                self.layer_trace.append(x.clone())
        h = ops.residual_scale_rms(x, y, m, norm=self.final_norm, w_shift=NORM_SHIFT, out_dtype=torch.float32, eps=eps)
        if want_rows is None or want_rows.numel() == 0:
            return None
        logits = lin(h.index_select(0, want_rows), self.embed, torch.float32)
        return logits.mul_(cfg.logit_scale) if cfg.logit_scale != 1.0 else logits

    layer_trace = None      # tests: set to a list to collect the residual stream after every layer run
