"""Zaronex: a decoder-only design of pre-normed layers, x <- x + mixer(norm1(x)), x <- x + ff(norm2(x)) with plain RMS norms, whose
residual stream is averaged over depth: with X_0 the embedding output and X_(i+1) the result of layer i, the next layer (and after the
last one the output norm) reads sum_j dwa_i[j] X_j over j = 0 .. i + 1, a learned weighting per layer.  The output head is a tensor of
its own.

Mixers:
  "latent_attention"  attention over a cached low-rank latent plus one shared rotated key part; the queries go through an RMS-normed
                      latent too; interleaved rotary pairs on the rotated part, a sliding window, a sigmoid output gate per element
                      (krasis_b200.mixers.WindowLatentAttention)
  "parallel"          two mixers side by side on the same input, each output RMS-normed over the width, averaged:
                      left   grouped-query attention with biased projections, rotation of dimension i with i + dims / 2 on the first
                             rot.dims dimensions, a sliding window plus one mean-pooled key / value per block of mask.pool positions that
                             lies wholly before the window, a softmax sink per head, a sigmoid output gate per element
                             (krasis_b200.mixers.MultiMapAttention)
                      right  gated linear attention with a decay per key channel (krasis_b200.mixers.GatedLinearAttention)
  "parallel_2"        left   grouped-query attention with one RMS norm over the whole of q and of k, interleaved rotary pairs with
                             linear position scaling, values cached rotated by their positions and the output turned back, a sliding
                             window
                      right  selective scan (krasis_b200.mixers.SelectiveScan)
Feed-forward: dense, down(gelu_tanh(gate h) * (up h)), or none.

config.json keys: architecture, vocab, width, norm.eps, layers [{type, mixer, mlp: null | {kind: "dense", ff}}] with mixer
  latent_attention: heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask.size, rot {base, dims, scaling.factor}
  attention (left): heads, kv_heads, dim, vdim, scale, mask {size, pool}, rot {base, dims, scaling.factor}
  gated linear attention (right of parallel): heads, dim, vdim, tau;  selective scan (right of parallel_2): inner, state, dt_rank, conv.
Tensor names: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.dwa, l<i>.mlp.{gate, up, down},
  latent_attention: l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o};
  left: l<i>.mix.left.{q, k, v}[.b], {q, k}.norm, sink, g, o;  right: l<i>.mix.right.{q, k, v, g, a1, a2, a2.b, norm, o} |
  l<i>.mix.right.{in, conv, conv.b, x, dt, dt.b, A_log, D, o};  l<i>.mix.{left, right}.out.
What a left mixer has beside its projections follows from the tensors and keys that are present (biases, whole norms, sink, gate,
mask.pool, rot.scaling); the pair layout and the rotated values belong to the mixer type.

The model exposes the step interface of `krasis_b200.scheduler`: `make_caches`, `forward_step(tables, want_rows)`.
The residual stream and its depth stack, every norm, attention scores, and everything that feeds a recurrence are fp32; `dtype`
(bfloat16 or float32) is the type of weights, GEMM inputs and the key / value cache.
"""
import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from . import seqops as ops
from .attention import HeadKVCache, RecurrentStatePool
from .mixers import (GatedLinearAttention, GatedMLP, MultiMapAttention, SelectiveScan, SideBySide, WindowLatentAttention, lin,
                     rotary_table)

# what the mixer type fixes for its left attention: (pairs are halves i / i + dims / 2, values are cached rotated)
LEFT_FORM = {"parallel": (True, False), "parallel_2": (False, True)}
MIXERS = ("latent_attention",) + tuple(LEFT_FORM)


@dataclass
class ZaronexConfig:
    vocab: int
    width: int
    eps: float
    layers: List[dict]
    raw: dict = field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "ZaronexConfig":
        cfg = cls(vocab=int(raw["vocab"]), width=int(raw["width"]), eps=float(raw["norm"]["eps"]), layers=list(raw["layers"]), raw=raw)
        for i, L in enumerate(cfg.layers):
            if L["type"] not in MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
            mlp = L.get("mlp")
            if mlp and mlp.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            if L["type"] in LEFT_FORM:
                m = L["mixer"]["left"]
                if m["heads"] % m["kv_heads"]:
                    raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
        return cfg


def _sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix):].replace(".", "_"): v for k, v in weights.items() if k.startswith(prefix)}


def _rot(m: dict):
    """(rotated dims, base, linear position factor) of a mixer's rot entry."""
    rot = m.get("rot") or {}
    return int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), float((rot.get("scaling") or {}).get("factor", 1.0))


def random_weights(cfg: ZaronexConfig, seed: int = 0) -> dict:
    """Random tensors of the design's names and shapes (bf16-representable fp32 on the CPU): tests and benchmarks."""
    g = torch.Generator().manual_seed(seed)
    W = cfg.width
    r = lambda *s, sd=1.0: (torch.randn(*s, generator=g) * sd).to(torch.bfloat16).float()
    nw = lambda n: (1.0 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).float()
    w = {"embed": r(cfg.vocab, W), "head": r(cfg.vocab, W, sd=W ** -0.5), "final.norm": nw(W)}
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L["mixer"]
        w[p + "norm1"] = nw(W)
        if L["type"] == "latent_attention":
            H, dn, dr, dv, rk, rq = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            w.update({p + "mix.dq": r(rq, W, sd=W ** -0.5), p + "mix.dq.norm": nw(rq), p + "mix.uq": r(H * (dn + dr), rq, sd=rq ** -0.5),
                      p + "mix.dkv": r(rk + dr, W, sd=W ** -0.5), p + "mix.dkv.norm": nw(rk), p + "mix.uk": r(H * dn, rk, sd=rk ** -0.5),
                      p + "mix.uv": r(H * dv, rk, sd=rk ** -0.5), p + "mix.g": r(H * dv, W, sd=W ** -0.5),
                      p + "mix.o": r(W, H * dv, sd=(H * dv) ** -0.5)})
        else:
            a, q = m["left"], p + "mix.left."
            H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for nm, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                w[q + nm] = r(rows, W, sd=W ** -0.5)
            w[q + "o"] = r(W, H * dv, sd=(H * dv) ** -0.5)
            if L["type"] == "parallel":
                for nm, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    w[q + nm + ".b"] = r(rows, sd=0.1)
                w.update({q + "sink": r(H), q + "g": r(H * dv, W, sd=W ** -0.5)})
                b, q = m["right"], p + "mix.right."
                Hr, dk, dvr = b["heads"], b["dim"], b["vdim"]
                rk = max(1, min(W, 16))
                w.update({q + "q": r(Hr * dk, W, sd=W ** -0.5), q + "k": r(Hr * dk, W, sd=W ** -0.5), q + "v": r(Hr * dvr, W, sd=W ** -0.5),
                          q + "g": r(Hr * dvr, W, sd=W ** -0.5), q + "a1": r(rk, W, sd=W ** -0.5), q + "a2": r(Hr * dk, rk, sd=rk ** -0.5),
                          q + "a2.b": (r(Hr * dk) + 3.0).to(torch.bfloat16).float(), q + "norm": nw(dvr),
                          q + "o": r(W, Hr * dvr, sd=(Hr * dvr) ** -0.5)})
            else:
                w.update({q + "q.norm": nw(H * d), q + "k.norm": nw(G * d)})
                b, q = m["right"], p + "mix.right."
                C, N, R, K = b["inner"], b["state"], b["dt_rank"], b["conv"]
                w.update({q + "in": r(2 * C, W, sd=W ** -0.5), q + "conv": r(C, K, sd=0.5), q + "conv.b": r(C, sd=0.1),
                          q + "x": r(R + 2 * N, C, sd=C ** -0.5), q + "dt": r(C, R, sd=R ** -0.5), q + "dt.b": (r(C) - 2.0).to(torch.bfloat16).float(),
                          q + "A_log": torch.log(1.0 + torch.arange(N, dtype=torch.float32)).repeat(C, 1).to(torch.bfloat16).float(),
                          q + "D": r(C), q + "o": r(W, C, sd=C ** -0.5)})
            w.update({p + "mix.left.out": nw(W), p + "mix.right.out": nw(W)})
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            w.update({p + "norm2": nw(W), p + "mlp.gate": r(F, W, sd=W ** -0.5), p + "mlp.up": r(F, W, sd=W ** -0.5),
                      p + "mlp.down": r(W, F, sd=F ** -0.5)})
        c = torch.rand(i + 2, generator=g) + 0.1
        w[p + "dwa"] = (c / c.sum()).to(torch.bfloat16).float()
    return w


class ZaronexModel:
    """Weights on the device plus the step function; caches and state slots are made by `make_caches` for a serving session."""

    architecture = "Zaronex"
    page_size = 64

    def __init__(self, cfg: ZaronexConfig, weights: dict, dtype=torch.bfloat16, device=0):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype: bfloat16 or float32")
        if not torch.cuda.is_available():
            raise RuntimeError("ZaronexModel needs a CUDA device (krasis_b200 has no CPU path)")
        ops.load()
        self.cfg, self.dtype = cfg, dtype
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        dev, eps = self.device, cfg.eps
        d = lambda t: t.to(device=dev, dtype=dtype).contiguous()
        f = lambda t: t.to(device=dev, dtype=torch.float32).contiguous()
        self.embed, self.head, self.final_norm = d(weights["embed"]), d(weights["head"]), f(weights["final.norm"])
        self.layers = []
        for i, L in enumerate(cfg.layers):
            p, m = f"l{i}.", L["mixer"]
            lay = {"type": L["type"], "norm1": f(weights[p + "norm1"]), "dwa": f(weights[p + "dwa"])}
            if lay["dwa"].numel() != i + 2:
                raise ValueError(f"layer {i}: the depth average needs {i + 2} weights")
            if L["type"] == "latent_attention":
                dims, base, factor = _rot(m)
                lay["mixer"] = WindowLatentAttention(_sub(weights, p + "mix."), m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"],
                                                     m["scale"], (m.get("mask") or {}).get("size"), dims, base, None, eps, dtype, dev,
                                                     rot_freq=rotary_table(dims, base, factor))
            else:
                halves, rot_values = LEFT_FORM[L["type"]]
                a, b = m["left"], m["right"]
                lw, rw = _sub(weights, p + "mix.left."), _sub(weights, p + "mix.right.")
                lw.pop("out"), rw.pop("out")
                dims, base, factor = _rot(a)
                mask = a.get("mask") or {}
                left = MultiMapAttention(lw, a["heads"], a["kv_heads"], 1, a["dim"], a["vdim"], a["scale"], eps, dtype, dev,
                                         window=mask.get("size"), rot_dims=dims, rot_base=base, rot_factor=factor, rot_half=halves,
                                         norm_whole="q_norm" in lw, pool=mask.get("pool") or 0, rot_values=rot_values,
                                         gate_per_element=True)
                if L["type"] == "parallel":
                    right = GatedLinearAttention(rw, b["heads"], b["dim"], b["vdim"], b["tau"], eps, dtype, dev)
                else:
                    right = SelectiveScan(rw, b["inner"], b["state"], b["dt_rank"], b["conv"], dtype, dev)
                lay["mixer"] = SideBySide(left, right, weights[p + "mix.left.out"], weights[p + "mix.right.out"], eps, dev)
            if L.get("mlp"):
                lay["norm2"] = f(weights[p + "norm2"])
                lay["mlp"] = GatedMLP(_sub(weights, p + "mlp."), dtype, dev, act="gelu_tanh")
            else:
                lay["mlp"] = None
            self.layers.append(lay)

    # ------------------------------------------------------------------------------------------- construction
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype=torch.bfloat16, device=0, **_):
        from . import loader
        cfg = ZaronexConfig.from_dict(json.load(open(os.path.join(model_dir, "config.json"))))
        return cls(cfg, loader.read_named_tensors(model_dir), dtype=dtype, device=device)

    @classmethod
    def random(cls, cfg: ZaronexConfig, seed: int = 0, dtype=torch.bfloat16, device=0):
        return cls(cfg, random_weights(cfg, seed), dtype=dtype, device=device)

    # ------------------------------------------------------------------------------------------- serving interface
    def make_caches(self, max_tokens: int, max_requests: int):
        """(paged cache, state pool) for a session that holds at most max_tokens tokens (each request rounded up to whole pages) in at
        most max_requests live requests.  Every layer has a cache of its own (latents and the rotated key part, or keys and values with
        the pooled blocks where the layer has them); the right-hand mixers keep their recurrent state in the slots."""
        pages = (max_tokens + self.page_size - 1) // self.page_size
        pool = RecurrentStatePool(max_requests, self.device)
        dims, self._state = [], []
        for lay in self.layers:
            mixer = lay["mixer"]
            if isinstance(mixer, SideBySide):
                dims.append(mixer.left.cache_dims())
                self._state.append(mixer.right.register_state(pool))
            else:
                dims.append(mixer.cache_dims())
                self._state.append(None)
        self.kv_cache = HeadKVCache(dims, self.device, max_pages=max(pages, 1), dtype=self.dtype, page_size=self.page_size)
        self.state_pool = pool
        return self.kv_cache, pool

    def _mix(self, i: int, h: torch.Tensor, tb: ops.StepTables) -> torch.Tensor:
        mixer, ps = self.layers[i]["mixer"], self.kv_cache.page_size
        kc, vc = self.kv_cache.get_layer_caches(i)
        if not isinstance(mixer, SideBySide):
            return mixer.forward(h, tb, kc, vc, ps)
        y_left = mixer.left.forward(h, tb, kc, vc, ps, pooled=self.kv_cache.get_pooled_caches(i))
        st = self._state[i]
        y_right = mixer.right.forward(h, tb, *st) if isinstance(st, tuple) else mixer.right.forward(h, tb, st)
        return mixer.merge(y_left, y_right)

    def forward_step(self, tb: ops.StepTables, want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every layer; returns fp32 logits [len(want_rows), vocab] (None if nothing is wanted)."""
        eps, dt, n = self.cfg.eps, self.dtype, len(self.layers)
        x = ops.embed(self.embed, tb.tokens, 1.0)
        stack = torch.empty((n + 1,) + tuple(x.shape), dtype=torch.float32, device=x.device)      # X_0 .. X_n of this step's tokens
        stack[0].copy_(x)
        h = ops.residual_scale_rms(x, norm=self.layers[0]["norm1"], out_dtype=dt, eps=eps) if n else None
        for i, lay in enumerate(self.layers):
            y = self._mix(i, h, tb)
            if lay["mlp"] is not None:
                h = ops.residual_scale_rms(x, y, 1.0, norm=lay["norm2"], out_dtype=dt, eps=eps)
                y = lay["mlp"].forward(h)
            last = i + 1 == n
            # X_(i+1) = x + y joins the stack, x becomes the weighted sum of the stack, h its norm for the next layer / the head
            h = ops.depth_mix(stack, i + 2, lay["dwa"], x, y, norm=self.final_norm if last else self.layers[i + 1]["norm1"],
                              out_dtype=torch.float32 if last else dt, eps=eps)
            if self.layer_trace is not None:
                self.layer_trace.append(x.clone())
        if n == 0:
            h = ops.residual_scale_rms(x, norm=self.final_norm, out_dtype=torch.float32, eps=eps)
        if want_rows is None or want_rows.numel() == 0:
            return None
        return lin(h.index_select(0, want_rows), self.head, torch.float32)

    layer_trace = None      # tests: set to a list to collect the residual stream after every layer
