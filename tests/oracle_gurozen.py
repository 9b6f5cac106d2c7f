"""Plain float64 restatement of the Gurozen design, one function per mechanism, written from the design's equations.  It shares no
code with the package; it is slow on purpose (explicit loops over tokens, heads and keys) and runs on the CPU with numpy alone.

Notation: h [T, W] is a sublayer's input, weights are [out, in] and applied as h @ w.T; names follow the checkpoint's tensor names
with the layer prefix removed ("q", "q.b", "q.conv", "q.norm", ...)."""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


def rms_unit(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_around_zero(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def causal_conv(u, taps):
    """u [T, C], taps [C, K]: y[t] = sum_j taps[:, j] u[t - K + 1 + j], zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    y = np.zeros_like(u)
    for t in range(T):
        for j in range(K):
            src = t - K + 1 + j
            if src >= 0:
                y[t] += taps[:, j] * u[src]
    return y


def rot_frequencies(rot):
    """f_i = base^(-2i / dims), rescaled by wavelength against the original length."""
    dims = rot["dims"]
    f = np.array([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < sc["original"] / sc["high"]:
            continue
        if wave > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
    return out


def rotate_half(x, positions, rot):
    """x [T, heads, d]: dimension i turns with dimension i + dims / 2 by the angle position * f_i; the rest passes."""
    if not rot or not rot.get("dims"):
        return x
    dims, f = rot["dims"], rot_frequencies(rot)
    y = x.copy()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * f[i]
            c, s = math.cos(a), math.sin(a)
            u, v = x[t, :, i], x[t, :, i + dims // 2]
            y[t, :, i] = u * c - v * s
            y[t, :, i + dims // 2] = v * c + u * s
    return y


def attention(h, w, m, eps, first_position=0):
    """Grouped-query causal softmax attention with convolved projections, whole-projection q / k norms, rotation and a tanh cap."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for n in ("q", "k", "v"):
        u = h @ w[n].T + w[n + ".b"]
        proj[n] = causal_conv(u, w[n + ".conv"]) if m.get("conv") else u
    q = rms_unit(proj["q"], eps) * w["q.norm"]
    k = rms_unit(proj["k"], eps) * w["k.norm"]
    pos = [first_position + t for t in range(T)]
    q = rotate_half(q.reshape(T, H, d), pos, m.get("rot"))
    k = rotate_half(k.reshape(T, G, d), pos, m.get("rot"))
    v = proj["v"].reshape(T, G, dv)
    cap = m.get("softcap") or 0.0
    out = np.zeros((T, H, dv))
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            sc = (k[:t + 1, g] @ q[t, hh]) * m["scale"]
            if cap:
                sc = cap * np.tanh(sc / cap)
            p = np.exp(sc - sc.max())
            out[t, hh] = (p / p.sum()) @ v[:t + 1, g]
    return out.reshape(T, H * dv) @ w["o"].T


def channel_delta(h, w, m, eps, return_state=False):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, d)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, d)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w["b"].T)
    step = softplus((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(T, H, d)
    decay = np.exp(-np.exp(w["A_log"])[None, :, None] * step)
    gate = sigmoid((h @ w["g1"].T) @ w["g2"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    states = []
    for hh in range(H):
        kh = hh // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = decay[t, hh][:, None] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, kh])
            S = S + np.outer(k[t, kh], u)
            out[t, hh] = S.T @ q[t, kh]
        states.append(S)
    out = rms_unit(out, eps) * w["norm"] * gate
    y = out.reshape(T, H * dv) @ w["o"].T
    return (y, np.stack(states)) if return_state else y


def dense_ff(h, w):
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def squared_relu_expert(h, up, down):
    return (np.maximum(h @ up.T, 0.0) ** 2) @ down.T


def route(h, router_w, rt):
    """(chosen experts [T, top], their weights [T, top]): sigmoid scores, groups ranked by their best two members added up, top-k
    among the kept groups (ties to the lower index), weights renormalised and scaled."""
    T = h.shape[0]
    E, top = rt["experts"], rt["top"]
    grp = rt.get("groups") or {"count": 1, "keep": 1}
    s = sigmoid(h @ router_w.T)
    size = E // grp["count"]
    ids, wts = np.zeros((T, top), dtype=np.int64), np.zeros((T, top))
    for t in range(T):
        gscore = [np.sort(s[t, gi * size:(gi + 1) * size])[-2:].sum() for gi in range(grp["count"])]
        kept = sorted(range(grp["count"]), key=lambda gi: (-gscore[gi], gi))[:grp["keep"]]
        cand = [e for e in range(E) if e // size in kept]
        chosen = sorted(cand, key=lambda e: (-s[t, e], e))[:top]
        ids[t] = chosen
        wts[t] = s[t, chosen] / (s[t, chosen].sum() + 1e-20) * rt.get("scale", 1.0)
    return ids, wts


def moe_ff(h, w, mlp):
    ids, wts = route(h, w["router"], mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], wts[t]):
            out[t] += a * squared_relu_expert(h[t:t + 1], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out += sigmoid(h @ w["shared.sg"].T) * squared_relu_expert(h, w["shared.up"], w["shared.down"])
    return out


def layer_runs(raw):
    """[(layer, True where a pass of the looped span starts)]."""
    n, lp = len(raw["layers"]), raw.get("loop")
    if not lp or lp["times"] < 1 or lp["stop"] <= lp["start"]:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(lp["start"])]
    for _ in range(lp["times"]):
        runs += [(i, i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, False) for i in range(lp["stop"], n)]


def sub(w, prefix):
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def forward(raw, w, tokens, collect=None):
    """Logits [T, vocab] of one sequence; `collect` (a list) receives the residual stream after every layer run."""
    eps, mult = raw["norm"]["eps"], raw.get("residual_mult", 1.0)
    x = norm_around_zero(w["embed"][np.asarray(tokens)], w["embed.norm"], eps)
    x0 = x
    for li, starts in layer_runs(raw):
        L, p = raw["layers"][li], f"l{li}."
        if starts:
            x = np.concatenate([x, x0], -1) @ w["loop.in"].T
        h = norm_around_zero(x, w[p + "norm1"], eps)
        mix = attention if L["type"] == "attention" else channel_delta
        x = x + mult * mix(h, sub(w, p + "mix."), L["mixer"], eps)
        if L.get("mlp"):
            h = norm_around_zero(x, w[p + "norm2"], eps)
            ff = dense_ff if L["mlp"].get("kind", "dense") == "dense" else (lambda a, b: moe_ff(a, b, L["mlp"]))
            x = x + mult * ff(h, sub(w, p + "mlp."))
        if collect is not None:
            collect.append(x.copy())
    return norm_around_zero(x, w["final.norm"], eps) @ w["embed"].T * raw.get("logit_scale", 1.0)
