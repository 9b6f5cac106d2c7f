"""Plain float64 restatement of the Zaronex design, one function per mechanism, written from the design's equations.  It shares no
code with the package; it is slow on purpose (explicit loops over tokens, heads and keys) and runs on the CPU with numpy alone.

Notation: h [T, W] is a sublayer's input, weights are [out, in] and applied as h @ w.T; `w` dictionaries hold a mixer's tensors under
their checkpoint names with the prefix removed ("q", "q.b", "q.norm", "left.q", ...).  Every function takes one whole sequence whose
first token has position 0."""
import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.where(z > 30.0, z, np.log1p(np.exp(np.minimum(z, 30.0))))


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


# ----------------------------------------------------------------------------------------------------------- rotary positions
def pair_frequencies(dims, base, factor=1.0):
    return np.array([base ** (-2.0 * i / dims) / factor for i in range(dims // 2)], dtype=np.float64)


def turn(x, angle_sign, positions, freqs, halves):
    """x [T, ..., d]: the first 2 len(freqs) dimensions turn by sign * position * f_m in pairs (m, m + n) if halves else (2m, 2m + 1)."""
    n = len(freqs)
    y = x.copy()
    for t, p in enumerate(positions):
        for m in range(n):
            a = angle_sign * p * freqs[m]
            c, s = math.cos(a), math.sin(a)
            iu, iv = (m, m + n) if halves else (2 * m, 2 * m + 1)
            u, v = x[t, ..., iu], x[t, ..., iv]
            y[t, ..., iu] = u * c - v * s
            y[t, ..., iv] = v * c + u * s
    return y


def rot_of(m):
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    factor = float((rot.get("scaling") or {}).get("factor", 1.0))
    return dims, float(rot.get("base", 10000.0)), factor


# ----------------------------------------------------------------------------------------------------------- softmax attention
def visible_softmax(q, keys, values, scale, sink=None):
    """One query q [d] over keys [n, d] / values [n, dv]; the sink adds exp(sink) to the denominator only."""
    s = keys @ q * scale
    top = s.max() if sink is None else max(s.max(), sink)
    e = np.exp(s - top)
    den = e.sum() + (math.exp(sink - top) if sink is not None else 0.0)
    return (e[:, None] * values).sum(0) / den


def window_keys(i, size):
    return list(range(max(0, i - size + 1), i + 1))


def pooled_blocks(i, size, pool):
    """Blocks of `pool` positions that lie wholly before the window of position i."""
    out, b = [], 0
    while b * pool + pool - 1 <= i - size:
        out.append(b)
        b += 1
    return out


def grouped_window_attention(h, w, m, eps, positions, value_turn=False, cache_round=None):
    """Grouped-query softmax attention under a sliding window, with the options the config and tensors switch on: biases, a norm over
    the whole of q and of k, partial rotation in either pair layout with linear scaling, mean-pooled blocks before the window, a
    sink in the denominator, rotated values, a sigmoid output gate.  Returns [T, W].  halves: `m["halves"]` (set by the caller)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ w["q"].T, h @ w["k"].T, h @ w["v"].T
    if "q.b" in w:
        q, k, v = q + w["q.b"], k + w["k.b"], v + w["v.b"]
    if "q.norm" in w:
        q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    dims, base, factor = rot_of(m)
    halves = m["halves"]
    if dims:
        f = pair_frequencies(dims, base, factor)
        q, k = turn(q, 1.0, positions, f, halves), turn(k, 1.0, positions, f, halves)
    fv = pair_frequencies(dv, base) if value_turn else None
    if value_turn:
        v = turn(v, 1.0, positions, fv, halves)
    if cache_round is not None:
        k, v = cache_round(k), cache_round(v)
    size, pool = m["mask"]["size"], m["mask"].get("pool")
    out = np.zeros((T, H, dv))
    for i in range(T):
        js = window_keys(i, size)
        for hh in range(H):
            g = hh // (H // G)
            keys, vals = [k[j, g] for j in js], [v[j, g] for j in js]
            if pool:
                for b in pooled_blocks(i, size, pool):
                    keys.append(k[b * pool:(b + 1) * pool, g].mean(0))
                    vals.append(v[b * pool:(b + 1) * pool, g].mean(0))
            sink = float(w["sink"][hh]) if "sink" in w else None
            out[i, hh] = visible_softmax(q[i, hh], np.array(keys), np.array(vals), m["scale"], sink)
    if value_turn:
        out = turn(out, -1.0, positions, fv, halves)
    out = out.reshape(T, H * dv)
    if "g" in w:
        out = out * sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def latent_attention(h, w, m, eps, positions):
    """Queries through a normed latent; keys and values from a normed latent c plus one rotated key part shared by the heads."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, dn + dr)
    kv = h @ w["dkv"].T
    c = rms_norm(kv[:, :r], w["dkv.norm"], eps)
    _, base, factor = rot_of(m)
    f = pair_frequencies(dr, base, factor)
    kr = turn(kv[:, r:], 1.0, positions, f, False)
    qr = turn(q[:, :, dn:], 1.0, positions, f, False)
    kn = (c @ w["uk"].T).reshape(T, H, dn)
    vv = (c @ w["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        js = window_keys(i, m["mask"]["size"])
        for hh in range(H):
            keys = np.array([np.concatenate([kn[j, hh], kr[j]]) for j in js])
            qq = np.concatenate([q[i, hh, :dn], qr[i, hh]])
            out[i, hh] = visible_softmax(qq, keys, np.array([vv[j, hh] for j in js]), m["scale"])
    out = out.reshape(T, H * dv) * sigmoid(h @ w["g"].T)
    return out @ w["o"].T


# ----------------------------------------------------------------------------------------------------------- recurrences
def gated_linear_attention(h, w, m, eps, state=None):
    """S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t per head; alpha = sigmoid(z)^(1 / tau) per key channel."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ w["q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, d)
    S = np.zeros((H, d, dv)) if state is None else state
    o = np.zeros((T, H, dv))
    for t in range(T):
        for hh in range(H):
            S[hh] = alpha[t, hh][:, None] * S[hh] + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    o = rms_norm(o, w["norm"], eps).reshape(T, H * dv) * silu(h @ w["g"].T)
    return o @ w["o"].T


def causal_conv(u, taps, bias):
    """u [T, C], taps [C, K]: y[t] = bias + sum_j taps[:, j] u[t - K + 1 + j], zeros before the start."""
    T, _ = u.shape
    K = taps.shape[1]
    y = np.tile(bias, (T, 1)).astype(np.float64)
    for t in range(T):
        for j in range(K):
            src = t - K + 1 + j
            if src >= 0:
                y[t] += taps[:, j] * u[src]
    return y


def selective_scan(h, w, m):
    """Mamba: S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n; y_c = sum_n S[c, n] C_n + D_c x_c; out = W_o (y silu(z))."""
    T = h.shape[0]
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = h @ w["in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w["conv"], w["conv.b"]))
    p = x @ w["x"].T
    dt = softplus(p[:, :R] @ w["dt"].T + w["dt.b"])
    B, Cc = p[:, R:R + N], p[:, R + N:R + 2 * N]
    A = -np.exp(w["A_log"])
    S = np.zeros((inner, N))
    y = np.zeros((T, inner))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ Cc[t] + w["D"] * x[t]
    return (y * silu(z)) @ w["o"].T


# ----------------------------------------------------------------------------------------------------------- sublayers and model
def gated_ff(h, w):
    return (gelu_tanh(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def side_by_side(left, right, w, eps):
    return 0.5 * (rms_norm(left, w["left.out"], eps) + rms_norm(right, w["right.out"], eps))


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def mixer(kind, h, w, m, eps, positions):
    if kind == "latent_attention":
        return latent_attention(h, w, m, eps, positions)
    if kind == "parallel":
        lm = dict(m["left"], halves=True)
        left = grouped_window_attention(h, sub(w, "left."), lm, eps, positions)
        right = gated_linear_attention(h, sub(w, "right."), m["right"], eps)
        return side_by_side(left, right, w, eps)
    if kind == "parallel_2":
        lm = dict(m["left"], halves=False)
        left = grouped_window_attention(h, sub(w, "left."), lm, eps, positions, value_turn=True)
        right = selective_scan(h, sub(w, "right."), m["right"])
        return side_by_side(left, right, w, eps)
    raise ValueError(kind)


def forward(cfg, weights, tokens, trace=None):
    """Logits [T, vocab] of one sequence; trace (a list) collects the stream after every layer (after the depth average)."""
    W64 = {k: np.asarray(v, dtype=np.float64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    positions = list(range(len(tokens)))
    x = W64["embed"][np.asarray(tokens)]
    stack = [x]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = x + mixer(L["type"], rms_norm(x, W64[p + "norm1"], eps), sub(W64, p + "mix."), L["mixer"], eps, positions)
        if L.get("mlp"):
            y = y + gated_ff(rms_norm(y, W64[p + "norm2"], eps), sub(W64, p + "mlp."))
        stack.append(y)
        x = sum(W64[p + "dwa"][j] * stack[j] for j in range(i + 2))
        if trace is not None:
            trace.append(x.copy())
    return rms_norm(x, W64["final.norm"], eps) @ W64["head"].T
