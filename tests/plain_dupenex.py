"""A plain, slow Dupenex in 64-bit numpy: one function per mechanism, whole sequences only.

It shares nothing with the engine: no kernels, no cache, no step function. A sequence goes in whole and the logits
of every position come out; every recurrence is a Python loop over the tokens, every attention row a loop over the
keys it may see. `w` maps tensor names to 64-bit arrays, `cfg` is the parsed config.json.

Notation. T tokens, E the model's width, n(v) = v / sqrt(mean(v^2) + eps) * weight.
A layer without `streams` is x <- x + mixer(n1(x)); x <- x + ff(n2(x)). With `streams` = s the model carries s
copies X[0..s-1] of the stream (all the embedding output at first); sublayer c of a layer has a read vector r, a
write vector o and an s x s matrix M (rows: from, columns: to):
    y = sublayer(n(sum_a r[a] X[a]));   X'[b] = sum_a M[a, b] X[a] + o[b] y   (all b from the old X),
and the model's output stream is sum_a X[a]. Layers start..stop-1 of `loop` run `times` passes in a row with the
same weights and nothing between the passes.
"""
from __future__ import annotations

import math

import numpy as np

ROUND = None  # a function that rounds an array to the engine's 16-bit format, or None: exact


def mm(a, W):
    """a W^T; with `ROUND` set, `a` is rounded first, as a 16-bit engine rounds what enters a contraction."""
    return (ROUND(a) if ROUND is not None else a) @ W.T


def rms(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def softplus(v):
    return np.logaddexp(0.0, v)


def log_sigmoid(v):
    return -np.logaddexp(0.0, -v)


def short_conv(x, taps_w):
    """Causal convolution along time per channel: y_t[c] = sum_j w[c, j] x_(t - (K-1) + j)[c], zeros before the
    start (the last column weighs the current token). x: [T, C], taps_w: [C, K]."""
    T, C = x.shape
    K = taps_w.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    y = np.zeros_like(x)
    for t in range(T):
        for j in range(K):
            y[t] += taps_w[:, j] * padded[t + j]
    return y


def rotate_adjacent(v, positions, base, dims):
    """Pairs (2i, 2i+1) of the first `dims` entries of the last axis turn by p * base^(-2i/dims). v: [T, heads, d]."""
    out = v.copy()
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * float(base) ** (-2.0 * i / dims)
            c, s = math.cos(a), math.sin(a)
            x0, x1 = v[t, :, 2 * i].copy(), v[t, :, 2 * i + 1].copy()
            out[t, :, 2 * i] = x0 * c - x1 * s
            out[t, :, 2 * i + 1] = x1 * c + x0 * s
    return out


# ----------------------------------------------------------------------------------------------- mixers
def channel_delta(h, w, p, m, eps):
    """Delta rule with a decay per head and key channel. Per head S [dim, vdim], token by token:
    S <- g[:, None] * S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(mm(h, w[p + "q"]), w[p + "q.conv"])).reshape(T, G, d)
    k = silu(short_conv(mm(h, w[p + "k"]), w[p + "k.conv"])).reshape(T, G, d)
    v = silu(short_conv(mm(h, w[p + "v"]), w[p + "v.conv"])).reshape(T, H, dv)
    q = q / np.sqrt(np.sum(q * q, axis=-1, keepdims=True) + 1e-6) * d ** -0.5
    k = k / np.sqrt(np.sum(k * k, axis=-1, keepdims=True) + 1e-6)
    beta = sigmoid(mm(h, w[p + "b"]))  # [T, H]
    rate = softplus(mm(mm(h, w[p + "a1"]), w[p + "a2"]) + w[p + "dt_bias"]).reshape(T, H, d)
    g = np.exp(-np.exp(w[p + "A_log"])[None, :, None] * rate)
    gate = sigmoid(mm(mm(h, w[p + "g1"]), w[p + "g2"])).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for a in range(H):
        kv = a // (H // G)
        S = np.zeros((d, dv))
        for t in range(T):
            S = g[t, a][:, None] * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            out[t, a] = S.T @ q[t, kv]
    out = rms(out, eps) * w[p + "norm"] * gate
    return mm(out.reshape(T, H * dv), w[p + "o"])


def window_attention(h, w, p, m):
    """Softmax attention over the last `mask.size` keys (all without a mask), rotary q and k, a sigmoid gate on the
    concatenated heads."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = mm(h, w[p + "q"]).reshape(T, H, d)
    k = mm(h, w[p + "k"]).reshape(T, G, d)
    v = mm(h, w[p + "v"]).reshape(T, G, dv)
    if m.get("rot"):
        q = rotate_adjacent(q, range(T), m["rot"]["base"], m["rot"]["dims"])
        k = rotate_adjacent(k, range(T), m["rot"]["base"], m["rot"]["dims"])
    if ROUND is not None:
        k, v = ROUND(k), ROUND(v)  # the cache holds 16-bit keys and values
    size = m["mask"]["size"] if m.get("mask") else None
    scale = m["scale"] if m.get("scale") is not None else d ** -0.5
    out = np.zeros((T, H, dv))
    for t in range(T):
        lo = 0 if size is None else max(0, t - size + 1)
        for a in range(H):
            kv = a // (H // G)
            s = np.array([q[t, a] @ k[j, kv] for j in range(lo, t + 1)]) * scale
            e = np.exp(s - s.max())
            pr = e / e.sum()
            out[t, a] = pr @ v[lo:t + 1, kv]
    gate = sigmoid(mm(h, w[p + "g"]))
    return mm(out.reshape(T, H * dv) * gate, w[p + "o"])


def matrix_memory(h, w, p, m, eps):
    """A matrix memory with exponential gates kept stable by a running maximum r (0 at the start):
    r' = max(f + r, i);  S <- exp(f + r - r') S + exp(i - r') k v^T;  z likewise from k alone;
    o = S^T q / (max(|z . q|, exp(-r')) + 1e-6)."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = mm(h, w[p + "q"]).reshape(T, H, d) * d ** -0.5
    k = mm(h, w[p + "k"]).reshape(T, H, d)
    v = mm(h, w[p + "v"]).reshape(T, H, dv)
    gi = cap * np.tanh((mm(h, w[p + "i"]) + w[p + "i.b"]) / cap)
    gf = log_sigmoid(cap * np.tanh((mm(h, w[p + "f"]) + w[p + "f.b"]) / cap))
    out = np.zeros((T, H, dv))
    for a in range(H):
        S, z, r = np.zeros((d, dv)), np.zeros(d), 0.0
        for t in range(T):
            r_new = max(gf[t, a] + r, gi[t, a])
            keep, take = math.exp(gf[t, a] + r - r_new), math.exp(gi[t, a] - r_new)
            S = keep * S + take * np.outer(k[t, a], v[t, a])
            z = keep * z + take * k[t, a]
            r = r_new
            out[t, a] = S.T @ q[t, a] / (max(abs(z @ q[t, a]), math.exp(-r)) + 1e-6)
    out = rms(out, eps).reshape(T, H * dv) * w[p + "norm"] * sigmoid(mm(h, w[p + "g"]))
    return mm(out, w[p + "o"])


def side_by_side(h, w, p, m, eps):
    left = window_attention(h, w, p + "left.", m["left"])
    right = matrix_memory(h, w, p + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[p + "left.out"] + rms(right, eps) * w[p + "right.out"])


# ----------------------------------------------------------------------------------------------- feed-forwards
def dense_ff(f, w, p):
    return mm(silu(mm(f, w[p + "gate"])) * mm(f, w[p + "up"]), w[p + "down"])


def routed_ff(f, w, p, mlp):
    """Every token goes to the `top` experts with the largest router logits, weighted by the softmax over those
    logits alone; an expert is down(relu(up f)^2)."""
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = mm(f, w[p + "router"])
    out = np.zeros((f.shape[0], w[p + "e0.down"].shape[0]))
    for t in range(f.shape[0]):
        chosen = sorted(range(n), key=lambda e: (-z[t, e], e))[:top]
        zs = np.array([z[t, e] for e in chosen])
        pr = np.exp(zs - zs.max())
        pr = pr / pr.sum()
        for e, g in zip(chosen, pr):
            a = np.maximum(mm(f[t:t + 1], w[p + f"e{e}.up"]), 0.0) ** 2
            out[t] += g * mm(a, w[p + f"e{e}.down"])[0]
    return out


# ----------------------------------------------------------------------------------------------- the model
def run_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def mixer(h, w, i, layer, eps):
    p = f"l{i}.mix."
    if layer["type"] == "channel_delta":
        return channel_delta(h, w, p, layer["mixer"], eps)
    if layer["type"] == "parallel":
        return side_by_side(h, w, p, layer["mixer"], eps)
    raise ValueError(layer["type"])


def feed_forward(f, w, i, layer):
    mlp = layer["mlp"]
    if mlp.get("kind", "dense") == "moe":
        return routed_ff(f, w, f"l{i}.mlp.", mlp)
    return dense_ff(f, w, f"l{i}.mlp.")


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence. `layers_out`: a list that receives the stream (summed over the
    copies) after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][np.asarray(tokens)]
    s = cfg.get("streams")
    X = [x.copy() for _ in range(s)] if s else None
    for i in run_order(cfg):
        layer = cfg["layers"][i]
        subs = [(1, lambda h, i=i, layer=layer: mixer(h, w, i, layer, eps))]
        if layer.get("mlp"):
            subs.append((2, lambda f, i=i, layer=layer: feed_forward(f, w, i, layer)))
        for c, fn in subs:
            nw = w[f"l{i}.norm{c}"]
            if X is None:
                x = x + fn(rms(x, eps) * nw)
                continue
            r, o, M = w[f"l{i}.hc{c}.in"], w[f"l{i}.hc{c}.out"], w[f"l{i}.hc{c}.mix"]
            y = fn(rms(sum(r[a] * X[a] for a in range(s)), eps) * nw)
            X = [sum(M[a, b] * X[a] for a in range(s)) + o[b] * y for b in range(s)]
        if layers_out is not None:
            layers_out.append(x.copy() if X is None else sum(X))
    if X is not None:
        x = sum(X)
    return mm(rms(x, eps) * w["final.norm"], w["head"])
