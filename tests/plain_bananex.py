"""A plain, slow Bananex in 64-bit numpy: one function per mechanism, whole sequences only.

It shares nothing with the engine: no kernels, no cache, no step function. A sequence goes in whole and the
logits of every position come out; every recurrence is a Python loop over the tokens, every attention row a loop
over the keys it may see. `w` maps tensor names to 64-bit arrays, `cfg` is the parsed config.json.

Notation. T tokens, E the model's width. A layer is
    x <- x + n1b(mixer(shift(n1(x)))),   x <- x + n2b(ff(n2(x)))
with n(v) = v / sqrt(mean(v^2) + eps) * g for a single number g, and shift(h)_t = h_t + (h_(t-1) - h_t) * s
(h_(-1) = 0, s a vector). Layers start..stop-1 run `times` passes with the same weights; before pass t
x <- W [x; e] + step_t, with e the embedding output.
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


def gelu_erf(v):
    return 0.5 * v * (1.0 + np.vectorize(math.erf)(v / math.sqrt(2.0)))


def token_shift(h, s):
    """h_t + (h_(t-1) - h_t) * s with zeros before the first token."""
    prev = np.concatenate([np.zeros_like(h[:1]), h[:-1]], axis=0)
    return h + (prev - h) * s


def rotate_adjacent(v, positions, base, dims):
    """Pairs (2i, 2i+1) of the first `dims` entries of the last axis turn by p * base^(-2i/dims)."""
    out = v.copy()
    i = np.arange(dims // 2, dtype=np.float64)
    f = np.power(float(base), -2.0 * i / dims)
    shape = [len(positions)] + [1] * (v.ndim - 2) + [dims // 2]
    a = (np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]).reshape(shape)
    u, t = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = u * np.cos(a) - t * np.sin(a)
    out[..., 1:dims:2] = t * np.cos(a) + u * np.sin(a)
    return out


def latent_attention(h, w, p, m, eps):
    """Keys and values come from a low-rank latent; one rotated key part is shared by the heads."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    win = m["mask"]["size"] if m.get("mask") else T  # no mask: every earlier key
    pos = np.arange(T)
    q = mm(h, w[p + "q"]).reshape(T, H, dn + dr)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q_plain, q_rot = q[..., :dn], rotate_adjacent(q[..., dn:], pos, rot["base"], rot["dims"])
    dkv = mm(h, w[p + "dkv"])
    c = rms(dkv[:, :r], eps) * w[p + "dkv.norm"]
    if ROUND is not None:  # the cache holds 16-bit values
        c = ROUND(c)
    k_rot = rotate_adjacent(dkv[:, r:], pos, rot["base"], rot["dims"])  # [T, dr], every head's
    if ROUND is not None:
        k_rot = ROUND(k_rot)
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for i in range(T):
        lo = max(0, i - win + 1)
        for a in range(H):
            s = np.array([(q_plain[i, a] @ k_plain[j, a] + q_rot[i, a] @ k_rot[j]) * m["scale"]
                          for j in range(lo, i + 1)])
            e = np.exp(s - s.max())
            out[i, a] = (e / e.sum()) @ v[lo:i + 1, a]
    gate = sigmoid(mm(h, w[p + "g"]))
    return mm(out.reshape(T, H * dv) * gate, w[p + "o"])


def mingru(h, w, p, m):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t, gates from the current token alone."""
    z = sigmoid(mm(h, w[p + "z"]) + w[p + "z.b"])
    u = mm(h, w[p + "x"]) + w[p + "x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(m["width"])
    states = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        states[t] = S
    return mm(states * silu(mm(h, w[p + "g"])), w[p + "o"])


def mamba2(h, w, p, m, eps):
    """Selective state space with a scalar decay per head; S is [state, vdim] per head."""
    T = h.shape[0]
    H, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = H * P
    proj = mm(h, w[p + "in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    padded = np.concatenate([np.zeros((taps - 1, xbc.shape[1])), xbc], axis=0)
    conv = np.zeros_like(xbc)
    for t in range(T):
        conv[t] = np.sum(padded[t:t + taps].T * w[p + "conv"], axis=1) + w[p + "conv.b"]
    conv = silu(conv)
    x = conv[:, :inner].reshape(T, H, P)
    B = conv[:, inner:inner + G * N].reshape(T, G, N)
    C = conv[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :] * dt)
    y = np.zeros((T, H, P))
    S = np.zeros((H, N, P))
    for t in range(T):
        for a in range(H):
            g = a // (H // G)
            S[a] = decay[t, a] * S[a] + dt[t, a] * np.outer(B[t, g], x[t, a])
            y[t, a] = S[a].T @ C[t, g] + w[p + "D"][a] * x[t, a]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return mm(y, w[p + "o"])


def dense_ff(h, w, p):
    return mm(gelu_erf(mm(h, w[p + "up"]) + w[p + "up.b"]), w[p + "down"]) + w[p + "down.b"]


def layer(x, w, i, spec, eps):
    p = f"l{i}."
    h = token_shift(rms(x, eps) * w[p + "norm1"], w[p + "shift"])
    kind, m = spec["type"], spec["mixer"]
    if kind == "latent_attention":
        y = latent_attention(h, w, p + "mix.", m, eps)
    elif kind == "mingru":
        y = mingru(h, w, p + "mix.", m)
    elif kind == "mamba2":
        y = mamba2(h, w, p + "mix.", m, eps)
    else:
        raise ValueError(kind)
    x = x + rms(y, eps) * w[p + "norm1b"]
    if spec.get("mlp") is not None:
        f = dense_ff(rms(x, eps) * w[p + "norm2"], w, p + "mlp.")
        x = x + rms(f, eps) * w[p + "norm2b"]
    return x


def run_order(cfg):
    """[(layer, pass or None, first of its pass)] in the order the layers run."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None, False) for i in range(a)]
    for t in range(times):
        order += [(i, t, i == a) for i in range(a, b)]
    return order + [(i, None, False) for i in range(b, n)]


def forward(cfg, w, tokens, trace=None):
    """Logits [T, vocab] of one whole sequence; `trace` (a list) receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    e = x.copy()
    for i, t, first in run_order(cfg):
        if first:
            x = mm(np.concatenate([x, e], axis=1), w["loop.in"]) + w["loop.step"][t]
        x = layer(x, w, i, cfg["layers"][i], eps)
        if trace is not None:
            trace.append(x.copy())
    return mm(rms(x, eps) * w["final.norm"], w["head"]) * cfg["logit_scale"]
