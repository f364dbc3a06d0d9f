"""Babotar in plain float64 NumPy, one function per mechanism, written from the architecture's equations and sharing no
code with the engine. Slow on purpose: every recurrence is a visible loop over tokens, every attention a loop over
(head, query, key).

Notation: T tokens, d model width, a sequence's positions count from 0. ``W`` maps tensor names to float64 arrays
(matrices stored [out, in] and applied as W x); ``p`` is the prefix of a part's tensor names; ``m`` the part's sizes as
config.json gives them.
"""
import math

import numpy as np


def logistic(x):
    return 1.0 / (1.0 + np.exp(-np.asarray(x, dtype=np.float64)))


def silu(x):
    return x * logistic(x)


def softplus(x):
    return np.logaddexp(0.0, x)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(x, w, eps):
    """(x - mean) / sqrt(var + eps) * w over the last axis; var = mean of squared deviations; no bias."""
    mu = x.mean(-1, keepdims=True)
    var = ((x - mu) ** 2).mean(-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def causal_conv(x, w):
    """x [T, C], w [C, taps] (last column weighs the current token): y_t = sum_j w[:, j] x_(t - taps + 1 + j), zeros before
    the start."""
    T, taps = x.shape[0], w.shape[1]
    y = np.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - taps + 1 + j
            if src >= 0:
                y[t] += w[:, j] * x[src]
    return y


def rotary_frequencies(rot):
    """The dims/2 angular frequencies of a rotation, with the long-context rescaling when ``rot`` has ``scaling``, and the
    factor that cos and sin carry."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    f = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    sc = rot.get("scaling")
    if sc is None:
        return f, 1.0

    def turn_dim(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(sc["fast"])), 0)
    hi = min(math.ceil(turn_dim(sc["slow"])), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / sc["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(sc["factor"]) + 1.0


def rotate_half(x, positions, rot):
    """x [T, heads, D]: channel i < dims/2 is paired with channel i + dims/2; the rest pass unchanged."""
    freq, mag = rotary_frequencies(rot)
    half = rot["dims"] // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    a, b = x[..., :half], x[..., half:2 * half]
    out[..., :half] = a * c - b * s
    out[..., half:2 * half] = b * c + a * s
    return out


def lightning(h, W, p, m, eps):
    """Linear attention with one fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; the heads are
    normed together, gated, projected."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).reshape(T, H, D)
    k = silu(h @ W[p + "k"].T).reshape(T, H, D)
    v = silu(h @ W[p + "v"].T).reshape(T, H, V)
    o = np.zeros((T, H, V))
    for head in range(H):
        S = np.zeros((D, V))
        for t in range(T):
            S = m["decay"][head] * S + np.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_unit(o.reshape(T, H * V), eps) * W[p + "norm"]
    return (o * logistic(h @ W[p + "g"].T)) @ W[p + "o"].T


def talking_softmax_attention(h, W, p, m):
    """Causal grouped-query attention: biased projections, rotation, capped scores, a softmax whose denominator holds one
    more unit (a key of score 0 without a value), the heads' weights mixed by a matrix before they meet the values."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).reshape(T, H, D)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).reshape(T, G, D)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).reshape(T, G, V)
    pos = np.arange(T)
    if m.get("rot") is not None:
        q, k = rotate_half(q, pos, m["rot"]), rotate_half(k, pos, m["rot"])
    weights = np.zeros((H, T, T))
    for head in range(H):
        g = head // (H // G)
        for i in range(T):
            s = np.array([q[i, head] @ k[j, g] * m["scale"] for j in range(i + 1)])
            if m.get("softcap") is not None:
                s = m["softcap"] * np.tanh(s / m["softcap"])
            e = np.exp(s)
            weights[head, i, :i + 1] = e / (1.0 + e.sum())
    mixed = np.einsum("hg,gij->hij", W[p + "talk"], weights)
    out = np.zeros((T, H, V))
    for head in range(H):
        out[:, head] = mixed[head] @ v[:, head // (H // G)]
    return out.reshape(T, H * V) @ W[p + "o"].T


def gated_delta(h, W, p, m, eps):
    """Gated delta rule with one decay per head: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m.get("kv_heads", m["heads"]), m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, D)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, D)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = logistic(h @ W[p + "b"].T)
    g = np.exp(-np.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = silu(h @ W[p + "g"].T).reshape(T, H, V)
    o = np.zeros((T, H, V))
    for head in range(H):
        kv = head // (H // G)
        S = np.zeros((D, V))
        for t in range(T):
            S = g[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + np.outer(k[t, kv], u)
            o[t, head] = S.T @ q[t, kv]
    o = rms_unit(o, eps) * W[p + "norm"] * gate
    return o.reshape(T, H * V) @ W[p + "o"].T


def parallel(h, W, p, m, eps):
    return (m.get("left_scale", 1.0) * talking_softmax_attention(h, W, p + "left.", m["left"])
            + m.get("right_scale", 1.0) * gated_delta(h, W, p + "right.", m["right"], eps))


def dense_ff(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def mixer(kind, h, W, p, m, eps):
    if kind == "lightning":
        return lightning(h, W, p, m, eps)
    if kind == "parallel":
        return parallel(h, W, p, m, eps)
    raise ValueError(kind)


def forward(cfg, W, tokens, collect=None):
    """tokens -> logits [T, vocab]. ``collect`` (a list) receives the summed residual after every layer."""
    T = len(tokens)
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = W["embed"][np.asarray(tokens)] + W["pos"][np.arange(T)]
    streams = cfg.get("streams")
    xs = [x.copy() for _ in range(streams)] if streams else None
    for i, L in enumerate(cfg["layers"]):
        t = f"l{i}."
        branches = [(1, lambda u: mixer(L["type"], u, W, t + "mix.", L["mixer"], eps))]
        if L.get("mlp") is not None:
            branches.append((2, lambda u: dense_ff(u, W, t + "mlp.")))
        for number, branch in branches:
            hc = f"{t}hc{number}."
            u = sum(W[hc + "in"][s] * xs[s] for s in range(streams)) if streams else x
            u = layer_norm(u, W[f"{t}norm{number}"], eps)
            if number == 1 and cfg.get("canon") is not None:
                u = u + causal_conv(u, W[t + "canon1"])
            y = branch(u)
            if streams:
                xs = [sum(W[hc + "mix"][s, to] * xs[s] for s in range(streams)) + mult * W[hc + "out"][to] * y
                      for to in range(streams)]
            else:
                x = x + mult * y
        if collect is not None:
            collect.append(sum(xs) if streams else x.copy())
    x = sum(xs) if streams else x
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T
