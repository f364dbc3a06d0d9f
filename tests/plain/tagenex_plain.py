"""Tagenex in plain float64 NumPy, one function per mechanism, written from the architecture's equations and sharing no
code with the engine. Slow on purpose: every sum is a visible loop or a single matrix product over a whole sequence.

Notation: T tokens, d model width, a sequence's positions count from 0. ``W`` maps tensor names to float64 arrays
(matrices stored [out, in] and applied as W x). A layer is x += norm1(mixer(x)); x += norm2(ff(x)): the branches read the
residual itself, and only their outputs are normed.
"""
import numpy as np

#: the slope inside the feed-forwards' gate activation, g * logistic(SLOPE * g)
SLOPE = 1.702


def logistic(x):
    return 1.0 / (1.0 + np.exp(-np.asarray(x, dtype=np.float64)))


def rms_unit(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (eps inside the root, plain gain)."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def visible(i, j, window):
    """Whether position i sees position j: itself and the window - 1 tokens before it (no window: all earlier ones)."""
    return j <= i and (window is None or i - j < window)


def distance_bias(r1, r2, distance):
    """What is taken off the score of a key ``distance`` tokens back: r1 ln(1 + r2 distance), zero for the token itself."""
    return r1 * np.log1p(r2 * distance)


def sink_softmax(scores, sink):
    """Weights of the visible keys when the denominator also holds exp(sink): they add up to less than one."""
    m = max(float(np.max(scores)), float(sink))
    e = np.exp(np.asarray(scores) - m)
    return e / (e.sum() + np.exp(sink - m))


def mix_values(v, v_first, lam):
    """(1 - lam) v + lam v_first; the first mixing layer (v_first None) keeps its own values."""
    return v if v_first is None else (1.0 - lam) * v + lam * v_first


def attention(h, W, p, m, eps, v_first=None):
    """h [T, d] -> ([T, d] before the branch norm, the values [T, G, V] that this layer keeps)."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, D)
    k = (h @ W[p + "k"].T).reshape(T, G, D)
    v = (h @ W[p + "v"].T).reshape(T, G, V)
    q, k = rms_unit(q, W[p + "q.norm"], eps), rms_unit(k, W[p + "k.norm"], eps)
    if m.get("v_mix"):
        v = mix_values(v, v_first, float(W[p + "vmix"]))
    gate = logistic(h @ W[p + "g"].T)                          # [T, H]
    window = m["mask"]["size"] if m.get("mask") is not None else None
    out = np.zeros((T, H, V))
    for head in range(H):
        g = head // (H // G)
        r1, r2, sink = W[p + "r1"][head], W[p + "r2"][head], W[p + "sink"][head]
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, window)]
            s = np.array([q[i, head] @ k[j, g] * m["scale"] - distance_bias(r1, r2, i - j) for j in js])
            w = sink_softmax(s, sink)
            for a, j in zip(w, js):
                out[i, head] += a * v[j, g]
            out[i, head] *= gate[i, head]
    return out.reshape(T, H * V) @ W[p + "o"].T, v


def gated_unit(g, u, limit):
    """min(g, limit) * logistic(SLOPE min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
    g = np.minimum(g, limit)
    u = np.clip(u, -limit, limit)
    return g * logistic(SLOPE * g) * (u + 1.0)


def dense_ff(h, W, p, mlp):
    y = gated_unit(h @ W[p + "gate"].T + W[p + "gate.b"], h @ W[p + "up"].T + W[p + "up.b"], mlp["limit"])
    return y @ W[p + "down"].T + W[p + "down.b"]


def route(h, W, p, mlp):
    """([T, top] chosen experts, [T, top] weights): the ``top`` largest logits (lowest index among equals), softmax over
    the chosen logits alone."""
    z = h @ W[p + "router"].T + W[p + "router.b"]
    top = mlp["router"]["top"]
    order = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, order, axis=-1)
    e = np.exp(zc - zc.max(-1, keepdims=True))
    return order, e / e.sum(-1, keepdims=True)


def expert(h_row, W, p, e, limit):
    q = f"{p}e{e}."
    return gated_unit(W[q + "gate"] @ h_row, W[q + "up"] @ h_row, limit) @ W[q + "down"].T


def moe_ff(h, W, p, mlp):
    order, weight = route(h, W, p, mlp)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for k in range(order.shape[1]):
            out[t] += weight[t, k] * expert(h[t], W, p, int(order[t, k]), mlp["expert"]["limit"])
    return out


def feed_forward(h, W, p, mlp):
    return dense_ff(h, W, p, mlp) if mlp["kind"] == "dense" else moe_ff(h, W, p, mlp)


def forward(cfg, W, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the residual after every layer [L, T, d])."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(tokens)]
    v_first, after = None, []
    for i, L in enumerate(cfg["layers"]):
        t = f"l{i}."
        y, v = attention(x, W, t + "mix.", L["mixer"], eps, v_first)
        if L["mixer"].get("v_mix") and v_first is None:
            v_first = v
        x = x + rms_unit(y, W[t + "norm1"], eps)
        if L.get("mlp") is not None:
            x = x + rms_unit(feed_forward(x, W, t + "mlp.", L["mlp"]), W[t + "norm2"], eps)
        after.append(x.copy())
    logits = rms_unit(x, W["final.norm"], eps) @ W["head"].T
    return (logits, np.array(after)) if keep_layers else logits
