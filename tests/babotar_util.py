"""Small Babotar models for the tests: configurations, random weights, a model folder. Weights are drawn in float64, rounded
to bfloat16, and both the file and the plain implementation get the rounded values, so that the two compute from the same
numbers. ``zurerax_util.run_schedule`` drives an engine for these models too."""
import json
import os

import numpy as np
import torch

from glassbox_b200.weights.safetensors_io import write_safetensors


def dense(ff):
    return {"kind": "dense", "ff": ff}


def lightning(heads, dim, vdim, decay, mlp=None):
    assert len(decay) == heads
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def left(heads, kv_heads, dim, vdim, rotation=None, softcap=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if rotation is not None:
        m["rot"] = rotation
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def parallel(lf, rt, left_scale=None, right_scale=None, mlp=None):
    m = {"left": lf, "right": rt}
    if left_scale is not None:
        m["left_scale"] = left_scale
    if right_scale is not None:
        m["right_scale"] = right_scale
    return {"type": "parallel", "mixer": m, "mlp": mlp}


def config(vocab, width, layers, streams=None, mult=None, taps=None, max_positions=512, eps=1e-6):
    cfg = {"architecture": "Babotar", "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": eps},
           "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if mult is not None:
        cfg["residual_mult"] = mult
    if taps is not None:
        cfg["canon"] = {"taps": taps}
    return cfg


CONFIGS = {
    # nothing a power of two; two streams; a convolution of two taps on the mixers' input and one of four in the delta rule;
    # grouped heads on both sides with unlike group sizes; a rotation of a part of the head with stretched frequencies (the
    # ramp lies inside the pairs); value sizes unlike key sizes; a layer without a feed-forward; layers in another order
    "odd": lambda: config(203, 56, [
        parallel(left(6, 2, 20, 12, rot(12, 1000.0, (4.0, 64, 8.0, 2.0)), softcap=5.0, scale=0.3),
                 right(4, 2, 12, 6, 4), 0.5, 1.3, dense(40)),
        lightning(3, 10, 6, (0.5, 0.9, 0.99), dense(24)),
        lightning(2, 12, 20, (1.0, 0.75), None),
        parallel(left(4, 4, 16, 24, rot(16, 50.0), softcap=2.0), right(2, 1, 20, 12, 2), 1.1, 0.4, dense(72)),
    ], streams=2, mult=0.8, taps=2, eps=1e-5),
    # sizes the vector loads and the tensor-core kernels are built for; four streams, four taps
    "even": lambda: config(320, 128, [
        lightning(4, 64, 64, (0.9, 0.95, 0.99, 0.999), dense(256)),
        parallel(left(8, 2, 64, 64, rot(64, 10000.0, (8.0, 128, 16.0, 1.0)), softcap=30.0), right(4, 2, 64, 64, 4), 0.7, 0.8, dense(128)),
        parallel(left(4, 4, 32, 32, rot(16, 10000.0), softcap=10.0), right(4, 4, 32, 32, 3), 1.0, 1.0, None),
        lightning(2, 128, 64, (0.97, 0.8), dense(64)),
        parallel(left(4, 1, 128, 64, rot(128, 500.0)), right(2, 1, 128, 128, 2), 0.9, 0.6, dense(128)),
    ], streams=4, mult=0.6, taps=4),
    # what the design lets a model leave out: no streams, no convolution on the input, no factor on the branches, no
    # rotation, no cap, no stretching, layers without a feed-forward, branch weights left to their default
    "plain": lambda: config(97, 48, [
        parallel(left(3, 1, 16, 16), right(2, 2, 8, 8, 3), mlp=dense(24)),
        lightning(2, 8, 24, (0.9, 0.6), None),
        parallel(left(4, 2, 8, 16, rot(8, 100.0)), right(4, 1, 16, 8, 1), mlp=None),
    ]),
    # ones: one learned stream, one tap everywhere (the convolutions see the current token only), one head, one channel of
    # value, a feed-forward of one unit, a decay of one (nothing is forgotten) and of zero (only the current token counts)
    "ones": lambda: config(61, 32, [
        lightning(1, 8, 8, (1.0,), dense(1)),
        parallel(left(1, 1, 8, 1, rot(2, 10.0, (2.0, 8, 2.0, 1.0))), right(1, 1, 8, 1, 1), 1.0, 1.0, dense(8)),
        lightning(2, 4, 1, (0.0, 0.5), None),
    ], streams=1, mult=1.0, taps=1),
    # sizes that fit no vector width: odd row lengths everywhere, so every kernel's aligned fast path must step aside
    "ragged": lambda: config(67, 50, [
        parallel(left(3, 1, 10, 7, rot(6, 77.0, (3.0, 32, 4.0, 1.0)), softcap=4.0), right(3, 1, 9, 7, 3), 0.75, 1.2, dense(11)),
        lightning(3, 7, 5, (0.9, 0.8, 0.7), dense(9)),
    ], streams=5, mult=0.9, taps=5),
}


def tensor_shapes(cfg):
    d = cfg["width"]
    shapes = {"embed": (cfg["vocab"], d), "pos": (cfg["max_positions"], d), "final.norm": (d,), "head": (cfg["vocab"], d)}
    S = cfg.get("streams")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        shapes[p + "norm1"] = (d,)
        if cfg.get("canon") is not None:
            shapes[p + "canon1"] = (d, cfg["canon"]["taps"])
        for q in (1, 2) if L["mlp"] is not None else (1,):
            if S is not None:
                shapes.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        if L["type"] == "lightning":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * D, d), p + "mix.k": (H * D, d), p + "mix.v": (H * V, d), p + "mix.g": (H * V, d),
                           p + "mix.o": (d, H * V), p + "mix.norm": (H * V,)})
        else:
            a, r = m["left"], m["right"]
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            lp = p + "mix.left."
            shapes.update({lp + "q": (H * D, d), lp + "q.b": (H * D,), lp + "k": (G * D, d), lp + "k.b": (G * D,),
                           lp + "v": (G * V, d), lp + "v.b": (G * V,), lp + "talk": (H, H), lp + "o": (d, H * V)})
            H, G, D, V, taps = r["heads"], r["kv_heads"], r["dim"], r["vdim"], r["conv"]
            rp = p + "mix.right."
            shapes.update({rp + "q": (G * D, d), rp + "q.conv": (G * D, taps), rp + "k": (G * D, d), rp + "k.conv": (G * D, taps),
                           rp + "v": (H * V, d), rp + "v.conv": (H * V, taps), rp + "b": (H, d), rp + "A_log": (H,), rp + "norm": (V,),
                           rp + "a": (H, d), rp + "dt_bias": (H,), rp + "g": (H * V, d), rp + "o": (d, H * V)})
        if L["mlp"] is not None:
            ff = L["mlp"]["ff"]
            shapes.update({p + "norm2": (d,), p + "mlp.gate": (ff, d), p + "mlp.up": (ff, d), p + "mlp.down": (d, ff)})
    return shapes


def _bf16(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def random_weights(cfg, seed, sharpen=1.0):
    """{name: bfloat16 tensor}. Matrices are N(0, 1/in), so that every projection of a unit row is of order one; ``sharpen``
    multiplies the attention's query projections, so that a few keys carry each softmax; the heads' mixing matrix is the
    identity plus noise of a third of it; stream weights lie around a plain residual."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name == "embed":
            w = rng.standard_normal(shape)
        elif name == "pos":
            w = rng.standard_normal(shape) * 0.5
        elif leaf == "conv":
            w = rng.standard_normal(shape) * 0.6
        elif leaf == "canon1":
            w = rng.standard_normal(shape) * 0.4
        elif leaf == "talk":
            w = np.eye(shape[0]) + rng.standard_normal(shape) * 0.3
        elif leaf == "mix" and ".hc" in name:
            w = np.eye(shape[0]) * 0.8 + rng.standard_normal(shape) * 0.15
        elif leaf == "in":
            w = 1.0 / shape[0] + rng.standard_normal(shape) * 0.2
        elif leaf == "out":
            w = 1.0 + rng.standard_normal(shape) * 0.3
        elif len(shape) == 2:
            w = rng.standard_normal(shape) / np.sqrt(shape[1])
            if name.endswith("left.q"):
                w *= sharpen
        elif leaf == "b":
            w = rng.standard_normal(shape) * 0.5
        elif leaf in ("norm1", "norm2", "norm"):
            w = 1.0 + rng.standard_normal(shape) * 0.2
        elif leaf == "A_log":
            w = rng.uniform(-2.0, 0.5, shape)
        elif leaf == "dt_bias":
            w = rng.standard_normal(shape)
        else:
            raise AssertionError(name)
        out[name] = _bf16(w)
    return out


def as_float64(tensors):
    return {k: v.float().numpy().astype(np.float64) for k, v in tensors.items()}


def write_model(folder, cfg, tensors):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), {k: v.contiguous() for k, v in tensors.items()})
    return folder
