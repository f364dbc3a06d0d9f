"""Small Tagenex models for the tests: configurations, random weights, a model folder. Weights are drawn in float64,
rounded to bfloat16, and both the file and the plain implementation get the rounded values, so that the two compute from
the same numbers. ``zurerax_util.run_schedule`` drives an engine for these models too."""
import json
import os

import numpy as np
import torch

from glassbox_b200.weights.safetensors_io import write_safetensors


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, top, ff, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def attn(heads, kv_heads, dim, vdim, window=None, scale=None, v_mix=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale if scale is not None else dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return {"type": "attention", "mixer": m, "mlp": mlp}


def config(vocab, width, layers, eps=1e-6):
    return {"architecture": "Tagenex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


CONFIGS = {
    # nothing a power of two; the first mixing layer is not layer 0 and a layer between two mixing ones does not mix; the
    # layers differ in heads, sizes and windows (shorter and longer than a page); value size unlike key size; one layer
    # without a feed-forward; both kinds of feed-forward with unlike limits
    "odd": lambda: config(203, 56, [
        attn(6, 2, 20, 12, window=7, mlp=dense(40, 1.5)),
        attn(6, 3, 12, 8, window=19, v_mix=True, scale=0.4, mlp=moe(6, 2, 24, 0.75)),
        attn(4, 4, 16, 24, window=11, v_mix=False, mlp=None),
        attn(3, 3, 20, 8, window=23, v_mix=True, mlp=dense(72, 3.0)),
        attn(6, 3, 8, 8, v_mix=True, mlp=moe(5, 3, 20, 2.5)),
    ], eps=1e-5),
    # sizes the vector loads and the tensor-core kernels are built for; a window of 33 (two pages plus one), one of 48
    # (three whole pages), one of 100 (longer than a tile of rows)
    "even": lambda: config(320, 128, [
        attn(8, 2, 64, 64, window=33, v_mix=True, mlp=moe(16, 4, 32, 1.0)),
        attn(4, 2, 128, 64, window=48, v_mix=True, scale=0.2, mlp=dense(256, 2.0)),
        attn(4, 4, 32, 32, window=100, mlp=moe(4, 2, 128, 4.0)),
        attn(2, 1, 32, 128, window=64, v_mix=False, mlp=dense(64, 0.5)),
        attn(2, 2, 64, 64, window=17, v_mix=True, mlp=None),
    ]),
    # what the design lets a model leave out: no window anywhere, no value mixing, layers without a feed-forward
    "plain": lambda: config(97, 48, [
        attn(3, 1, 16, 16, mlp=dense(24, 2.0)),
        attn(2, 2, 8, 24, mlp=None),
        attn(4, 2, 8, 16, v_mix=False, mlp=moe(3, 3, 16, 1.0)),
    ]),
    # ones: one head, a window of one token (a position sees itself and the sink alone), a window of two, one expert,
    # one of several experts per token (its weight is then exactly one), a single mixing layer (nothing ever mixes into it)
    "ones": lambda: config(61, 32, [
        attn(1, 1, 8, 8, window=1, mlp=moe(1, 1, 8, 1.0)),
        attn(2, 1, 8, 8, window=2, v_mix=True, mlp=moe(4, 1, 8, 2.0)),
        attn(1, 1, 16, 1, window=3, mlp=dense(1, 1.0)),
    ]),
    # sizes that fit no vector width: odd row lengths everywhere, so every kernel's aligned fast path must step aside
    "ragged": lambda: config(67, 50, [
        attn(3, 1, 10, 7, window=5, v_mix=True, mlp=moe(6, 2, 9, 1.25)),
        attn(1, 1, 13, 7, window=9, v_mix=True, mlp=dense(11, 2.0)),
    ]),
}


def tensor_shapes(cfg):
    d = cfg["width"]
    shapes = {"embed": (cfg["vocab"], d), "final.norm": (d,), "head": (cfg["vocab"], d)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        shapes.update({p + "norm1": (d,), p + "mix.q": (H * D, d), p + "mix.k": (G * D, d), p + "mix.v": (G * V, d),
                       p + "mix.g": (H, d), p + "mix.o": (d, H * V), p + "mix.q.norm": (D,), p + "mix.k.norm": (D,),
                       p + "mix.r1": (H,), p + "mix.r2": (H,), p + "mix.sink": (H,), p + "mix.vmix": ()})
        f = L["mlp"]
        if f is None:
            continue
        shapes[p + "norm2"] = (d,)
        if f["kind"] == "dense":
            shapes.update({p + "mlp.gate": (f["ff"], d), p + "mlp.gate.b": (f["ff"],), p + "mlp.up": (f["ff"], d),
                           p + "mlp.up.b": (f["ff"],), p + "mlp.down": (d, f["ff"]), p + "mlp.down.b": (d,)})
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            shapes.update({p + "mlp.router": (E, d), p + "mlp.router.b": (E,)})
            for e in range(E):
                shapes.update({p + f"mlp.e{e}.gate": (ff, d), p + f"mlp.e{e}.up": (ff, d), p + f"mlp.e{e}.down": (d, ff)})
    return shapes


def _bf16(a):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(torch.bfloat16)


def random_weights(cfg, seed):
    """{name: bfloat16 tensor}. Matrices are N(0, 1/in), so that every projection of a unit row is of order one; the
    feed-forwards' first products are wider, so that the clamps cut a good part of their outputs on both sides; the
    distance bias is large enough to reorder keys (r1 around 0.5, r2 positive), sinks and router biases of the order of
    the scores they stand beside."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name in ("embed", "head"):
            w = rng.standard_normal(shape) * (1.0 if name == "embed" else 1.0 / np.sqrt(shape[1]))
        elif name.endswith("mlp.router"):
            w = rng.standard_normal(shape) * 2.0 / np.sqrt(shape[1])
        elif leaf in ("gate", "up"):
            w = rng.standard_normal(shape) * 1.5 / np.sqrt(shape[1])
        elif len(shape) == 2:
            w = rng.standard_normal(shape) / np.sqrt(shape[1])
        elif leaf == "r1":
            w = rng.uniform(0.1, 1.0, shape)
        elif leaf == "r2":
            w = rng.uniform(0.05, 2.0, shape)
        elif leaf == "sink":
            w = rng.standard_normal(shape) * 1.5
        elif leaf == "vmix":
            w = rng.uniform(0.2, 0.7)
        elif name.endswith("router.b"):
            w = rng.standard_normal(shape) * 0.7
        elif leaf == "b":
            w = rng.standard_normal(shape) * 0.5
        elif leaf in ("norm1", "norm2", "norm"):
            w = 1.0 + rng.standard_normal(shape) * 0.2
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
