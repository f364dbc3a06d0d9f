"""Tagenex: a decoder whose layers norm their branches on the way out only (x += norm1(mixer(x)); x += norm2(ff(x)), the
branches reading the residual itself), whose mixers are sliding-window grouped-query softmax attention without a rotation
(query/key RMS norm per head, a logarithmic bias on the distance with two learned numbers per head, a learned sink logit
per head in the softmax's denominator, values mixed with those of the first mixing layer before they are cached, a sigmoid
output gate per head), and whose feed-forwards are either a dense clamped gated unit with biases or a mixture of such
units without biases, routed by the largest logits with softmax weights over the chosen ones.

This file only *describes* the architecture: which config.json keys it reads and how tensor names map onto part parameters.
The math lives in the parts (``parts/sink_attention.py``, ``parts/mlp.py``, ``parts/moe.py``, ``parts/block.py``).

config.json: ``architecture`` "Tagenex"; ``vocab``, ``width``; ``norm.eps``; ``layers``: a list of {``type``: "attention",
``mixer``: {``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size`` (absent: every earlier token is visible),
``v_mix`` (absent: false)}, ``mlp``: {``kind``: "dense", ``ff``, ``limit``} or {``kind``: "moe", ``expert``: {``ff``,
``limit``}, ``router``: {``experts``, ``top``}} or null}. Tensors of layer i start with ``l<i>.``: ``norm1``, ``norm2``,
``mix.q``, ``mix.k``, ``mix.v``, ``mix.g``, ``mix.o``, ``mix.q.norm``, ``mix.k.norm``, ``mix.r1``, ``mix.r2``, ``mix.sink``,
``mix.vmix``; dense: ``mlp.gate``, ``mlp.up``, ``mlp.down`` with ``.b``; routed: ``mlp.router``, ``mlp.router.b``,
``mlp.e<j>.gate``, ``.up``, ``.down``; ``embed``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.specs import (ClampedGluSpec, ConfigError, LayerSpec, ModelConfig, RmsNormSpec, RoutedExpertsSpec, RunSpec,
                            SinkAttentionSpec)
from ..weights.binding import Ignorable, Stacked

NAME = "Tagenex"
#: no key limits the length of a sequence and no table depends on it, so this only bounds requests
DEFAULT_MAX_POSITION = 1 << 20
#: the slope inside the gate activation g * sigmoid(slope * g) of both kinds of feed-forward
GLU_SLOPE = 1.702


def _get(d, key: str, where: str):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _pos_int(d, key: str, where: str) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    return v


def _number(d, key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _mixer(kind: str, m: dict, where: str, eps: float, source_seen: bool):
    if kind != "attention":
        raise ConfigError(f"config.json: {where}: unknown layer type {kind!r}")
    heads, kv_heads = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    v_mix = m.get("v_mix", False)
    if not isinstance(v_mix, bool):
        raise ConfigError(f"config.json: {where}.v_mix must be true or false, got {v_mix!r}")
    window = _pos_int(m["mask"], "size", where + ".mask") if m.get("mask") is not None else None
    return SinkAttentionSpec(num_heads=heads, num_kv_heads=kv_heads, head_dim=_pos_int(m, "dim", where),
                             value_dim=_pos_int(m, "vdim", where), scale=_number(m, "scale", where), window=window, qk_norm_eps=eps,
                             distance_bias=True, sink=True, value_mix=("mixed" if source_seen else "source") if v_mix else "none",
                             output_gate=True)


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    kind = _get(mlp, "kind", where)
    if kind == "dense":
        return ClampedGluSpec(intermediate_size=_pos_int(mlp, "ff", where), limit=_number(mlp, "limit", where), slope=GLU_SLOPE,
                              bias=True)
    if kind == "moe":
        router, expert = _get(mlp, "router", where), _get(mlp, "expert", where)
        experts, top = _pos_int(router, "experts", where + ".router"), _pos_int(router, "top", where + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {where}.router: {top} of {experts} experts per token")
        return RoutedExpertsSpec(num_experts=experts, top_k=top, expert_size=_pos_int(expert, "ff", where + ".expert"),
                                 correction=False, shared_size=0, shared_gate=False, scoring="softmax_chosen", router_bias=True,
                                 activation="clamped_glu", limit=_number(expert, "limit", where + ".expert"), glu_slope=GLU_SLOPE)
    raise ConfigError(f"config.json: {where}: unknown kind {kind!r}")


def parse_tagenex_config(raw: dict) -> ModelConfig:
    vocab = _pos_int(raw, "vocab", "top level")
    width = _pos_int(raw, "width", "top level")
    eps = _number(_get(raw, "norm", "top level"), "eps", "norm")
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
    layers_raw = _get(raw, "layers", "top level")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    max_pos = raw.get("max_position", DEFAULT_MAX_POSITION)
    if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
        raise ConfigError(f"config.json: 'max_position' must be a positive integer, got {max_pos!r}")
    norm = RmsNormSpec(eps=eps)
    layers, schedule = [], []
    source = None                      # (layer, key/value heads * value size) of the first layer that mixes values
    for i, L in enumerate(layers_raw):
        where = f"layers[{i}]"
        mixer = _mixer(_get(L, "type", where), _get(L, "mixer", where), where, eps, source is not None)
        if mixer.value_mix != "none":
            size = mixer.num_kv_heads * mixer.value_dim
            if source is None:
                source = (i, size)
            elif size != source[1]:
                raise ConfigError(f"config.json: {where}: its values ({size} numbers per token) cannot be mixed with those of "
                                  f"layers[{source[0]}] ({source[1]})")
        ffn = _feed_forward(L.get("mlp"), where + ".mlp")
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=None, ffn_norm=None, arrangement="branch_norm",
                                mixer_post_norm=norm, ffn_post_norm=norm if ffn is not None else None))
        schedule.append(RunSpec(layer=i, cache=i))
    return ModelConfig(architecture=NAME, vocab_size=vocab, hidden_size=width, max_position=max_pos, tie_word_embeddings=False,
                       layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, raw=dict(raw))


def bind_tagenex_weights(config: ModelConfig) -> dict:
    b = {"embed.weight": Stacked(("embed",)), "final_norm.weight": Stacked(("final.norm",)), "head.weight": Stacked(("head",))}
    unused = []
    for i, layer in enumerate(config.layers):
        p, t = f"layers.{i}", f"l{i}"
        m = f"{t}.mix"
        b[f"{p}.mixer_post_norm.weight"] = Stacked((f"{t}.norm1",))
        b[f"{p}.mixer.w_in"] = Stacked((f"{m}.q", f"{m}.k", f"{m}.v", f"{m}.g"))
        b[f"{p}.mixer.q_norm"] = Stacked((f"{m}.q.norm",))
        b[f"{p}.mixer.k_norm"] = Stacked((f"{m}.k.norm",))
        b[f"{p}.mixer.r1"] = Stacked((f"{m}.r1",))
        b[f"{p}.mixer.r2"] = Stacked((f"{m}.r2",))
        b[f"{p}.mixer.sink"] = Stacked((f"{m}.sink",))
        b[f"{p}.mixer.wo"] = Stacked((f"{m}.o",))
        if layer.mixer.value_mix == "mixed":
            b[f"{p}.mixer.value_mix"] = Stacked((f"{m}.vmix",))
        else:
            unused.append(f"{m}.vmix")          # stored for every layer, read by those that mix in another layer's values
        if layer.ffn is None:
            continue
        f = f"{t}.mlp"
        b[f"{p}.ffn_post_norm.weight"] = Stacked((f"{t}.norm2",))
        if isinstance(layer.ffn, ClampedGluSpec):
            b[f"{p}.ffn.w_gate_up"] = Stacked((f"{f}.gate", f"{f}.up"))
            b[f"{p}.ffn.b_gate_up"] = Stacked((f"{f}.gate.b", f"{f}.up.b"))
            b[f"{p}.ffn.w_down"] = Stacked((f"{f}.down",))
            b[f"{p}.ffn.b_down"] = Stacked((f"{f}.down.b",))
        else:
            E = layer.ffn.num_experts
            b[f"{p}.ffn.router"] = Stacked((f"{f}.router",))
            b[f"{p}.ffn.router_bias"] = Stacked((f"{f}.router.b",))
            b[f"{p}.ffn.w_up"] = Stacked(tuple(f"{f}.e{j}.{which}" for j in range(E) for which in ("gate", "up")))
            b[f"{p}.ffn.w_down"] = Stacked(tuple(f"{f}.e{j}.down" for j in range(E)))
    if unused:
        b[Ignorable.KEY] = Ignorable(tuple(unused))
    return b


def make_tagenex_raw_config(*, vocab: int, width: int, layers: list, norm_eps: float = 1e-5) -> dict:
    """``layers``: a list of dicts as config.json holds them ({"type", "mixer", "mlp"})."""
    return {"architecture": NAME, "vocab": vocab, "width": width, "norm": {"eps": norm_eps}, "layers": layers}


register_architecture(Architecture(name=NAME, parse=parse_tagenex_config, bind=bind_tagenex_weights,
                                   make_raw_config=make_tagenex_raw_config), replace=True)
