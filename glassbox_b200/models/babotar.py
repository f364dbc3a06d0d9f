"""Babotar: a decoder with a learned position vector on the embedding, whose layers mix tokens either with lightning
attention (linear attention with one fixed decay per head, the heads normed together and gated) or with two mixers side by
side on the same input: softmax attention whose heads exchange their weights (biased projections, a rotation of the leading
channels with stretched frequencies, capped scores, one more unit in the softmax's denominator) and a gated delta rule with
one decay per head; whose feed-forwards are gated units with the tanh form of GELU; whose norms are layer norms without
bias; whose mixers read their normed input through a short causal convolution added to it; whose branches are scaled by a
constant; and whose residual may be kept as several streams (hyper-connections).

This file only *describes* the architecture: which config.json keys it reads and how tensor names map onto part parameters.
The math lives in the parts (``parts/linear_attention.py``, ``parts/talking_attention.py``, ``parts/delta_rule.py``,
``parts/parallel.py``, ``parts/mlp.py``, ``parts/block.py``, ``parts/embedding.py``).

config.json: ``architecture`` "Babotar"; ``vocab``, ``width``, ``max_positions``; ``norm.eps``; ``residual_mult`` (absent: 1);
``streams`` (absent: one plain residual row); ``canon.taps`` (absent: no convolution on the mixers' input); ``layers``: a list
of {``type``: "lightning" | "parallel", ``mixer``: sizes, ``mlp``: {``kind``: "dense", ``ff``} or null}. A lightning mixer
gives ``heads``, ``dim``, ``vdim``, ``decay`` (a list, one per head); a parallel mixer ``left`` (``heads``, ``kv_heads``,
``dim``, ``vdim``, ``scale``, ``softcap`` (absent: none), ``rot``: {``base``, ``dims``, ``scaling``: {``factor``,
``original``, ``fast``, ``slow``} (absent: plain frequencies)} (absent: no rotation)), ``right`` (``heads``, ``kv_heads``,
``dim``, ``vdim``, ``conv``), ``left_scale``, ``right_scale``. Tensors of layer i start with ``l<i>.``: ``norm1`` (mixer
``mix.*``), ``norm2`` (feed-forward ``mlp.*``), ``hc1.*`` / ``hc2.*`` (``in``, ``out``, ``mix`` of the two branches' stream
mixing), ``canon1``; ``embed``, ``pos``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.specs import (ConfigError, DecayLinearAttentionSpec, GeluGluSpec, HeadDeltaSpec, LayerNormSpec, LayerSpec, ModelConfig,
                            NoPositionSpec, ParallelMixerSpec, PositionalEmbeddingSpec, RopeRescaleSpec, RopeSpec, RunSpec,
                            TalkingAttentionSpec)
from ..weights.binding import Stacked

NAME = "Babotar"


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


def _heads(m: dict, where: str):
    heads = _pos_int(m, "heads", where)
    kv_heads = _pos_int(m, "kv_heads", where) if "kv_heads" in m else heads
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}: heads {heads} is not a multiple of kv_heads {kv_heads}")
    return heads, kv_heads


def _left(m: dict, where: str, max_pos: int):
    heads, kv_heads = _heads(m, where)
    dim = _pos_int(m, "dim", where)
    position = NoPositionSpec()
    if m.get("rot") is not None:
        rot = m["rot"]
        dims = _pos_int(rot, "dims", where + ".rot")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {where}: rot.dims {dims} must be even and at most dim {dim}")
        base = _number(rot, "base", where + ".rot")
        if not base > 1:
            raise ConfigError(f"config.json: {where}.rot.base must be above 1, got {base!r}")
        rescale = None
        if rot.get("scaling") is not None:
            sc, w = rot["scaling"], where + ".rot.scaling"
            rescale = RopeRescaleSpec(factor=_number(sc, "factor", w), original=_number(sc, "original", w),
                                      fast=_number(sc, "fast", w), slow=_number(sc, "slow", w))
            if not (rescale.factor > 0 and rescale.original > 0 and rescale.fast > 0 and rescale.slow > 0):
                raise ConfigError(f"config.json: {w}: factor, original, fast and slow must be positive")
        position = RopeSpec(theta=base, rotary_dim=dims, max_position=max_pos, pairing="half", rescale=rescale)
    softcap = _number(m, "softcap", where) if m.get("softcap") is not None else None
    if softcap is not None and not softcap > 0:
        raise ConfigError(f"config.json: {where}.softcap must be positive, got {softcap!r}")
    return TalkingAttentionSpec(num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=_pos_int(m, "vdim", where),
                                scale=_number(m, "scale", where), position=position, softcap=softcap, unit_sink=True, bias=True,
                                talk=True, window=None)


def _right(m: dict, where: str, eps: float):
    heads, kv_heads = _heads(m, where)
    return HeadDeltaSpec(num_heads=heads, num_kv_heads=kv_heads, key_dim=_pos_int(m, "dim", where),
                         value_dim=_pos_int(m, "vdim", where), conv_taps=_pos_int(m, "conv", where), norm_eps=eps, gate="silu")


def _mixer(kind: str, m: dict, where: str, eps: float, max_pos: int):
    if kind == "lightning":
        heads = _pos_int(m, "heads", where)
        decay = _get(m, "decay", where)
        if not isinstance(decay, list) or len(decay) != heads or not all(
                isinstance(g, (int, float)) and not isinstance(g, bool) and 0 <= g <= 1 for g in decay):
            raise ConfigError(f"config.json: {where}.decay must list one number in [0, 1] per head ({heads})")
        return DecayLinearAttentionSpec(num_heads=heads, head_dim=_pos_int(m, "dim", where), value_dim=_pos_int(m, "vdim", where),
                                        decay=tuple(float(g) for g in decay), norm_eps=eps)
    if kind == "parallel":
        return ParallelMixerSpec(left=_left(_get(m, "left", where), where + ".left", max_pos),
                                 right=_right(_get(m, "right", where), where + ".right", eps),
                                 left_scale=_number(m, "left_scale", where) if "left_scale" in m else 1.0,
                                 right_scale=_number(m, "right_scale", where) if "right_scale" in m else 1.0)
    raise ConfigError(f"config.json: {where}: unknown layer type {kind!r}")


def _feed_forward(mlp, where: str):
    if mlp is None:
        return None
    if _get(mlp, "kind", where) != "dense":
        raise ConfigError(f"config.json: {where}: unknown kind {mlp['kind']!r}")
    return GeluGluSpec(intermediate_size=_pos_int(mlp, "ff", where))


def parse_babotar_config(raw: dict) -> ModelConfig:
    vocab = _pos_int(raw, "vocab", "top level")
    width = _pos_int(raw, "width", "top level")
    max_pos = _pos_int(raw, "max_positions", "top level")
    eps = _number(_get(raw, "norm", "top level"), "eps", "norm")
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
    learned = raw.get("streams") is not None
    streams = _pos_int(raw, "streams", "top level") if learned else 1
    if streams > 8:
        raise ConfigError(f"config.json: {streams} streams; at most 8 are supported")
    mult = _number(raw, "residual_mult", "top level") if raw.get("residual_mult") is not None else 1.0
    taps = _pos_int(raw["canon"], "taps", "canon") if raw.get("canon") is not None else 0
    if taps > 64:
        raise ConfigError(f"config.json: canon.taps {taps}; at most 64 are supported")
    layers_raw = _get(raw, "layers", "top level")
    if not isinstance(layers_raw, list) or not layers_raw:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    norm = LayerNormSpec(eps=eps, bias=False)
    layers, schedule = [], []
    for i, L in enumerate(layers_raw):
        where = f"layers[{i}]"
        mixer = _mixer(_get(L, "type", where), _get(L, "mixer", where), where + ".mixer", eps, max_pos)
        ffn = _feed_forward(L.get("mlp"), where + ".mlp")
        # without 'streams' the residual is one row that every branch reads as it is and adds to: hyper-connections over one
        # stream with no learned weights
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm if ffn is not None else None,
                                arrangement="hyper_connections", streams=streams, learned_streams=learned, branch_scale=mult,
                                mixer_input_conv=taps))
        schedule.append(RunSpec(layer=i, cache=i))
    return ModelConfig(architecture=NAME, vocab_size=vocab, hidden_size=width, max_position=max_pos, tie_word_embeddings=False,
                       layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, raw=dict(raw),
                       embedding=PositionalEmbeddingSpec(max_position=max_pos), residual_streams=streams)


def bind_babotar_weights(config: ModelConfig) -> dict:
    b = {"embed.weight": Stacked(("embed",)), "embed.positions": Stacked(("pos",)), "final_norm.weight": Stacked(("final.norm",)),
         "head.weight": Stacked(("head",))}
    for i, layer in enumerate(config.layers):
        p, t = f"layers.{i}", f"l{i}"
        m = f"{t}.mix"
        branches = [("mixer", "norm1", "hc1")] + ([("ffn", "norm2", "hc2")] if layer.ffn is not None else [])
        for part, norm, hc in branches:
            b[f"{p}.{part}_norm.weight"] = Stacked((f"{t}.{norm}",))
            if layer.learned_streams:
                b[f"{p}.{part}_streams.read"] = Stacked((f"{t}.{hc}.in",))
                b[f"{p}.{part}_streams.write"] = Stacked((f"{t}.{hc}.out",))
                b[f"{p}.{part}_streams.mix"] = Stacked((f"{t}.{hc}.mix",))
        if layer.mixer_input_conv:
            b[f"{p}.mixer_conv.weight"] = Stacked((f"{t}.canon1",))
        if isinstance(layer.mixer, DecayLinearAttentionSpec):
            b[f"{p}.mixer.w_in"] = Stacked((f"{m}.q", f"{m}.k", f"{m}.v", f"{m}.g"))
            b[f"{p}.mixer.out_norm"] = Stacked((f"{m}.norm",))
            b[f"{p}.mixer.wo"] = Stacked((f"{m}.o",))
        else:
            lf, rt = f"{m}.left", f"{m}.right"
            b[f"{p}.mixer.left.w_in"] = Stacked((f"{lf}.q", f"{lf}.k", f"{lf}.v"))
            b[f"{p}.mixer.left.b_in"] = Stacked((f"{lf}.q.b", f"{lf}.k.b", f"{lf}.v.b"))
            b[f"{p}.mixer.left.talk"] = Stacked((f"{lf}.talk",))
            b[f"{p}.mixer.left.wo"] = Stacked((f"{lf}.o",))
            b[f"{p}.mixer.right.w_in"] = Stacked((f"{rt}.q", f"{rt}.k", f"{rt}.v", f"{rt}.a", f"{rt}.b", f"{rt}.g"))
            b[f"{p}.mixer.right.conv"] = Stacked((f"{rt}.q.conv", f"{rt}.k.conv", f"{rt}.v.conv"))
            b[f"{p}.mixer.right.dt_bias"] = Stacked((f"{rt}.dt_bias",))
            b[f"{p}.mixer.right.a_log"] = Stacked((f"{rt}.A_log",))
            b[f"{p}.mixer.right.out_norm"] = Stacked((f"{rt}.norm",))
            b[f"{p}.mixer.right.wo"] = Stacked((f"{rt}.o",))
        if layer.ffn is not None:
            f = f"{t}.mlp"
            b[f"{p}.ffn.w_gate_up"] = Stacked((f"{f}.gate", f"{f}.up"))
            b[f"{p}.ffn.w_down"] = Stacked((f"{f}.down",))
    return b


def make_babotar_raw_config(*, vocab: int, width: int, max_positions: int, layers: list, streams=None, residual_mult=None,
                            canon_taps=None, norm_eps: float = 1e-6) -> dict:
    """``layers``: a list of dicts as config.json holds them ({"type", "mixer", "mlp"})."""
    raw = {"architecture": NAME, "vocab": vocab, "width": width, "max_positions": max_positions, "norm": {"eps": norm_eps},
           "layers": layers}
    if streams is not None:
        raw["streams"] = streams
    if residual_mult is not None:
        raw["residual_mult"] = residual_mult
    if canon_taps is not None:
        raw["canon"] = {"taps": canon_taps}
    return raw


register_architecture(Architecture(name=NAME, parse=parse_babotar_config, bind=bind_babotar_weights,
                                   make_raw_config=make_babotar_raw_config), replace=True)
