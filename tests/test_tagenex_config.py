"""Tagenex without a GPU: the configuration reader (every optional key present and absent, every refusal), the binding of
tensor names to parameters, and properties of the plain implementation that the GPU tests compare against."""
import numpy as np
import pytest

import glassbox_b200  # noqa: F401  (registers the architectures)
from glassbox_b200.config.registry import get_architecture, parse_config
from glassbox_b200.config.specs import ClampedGluSpec, ConfigError, RmsNormSpec, RoutedExpertsSpec, SinkAttentionSpec
from glassbox_b200.engine.model import DecoderModel
from glassbox_b200.parts.base import PagedKvSpec
from plain import tagenex_plain as plain
import tagenex_util as tu


@pytest.mark.parametrize("name", sorted(tu.CONFIGS))
def test_every_tensor_is_bound_or_named_as_unused(name):
    from glassbox_b200.weights.binding import Ignorable
    raw = tu.CONFIGS[name]()
    config = parse_config(raw)
    model = DecoderModel(config)
    specs, binding = model.param_specs(), get_architecture("Tagenex").bind(config)
    unused = binding.pop(Ignorable.KEY, None)
    assert set(binding) == set(specs)
    shapes = tu.tensor_shapes(raw)
    named = [n for path in specs for n in binding[path].names] + list(unused.names if unused else ())
    assert sorted(named) == sorted(shapes)
    for path, spec in specs.items():
        names = binding[path].names
        rows = spec.pieces if len(names) > 1 else ((spec.shape[0],) if spec.shape else ())
        for n, r in zip(names, rows):
            assert tuple(shapes[n]) == (r,) + tuple(spec.shape[1:]), n
    # the mixing number is read by the layers that mix another layer's values in, and by no other
    mixing = [i for i, L in enumerate(raw["layers"]) if L["mixer"].get("v_mix")]
    assert sorted(unused.names if unused else ()) == sorted(f"l{i}.mix.vmix" for i in range(len(raw["layers"])) if i not in mixing[1:])


def test_what_the_reader_makes_of_the_keys():
    config = parse_config(tu.CONFIGS["odd"]())
    assert config.vocab_size == 203 and config.hidden_size == 56 and not config.tie_word_embeddings
    assert isinstance(config.final_norm, RmsNormSpec) and config.final_norm.eps == 1e-5
    assert all(l.arrangement == "branch_norm" and l.mixer_norm is None and l.ffn_norm is None for l in config.layers)
    assert all(l.mixer_post_norm.eps == 1e-5 for l in config.layers)
    a, b, c, d, e = config.layers
    assert isinstance(a.mixer, SinkAttentionSpec)
    assert (a.mixer.num_heads, a.mixer.num_kv_heads, a.mixer.head_dim, a.mixer.value_dim, a.mixer.window) == (6, 2, 20, 12, 7)
    assert a.mixer.scale == 20 ** -0.5 and a.mixer.qk_norm_eps == 1e-5 and a.mixer.sink and a.mixer.distance_bias and a.mixer.output_gate
    # layer 0 has no v_mix key, layer 1 is the first that mixes (the source), layer 2 says false, layers 3 and 4 mix
    assert [l.mixer.value_mix for l in config.layers] == ["none", "source", "none", "mixed", "mixed"]
    assert b.mixer.scale == 0.4 and e.mixer.window is None
    assert isinstance(a.ffn, ClampedGluSpec) and (a.ffn.intermediate_size, a.ffn.limit, a.ffn.slope, a.ffn.bias) == (40, 1.5, 1.702, True)
    assert isinstance(b.ffn, RoutedExpertsSpec) and (b.ffn.num_experts, b.ffn.top_k, b.ffn.expert_size, b.ffn.limit) == (6, 2, 24, 0.75)
    assert b.ffn.scoring == "softmax_chosen" and b.ffn.router_bias and b.ffn.activation == "clamped_glu" and b.ffn.shared_size == 0
    assert c.ffn is None and c.ffn_post_norm is None and d.ffn.limit == 3.0
    specs = DecoderModel(config).cache_layer_specs()
    assert specs[0] == PagedKvSpec(2, 20, 7, value_dim=12) and specs[4] == PagedKvSpec(3, 8, None, value_dim=8)
    assert [(r.layer, r.cache) for r in config.schedule] == [(i, i) for i in range(5)]


def _broken(change):
    raw = tu.CONFIGS["odd"]()
    change(raw)
    return raw


@pytest.mark.parametrize("change, word", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].pop("eps"), "eps"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
    (lambda r: r.update(layers=[]), "layers"),
    (lambda r: r["layers"][0].update(type="conv"), "conv"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=4), "multiple"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda r: r["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "size"),
    (lambda r: r["layers"][1]["mixer"].update(v_mix=1), "v_mix"),
    (lambda r: r["layers"][3]["mixer"].update(vdim=12), "mixed"),           # 3 x 12 values cannot mix with layer 1's 3 x 8
    (lambda r: r["layers"][0]["mlp"].update(kind="glu"), "glu"),
    (lambda r: r["layers"][0]["mlp"].pop("limit"), "limit"),
    (lambda r: r["layers"][1]["mlp"]["router"].update(top=7), "7 of 6"),
    (lambda r: r["layers"][1]["mlp"]["expert"].pop("ff"), "ff"),
])
def test_refusals_name_the_key(change, word):
    with pytest.raises(ConfigError) as e:
        parse_config(_broken(change))
    assert word in str(e.value)


def test_random_weights_mode_writes_a_loadable_folder():
    from glassbox_b200.weights.random_init import random_tensors
    raw = tu.CONFIGS["odd"]()
    tensors = random_tensors(raw, seed=3)
    want = tu.tensor_shapes(raw)
    assert set(tensors) <= set(want) and {n for n in want if not n.endswith("mix.vmix")} <= set(tensors)
    for name, t in tensors.items():
        assert tuple(t.shape) == tuple(want[name]), name
    assert float(tensors["l0.mix.r2"].float().min()) > 0            # the logarithm's argument stays above one
    assert abs(float(tensors["l0.mlp.down.b"].float().mean())) < 0.3     # biases around zero, not one


# ------------------------------------------------------------------------------- the plain implementation itself
def _identity_mixer(D, heads=1, **extra):
    W = {"q": np.eye(heads * D), "k": np.eye(D), "v": np.eye(D), "q.norm": np.ones(D), "k.norm": np.ones(D), "o": np.eye(heads * D),
         "g": np.zeros((heads, heads * D)), "r1": np.zeros(heads), "r2": np.ones(heads), "sink": np.full(heads, -1e9),
         "vmix": np.array(0.0)}
    W.update(extra)
    return W


def test_plain_attention_without_bias_or_sink_is_a_windowed_mean():
    """Equal scores, no bias, a sink of minus infinity, a gate logit of zero: half the mean of the visible values."""
    T, D = 12, 4
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 0.0, "mask": {"size": 5}}
    h = np.ones((T, D)) + 0.01 * np.arange(T)[:, None] * np.arange(1, D + 1)
    out, kept = plain.attention(h, _identity_mixer(D), "", m, 1e-6)
    for i in range(T):
        np.testing.assert_allclose(out[i], 0.5 * h[max(0, i - 4):i + 1].mean(0), rtol=1e-9)
    np.testing.assert_array_equal(kept[:, 0], h)
    assert plain.visible(7, 3, 5) and not plain.visible(7, 2, 5) and plain.visible(7, 7, 1) and not plain.visible(7, 6, 1)
    assert plain.visible(7, 0, None) and not plain.visible(3, 4, None)


def test_plain_sink_takes_its_share_and_the_bias_grows_with_distance():
    w = plain.sink_softmax(np.array([0.0, 0.0, 0.0]), 0.0)
    np.testing.assert_allclose(w, [0.25] * 3)                                    # the sink counts once, like a fourth key
    w = plain.sink_softmax(np.array([1.0]), 1.0 + np.log(3.0))
    np.testing.assert_allclose(w, [0.25])
    np.testing.assert_allclose(plain.sink_softmax(np.array([700.0, 699.0]), -700.0).sum(), 1.0)    # (no overflow either way)
    assert plain.distance_bias(0.7, 1.3, 0) == 0.0
    np.testing.assert_allclose(plain.distance_bias(0.5, 2.0, 3), 0.5 * np.log(7.0))
    # with equal dot products a bias r1 = 1, r2 = 1 weighs a key at distance k as 1 / (1 + k)
    T, D = 4, 2
    m = {"heads": 1, "kv_heads": 1, "dim": D, "vdim": D, "scale": 0.0}
    h = np.eye(T, D) + 1.0
    out, _ = plain.attention(h, _identity_mixer(D, r1=np.ones(1)), "", m, 1e-6)
    wts = np.array([1 / 4, 1 / 3, 1 / 2, 1.0])
    np.testing.assert_allclose(out[3], 0.5 * (wts[:, None] * h).sum(0) / wts.sum(), rtol=1e-9)


def test_plain_values_mix_with_the_first_mixing_layers_only():
    v, first = np.full((2, 1, 3), 4.0), np.full((2, 1, 3), 1.0)
    np.testing.assert_array_equal(plain.mix_values(v, None, 0.3), v)
    np.testing.assert_allclose(plain.mix_values(v, first, 0.25), np.full((2, 1, 3), 3.25))
    # in a whole model: three mixing layers; the third mixes with the first one's values, not with the second's mixed ones
    cfg = tu.config(11, 8, [tu.attn(1, 1, 4, 4, v_mix=True), tu.attn(1, 1, 4, 4, v_mix=True), tu.attn(1, 1, 4, 4, v_mix=True)])
    W = tu.as_float64(tu.random_weights(cfg, 2))
    toks = [1, 5, 3, 7]
    base = plain.forward(cfg, W, toks)
    W2 = dict(W); W2["l0.mix.vmix"] = np.array(0.9)                              # the first layer's number is never read
    np.testing.assert_array_equal(plain.forward(cfg, W2, toks), base)
    W3 = dict(W); W3["l2.mix.vmix"] = np.array(1.0)                              # layer 2 then attends over layer 0's values alone
    x = W["embed"][toks]
    y0, v0 = plain.attention(x, W, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6)
    x1 = x + plain.rms_unit(y0, W["l0.norm1"], 1e-6)
    y1, _ = plain.attention(x1, W, "l1.mix.", cfg["layers"][1]["mixer"], 1e-6, v0)
    x2 = x1 + plain.rms_unit(y1, W["l1.norm1"], 1e-6)
    _, v2 = plain.attention(x2, W3, "l2.mix.", cfg["layers"][2]["mixer"], 1e-6, v0)
    np.testing.assert_allclose(v2, v0)


def test_plain_gated_unit_clamps_one_side_of_the_gate_and_both_of_the_other():
    assert plain.gated_unit(np.array(-50.0), np.array(0.0), 2.0) == pytest.approx(0.0, abs=1e-30)   # the gate has no floor
    np.testing.assert_allclose(plain.gated_unit(np.array(9.0), np.array(0.0), 2.0), 2.0 * plain.logistic(1.702 * 2.0))
    np.testing.assert_allclose(plain.gated_unit(np.array(1.0), np.array(-9.0), 2.0), plain.logistic(1.702) * (-1.0))
    np.testing.assert_allclose(plain.gated_unit(np.array(1.0), np.array(9.0), 2.0), plain.logistic(1.702) * 3.0)
    np.testing.assert_allclose(plain.gated_unit(np.array(1.0), np.array(-1.0), 2.0), 0.0)           # u + 1 = 0


def test_plain_router_weighs_the_chosen_logits_alone():
    W = {"router": np.eye(4), "router.b": np.array([0.0, 0.0, 0.0, 2.5])}
    h = np.array([[3.0, 1.0, 2.0, 0.0], [0.0, 0.0, 0.0, -2.5]])
    order, weight = plain.route(h, W, "", {"router": {"experts": 4, "top": 2}})
    np.testing.assert_array_equal(order, [[0, 3], [0, 1]])                       # the bias is part of the logit; equals: lowest index
    np.testing.assert_allclose(weight[0], [1 / (1 + np.exp(-0.5)), 1 / (1 + np.exp(0.5))])
    np.testing.assert_allclose(weight[1], [0.5, 0.5])
    _, one = plain.route(h, W, "", {"router": {"experts": 4, "top": 1}})
    np.testing.assert_array_equal(one, [[1.0], [1.0]])


def test_plain_layer_norms_the_branch_and_not_its_input():
    """Scaling the embedding scales what the branches read: a layer that normed its input would not notice."""
    cfg = tu.config(11, 8, [tu.attn(2, 1, 4, 4, mlp=tu.dense(6, 2.0))])
    W = tu.as_float64(tu.random_weights(cfg, 1))
    toks = [3, 1, 4, 1, 5]
    _, layers = plain.forward(cfg, W, toks, keep_layers=True)
    x = W["embed"][toks]
    branch = layers[0] - x
    y, _ = plain.attention(x, W, "l0.mix.", cfg["layers"][0]["mixer"], 1e-6)
    after_mixer = x + plain.rms_unit(y, W["l0.norm1"], 1e-6)
    np.testing.assert_allclose(branch, after_mixer - x + plain.rms_unit(plain.dense_ff(after_mixer, W, "l0.mlp.", cfg["layers"][0]["mlp"]),
                                                                      W["l0.norm2"], 1e-6))
    W2 = dict(W); W2["embed"] = 2.0 * W["embed"]
    _, layers2 = plain.forward(cfg, W2, toks, keep_layers=True)
    assert np.abs((layers2[0] - 2.0 * x) - branch).max() > 1e-3
