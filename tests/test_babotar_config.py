"""Babotar without a GPU: the configuration reader (every optional key present and absent, every refusal), the binding of
tensor names to parameters, cache layers that keep pages and states together, and properties of the plain implementation
that the GPU tests compare against."""
import math

import numpy as np
import pytest

import glassbox_b200  # noqa: F401  (registers the architectures)
from glassbox_b200.config.registry import get_architecture, parse_config
from glassbox_b200.config.specs import (ConfigError, DecayLinearAttentionSpec, GeluGluSpec, HeadDeltaSpec, LayerNormSpec, NoPositionSpec,
                                        ParallelMixerSpec, PositionalEmbeddingSpec, TalkingAttentionSpec)
from glassbox_b200.engine.model import DecoderModel
from glassbox_b200.parts.base import CombinedCacheSpec, PagedKvSpec, StateSpec, combine_cache_specs
from plain import babotar_plain as plain
import babotar_util as bu


@pytest.mark.parametrize("name", sorted(bu.CONFIGS))
def test_every_tensor_is_bound(name):
    raw = bu.CONFIGS[name]()
    config = parse_config(raw)
    model = DecoderModel(config)
    specs, binding = model.param_specs(), get_architecture("Babotar").bind(config)
    assert set(binding) == set(specs)
    shapes = bu.tensor_shapes(raw)
    assert sorted(n for path in specs for n in binding[path].names) == sorted(shapes)
    for path, spec in specs.items():
        names = binding[path].names
        rows = spec.pieces if len(names) > 1 else ((spec.shape[0],) if spec.shape else ())
        for n, r in zip(names, rows):
            assert tuple(shapes[n]) == (r,) + tuple(spec.shape[1:]), n


def test_what_the_reader_makes_of_the_keys():
    config = parse_config(bu.CONFIGS["odd"]())
    assert config.vocab_size == 203 and config.hidden_size == 56 and config.max_position == 512 and config.residual_streams == 2
    assert config.embedding == PositionalEmbeddingSpec(max_position=512)
    assert config.final_norm == LayerNormSpec(eps=1e-5, bias=False)
    assert all(l.arrangement == "hyper_connections" and l.streams == 2 and l.learned_streams and l.branch_scale == 0.8
               and l.mixer_input_conv == 2 and l.mixer_norm == config.final_norm for l in config.layers)
    a, b, c, d = config.layers
    assert isinstance(a.mixer, ParallelMixerSpec) and (a.mixer.left_scale, a.mixer.right_scale) == (0.5, 1.3)
    lf, rt = a.mixer.left, a.mixer.right
    assert isinstance(lf, TalkingAttentionSpec) and (lf.num_heads, lf.num_kv_heads, lf.head_dim, lf.value_dim) == (6, 2, 20, 12)
    assert lf.scale == 0.3 and lf.softcap == 5.0 and lf.unit_sink and lf.bias and lf.talk and lf.window is None
    assert (lf.position.theta, lf.position.rotary_dim, lf.position.pairing, lf.position.max_position) == (1000.0, 12, "half", 512)
    assert (lf.position.rescale.factor, lf.position.rescale.original, lf.position.rescale.fast, lf.position.rescale.slow) == (4.0, 64, 8.0, 2.0)
    assert rt == HeadDeltaSpec(num_heads=4, num_kv_heads=2, key_dim=12, value_dim=6, conv_taps=4, norm_eps=1e-5, gate="silu")
    assert b.mixer == DecayLinearAttentionSpec(num_heads=3, head_dim=10, value_dim=6, decay=(0.5, 0.9, 0.99), norm_eps=1e-5)
    assert a.ffn == GeluGluSpec(40) and c.ffn is None and c.ffn_norm is None
    assert d.mixer.left.position.rescale is None
    specs = DecoderModel(config).cache_layer_specs()
    assert specs[0] == CombinedCacheSpec(PagedKvSpec(2, 20, None, value_dim=12),
                                         (("mixer.right", StateSpec((4 * 12 * 6 + 3 * (2 * 2 * 12 + 4 * 6),))), ("input_conv", StateSpec((56,)))))
    assert specs[1] == CombinedCacheSpec(None, (("mixer", StateSpec((3 * 10 * 6,))), ("input_conv", StateSpec((56,)))))


def test_what_a_config_may_leave_out():
    config = parse_config(bu.CONFIGS["plain"]())
    assert config.residual_streams == 1
    assert all(l.streams == 1 and not l.learned_streams and l.branch_scale == 1.0 and l.mixer_input_conv == 0 for l in config.layers)
    a, b, c = config.layers
    assert isinstance(a.mixer.left.position, NoPositionSpec) and a.mixer.left.softcap is None
    assert (a.mixer.left_scale, a.mixer.right_scale) == (1.0, 1.0) and c.mixer.left.position.rescale is None
    model = DecoderModel(config)
    assert not any("streams" in p or "mixer_conv" in p for p in model.param_specs())
    # without a convolution on the input the layer's cache layer is its mixer's
    assert model.cache_layer_specs()[1] == StateSpec((2 * 8 * 24,))
    assert model.cache_layer_specs()[0] == CombinedCacheSpec(PagedKvSpec(1, 16, None, value_dim=16), (("right", StateSpec((2 * 8 * 8 + 2 * 48,))),))
    one = parse_config(bu.CONFIGS["ones"]())
    assert one.residual_streams == 1 and all(l.learned_streams and l.mixer_input_conv == 1 for l in one.layers)


def _broken(change):
    raw = bu.CONFIGS["odd"]()
    change(raw)
    return raw


@pytest.mark.parametrize("change, word", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r.pop("max_positions"), "max_positions"),
    (lambda r: r.__setitem__("streams", 9), "streams"),
    (lambda r: r.__setitem__("streams", 0), "streams"),
    (lambda r: r["norm"].__setitem__("eps", 0.0), "eps"),
    (lambda r: r["canon"].__setitem__("taps", 0), "taps"),
    (lambda r: r["layers"][0].__setitem__("type", "conv"), "unknown layer type"),
    (lambda r: r["layers"][0]["mixer"]["left"].__setitem__("kv_heads", 4), "multiple"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 13), "even"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"].__setitem__("dims", 22), "at most dim"),
    (lambda r: r["layers"][0]["mixer"]["left"].__setitem__("softcap", -1.0), "softcap"),
    (lambda r: r["layers"][0]["mixer"]["left"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda r: r["layers"][0]["mixer"]["right"].pop("conv"), "conv"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.9]), "decay"),
    (lambda r: r["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.9, 1.5]), "decay"),
    (lambda r: r["layers"][0]["mlp"].__setitem__("kind", "moe"), "unknown kind"),
    (lambda r: r.__setitem__("layers", []), "layers"),
])
def test_refusals_name_the_key(change, word):
    with pytest.raises(ConfigError) as e:
        parse_config(_broken(change))
    assert word in str(e.value)


def test_cache_specs_combine():
    paged, st = PagedKvSpec(2, 8, None, value_dim=4), StateSpec((5,))
    assert combine_cache_specs([("", paged)]) is paged
    assert combine_cache_specs([("left", paged), ("right", None)]) is paged
    assert combine_cache_specs([("left", None), ("right", st)]) == CombinedCacheSpec(None, (("right", st),))
    both = combine_cache_specs([("left", paged), ("right", st)])
    assert both == CombinedCacheSpec(paged, (("right", st),))
    assert combine_cache_specs([("mixer", both), ("conv", st)]) == CombinedCacheSpec(paged, (("mixer.right", st), ("conv", st)))
    with pytest.raises(ValueError):
        combine_cache_specs([("left", paged), ("right", paged)])


# ----------------------------------------------------------------------------- the plain implementation's own equations
def test_stretched_frequencies():
    """Pairs that turn often keep their frequency, slow pairs are slowed by the factor, the ramp lies between, and the table
    the engine builds holds the same angles and the factor on sine and cosine."""
    from glassbox_b200.config.specs import RopeRescaleSpec
    from glassbox_b200.parts.rope import rotary_table
    r = bu.rot(32, 10000.0, (8.0, 256, 16.0, 1.0))
    f, mag = plain.rotary_frequencies(r)
    base = np.array([10000.0 ** (-2.0 * i / 32) for i in range(16)])
    turns = 256 * base / (2 * math.pi)
    assert mag == pytest.approx(0.1 * math.log(8.0) + 1.0)
    assert np.allclose(f[turns > 20], base[turns > 20]) and np.allclose(f[turns < 0.8], base[turns < 0.8] / 8.0)
    assert np.all(f <= base + 1e-15) and np.all(f >= base / 8.0 - 1e-15) and np.any((f < base * 0.99) & (f > base / 8.0 * 1.01))
    table = rotary_table(10000.0, 32, 300, RopeRescaleSpec(8.0, 256, 16.0, 1.0)).numpy()
    ang = np.arange(300)[:, None] * f[None, :]
    assert np.abs(table[..., 0] - np.cos(ang) * mag).max() < 3e-5 and np.abs(table[..., 1] - np.sin(ang) * mag).max() < 3e-5
    plain_table = rotary_table(10000.0, 32, 300).numpy()
    assert np.abs(plain_table[..., 0] - np.cos(np.arange(300)[:, None] * base[None, :])).max() < 3e-5


def test_rotation_keeps_relative_angles():
    rng = np.random.default_rng(0)
    r = bu.rot(8, 100.0)
    q, k = rng.standard_normal((1, 1, 12)), rng.standard_normal((1, 1, 12))
    a = plain.rotate_half(q, [7], r)[0, 0] @ plain.rotate_half(k, [3], r)[0, 0]
    b = plain.rotate_half(q, [29], r)[0, 0] @ plain.rotate_half(k, [25], r)[0, 0]
    assert a == pytest.approx(b)
    assert np.array_equal(plain.rotate_half(q, [5], r)[..., 8:], q[..., 8:])          # the rest passes unchanged


def test_the_sink_takes_its_share_and_an_identity_mix_changes_nothing():
    rng = np.random.default_rng(1)
    H, G, D, V, T = 2, 1, 4, 3, 6
    m = bu.left(H, G, D, V, scale=0.5)
    W = {"q": np.zeros((H * D, 5)), "k": np.zeros((G * D, 5)), "v": rng.standard_normal((G * V, 5)), "q.b": np.zeros(H * D),
         "k.b": np.zeros(G * D), "v.b": np.zeros(G * V), "talk": np.eye(H), "o": np.eye(H * V)}
    h = rng.standard_normal((T, 5))
    out = plain.talking_softmax_attention(h, W, "", m).reshape(T, H, V)
    v = h @ W["v"].T
    for t in range(T):                                  # all scores 0: each of t + 1 keys and the sink weigh 1 / (t + 2)
        assert np.allclose(out[t, 0], v[:t + 1].sum(0) / (t + 2))
    W["talk"] = np.array([[0.0, 2.0], [1.0, 0.0]])
    W["q"], W["k"] = rng.standard_normal((H * D, 5)), rng.standard_normal((G * D, 5))
    mixed = plain.talking_softmax_attention(h, W, "", m).reshape(T, H, V)
    W["talk"] = np.eye(H)
    own = plain.talking_softmax_attention(h, W, "", m).reshape(T, H, V)
    assert np.allclose(mixed[:, 0], 2.0 * own[:, 1]) and np.allclose(mixed[:, 1], own[:, 0])      # one shared key/value head


def test_the_delta_rule_recalls_what_it_stored():
    """With no decay, beta one and orthonormal keys, reading with a stored key returns its value."""
    D, V, T = 4, 3, 4
    rng = np.random.default_rng(2)
    S = np.zeros((D, V))
    keys, vals = np.eye(D), rng.standard_normal((T, V))
    for t in range(T):
        u = 1.0 * (vals[t] - S.T @ keys[t])
        S = S + np.outer(keys[t], u)
    for t in range(T):
        assert np.allclose(S.T @ keys[t], vals[t])


def test_lightning_with_decay_one_is_a_running_sum_and_with_zero_forgets():
    rng = np.random.default_rng(3)
    T, D, V = 5, 3, 2
    h = rng.standard_normal((T, 2 * D + 2 * V))
    eye = np.eye(2 * D + 2 * V)
    W = {"q": eye[:D], "k": eye[D:2 * D], "v": eye[2 * D:2 * D + V], "g": eye[2 * D + V:], "o": np.eye(V), "norm": np.ones(V)}
    q, k, v = plain.silu(h[:, :D]), plain.silu(h[:, D:2 * D]), plain.silu(h[:, 2 * D:2 * D + V])
    gate = plain.logistic(h[:, 2 * D + V:])
    for decay, keep in ((1.0, lambda t, j: 1.0), (0.0, lambda t, j: float(t == j))):
        out = plain.lightning(h, W, "", {"heads": 1, "dim": D, "vdim": V, "decay": [decay]}, 1e-6)
        for t in range(T):
            o = sum(keep(t, j) * (q[t] @ k[j]) * v[j] for j in range(t + 1))
            assert np.allclose(out[t], plain.rms_unit(o, 1e-6) * gate[t])


def test_convolution_and_streams():
    x = np.arange(12.0).reshape(6, 2)
    w = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = plain.causal_conv(x, w)
    assert np.array_equal(y[:, 1], x[:, 1]) and y[0, 0] == 0.0 and y[2, 0] == 1.0 * 0 + 10.0 * 2 + 100.0 * 4
    # one learned stream with unit weights is the plain residual with the factor on every branch
    cfg = bu.CONFIGS["ones"]()
    W = bu.as_float64(bu.random_weights(cfg, 3))
    for k in W:
        if ".hc" in k:
            W[k] = np.ones_like(W[k])
    cfg["residual_mult"] = 0.5
    a = plain.forward(cfg, W, [3, 1, 4, 1, 5])
    cfg2 = dict(cfg)
    cfg2.pop("streams")
    assert np.allclose(a, plain.forward(cfg2, W, [3, 1, 4, 1, 5]))
