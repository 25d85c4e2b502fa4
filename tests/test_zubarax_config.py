"""Zubarax without a GPU: the reader of its config.json and its messages, the layout of parts and schedule entries, the
declared tensors against the names a checkpoint uses, and the plain implementation's mechanisms against hand-made cases."""
import copy

import numpy as np
import pytest

import plain_zubarax as pz
import zubarax_util as zu
from mimirmind_b200.config.model_config import ConfigError
from mimirmind_b200.registry import get_architecture, is_supported_architecture
from mimirmind_b200.weights.store import expected_tensors


def spec_of(cfg):
    entry = get_architecture("Zubarax")
    return entry.build_spec(entry.parse_config(cfg, "config.json"))


def test_the_architecture_is_registered_and_read():
    assert is_supported_architecture("Zubarax")
    cfg = get_architecture("Zubarax").parse_config(zu.CONFIGS["A"], "config.json")
    assert (cfg.vocab, cfg.width, cfg.alpha, cfg.embedding_scale) == (101, 64, 2.0, 4.0)
    assert [layer.weights_of for layer in cfg.layers] == [None, None, 0, None, 1]
    assert cfg.layers[0].mixer.left.rot_dims == 12 and cfg.layers[3].mixer.left.rot_dims == 0 and cfg.layers[3].mixer.left.conv == 0
    assert cfg.layers[0].mlp.shared.ff == 24 and cfg.layers[1].mlp.shared is None and cfg.layers[3].mlp is None
    bare = get_architecture("Zubarax").parse_config(zu.CONFIGS["C"], "config.json")
    assert bare.alpha == 1.0 and bare.embedding_scale == 1.0


@pytest.mark.parametrize("name", sorted(zu.CONFIGS))
def test_declared_tensors_are_the_checkpoints(name):
    cfg = zu.CONFIGS[name]
    spec = spec_of(cfg)
    exp = expected_tensors(spec)
    have = zu.tensor_shapes(cfg)
    required = {k for k, v in exp.items() if not v.optional}
    assert required == set(have)
    for k, shape in have.items():
        assert tuple(exp[k].shape) == tuple(shape), k


def test_layers_that_share_tensors_are_schedule_entries_of_their_own():
    spec = spec_of(zu.CONFIGS["A"])
    assert len(spec.layers) == 3 and [l.prefix for l in spec.layers] == ["l0.", "l1.", "l3."]
    assert [(e.layer, e.cache_from) for e in spec.schedule] == [(0, None), (1, None), (0, None), (2, None), (1, None)]
    assert spec.layers[2].feed_forward.kind == "none" and spec.layers[0].block.kind == "post_norm" and spec.layers[0].block["alpha"] == 2.0
    left = spec.layers[0].mixer["left"]
    assert left.kind == "talking_attention" and left["rotary"] == {"dims": 12, "base": 100.0} and spec.layers[2].mixer["left"]["rotary"] is None
    assert spec.layers[0].mixer["right"]["decay"] == "forget_gate" and spec.head["tied_to"] == "embed"
    ffn = spec.layers[0].feed_forward
    assert (ffn["scoring"], ffn["weight_on"], ffn["activation"], ffn["limit"], ffn["shared"]["limit"]) == ("sigmoid", "input", "clamped", 1.5, 0.8)


@pytest.mark.parametrize("edit,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["layers"][0]["mixer"]["left"].pop("scale"), "layers[0].mixer.left.scale"),
    (lambda c: c["layers"][0]["mixer"].pop("right_scale"), "layers[0].mixer.right_scale"),
    (lambda c: c["layers"][0]["mixer"]["left"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][0].update(type="serial"), "'parallel'"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "'moe'"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "cannot be chosen"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "layers[0].mlp.expert.limit"),
    (lambda c: c["layers"][2].update(weights_of=4), "tensors of its own"),
    (lambda c: c["layers"][2]["mixer"].update(left_scale=9.0), "another mixer"),
])
def test_what_the_reader_refuses(edit, message):
    cfg = copy.deepcopy(zu.CONFIGS["A"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        get_architecture("Zubarax").parse_config(cfg, "config.json")
    assert message in str(e.value)


# ---- the plain mechanisms against hand-made cases -----------------------------------------------------------------------
def test_plain_convolution_and_rotation():
    u = np.arange(1.0, 6.0)[:, None] * np.ones((1, 2))
    taps = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]])
    y = pz.short_conv(u, taps)
    assert np.allclose(y[:, 0], [100.0, 210.0, 321.0, 432.0, 543.0]) and np.allclose(y[:, 1], u[:, 1])
    x = np.zeros((2, 1, 6))
    x[:, 0, 0] = 1.0
    x[:, 0, 5] = 7.0
    r = pz.rotate_half(x, [0, 3], 4, 10.0)
    assert np.allclose(r[0], x[0]) and np.allclose(r[1, 0], [np.cos(3.0), 0.0, np.sin(3.0), 0.0, 0.0, 7.0])


def test_plain_mixed_heads_and_sink():
    rng = np.random.RandomState(0)
    q, k, v = rng.randn(5, 2, 4), rng.randn(5, 1, 4), rng.randn(5, 1, 3)
    none = np.array([-1e9, -1e9])
    plain = pz.talking_sink_attention_core(q, k, v, np.eye(2), none, 0.5)
    s = (q[4, 1] @ k[:, 0].T) * 0.5
    p = np.exp(s - s.max())
    assert np.allclose(plain[4, 1], (p / p.sum()) @ v[:, 0])
    swapped = pz.talking_sink_attention_core(q, k, v, np.array([[0.0, 1.0], [1.0, 0.0]]), none, 0.5)
    assert np.allclose(swapped[:, 0], plain[:, 1]) and np.allclose(swapped[:, 1], plain[:, 0])
    # a sink as large as the only score takes half of the first token's weight
    one = pz.talking_sink_attention_core(q[:1], k[:1], v[:1], np.eye(2), np.array([(q[0, 0] @ k[0, 0]) * 0.5, -1e9]), 0.5)
    assert np.allclose(one[0, 0], 0.5 * v[0, 0]) and np.allclose(one[0, 1], v[0, 0])


def test_plain_forget_gate_state():
    q = np.ones((3, 1, 2))
    f = np.array([[[0.5, 0.0]], [[0.5, 1.0]], [[0.0, 0.25]]])
    v = np.array([[[2.0]], [[4.0]], [[8.0]]])
    o = pz.hgrn2_core(q, f, v)
    # row 0: 1, 0.5 + 2, 8; row 1: 2, 2, 0.5 + 6
    assert np.allclose(o[:, 0, 0], [1.0 + 2.0, 2.5 + 2.0, 8.0 + 6.5])


def test_plain_experts_weigh_their_input():
    rng = np.random.RandomState(1)
    w = {"r": rng.randn(3, 4)}
    for e in range(3):
        w.update({f"e{e}.gate": rng.randn(5, 4), f"e{e}.up": rng.randn(5, 4), f"e{e}.down": rng.randn(4, 5)})
    w["router"] = w.pop("r")
    h = rng.randn(2, 4)
    idx, s = pz.router_choice(h, w["router"], 2)
    z = 1.0 / (1.0 + np.exp(-(h @ w["router"].T)))
    assert np.array_equal(idx[0], np.argsort(-z[0])[:2]) and np.allclose(s[0], np.sort(z[0])[::-1][:2])
    out = pz.experts_feed_forward(h, w, "", {"router": {"top": 2}, "expert": {"limit": 0.5}})
    e0 = int(idx[0, 0])
    g = np.minimum((s[0, 0] * h[0]) @ w[f"e{e0}.gate"].T, 0.5)
    u = np.clip((s[0, 0] * h[0]) @ w[f"e{e0}.up"].T, -0.5, 0.5)
    first = (g / (1.0 + np.exp(-1.702 * g)) * (u + 1.0)) @ w[f"e{e0}.down"].T
    other = pz.clamped_expert(s[0, 1] * h[:1], w, f"e{int(idx[0, 1])}", 0.5)[0]
    assert np.allclose(out[0], first + other)
