"""Tupunex without a GPU: the configuration reader, the layout of parts and the order of layer runs, the tensor list, and
the plain implementation's mechanisms against hand-made cases."""
import copy

import numpy as np
import pytest

import plain_tupunex as pt
import tupunex_util as tu


def parse(cfg):
    from mimirmind_b200.registry import get_architecture
    entry = get_architecture("Tupunex")
    parsed = entry.parse_config(cfg, "config.json")
    return parsed, entry.build_spec(parsed)


def test_every_size_and_constant_comes_from_the_file():
    parsed, spec = parse(tu.CONFIGS["A"])
    assert (spec.vocab_size, spec.hidden_size, len(spec.layers)) == (101, 64, 4)
    assert [layer.mixer.kind for layer in spec.layers] == ["differential_attention", "latent_attention"] * 2
    assert all(layer.block.kind == "stream_connections" for layer in spec.layers)
    assert all(layer.mixer_norm.kind == "rmsnorm" and layer.mixer_norm["eps"] == 1e-5 for layer in spec.layers)
    assert spec.embedding["scale"] == 1.5 and spec.embedding["copies"] == 3 and spec.final_norm["streams"] == 3
    a = spec.layers[0].mixer
    assert (a["heads"], a["kv_heads"], a["key_dim"], a["value_dim"], a["window"], a["scale"], a["softcap"], a["diff"], a["conv"]) == \
        (4, 2, 16, 24, 23, 0.4, 4.0, 0.3, 4)
    assert a["eps"] == 1e-5 and a["bias"] and a["g"] == "mix.g"
    m = spec.layers[1].mixer
    assert (m["heads"], m["key_dim"], m["rot_dim"], m["value_dim"], m["rank"], m["scale"]) == (3, 8, 12, 10, 20, 0.35)
    assert m["rotary"] == {"dims": 12, "base": 300.0}
    c = spec.layers[0].extras["mixer_connection"]
    assert (c.kind, c.category, c["streams"], c["read"], c["mix"], c["write"], c["scale"]) == \
        ("hyper_connection", "connection", 3, "hc1.in", "hc1.mix", "hc1.out", "ls1")
    assert spec.layers[0].extras["ffn_connection"]["scale"] == "ls2"
    ff = spec.layers[0].feed_forward
    assert (ff.kind, ff["intermediate"]) == ("swiglu", 96)
    assert spec.layers[2].feed_forward.kind == "none" and "ffn_connection" not in spec.layers[2].extras


def test_a_loop_runs_its_layers_in_a_row_each_pass_with_a_cache_of_its_own():
    parsed, spec = parse(tu.CONFIGS["A"])
    assert parsed.order() == (0, 1, 2, 1, 2, 1, 2, 3)
    assert [(e.layer, e.cache_from) for e in spec.schedule] == [(i, None) for i in (0, 1, 2, 1, 2, 1, 2, 3)]
    assert parse(tu.CONFIGS["B"])[0].order() == (0, 1, 1, 2)
    assert parse(tu.CONFIGS["C"])[0].order() == (0, 1, 2, 3, 4)
    assert parse(tu.CONFIGS["D"])[0].order() == (0, 1, 0, 1)
    for name, cfg in tu.CONFIGS.items():
        assert list(parse(cfg)[0].order()) == tu.layer_order(cfg) == pt.layer_order(cfg)
    once = copy.deepcopy(tu.CONFIGS["A"])
    once["loop"]["times"] = 1
    assert parse(once)[0].order() == (0, 1, 2, 3)
    empty = copy.deepcopy(tu.CONFIGS["A"])
    empty["loop"] = {"start": 2, "stop": 2, "times": 5}
    assert parse(empty)[0].order() == (0, 1, 2, 3)


def test_what_may_be_absent():
    parsed, spec = parse(tu.CONFIGS["C"])
    first, third = parsed.layers[0].mixer, parsed.layers[2].mixer
    assert (first.window, first.conv, first.softcap, first.diff) == (1, 1, 0.0, 0.0)
    assert (third.window, third.conv, third.softcap) == (0, 0, 0.0)
    assert parsed.streams == 1 and parsed.loop is None and parsed.embedding_scale == 1.0
    plain, spec = parse(tu.CONFIGS["D"])
    assert plain.streams == 0 and spec.embedding["copies"] == 1 and spec.final_norm["streams"] == 1
    assert spec.layers[0].extras["mixer_connection"]["streams"] == 0


@pytest.mark.parametrize("name", sorted(tu.CONFIGS))
def test_the_declared_tensors_are_the_checkpoints(name):
    from mimirmind_b200.weights.store import expected_tensors
    _, spec = parse(tu.CONFIGS[name])
    declared = expected_tensors(spec)
    assert {k: tuple(v.shape) for k, v in declared.items() if not v.optional} == tu.tensor_shapes(tu.CONFIGS[name])
    # a layer without a feed-forward may still carry the second sublayer's norm, scale and stream weights: allowed, never read
    spare = {k for k, v in declared.items() if v.optional}
    S = tu.CONFIGS[name].get("streams")
    want = set()
    for i, layer in enumerate(tu.CONFIGS[name]["layers"]):
        if layer["mlp"] is None:
            want |= {f"l{i}.norm2", f"l{i}.ls2"} | ({f"l{i}.hc2.in", f"l{i}.hc2.out", f"l{i}.hc2.mix"} if S else set())
    assert spare == want


def _edit(path, value=None, delete=False):
    def apply(cfg):
        node = cfg
        for key in path[:-1]:
            node = node[key]
        if delete:
            del node[path[-1]]
        else:
            node[path[-1]] = value
    return apply


@pytest.mark.parametrize("edit,message", [
    (_edit(["width"], delete=True), "missing required key 'width'"),
    (_edit(["norm", "eps"], delete=True), "missing required key 'norm.eps'"),
    (_edit(["layers", 0, "mixer", "diff"], delete=True), "missing required key 'layers[0].mixer.diff'"),
    (_edit(["layers", 0, "mixer", "kv_heads"], 3), "not a multiple of kv_heads"),
    (_edit(["layers", 1, "mixer", "kv_rank"], delete=True), "missing required key 'layers[1].mixer.kv_rank'"),
    (_edit(["layers", 1, "mixer", "rot", "dims"], 13), "must be even and at most rot_dim"),
    (_edit(["layers", 1, "mixer", "rot", "dims"], 14), "must be even and at most rot_dim"),
    (_edit(["layers", 1, "type"], "attn"), "is not one of 'attention', 'latent_attention'"),
    (_edit(["layers", 0, "mlp", "kind"], "moe"), "is not 'dense'"),
    (_edit(["loop", "stop"], 9), "'loop' runs layers"),
    (_edit(["streams"], 9), "at most 8 residual streams"),
    (_edit(["layers", 0, "mixer", "mask", "size"], 0), "must be an integer >= 1"),
    (_edit(["layers"], []), "non-empty list"),
])
def test_a_wrong_configuration_names_its_key(edit, message):
    from mimirmind_b200.config.model_config import ConfigError
    cfg = copy.deepcopy(tu.CONFIGS["A"])
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        parse(cfg)
    assert message in str(e.value)


def test_the_model_class_is_chosen_by_the_architecture_key():
    from mimirmind_b200.registry import architecture_name, is_supported_architecture
    assert architecture_name(tu.CONFIGS["A"]) == "Tupunex" and is_supported_architecture("Tupunex")


# ---- the plain mechanisms against hand-made cases ---------------------------------------------------------------------
def test_plain_convolution():
    u = np.array([[1.0, 10.0], [2.0, 20.0], [3.0, 30.0], [4.0, 40.0]])
    taps = np.array([[100.0, 10.0, 1.0], [0.0, 0.0, 2.0]])            # last column: the current token
    y = pt.causal_conv(u, taps)
    assert np.allclose(y[:, 0], [1.0, 12.0, 123.0, 234.0]) and np.allclose(y[:, 1], [20.0, 40.0, 60.0, 80.0])


def test_plain_window_and_cap():
    vis = pt.window_visible(5, 2)
    assert vis.tolist() == [[True, False, False, False, False], [True, True, False, False, False], [False, True, True, False, False],
                            [False, False, True, True, False], [False, False, False, True, True]]
    assert pt.window_visible(3, 0).tolist() == [[True, False, False], [True, True, False], [True, True, True]]
    assert abs(pt.soft_cap(np.array([1000.0]), 5.0)[0] - 5.0) < 1e-9 and abs(pt.soft_cap(np.array([0.01]), 5.0)[0] - 0.01) < 1e-7


def test_plain_differential_attention_takes_the_second_map_off_the_first():
    """One head, two tokens, values that are unit vectors: the first map looks at token 0, the second at token 1."""
    big = 50.0
    q = np.zeros((2, 1, 2, 2))
    k = np.zeros((2, 1, 2, 2))
    k[0, 0, 0] = [1.0, 0.0]
    k[1, 0, 0] = [0.0, 1.0]
    k[0, 0, 1] = [1.0, 0.0]
    k[1, 0, 1] = [0.0, 1.0]
    q[1, 0, 0] = [big, 0.0]        # map 1 of token 1 -> key 0
    q[1, 0, 1] = [0.0, big]        # map 2 of token 1 -> key 1
    v = np.array([[[1.0, 0.0]], [[0.0, 1.0]]])
    lam, diff = 0.25, 0.2
    out = pt.differential_attention_core(q, k, v, 1.0, 0.0, 0, lam, diff, 0.0)
    want = np.array([1.0, -lam])
    want = want / np.sqrt(np.mean(want * want)) * (1.0 - diff)
    assert np.allclose(out[1, 0], want, atol=1e-9)
    # token 0 sees only itself in both maps: (1 - lam) v0, whose sign and size the norm keeps as sqrt(2) (1 - diff) on the first place
    assert np.allclose(out[0, 0], [np.sqrt(2.0) * (1.0 - diff), 0.0], atol=1e-9)
    assert abs(pt.differential_lambda(np.array([1.0, 2.0]), np.array([0.5, 0.0]), np.array([0.0, 1.0]), np.array([3.0, 0.0]), 0.3)
               - (np.exp(0.5) - 1.0 + 0.3)) < 1e-12


def test_plain_rotation_pairs_the_halves():
    x = np.array([[1.0, 2.0, 3.0, 4.0, 9.0]])
    y = pt.rotate_half(x, np.array([1.0]), 4, 100.0)
    a0, a1 = 1.0, 100.0 ** -0.5
    assert np.allclose(y[0], [np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1), 3 * np.cos(a0) + np.sin(a0),
                              4 * np.cos(a1) + 2 * np.sin(a1), 9.0])
    assert np.allclose(pt.rotate_half(x, np.array([0.0]), 4, 100.0), x)


def test_plain_streams():
    streams = np.array([[[1.0, 2.0]], [[10.0, 20.0]]])                  # S = 2, one token, width 2
    assert np.allclose(pt.hyper_in(streams, np.array([0.5, 2.0])), [[20.5, 41.0]])
    mix = np.array([[1.0, 3.0], [0.0, 1.0]])                            # [from, to]
    out = pt.hyper_out(streams, np.array([[100.0, 200.0]]), mix, np.array([1.0, -1.0]))
    assert np.allclose(out[0], [[101.0, 202.0]]) and np.allclose(out[1], [[3.0 + 10.0 - 100.0, 6.0 + 20.0 - 200.0]])


def test_plain_latent_attention_equals_its_absorbed_form():
    """Scores and values computed through the per-head up-projections equal those computed on the latent itself."""
    rng = np.random.RandomState(3)
    T, D, H, dk, dr, dv, r = 6, 10, 2, 4, 4, 3, 5
    m = {"heads": H, "dim": dk, "rot_dim": dr, "vdim": dv, "kv_rank": r, "scale": 0.3, "rot": {"dims": dr, "base": 50.0}}
    w = {"q": rng.randn(H * (dk + dr), D), "dkv": rng.randn(r + dr, D), "dkv.norm": 1 + 0.1 * rng.randn(r), "uk": rng.randn(H * dk, r),
         "uv": rng.randn(H * dv, r), "g": rng.randn(H, D), "o": rng.randn(D, H * dv)}
    h = rng.randn(T, D)
    want = pt.latent_attention(h, w, m, 1e-6)
    pos = np.arange(T, dtype=np.float64)
    q = (h @ w["q"].T).reshape(T, H, dk + dr)
    down = h @ w["dkv"].T
    c = pt.rms_norm(down[:, :r], w["dkv.norm"], 1e-6)
    k_rot = pt.rotate_half(down[:, r:], pos, dr, 50.0)
    q_rot = pt.rotate_half(q[:, :, dk:], pos, dr, 50.0)
    out = np.zeros((T, H, dv))
    for i in range(H):
        q_abs = q[:, i, :dk] @ w["uk"][i * dk:(i + 1) * dk]              # [T, r]
        s = (q_abs @ c.T + q_rot[:, i] @ k_rot.T) * 0.3
        p = pt.softmax_rows(s, pt.window_visible(T, 0))
        out[:, i] = (p @ c) @ w["uv"][i * dv:(i + 1) * dv].T
    out = out * pt.sigmoid(h @ w["g"].T)[:, :, None]
    assert np.allclose(out.reshape(T, H * dv) @ w["o"].T, want, atol=1e-10)


def test_a_loop_of_one_pass_and_a_plain_residual_in_the_plain_model():
    cfg = copy.deepcopy(tu.CONFIGS["D"])
    w = {k: v.astype(np.float64) for k, v in tu.random_weights(cfg, 5).items()}
    toks = [3, 1, 4, 1, 5, 9, 2, 6]
    twice = pt.forward(cfg, w, toks)
    cfg["loop"]["times"] = 1
    once = pt.forward(cfg, w, toks)
    del cfg["loop"]
    assert np.array_equal(once, pt.forward(cfg, w, toks)) and not np.allclose(once, twice)
    # one stream that is read, carried on and written with ones is the ordinary residual sum
    cfg["streams"] = 1
    for i, layer in enumerate(cfg["layers"]):
        for q in (1, 2):
            w.update({f"l{i}.hc{q}.in": np.ones(1), f"l{i}.hc{q}.out": np.ones(1), f"l{i}.hc{q}.mix": np.ones((1, 1))})
    assert np.allclose(pt.forward(cfg, w, toks), once, atol=1e-12)
