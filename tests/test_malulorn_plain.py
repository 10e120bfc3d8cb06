"""The Malulorn oracle against the same mechanisms written the other way round, and the configuration, tensor list
and schedule of the product - all without a GPU."""
import json

import numpy as np
import pytest

import plain_malulorn as pm
import tiny_malulorn as tm
from cpp_minilamma_b200.config.base import ConfigError, config_from_dict
from cpp_minilamma_b200.config.malulorn import MalulornConfig
from cpp_minilamma_b200.models.malulorn import build_malulorn_spec


def test_sink_attention_row_by_row():
    """The oracle's dense form against one query at a time: p_j = exp(s_j) / (1 + sum exp(s_j))."""
    rng = np.random.RandomState(1)
    m = {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 5, "scale": 0.4, "q_temp": {"coef": 0.5, "every": 3}}
    D, T = 12, 11
    W = {"q": rng.randn(24, D), "k": rng.randn(12, D), "v": rng.randn(10, D), "g": rng.randn(4, D), "o": rng.randn(D, 20)}
    h = rng.randn(T, D)
    got = pm.sink_attention(h, W, "", m)
    want = np.zeros((T, D))
    for i in range(T):
        temp = 1 + 0.5 * np.log((i + 1) // 3 + 1)
        heads = []
        for head in range(4):
            q = (W["q"] @ h[i])[head * 6:(head + 1) * 6] * temp
            kv = head // 2
            s = np.array([0.4 * q @ (W["k"] @ h[j])[kv * 6:(kv + 1) * 6] for j in range(i + 1)])
            p = np.exp(s) / (1 + np.exp(s).sum())
            o = sum(p[j] * (W["v"] @ h[j])[kv * 5:(kv + 1) * 5] for j in range(i + 1))
            heads.append(o / (1 + np.exp(-(W["g"] @ h[i])[head])))
        want[i] = W["o"] @ np.concatenate(heads)
    assert np.abs(got - want).max() < 1e-10
    # the first token sees one key, yet its weight is not one: the sink takes its share
    assert np.abs(pm.sink_attention(h[:1], W, "", m) - want[:1]).max() < 1e-10


def test_latent_attention_equals_its_absorbed_form():
    """Expanding keys and values per head (the oracle) and attending over the latent rows themselves
    (q~ = W_uk^T q, values = c, then W_uv) are the same function."""
    rng = np.random.RandomState(2)
    m = {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 5, "kv_rank": 7, "scale": 0.3, "rot": {"base": 50.0, "dims": 4}}
    D, T, eps = 10, 9, 1e-5
    W = {"q": rng.randn(30, D), "dkv": rng.randn(11, D), "dkv.norm": 1 + 0.3 * rng.randn(7), "uk": rng.randn(18, 7),
         "uv": rng.randn(15, 7), "g": rng.randn(15, D), "o": rng.randn(D, 15)}
    h = rng.randn(T, D)
    got = pm.latent_attention(h, W, "", m, eps)
    pos = np.arange(T, dtype=np.float64)
    q = (h @ W["q"].T).reshape(T, 3, 10)
    down = h @ W["dkv"].T
    c = pm.rms(down[:, :7], eps) * W["dkv.norm"]
    rows = np.concatenate([c, pm.rotate_pairs(down[:, 7:], pos, 50.0)], axis=1)  # what a cache would hold
    heads = []
    for head in range(3):
        q_abs = np.concatenate([q[:, head, :6] @ W["uk"][head * 6:(head + 1) * 6], pm.rotate_pairs(q[:, head, 6:], pos, 50.0)], axis=1)
        s = np.where(pm.causal_mask(T), 0.3 * q_abs @ rows.T, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        heads.append((p @ c) @ W["uv"][head * 5:(head + 1) * 5].T)
    want = (np.concatenate(heads, axis=1) * pm.sigmoid(h @ W["g"].T)) @ W["o"].T
    assert np.abs(got - want).max() < 1e-10


def test_rotation_is_a_turn_by_position_times_frequency():
    x = np.array([[1.0, 0.0, 0.0, 2.0]])
    out = pm.rotate_pairs(np.repeat(x, 3, axis=0), np.array([0.0, 1.0, 5.0]), 16.0)
    assert np.allclose(out[0], x[0])
    assert np.allclose(out[1], [np.cos(1.0), np.sin(1.0), -2 * np.sin(0.25), 2 * np.cos(0.25)])
    assert np.allclose(out[2], [np.cos(5.0), np.sin(5.0), -2 * np.sin(1.25), 2 * np.cos(1.25)])


def test_routing_takes_the_largest_logits_and_weighs_them_alone():
    W = {"router": np.eye(4), "router.b": np.array([0.0, 0.0, 0.5, 0.0])}
    h = np.array([[1.0, 2.0, 1.6, -1.0], [0.0, 0.0, -1.0, 0.0]])
    chosen, weights = pm.route(h, W, "", 2)
    assert chosen.tolist() == [[2, 1], [0, 1]]          # 2.1 > 2.0; a tie goes to the lower index
    e = np.exp([2.1, 2.0])
    assert np.allclose(weights[0], e / e.sum()) and np.allclose(weights[1], [0.5, 0.5])
    _, all_of_them = pm.route(h, W, "", 4)
    assert np.allclose(all_of_them.sum(axis=1), 1.0)


def test_layer_norm_uses_the_mean_squared_deviation():
    x = np.array([[1.0, 3.0, 5.0, 7.0]])
    out = pm.layer_norm(x, np.array([1.0, 2.0, 1.0, 1.0]), np.array([0.0, 0.0, 0.5, 0.0]), 0.0)
    z = (x - 4.0) / np.sqrt(5.0)
    assert np.allclose(out, z * [1, 2, 1, 1] + [0, 0, 0.5, 0])


@pytest.mark.parametrize("name", list(tm.CONFIGS))
def test_configuration_round_trip_and_tensor_list(name):
    raw = tm.CONFIGS[name]()
    config = config_from_dict(raw)
    assert isinstance(config, MalulornConfig)
    again = config_from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config
    from cpp_minilamma_b200.engine.model import Model
    import torch
    model = Model(build_malulorn_spec(config), torch.float32, "cpu", max_positions=8)
    listed = {s.name: tuple(s.shape) for s in model.weight_specs() if not s.optional}
    assert listed == tm.tensor_shapes(raw)
    # the schedule: the stretch's first layer of every pass is entered through the re-entry product
    order = [(e.layer, None if e.enter is None else e.enter[1]) for e in model.spec.schedule]
    assert [(i, run if first else None) for i, run, first in pm.schedule(raw)] == order
    assert [e.layer for e in model.spec.schedule] == [i for i, _, _ in pm.schedule(raw)]


def test_configuration_faults_are_named():
    good = tm.CONFIGS["mixed"]()
    for change, word in [(lambda c: c["layers"][0].update(type="window_attention"), "type"),
                         (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "multiple"),
                         (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=6), "rot"),
                         (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
                         (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
                         (lambda c: c["layers"][1]["mixer"]["q_temp"].update(every=0), "every"),
                         (lambda c: c.update(loop={"start": 2, "stop": 9, "times": 2}), "loop"),
                         (lambda c: c.pop("norm"), "norm")]:
        raw = json.loads(json.dumps(good))
        change(raw)
        with pytest.raises(ConfigError) as caught:
            config_from_dict(raw)
        assert word in str(caught.value)


def test_oracle_forward_shapes_and_layer_trace():
    raw = tm.CONFIGS["mixed"]()
    W = {k: v.astype(np.float64) for k, v in tm.make_weights(raw, 3).items()}
    toks = tm.tokens(raw, 20, 1)
    logits, after = pm.forward(raw, W, toks, with_layers=True)
    assert logits.shape == (20, raw["vocab"]) and after.shape == (6, 20, raw["width"])
    # causal: a prefix gives the same logits
    assert np.abs(pm.forward(raw, W, toks[:9]) - logits[:9]).max() < 1e-9


def test_command_line_random_then_inspect(tmp_path, capsys):
    """`random` writes a folder from a configuration file (every tensor of the list, bfloat16), `inspect` reads it
    back, and the oracle can run it."""
    from cpp_minilamma_b200.cli import main
    raw = tm.CONFIGS["mixed"]()
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(raw))
    assert main(["random", str(tmp_path / "m"), "--config", str(cfg), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "architecture: Malulorn" in out and "status=ok" in out
    assert "tensor l1.mlp.e6.down [56, 16] bfloat16" in out and "tensor loop.step [2, 56] bfloat16" in out
    assert "tensor l3.mix.dkv.norm [24] bfloat16" in out
    config, W = pm.read_folder(tmp_path / "m")
    # a layer without a feed-forward: the folder holds its second norm all the same (ones and zeros would do)
    assert set(W) - set(tm.tensor_shapes(raw)) == {"l2.norm2", "l2.norm2.b"}
    logits = pm.forward(config, W, tm.tokens(raw, 12, 5))
    assert logits.shape == (12, raw["vocab"]) and np.isfinite(logits).all()
