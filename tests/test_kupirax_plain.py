"""The Kupirax oracle against itself and the configuration reader, without a GPU: every recurrence of
`plain_kupirax` is compared with the same mechanism written the other way round (a sum over earlier tokens
instead of a state carried along), so that the oracle's reading of the equations does not rest on one form."""
import math

import numpy as np
import pytest

import cpp_minilamma_b200 as ml
import plain_kupirax as pk
import tiny_kupirax as tk


def test_retention_as_a_sum_over_earlier_tokens():
    cfg = tk.CONFIGS["retention_only"]()
    W = {k: v.astype(np.float64) for k, v in tk.make_weights(cfg, 1).items()}
    m = cfg["layers"][0]["mixer"]
    rng = np.random.RandomState(0)
    h = rng.randn(9, cfg["width"])
    got = pk.retention(h, W, "l0.mix.", m, 1e-5)
    T, H, d, dv = 9, m["heads"], m["dim"], m["vdim"]
    q = pk.rotate((h @ W["l0.mix.q"].T).reshape(T, H, d), range(T), m["rot"], False)
    k = pk.rotate((h @ W["l0.mix.k"].T).reshape(T, H, d), range(T), m["rot"], False) / math.sqrt(d)
    v = (h @ W["l0.mix.v"].T).reshape(T, H, dv)
    o = np.zeros((T, H, dv))
    for t in range(T):
        for head in range(H):
            for j in range(t + 1):
                o[t, head] += m["decay"][head] ** (t - j) * (q[t, head] @ k[j, head]) * v[j, head]
    want = (pk.rms(o, 1e-5).reshape(T, -1) * pk.silu(h @ W["l0.mix.g"].T)) @ W["l0.mix.o"].T
    np.testing.assert_allclose(got, want, rtol=1e-9, atol=1e-12)


def test_rotation_pairs_and_untouched_dimensions():
    rot = {"base": 10.0, "dims": 4}
    x = np.arange(1.0, 13.0).reshape(1, 2, 6)
    for interleaved, pairs in ((True, [(0, 1), (2, 3)]), (False, [(0, 2), (1, 3)])):
        y = pk.rotate(x, [3], rot, interleaved)
        np.testing.assert_array_equal(y[..., 4:], x[..., 4:])
        for i, (a, b) in enumerate(pairs):
            ang = 3 * 10.0 ** (-2.0 * i / 4)
            np.testing.assert_allclose(y[0, :, a], x[0, :, a] * math.cos(ang) - x[0, :, b] * math.sin(ang))
            np.testing.assert_allclose(y[0, :, b], x[0, :, b] * math.cos(ang) + x[0, :, a] * math.sin(ang))


def test_frequency_scaling_keeps_short_waves_and_slows_long_ones():
    rot = {"base": 10000.0, "dims": 32, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = pk.rotary_frequencies({"base": 10000.0, "dims": 32})
    scaled = pk.rotary_frequencies(rot)
    lam = 2 * math.pi / plain
    assert np.all(scaled[lam < 16] == plain[lam < 16])
    np.testing.assert_allclose(scaled[lam > 64], plain[lam > 64] / 8.0)
    between = (lam >= 16) & (lam <= 64)
    assert between.any() and np.all(scaled[between] <= plain[between]) and np.all(scaled[between] >= plain[between] / 8)


def test_chunk_mask_counts_from_position_zero():
    cfg = tk.CONFIGS["attention_only"]()
    W = {k: v.astype(np.float64) for k, v in tk.make_weights(cfg, 2).items()}
    m = cfg["layers"][0]["mixer"]
    h = np.random.RandomState(3).randn(20, cfg["width"])
    whole = pk.attention(h, W, "l0.mix.", m, 1e-5)
    # a token at the start of a chunk sees only itself: its output does not change when all earlier inputs do
    other = h.copy()
    other[:16] += 1.0
    changed = pk.attention(other, W, "l0.mix.", m, 1e-5)
    np.testing.assert_allclose(changed[16], whole[16], rtol=1e-12)
    assert np.abs(changed[15] - whole[15]).max() > 1e-3


def test_delta_rule_reads_its_own_write():
    cfg = tk.CONFIGS["delta_only"]()
    W = {k: v.astype(np.float64) for k, v in tk.make_weights(cfg, 4).items()}
    h = np.random.RandomState(5).randn(1, cfg["width"])
    out = pk.channel_delta(h, W, "l0.mix.", cfg["layers"][0]["mixer"], 1e-5)
    assert np.abs(out).max() > 1e-6  # from a zero state the first token's output is its own write read back


def test_schedule_with_a_loop():
    cfg = tk.CONFIGS["mixed"]()
    assert pk.schedule(cfg) == [0, 1, 2, 1, 2, 3, 4]
    typed = ml.config_from_dict(cfg)
    assert typed.schedule() == pk.schedule(cfg)
    assert ml.config_from_dict(typed.to_dict()).to_dict() == typed.to_dict()


def test_configuration_faults_are_named():
    cfg = tk.CONFIGS["mixed"]()
    cfg["layers"][0]["type"] = "something"
    with pytest.raises(ml.ConfigError, match="type"):
        ml.config_from_dict(cfg)
    cfg = tk.CONFIGS["mixed"]()
    cfg["layers"][0]["mixer"]["decay"] = [0.5]
    with pytest.raises(ml.ConfigError, match="decay"):
        ml.config_from_dict(cfg)
    cfg = tk.CONFIGS["mixed"]()
    cfg["loop"] = {"start": 3, "stop": 9, "times": 2}
    with pytest.raises(ml.ConfigError, match="loop"):
        ml.config_from_dict(cfg)
    cfg = tk.CONFIGS["mixed"]()
    cfg["layers"][1]["mlp"] = {"kind": "routed", "ff": 8}
    with pytest.raises(ml.ConfigError, match="kind"):
        ml.config_from_dict(cfg)


def test_tensor_list_matches_the_folder(tmp_path):
    import torch
    for name in tk.CONFIGS:
        folder, cfg, _ = tk.make_folder(name, tmp_path / name)
        model = ml.build_model(ml.load_config(folder), "float32", "cpu", max_positions=8)
        specs = {s.name: s.shape for s in model.weight_specs()}
        shapes = tk.tensor_shapes(cfg)
        assert set(specs) == set(shapes)
        for n, shape in specs.items():
            assert all(a == -1 or a == b for a, b in zip(shape, shapes[n])), n
        needs = model.cache_needs()
        assert len(needs) == len(pk.schedule(cfg))  # every run of a looped layer has a cache or state of its own


def test_command_line_writes_and_inspects_a_random_folder(tmp_path, capsys):
    """`random` needs the sizes that only tensors give (the low-rank pairs' inner sizes) named in the configuration."""
    import json
    from cpp_minilamma_b200.cli import main
    cfg = tk.CONFIGS["mixed"]()
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    assert main(["random", str(tmp_path / "m"), "--config", str(tmp_path / "c.json")]) == 1
    assert "configuration must name it" in capsys.readouterr().err
    for layer in cfg["layers"]:
        if layer["type"] == "channel_delta":
            layer["mixer"]["decay_rank"], layer["mixer"]["gate_rank"] = tk.RANKS
    (tmp_path / "c.json").write_text(json.dumps(cfg))
    assert main(["random", str(tmp_path / "m"), "--config", str(tmp_path / "c.json"), "--seed", "3"]) == 0
    assert main(["inspect", str(tmp_path / "m")]) == 0
    out = capsys.readouterr().out
    assert "architecture: Kupirax" in out and "tensor l4.mix.q.conv [16, 5] bfloat16" in out and "status=ok" in out
    model = ml.build_model(ml.load_config(tmp_path / "m"), "float32", "cpu", max_positions=8)
    assert {s.name for s in model.weight_specs()} == set(tk.tensor_shapes(cfg))
