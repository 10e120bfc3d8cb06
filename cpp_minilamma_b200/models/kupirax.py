"""The Kupirax decoder as data: `KupiraxConfig` -> `ModelSpec`.

A token embedding followed by a norm on the stream, then layers in which one norm feeds a mixer and a
feed-forward side by side (`parallel` block), a final norm and an untied head.  A layer's mixer is chunked
grouped-query attention with a norm over the whole q and k projections, retention, or the gated delta rule with
a decay per key channel; a stretch of layers may run several times in a row with the same weights, every run
with a cache or state of its own (the schedule names those layers again).  This file is the only one that knows
Kupirax's tensor names: `embed`, `embed.norm`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`,
`final.norm`, `head`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.kupirax import KupiraxConfig, KupiraxLayer, Rotation
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _rotary(rot: Rotation, interleaved: bool):
    if rot is None or rot.dims == 0:
        return None
    scaling = None
    if rot.scaling:
        scaling = {"factor": rot.scaling["factor"], "low_freq_factor": rot.scaling["low"],
                   "high_freq_factor": rot.scaling["high"],
                   "original_max_position_embeddings": rot.scaling["original"]}
    return PartSpec("rotary", {"head_dim": rot.dims, "theta": rot.base, "scaling": scaling, "interleaved": interleaved})


def _mixer(layer: KupiraxLayer, prefix: str, eps: float) -> PartSpec:
    mix = prefix + "mix."
    if layer.type == "attention":
        return PartSpec("chunked_attention", {
            "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim, "v_head_dim": layer.vdim,
            "scale": layer.scale, "chunk": layer.chunk, "window": 0,
            "position": _rotary(layer.rot, interleaved=True), "rotary_dims": layer.rot.dims if layer.rot else 0,
            "qk_norm": {"q": mix + "q.norm", "k": mix + "k.norm", "eps": eps},
            "names": {p: mix + p for p in ("q", "k", "v", "o")}})
    if layer.type == "retention":
        return PartSpec("retention", {
            "n_heads": layer.heads, "head_dim": layer.dim, "v_head_dim": layer.vdim, "decay": list(layer.decay),
            "eps": eps, "position": _rotary(layer.rot, interleaved=False),
            "rotary_dims": layer.rot.dims if layer.rot else 0,
            "names": {p: mix + p for p in ("q", "k", "v", "g", "o")}})
    return PartSpec("gated_delta_rule", {
        "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim, "v_head_dim": layer.vdim,
        "conv": layer.conv, "eps": eps, "unit_eps": 1e-6,
        "decay_rank": layer.decay_rank or -1, "gate_rank": layer.gate_rank or -1,
        "names": {p: mix + p for p in ("q", "k", "v", "b", "a1", "a2", "dt_bias", "A_log", "g1", "g2", "norm", "o")}})


def build_kupirax_spec(config: KupiraxConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rms_norm", {"width": config.width, "eps": config.eps, "name": name})

    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        feed_forward = PartSpec("none") if not layer.ff else PartSpec("swiglu", {
            "intermediate": layer.ff, "names": {p: prefix + "mlp." + p for p in ("gate", "up", "down")},
            "bare_names": True})
        layers.append(LayerSpec(block=PartSpec("parallel"), mixer=_mixer(layer, prefix, config.eps),
                                feed_forward=feed_forward, norms={"input": norm(prefix + "norm1")}))
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "name": "embed", "norm": norm("embed.norm")}),
        layers=layers, schedule=[ScheduleEntry(i) for i in config.schedule()],
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab": config.vocab, "name": "head", "tied_to": None}))


register_architecture("Kupirax", KupiraxConfig, build_kupirax_spec)
