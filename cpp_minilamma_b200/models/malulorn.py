"""The Malulorn decoder as data: `MalulornConfig` -> `ModelSpec`.

A token embedding, then pre-norm layers (layer norms with weight and bias) whose mixer is grouped-query attention
without rotation - query temperature, a sink in the softmax, a gate per head - or attention over a shared low-rank
latent with one rotated key part and a gate per element, and whose feed-forward routes every token through a few
small experts beside a shared one; a stretch of layers may run several times in a row with the same weights, every
pass with caches of its own and entered through a product that mixes the stream with the embedding's output; a final
layer norm and an untied head.  This file is the only one that knows Malulorn's tensor names: `embed`, `loop.in`,
`loop.step`, `l<i>.norm1(.b)`, `l<i>.norm2(.b)`, `l<i>.mix.*`, `l<i>.mlp.{router(.b), e<k>.*, shared.*}`,
`final.norm(.b)`, `head`.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.malulorn import MalulornConfig, MalulornLayer
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _mixer(layer: MalulornLayer, prefix: str, eps: float) -> PartSpec:
    mix = prefix + "mix."
    if layer.type == "attention":
        return PartSpec("chunked_attention", {
            "n_heads": layer.heads, "n_kv_heads": layer.kv_heads, "head_dim": layer.dim, "v_head_dim": layer.vdim,
            "scale": layer.scale, "chunk": 0, "window": 0, "position": None, "rotary_dims": 0, "qk_norm": None,
            "q_temp": {"coef": layer.q_temp_coef, "every": layer.q_temp_every} if layer.q_temp_every else None,
            "sink": True, "gate": "head", "names": {p: mix + p for p in ("q", "k", "v", "g", "o")}})
    position = None
    if layer.rot_dim:
        position = PartSpec("rotary", {"head_dim": layer.rot_dim, "theta": layer.rot.base, "scaling": None,
                                       "interleaved": True})
    names = {p: mix + p for p in ("q", "dkv", "uk", "uv", "g", "o")}
    names["dkv_norm"] = mix + "dkv.norm"
    return PartSpec("latent_attention", {
        "n_heads": layer.heads, "head_dim": layer.dim, "rot_dim": layer.rot_dim, "v_head_dim": layer.vdim,
        "kv_rank": layer.kv_rank, "scale": layer.scale, "eps": eps, "position": position, "gate": True, "names": names})


def _feed_forward(layer: MalulornLayer, prefix: str) -> PartSpec:
    mlp = layer.mlp
    if mlp is None:
        return PartSpec("none")
    pre = prefix + "mlp."
    if mlp.kind == "dense":
        return PartSpec("swiglu", {"intermediate": mlp.ff, "names": {p: pre + p for p in ("gate", "up", "down")},
                                   "bare_names": True})
    shared = None
    if mlp.shared_ff:
        shared = {"intermediate": mlp.shared_ff, "names": {p: pre + "shared." + p for p in ("gate", "up", "down")},
                  "bare_names": True}
    return PartSpec("routed", {"experts": mlp.experts, "top": mlp.top, "intermediate": mlp.ff, "router_bias": True,
                               "names": {"router": pre + "router", "router_bias": pre + "router.b",
                                         "expert": pre + "e{e}.{p}"}, "shared": shared})


def build_malulorn_spec(config: MalulornConfig) -> ModelSpec:
    def norm(name, optional=False):
        return PartSpec("layer_norm", {"width": config.width, "eps": config.eps, "name": name, "bias": name + ".b",
                                       "optional": optional})

    layers = []
    for i, layer in enumerate(config.layers):
        prefix = f"l{i}."
        # a layer without a feed-forward has nothing behind its second norm; a folder may leave those tensors out
        layers.append(LayerSpec(block=PartSpec("pre_norm"), mixer=_mixer(layer, prefix, config.eps),
                                feed_forward=_feed_forward(layer, prefix),
                                norms={"input": norm(prefix + "norm1"),
                                       "post_mixer": norm(prefix + "norm2", optional=layer.mlp is None)}))
    stream_ops = []
    if config.loop_times > 0:
        # a loop over no layers is never entered; its tensors may be in the folder all the same
        stream_ops.append(PartSpec("reentry", {"passes": config.loop_times, "names": {"in": "loop.in", "step": "loop.step"},
                                               "optional": not config.loops}))
    schedule = [ScheduleEntry(i, enter=None if run is None else (0, run)) for i, run in config.schedule()]
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab, max_positions=config.max_positions,
        embedding=PartSpec("token_embedding", {"vocab": config.vocab, "name": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab": config.vocab, "name": "head", "tied_to": None}),
        stream_ops=stream_ops)


register_architecture("Malulorn", MalulornConfig, build_malulorn_spec)
