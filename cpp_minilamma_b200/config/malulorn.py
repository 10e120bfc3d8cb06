"""`MalulornConfig`: the configuration of the Malulorn decoder, typed and checked.

A Malulorn folder's config.json names the design in "architecture" and gives every size and constant:

    vocab, width, norm.eps
    layers[i].type     "attention" | "latent_attention"
    layers[i].mixer    attention: heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (optional)
                       latent_attention: heads, dim, rot_dim, vdim, kv_rank, scale, rot {base, dims}
    layers[i].mlp      {"kind": "moe", "router": {experts, top}, "expert": {ff}, "shared": {ff} or null},
                       {"kind": "dense", "ff": n}, or null for a layer without a feed-forward
    loop               {"start", "stop", "times"}: layers start .. stop - 1 run `times` times in a row, each pass
                       entered through the re-entry product; absent: every layer runs once and nothing is re-entered

Nothing here knows tensor names or kernels; `models/malulorn.py` turns the typed configuration into parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, take_float, take_int
from .kupirax import Rotation, _object

MIXER_TYPES = ("attention", "latent_attention")


@dataclass
class MalulornFeedForward:
    kind: str                 # "moe" or "dense"
    ff: int                   # an expert's width (moe) or the layer's (dense)
    experts: int = 0
    top: int = 0
    shared_ff: int = 0        # 0: no shared expert

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> Optional["MalulornFeedForward"]:
        if raw is None:
            return None
        raw = _object(raw, what)
        kind = raw.get("kind")
        if kind == "dense":
            return cls("dense", take_int(raw, "ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"config.json: {what}.kind {kind!r} is not supported (known: moe, dense)")
        router = _object(raw.get("router"), what + ".router")
        out = cls("moe", take_int(_object(raw.get("expert"), what + ".expert"), "ff", minimum=1),
                  experts=take_int(router, "experts", minimum=1), top=take_int(router, "top", minimum=1))
        if raw.get("shared") is not None:
            out.shared_ff = take_int(_object(raw["shared"], what + ".shared"), "ff", minimum=1)
        if out.top > out.experts:
            raise ConfigError(f"config.json: {what}: top {out.top} of {out.experts} experts")
        return out

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff},
                "shared": {"ff": self.shared_ff} if self.shared_ff else None}


@dataclass
class MalulornLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    scale: float
    kv_heads: int = 0                    # attention
    q_temp_coef: float = 0.0             # attention: query temperature, every == 0: none
    q_temp_every: int = 0
    rot_dim: int = 0                     # latent_attention
    kv_rank: int = 0
    rot: Optional[Rotation] = None
    mlp: Optional[MalulornFeedForward] = None

    @classmethod
    def from_dict(cls, raw: Any, index: int) -> "MalulornLayer":
        what = f"layers[{index}]"
        raw = _object(raw, what)
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {what}.type {kind!r} is not one of {', '.join(MIXER_TYPES)}")
        m = _object(raw.get("mixer"), what + ".mixer")
        heads, dim = take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1)
        layer = cls(type=kind, heads=heads, dim=dim, vdim=take_int(m, "vdim", default=dim, minimum=1), scale=0.0)
        if kind == "attention":
            layer.kv_heads = take_int(m, "kv_heads", default=heads, minimum=1)
            layer.scale = take_float(m, "scale", default=dim ** -0.5)
            if heads % layer.kv_heads:
                raise ConfigError(f"config.json: {what}: {heads} heads are not a multiple of {layer.kv_heads} kv_heads")
            if m.get("q_temp") is not None:
                q_temp = _object(m["q_temp"], what + ".mixer.q_temp")
                layer.q_temp_coef = take_float(q_temp, "coef")
                layer.q_temp_every = take_int(q_temp, "every", minimum=1)
        else:
            layer.rot_dim = take_int(m, "rot_dim", default=0, minimum=0)
            layer.kv_rank = take_int(m, "kv_rank", minimum=1)
            layer.scale = take_float(m, "scale", default=(dim + layer.rot_dim) ** -0.5)
            layer.rot = Rotation.from_dict(m.get("rot"), what + ".mixer.rot")
            if layer.rot_dim:
                if layer.rot is None or layer.rot.dims != layer.rot_dim or layer.rot.scaling:
                    raise ConfigError(f"config.json: {what}: the {layer.rot_dim} rotated dimensions need "
                                      "'rot' with the same 'dims' and no scaling")
            elif layer.rot is not None and layer.rot.dims:
                raise ConfigError(f"config.json: {what}: 'rot' without rotated dimensions")
        layer.mlp = MalulornFeedForward.from_dict(raw.get("mlp"), what + ".mlp")
        return layer

    def to_dict(self) -> Dict[str, Any]:
        m: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.type == "attention":
            m["kv_heads"] = self.kv_heads
            if self.q_temp_every:
                m["q_temp"] = {"coef": self.q_temp_coef, "every": self.q_temp_every}
        else:
            m.update(rot_dim=self.rot_dim, kv_rank=self.kv_rank)
            if self.rot is not None:
                m["rot"] = self.rot.to_dict()
        return {"type": self.type, "mixer": m, "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass
class MalulornConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 1e-5
    layers: List[MalulornLayer] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0            # 0: no looped stretch (and so no re-entry)
    max_positions: int = 1 << 20   # not part of the design: the most positions a sequence may have
    torch_dtype: str = "bfloat16"  # storage of a folder written from this configuration

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MalulornConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=take_int(raw, "vocab", minimum=1), width=take_int(raw, "width", minimum=1),
                     eps=take_float(_object(raw.get("norm"), "'norm'"), "eps"),
                     layers=[MalulornLayer.from_dict(l, i) for i, l in enumerate(layers)])
        if raw.get("loop") is not None:
            loop = _object(raw["loop"], "'loop'")
            config.loop_start = take_int(loop, "start", minimum=0)
            config.loop_stop = take_int(loop, "stop", minimum=0)
            config.loop_times = take_int(loop, "times", minimum=1)
        config.max_positions = take_int(raw, "max_positions", default=cls.max_positions, minimum=1)
        config.torch_dtype = raw.get("torch_dtype", "bfloat16")
        return config

    def validate(self) -> None:
        if self.eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if not 0 <= self.loop_start <= self.loop_stop <= len(self.layers):
            raise ConfigError(f"config.json: loop [{self.loop_start}, {self.loop_stop}) does not lie inside the "
                              f"{len(self.layers)} layers")

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def loops(self) -> bool:
        return self.loop_times > 0 and self.loop_stop > self.loop_start

    def schedule(self) -> List[tuple]:
        """(layer, pass of the looped stretch if the layer is the first of a pass, else None) in running order."""
        n = len(self.layers)
        if not self.loops:
            return [(i, None) for i in range(n)]
        order = [(i, None) for i in range(self.loop_start)]
        for run in range(self.loop_times):
            order += [(i, run if i == self.loop_start else None) for i in range(self.loop_start, self.loop_stop)]
        return order + [(i, None) for i in range(self.loop_stop, n)]

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture or "Malulorn", "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps}, "layers": [l.to_dict() for l in self.layers],
                               "max_positions": self.max_positions, "torch_dtype": self.torch_dtype}
        if self.loops:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out
