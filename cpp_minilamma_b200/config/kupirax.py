"""`KupiraxConfig`: the configuration of the Kupirax decoder, typed and checked.

A Kupirax folder's config.json names the design in "architecture" and gives every size and constant:

    vocab, width, norm.eps
    layers[i].type     "attention" | "retention" | "channel_delta"
    layers[i].mixer    the mixer's sizes (heads, kv_heads, dim, vdim, ...) and constants
    layers[i].mlp      {"kind": "dense", "ff": n} or null
    loop               {"start", "stop", "times"}: layers start .. stop - 1 run `times` times in a row

Nothing here knows tensor names or kernels; `models/kupirax.py` turns the typed configuration into parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .base import ConfigError, ModelConfig, take_float, take_int

MIXER_TYPES = ("attention", "retention", "channel_delta")


def _object(raw: Any, what: str) -> Dict[str, Any]:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {what} must be an object")
    return raw


@dataclass
class Rotation:
    """Rotary positions on the first `dims` dimensions of a head; `scaling` rescales the frequencies by
    wavelength (keys factor, low, high, original) or is None."""

    base: float
    dims: int
    scaling: Optional[Dict[str, float]] = None

    @classmethod
    def from_dict(cls, raw: Any, what: str) -> Optional["Rotation"]:
        if raw is None:
            return None
        raw = _object(raw, what)
        scaling = None
        if raw.get("scaling") is not None:
            sc = _object(raw["scaling"], what + ".scaling")
            scaling = {"factor": take_float(sc, "factor"), "low": take_float(sc, "low"),
                       "high": take_float(sc, "high"), "original": float(take_int(sc, "original", minimum=1))}
            if not scaling["high"] > scaling["low"] > 0 or scaling["factor"] <= 0:
                raise ConfigError(f"config.json: {what}.scaling needs high > low > 0 and a positive factor")
        rot = cls(base=take_float(raw, "base"), dims=take_int(raw, "dims", minimum=0), scaling=scaling)
        if rot.dims % 2 or rot.base <= 0:
            raise ConfigError(f"config.json: {what} needs an even 'dims' and a positive 'base'")
        return rot

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling:
            out["scaling"] = {"factor": self.scaling["factor"], "low": self.scaling["low"],
                              "high": self.scaling["high"], "original": int(self.scaling["original"])}
        return out


@dataclass
class KupiraxLayer:
    type: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0                   # attention: key/value heads; channel_delta: q/k heads
    rot: Optional[Rotation] = None      # attention, retention
    scale: float = 0.0                  # attention
    chunk: int = 0                      # attention: mask.size (0: plain causal)
    decay: List[float] = field(default_factory=list)  # retention
    conv: int = 0                       # channel_delta: taps
    decay_rank: int = 0                 # channel_delta: inner sizes of the two low-rank pairs; 0: as the
    gate_rank: int = 0                  # tensors of the folder have them (config.json need not give them)
    ff: int = 0                         # feed-forward width, 0: none

    @classmethod
    def from_dict(cls, raw: Any, index: int) -> "KupiraxLayer":
        what = f"layers[{index}]"
        raw = _object(raw, what)
        kind = raw.get("type")
        if kind not in MIXER_TYPES:
            raise ConfigError(f"config.json: {what}.type {kind!r} is not one of {', '.join(MIXER_TYPES)}")
        m = _object(raw.get("mixer"), what + ".mixer")
        heads, dim = take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1)
        layer = cls(type=kind, heads=heads, dim=dim, vdim=take_int(m, "vdim", default=dim, minimum=1))
        if kind == "attention":
            layer.kv_heads = take_int(m, "kv_heads", default=heads, minimum=1)
            layer.rot = Rotation.from_dict(m.get("rot"), what + ".mixer.rot")
            layer.scale = take_float(m, "scale", default=dim ** -0.5)
            if m.get("mask") is not None:
                layer.chunk = take_int(_object(m["mask"], what + ".mixer.mask"), "size", minimum=1)
        elif kind == "retention":
            layer.rot = Rotation.from_dict(m.get("rot"), what + ".mixer.rot")
            decay = m.get("decay")
            if not isinstance(decay, list) or len(decay) != layer.heads or \
                    any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in decay):
                raise ConfigError(f"config.json: {what}.mixer.decay must list one number per head")
            layer.decay = [float(x) for x in decay]
        else:
            layer.kv_heads = take_int(m, "kv_heads", default=heads, minimum=1)
            layer.conv = take_int(m, "conv", minimum=1)
            layer.decay_rank = take_int(m, "decay_rank", default=0, minimum=0)
            layer.gate_rank = take_int(m, "gate_rank", default=0, minimum=0)
        if layer.kv_heads and layer.heads % layer.kv_heads:
            raise ConfigError(f"config.json: {what}: {layer.heads} heads are not a multiple of {layer.kv_heads} kv_heads")
        if layer.rot is not None and layer.rot.dims > layer.dim:
            raise ConfigError(f"config.json: {what}: {layer.rot.dims} rotated dimensions of a head of {layer.dim}")
        mlp = raw.get("mlp")
        if mlp is not None:
            mlp = _object(mlp, what + ".mlp")
            if mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: {what}.mlp.kind {mlp.get('kind')!r} is not supported (known: dense)")
            layer.ff = take_int(mlp, "ff", minimum=1)
        return layer

    def to_dict(self) -> Dict[str, Any]:
        m: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim}
        if self.type == "attention":
            m.update(kv_heads=self.kv_heads, scale=self.scale)
            if self.rot is not None:
                m["rot"] = self.rot.to_dict()
            if self.chunk:
                m["mask"] = {"size": self.chunk}
        elif self.type == "retention":
            m["decay"] = list(self.decay)
            if self.rot is not None:
                m["rot"] = self.rot.to_dict()
        else:
            m.update(kv_heads=self.kv_heads, conv=self.conv)
            if self.decay_rank:
                m["decay_rank"] = self.decay_rank
            if self.gate_rank:
                m["gate_rank"] = self.gate_rank
        return {"type": self.type, "mixer": m, "mlp": {"kind": "dense", "ff": self.ff} if self.ff else None}


@dataclass
class KupiraxConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    eps: float = 1e-6
    layers: List[KupiraxLayer] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    max_positions: int = 1 << 20   # not part of the design: the most positions a sequence may have (tables are built for what the cache holds)
    torch_dtype: str = "bfloat16"  # storage of a folder written from this configuration

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "KupiraxConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab=take_int(raw, "vocab", minimum=1), width=take_int(raw, "width", minimum=1),
                     eps=take_float(_object(raw.get("norm"), "'norm'"), "eps"),
                     layers=[KupiraxLayer.from_dict(l, i) for i, l in enumerate(layers)])
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

    def schedule(self) -> List[int]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        return (list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times
                + list(range(self.loop_stop, n)))

    def to_dict(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture or "Kupirax", "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.eps}, "layers": [l.to_dict() for l in self.layers],
                               "max_positions": self.max_positions, "torch_dtype": self.torch_dtype}
        if self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out
