"""Typed configuration of the Nafevik decoder, read from config.json's own keys.

    architecture    "Nafevik"
    vocab, width, max_positions
    norm.eps, residual_mult
    canon.taps      taps of the short causal convolution that each sublayer's input passes (absent: none)
    layers[]        type ("attention"), mixer {heads, kv_heads, dim, vdim, scale, mask.size, rot{base, dims,
                    scaling{factor, original, fast, slow}}}, mlp {kind "dense", ff} or null
    loop            {start, stop, times}: layers start..stop-1 run `times` times in a row (absent: each layer once)

Every size and constant is a parameter; a key that is absent switches its mechanism off where the design allows
that (`canon`, `loop`, a mixer's `mask`, `rot` and `rot.scaling`, a layer's `mlp`).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Optional

from .model_config import ConfigError

MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense",)


def _positive_int(value, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {value!r}")
    return value


def _number(value, what: str, positive: bool = True) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(float(value)):
        raise ConfigError(f"config.json: {what} must be a finite number, got {value!r}")
    if positive and not float(value) > 0:
        raise ConfigError(f"config.json: {what} must be positive, got {value!r}")
    return float(value)


def _section(raw: dict, key: str, what: str) -> dict:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {what} needs an object {key!r}")
    return value


@dataclass(frozen=True)
class NafevikConfig:
    width: int
    vocab: int
    max_positions: int
    norm_eps: float
    residual_mult: float
    layers: tuple                      # of dicts as in config.json (validated)
    canon_taps: int = 0                # 0: no input convolution
    loop: Optional[tuple] = None       # (start, stop, times)
    initializer_range: float = 0.02
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "NafevikConfig":
        width = _positive_int(raw.get("width"), "width")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        checked = []
        for i, layer in enumerate(layers):
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is not known; known: {MIXER_TYPES}")
            mixer = _section(layer, "mixer", f"layers[{i}]")
            heads = _positive_int(mixer.get("heads"), f"layers[{i}].mixer.heads")
            kv_heads = _positive_int(mixer.get("kv_heads", heads), f"layers[{i}].mixer.kv_heads")
            if heads % kv_heads:
                raise ConfigError(f"config.json: layers[{i}].mixer.heads must be a multiple of kv_heads")
            dim = _positive_int(mixer.get("dim"), f"layers[{i}].mixer.dim")
            _positive_int(mixer.get("vdim", dim), f"layers[{i}].mixer.vdim")
            _number(mixer.get("scale"), f"layers[{i}].mixer.scale")
            if mixer.get("mask") is not None:
                _positive_int(_section(mixer, "mask", f"layers[{i}].mixer").get("size"), f"layers[{i}].mixer.mask.size")
            rot = mixer.get("rot")
            if rot is not None:
                dims = _positive_int(rot.get("dims"), f"layers[{i}].mixer.rot.dims")
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: layers[{i}].mixer.rot.dims must be even and at most dim")
                _number(rot.get("base"), f"layers[{i}].mixer.rot.base")
                scaling = rot.get("scaling")
                if scaling is not None:
                    for key in ("factor", "original", "fast", "slow"):
                        _number(scaling.get(key), f"layers[{i}].mixer.rot.scaling.{key}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp.get('kind')!r} is not known; known: {MLP_KINDS}")
                _positive_int(mlp.get("ff"), f"layers[{i}].mlp.ff")
            checked.append(copy.deepcopy(layer))
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = loop.get("start"), loop.get("stop"), loop.get("times")
            for name, value in (("start", start), ("stop", stop)):
                if isinstance(value, bool) or not isinstance(value, int) or value < 0:
                    raise ConfigError(f"config.json: loop.{name} must be a non-negative integer")
            _positive_int(times, "loop.times")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
            loop = (start, stop, times)
        canon = raw.get("canon")
        taps = 0 if canon is None else _positive_int(canon.get("taps"), "canon.taps")
        known = {"architecture", "vocab", "width", "max_positions", "norm", "residual_mult", "layers", "loop", "canon",
                 "initializer_range"}
        return cls(width=width, vocab=_positive_int(raw.get("vocab"), "vocab"),
                   max_positions=_positive_int(raw.get("max_positions"), "max_positions"),
                   norm_eps=_number(_section(raw, "norm", "the model").get("eps"), "norm.eps"),
                   residual_mult=_number(raw.get("residual_mult", 1.0), "residual_mult", positive=False),
                   layers=tuple(checked), canon_taps=taps, loop=loop,
                   initializer_range=float(raw.get("initializer_range", 0.02)),
                   extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        out = {"architecture": "Nafevik", "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "layers": copy.deepcopy(list(self.layers)), "initializer_range": self.initializer_range}
        if self.canon_taps:
            out["canon"] = {"taps": self.canon_taps}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        out.update(self.extra)
        return out

    def layer_runs(self) -> list:
        """The order in which layers run: (layer, pass of the loop or None, first of its pass)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None, False) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, None, False) for i in range(start)]
        for t in range(times):
            runs += [(i, t, i == start) for i in range(start, stop)]
        return runs + [(i, None, False) for i in range(stop, n)]

    def validate_capacity(self, capacity: int) -> None:
        if not 0 < capacity <= self.max_positions:
            raise ConfigError(f"context capacity {capacity} exceeds the model's max_positions {self.max_positions}")
