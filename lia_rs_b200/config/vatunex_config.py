"""Typed configuration of the Vatunex decoder, read from config.json's own keys.

    architecture    "Vatunex"
    vocab, width
    norm.eps
    layers[]        type: which mixer the layer has; mixer: its sizes; mlp {kind "dense", ff} or null
      "latent_attention"  mixer {heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, mask.size (absent: all keys),
                                 rot {base, dims, scaling (absent: plain)}}
      "attention"         mixer {heads, kv_heads (absent: heads), dim, vdim (absent: dim), scale, v_mix (absent: false),
                                 mask.size (absent: all keys), rot {base, dims, scaling {factor, low, high, original}}
                                 (absent: no rotation)}
      "mamba1"            mixer {inner, state, dt_rank, conv}

Every size and constant is a parameter.  The design has no table of positions and no limit of its own on a request's
length.  `initializer_range` (absent: 0.02) only serves the random-weights mode."""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .model_config import ConfigError
from .nafevik_config import _number, _positive_int, _section

MIXER_TYPES = ("latent_attention", "attention", "mamba1")
MLP_KINDS = ("dense",)


def _rot(mixer: dict, limit: int, where: str, needed: bool) -> None:
    rot = mixer.get("rot")
    if rot is None:
        if needed:
            raise ConfigError(f"config.json: {where} needs an object 'rot'")
        return
    dims = _positive_int(rot.get("dims"), f"{where}.rot.dims")
    if dims % 2 or dims > limit:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most {limit}")
    _number(rot.get("base"), f"{where}.rot.base")
    scaling = rot.get("scaling")
    if scaling is not None:
        for key in ("factor", "low", "high", "original"):
            _number(scaling.get(key), f"{where}.rot.scaling.{key}")
        if float(scaling["low"]) == float(scaling["high"]):
            raise ConfigError(f"config.json: {where}.rot.scaling.low and .high must differ")


def _mask(mixer: dict, where: str) -> None:
    if mixer.get("mask") is not None:
        _positive_int(_section(mixer, "mask", where).get("size"), f"{where}.mask.size")


@dataclass(frozen=True)
class VatunexConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: tuple                      # of dicts as in config.json (validated)
    initializer_range: float = 0.02
    extra: dict = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: dict) -> "VatunexConfig":
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
            where = f"layers[{i}].mixer"
            mixer = _section(layer, "mixer", f"layers[{i}]")
            if kind == "latent_attention":
                for key in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"):
                    _positive_int(mixer.get(key), f"{where}.{key}")
                _number(mixer.get("scale"), f"{where}.scale")
                _rot(mixer, mixer["rot_dim"], where, needed=True)
                _mask(mixer, where)
            elif kind == "attention":
                heads = _positive_int(mixer.get("heads"), f"{where}.heads")
                kv_heads = _positive_int(mixer.get("kv_heads", heads), f"{where}.kv_heads")
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
                dim = _positive_int(mixer.get("dim"), f"{where}.dim")
                _positive_int(mixer.get("vdim", dim), f"{where}.vdim")
                _number(mixer.get("scale"), f"{where}.scale")
                if not isinstance(mixer.get("v_mix", False), bool):
                    raise ConfigError(f"config.json: {where}.v_mix must be true or false")
                _rot(mixer, dim, where, needed=False)
                _mask(mixer, where)
            else:
                for key in ("inner", "state", "dt_rank", "conv"):
                    _positive_int(mixer.get(key), f"{where}.{key}")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind is not known; known: {MLP_KINDS}")
                _positive_int(mlp.get("ff"), f"layers[{i}].mlp.ff")
            checked.append(copy.deepcopy(layer))
        mixed = [l["mixer"] for l in checked if l["type"] == "attention" and l["mixer"].get("v_mix")]
        sizes = {(m.get("kv_heads", m["heads"]), m.get("vdim", m["dim"])) for m in mixed}
        if len(sizes) > 1:
            raise ConfigError("config.json: layers that mix values must agree in kv_heads and vdim")
        known = {"architecture", "vocab", "width", "norm", "layers", "initializer_range"}
        return cls(width=width, vocab=_positive_int(raw.get("vocab"), "vocab"),
                   norm_eps=_number(_section(raw, "norm", "the model").get("eps"), "norm.eps"),
                   layers=tuple(checked), initializer_range=float(raw.get("initializer_range", 0.02)),
                   extra={k: v for k, v in raw.items() if k not in known})

    def to_dict(self) -> dict:
        out = {"architecture": "Vatunex", "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "layers": copy.deepcopy(list(self.layers))}
        if self.initializer_range != 0.02:
            out["initializer_range"] = self.initializer_range
        out.update(self.extra)
        return out
