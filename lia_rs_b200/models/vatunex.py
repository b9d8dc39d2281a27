"""Vatunex: a decoder whose layers carry a norm before and after each sublayer (RMS norms whose stored weight is used as
one plus itself) and whose mixer is, layer by layer, one of: attention through latents inside a sliding window;
grouped-query attention with biases, per-head norms of q and k, band-scaled rotary frequencies, a sink in the softmax
and values mixed with those of the first such layer; a selective-scan recurrence.  The feed-forward is dense with the
tanh form of GELU, or absent.  No position table; a final norm and an untied head.  This file only translates a
`VatunexConfig` into a `ModelSpec`: every mechanism is a registered part.

Checkpoint names: embed, l<i>.norm1, l<i>.norm1b, l<i>.norm2, l<i>.norm2b, l<i>.mix.*, l<i>.mlp.{up,down},
final.norm, head."""
from __future__ import annotations

from ..config import VatunexConfig, register_architecture
from ..parts import LayerSpec, PartSpec
from .decoder import ModelSpec


def build_vatunex(config: VatunexConfig) -> ModelSpec:
    width, eps = config.width, config.norm_eps
    norm = PartSpec("rmsnorm", {"hidden": width, "eps": eps, "tensor": "", "one_plus": True})
    layers, mixing_seen = [], False
    for layer in config.layers:
        kind, m = layer["type"], layer["mixer"]
        window = m["mask"]["size"] if m.get("mask") else None
        if kind == "latent_attention":
            mixer = PartSpec("latent_attention", {
                "hidden": width, "heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "v_head_dim": m["vdim"],
                "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": m["scale"], "window": window, "norm_eps": eps,
                "rot": m["rot"]})
        elif kind == "attention":
            mix = None
            if m.get("v_mix"):
                mix, mixing_seen = ("mixed" if mixing_seen else "source"), True
            mixer = PartSpec("sink_attention", {
                "hidden": width, "heads": m["heads"], "kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
                "v_head_dim": m.get("vdim", m["dim"]), "scale": m["scale"], "window": window, "sink": True, "biases": True,
                "qk_norm": True, "norm_eps": eps, "rot": m.get("rot"), "value_mix": mix})
        else:
            mixer = PartSpec("selective_scan", {"hidden": width, "inner": m["inner"], "state": m["state"],
                                                "dt_rank": m["dt_rank"], "taps": m["conv"]})
        mlp = layer.get("mlp")
        feed_forward = None if mlp is None else PartSpec("dense_act", {
            "hidden": width, "intermediate": mlp["ff"], "activation": "gelu_tanh", "names": {"up": "up", "down": "down"}})
        layers.append(LayerSpec(
            mixer=mixer, feed_forward=feed_forward, norm=norm, arrangement="sandwich",
            names={"norm1": "norm1", "norm1b": "norm1b", "norm2": "norm2", "norm2b": "norm2b", "mixer": "mix.",
                   "feed_forward": "mlp."}))
    return ModelSpec(hidden_size=width, vocab_size=config.vocab, max_positions=None, layers=layers, final_norm=norm,
                     embedding_name="embed", head_name="head", layer_prefix="l{}.", final_norm_prefix="final.norm")


register_architecture(("Vatunex",), VatunexConfig, build_vatunex)
