"""Nafevik: a decoder with learned positions added to the embedding; parallel layers (one RMSNorm whose output, passed
through a short causal convolution of its own for each sublayer, feeds a gated sigmoid attention and a SwiGLU
feed-forward, both added to the stream times `residual_mult`); a run of layers that repeats with the same weights,
each pass with caches and states of its own and the embedding output re-injected ahead of it; a final RMSNorm and an
untied head.  This file only translates a `NafevikConfig` into a `ModelSpec`: every mechanism is a registered part.

Checkpoint names: embed, pos, loop.in, loop.step, l<i>.norm1, l<i>.mix.{q,k,v,pb,g,o}, l<i>.mlp.{gate,up,down},
l<i>.canon1, l<i>.canon2, final.norm, head."""
from __future__ import annotations

from ..config import NafevikConfig, register_architecture
from ..parts import LayerSpec, PartSpec
from .decoder import ModelSpec, ScheduleEntry


def build_nafevik(config: NafevikConfig) -> ModelSpec:
    width = config.width
    layers = []
    for layer in config.layers:
        mixer = layer["mixer"]
        rot = mixer.get("rot")
        position = PartSpec("rotary_pairs", {"base": rot["base"], "rotary_dim": rot["dims"], "scaling": rot.get("scaling")}
                            if rot else {"base": 2.0, "rotary_dim": 0, "scaling": None})
        heads, dim = mixer["heads"], mixer["dim"]
        attention = PartSpec("sigmoid_attention", {
            "hidden": width, "heads": heads, "kv_heads": mixer.get("kv_heads", heads), "head_dim": dim,
            "v_head_dim": mixer.get("vdim", dim), "scale": mixer["scale"], "window": None,
            "chunk": mixer["mask"]["size"] if mixer.get("mask") else None, "position": position})
        mlp = layer.get("mlp")
        feed_forward = None if mlp is None else PartSpec("swiglu", {
            "hidden": width, "intermediate": mlp["ff"], "names": {"gate": "gate", "up": "up", "down": "down"}})
        options = {}
        if config.canon_taps:
            options["input_conv"] = {"taps": config.canon_taps, "names": ("canon1", "canon2")}
        layers.append(LayerSpec(
            mixer=attention, feed_forward=feed_forward,
            norm=PartSpec("rmsnorm", {"hidden": width, "eps": config.norm_eps, "tensor": ""}),
            arrangement="parallel", residual_scale=config.residual_mult, options=options,
            names={"norm1": "norm1", "mixer": "mix.", "feed_forward": "mlp."}))
    schedule, junctions = [], {}
    for position, (layer, loop_pass, first_of_pass) in enumerate(config.layer_runs()):
        schedule.append(ScheduleEntry(layer, cache=position))          # every run of a layer has a cache of its own
        if first_of_pass:
            junctions[position] = PartSpec("reinject", {"hidden": width, "row": loop_pass, "rows": config.loop[2],
                                                        "names": {"weight": "loop.in", "bias": "loop.step"}})
    return ModelSpec(
        hidden_size=width, vocab_size=config.vocab, max_positions=config.max_positions, layers=layers,
        final_norm=PartSpec("rmsnorm", {"hidden": width, "eps": config.norm_eps, "tensor": ""}),
        schedule=schedule, embedding_name="embed", head_name="head", layer_prefix="l{}.",
        final_norm_prefix="final.norm", position_table_name="pos", junctions=junctions)


register_architecture(("Nafevik",), NafevikConfig, build_nafevik)
