"""Tiny Nafevik configurations for the tests, their model folders with random weights, and the comparison with the
plain implementation (tests/plain_nafevik.py).

The configurations differ in everything that config.json gives: widths, vocabularies, head counts and groups (1, 2,
3 and 4 query heads per kv head), key and value head sizes (equal and unequal, powers of two and not), the share
of a head that is rotated (all of it, part of it, none), frequency scaling present and absent, block sizes of the
attention that are no multiple of the page size (and a layer without blocks), 2, 3 and 4 taps of the input
convolution (and none), loops of 1, 2 and 3 passes that start at the first layer or later and end at the last layer
or earlier (and no loop), a layer without a feed-forward, layers of different sizes in one model, residual
multipliers."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_nafevik


def _layer(heads, kv_heads, dim, vdim, scale, chunk, rot, ff):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        mixer["mask"] = {"size": chunk}
    if rot:
        mixer["rot"] = rot
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


_SCALED = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}

NAFEVIK = {
    "naf-A": dict(
        config={"architecture": "Nafevik", "vocab": 97, "width": 64, "max_positions": 256, "norm": {"eps": 1e-5},
                "residual_mult": 0.5, "canon": {"taps": 3}, "initializer_range": 0.08,
                "layers": [_layer(4, 2, 16, 16, 0.25, 24, {"base": 10000.0, "dims": 16, "scaling": _SCALED}, 96),
                           _layer(4, 2, 16, 16, 0.25, 24, {"base": 10000.0, "dims": 16, "scaling": _SCALED}, 96),
                           _layer(4, 2, 16, 16, 0.25, 24, {"base": 10000.0, "dims": 16, "scaling": _SCALED}, 96)],
                "loop": {"start": 1, "stop": 2, "times": 3}},
        seed=1, page_size=8, sharpen=2.0),
    "naf-B": dict(
        config={"architecture": "Nafevik", "vocab": 131, "width": 96, "max_positions": 192, "norm": {"eps": 3e-6},
                "residual_mult": 0.8, "canon": {"taps": 2}, "initializer_range": 0.06,
                "layers": [_layer(3, 1, 32, 16, 0.2, 7, {"base": 500.0, "dims": 8}, 80),
                           _layer(2, 2, 16, 48, 0.3, None, {"base": 3000.0, "dims": 16, "scaling": _SCALED}, None),
                           _layer(6, 2, 8, 24, 0.4, 33, None, 120)],
                "loop": {"start": 0, "stop": 3, "times": 2}},
        seed=2, page_size=4, sharpen=2.5),
    "naf-C": dict(
        config={"architecture": "Nafevik", "vocab": 211, "width": 128, "max_positions": 640, "norm": {"eps": 1e-6},
                "residual_mult": 1.0, "initializer_range": 0.05,
                "layers": [_layer(4, 1, 64, 64, 0.125, 40, {"base": 25000.0, "dims": 32}, 192),
                           _layer(4, 1, 64, 64, 0.125, 40, {"base": 25000.0, "dims": 32}, 192)]},
        seed=3, page_size=16, sharpen=1.5),
    "naf-D": dict(
        config={"architecture": "Nafevik", "vocab": 157, "width": 80, "max_positions": 320, "norm": {"eps": 2e-5},
                "residual_mult": 0.35, "canon": {"taps": 4}, "initializer_range": 0.07,
                "layers": [_layer(2, 2, 40, 24, 0.16, 50, {"base": 1000.0, "dims": 40, "scaling":
                                                           {"factor": 2.0, "original": 32, "fast": 8.0, "slow": 1.0}}, 100),
                           _layer(4, 1, 128, 128, 0.09, 64, {"base": 1e6, "dims": 64}, 64)],
                "loop": {"start": 1, "stop": 2, "times": 1}},
        seed=4, page_size=16, sharpen=1.5),
}


def make_model(folder: str, name: str) -> dict:
    """The folder through the package's random-weights mode; then q and k are scaled up (peaked weights: a wrong or
    missing key shows), the heads' score biases are set to values between -3 and 1, and the norm weights are moved
    off 1.  Returns {dir, config, weights (by checkpoint name, as stored), page_size, name}."""
    from safetensors.torch import load_file, save_file

    from lia_rs_b200.config import NafevikConfig
    from lia_rs_b200.weights import write_random_model
    entry = NAFEVIK[name]
    write_random_model(NafevikConfig.from_dict(entry["config"]), folder, seed=entry["seed"])
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    generator = torch.Generator().manual_seed(entry["seed"] + 100)
    for key in list(weights):
        if key.endswith(".mix.q") or key.endswith(".mix.k"):
            weights[key] = (weights[key].float() * entry["sharpen"]).to(torch.bfloat16)
        elif key.endswith(".mix.pb"):
            weights[key] = (torch.rand(weights[key].shape, generator=generator) * 4.0 - 3.0).to(torch.bfloat16)
        elif key.endswith("norm1") or key == "final.norm":
            weights[key] = (1.0 + 0.2 * torch.randn(weights[key].shape, generator=generator)).to(torch.bfloat16)
        elif key.endswith("canon1") or key.endswith("canon2"):
            weights[key] = (0.5 * torch.randn(weights[key].shape, generator=generator)).to(torch.bfloat16)
        elif key in ("pos", "loop.step"):
            weights[key] = (weights[key].float() * 3.0).to(torch.bfloat16)
    save_file(weights, path)
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return dict(dir=folder, config=config, weights=weights, page_size=entry["page_size"], name=name)


_CACHE = {}


def plain_logits(model: dict, tokens, dtype: str = "float32") -> torch.Tensor:
    key = (model["name"], tuple(tokens), dtype)
    if key not in _CACHE:
        store = plain_nafevik.exact if dtype == "float32" else plain_nafevik.to_bf16
        _CACHE[key] = plain_nafevik.forward(model["config"], model["weights"], tokens, store=store)
    return _CACHE[key]


def longest_sum(config: dict) -> int:
    sizes = [2 * config["width"]]
    for layer in config["layers"]:
        mixer = layer["mixer"]
        sizes.append(mixer["heads"] * max(mixer["dim"], mixer.get("vdim", mixer["dim"])))
        if layer.get("mlp"):
            sizes.append(layer["mlp"]["ff"])
    return max(sizes)


def assert_close(actual, reference, dtype: str, what: str, config: dict):
    """32-bit: 4 K 2^-24 of the largest logit per layer run that the sums pass through (K the model's longest sum).
    bfloat16: against the plain model that rounds where the serving path stores 16-bit values; what remains is the
    order of the sums and an element here and there that rounds the other way: 1e-2 of the largest logit, times the
    root of the number of layer runs over 3 (rounding noise of a run adds to that of the runs before)."""
    actual = torch.as_tensor(np.asarray(actual), dtype=torch.float64)
    reference = reference.to(torch.float64)
    assert actual.shape == reference.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(reference.shape)}"
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    runs = len(plain_nafevik.layer_runs(config))
    scale = max(1.0, float(reference.abs().max()))
    if dtype == "float32":
        limit = 4.0 * longest_sum(config) * 2.0 ** -24 * scale * runs
    else:
        limit = 1e-2 * scale * max(1.0, (runs / 3.0) ** 0.5)
    error = (actual - reference).abs()
    worst = float(error.max())
    if worst > limit:
        row = int(error.max(dim=-1).values.argmax()) if error.dim() > 1 else 0
        raise AssertionError(f"{what}: max abs error {worst:.3e} > {limit:.3e} (first at wanted row {row})")
