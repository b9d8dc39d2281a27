"""Tiny Vatunex configurations for the tests, their model folders with random weights, and the comparison with the
plain implementation (tests/plain_vatunex.py).

The configurations differ in everything that config.json gives: widths and vocabularies; the order of the three kinds
of layer (each kind first, last and alone somewhere); latent attention with 1, 2, 3 and 4 heads, ranks smaller and
larger than the width, a model of scans alone, windows that are no multiple of the page size, one layer without a window; attention with 1, 2
and 4 query heads per kv head, key and value head sizes equal and unequal, rotation of all, part or none of a head, band
scaling present and absent, a window on one layer, value mixing in none, two or three layers; scans with 1 to 4 taps,
state sizes from 3 to 24 (one to four lanes a channel) and ranks of 1 and more; layers without a feed-forward."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

import plain_vatunex


def _latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, window, base, ff):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _attention(heads, kv_heads, dim, vdim, scale, rot, v_mix, window, ff):
    mixer = {"heads": heads, "dim": dim, "scale": scale}
    if kv_heads:
        mixer["kv_heads"] = kv_heads
    if vdim:
        mixer["vdim"] = vdim
    if rot:
        mixer["rot"] = rot
    if v_mix is not None:
        mixer["v_mix"] = v_mix
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _scan(inner, state, dt_rank, conv, ff):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


_BANDS = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}

VATUNEX = {
    "vat-A": dict(
        config={"architecture": "Vatunex", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "initializer_range": 0.08,
                "layers": [_latent(2, 16, 8, 24, 32, 40, 0.2, 21, 10000.0, 96),
                           _attention(4, 2, 16, 8, 0.25, {"base": 10000.0, "dims": 8, "scaling": _BANDS}, True, None, 96),
                           _scan(96, 8, 4, 3, 80),
                           _attention(4, 2, 24, 8, 0.2, {"base": 500.0, "dims": 24}, True, 13, None),
                           _latent(3, 8, 4, 8, 16, 72, 0.3, 9, 300.0, 64)]},
        seed=1, page_size=8, sharpen=2.0),
    "vat-B": dict(
        config={"architecture": "Vatunex", "vocab": 131, "width": 96, "norm": {"eps": 3e-6}, "initializer_range": 0.06,
                "layers": [_scan(72, 5, 3, 4, 120),
                           _attention(3, None, 24, None, 0.2, None, False, None, 80),
                           _latent(1, 32, 16, 16, 48, 24, 0.18, None, 2000.0, None),
                           _scan(40, 24, 1, 1, 48)]},
        seed=2, page_size=4, sharpen=2.5),
    "vat-C": dict(
        config={"architecture": "Vatunex", "vocab": 211, "width": 128, "norm": {"eps": 1e-6}, "initializer_range": 0.05,
                "layers": [_attention(4, 1, 128, 128, 0.09, {"base": 25000.0, "dims": 64, "scaling":
                                                             {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 32}}, True, None, 192),
                           _latent(4, 64, 32, 48, 96, 64, 0.1, 40, 25000.0, 192),
                           _attention(4, 1, 128, 128, 0.09, {"base": 25000.0, "dims": 128}, True, None, 192),
                           _scan(256, 16, 8, 2, 192),
                           _attention(8, 2, 64, 64, 0.125, {"base": 1e6, "dims": 32}, False, 50, 64)]},
        seed=3, page_size=16, sharpen=1.5),
    "vat-D": dict(
        config={"architecture": "Vatunex", "vocab": 157, "width": 80, "norm": {"eps": 2e-5}, "initializer_range": 0.07,
                "layers": [_latent(4, 24, 16, 40, 56, 32, 0.15, 33, 1000.0, 100),
                           _scan(160, 3, 5, 2, None),
                           _latent(4, 24, 16, 40, 56, 32, 0.15, 17, 1000.0, 100)]},
        seed=4, page_size=16, sharpen=1.5),
    "vat-E": dict(          # no attention at all: the engine runs without a page pool, on state slots alone
        config={"architecture": "Vatunex", "vocab": 83, "width": 56, "norm": {"eps": 1e-5}, "initializer_range": 0.08,
                "layers": [_scan(88, 6, 2, 3, 72), _scan(64, 10, 7, 5, None)]},
        seed=5, page_size=8, sharpen=1.0),
}


def random_configuration(seed: int) -> dict:
    """A configuration drawn at random: 3 to 6 layers of the three kinds in any order, sizes that are and are not
    multiples of 8, 16 or 32, every optional key present or absent."""
    import random
    rng = random.Random(seed)
    width = rng.choice([48, 64, 72, 96, 128, 144])
    if seed % 3 == 0:
        width = random.Random(seed).choice([50, 66, 100, 257])          # rows that no 16-byte access fits
    mixing = (rng.choice([1, 2]), rng.choice([8, 16, 24, 32]))            # kv heads and value size of the layers that mix values
    layers = []
    for _ in range(rng.randint(3, 6)):
        kind = rng.choice(["latent", "attention", "scan"])
        ff = rng.choice([None, 40, 96, 160, 200])
        if kind == "latent":
            rot_dim = rng.choice([4, 8, 16, 32])
            layers.append(_latent(rng.choice([1, 2, 3, 4, 5]), rng.choice([8, 16, 24, 64]), rot_dim, rng.choice([8, 16, 40]),
                                  rng.choice([16, 32, 48, 64, 96, 128]), rng.choice([16, 24, 64, 100]), rng.uniform(0.1, 0.3),
                                  rng.choice([None, 5, 16, 31, 64]), rng.choice([100.0, 10000.0, 500000.0]), ff))
        elif kind == "attention":
            mixes = rng.random() < 0.6
            kv = mixing[0] if mixes else rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 32, 48, 64, 128])
            vdim = mixing[1] if mixes else rng.choice([None, 8, dim])
            rot = None
            if rng.random() < 0.8:
                rot = {"base": rng.choice([100.0, 10000.0, 1e6]), "dims": rng.choice([d for d in (2, 4, 8, 16, 32, dim) if d <= dim])}
                if rng.random() < 0.5:
                    rot["scaling"] = {"factor": rng.choice([2.0, 4.0, 8.0]), "low": 1.0, "high": rng.choice([2.0, 4.0, 16.0]),
                                      "original": rng.choice([16, 64, 512])}
            group = rng.choice([1, 2, 4])
            named = kv if group > 1 or rng.random() < 0.5 else None          # heads == kv_heads: the key may be absent
            layers.append(_attention(kv * group, named, dim, vdim, rng.uniform(0.08, 0.3), rot,
                                     True if mixes else rng.choice([None, False]), rng.choice([None, None, 7, 32, 50]), ff))
        else:
            layers.append(_scan(rng.choice([24, 64, 100, 192]), rng.choice([1, 4, 8, 12, 16, 33]), rng.choice([1, 2, 8, 12]),
                                rng.choice([1, 2, 3, 4, 5]), ff))
    return {"architecture": "Vatunex", "vocab": rng.choice([61, 128, 250]), "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 3e-5])},
            "initializer_range": 0.07, "layers": layers}


def make_model(folder: str, name: str) -> dict:
    """The folder through the package's random-weights mode; then the weights are moved to where a fault shows: the
    matrices that make queries and keys are scaled up (peaked attention weights: a wrong, missing or extra key changes
    the output), norm weights and biases are spread, the mixing scalars lie well inside (0, 1), the scan's decays, step
    biases and taps are spread so that state carried wrongly shows after a few tokens.
    Returns {dir, config, weights (by checkpoint name, as stored), page_size, name}."""
    from safetensors.torch import load_file, save_file

    from lia_rs_b200.config import VatunexConfig
    from lia_rs_b200.weights import write_random_model
    entry = VATUNEX[name] if name in VATUNEX else dict(config=random_configuration(int(name.split("-")[1])), seed=int(name.split("-")[1]),
                                                        page_size=(4, 8, 16)[int(name.split("-")[1]) % 3], sharpen=2.0)
    write_random_model(VatunexConfig.from_dict(entry["config"]), folder, seed=entry["seed"])
    path = os.path.join(folder, "model.safetensors")
    weights = load_file(path)
    g = torch.Generator().manual_seed(entry["seed"] + 100)
    bf16 = lambda t: t.to(torch.bfloat16)
    for key in list(weights):
        shape = weights[key].shape
        tail = key.split(".", 1)[1] if "." in key else key
        if tail in ("mix.q", "mix.k", "mix.uq", "mix.uk", "mix.dkv"):
            weights[key] = bf16(weights[key].float() * entry["sharpen"])
        elif "norm" in tail and tail.startswith("mix."):
            weights[key] = bf16(1.0 + 0.3 * torch.randn(shape, generator=g))
        elif "norm" in key:
            weights[key] = bf16(0.3 * torch.randn(shape, generator=g))
        elif tail.endswith(".b") and tail != "mix.dt.b":
            weights[key] = bf16(0.5 * torch.randn(shape, generator=g))
        elif tail == "mix.vmix":
            weights[key] = bf16(torch.tensor(0.3 + 0.4 * float(torch.rand((), generator=g))))
        elif tail == "mix.A_log":
            weights[key] = bf16(torch.log(0.2 + 3.0 * torch.rand(shape, generator=g)))
        elif tail == "mix.dt.b":
            weights[key] = bf16(torch.randn(shape, generator=g) - 1.0)
        elif tail == "mix.D":
            weights[key] = bf16(1.0 + 0.5 * torch.randn(shape, generator=g))
        elif tail == "mix.conv":
            weights[key] = bf16(0.6 * torch.randn(shape, generator=g))
        elif tail in ("mix.x", "mix.dt"):
            weights[key] = bf16(weights[key].float() * 3.0)
    save_file(weights, path)
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    return dict(dir=folder, config=config, weights=weights, page_size=entry["page_size"], name=name)


_CACHE = {}


def plain_logits(model: dict, tokens) -> torch.Tensor:
    key = (model["name"], tuple(tokens))
    if key not in _CACHE:
        _CACHE[key] = plain_vatunex.forward(model["config"], model["weights"], list(tokens))
    return _CACHE[key]


def longest_sum(config: dict) -> int:
    sizes = [config["width"]]
    for layer in config["layers"]:
        m = layer["mixer"]
        if layer["type"] == "mamba1":
            sizes.append(m["inner"])
        else:
            sizes.append(m["heads"] * max(m["dim"] + m.get("rot_dim", 0), m.get("vdim", m["dim"]), m.get("kv_rank", 0)))
        if layer.get("mlp"):
            sizes.append(layer["mlp"]["ff"])
    return max(sizes)


def assert_close(actual, reference, dtype: str, what: str, config: dict):
    """Against the exact (64-bit) model.  32-bit: every logit within 8 K 2^-24 of the largest logit per layer that the
    sums pass through (K the model's longest sum).  bfloat16: every row's root-mean-square error within 2.5e-2 of the
    largest logit, times the root of the number of layers over 3 (rounding noise of a layer adds to that of the layers
    before; a recurrent layer carries its rounding along the sequence and counts as four), and no single logit further
    off than three times that (a norm directly behind a sublayer magnifies the rounding of a small output, so single rows
    stand out however the work is cut)."""
    actual = torch.as_tensor(np.asarray(actual), dtype=torch.float64)
    reference = reference.to(torch.float64)
    assert actual.shape == reference.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(reference.shape)}"
    assert torch.isfinite(actual).all(), f"{what}: non-finite logits"
    layers = len(config["layers"])
    scale = max(1.0, float(reference.abs().max()))
    error = (actual - reference).abs()
    if dtype == "float32":
        limit = 8.0 * longest_sum(config) * 2.0 ** -24 * scale * layers
        worst = float(error.max())
    else:
        weighted = layers + 3 * sum(1 for layer in config["layers"] if layer["type"] == "mamba1")
        limit = 2.5e-2 * scale * max(1.0, (weighted / 3.0) ** 0.5)
        worst = max(float((error ** 2).mean(dim=-1).sqrt().max()), float(error.max()) / 3.0)
    if worst > limit:
        row = int(error.max(dim=-1).values.argmax()) if error.dim() > 1 else 0
        raise AssertionError(f"{what}: error {worst:.3e} > {limit:.3e} (largest at wanted row {row})")
