"""What needs no GPU of the Vatunex decoder: its configuration and its refusals, the registry, the model description
(tensor names, parts chosen layer by layer, caches and states), random weights through the loader, the band-scaled rotary
frequencies against the plain implementation, and the cache manager with the needs of its mixers (latents in pages of
their own under a window beside whole-context pages)."""
import copy
import json
import random

import pytest
import torch

import plain_vatunex
import vatunex_helpers as vh
from lia_rs_b200.cache import CacheManager
from lia_rs_b200.config import ConfigError, VatunexConfig, resolve_architecture
from lia_rs_b200.parts import KVCacheRequest
from lia_rs_b200.parts.rotary import band_scaled_frequencies


@pytest.mark.parametrize("name", list(vh.VATUNEX))
def test_configuration_round_trip_and_registry(name):
    raw = vh.VATUNEX[name]["config"]
    architecture = resolve_architecture(raw)
    assert architecture.name == "Vatunex" and architecture.config_class is VatunexConfig
    config = VatunexConfig.from_dict(raw)
    again = VatunexConfig.from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config and again.to_dict() == config.to_dict()
    assert [l["type"] for l in config.layers] == [l["type"] for l in raw["layers"]]


def test_configuration_refusals():
    good = vh.VATUNEX["vat-A"]["config"]

    def broken(change):
        raw = copy.deepcopy(good)
        change(raw)
        return raw

    cases = [
        (lambda r: r["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=32), "at most"),
        (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=10), "at most"),
        (lambda r: r["layers"][0]["mixer"].pop("rot"), "needs an object 'rot'"),
        (lambda r: r["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
        (lambda r: r["layers"][2].update(type="recurrent"), "not known"),
        (lambda r: r["layers"][2]["mlp"].update(kind="experts"), "not known"),
        (lambda r: r["layers"][2]["mixer"].update(conv=0), "conv"),
        (lambda r: r["layers"][3]["mixer"].update(vdim=16), "agree in kv_heads and vdim"),
        (lambda r: r["layers"][1]["mixer"]["rot"]["scaling"].update(low=4.0), "must differ"),
        (lambda r: r.pop("width"), "width"),
        (lambda r: r["norm"].pop("eps"), "norm.eps"),
        (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    ]
    for change, words in cases:
        with pytest.raises(ConfigError, match=words):
            VatunexConfig.from_dict(broken(change))
    # sizes beyond the kernels are refused when the model is described, before any tensor is read
    architecture = resolve_architecture(good)
    for change, words in [(lambda r: r["layers"][2]["mixer"].update(conv=9), "taps"),
                          (lambda r: r["layers"][2]["mixer"].update(state=300), "states"),
                          (lambda r: r["layers"][0]["mixer"].update(kv_rank=600), "kv_rank")]:
        with pytest.raises(ValueError, match=words):
            architecture.build(VatunexConfig.from_dict(broken(change)))


@pytest.mark.parametrize("name", list(vh.VATUNEX))
def test_model_description(name):
    raw = vh.VATUNEX[name]["config"]
    config = VatunexConfig.from_dict(raw)
    spec = resolve_architecture(raw).build(config)
    assert spec.max_positions is None and spec.position_table_name is None and not spec.junctions
    kinds = {"latent_attention": "latent_attention", "attention": "sink_attention", "mamba1": "selective_scan"}
    assert [l.mixer.kind for l in spec.layers] == [kinds[l["type"]] for l in raw["layers"]]
    assert all(l.arrangement == "sandwich" and l.norm.params["one_plus"] for l in spec.layers)
    names = {s.name: tuple(s.shape) for s in spec.tensor_specs() if not s.optional}
    width = raw["width"]
    assert names["embed"] == (raw["vocab"], width) and names["head"] == (raw["vocab"], width) and names["final.norm"] == (width,)
    sources = 0
    for i, layer in enumerate(raw["layers"]):
        m, p = layer["mixer"], f"l{i}."
        assert names[p + "norm1"] == (width,) and names[p + "norm1b"] == (width,)
        assert (p + "norm2" in names) == (layer["mlp"] is not None) == (p + "mlp.up" in names)
        if layer["mlp"]:
            assert names[p + "mlp.up"] == (layer["mlp"]["ff"], width) and names[p + "mlp.down"] == (width, layer["mlp"]["ff"])
        if layer["type"] == "latent_attention":
            assert names[p + "mix.dkv"] == (m["kv_rank"] + m["rot_dim"], width)
            assert names[p + "mix.uq"] == (m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"])
            assert names[p + "mix.uk"] == (m["heads"] * m["dim"], m["kv_rank"]) and names[p + "mix.uv"] == (m["heads"] * m["vdim"], m["kv_rank"])
            assert spec.cache_requests()[i] == KVCacheRequest(1, m["kv_rank"], m.get("mask", {}).get("size"), v_head_dim=m["rot_dim"])
        elif layer["type"] == "attention":
            kv, dv = m.get("kv_heads", m["heads"]), m.get("vdim", m["dim"])
            assert names[p + "mix.v"] == (kv * dv, width) and names[p + "mix.o.b"] == (width,) and names[p + "mix.q.norm"] == (m["dim"],)
            assert (p + "mix.vmix" in names) == bool(m.get("v_mix"))
            if m.get("v_mix"):
                assert names[p + "mix.vmix"] == ()
                assert spec.layers[i].mixer.params["value_mix"] == ("mixed" if sources else "source")
                sources += 1
            assert spec.cache_requests()[i] == KVCacheRequest(kv, m["dim"], m.get("mask", {}).get("size"), v_head_dim=dv)
        else:
            assert names[p + "mix.x"] == (m["dt_rank"] + 2 * m["state"], m["inner"]) and names[p + "mix.conv"] == (m["inner"], m["conv"])
            assert i not in spec.cache_requests()
            assert spec.state_requests()[i].shape == ((m["conv"] - 1) * m["inner"] + m["inner"] * m["state"],)
    # a layer without a feed-forward tolerates the absent sublayer's norms in a checkpoint
    optional = {s.name for s in spec.tensor_specs() if s.optional}
    assert optional == {f"l{i}.{n}" for i, l in enumerate(raw["layers"]) if l["mlp"] is None for n in ("norm2", "norm2b")}


@pytest.mark.parametrize("name", ["vat-A", "vat-B"])
def test_random_weights_pass_the_loader(tmp_path, name):
    from lia_rs_b200.weights import load_weights, write_random_model
    raw = vh.VATUNEX[name]["config"]
    config = VatunexConfig.from_dict(raw)
    folder = write_random_model(config, str(tmp_path / "m"), seed=5)
    spec = resolve_architecture(raw).build(config)
    tensors = load_weights(folder, spec.tensor_specs())
    assert set(tensors) == {s.name for s in spec.tensor_specs() if not s.optional}
    assert float(tensors["l0.norm1"].float().abs().max()) < 1.0          # norm weights lie around zero in this design
    if name == "vat-A":
        assert tensors["l1.mix.vmix"].shape == () and tensors["l3.mix.vmix"].shape == ()      # scalars are stored and read back


def test_band_scaled_frequencies_against_the_plain_ones():
    for base, dims, scaling in [(10000.0, 16, None), (30000.0, 20, {"factor": 3.0, "low": 1.0, "high": 6.0, "original": 256}),
                                (500.0, 64, {"factor": 8.0, "low": 0.5, "high": 16.0, "original": 100}),
                                (1e6, 128, {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 32})]:
        ours = band_scaled_frequencies(base, dims, scaling)
        plain = plain_vatunex.rotary_frequencies(base, dims, scaling)
        assert ours.shape == plain.shape and torch.allclose(ours, plain, rtol=1e-13, atol=0)
        if scaling:          # all three bands occur in the larger cases
            ratio = ours / plain_vatunex.rotary_frequencies(base, dims, None)
            assert float(ratio.max()) <= 1.0 + 1e-12 and float(ratio.min()) >= 1.0 / scaling["factor"] - 1e-12


def test_cache_manager_with_latent_and_whole_context_groups():
    """Latent pages under a window beside whole-context pages: random admissions, portions and releases keep the
    invariants; the window group gives pages back as a request moves on, the other does not."""
    latent = KVCacheRequest(1, 32, 21, v_head_dim=8)
    whole = KVCacheRequest(2, 16, None, v_head_dim=8)
    manager = CacheManager({0: latent, 1: whole, 4: latent}, {}, num_pages=40, page_size=8, max_slots=3,
                           max_context=200, dtype=torch.float32)
    assert len(manager.groups) == 2
    window_group = manager.group_of[0]
    assert manager.group_of[4] is window_group and window_group.v[0].shape[-1] == 8 and window_group.k[0].shape[-1] == 32
    rng = random.Random(7)
    at = {}
    for _ in range(300):
        if at and rng.random() < 0.15:
            slot = rng.choice(list(at))
            manager.release(slot)
            del at[slot]
        elif len(at) < 3 and rng.random() < 0.3:
            at[manager.admit()] = 0
        elif at:
            slot = rng.choice(list(at))
            count = rng.choice([1, 1, 2, 5, 17])
            if at[slot] + count <= 200 and manager.ensure(slot, at[slot], at[slot] + count):
                at[slot] += count
                held = window_group.held_by(slot)
                assert held <= (21 + count + 2 * 8) // 8 + 1            # only what the window and the portion span
        manager.check()
