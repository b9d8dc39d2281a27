"""What needs no GPU of the Nafevik decoder: its configuration and its refusals, the registry, the model description
(tensor names, the order of layer runs, caches and states of every run, junctions), random weights through the
loader, the scaled rotary frequencies, and the cache manager's rule for attention in blocks (pages before a request's
current block are given back; values may have a head size of their own)."""
import copy
import json
import random

import pytest
import torch

import nafevik_helpers as nh
import plain_nafevik
from lia_rs_b200.cache import CacheManager
from lia_rs_b200.config import ConfigError, NafevikConfig, resolve_architecture
from lia_rs_b200.parts import KVCacheRequest, StateRequest
from lia_rs_b200.parts.rotary import scaled_frequencies


@pytest.mark.parametrize("name", list(nh.NAFEVIK))
def test_configuration_round_trip_and_registry(name):
    raw = nh.NAFEVIK[name]["config"]
    architecture = resolve_architecture(raw)
    assert architecture.name == "Nafevik" and architecture.config_class is NafevikConfig
    config = NafevikConfig.from_dict(raw)
    again = NafevikConfig.from_dict(json.loads(json.dumps(config.to_dict())))
    assert again == config and again.to_dict() == config.to_dict()
    assert config.canon_taps == raw.get("canon", {}).get("taps", 0)
    assert [i for i, _, _ in config.layer_runs()] == [i for i, _ in plain_nafevik.layer_runs(raw)]
    assert [t for _, t, first in config.layer_runs() if first] == [t for _, t in plain_nafevik.layer_runs(raw) if t is not None]


def test_configuration_refusals():
    good = nh.NAFEVIK["naf-A"]["config"]

    def broken(change):
        raw = copy.deepcopy(good)
        change(raw)
        return raw

    cases = [
        (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
        (lambda r: r["layers"][1]["mixer"]["rot"].update(dims=32), "at most dim"),
        (lambda r: r["layers"][2].update(type="recurrent"), "not known"),
        (lambda r: r["layers"][2]["mlp"].update(kind="experts"), "not known"),
        (lambda r: r["loop"].update(stop=9), "does not lie within"),
        (lambda r: r["loop"].update(times=0), "positive integer"),
        (lambda r: r.pop("width"), "width"),
        (lambda r: r["norm"].pop("eps"), "norm.eps"),
        (lambda r: r["canon"].update(taps=0), "canon.taps"),
        (lambda r: r["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
    ]
    for change, words in cases:
        with pytest.raises(ConfigError, match=words):
            NafevikConfig.from_dict(broken(change))
    with pytest.raises(ConfigError, match="unsupported model architecture"):
        resolve_architecture({"architecture": "Somethingelse"})
    # too many taps for the kernel is refused when the model is described, before any tensor is read
    with pytest.raises(ValueError, match="taps"):
        resolve_architecture(good).build(NafevikConfig.from_dict(broken(lambda r: r["canon"].update(taps=9))))


def test_model_description_of_a_looped_model():
    raw = nh.NAFEVIK["naf-B"]["config"]                       # three layers of different sizes, all looped twice
    spec = resolve_architecture(raw).build(NafevikConfig.from_dict(raw))
    names = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    assert names["embed"] == (131, 96) and names["pos"] == (192, 96) and names["head"] == (131, 96)
    assert names["loop.in"] == (96, 192) and names["loop.step"] == (2, 96) and names["final.norm"] == (96,)
    assert names["l0.mix.q"] == (96, 96) and names["l0.mix.k"] == (32, 96) and names["l0.mix.v"] == (16, 96)
    assert names["l0.mix.pb"] == (3,) and names["l0.mix.g"] == (3, 96) and names["l0.mix.o"] == (96, 48)
    assert names["l1.mix.v"] == (96, 96) and names["l1.norm1"] == (96,) and names["l1.canon1"] == (96, 2)
    assert "l1.mlp.gate" not in names and "l1.canon2" not in names          # a layer without a feed-forward
    assert names["l2.mlp.gate"] == (120, 96) and names["l2.mlp.down"] == (96, 120) and names["l2.canon2"] == (96, 2)
    assert len(names) == 6 + (7 + 3 + 2) + (7 + 1) + (7 + 3 + 2)      # model-wide, then each layer's: norm and mixer, feed-forward, taps
    assert [e.layer for e in spec.schedule] == [0, 1, 2, 0, 1, 2]
    assert [e.cache for e in spec.schedule] == list(range(6))             # every run has a cache of its own
    assert sorted(spec.junctions) == [0, 3]                                  # ahead of the first layer of each pass
    assert [spec.junctions[p].params["row"] for p in (0, 3)] == [0, 1]
    needs = spec.cache_requests()
    assert needs[0] == needs[3] == KVCacheRequest(1, 32, None, v_head_dim=16, chunk=7)
    assert needs[1] == KVCacheRequest(2, 16, None, v_head_dim=48, chunk=None)
    states = spec.state_requests()
    assert sorted(states, key=str) == [("layer", p) for p in range(6)]
    assert all(request == StateRequest((1, 96), torch.float32) for request in states.values())
    # no loop, no convolution: no junction, no state, the plain order
    plain_raw = nh.NAFEVIK["naf-C"]["config"]
    plain_spec = resolve_architecture(plain_raw).build(NafevikConfig.from_dict(plain_raw))
    assert not plain_spec.junctions and not plain_spec.state_requests() and "loop.in" not in {s.name for s in plain_spec.tensor_specs()}
    assert [e.layer for e in plain_spec.schedule] == [0, 1]


def test_random_weights_load_by_name(tmp_path):
    from lia_rs_b200.weights import Archive, load_weights
    model = nh.make_model(str(tmp_path / "m"), "naf-D")
    raw = model["config"]
    spec = resolve_architecture(raw).build(NafevikConfig.from_dict(raw))
    tensors = load_weights(model["dir"], spec.tensor_specs())
    assert set(tensors) == set(Archive(model["dir"]).names()) == {s.name for s in spec.tensor_specs()}
    assert tensors["l1.mix.q"].dtype == torch.bfloat16 and tuple(tensors["l0.canon2"].shape) == (80, 4)
    logits = plain_nafevik.forward(raw, model["weights"], [1, 2, 3, 4, 5])
    assert logits.shape == (5, 157) and torch.isfinite(logits).all() and float(logits.std()) > 1e-3


def test_scaled_frequencies_against_the_plain_formula():
    for base, dims, scaling in [(10000.0, 64, None), (30000.0, 56, {"factor": 6.0, "original": 256, "fast": 24.0, "slow": 1.5}),
                                (500.0, 8, {"factor": 32.0, "original": 4096, "fast": 4.0, "slow": 2.0}),
                                (1e6, 128, {"factor": 1.5, "original": 64, "fast": 64.0, "slow": 0.5})]:
        freq, magnitude = scaled_frequencies(base, dims, scaling)
        want, want_magnitude = plain_nafevik.rotary_frequencies(base, dims, scaling)
        assert torch.allclose(freq, want, rtol=1e-13, atol=0) and abs(magnitude - want_magnitude) < 1e-14
        if scaling:
            plain_freq = plain_nafevik.rotary_frequencies(base, dims)[0]
            assert torch.all(freq <= plain_freq * (1 + 1e-12)) and torch.all(freq >= plain_freq / scaling["factor"] * (1 - 1e-12))


def test_cache_gives_back_the_pages_before_a_request_block():
    """Blocks of 10 positions on pages of 4: a token at position 23 reads keys 20..23, so pages 0..4 (positions
    0..19) are given back; a portion that begins in one block and ends in the next keeps the first one's pages."""
    need = KVCacheRequest(2, 16, None, v_head_dim=24, chunk=10)
    m = CacheManager({0: need, 1: need, 2: KVCacheRequest(2, 16, None)}, {}, 16, 4, 3, 128, torch.float32, "cpu")
    assert len(m.groups) == 2
    blocked = m.group_of[0]
    assert m.kv_view(0, True).v_pages.shape == (16, 4, 2, 24) and m.kv_view(0, True).k_pages.shape == (16, 4, 2, 16)
    s = m.admit()
    assert m.ensure(s, 0, 19) and blocked.held_by(s) == 5 and m.group_of[2].held_by(s) == 5
    assert m.ensure(s, 19, 24)                                   # begins at 19: block 10..19 starts on page 2
    assert blocked.tables[s][:2] == [-1, -1] and blocked.held_by(s) == 4 and m.group_of[2].held_by(s) == 6
    assert m.ensure(s, 24, 25) and blocked.held_by(s) == 2       # position 24 reads 20..24: pages 5 and 6
    assert blocked.tables[s][:5] == [-1] * 5
    m.check()
    m.flush()
    assert blocked.device_table[s, :7].tolist() == blocked.tables[s][:7]
    m.release(s)
    assert blocked.pool.in_use() == 0
    # random orders keep the invariants, and a block's pages are there while its tokens come
    rng = random.Random(5)
    at = {}
    for _ in range(300):
        live = m.live_slots()
        action = rng.random()
        if action < 0.2 and m.free_slots():
            at[m.admit()] = 0
        elif action < 0.3 and live:
            slot = rng.choice(live)
            m.release(slot)
            del at[slot]
        elif live:
            slot = rng.choice(live)
            count = rng.randint(1, 9)
            if at[slot] + count <= 128 and m.ensure(slot, at[slot], at[slot] + count):
                first_key = at[slot] // 10 * 10
                table = blocked.tables[slot]
                assert all(table[b] >= 0 for b in range(first_key // 4, (at[slot] + count - 1) // 4 + 1))
                at[slot] += count
        m.check()
