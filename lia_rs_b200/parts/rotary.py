"""Rotary position encoding, rotate-half over the first `rotary_dim` elements of each head
(src/gpu/kernels/llama.rs:44-55): inv_i = theta^(-2i/rotary_dim), angle = position * inv_i.
The inverse frequencies are computed in 64-bit on the host and rounded once to 32-bit; angle,
sine and cosine are 32-bit on the device.  Fused with the append of keys and values to the cache.
Parameters: theta, rotary_dim.  `none` encodes nothing and only appends."""
from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # positions are read on the device

    @staticmethod
    def check_params(params):
        rotary_dim, theta = int(params["rotary_dim"]), float(params["theta"])
        if rotary_dim % 2 or rotary_dim <= 0 or not theta > 0:
            raise ValueError("rotary encoding needs an even positive rotary_dim and theta > 0")

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.rotary_dim = int(params["rotary_dim"])
        theta = float(params["theta"])
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        inv = 1.0 / (theta ** (2.0 * i / self.rotary_dim))
        self.inv_freq = inv.to(torch.float32).to(runtime.device)

    def rotate_half(self):
        return self.rotary_dim, self.inv_freq

    def encode_and_store(self, ctx, qkv, q_out, kv, nq, nkv, d):
        self.runtime.ops.rope_kv_write(qkv, ctx.positions, ctx.slots, kv.block_table, q_out, kv.k_pages,
                                       kv.v_pages, nq, nkv, d, self.rotary_dim, self.inv_freq,
                                       write_kv=kv.writes, error_flag=ctx.error_flag)


@register_position_encoding("none")
class NoEncoding(PositionEncoding):
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # positions are read on the device

    def rotate_half(self):
        return 0, None

    def encode_and_store(self, ctx, qkv, q_out, kv, nq, nkv, d):
        self.runtime.ops.rope_kv_write(qkv, ctx.positions, ctx.slots, kv.block_table, q_out, kv.k_pages,
                                       kv.v_pages, nq, nkv, d, 0, None, write_kv=kv.writes,
                                       error_flag=ctx.error_flag)


def scaled_frequencies(base: float, rotary_dim: int, scaling=None):
    """(frequencies [rotary_dim / 2] in 64-bit, magnitude) of a rotary encoding with f_i = base^(-2i/rotary_dim).

    `scaling` (None: plain) holds `factor`, `original`, `fast`, `slow`: the wavelength-dependent interpolation in
    which a pair that turns more than `fast` times over `original` positions keeps its frequency, one that turns
    fewer than `slow` times has it divided by `factor`, and those between are blended linearly in the pair's
    index: with index(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln base), lo = max(floor(index(fast)), 0),
    hi = min(ceil(index(slow)), rotary_dim - 1), blend_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1),
        f_i' = f_i / factor * blend_i + f_i * (1 - blend_i),
    and sine and cosine are multiplied by the magnitude 0.1 ln(factor) + 1."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / rotary_dim)
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index(float(scaling["slow"]))), rotary_dim - 1)
    blend = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * blend + freq * (1.0 - blend), 0.1 * math.log(factor) + 1.0


def band_scaled_frequencies(base: float, rotary_dim: int, scaling=None):
    """Frequencies [rotary_dim / 2] in 64-bit of a rotary encoding with f_i = base^(-2i/rotary_dim).

    `scaling` (None: plain) holds `factor`, `low`, `high`, `original`: the interpolation by wavelength bands in which,
    with l_i = 2 pi / f_i, a pair whose wavelength is shorter than original / high keeps its frequency, one whose
    wavelength is longer than original / low has it divided by `factor`, and those between are blended,
        s_i = (original / l_i - low) / (high - low),   f_i' = (1 - s_i) f_i / factor + s_i f_i.
    Sine and cosine keep their magnitude."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    freq = float(base) ** (-2.0 * i / rotary_dim)
    if not scaling:
        return freq
    factor, low, high, original = (float(scaling[key]) for key in ("factor", "low", "high", "original"))
    wavelength = 2.0 * math.pi / freq
    blend = (original / wavelength - low) / (high - low)
    blended = (1.0 - blend) * freq / factor + blend * freq
    return torch.where(wavelength < original / high, freq, torch.where(wavelength > original / low, freq / factor, blended))


@register_position_encoding("rotary_pairs")
class RotaryPairs(PositionEncoding):
    """Rotary encoding in which element 2i of a head is paired with element 2i+1 (the interleaved layout), over
    the first `rotary_dim` elements; the rest pass unchanged.  Parameters: base, rotary_dim (0: nothing is encoded),
    scaling (see `scaled_frequencies`; None: plain).  The frequencies are computed in 64-bit on the host and
    rounded once to 32-bit; angle, sine and cosine are 32-bit on the device.  Keys and values may have different
    head sizes (`v_dim`).  It is not the rotate-half form, so it never rides inside the decode attention kernel."""
    graph_safe = True

    def graph_key(self, ctx) -> tuple:
        return ()                    # positions are read on the device

    @staticmethod
    def check_params(params):
        rotary_dim = int(params["rotary_dim"])
        if rotary_dim % 2 or rotary_dim < 0 or (rotary_dim and not float(params["base"]) > 1):
            raise ValueError("pairwise rotary encoding needs an even rotary_dim and a base above 1")

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.rotary_dim = int(params["rotary_dim"])
        self.freq, self.magnitude = None, 1.0
        if self.rotary_dim:
            freq, self.magnitude = scaled_frequencies(params["base"], self.rotary_dim, params.get("scaling"))
            self.freq = freq.to(torch.float32).to(runtime.device)

    def pairs_record(self):
        """(rotary_dim, frequencies, magnitude): all a kernel needs to apply this encoding itself."""
        return self.rotary_dim, self.freq, self.magnitude

    def encode_and_store(self, ctx, qkv, q_out, kv, nq, nkv, d, v_dim=None):
        self.runtime.ops.rotary_pairs_kv_write(qkv, ctx.positions, ctx.slots, kv.block_table, q_out, kv.k_pages,
                                               kv.v_pages, nq, nkv, d, d if v_dim is None else v_dim, self.rotary_dim,
                                               self.freq, self.magnitude, write_kv=kv.writes,
                                               error_flag=ctx.error_flag)
