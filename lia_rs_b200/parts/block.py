"""Arrangements of a layer's parts.

`sandwich` (a norm before and after each sublayer) and `parallel` are described at their classes.

`prenorm`: r = h + s * mixer(norm1(h)); h' = r + s * ffn(norm2(r))
(src/inference/llama_fusion.rs:41-117; s is MiniCPM's scale_depth / sqrt(layers), 1 for plain
Llama).  Checkpoint names: input_layernorm, self_attn, post_attention_layernorm, mlp
(src/inference/huggingface/minicpm5.rs:31-68); a layer spec may override them."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..weights import TensorSpec
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, Arrangement, DeferredNorm, PartSpec, StateRequest, lookup,
                   register_arrangement)


@dataclass(frozen=True)
class LayerSpec:
    """`norm` is the norm at every place of the arrangement; `norms` names other norms for single places
    (for the pre-norm arrangement the places are "norm1" and "norm2")."""
    mixer: PartSpec
    feed_forward: Optional[PartSpec]     # None: the layer has no feed-forward (an arrangement that allows it)
    norm: PartSpec
    arrangement: str = "prenorm"
    residual_scale: float = 1.0
    norms: dict = field(default_factory=dict, hash=False, compare=False)
    options: dict = field(default_factory=dict, hash=False, compare=False)      # what else the arrangement is told
    names: dict = field(default_factory=lambda: {"norm1": "input_layernorm.", "mixer": "self_attn.",
                                                 "norm2": "post_attention_layernorm.", "feed_forward": "mlp."},
                        hash=False, compare=False)

    def norm_at(self, place: str) -> PartSpec:
        return self.norms.get(place, self.norm)


@register_arrangement("prenorm")
class PreNormBlock(Arrangement):
    supports_rows = True

    @staticmethod
    def _classes(spec: LayerSpec):
        norm1, norm2 = spec.norm_at("norm1"), spec.norm_at("norm2")
        return ((lookup(NORMS, norm1.kind, "norm"), norm1.params), (lookup(MIXERS, spec.mixer.kind, "mixer"), spec.mixer.params),
                (lookup(NORMS, norm2.kind, "norm"), norm2.params),
                (lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward"), spec.feed_forward.params))

    @staticmethod
    def check(spec: LayerSpec) -> None:
        for cls, params in PreNormBlock._classes(spec):
            cls.check_params(params)

    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str) -> list:
        n = spec.names
        places = (n["norm1"], n["mixer"], n["norm2"], n["feed_forward"])
        return [t for (cls, params), place in zip(PreNormBlock._classes(spec), places)
                for t in cls.tensor_specs(params, prefix + place)]

    def __init__(self, spec: LayerSpec, tensors: dict, prefix: str, runtime):
        n = spec.names
        self.runtime = runtime
        self.scale = float(spec.residual_scale)
        places = (n["norm1"], n["mixer"], n["norm2"], n["feed_forward"])
        self.norm1, self.mixer, self.norm2, self.feed_forward = (
            cls(params, tensors, prefix + place, runtime) for (cls, params), place in zip(self._classes(spec), places))
        self.graph_safe = all(part.graph_safe for part in (self.norm1, self.mixer, self.norm2, self.feed_forward))
        if self.mixer.output_bias is not None:
            raise ValueError("the pre-norm arrangement does not add a mixer's output bias")

    def graph_key(self, ctx) -> tuple:
        return (self.norm1.graph_key(ctx) + self.mixer.graph_key(ctx) + self.norm2.graph_key(ctx) +
                self.feed_forward.graph_key(ctx))

    def _normed(self, ctx, norm, part, source):
        """The input of `part`: `norm(source)`, left to the part's first product where the part can take that."""
        deferred = DeferredNorm(ctx, norm, source)
        return deferred if part.takes_deferred_norm else deferred.tensor()

    def forward(self, ctx, residual, kv=None, state=None, rows=None, n_rows=None):
        x = self._normed(ctx, self.norm1, self.mixer, residual)
        if rows is None:
            self.mixer.forward(ctx, x, residual, self.scale, kv=kv, state=state)
            self.feed_forward.forward(ctx, self._normed(ctx, self.norm2, self.feed_forward, residual), residual, self.scale)
            return None
        # Only `rows` matter after this layer (the reference prunes the last layer the same way:
        # src/inference/llama_fusion.rs:45-60): the mixer brings the cache up to date for every token; the output
        # projection, the second norm, the feed-forward and both residual sums run on the picked rows alone.
        picked = ctx.buffer("block.picked", (n_rows, residual.shape[1]), residual.dtype)
        if n_rows and self.mixer.supports_rows:
            self.runtime.ops.gather_rows(residual, rows, picked)
        if self.mixer.supports_rows:
            self.mixer.forward(ctx, x, picked, self.scale, kv=kv, state=state, rows=rows, n_rows=n_rows)
        else:
            self.mixer.forward(ctx, x, residual, self.scale, kv=kv, state=state)
            if n_rows:
                self.runtime.ops.gather_rows(residual, rows, picked)
        if n_rows:
            self.feed_forward.forward(ctx, self._normed(ctx, self.norm2, self.feed_forward, picked), picked, self.scale)
        return picked


@register_arrangement("sandwich")
class SandwichBlock(Arrangement):
    """A norm before and after each sublayer:

        x <- x + post1(mixer(pre1(x)));   x <- x + post2(feed_forward(pre2(x)))

    The sublayer's output goes to a 32-bit buffer of its own (it cannot join the stream before its norm); one kernel
    norms it, adds it to the stream and, when many tokens follow, norms the new stream for the next sublayer in the same
    pass (csrc/norm_residual.cu; with few tokens the next sublayer's first product norms its input itself).  The four
    norms must be RMS norms (`rms_record`).  The feed-forward may be absent (then there is no pre2 and post2).  A mixer's
    `output_bias` is added ahead of post1.  `residual_scale` has no meaning here (a norm follows the sublayer) and must
    be 1.  Checkpoint names: `names["norm1"]`, `["norm1b"]`, `["mixer"]`, `["norm2"]`, `["norm2b"]`, `["feed_forward"]`."""

    PLACES = ("norm1", "norm1b", "norm2", "norm2b")

    @staticmethod
    def _classes(spec: LayerSpec):
        """[(class, params, place)] of the norms that exist, the mixer and the feed-forward."""
        places = SandwichBlock.PLACES if spec.feed_forward is not None else SandwichBlock.PLACES[:2]
        out = [(lookup(NORMS, spec.norm_at(p).kind, "norm"), spec.norm_at(p).params, p) for p in places]
        out.append((lookup(MIXERS, spec.mixer.kind, "mixer"), spec.mixer.params, "mixer"))
        if spec.feed_forward is not None:
            out.append((lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward"), spec.feed_forward.params, "feed_forward"))
        return out

    @staticmethod
    def check(spec: LayerSpec) -> None:
        for cls, params, _ in SandwichBlock._classes(spec):
            cls.check_params(params)
        if float(spec.residual_scale) != 1.0:
            raise ValueError("the sandwich arrangement takes no residual scale")

    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str) -> list:
        specs = [t for cls, params, place in SandwichBlock._classes(spec) for t in cls.tensor_specs(params, prefix + spec.names[place])]
        if spec.feed_forward is None:
            # a checkpoint may carry the norms of the absent sublayer all the same: taken if there, never used
            for place in SandwichBlock.PLACES[2:]:
                norm = spec.norm_at(place)
                specs += [TensorSpec(t.name, t.shape, t.kind, optional=True)
                          for t in lookup(NORMS, norm.kind, "norm").tensor_specs(norm.params, prefix + spec.names[place])]
        return specs

    def __init__(self, spec: LayerSpec, tensors: dict, prefix: str, runtime):
        self.runtime = runtime
        parts = {place: cls(params, tensors, prefix + spec.names[place], runtime) for cls, params, place in self._classes(spec)}
        self.mixer, self.feed_forward = parts["mixer"], parts.get("feed_forward")
        self.pre1, self.pre2 = parts["norm1"], parts.get("norm2")
        self.post = {}
        for place in ("norm1b", "norm2", "norm2b"):
            if place in parts:
                record = parts[place].rms_record()
                if record is None:
                    raise ValueError("the sandwich arrangement needs RMS norms")
                self.post[place] = (record[0].to(torch.float32).contiguous(), float(record[1]))
        self.graph_safe = all(part.graph_safe for part in parts.values())
        self._parts = list(parts.values())

    def graph_key(self, ctx) -> tuple:
        key = ()
        for part in self._parts:
            key += part.graph_key(ctx)
        return key

    def forward(self, ctx, residual, kv=None, state=None):
        ops = self.runtime.ops
        deferred = DeferredNorm(ctx, self.pre1, residual)
        x = deferred if self.mixer.takes_deferred_norm else deferred.tensor()
        y = ctx.buffer("block.sublayer", tuple(residual.shape), torch.float32)
        if self.mixer.can_store:
            self.mixer.forward(ctx, x, y, 1.0, kv=kv, state=state, store=True)
        else:
            y.zero_()
            self.mixer.forward(ctx, x, y, 1.0, kv=kv, state=state)
        weight, eps = self.post["norm1b"]
        if self.feed_forward is None:
            ops.norm_residual(y, weight, residual, eps, bias=self.mixer.output_bias)
            return None
        if self.feed_forward.takes_deferred_norm and residual.shape[0] <= ops.STREAM_MAX_TOKENS:
            ops.norm_residual(y, weight, residual, eps, bias=self.mixer.output_bias)
            x = DeferredNorm(ctx, self.pre2, residual, buffer_name="block.x2")
        else:
            next_weight, next_eps = self.post["norm2"]
            x = ctx.buffer("block.x2", tuple(residual.shape), self.runtime.compute_dtype)
            ops.norm_residual(y, weight, residual, eps, bias=self.mixer.output_bias, next_weight=next_weight, next_out=x,
                              next_eps=next_eps)
        if self.feed_forward.can_store:
            self.feed_forward.forward(ctx, x, y, 1.0, store=True)
        else:
            y.zero_()
            self.feed_forward.forward(ctx, x, y, 1.0)
        weight, eps = self.post["norm2b"]
        ops.norm_residual(y, weight, residual, eps)
        return None


@register_arrangement("parallel")
class ParallelBlock(Arrangement):
    """One norm, both sublayers read its output, one residual sum:

        h = norm(x);   x <- x + s * (mixer(a(h)) + feed_forward(b(h)))

    a and b are the identity, or, with `options["input_conv"] = {"taps": n, "names": (mixer's, feed-forward's)}`,
    a short causal convolution over time on each channel added to its input, y_t = h_t + sum_j c[:, j] h_(t-n+1+j)
    (c [hidden, n], zeros before the sequence's start), with taps of its own for each sublayer.  The last n - 1
    normed rows of a request are the arrangement's state (one tensor for both sublayers: they read the same rows).
    The norm must be an RMSNorm (`rms_record`): norm and convolution are one kernel (csrc/short_conv.cu).  The
    feed-forward may be absent.  Checkpoint names: `names["norm1"]`, `names["mixer"]`, `names["feed_forward"]`."""
    supports_rows = True

    @staticmethod
    def _classes(spec: LayerSpec):
        norm = spec.norm_at("norm1")
        out = [(lookup(NORMS, norm.kind, "norm"), norm.params), (lookup(MIXERS, spec.mixer.kind, "mixer"), spec.mixer.params)]
        if spec.feed_forward is not None:
            out.append((lookup(FEED_FORWARDS, spec.feed_forward.kind, "feed-forward"), spec.feed_forward.params))
        return out

    @staticmethod
    def _conv(spec: LayerSpec):
        conv = spec.options.get("input_conv")
        if not conv:
            return 0, ()
        names = tuple(conv["names"])[:2 if spec.feed_forward is not None else 1]
        return int(conv["taps"]), names

    @staticmethod
    def check(spec: LayerSpec) -> None:
        for cls, params in ParallelBlock._classes(spec):
            cls.check_params(params)
        taps, _ = ParallelBlock._conv(spec)
        if taps and not 1 <= taps <= 8:
            raise ValueError(f"input convolution: {taps} taps; the kernel takes 1..8")

    @staticmethod
    def _hidden(spec: LayerSpec) -> int:
        return int(spec.norm_at("norm1").params["hidden"])

    @staticmethod
    def tensor_specs(spec: LayerSpec, prefix: str) -> list:
        n = spec.names
        places = (n["norm1"], n["mixer"], n["feed_forward"])
        out = [t for (cls, params), place in zip(ParallelBlock._classes(spec), places)
               for t in cls.tensor_specs(params, prefix + place)]
        taps, names = ParallelBlock._conv(spec)
        return out + [TensorSpec(prefix + name, (ParallelBlock._hidden(spec), taps)) for name in names]

    @staticmethod
    def state_request(spec: LayerSpec):
        taps, _ = ParallelBlock._conv(spec)
        return StateRequest((taps - 1, ParallelBlock._hidden(spec)), torch.float32) if taps > 1 else None

    def __init__(self, spec: LayerSpec, tensors: dict, prefix: str, runtime):
        n = spec.names
        self.runtime = runtime
        self.scale = float(spec.residual_scale)
        places = (n["norm1"], n["mixer"], n["feed_forward"])
        parts = [cls(params, tensors, prefix + place, runtime) for (cls, params), place in zip(self._classes(spec), places)]
        self.norm, self.mixer = parts[0], parts[1]
        self.feed_forward = parts[2] if len(parts) > 2 else None
        self.hidden = self._hidden(spec)
        self.taps, names = self._conv(spec)
        self.conv_weights = []
        if self.taps:
            record = self.norm.rms_record()
            if record is None:
                raise ValueError("the parallel arrangement's input convolution needs an RMSNorm")
            self.norm_weight, self.eps = record
            self.conv_weights = [tensors[prefix + name].to(self.norm_weight.dtype).contiguous() for name in names]
        self.graph_safe = all(part.graph_safe for part in parts)
        if self.mixer.output_bias is not None:
            raise ValueError("the parallel arrangement does not add a mixer's output bias")

    def graph_key(self, ctx) -> tuple:
        key = self.norm.graph_key(ctx) + self.mixer.graph_key(ctx)
        return key + (self.feed_forward.graph_key(ctx) if self.feed_forward is not None else ())

    def _inputs(self, ctx, residual, own_state):
        """(the mixer's input, the feed-forward's input) in the compute element type."""
        rt, n = self.runtime, residual.shape[0]
        a = ctx.buffer("block.x", (n, self.hidden), rt.compute_dtype)
        if not self.taps:
            self.norm.forward(ctx, residual, a)
            return a, a
        b = ctx.buffer("block.x2", (n, self.hidden), rt.compute_dtype) if self.feed_forward is not None else None
        single = ctx.decode_only
        tail = None if single or self.taps <= 1 else ctx.buffer("block.conv_tail", (n, self.hidden), torch.float32)
        rt.ops.short_conv(residual, self.norm_weight, self.conv_weights[0],
                          self.conv_weights[1] if b is not None else None, ctx.positions, ctx.slots, own_state, tail,
                          a, b, self.eps, single)
        return a, b

    def forward(self, ctx, residual, kv=None, state=None, rows=None, n_rows=None, own_state=None):
        a, b = self._inputs(ctx, residual, own_state)
        if rows is None:
            self.mixer.forward(ctx, a, residual, self.scale, kv=kv, state=state)
            if self.feed_forward is not None:
                self.feed_forward.forward(ctx, b, residual, self.scale)
            return None
        # only `rows` matter after this layer: cache and state have been brought up to date for every token above and
        # in the mixer; the output projection, the feed-forward and the residual sum run on the picked rows alone
        picked = ctx.buffer("block.picked", (n_rows, residual.shape[1]), residual.dtype)
        if n_rows:
            self.runtime.ops.gather_rows(residual, rows, picked)
        if self.mixer.supports_rows:
            self.mixer.forward(ctx, a, picked, self.scale, kv=kv, state=state, rows=rows, n_rows=n_rows)
        else:
            full = ctx.buffer("block.mixed", tuple(residual.shape), residual.dtype)
            full.zero_()
            self.mixer.forward(ctx, a, full, self.scale, kv=kv, state=state)
            if n_rows:
                mixed = ctx.buffer("block.mixed_rows", (n_rows, residual.shape[1]), residual.dtype)
                self.runtime.ops.gather_rows(full, rows, mixed)
                picked.add_(mixed)
        if n_rows and self.feed_forward is not None:
            b_rows = ctx.buffer("block.x2_rows", (n_rows, self.hidden), self.runtime.compute_dtype)
            self.runtime.ops.gather_rows(b, rows, b_rows)
            self.feed_forward.forward(ctx, b_rows, picked, self.scale)
        return picked


def build_layer(spec: LayerSpec, tensors: dict, prefix: str, runtime):
    return lookup(ARRANGEMENTS, spec.arrangement, "arrangement")(spec, tensors, prefix, runtime)


def check_layer(spec: LayerSpec) -> None:
    """Raise ValueError if a part of the layer refuses its parameters (no device needed)."""
    arrangement = lookup(ARRANGEMENTS, spec.arrangement, "arrangement")
    if hasattr(arrangement, "check"):
        arrangement.check(spec)


def layer_tensor_specs(spec: LayerSpec, prefix: str) -> list:
    return lookup(ARRANGEMENTS, spec.arrangement, "arrangement").tensor_specs(spec, prefix)
