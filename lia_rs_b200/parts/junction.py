"""Junctions: what a model does to the residual stream between two layers.

`reinject`: x <- W [x; x0] + b, with x0 the embedding output of the same tokens, W [hidden, 2 hidden] (x's half
first) and b one row of a table [rows, hidden] chosen when the model is put together (a model that runs a group of
layers several times re-injects ahead of every pass, each pass with its own row).  The two streams are laid side by
side in the product's element type, x is set to b, and the product adds into it: the sum stays 32-bit.
Parameters: hidden, row, rows, names {"weight", "bias"} (checkpoint names; the junction's prefix is empty)."""
from __future__ import annotations

from ..weights import TensorSpec
from .base import Junction, register_junction
from .linear import ACCUM, linear, prepare_weight


@register_junction("reinject")
class Reinject(Junction):
    graph_safe = True
    needs_first = True

    def graph_key(self, ctx) -> tuple:
        return ()

    @staticmethod
    def tensor_specs(params, prefix):
        h = params["hidden"]
        return [TensorSpec(prefix + params["names"]["weight"], (h, 2 * h)),
                TensorSpec(prefix + params["names"]["bias"], (params["rows"], h))]

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden = int(params["hidden"])
        self.weight = prepare_weight(tensors[prefix + params["names"]["weight"]], runtime)
        self.bias = tensors[prefix + params["names"]["bias"]][int(params["row"])].contiguous()

    def forward(self, ctx, residual, first):
        rt, n = self.runtime, residual.shape[0]
        side_by_side = ctx.buffer("junction.in", (n, 2 * self.hidden), rt.compute_dtype)
        rt.ops.reinject_input(residual, first, self.bias, side_by_side)
        linear(rt, ACCUM, side_by_side, self.weight, residual, 1.0, error_flag=ctx.error_flag, name="reinject")
