"""A recurrent mixer with input-dependent decay (a selective state-space scan).

    [u | z] = W_in x                                   (`inner` channels each)
    u <- silu(conv(u)):  conv(u)_t[c] = b[c] + sum_j w[c, j] u_(t - taps + 1 + j)[c], zeros before the sequence's start
    [r | B | C] = W_x u                                (`dt_rank`, `state`, `state` elements)
    dt = softplus(W_dt r + b_dt)                       (one step size per channel);   A = -exp(A_log)  [inner, state]
    S_t[c, n] = exp(dt[c] A[c, n]) S_(t-1)[c, n] + dt[c] u[c] B[n],   S_(-1) = 0
    y[c] = sum_n S_t[c, n] C[n] + D[c] u[c];   out = W_o (y * silu(z))

What a request carries from token to token is one 32-bit state per slot: the convolution's last taps - 1 inputs and
S.  The products may run in the compute element type; the convolution and its activation, step sizes, decays,
exponentials, the state and the sums over it are 32-bit (csrc/selective_scan.cu).  A step's runs (prompt portions and
single tokens) are walked token by token on the device, so a portion cut anywhere continues from the slot's state.  In a
step of many tokens the portions are cut into chunks of 64 tokens that run side by side: the recurrence is linear in the
state, so a chunk's end state is its end state from zero plus the decayed state it started from.

Parameters: hidden, inner, state, dt_rank, taps, and optionally `names` (checkpoint names behind the part's prefix)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import Mixer, StateRequest, register_mixer
from .linear import ACCUM, STORE, linear, prepare_weight


@register_mixer("selective_scan")
class SelectiveScan(Mixer):
    graph_safe = True
    takes_deferred_norm = True
    can_store = True
    CHUNKED_FROM = 256        # tokens of a step from which its portions are cut into chunks that run side by side
    NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "x": "x", "dt": "dt", "dt_bias": "dt.b", "A_log": "A_log",
             "D": "D", "o": "o"}

    def graph_key(self, ctx) -> tuple:
        return ()

    @staticmethod
    def _names(params, prefix):
        return {key: prefix + name for key, name in {**SelectiveScan.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        inner, states, rank, taps = (int(params[k]) for k in ("inner", "state", "dt_rank", "taps"))
        if inner <= 0 or rank <= 0:
            raise ValueError("selective scan: inner and dt_rank must be positive")
        if not 1 <= taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"selective scan: {taps} taps; the kernel takes 1..{ops.CONV_MAX_TAPS}")
        if not 1 <= states <= ops.SCAN_MAX_STATES:
            raise ValueError(f"selective scan: {states} states; the kernel takes 1..{ops.SCAN_MAX_STATES}")

    @staticmethod
    def tensor_specs(params, prefix):
        h, inner, states, rank, taps = (int(params[k]) for k in ("hidden", "inner", "state", "dt_rank", "taps"))
        n = SelectiveScan._names(params, prefix)
        return [TensorSpec(n["in"], (2 * inner, h)), TensorSpec(n["conv"], (inner, taps)), TensorSpec(n["conv_bias"], (inner,)),
                TensorSpec(n["x"], (rank + 2 * states, inner)), TensorSpec(n["dt"], (inner, rank)),
                TensorSpec(n["dt_bias"], (inner,)), TensorSpec(n["A_log"], (inner, states)), TensorSpec(n["D"], (inner,)),
                TensorSpec(n["o"], (h, inner))]

    @staticmethod
    def state_request(params):
        inner, states, taps = int(params["inner"]), int(params["state"]), int(params["taps"])
        return StateRequest(((taps - 1) * inner + inner * states,), torch.float32)

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.check_params(params)
        self.hidden, self.inner = int(params["hidden"]), int(params["inner"])
        self.states, self.rank, self.taps = int(params["state"]), int(params["dt_rank"]), int(params["taps"])
        n = self._names(params, prefix)
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.w_in = prepare_weight(tensors[n["in"]], runtime)
        self.w_x = prepare_weight(tensors[n["x"]], runtime)
        self.w_dt = prepare_weight(tensors[n["dt"]], runtime)
        self.w_o = prepare_weight(tensors[n["o"]], runtime)
        self.conv, self.conv_bias = f32(tensors[n["conv"]]), f32(tensors[n["conv_bias"]])
        self.dt_bias, self.skip = f32(tensors[n["dt_bias"]]), f32(tensors[n["D"]])
        self.decay = (-torch.exp(tensors[n["A_log"]].to(torch.float32))).contiguous()

    def forward(self, ctx, x, residual, scale, kv=None, state=None, store=False):
        rt, n = self.runtime, x.shape[0]
        inner, states, rank, taps = self.inner, self.states, self.rank, self.taps
        flag, dtype = ctx.error_flag, rt.compute_dtype
        slots = state.shape[0]
        split = (taps - 1) * inner
        conv_state = state[:, :split].view(slots, taps - 1, inner) if taps > 1 else None
        scan_state = state[:, split:].view(slots, inner, states)
        uz = ctx.buffer("scan.in", (n, 2 * inner), torch.float32)
        linear(rt, STORE, x, self.w_in, uz, error_flag=flag, name="in")
        u = ctx.buffer("scan.u", (n, inner), torch.float32)
        u_rounded = ctx.buffer("scan.u_rounded", (n, inner), dtype) if dtype != torch.float32 else None
        single = ctx.decode_only                  # single tokens only: the convolution leaves its new state itself
        ops.causal_conv(uz, self.conv, self.conv_bias, conv_state, ctx.positions, ctx.slots, u, u_rounded, act=1,
                        update_single=single)
        if taps > 1 and not single:
            ops.conv_state_update(uz, conv_state, ctx.positions, ctx.slots, inner)
        projected = ctx.buffer("scan.x", (n, rank + 2 * states), torch.float32)
        linear(rt, STORE, u if u_rounded is None else u_rounded, self.w_x, projected, error_flag=flag, name="x")
        low = ctx.buffer("scan.dt_in", (n, rank), dtype)
        ops.activation_rows(projected[:, :rank], low, ops.ACT_NONE)
        dt_raw = ctx.buffer("scan.dt", (n, inner), torch.float32)
        linear(rt, STORE, low, self.w_dt, dt_raw, error_flag=flag, name="dt")
        y = ctx.buffer("scan.y", (n, inner), dtype)
        chunk_scratch = None
        if ctx.n_prefill_segments and n >= self.CHUNKED_FROM:
            words = ops.selective_scan_chunk_floats(n, ctx.n_prefill_segments, inner, states)
            chunk_scratch = ctx.runtime.scratch("scan.chunks", words, torch.float32)
        ops.selective_scan(u, dt_raw, self.dt_bias, self.decay, projected, rank, rank + states, self.skip, uz[:, inner:],
                           scan_state, ctx.prefill_segments, ctx.n_prefill_segments, ctx.decode_rows, ctx.slots, y,
                           chunk_scratch=chunk_scratch)
        linear(rt, STORE if store else ACCUM, y, self.w_o, residual, scale, error_flag=flag, name="o")
