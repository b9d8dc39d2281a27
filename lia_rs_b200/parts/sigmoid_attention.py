"""Grouped-query attention without a softmax, over the paged cache, with a gate on each head's output.

    q = Wq x, k = Wk x, v = Wv x, g = Wg x (one logit per query head); no biases
    position encoding of q and k, append of k and v to the pages
    weight of a visible key j for head h:  sigmoid(scale * (q_h . k_j) + bias_h)        (not normalised over keys)
    head h's output:  sigmoid(g_h) * sum_j weight_j v_j;  the heads side by side through Wo into the residual stream

A token sees the keys j <= its position p that lie in the last `window` positions (if a window is set) and in p's own
block of `chunk` positions, floor(j / chunk) == floor(p / chunk) (if a chunk is set; blocks are counted from position
0 of the sequence, however the prompt was cut into steps).  Keys have head size `head_dim`, values `v_head_dim`.
Scores, weights and the sums over keys are 32-bit; so are the gate and its sigmoid.

The four projections are one product against [Wq; Wk; Wv; Wg] (zero rows bring the row count to a multiple of
8) whose 32-bit rows the encoding kernel and the attention kernel read in place.

Parameters: hidden, heads, kv_heads, head_dim, v_head_dim, scale, window, chunk, position (a PartSpec), and
`names` (checkpoint names of q, k, v, o, gate and bias behind the part's prefix).

`PagedSigmoidAttention` chooses the kernels: bfloat16 with head sizes that the tensor-core kernel takes (multiples of
8 up to 128) goes to csrc/sigmoid_attention_tc.cu (prompt portions and single tokens alike);
everything else, and the whole 32-bit path, to the kernel for every size (csrc/sigmoid_attention.cu).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import KVCacheRequest, Mixer, POSITION_ENCODINGS, lookup, register_mixer
from .linear import ACCUM, STORE, linear, prepare_weight


class PagedSigmoidAttention:
    """Sigmoid-weighted attention of a step's tokens over a paged cache: which kernel serves which rows."""

    @staticmethod
    def check(heads: int, kv_heads: int, head_dim: int, v_head_dim: int) -> None:
        if heads <= 0 or kv_heads <= 0 or heads % kv_heads:
            raise ValueError("attention: heads must be a positive multiple of kv_heads")
        for name, size in (("head_dim", head_dim), ("v_head_dim", v_head_dim)):
            if size <= 0 or size > ops.ATTENTION_HEAD_DIM_MAX:
                raise ValueError(f"attention: {name} {size} is not within 1..{ops.ATTENTION_HEAD_DIM_MAX} "
                                 f"(what the attention kernels take)")

    def __init__(self, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, v_head_dim: int, window, chunk,
                 scale: float, head_bias=None):
        self.check(heads, kv_heads, head_dim, v_head_dim)
        self.nq, self.nkv, self.d, self.dv = int(heads), int(kv_heads), int(head_dim), int(v_head_dim)
        self.window, self.chunk, self.scale = window, chunk, float(scale)
        self.head_bias = head_bias
        self.group = self.nq // self.nkv
        self.per_tile = ops.sigmoid_attention_tc_tokens_per_tile(self.group, self.d, self.dv) if dtype == torch.bfloat16 else 0
        self.variant = "tensor" if self.per_tile else "generic"

    def graph_key(self, ctx) -> tuple:
        """What of a step's shape the launches depend on beyond the numbers of tokens, single-token entries and
        portions: into how many tiles the tensor-core kernel cuts the portions (where they begin and how long each is,
        the kernel reads on the device)."""
        if self.variant != "tensor" or not ctx.n_prefill_segments:
            return ()
        return (self.per_tile, ops.sigmoid_attention_tc_tiles(ctx.segments, self.per_tile))

    def single_splits(self, ctx, rows: int) -> dict:
        """Into how many ranges the tensor-core kernel cuts the key tiles of each single token (and their scratch): as
        many as give every SM a CTA, no more than a token can have tiles at the step's context bucket, its window and
        its block, at most 8.  It depends on the number of rows and the context bucket alone, as a captured step needs."""
        longest = min(ctx.context_bucket, self.window or ctx.context_bucket, self.chunk or ctx.context_bucket)
        splits = max(1, min(ctx.runtime.sm_count // max(1, rows * self.nkv), 8, (longest + 127) // 128))
        if splits == 1:
            return {}
        words = splits * ctx.n_tokens * self.nq * self.dv
        return dict(splits=splits, partial=ctx.runtime.scratch("sattn.partial", words, torch.float32))

    def visible(self, position: int) -> int:
        first = 0
        if self.window:
            first = max(first, position - self.window + 1)
        if self.chunk:
            first = max(first, position // self.chunk * self.chunk)
        return position + 1 - first

    def _work(self, ctx, element_size: int):
        """(cache bytes the single-token rows read, flops of the prompt portions), for the profile only."""
        if ops._profiler is None:
            return 0, 0
        keys = sum(self.visible(start) for _, start, count, _ in ctx.segments if count == 1)
        pairs = sum(self.visible(start + i) for _, start, count, _ in ctx.segments if count > 1 for i in range(count))
        return keys * self.nkv * (self.d + self.dv) * element_size, 2 * self.nq * (self.d + self.dv) * pairs

    def forward_fused(self, ctx, projected, kv, out, pairs, gate=None, gate_stride=0) -> bool:
        """For a step of single decoded tokens, the tensor-core variant and a pairwise rotary (or no) encoding
        (`pairs`: what the encoding answers to `pairs_record()`): encoding of q and k, append of k and v to `kv`, and
        attention in one kernel, from the product's 32-bit rows `projected`.  Returns False, having done nothing, when
        the step or this attention is not of that kind; the caller then encodes and attends separately."""
        if self.variant != "tensor" or pairs is None or not ctx.decode_only or kv.k_pages.dtype != torch.bfloat16:
            return False
        rotary_dim, freq, magnitude = pairs
        work_bytes, _ = self._work(ctx, 2)
        ops.sigmoid_attention_tc(None, kv.k_pages, kv.v_pages, None, 0, 0, ctx.decode_rows, ctx.positions, ctx.slots,
                                 kv.block_table, out, self.nq, self.nkv, self.d, self.dv, self.window, self.chunk, self.scale,
                                 self.head_bias, gate, gate_stride, error_flag=ctx.error_flag, label="fused",
                                 work_bytes=work_bytes, fused_rows=projected, freq=freq, rotary_dim=rotary_dim,
                                 magnitude=magnitude, write_kv=kv.writes, **self.single_splits(ctx, ctx.n_tokens))
        return True

    def forward(self, ctx, q, kv, out, gate=None, gate_stride=0, rows=None, n_rows=None):
        """out[t] = gated attention of token t's encoded queries over `kv` (this step's keys and values already
        appended), for every token of the step or for the batch indices in the device tensor `rows`."""
        if rows is not None and n_rows == 0:
            return
        work_bytes, work_flops = self._work(ctx, q.element_size())
        if self.variant == "tensor" and rows is not None:
            # a few wanted rows (the last tokens of portions, in a model's last layer): each as a single token
            ops.sigmoid_attention_tc(q, kv.k_pages, kv.v_pages, None, 0, 0, rows[:n_rows], ctx.positions, ctx.slots,
                                     kv.block_table, out, self.nq, self.nkv, self.d, self.dv, self.window, self.chunk,
                                     self.scale, self.head_bias, gate, gate_stride, error_flag=ctx.error_flag, label="rows",
                                     **self.single_splits(ctx, n_rows))
            return
        if self.variant == "tensor":
            tiles = ops.sigmoid_attention_tc_tiles(ctx.segments, self.per_tile) if ctx.n_prefill_segments else 0
            ops.sigmoid_attention_tc(q, kv.k_pages, kv.v_pages, ctx.prefill_segments, ctx.n_prefill_segments, tiles,
                                     ctx.decode_rows, ctx.positions, ctx.slots, kv.block_table, out, self.nq, self.nkv,
                                     self.d, self.dv, self.window, self.chunk, self.scale, self.head_bias, gate, gate_stride,
                                     error_flag=ctx.error_flag, work_bytes=work_bytes, work_flops=work_flops,
                                     **(self.single_splits(ctx, ctx.n_single) if not ctx.n_prefill_segments else {}))
            return
        ops.sigmoid_attention_generic(q, kv.k_pages, kv.v_pages, ctx.positions, ctx.slots, kv.block_table, out, self.nq,
                                      self.nkv, self.d, self.dv, self.window, self.chunk, self.scale, self.head_bias,
                                      gate, gate_stride, rows=None if rows is None else rows[:n_rows],
                                      error_flag=ctx.error_flag, work_bytes=work_bytes)


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    graph_safe = True
    supports_rows = True
    NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "bias": "pb"}

    @staticmethod
    def _names(params, prefix):
        return {key: prefix + name for key, name in {**SigmoidAttention.NAMES, **params.get("names", {})}.items()}

    @staticmethod
    def check_params(params):
        PagedSigmoidAttention.check(int(params["heads"]), int(params["kv_heads"]), int(params["head_dim"]),
                                    int(params["v_head_dim"]))
        position = params["position"]
        lookup(POSITION_ENCODINGS, position.kind, "position encoding").check_params(position.params)
        for key in ("window", "chunk"):
            if params.get(key) is not None and int(params[key]) <= 0:
                raise ValueError(f"attention: {key} must be positive or None")

    @staticmethod
    def tensor_specs(params, prefix):
        h, nq, nkv = params["hidden"], params["heads"], params["kv_heads"]
        d, dv = params["head_dim"], params["v_head_dim"]
        n = SigmoidAttention._names(params, prefix)
        return [TensorSpec(n["q"], (nq * d, h)), TensorSpec(n["k"], (nkv * d, h)), TensorSpec(n["v"], (nkv * dv, h)),
                TensorSpec(n["bias"], (nq,)), TensorSpec(n["gate"], (nq, h)), TensorSpec(n["o"], (h, nq * dv))]

    @staticmethod
    def cache_request(params):
        return KVCacheRequest(params["kv_heads"], params["head_dim"], params.get("window"),
                              v_head_dim=params["v_head_dim"], chunk=params.get("chunk"))

    def __init__(self, params, tensors, prefix, runtime):
        super().__init__(params, tensors, prefix, runtime)
        self.hidden = int(params["hidden"])
        self.nq, self.nkv = int(params["heads"]), int(params["kv_heads"])
        self.d, self.dv = int(params["head_dim"]), int(params["v_head_dim"])
        n = self._names(params, prefix)
        parts = [tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["gate"]]]
        self.gate_offset = (self.nq + self.nkv) * self.d + self.nkv * self.dv
        used = self.gate_offset + self.nq
        self.width = (used + 7) // 8 * 8
        if self.width > used:
            parts.append(torch.zeros((self.width - used, self.hidden), dtype=parts[0].dtype, device=parts[0].device))
        self.w_in = prepare_weight(torch.cat(parts, dim=0), runtime)
        self.w_o = prepare_weight(tensors[n["o"]], runtime)
        position = params["position"]
        self.position = lookup(POSITION_ENCODINGS, position.kind, "position encoding")(
            position.params, tensors, prefix, runtime)
        self.graph_safe = bool(self.position.graph_safe)
        self.attention = PagedSigmoidAttention(runtime.compute_dtype, self.nq, self.nkv, self.d, self.dv,
                                               params.get("window"), params.get("chunk"), float(params["scale"]),
                                               head_bias=tensors[n["bias"]].to(torch.float32).contiguous())

    def graph_key(self, ctx) -> tuple:
        return self.position.graph_key(ctx) + self.attention.graph_key(ctx)

    def forward(self, ctx, x, residual, scale, kv=None, state=None, rows=None, n_rows=None):
        """`rows` (device int32, `n_rows` of them): only these tokens' outputs are needed; `residual` then holds those
        rows alone ([n_rows, hidden]); keys and values of every token are still appended."""
        rt, n = self.runtime, x.shape[0]
        nq, nkv, d, dv = self.nq, self.nkv, self.d, self.dv
        flag = ctx.error_flag
        projected = ctx.buffer("sattn.in", (n, self.width), torch.float32)
        linear(rt, STORE, x, self.w_in, projected, error_flag=flag, name="qkvg")
        o = ctx.buffer("sattn.o", (n, nq * dv), rt.compute_dtype)
        gate = projected[:, self.gate_offset:]
        if rows is None and self.attention.forward_fused(ctx, projected, kv, o, self.position.pairs_record(), gate=gate,
                                                         gate_stride=self.width):
            linear(rt, ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
            return
        q = ctx.buffer("sattn.q", (n, nq * d), rt.compute_dtype)
        self.position.encode_and_store(ctx, projected, q, kv, nq, nkv, d, v_dim=dv)
        if rows is None:
            self.attention.forward(ctx, q, kv, o, gate=gate, gate_stride=self.width)
            linear(rt, ACCUM, o, self.w_o, residual, scale, error_flag=flag, name="o")
            return
        if n_rows == 0:
            return
        self.attention.forward(ctx, q, kv, o, gate=gate, gate_stride=self.width, rows=rows, n_rows=n_rows)
        picked = ctx.buffer("sattn.o_rows", (n_rows, nq * dv), rt.compute_dtype)
        rt.ops.gather_rows(o, rows, picked)
        linear(rt, ACCUM, picked, self.w_o, residual, scale, error_flag=flag, name="o")
