"""Each mechanism of the Vatunex decoder alone, as its kernel, against the plain functions (tests/plain_vatunex.py): the
norm that joins a sublayer's output to the stream; the activation between a dense feed-forward's products; softmax
attention with two-part keys, values of their own size, a window and a sink, where ONE key decides (far back among
hundreds, at a page border, just inside and just outside the window, in prompt rows and for chosen rows); the
tensor-core kernel for attention in a latent's space against the kernel for every size, whole and cut into ranges; the
preparation of q, k, v (bias, per-head norm, rotation, value mixing, append) and of latents; the short convolution and
the selective scan with their state carried over steps of unequal runs on reused slots; products of many heads at once."""
import math

import numpy as np
import pytest
import torch

import plain_vatunex as pv

pytestmark = pytest.mark.gpu
F64 = torch.float64


def dev(t, dtype=None):
    return t.to("cuda", dtype=dtype) if dtype else t.to("cuda")


def ints(values):
    return torch.tensor(list(values), dtype=torch.int32, device="cuda")


class Pages:
    """A paged cache for the tests: `slots` requests, each with its pages in a shuffled order of the pool."""

    def __init__(self, slots, max_tokens, page_size, seed=0):
        self.page_size = page_size
        self.blocks = (max_tokens + page_size - 1) // page_size
        self.num_pages = slots * self.blocks + 3
        order = torch.randperm(self.num_pages, generator=torch.Generator().manual_seed(seed))[:slots * self.blocks]
        self.table = order.view(slots, self.blocks).to(torch.int32).cuda().contiguous()

    def empty(self, heads, dim, dtype):
        return torch.zeros((self.num_pages, self.page_size, heads, dim), dtype=dtype, device="cuda")

    def fill(self, pages, slot, values):
        """values [T, heads, dim] at positions 0..T-1 of `slot`."""
        for pos in range(values.shape[0]):
            page = int(self.table[slot, pos // self.page_size])
            pages[page, pos % self.page_size] = values[pos].to(pages.dtype)


def test_norm_residual_and_next_norm():
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(1)
    for rows, hidden, with_bias, dtype in [(5, 96, True, torch.bfloat16), (37, 257, False, torch.float32), (3, 2048, True, torch.float32)]:
        y, x = torch.randn(rows, hidden, generator=g), torch.randn(rows, hidden, generator=g) * 3
        w1, w2 = torch.randn(hidden, generator=g), torch.randn(hidden, generator=g)
        bias = torch.randn(hidden, generator=g) if with_bias else None
        want_x = x.to(F64) + pv.norm_plain(y.to(F64) + (bias.to(F64) if with_bias else 0.0), w1, 1e-5)
        want_next = pv.norm_plain(want_x, w2, 2e-6)
        residual, out = dev(x), torch.empty(rows, hidden, dtype=dtype, device="cuda")
        ops.norm_residual(dev(y), dev(w1), residual, 1e-5, bias=dev(bias) if with_bias else None, next_weight=dev(w2),
                          next_out=out, next_eps=2e-6)
        assert torch.allclose(residual.cpu().to(F64), want_x, atol=2e-5, rtol=1e-5)
        tolerance = 1e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(out.float().cpu().to(F64), want_next, atol=tolerance, rtol=tolerance)
        residual = dev(x)
        ops.norm_residual(dev(y), dev(w1), residual, 1e-5, bias=dev(bias) if with_bias else None)
        assert torch.allclose(residual.cpu().to(F64), want_x, atol=2e-5, rtol=1e-5)


def test_activation_rows():
    from lia_rs_b200.kernels import ops
    x = torch.randn(19, 70, generator=torch.Generator().manual_seed(2)) * 3
    wide = dev(x)
    for act, plain in [(ops.ACT_GELU_TANH, pv.gelu_tanh), (ops.ACT_SILU, lambda z: z * torch.sigmoid(z)), (ops.ACT_NONE, lambda z: z)]:
        out = torch.empty(19, 33, dtype=torch.float32, device="cuda")
        ops.activation_rows(wide[:, 5:38], out, act)                   # a view: columns of wider rows
        assert torch.allclose(out.cpu().to(F64), plain(x[:, 5:38].to(F64)), atol=2e-6, rtol=2e-6)
        half = torch.empty(19, 33, dtype=torch.bfloat16, device="cuda")
        ops.activation_rows(wide[:, 5:38], half, act)
        assert torch.allclose(half.float().cpu().to(F64), plain(x[:, 5:38].to(F64)), atol=3e-2, rtol=1e-2)


def _one_key_case(T, H, G, d, dv, decisive, seed):
    """q, k, v [T, ., .] where for every query position i the key at i - decisive(i) (if >= 0) has by far the largest
    score: k there points along q_i... built the other way round: every key j gets a direction of its own and query i
    points along the direction of its decisive key."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(T, G, d, generator=g, dtype=F64)
    k = k / k.norm(dim=-1, keepdim=True)
    q = 0.3 * torch.randn(T, H, d, generator=g, dtype=F64)
    for i in range(T):
        j = i - decisive(i)
        if j >= 0:
            for h in range(H):
                q[i, h] += 9.0 * k[j, h // (H // G)]
    v = torch.randn(T, G, dv, generator=g, dtype=F64)
    return q, k, v


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_general_where_one_key_decides(dtype):
    """A window of 37 on pages of 8: the decisive key lies far back (outside: it must not count), at the window's first
    key (just inside), one before it (just outside), at page borders, at the query itself; with and without a sink, heads
    in groups, values smaller than keys."""
    from lia_rs_b200.kernels import ops
    T, H, G, d, dv, page = 300, 4, 2, 24, 8, 8
    cache = Pages(2, T, page, seed=3)
    for window, sink in [(37, True), (None, True), (37, False), (None, False)]:
        offsets = [0, 1, 7, 8, 9, 36, 37, 38, 100, 250]            # 36: the window's first key; 37: just outside
        q, k, v = _one_key_case(T, H, G, d, dv, lambda i: offsets[i % len(offsets)], seed=5)
        round_trip = (lambda t: t.to(dtype).to(F64))
        q, k, v = round_trip(q), round_trip(k), round_trip(v)
        want = pv.softmax_attention(q, k, v, 1.0, window=window, sink=sink)
        k_pages, v_pages = cache.empty(G, d, dtype), cache.empty(G, dv, dtype)
        cache.fill(k_pages, 1, k)
        cache.fill(v_pages, 1, v)
        positions, slots = ints(range(T)), ints([1] * T)
        out = torch.zeros(T, H * dv, dtype=dtype, device="cuda")
        qd = dev(q.reshape(T, H * d), dtype)
        ops.attention_general(qd, (H * d, d), None, None, k_pages, None, v_pages, dv, dv, positions, slots, cache.table, out,
                              (H * dv, dv), T, H, G, window, 1.0, sink=sink)
        tolerance = 2e-5 if dtype == torch.float32 else 2e-2
        got = out.float().cpu().to(F64).view(T, H, dv)
        assert torch.allclose(got, want, atol=tolerance, rtol=tolerance), (window, sink, float((got - want).abs().max()))
        # chosen rows only, in another order; the others stay as they were
        out.zero_()
        rows = [250, 37, 299, 8]
        ops.attention_general(qd, (H * d, d), None, None, k_pages, None, v_pages, dv, dv, positions, slots, cache.table, out,
                              (H * dv, dv), T, H, G, window, 1.0, sink=sink, rows=ints(rows))
        got = out.float().cpu().to(F64).view(T, H, dv)
        assert torch.allclose(got[rows], want[rows], atol=tolerance, rtol=tolerance)
        assert float(got[[0, 100, 251]].abs().max()) == 0.0


@pytest.mark.parametrize("heads,rank,dr,window", [(4, 64, 16, 45), (16, 128, 32, None), (3, 32, 16, 33), (20, 96, 64, 70)])
def test_latent_attention_kernel_against_the_kernel_for_every_size(heads, rank, dr, window):
    """bfloat16: the tensor-core kernel, whole and cut into 2, 3 and 7 ranges, against `attention_general` on the same
    pages; two requests in one call (a prompt portion in the middle of a request and single tokens), one decisive key per
    query at the window's edges; then against the plain softmax over the two-part keys."""
    from lia_rs_b200.kernels import ops
    dtype, page = torch.bfloat16, 16
    T = 200
    cache = Pages(3, T, page, seed=11)
    offsets = [0, 1, 15, 16, 17, (window or 150) - 1, window or 151, 120]
    q, k, _ = _one_key_case(T, heads, 1, rank + dr, 8, lambda i: offsets[i % len(offsets)], seed=13)
    q, k = q.to(dtype), k.to(dtype)
    latent_pages, part_pages = cache.empty(1, rank, dtype), cache.empty(1, dr, dtype)
    for slot in (0, 2):
        cache.fill(latent_pages, slot, k[:, :, :rank])
        cache.fill(part_pages, slot, k[:, :, rank:])
    # slot 0: positions 60..179 as a portion; slot 2: single tokens at 0, 5, 199
    where = list(range(60, 180)) + [0, 5, 199]
    slots = [0] * 120 + [2, 2, 2]
    n = len(where)
    q_here = q[where]                                                    # [n, heads, rank + dr]
    q1 = dev(q_here[:, :, :rank].transpose(0, 1).contiguous())           # [heads, n, rank]
    q2 = dev(q_here[:, :, rank:].reshape(n, heads * dr).contiguous())
    positions, slot_ids = ints(where), ints(slots)
    reference = torch.zeros(heads, n, rank, dtype=dtype, device="cuda")
    ops.attention_general(q1, (rank, n * rank), q2, (heads * dr, dr), latent_pages, part_pages, latent_pages, rank, rank,
                          positions, slot_ids, cache.table, reference, (rank, n * rank), n, heads, 1, window, 0.7)
    want = pv.softmax_attention(q.to(F64), k.to(F64), k.to(F64)[:, :, :rank], 0.7, window=window)[where]     # [n, heads, rank]
    assert torch.allclose(reference.float().cpu().to(F64).transpose(0, 1), want, atol=2e-2, rtol=2e-2)
    for splits in (1, 2, 3, 7):
        out = torch.zeros(heads, n, rank, dtype=dtype, device="cuda")
        partial = torch.empty(splits * heads * n * (rank + 2), dtype=torch.float32, device="cuda") if splits > 1 else None
        ops.latent_attention(q1, q2, latent_pages, part_pages, positions, slot_ids, cache.table, out, heads, window, 0.7,
                             splits=splits, partial=partial)
        got = out.float().cpu().to(F64).transpose(0, 1)
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2), (splits, float((got - want).abs().max()))


def test_qkv_prepare_against_plain_functions():
    from lia_rs_b200.kernels import ops
    from lia_rs_b200.parts.rotary import band_scaled_frequencies
    g = torch.Generator().manual_seed(21)
    n, H, G, d, dv, page, dims = 23, 6, 2, 40, 24, 4, 16
    cache = Pages(2, 64, page, seed=4)
    rows = torch.randn(n, (H + G) * d + G * dv + 4, generator=g)                 # wider than needed: a padded product
    bias = torch.randn((H + G) * d + G * dv, generator=g)
    qn, kn = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    scaling = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 16}
    freq = band_scaled_frequencies(300.0, dims, scaling)
    where = list(range(7, 7 + n - 3)) + [0, 50, 33]
    slots = [0] * (n - 3) + [1, 1, -1]                                           # the last row belongs to nobody
    positions = torch.tensor(where)
    x = rows[:, :bias.numel()].to(F64) + bias.to(F64)
    q = pv.rotate_half(pv.norm_plain(x[:, :H * d].view(n, H, d), qn, 1e-5), positions, pv.rotary_frequencies(300.0, dims, scaling), dims)
    k = pv.rotate_half(pv.norm_plain(x[:, H * d:(H + G) * d].view(n, G, d), kn, 1e-5), positions,
                       pv.rotary_frequencies(300.0, dims, scaling), dims)
    v = x[:, (H + G) * d:].view(n, G, dv)
    first = torch.randn(n, G * dv, generator=g)
    for mode, lam in [(0, 0.0), (1, 0.0), (2, 0.35)]:
        k_pages, v_pages = cache.empty(G, d, torch.float32), cache.empty(G, dv, torch.float32)
        q_out = torch.zeros(n, H * d, device="cuda")
        v_first = dev(first.clone())
        ops.qkv_prepare(dev(rows), dev(bias), dev(qn), dev(kn), 1e-5, dev(freq, torch.float32), dims, mode, lam, v_first,
                        ints(where), ints(slots), cache.table, q_out, k_pages, v_pages, H, G, d, dv)
        want_v = v if mode < 2 else (1 - lam) * v + lam * first.to(F64).view(n, G, dv)
        for r in range(n - 1):
            page_id = int(cache.table[slots[r], where[r] // page])
            assert torch.allclose(q_out[r].cpu().to(F64), q[r].reshape(-1), atol=2e-5, rtol=2e-5)
            assert torch.allclose(k_pages[page_id, where[r] % page].cpu().to(F64), k[r], atol=2e-5, rtol=2e-5)
            assert torch.allclose(v_pages[page_id, where[r] % page].cpu().to(F64), want_v[r], atol=2e-5, rtol=2e-5)
        if mode == 1:
            assert torch.allclose(v_first[:n - 1].cpu().to(F64), v[:n - 1].reshape(n - 1, -1), atol=1e-6)
        assert float(q_out[n - 1].abs().max()) == 0.0                            # nobody's row: nothing written


def test_latent_prepare_against_plain_functions():
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(22)
    n, H, d, dr, rank, page = 11, 3, 12, 8, 20, 4
    cache = Pages(1, 64, page, seed=6)
    q_rows, shared = torch.randn(n, H * (d + dr), generator=g), torch.randn(n, rank + dr, generator=g)
    weight = 1 + 0.3 * torch.randn(rank, generator=g)
    freqs = pv.rotary_frequencies(50.0, dr)
    where = list(range(30, 30 + n))
    positions = torch.tensor(where)
    q_plain = torch.zeros(H, n, d, device="cuda")
    q_rot = torch.zeros(n, H * dr, device="cuda")
    latent_pages, part_pages = cache.empty(1, rank, torch.float32), cache.empty(1, dr, torch.float32)
    ops.latent_prepare(dev(q_rows), dev(shared), dev(weight), 3e-6, dev(freqs, torch.float32), dr, ints(where), ints([0] * n),
                       cache.table, q_plain, q_rot, latent_pages, part_pages, H, d, dr, rank)
    q = q_rows.to(F64).view(n, H, d + dr)
    assert torch.allclose(q_plain.cpu().to(F64).transpose(0, 1), q[:, :, :d], atol=1e-6)
    assert torch.allclose(q_rot.cpu().to(F64).view(n, H, dr), pv.rotate_half(q[:, :, d:], positions, freqs, dr), atol=2e-5, rtol=2e-5)
    latent = pv.norm_plain(shared.to(F64)[:, :rank], weight, 3e-6)
    part = pv.rotate_half(shared.to(F64)[:, None, rank:], positions, freqs, dr)[:, 0]
    for r in range(n):
        page_id = int(cache.table[0, where[r] // page])
        assert torch.allclose(latent_pages[page_id, where[r] % page, 0].cpu().to(F64), latent[r], atol=2e-5, rtol=2e-5)
        assert torch.allclose(part_pages[page_id, where[r] % page, 0].cpu().to(F64), part[r], atol=2e-5, rtol=2e-5)


def _runs(plan):
    """positions, slots and the device lists of a step from [(slot, start, count)]."""
    positions, slots, segments, singles, at = [], [], [], [], 0
    for slot, start, count in plan:
        positions += list(range(start, start + count))
        slots += [slot] * count
        if count > 1:
            segments += [at, start, count]
        else:
            singles.append(at)
        at += count
    return ints(positions), ints(slots), ints(segments) if segments else ints([0, 0, 0])[:0], len(segments) // 3, ints(singles)


@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_causal_conv_carries_its_inputs_over_steps(taps):
    """Three requests on two slots (the second slot is used again from zeroed state), runs of 1 to 9 tokens, shorter and
    longer than the taps, in steps that mix them; every request equals the convolution of its whole sequence."""
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(30 + taps)
    channels, wide = 70, 150
    weight, bias = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    xs = {r: torch.randn(length, wide, generator=g) for r, length in (("a", 30), ("b", 12), ("c", 17))}
    want = {}
    for r, x in xs.items():
        y = pv.causal_conv(x[:, :channels].to(F64), weight, bias)
        want[r] = y * torch.sigmoid(y)
    state = torch.zeros(2, max(taps - 1, 1), channels, device="cuda")[:, :taps - 1]
    slot_of, at, got = {"a": 0, "b": 1}, {"a": 0, "b": 0, "c": 0}, {r: [] for r in xs}
    steps = [[("a", 3), ("b", 1)], [("b", 2), ("a", 1)], [("a", 9), ("b", 9)], [("a", 1)], [("a", 2), ("c", 1)], [("c", 5), ("a", 7)],
             [("c", 1), ("a", 1)], [("a", 6), ("c", 10)]]
    for step in steps:
        if any(r == "c" for r, _ in step) and "c" not in slot_of:
            slot_of["c"] = 1                                           # b is done: its slot again, zeroed as at admission
            if taps > 1:
                state[1].zero_()
        plan = [(slot_of[r], at[r], count) for r, count in step]
        positions, slots, _, _, _ = _runs(plan)
        x = torch.cat([xs[r][at[r]:at[r] + count] for r, count in step])
        n = x.shape[0]
        out, copy = torch.empty(n, channels, device="cuda"), torch.empty(n, channels, dtype=torch.bfloat16, device="cuda")
        xd = dev(x)
        single = all(count == 1 for _, count in step)                  # then the convolution leaves the new state itself
        ops.causal_conv(xd, dev(weight), dev(bias), state if taps > 1 else None, positions, slots, out, copy, act=1,
                        update_single=single)
        if taps > 1 and not single:
            ops.conv_state_update(xd, state, positions, slots, channels)
        row = 0
        for r, count in step:
            got[r].append(out[row:row + count].cpu())
            assert torch.allclose(copy[row:row + count].float().cpu(), got[r][-1], atol=2e-2, rtol=1e-2)
            row += count
            at[r] += count
    for r in ("a", "c"):
        rows = torch.cat(got[r]).to(F64)
        assert torch.allclose(rows, want[r][:rows.shape[0]], atol=2e-5, rtol=2e-5), (r, taps)


@pytest.mark.parametrize("chunked", [False, True])
@pytest.mark.parametrize("states", [3, 8, 16, 24, 40])
def test_selective_scan_carries_its_state_over_steps(states, chunked):
    """Runs of 1 to 150 tokens of three requests on two slots; `chunked`: the portions are cut into chunks of 64 tokens
    that run side by side (one, two and three chunks a portion, beside single tokens), with the same results."""
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(40 + states)
    channels, rank = 50, 3
    A = -(0.2 + 3 * torch.rand(channels, states, generator=g))
    D, dt_bias = torch.randn(channels, generator=g), torch.randn(channels, generator=g) - 1
    seqs = {}
    for r, length in (("a", 230), ("b", 9), ("c", 133)):
        x, dt_raw, z = (torch.randn(length, channels, generator=g) for _ in range(3))
        bc = torch.randn(length, rank + 2 * states + 2, generator=g)
        dt = torch.nn.functional.softplus(dt_raw.to(F64) + dt_bias.to(F64))
        y = pv.selective_scan(x.to(F64), dt, A.to(F64), bc[:, rank:rank + states].to(F64), bc[:, rank + states:rank + 2 * states].to(F64), D.to(F64))
        seqs[r] = dict(x=x, dt=dt_raw, z=z, bc=bc, want=y * (z.to(F64) * torch.sigmoid(z.to(F64))))
    state = torch.zeros(2, channels * states + 5, device="cuda")[:, 5:].view(2, channels, states)     # a view: a slot's stride is its own
    slot_of, at, got = {"a": 0, "b": 1}, {r: 0 for r in seqs}, {r: [] for r in seqs}
    steps = [[("a", 4), ("b", 1)], [("b", 8), ("a", 1)], [("a", 1)], [("c", 2), ("a", 150)], [("a", 1), ("c", 1)], [("c", 130), ("a", 73)]]
    for step in steps:
        if any(r == "c" for r, _ in step) and "c" not in slot_of:
            slot_of["c"] = 1
            state[1].zero_()
        plan = [(slot_of[r], at[r], count) for r, count in step]
        _, slots, segments, n_segments, singles = _runs(plan)
        cat = lambda key: dev(torch.cat([seqs[r][key][at[r]:at[r] + count] for r, count in step]))
        x, dt, z, bc = cat("x"), cat("dt"), cat("z"), cat("bc")
        wide_z = torch.cat([torch.zeros_like(z), z], dim=1)                   # z as the second half of wider rows
        out = torch.empty(x.shape[0], channels, device="cuda")
        scratch = None
        if chunked and n_segments:
            scratch = torch.full((ops.selective_scan_chunk_floats(x.shape[0], n_segments, channels, states),), float("nan"), device="cuda")
        ops.selective_scan(x, dt, dev(dt_bias), dev(A), bc, rank, rank + states, dev(D), wide_z[:, channels:], state, segments,
                           n_segments, singles, slots, out, chunk_scratch=scratch)
        row = 0
        for r, count in step:
            got[r].append(out[row:row + count].cpu())
            row += count
            at[r] += count
    for r in ("a", "c"):
        rows = torch.cat(got[r]).to(F64)
        assert torch.allclose(rows, seqs[r]["want"][:rows.shape[0]], atol=1e-4, rtol=1e-4), (r, states, chunked)


def test_products_of_many_heads_at_once():
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(50)
    B, M, N, K = 5, 37, 24, 19
    a, w = torch.randn(B, M, K, generator=g), torch.randn(B, N, K, generator=g)
    want = torch.einsum("bmk,bnk->bmn", a.to(F64), w.to(F64))
    out = torch.zeros(M, B * N, device="cuda")
    ops.gemm_simt_batched(ops.GEMM_STORE, dev(a), dev(w), out.view(M, B, N).transpose(0, 1))      # heads side by side in a row
    assert torch.allclose(out.cpu().to(F64).view(M, B, N).transpose(0, 1), want, atol=1e-5, rtol=1e-5)
    half = torch.zeros(B, M, N, dtype=torch.bfloat16, device="cuda")
    ops.gemm_simt_batched(ops.GEMM_STORE, dev(a, torch.bfloat16), dev(w, torch.bfloat16), half)
    assert torch.allclose(half.float().cpu().to(F64), want, atol=0.15, rtol=3e-2)


@pytest.mark.parametrize("B,M,N,K", [(3, 37, 24, 40), (16, 300, 128, 64), (2, 129, 66, 8), (5, 1, 512, 128)])
def test_products_of_many_heads_on_the_tensor_cores(B, M, N, K):
    """Sizes that are no multiples of the kernel's tiles, K shorter than and not a multiple of a step, outputs side by
    side in a row and as planes."""
    from lia_rs_b200.kernels import ops
    g = torch.Generator().manual_seed(51)
    a, w = torch.randn(B, M, K, generator=g).to(torch.bfloat16), torch.randn(B, N, K, generator=g).to(torch.bfloat16)
    want = torch.einsum("bmk,bnk->bmn", a.to(F64), w.to(F64))
    planes = torch.zeros(B, M, N, dtype=torch.bfloat16, device="cuda")
    assert ops.gemm_mma_batched_accepts(dev(a), dev(w), planes)
    ops.gemm_mma_batched(dev(a), dev(w), planes)
    assert torch.allclose(planes.float().cpu().to(F64), want, atol=0.02 * K ** 0.5, rtol=1e-2)
    side_by_side = torch.zeros(M, B * N, dtype=torch.bfloat16, device="cuda")
    ops.gemm_mma_batched(dev(a), dev(w), side_by_side.view(M, B, N).transpose(0, 1))
    assert torch.equal(side_by_side.view(M, B, N).transpose(0, 1), planes)
    assert not ops.gemm_mma_batched_accepts(dev(a)[:, :, :K - 1], dev(w)[:, :, :K - 1], planes)      # K no multiple of 8


@pytest.mark.parametrize("M", [1, 8, 16])
def test_activation_in_the_few_token_products_epilogue(M):
    """The persistent few-token product with GELU or SiLU in its epilogue against the activation of the plain product,
    with and without the norm of its input rows inside the kernel; `linear` hands the product to 32-bit rows where
    another kernel serves it (more tokens) and says so."""
    from lia_rs_b200.kernels import ops
    from lia_rs_b200.parts import Runtime
    from lia_rs_b200.parts.linear import STORE, linear
    g = torch.Generator().manual_seed(60 + M)
    N, K = 328, 256
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16)
    product = a.to(F64) @ w.to(F64).T
    for act, plain in [(ops.ACT_GELU_TANH, pv.gelu_tanh), (ops.ACT_SILU, lambda z: z * torch.sigmoid(z))]:
        out = torch.zeros(M, N, dtype=torch.bfloat16, device="cuda")
        assert ops.gemm_stream_accepts(ops.GEMM_STORE, dev(a), dev(w), out)
        ops.gemm_stream(ops.GEMM_STORE, dev(a), dev(w), out, 0.5, activation=act)
        assert torch.allclose(out.float().cpu().to(F64), plain(0.5 * product), atol=2e-2, rtol=1e-2)
        rows = torch.randn(M, K, generator=g) * 2
        weight = 1 + 0.2 * torch.randn(K, generator=g)
        normed = pv.norm_plain(rows.to(F64), weight, 1e-5).to(torch.bfloat16).to(F64)
        ops.gemm_stream(ops.GEMM_STORE, dev(rows), dev(w), out, 1.0, norm_weight=dev(weight), eps=1e-5, activation=act)
        assert torch.allclose(out.float().cpu().to(F64), plain(normed @ w.to(F64).T), atol=3e-2, rtol=2e-2)
    runtime = Runtime("cuda:0", torch.bfloat16)
    for tokens, applied in [(M, True), (200, False)]:
        a = torch.randn(tokens, K, generator=g).to(torch.bfloat16)
        out = torch.zeros(tokens, N, dtype=torch.bfloat16, device="cuda")
        wide = torch.zeros(tokens, N, dtype=torch.float32, device="cuda")
        assert bool(linear(runtime, STORE, dev(a), dev(w), out, activation=ops.ACT_GELU_TANH, unactivated=wide)) == applied
        want = a.to(F64) @ w.to(F64).T
        if applied:
            assert torch.allclose(out.float().cpu().to(F64), pv.gelu_tanh(want), atol=2e-2, rtol=1e-2)
        else:
            assert torch.allclose(wide.cpu().to(F64), want, atol=1e-3, rtol=1e-3) and float(out.abs().max()) == 0.0
