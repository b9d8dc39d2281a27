"""Each new mechanism alone, its kernel against the plain implementation's function (tests/plain_nafevik.py): learned
positions, the re-injection's input, the norm with its short convolution and carried state, the pairwise rotary
encoding with scaled frequencies, and the sigmoid attention over a paged cache, with inputs made so that ONE key
decides the output: far back, at page borders, just inside and just outside a block or a window, in prompt portions
and in single decoded tokens."""
import math

import numpy as np
import pytest
import torch

import plain_nafevik as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from lia_rs_b200.kernels import ops as module
    module.lib()
    return module


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=DEV)


def close(actual, reference, dtype, what):
    actual, reference = actual.double().cpu(), reference.double()
    scale = max(1.0, float(reference.abs().max()))
    limit = (2e-5 if dtype == torch.float32 else 1.2e-2) * scale
    worst = float((actual - reference).abs().max())
    assert worst <= limit, f"{what}: {worst:.3e} > {limit:.3e}"


def test_embedding_with_learned_positions_and_reinjection_input():
    o = ops()
    g = torch.Generator().manual_seed(0)
    vocab, width, most = 53, 40, 31
    table = torch.randn(vocab, width, generator=g).to(torch.bfloat16)
    where = torch.randn(most, width, generator=g).to(torch.bfloat16)
    tokens, positions = [5, 52, 0, 17, 17], [0, 30, 7, 8, 3]
    out = torch.empty(5, width, dtype=torch.float32, device=DEV)
    copy = torch.empty_like(out)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.embedding_positions(i32(tokens), i32(positions), table.to(DEV), where.to(DEV), out, 1.0, copy=copy, error_flag=flag)
    want = table.double()[tokens] + where.double()[positions]
    assert torch.equal(out.cpu().double(), want) and torch.equal(copy, out) and int(flag.item()) == 0
    o.embedding_positions(i32([1]), i32([most]), table.to(DEV), where.to(DEV), out[:1], 1.0, error_flag=flag)
    assert int(flag.item()) == 1                                   # a position beyond the table is refused, not read
    for dtype in DTYPES:
        x = torch.randn(5, width, generator=g).to(DEV)
        first = torch.randn(5, width, generator=g).to(DEV)
        bias = torch.randn(width, generator=g).to(torch.bfloat16).to(DEV)
        both = torch.empty(5, 2 * width, dtype=dtype, device=DEV)
        before = x.clone()
        o.reinject_input(x, first, bias, both)
        assert torch.equal(both, torch.cat([before, first], dim=1).to(dtype))
        assert torch.equal(x, bias.float().expand(5, width))


@pytest.mark.parametrize("width", [72, 70])           # 16-byte accesses, four channels a thread; and a width that does not allow them
@pytest.mark.parametrize("taps", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("dtype", DTYPES)
def test_norm_and_short_convolution_with_carried_state(taps, dtype, width):
    """Three requests in three slots; their sequences come in steps of unequal runs (a run shorter than the taps, a
    run of one, single-token steps that move the state in the same kernel, rows of nobody).  Every output row equals
    the plain convolution of the whole sequence."""
    o = ops()
    g = torch.Generator().manual_seed(taps)
    eps, slots = 1e-5, 4
    norm_w = (1 + 0.3 * torch.randn(width, generator=g)).to(torch.bfloat16)
    c = [(0.7 * torch.randn(width, taps, generator=g)).to(torch.bfloat16) for _ in range(2)]
    lengths = {0: 23, 2: 9, 3: 14}
    x = {s: torch.randn(n, width, generator=g) * (1 + s) for s, n in lengths.items()}
    want = {}
    for s in lengths:
        h = plain.rms_norm(x[s].double(), norm_w, eps)
        want[s] = [plain.input_conv(h, c[0]), plain.input_conv(h, c[1])]
    state = torch.full((slots, max(taps - 1, 1), width), 7.0, device=DEV)[:, :taps - 1].contiguous()   # junk: zeroing is not relied on
    at = {s: 0 for s in lengths}
    got = {s: [[], []] for s in lengths}
    steps = [[(0, 1), (2, 2)], [(2, 1), (0, 1), (3, 1)], [(3, 1), (0, 1)], [(0, 5), (3, 2), (2, 1)], [(2, 1), (0, 1), (3, 1)],
             [(0, 14), (2, 4), (3, 9)]]
    for step in steps:
        rows, positions, slot_ids = [], [], []
        for s, count in step:
            rows.append(x[s][at[s]:at[s] + count])
            positions += range(at[s], at[s] + count)
            slot_ids += [s] * count
        single = all(count == 1 for _, count in step)
        if single:                                                   # rows of nobody behind a step of single tokens
            rows.append(torch.randn(2, width, generator=g))
            positions += [0, 0]
            slot_ids += [-1, -1]
        batch = torch.cat(rows).to(DEV)
        n = batch.shape[0]
        out = [torch.empty(n, width, dtype=dtype, device=DEV) for _ in range(2)]
        tail = torch.empty(n, width, device=DEV)
        o.short_conv(batch, norm_w.to(DEV), c[0].to(DEV), c[1].to(DEV), i32(positions), i32(slot_ids), state if taps > 1 else None,
                     tail, out[0], out[1], eps, single)
        row = 0
        for s, count in step:
            for r in range(2):
                got[s][r].append(out[r][row:row + count])
            at[s] += count
            row += count
    for s in lengths:
        assert at[s] == lengths[s]
        for r in range(2):
            close(torch.cat(got[s][r]), want[s][r], dtype, f"taps {taps} slot {s} reader {r}")
    # one reader alone (a layer without a feed-forward)
    batch = x[0][:6].to(DEV)
    alone = torch.empty(6, width, dtype=dtype, device=DEV)
    o.short_conv(batch, norm_w.to(DEV), c[1].to(DEV), None, i32(range(6)), i32([1] * 6), state if taps > 1 else None,
                 torch.empty(6, width, device=DEV), alone, None, eps, False)
    close(alone, want[0][1][:6], dtype, "one reader")
    # a long portion (eight rows a CTA, a token takes its earlier rows from the token ahead) behind a short one
    g = torch.Generator().manual_seed(99)
    long_x = torch.randn(1500, width, generator=g)
    h = plain.rms_norm(long_x.double(), norm_w, eps)
    want_long = [plain.input_conv(h, c[0]), plain.input_conv(h, c[1])]
    got_long = [[], []]
    at_long = 0
    for count in (3, 1200, 1, 296):
        batch = torch.cat([long_x[at_long:at_long + count], x[2][:5]]).to(DEV)          # another request's rows behind it
        n = batch.shape[0]
        out = [torch.empty(n, width, dtype=dtype, device=DEV) for _ in range(2)]
        o.short_conv(batch, norm_w.to(DEV), c[0].to(DEV), c[1].to(DEV), i32(list(range(at_long, at_long + count)) + list(range(5))),
                     i32([0] * count + [2] * 5), state if taps > 1 else None, torch.empty(n, width, device=DEV), out[0], out[1], eps, False)
        for r in range(2):
            got_long[r].append(out[r][:count])
            close(out[r][count:], want[2][r][:5], dtype, f"the rows behind the long portion, reader {r}")
        at_long += count
    for r in range(2):
        close(torch.cat(got_long[r]), want_long[r], dtype, f"long portions, reader {r}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,dv,dims,scaling", [(16, 16, 16, None), (56, 24, 32, {"factor": 3.0, "original": 40, "fast": 8.0, "slow": 1.0}),
                                               (64, 128, 0, None), (40, 8, 40, {"factor": 16.0, "original": 16, "fast": 4.0, "slow": 2.0})])
def test_pairwise_rotary_encoding_and_append(d, dv, dims, scaling, dtype):
    from lia_rs_b200.parts.rotary import scaled_frequencies
    o = ops()
    g = torch.Generator().manual_seed(d)
    nq, nkv, page, pages = 3, 2, 4, 9
    base = 300.0
    if dims:
        freq, magnitude = scaled_frequencies(base, dims, scaling)
        want_freq, want_magnitude = plain.rotary_frequencies(base, dims, scaling)
        assert torch.allclose(freq, want_freq, rtol=1e-14, atol=0) and abs(magnitude - want_magnitude) < 1e-15
        if scaling:
            assert not torch.allclose(freq, plain.rotary_frequencies(base, dims)[0])      # the scaling does something
    else:
        freq, magnitude = None, 1.0
    positions = [0, 1, 2, 33, 34, 5]
    slot_ids = [0, 0, 0, 1, 1, -1]
    n = len(positions)
    stride = (nq + nkv) * d + nkv * dv + 5                         # the rows hold more than q, k and v
    rows = torch.randn(n, stride, generator=g)
    table = torch.full((2, 12), -1, dtype=torch.int32)
    table[0, 0], table[1, 8] = 7, 2
    k_pages = torch.zeros(pages, page, nkv, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros(pages, page, nkv, dv, dtype=dtype, device=DEV)
    q_out = torch.zeros(n, nq * d, dtype=dtype, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    o.rotary_pairs_kv_write(rows.to(DEV), i32(positions), i32(slot_ids), table.to(DEV), q_out, k_pages, v_pages, nq, nkv, d, dv,
                            dims, None if freq is None else freq.float().to(DEV), magnitude, error_flag=flag)
    assert int(flag.item()) == 0
    q = rows[:, :nq * d].double().view(n, nq, d)
    k = rows[:, nq * d:(nq + nkv) * d].double().view(n, nkv, d)
    v = rows[:, (nq + nkv) * d:(nq + nkv) * d + nkv * dv].double().view(n, nkv, dv)
    if dims:
        where = torch.tensor(positions)
        q, k = plain.rotate_pairs(q, where, want_freq, want_magnitude, dims), plain.rotate_pairs(k, where, want_freq, want_magnitude, dims)
    close(q_out[:5].view(5, nq, d), q[:5], dtype, "q")
    for t, (p, s) in enumerate(zip(positions[:5], slot_ids[:5])):
        page_of = int(table[s, p // page])
        close(k_pages[page_of, p % page], k[t], dtype, f"k of token {t}")
        close(v_pages[page_of, p % page], v[t], dtype, f"v of token {t}")
    assert float(q_out[5].abs().max()) == 0.0                     # a row of nobody is skipped
    untouched = torch.ones(pages, dtype=torch.bool)
    untouched[[7, 2]] = False
    assert float(k_pages[untouched].abs().max()) == 0.0 and float(v_pages[untouched].abs().max()) == 0.0


def _paged(keys, values, page, pages, order, dtype):
    """Keys [T, G, d] and values [T, G, dv] of one request laid into pages in the given order of page numbers."""
    T = keys.shape[0]
    k_pages = torch.zeros(pages, page, keys.shape[1], keys.shape[2], dtype=dtype, device=DEV)
    v_pages = torch.zeros(pages, page, values.shape[1], values.shape[2], dtype=dtype, device=DEV)
    table = torch.full((1, (T + page - 1) // page + 2), -1, dtype=torch.int32)
    for block in range((T + page - 1) // page):
        table[0, block] = order[block]
        rows = slice(block * page, min(T, (block + 1) * page))
        k_pages[order[block], :rows.stop - rows.start] = keys[rows].to(dtype)
        v_pages[order[block], :rows.stop - rows.start] = values[rows].to(dtype)
    return k_pages, v_pages, table.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,chunk,window,page", [(4, 2, 16, 16, 24, None, 8), (3, 1, 56, 24, 50, None, 16), (2, 2, 64, 64, None, 37, 4),
                                                        (6, 2, 32, 40, 128, 100, 16), (8, 1, 128, 128, 64, None, 16), (1, 1, 8, 200, None, None, 4)])
def test_sigmoid_attention_one_key_decides(H, G, d, dv, chunk, window, page, dtype):
    """The heads' biases push every weight to nothing (sigmoid(-14)); one key per probe is made to score +14 against
    the probing query, so the output is that key's value if the key is visible and nothing if it is not.  Probes:
    the token itself, its predecessor, a far key, the first key of the token's block and the key before it, the
    oldest key of the window and the one before it, the keys on both sides of a page border.  Then random inputs
    against the plain function, for a prompt portion and for the same tokens one by one."""
    o = ops()
    g = torch.Generator().manual_seed(H * 100 + d)
    T, scale = 300, 0.5
    bias = torch.full((H,), -14.0)
    gate = torch.randn(T, H, generator=g)
    values = torch.randn(T, G, dv, generator=g)
    pages = (T + page - 1) // page + 3
    order = torch.randperm(pages, generator=g).tolist()
    probes = []
    for p in (0, 1, 129, 255, 299):
        first = 0
        if chunk:
            first = max(first, p // chunk * chunk)
        if window:
            first = max(first, p - window + 1)
        border = p // page * page
        for j in {p, p - 1, first, first - 1, first + 1, border, border - 1, p - 100, 0}:
            if 0 <= j <= p:
                probes.append((p, j, plain.visible(p, j, chunk, window)))
    if chunk or window:
        assert any(not seen for _, _, seen in probes)
    else:
        assert any(seen and p - j >= 100 for p, j, seen in probes)          # nothing hides a key hundreds back
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    for p, j, seen in probes:
        keys = torch.randn(T, G, d, generator=g) * 0.05
        query = torch.randn(H, d, generator=g)
        query = query / query.norm(dim=-1, keepdim=True)
        for kvh in range(G):                                         # the kv head's key j points along its first query head
            keys[j, kvh] = query[kvh * (H // G)] * (28.0 / scale)
        for h in range(H):
            query[h] = query[h // (H // G) * (H // G)]
        k_pages, v_pages, table = _paged(keys, values, page, pages, order, dtype)
        q = query.view(1, H * d).to(dtype).to(DEV)
        out = torch.empty(1, H * dv, dtype=dtype, device=DEV)
        o.sigmoid_attention_generic(q, k_pages, v_pages, i32([p]), i32([0]), table, out, H, G, d, dv, window, chunk, scale,
                                    bias.to(DEV), gate[p:p + 1].contiguous().to(DEV), H, error_flag=flag)
        got = out.view(H, dv).float().cpu()
        for h in range(H):
            want = values[j, h // (H // G)] * torch.sigmoid(gate[p, h]) if seen else torch.zeros(dv)
            assert float((got[h] - want).abs().max()) <= 0.03 * max(1.0, float(want.abs().max())), (p, j, seen, h)
    # random inputs, moderate scores: a prompt portion of all tokens, then single tokens, against the plain function
    keys = torch.randn(T, G, d, generator=g)
    query = torch.randn(T, H, d, generator=g)
    bias = torch.rand(H, generator=g) * 3 - 2.5
    scale = 1.0 / math.sqrt(d)
    store = plain.exact if dtype == torch.float32 else plain.to_bf16
    want = plain.sigmoid_attention(store(query.double()), store(keys.double()), store(values.double()), scale, bias, gate.double(),
                                   chunk=chunk, window=window)
    k_pages, v_pages, table = _paged(keys, values, page, pages, order, dtype)
    q = query.view(T, H * d).to(dtype).to(DEV)
    out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
    wide = torch.cat([torch.randn(T, 3, generator=g), gate], dim=1).contiguous().to(DEV)      # gate logits inside wider rows
    o.sigmoid_attention_generic(q, k_pages, v_pages, i32(range(T)), i32([0] * T), table, out, H, G, d, dv, window, chunk, scale,
                                bias.to(DEV), wide[:, 3:], H + 3, error_flag=flag)
    close(out.view(T, H, dv), want, dtype, "portion")
    picked = [0, 1, chunk or 7, (chunk or 7) - 1, 130, 299]
    one = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
    o.sigmoid_attention_generic(q, k_pages, v_pages, i32(range(T)), i32([0] * T), table, one, H, G, d, dv, window, chunk, scale,
                                bias.to(DEV), wide[:, 3:], H + 3, rows=i32(picked), error_flag=flag)
    assert torch.equal(one[picked], out[picked]) and float(one[2].abs().max()) == 0.0
    assert int(flag.item()) == 0


@pytest.mark.parametrize("H,G,d,dv,chunk,window,page", [(4, 1, 64, 64, 40, None, 16), (2, 2, 64, 64, None, 37, 4), (8, 1, 128, 128, 64, None, 16),
                                                        (16, 2, 128, 128, 130, 100, 8), (1, 1, 64, 64, None, None, 16), (4, 4, 128, 128, 300, None, 32),
                                                        (4, 2, 40, 40, 50, None, 8), (8, 2, 96, 24, 110, None, 16), (2, 1, 16, 112, None, 60, 4),
                                                        (4, 1, 72, 8, 33, None, 16), (3, 1, 32, 16, 7, None, 4), (10, 2, 64, 64, 90, None, 16),
                                                        (7, 7, 56, 56, None, None, 8)])
def test_sigmoid_attention_on_the_tensor_cores(H, G, d, dv, chunk, window, page):
    """The tcgen05 kernel (bfloat16, head sizes that are multiples of 8 up to 128, keys' and values' apart) against the plain function and against the kernel for every
    size: one portion of all tokens; two portions beside single tokens and a row of nobody; and the one-key probes
    at block, window and page edges as single decoded tokens."""
    o = ops()
    dtype = torch.bfloat16
    assert o.sigmoid_attention_tc_accepts(H // G, d, dv) and not o.sigmoid_attention_tc_accepts(H // G, d + 4, dv)
    assert not o.sigmoid_attention_tc_accepts(H // G, 136, dv)
    per_tile = o.sigmoid_attention_tc_tokens_per_tile(H // G, d, dv)
    g = torch.Generator().manual_seed(H * 10 + d)
    T = 300
    keys, values = torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    query = torch.randn(T, H, d, generator=g)
    gate = torch.randn(T, H, generator=g)
    bias = torch.rand(H, generator=g) * 3 - 2.5
    scale = 1.0 / math.sqrt(d)
    want = plain.sigmoid_attention(plain.to_bf16(query.double()), plain.to_bf16(keys.double()), plain.to_bf16(values.double()), scale,
                                   bias, gate.double(), chunk=chunk, window=window)
    pages = (T + page - 1) // page + 3
    order = torch.randperm(pages, generator=g).tolist()
    k_pages, v_pages, table = _paged(keys, values, page, pages, order, dtype)
    q = query.view(T, H * d).to(dtype).to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions, slots = i32(range(T)), i32([0] * T)
    gate_dev = gate.contiguous().to(DEV)

    def run(portions, singles, slot_ids=slots):
        out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
        segments = i32([x for first, count in portions for x in (first, first, count)]).view(-1, 3) if portions else None
        tiles = sum((count + per_tile - 1) // per_tile for _, count in portions)
        o.sigmoid_attention_tc(q, k_pages, v_pages, segments, len(portions), tiles, i32(singles) if singles else None, positions,
                               slot_ids, table, out, H, G, d, dv, window, chunk, scale, bias.to(DEV), gate_dev, H, error_flag=flag)
        return out

    whole = run([(0, T)], [])
    close(whole.view(T, H, dv), want, dtype, "one portion")
    generic = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
    o.sigmoid_attention_generic(q, k_pages, v_pages, positions, slots, table, generic, H, G, d, dv, window, chunk, scale, bias.to(DEV),
                                gate_dev, H, error_flag=flag)
    close(whole, generic.double().cpu(), dtype, "against the kernel for every size")
    nobody = slots.clone()
    nobody[7] = -1
    mixed = run([(10, 140), (150, 149)], [0, 5, 9, 299, 7], nobody)
    rows = [0, 5, 9] + list(range(10, 300))
    close(mixed[rows].view(len(rows), H, dv), want[rows], dtype, "portions beside single tokens")
    assert float(mixed[7].abs().max()) == 0.0 and float(mixed[6].abs().max()) == 0.0       # nobody's row and an absent row
    one_by_one = run([], list(range(0, T, 7)))
    close(one_by_one[::7].view(-1, H, dv), want[::7], dtype, "single tokens")
    # the same single tokens with their key tiles cut into ranges that a second kernel adds (more ranges than some have tiles)
    for splits in (2, 3, 5):
        cut = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
        o.sigmoid_attention_tc(q, k_pages, v_pages, None, 0, 0, i32(list(range(0, T, 7)) + [6]), positions, nobody.roll(-1), table, cut, H, G, d, dv,
                               window, chunk, scale, bias.to(DEV), gate_dev, H, error_flag=flag, splits=splits,
                               partial=torch.full((splits * T * H * dv,), float("nan"), device=DEV))
        close(cut[::7].view(-1, H, dv), want[::7], dtype, f"single tokens in {splits} ranges")
    # one key decides
    low = torch.full((H,), -14.0)
    for p in (1, 129, 255, 299):
        first = max(p // chunk * chunk if chunk else 0, p - window + 1 if window else 0)
        border = p // page * page
        for j in sorted({p, p - 1, first, first - 1, border, border - 1, p - 100, 0}):
            if not 0 <= j <= p:
                continue
            seen = plain.visible(p, j, chunk, window)
            probe_keys = torch.randn(T, G, d, generator=g) * 0.05
            probe = torch.randn(G, d, generator=g)
            probe = probe / probe.norm(dim=-1, keepdim=True)
            probe_keys[j] = probe * (28.0 / scale)
            kp, vp, _ = _paged(probe_keys, values, page, pages, order, dtype)
            qq = torch.zeros(T, H, d)
            qq[p] = probe.repeat_interleave(H // G, dim=0)
            out = torch.zeros(T, H * dv, dtype=dtype, device=DEV)
            o.sigmoid_attention_tc(qq.view(T, H * d).to(dtype).to(DEV), kp, vp, None, 0, 0, i32([p]), positions, slots, table, out, H, G,
                                   d, dv, window, chunk, scale, low.to(DEV), gate_dev, H, error_flag=flag)
            got = out[p].view(H, dv).float().cpu()
            for h in range(H):
                expect = values[j, h // (H // G)] * torch.sigmoid(gate[p, h]) if seen else torch.zeros(dv)
                assert float((got[h] - expect).abs().max()) <= 0.03 * max(1.0, float(expect.abs().max())), (p, j, seen, h)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0


@pytest.mark.parametrize("H,G,d,dv,dims,chunk,page", [(4, 2, 64, 64, 64, 40, 16), (8, 1, 128, 128, 32, None, 8), (4, 1, 56, 24, 56, 100, 16),
                                                      (3, 3, 16, 40, 0, 7, 4)])
def test_single_tokens_encoded_and_appended_inside_the_attention_kernel(H, G, d, dv, dims, chunk, page):
    """A step of single tokens through the one kernel that encodes q and k, appends k and v and attends, against the
    encoding kernel followed by the attention kernel: the same outputs and the same pages (to 16-bit rounding: the two
    may contract their multiplications differently), the other pages untouched, a row of nobody skipped."""
    from lia_rs_b200.parts.rotary import scaled_frequencies
    o = ops()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(d + dv)
    contexts = [0, 1, 39, 40, 130, 255, 77]                        # each token's position: its request holds that many keys
    slot_ids = [0, 1, 2, 3, 4, 5, -1]
    n, slots = len(contexts), 6
    blocks = 256 // page + 1
    pages = slots * blocks + 2
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((slots, blocks), -1, dtype=torch.int32)
    k_pages = torch.zeros(pages, page, G, d)
    v_pages = torch.zeros(pages, page, G, dv)
    for s in range(slots):
        for b in range(contexts[s] // page + 1):
            table[s, b] = order[s * blocks + b]
            held = min(page, contexts[s] - b * page)               # keys of earlier steps in this page
            if held > 0:
                k_pages[table[s, b], :held] = torch.randn(held, G, d, generator=g)
                v_pages[table[s, b], :held] = torch.randn(held, G, dv, generator=g)
    width = ((H + G) * d + G * dv + H + 7) // 8 * 8
    rows = torch.randn(n, width, generator=g).to(DEV)
    gate_offset = (H + G) * d + G * dv
    freq, magnitude = (scaled_frequencies(700.0, dims, {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}) if dims else (None, 1.0))
    freq = None if freq is None else freq.float().to(DEV)
    bias = (torch.rand(H, generator=g) * 2 - 2).to(DEV)
    positions, slot_dev, table = i32(contexts), i32(slot_ids), table.to(DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    singles = i32(range(n))
    # apart: the encoding kernel, then the attention kernel
    ka, va = k_pages.to(dtype).to(DEV), v_pages.to(dtype).to(DEV)
    q = torch.zeros(n, H * d, dtype=dtype, device=DEV)
    o.rotary_pairs_kv_write(rows, positions, slot_dev, table, q, ka, va, H, G, d, dv, dims, freq, magnitude, error_flag=flag)
    apart = torch.zeros(n, H * dv, dtype=dtype, device=DEV)
    o.sigmoid_attention_tc(q, ka, va, None, 0, 0, singles, positions, slot_dev, table, apart, H, G, d, dv, None, chunk, scale, bias,
                           rows[:, gate_offset:], width, error_flag=flag)
    # together
    kb, vb = k_pages.to(dtype).to(DEV), v_pages.to(dtype).to(DEV)
    together = torch.zeros(n, H * dv, dtype=dtype, device=DEV)
    o.sigmoid_attention_tc(None, kb, vb, None, 0, 0, singles, positions, slot_dev, table, together, H, G, d, dv, None, chunk, scale, bias,
                           rows[:, gate_offset:], width, error_flag=flag, fused_rows=rows, freq=freq, rotary_dim=dims, magnitude=magnitude)
    # and with every token's tiles cut into ranges: the range that holds the token's own key appends it
    kc, vc = k_pages.to(dtype).to(DEV), v_pages.to(dtype).to(DEV)
    ranged = torch.zeros(n, H * dv, dtype=dtype, device=DEV)
    o.sigmoid_attention_tc(None, kc, vc, None, 0, 0, singles, positions, slot_dev, table, ranged, H, G, d, dv, None, chunk, scale, bias,
                           rows[:, gate_offset:], width, error_flag=flag, fused_rows=rows, freq=freq, rotary_dim=dims, magnitude=magnitude,
                           splits=3, partial=torch.full((3 * n * H * dv,), float("nan"), device=DEV))
    close(ranged, apart.double().cpu(), dtype, "outputs in ranges")
    assert torch.equal(kc, kb) and torch.equal(vc, vb)
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    close(together, apart.double().cpu(), dtype, "outputs")
    close(kb, ka.double().cpu(), dtype, "key pages")
    close(vb, va.double().cpu(), dtype, "value pages")
    assert float(together[:6].abs().max()) > 0 and float(together[6].abs().max()) == 0.0
    changed = (kb.float() != k_pages.to(dtype).to(DEV).float()).flatten(1).any(dim=1).nonzero().flatten().tolist()
    assert sorted(changed) == sorted(int(table[s, contexts[s] // page]) for s in range(slots))      # one page a request, no other
