"""A plain, slow implementation of the Nafevik decoder in dense 64-bit torch operations over whole sequences: one
function per mechanism, each written from the mechanism's equations (stated in its docstring) and sharing no code
with the package.  `store` stands for the rounding that the bfloat16 serving path applies where it keeps 16-bit
values (identity for the exact model)."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def exact(x):
    return x


def to_bf16(x):
    return x.to(torch.bfloat16).to(F64)


def embed_with_positions(tokens, table, position_table):
    """x_t = table[token_t] + position_table[t], positions counted from 0."""
    t = torch.as_tensor(tokens, dtype=torch.long)
    return table.to(F64)[t] + position_table.to(F64)[torch.arange(len(t))]


def rms_norm(x, weight, eps):
    """y = x / sqrt(mean(x^2) + eps) * weight, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight.to(F64)


def input_conv(h, taps_weight):
    """y_t = h_t + sum_{j=0}^{n-1} c[:, j] * h_{t-n+1+j}, rows before the sequence's start are zero; c [width, n]."""
    c = taps_weight.to(F64)
    n = c.shape[1]
    out = h.clone()
    for t in range(h.shape[0]):
        for j in range(n):
            source = t - n + 1 + j
            if source >= 0:
                out[t] += c[:, j] * h[source]
    return out


def rotary_frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2.  With scaling {factor, original, fast, slow}:
    where(t) = dims ln(original / (2 pi t)) / (2 ln base); lo = max(floor(where(fast)), 0);
    hi = min(ceil(where(slow)), dims - 1); r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
    f_i <- f_i / factor * r_i + f_i (1 - r_i); returns also the magnitude 0.1 ln(factor) + 1 (1 without scaling)."""
    freqs, magnitude = [], 1.0
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            where = lambda t: dims * math.log(scaling["original"] / (2 * math.pi * t)) / (2 * math.log(base))
            lo = max(math.floor(where(scaling["fast"])), 0)
            hi = min(math.ceil(where(scaling["slow"])), dims - 1)
            r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f = f / scaling["factor"] * r + f * (1.0 - r)
            magnitude = 0.1 * math.log(scaling["factor"]) + 1.0
        freqs.append(f)
    return torch.tensor(freqs, dtype=F64), magnitude


def rotate_pairs(x, positions, freqs, magnitude, dims):
    """x [T, heads, d]: for i < dims/2 the pair (x[2i], x[2i+1]) = (u, v) at position p becomes
    (u c - v s, v c + u s), c = magnitude cos(p f_i), s = magnitude sin(p f_i); elements from dims on are kept."""
    out = x.clone()
    for i in range(dims // 2):
        angle = positions.to(F64) * freqs[i]
        c, s = (magnitude * torch.cos(angle))[:, None], (magnitude * torch.sin(angle))[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def visible(i, j, chunk=None, window=None):
    """Whether position i sees key j: j <= i; same block of `chunk` positions (counted from 0); within `window`."""
    if j > i:
        return False
    if chunk and i // chunk != j // chunk:
        return False
    if window and j < i - window + 1:
        return False
    return True


def sigmoid_attention(q, k, v, scale, head_bias, gate_logits, chunk=None, window=None, positions=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads kv head h // (H / G);
    out[t, h] = sigmoid(gate[t, h]) * sum_{j visible from t} sigmoid(scale q[t,h].k[j,g] + bias[h]) v[j, g]."""
    T, H, _ = q.shape
    G = k.shape[1]
    positions = list(range(T)) if positions is None else [int(p) for p in positions]
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    for h in range(H):
        g = h // (H // G)
        scores = (q[:, h] @ k[:, g].T) * scale + float(head_bias[h])
        weights = torch.sigmoid(scores)
        mask = torch.tensor([[visible(positions[i], positions[j], chunk, window) for j in range(T)] for i in range(T)])
        out[:, h] = (weights * mask) @ v[:, g]
    return out * torch.sigmoid(gate_logits)[:, :, None]


def swiglu(x, gate, up, down, store=exact):
    """down (silu(gate x) * (up x)), silu(z) = z sigmoid(z)."""
    a, b = x @ gate.to(F64).T, x @ up.to(F64).T
    return store(a * torch.sigmoid(a) * b) @ down.to(F64).T


def attention_sublayer(mixer, weights, prefix, x, positions, store=exact):
    H, G = mixer["heads"], mixer.get("kv_heads", mixer["heads"])
    d, dv = mixer["dim"], mixer.get("vdim", mixer["dim"])
    T = x.shape[0]
    W = lambda name: weights[prefix + name].to(F64)
    q, k, v = (x @ W("q").T).view(T, H, d), (x @ W("k").T).view(T, G, d), (x @ W("v").T).view(T, G, dv)
    rot = mixer.get("rot")
    if rot:
        freqs, magnitude = rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q = rotate_pairs(q, positions, freqs, magnitude, rot["dims"])
        k = rotate_pairs(k, positions, freqs, magnitude, rot["dims"])
    chunk = mixer["mask"]["size"] if mixer.get("mask") else None
    out = sigmoid_attention(store(q), store(k), store(v), mixer["scale"], W("pb"), x @ W("g").T, chunk=chunk)
    return store(out).reshape(T, H * dv) @ W("o").T


def reinject(x, first, weight, bias_row, store=exact):
    """x <- W [x; first] + b."""
    return store(torch.cat([x, first], dim=-1)) @ weight.to(F64).T + bias_row.to(F64)


def layer_runs(config):
    """(layer, pass of the loop when the run opens a pass, else None) in running order."""
    n, loop = len(config["layers"]), config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(config, weights, tokens, store=exact, trace=None):
    """64-bit logits [T, vocab] of the whole sequence.  `trace` (a list) receives the stream after every layer run."""
    T = len(tokens)
    positions = torch.arange(T)
    x = embed_with_positions(tokens, weights["embed"], weights["pos"])
    first = x
    eps, mult = config["norm"]["eps"], config.get("residual_mult", 1.0)
    for i, opens_pass in layer_runs(config):
        if opens_pass is not None:
            x = reinject(x, first, weights["loop.in"], weights["loop.step"][opens_pass], store)
        layer, prefix = config["layers"][i], f"l{i}."
        h = rms_norm(x, weights[prefix + "norm1"], eps)
        a = input_conv(h, weights[prefix + "canon1"]) if config.get("canon") else h
        y = attention_sublayer(layer["mixer"], weights, prefix + "mix.", store(a), positions, store)
        if layer.get("mlp"):
            b = input_conv(h, weights[prefix + "canon2"]) if config.get("canon") else h
            y = y + swiglu(store(b), weights[prefix + "mlp.gate"], weights[prefix + "mlp.up"],
                           weights[prefix + "mlp.down"], store)
        x = x + mult * y
        if trace is not None:
            trace.append(x)
    return store(rms_norm(x, weights["final.norm"], eps)) @ weights["head"].to(F64).T


def greedy(config, weights, prompt, count):
    tokens, out = list(prompt), []
    for _ in range(count):
        row = forward(config, weights, tokens)[-1]
        best = row.max()
        token = max(i for i in range(len(row)) if row[i] == best)      # the last maximum, as the engine's rule
        out.append(token)
        tokens.append(token)
    return out
