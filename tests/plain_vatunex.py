"""A plain, slow implementation of the Vatunex decoder in dense 64-bit torch operations over whole sequences: one
function per mechanism, each written from the mechanism's equations (stated in its docstring) and sharing no code
with the package.

The design: x = embed[token]; every layer is  x <- x + N1b(mixer(N1(x))),  x <- x + N2b(ff(N2(x)))  (the second
line only when the layer has a feed-forward), N(.) an RMS norm whose stored weight w is used as 1 + w; the mixer of a
layer is one of `latent_attention`, `attention`, `mamba1`; logits = head N(x)."""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis, eps inside the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    """rms(x) * (1 + w)."""
    return rms(x, eps) * (1.0 + w.to(F64))


def norm_plain(x, w, eps):
    """rms(x) * w."""
    return rms(x, eps) * w.to(F64)


def gelu_tanh(z):
    """0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))."""
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dense_mlp(h, up, down):
    """down gelu_tanh(up h)."""
    return gelu_tanh(h @ up.to(F64).T) @ down.to(F64).T


def rotary_frequencies(base, dims, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2.  With scaling {factor, low, high, original} and wavelength l_i = 2 pi / f_i:
    l_i < original/high keeps f_i; l_i > original/low gives f_i / factor; between them
    s = (original / l_i - low) / (high - low) and f_i <- (1 - s) f_i / factor + s f_i."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, original = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate_half(x, positions, freqs, dims):
    """x [T, heads, d]: for i < dims/2 the pair (u, v) = (x[i], x[i + dims/2]) at position p becomes
    (u cos a - v sin a, v cos a + u sin a), a = p f_i; elements from dims on pass unchanged."""
    out = x.clone()
    half = dims // 2
    angle = positions.to(F64)[:, None] * freqs[None, :]                  # [T, half]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[:, :, :half], x[:, :, half:dims]
    out[:, :, :half] = u * c - v * s
    out[:, :, half:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale, window=None, sink=False):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; head h reads kv head h // (H / G).  Token i sees j with
    0 <= i - j (< window if one is set).  weights p_ij = exp(s_ij) / (sink + sum_j exp(s_ij)), s = scale q.k, where
    `sink` adds 1 to the denominator (a key of score 0 without a value).  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    out = torch.zeros((T, H, v.shape[2]), dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink:
            m = torch.clamp(m, min=0.0)
        e = torch.exp(s - m)
        denominator = e.sum(dim=-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out[:, h] = (e / denominator) @ v[:, g]
    return out


def latent_attention(mixer, W, h, positions, eps):
    """Attention through latents.  c_q = rms(W_dq h) * w_dqn; q = W_uq c_q, per head [dim | rot_dim].
    W_dkv h = [a: kv_rank | r: rot_dim]; c = rms(a) * w_dkvn; per head k = [W_uk c | rotate(r)] (r shared by the
    heads), v = W_uv c; the rot_dim part of q is rotated too.  Softmax over a window of mask.size, no sink."""
    T = h.shape[0]
    H, d, dr, dv, rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    cq = norm_plain(h @ W("dq").T, W("dq.norm"), eps)
    q = (cq @ W("uq").T).view(T, H, d + dr)
    dkv = h @ W("dkv").T
    c = norm_plain(dkv[:, :rank], W("dkv.norm"), eps)
    freqs = rotary_frequencies(mixer["rot"]["base"], mixer["rot"]["dims"], mixer["rot"].get("scaling"))
    shared = rotate_half(dkv[:, None, rank:], positions, freqs, mixer["rot"]["dims"])          # [T, 1, dr]
    q_rot = rotate_half(q[:, :, d:], positions, freqs, mixer["rot"]["dims"])
    k = torch.cat([(c @ W("uk").T).view(T, H, d), shared.expand(T, H, dr)], dim=-1)
    qq = torch.cat([q[:, :, :d], q_rot], dim=-1)
    v = (c @ W("uv").T).view(T, H, dv)
    window = mixer["mask"]["size"] if mixer.get("mask") else None
    o = softmax_attention(qq, k, v, mixer["scale"], window=window, sink=False)
    return o.reshape(T, H * dv) @ W("o").T


def attention(mixer, W, h, positions, eps, shared_values):
    """Grouped-query attention with biases, per-head norms of q and k, scaled rotary frequencies, a sink in the softmax
    and value mixing.  q = W_q h + b_q (k, v alike); q_h <- rms(q_h) * w_qn, k_g <- rms(k_g) * w_kn; both rotated over
    the first rot.dims elements; with `v_mix`: the first such layer of the model leaves its v in `shared_values`, every
    later one uses v <- (1 - lambda) v + lambda v_first; causal, all keys; output W_o o + b_o."""
    T = h.shape[0]
    H, G, d, dv = mixer["heads"], mixer.get("kv_heads", mixer["heads"]), mixer["dim"], mixer.get("vdim", mixer["dim"])
    q = (h @ W("q").T + W("q.b")).view(T, H, d)
    k = (h @ W("k").T + W("k.b")).view(T, G, d)
    v = (h @ W("v").T + W("v.b")).view(T, G, dv)
    q, k = norm_plain(q, W("q.norm"), eps), norm_plain(k, W("k.norm"), eps)
    rot = mixer.get("rot")
    if rot:
        freqs = rotary_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
        q, k = rotate_half(q, positions, freqs, rot["dims"]), rotate_half(k, positions, freqs, rot["dims"])
    if mixer.get("v_mix"):
        if "first" not in shared_values:
            shared_values["first"] = v
        else:
            lam = float(W("vmix"))
            v = (1.0 - lam) * v + lam * shared_values["first"]
    window = mixer["mask"]["size"] if mixer.get("mask") else None
    o = softmax_attention(q, k, v, mixer["scale"], window=window, sink=True)
    return o.reshape(T, H * dv) @ W("o").T + W("o.b")


def causal_conv(x, taps, bias):
    """y_t[c] = bias[c] + sum_j taps[c, j] x_(t - n + 1 + j)[c], zeros before the start; taps [channels, n]."""
    T, n = x.shape[0], taps.shape[1]
    y = bias.to(F64)[None, :].repeat(T, 1)
    for j in range(n):
        shift = n - 1 - j
        if shift < T:
            y[shift:] += taps.to(F64)[:, j] * x[:T - shift]
    return y


def selective_scan(x, dt, A, B, C, D):
    """S_t[c, n] = exp(dt_t[c] A[c, n]) S_(t-1)[c, n] + dt_t[c] x_t[c] B_t[n], S_(-1) = 0;
    y_t[c] = sum_n S_t[c, n] C_t[n] + D[c] x_t[c]."""
    T, inner = x.shape
    S = torch.zeros((inner, A.shape[1]), dtype=F64)
    y = torch.zeros((T, inner), dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


def mamba1(mixer, W, h):
    """[x | z] = W_in h; x <- silu(conv(x)); [dt | B | C] = W_x x; dt <- softplus(W_dt dt + b_dt); A = -exp(A_log);
    y = scan(x, dt, A, B, C, D) * silu(z); output W_o y."""
    inner, rank, state = mixer["inner"], mixer["dt_rank"], mixer["state"]
    xz = h @ W("in").T
    x, z = xz[:, :inner], xz[:, inner:]
    x = causal_conv(x, W("conv"), W("conv.b"))
    x = x * torch.sigmoid(x)
    proj = x @ W("x").T
    dt = torch.nn.functional.softplus(proj[:, :rank] @ W("dt").T + W("dt.b"))
    B, C = proj[:, rank:rank + state], proj[:, rank + state:rank + 2 * state]
    y = selective_scan(x, dt, -torch.exp(W("A_log")), B, C, W("D"))
    return (y * (z * torch.sigmoid(z))) @ W("o").T


def forward(config, weights, tokens, return_layers=False):
    """Logits [T, vocab] (64-bit) of the whole sequence; with `return_layers` also the residual stream after every layer."""
    eps = float(config["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = weights["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)]
    shared_values, after = {}, []
    for i, layer in enumerate(config["layers"]):
        prefix = f"l{i}."
        W = lambda name, p=prefix: weights[p + "mix." + name].to(F64)
        h = norm_one_plus(x, weights[prefix + "norm1"], eps)
        kind = layer["type"]
        if kind == "latent_attention":
            y = latent_attention(layer["mixer"], W, h, positions, eps)
        elif kind == "attention":
            y = attention(layer["mixer"], W, h, positions, eps, shared_values)
        elif kind == "mamba1":
            y = mamba1(layer["mixer"], W, h)
        else:
            raise ValueError(f"unknown mixer {kind!r}")
        x = x + norm_one_plus(y, weights[prefix + "norm1b"], eps)
        if layer.get("mlp"):
            h = norm_one_plus(x, weights[prefix + "norm2"], eps)
            y = dense_mlp(h, weights[prefix + "mlp.up"], weights[prefix + "mlp.down"])
            x = x + norm_one_plus(y, weights[prefix + "norm2b"], eps)
        after.append(x.clone())
    logits = norm_one_plus(x, weights["final.norm"], eps) @ weights["head"].to(F64).T
    return (logits, torch.stack(after)) if return_layers else logits


def greedy(config, weights, prompt, count):
    """`count` tokens after `prompt`, each the largest logit's id (the largest id among equals)."""
    tokens, out = list(prompt), []
    for _ in range(count):
        row = forward(config, weights, tokens)[-1]
        best = row.max()
        token = max(i for i in range(len(row)) if row[i] == best)
        out.append(token)
        tokens.append(token)
    return out
