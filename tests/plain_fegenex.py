"""The Fegenex decoder written out plainly: whole sequences, no cache, no batching, float64
by default. One function per mechanism; nothing here is shared with the engine, which is
compared against it.

Notation. x_t is the residual stream at token t (position t), eps the norm constant.
  norm_g(x)      = x / sqrt(mean(x^2) + eps) * g                    (g one number)
  layer          : x <- x + norm_1b(mixer(norm_1(x)));  x <- x + norm_2b(ff(norm_2(x)))
  minGRU         : z = sigma(Wz h + bz), u = Wx h + bx, c = u + 1/2 (u >= 0) | sigma(u) (u < 0),
                   S_t = (1 - z) S_{t-1} + z c,  out = Wo (S_t * silu(Wg h))
  RG-LRU         : y = gelu(Wy h + by), u = conv(Wx h + bx) (causal, per channel),
                   per block b: r = sigma(Ra_b u_b + ra_b), i = sigma(Ri_b u_b + ri_b),
                   a = exp(-8 r softplus(lam)), S_t = a S_{t-1} + sqrt(1 - a^2) i u,
                   out = Wo (S_t * y)
  attention      : rotary on the first `dims` features of each q/k head (feature i with
                   i + dims/2, angle p * base^(-2i/dims)), softmax(q.k * scale) over j <= i,
                   the heads' weights mixed by T (w_h <- sum_g T[h,g] w_g), values optionally
                   blended with the first blending layer's values of the same token
  feed-forward   : Wdown (gelu(Wgate h) * (Wup h)),  gelu in its tanh form
"""

from __future__ import annotations

import math

import torch


def plain_gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def plain_scalar_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def plain_embedding(w, tokens):
    ids = torch.tensor(tokens, dtype=torch.long)
    return w["embed"][ids] + w["pos"][torch.arange(len(tokens))]


def plain_mingru(h, w, p):
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ w[p + "g"].T
    gate = gate * torch.sigmoid(gate)
    state = torch.zeros_like(u[0])
    rows = []
    for t in range(h.shape[0]):
        state = (1.0 - z[t]) * state + z[t] * cand[t]
        rows.append(state * gate[t])
    return torch.stack(rows) @ w[p + "o"].T


def plain_causal_conv(x, kernel, bias):
    """x [T, C], kernel [C, taps] whose last column meets the current token."""
    taps = kernel.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x])
    out = torch.zeros_like(x)
    for k in range(taps):
        out = out + padded[k:k + x.shape[0]] * kernel[:, k]
    return out + bias


def plain_rglru(h, w, p, blocks):
    y = plain_gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = plain_causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    width = u.shape[1]
    size = width // blocks
    ub = u.view(-1, blocks, size)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ra"], ub) + w[p + "ra.b"]).reshape(-1, width)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w[p + "ri"], ub) + w[p + "ri.b"]).reshape(-1, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    state = torch.zeros_like(u[0])
    rows = []
    for t in range(h.shape[0]):
        state = a[t] * state + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        rows.append(state * y[t])
    return torch.stack(rows) @ w[p + "o"].T


def plain_partial_rotary(x, dims, base):
    """x [T, heads, dim]; the first `dims` features of each head are rotated."""
    if not dims:
        return x
    half = dims // 2
    positions = torch.arange(x.shape[0], dtype=x.dtype)
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    angle = positions[:, None] * freq[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., dims:]], dim=-1)


def plain_mixed_head_attention(h, w, p, mixer, v_first):
    """Returns (output, values before blending). `v_first` is None in the first blending
    layer and in layers that do not blend."""
    heads, kv_heads = mixer["heads"], mixer["kv_heads"]
    dim, vdim = mixer["dim"], mixer["vdim"]
    tokens = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(tokens, heads, dim)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(tokens, kv_heads, dim)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(tokens, kv_heads, vdim)
    rot = mixer.get("rot") or {}
    q = plain_partial_rotary(q, rot.get("dims", 0), rot.get("base", 10000.0))
    k = plain_partial_rotary(k, rot.get("dims", 0), rot.get("base", 10000.0))
    own_v = v
    if v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    group = heads // kv_heads
    hidden = torch.triu(torch.ones(tokens, tokens, dtype=torch.bool), diagonal=1)
    weights = []
    for head in range(heads):
        scores = (q[:, head] @ k[:, head // group].T) * mixer["scale"]
        weights.append(torch.softmax(scores.masked_fill(hidden, float("-inf")), dim=-1))
    weights = torch.stack(weights)                                   # [heads, T, T]
    mixed = torch.einsum("hg,gij->hij", w[p + "talk"], weights)
    out = torch.stack([mixed[head] @ v[:, head // group] for head in range(heads)], dim=1)
    return out.reshape(tokens, heads * vdim) @ w[p + "o"].T + w[p + "o.b"], own_v


def plain_gated_gelu(h, w, p):
    return (plain_gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def plain_fegenex(raw: dict, tensors: dict, tokens: list[int], dtype=torch.float64):
    """Logits [T, vocab] and the residual stream after every layer [layers, T, width]."""
    w = {name: t.to(dtype) for name, t in tensors.items()}
    eps = raw["norm"]["eps"]
    x = plain_embedding(w, tokens)
    v_first = None
    after = []
    for index, layer in enumerate(raw["layers"]):
        p = f"l{index}."
        h = plain_scalar_norm(x, w[p + "norm1"], eps)
        kind, mixer = layer["type"], layer["mixer"]
        if kind == "mingru":
            mixed = plain_mingru(h, w, p + "mix.")
        elif kind == "rglru":
            mixed = plain_rglru(h, w, p + "mix.", mixer["blocks"])
        elif kind == "attention":
            blend = bool(mixer.get("v_mix"))
            mixed, own_v = plain_mixed_head_attention(h, w, p + "mix.", mixer,
                                                      v_first if blend else None)
            if blend and v_first is None:
                v_first = own_v
        else:
            raise ValueError(kind)
        x = x + plain_scalar_norm(mixed, w[p + "norm1b"], eps)
        if layer.get("mlp"):
            h = plain_scalar_norm(x, w[p + "norm2"], eps)
            x = x + plain_scalar_norm(plain_gated_gelu(h, w, p + "mlp."), w[p + "norm2b"], eps)
        after.append(x)
    logits = plain_scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return logits, torch.stack(after)
