"""A plain, slow Kinelix: whole sequences in float64, no cache, no batching, one function per
mechanism, written from the design's equations and sharing no code with the engine.

A Kinelix model is a stack of pre-norm layers, x <- x + ls1 * mixer(LN1(x)) and then (where the
layer has one) x <- x + ls2 * ff(LN2(x)), LN a layer norm with a weight and no bias. Mixers:

mamba2            [z | x | B | C | dt] = W_in h; (x, B, C) through a causal convolution with bias
                  and SiLU; dt = softplus(dt + dt_bias); per head S_t = exp(-exp(A_log) dt_t) S_(t-1)
                  + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t; y * silu(z), RMS norm in groups, W_o.
delta             q, k, v through causal convolutions (no bias) and SiLU; q, k to unit length per
                  head (q also times dim^-1/2); beta = sigmoid(W_b h); g = exp(-exp(A_log)
                  softplus(W_a h + dt_bias)); S <- g S; u = beta (v - S^T k); S <- S + k u^T;
                  o = S^T q; o / rms(o) * w * silu(W_g h); W_o.
latent_attention  q = W_q h; c = rmsnorm(W_dkv h) * w (or the c of another layer); per head
                  k = W_uk c, v = W_uv c; causal softmax of q.k * scale whose denominator also
                  holds exp(sink_h); W_o.
Feed-forwards: a SiLU-gated dense one, or routed experts (sigmoid scores, a correction that
only steers the choice, groups of neighbours of which the best few may be chosen from).
The stack ends in a layer norm, the head, and cap * tanh(logits / cap).
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, w, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w


def rms_norm(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def causal_conv(x, taps_w, bias=None):
    """x [T, C]; taps_w [C, taps], the last column is the current token's; zeros before the
    start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for k in range(taps):
        out = out + padded[k:k + T] * taps_w[:, k]
    if bias is not None:
        out = out + bias
    return out


def mamba2(h, w, p, m, eps):
    """h [T, width]; w: the tensor dictionary; p: the mixer's prefix; m: its sizes."""
    heads, vdim, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * vdim
    T = h.shape[0]
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, vdim)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)          # [T, heads]
    per = heads // G
    y = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        g = head // per
        S = torch.zeros(N, vdim, dtype=h.dtype)
        for t in range(T):
            S = decay[t, head] * S + dt[t, head] * torch.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + w[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def delta_rule(h, w, p, m, eps):
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, kv_heads, dim)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, kv_heads, dim)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, heads, vdim)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dim ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    g = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    per = heads // kv_heads
    o = torch.zeros(T, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        kh = head // per
        S = torch.zeros(dim, vdim, dtype=h.dtype)
        for t in range(T):
            S = g[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            o[t, head] = S.T @ q[t, kh]
    o = rms_norm(o, eps) * w[p + "norm"]
    o = o.reshape(T, heads * vdim) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def latent(h, w, p, eps):
    """The latent rows a layer caches: rmsnorm(W_dkv h) * weight."""
    return rms_norm(h @ w[p + "dkv"].T, eps) * w[p + "dkv.norm"]


def latent_attention(h, c, w, p, m):
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).reshape(T, heads, dim)
    k = (c @ w[p + "uk"].T).reshape(T, heads, dim)
    v = (c @ w[p + "uv"].T).reshape(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=h.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for head in range(heads):
        s = (q[:, head] @ k[:, head].T) * m["scale"]
        s = s.masked_fill(~mask, -math.inf)
        sink = w[p + "sink"][head]
        big = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - big)
        weights = e / (e.sum(-1, keepdim=True) + torch.exp(sink - big))
        out[:, head] = weights @ v[:, head]
    return out.reshape(T, heads * vdim) @ w[p + "o"].T


def gated(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, w, p, r):
    """(chosen experts [T, top], their weights [T, top])."""
    experts, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = groups["count"], groups["keep"]
    size = experts // count
    grouped = choice.reshape(-1, count, size)
    group_score = grouped.topk(min(2, size), -1).values.sum(-1)
    kept = group_score.topk(keep, -1).indices
    allowed = torch.zeros(h.shape[0], count, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    allowed = allowed.unsqueeze(-1).expand(-1, -1, size).reshape(-1, experts)
    chosen = choice.masked_fill(~allowed, -math.inf).topk(top, -1).indices
    return chosen, s.gather(1, chosen) * r["scale"]


def routed_experts(h, w, p, mlp):
    chosen, weights = route(h, w, p, mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            e_p = f"{p}e{e}."
            out[t] += a * gated(h[t:t + 1], w[e_p + "gate"], w[e_p + "up"], w[e_p + "down"])[0]
    return out


def forward(config: dict, tensors: dict, tokens, layers_out: list | None = None):
    """Logits [T, vocab] of one whole sequence; `layers_out` collects the stream after every
    layer."""
    w = {k: (v.to(F64) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    latents = {}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "mamba2":
            mixed = mamba2(h, w, p + "mix.", m, eps)
        elif layer["type"] == "delta":
            mixed = delta_rule(h, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                latents[i] = latent(h, w, p + "mix.", eps)
                c = latents[i]
            else:
                c = latents[m["kv_from"]]
            mixed = latent_attention(h, c, w, p + "mix.", m)
        else:
            raise ValueError(layer["type"])
        x = x + w[p + "ls1"] * mixed
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                out = gated(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
            else:
                out = routed_experts(h, w, p + "mlp.", mlp)
            x = x + w[p + "ls2"] * out
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
