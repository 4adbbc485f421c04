"""Mixers that carry a state of fixed size from token to token instead of keys and values.

Both keep their state in float32 in the slot the cache manager gave the request, start it
at zero, and run a step's tokens of each sequence in order from where the step before
left it. Everything inside the recurrence (gates, decays, the state) is float32; the
projections around it are products like any other.

`MinGRU`:  z = sigmoid(Wz x + bz), u = Wx x + bx, c = u + 1/2 where u >= 0 and sigmoid(u)
           where u < 0;  S_t = (1 - z) S_{t-1} + z c;  out = Wo (S_t * silu(Wg x)).
`GatedLinearRecurrence` (the recurrent block of Griffin: De et al., "Griffin: Mixing Gated
Linear Recurrences with Local Attention for Efficient Language Models"):
           y = gelu_tanh(Wy x + by); u = conv(Wx x + bx), a causal convolution per channel
           over `taps` tokens; per block b of the channels r = sigmoid(Ra_b u_b + ra_b) and
           i = sigmoid(Ri_b u_b + ri_b); a = exp(-decay_scale * r * softplus(lam));
           S_t = a S_{t-1} + sqrt(1 - a^2) * i * u;  out = Wo (S_t * y).
           Its state is S and the last taps - 1 inputs of the convolution.
"""

from __future__ import annotations

import torch

from .base import Mixer, StateNeed, TensorSpec, register_mixer


class MinGRU(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, width: int, prefix: str, names: dict | None = None,
                 bias_suffix: str = ".b"):
        self.hidden_size, self.width, self.prefix = hidden_size, width, prefix
        self.names = {"z": "z", "x": "x", "g": "g", "o": "o"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix
        self.in_weight = self.in_bias = self.out_weight = None

    def state_need(self):
        return StateNeed((self.width,), torch.float32)

    def tensor_specs(self):
        p, n, b, h, w = self.prefix, self.names, self.bias_suffix, self.hidden_size, self.width
        return [TensorSpec(p + n["z"], (w, h)), TensorSpec(p + n["z"] + b, (w,)),
                TensorSpec(p + n["x"], (w, h)), TensorSpec(p + n["x"] + b, (w,)),
                TensorSpec(p + n["g"], (w, h)), TensorSpec(p + n["o"], (h, w))]

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix
        mats = [setup.place(tensors[p + n[k]]) for k in ("z", "x", "g")]
        biases = [setup.place(tensors[p + n["z"] + b]), setup.place(tensors[p + n["x"] + b])]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats + biases) else mats[0].dtype
        # one product feeds the gate, the candidate and the output gate: rows [z; x; g]
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()
        self.in_bias = torch.cat([t.to(widest) for t in biases]
                                 + [torch.zeros(self.width, dtype=widest, device=mats[0].device)]
                                 ).contiguous()
        self.out_weight = setup.place(tensors[p + n["o"]])

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        pre = ctx.buffer("recurrent_in", tokens, 3 * self.width, dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        mixed = ctx.buffer("recurrent_mixed", tokens, self.width)
        ops.mingru_scan(pre, state, ctx.batch, mixed)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(mixed, self.out_weight, None, out)
        return out


class GatedLinearRecurrence(Mixer):
    capturable = True

    def __init__(self, hidden_size: int, width: int, blocks: int, taps: int, prefix: str,
                 decay_scale: float = 8.0, names: dict | None = None, bias_suffix: str = ".b"):
        if width % blocks:
            raise ValueError(f"width {width} does not divide into {blocks} blocks")
        if not 1 <= taps <= 16:
            raise ValueError(f"a convolution over {taps} tokens is not built (1 to 16)")
        self.hidden_size, self.width, self.blocks, self.taps = hidden_size, width, blocks, taps
        self.prefix = prefix
        self.decay_scale = float(decay_scale)
        self.names = {"y": "y", "x": "x", "conv": "conv", "ra": "ra", "ri": "ri", "lam": "lam",
                      "o": "o"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix

    def state_need(self):
        # row 0: S; row j >= 1: the convolution's input j tokens back
        return StateNeed((self.taps, self.width), torch.float32)

    def tensor_specs(self):
        p, n, b, h, w = self.prefix, self.names, self.bias_suffix, self.hidden_size, self.width
        size = w // self.blocks
        return [TensorSpec(p + n["y"], (w, h)), TensorSpec(p + n["y"] + b, (w,)),
                TensorSpec(p + n["x"], (w, h)), TensorSpec(p + n["x"] + b, (w,)),
                TensorSpec(p + n["conv"], (w, self.taps), std=0.3),
                TensorSpec(p + n["conv"] + b, (w,)),
                TensorSpec(p + n["ra"], (self.blocks, size, size), std=0.1),
                TensorSpec(p + n["ra"] + b, (self.blocks, size)),
                TensorSpec(p + n["ri"], (self.blocks, size, size), std=0.1),
                TensorSpec(p + n["ri"] + b, (self.blocks, size)),
                TensorSpec(p + n["lam"], (w,), std=0.5, mean=-1.0),
                TensorSpec(p + n["o"], (h, w))]

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix
        place = lambda name: setup.place(tensors[p + name])
        mats = [place(n["y"]), place(n["x"])]
        biases = [place(n["y"] + b), place(n["x"] + b)]
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats + biases) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()   # rows [y; x]
        self.in_bias = torch.cat([t.to(widest) for t in biases]).contiguous()
        # what stands inside the recurrence is float32: taps, gate matrices, decay
        self.conv = place(n["conv"]).float().contiguous()
        self.conv_bias = place(n["conv"] + b).float().contiguous()
        # [2][blocks][in][out]: input-major, the way the gate kernel reads it
        self.gate_weight = torch.stack([place(n["ra"]).float(), place(n["ri"]).float()]
                                       ).transpose(-1, -2).contiguous()
        self.gate_bias = torch.stack([place(n["ra"] + b).float(), place(n["ri"] + b).float()]).contiguous()
        self.softplus_lam = torch.nn.functional.softplus(place(n["lam"]).float()).contiguous()
        self.out_weight = place(n["o"])

    def forward(self, x, ctx, cache, state):
        tokens, ops, w = x.shape[0], ctx.ops, self.width
        pre = ctx.buffer("recurrent_in", tokens, 2 * w, dtype="float32")
        ops.linear(x, self.in_weight, self.in_bias, pre)
        u = ctx.buffer("recurrent_conv", tokens, w, dtype="float32")
        ops.causal_conv(pre, w, w, self.conv, self.conv_bias, state, ctx.batch, u)
        gates = ctx.buffer("recurrent_gates", tokens, 2 * w, dtype="float32")
        ops.block_gates(u, self.gate_weight, self.gate_bias, gates)
        mixed = ctx.buffer("recurrent_mixed", tokens, w)
        ops.gated_recurrence_scan(pre, u, gates, self.softplus_lam, self.decay_scale, state,
                                  ctx.batch, mixed)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(mixed, self.out_weight, None, out)
        return out


register_mixer("mingru", MinGRU)
register_mixer("gated_linear_recurrence", GatedLinearRecurrence)
