"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases
(mercury/model/qwen2.py:34-42, with act = SiLU). Gate and up are held as one packed matrix
`[2 * intermediate, hidden]` (gate rows first) so that one product feeds both. `activation`
is "silu" or "gelu_tanh" (0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))); `names` gives
the checkpoint's names of the three matrices behind `prefix`."""

from __future__ import annotations

import torch

from .base import FeedForward, TensorSpec, register_feed_forward


class GatedFeedForward(FeedForward):
    capturable = True
    accepts_pending_norm = True
    adds_to_residual = True

    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, prefix: str,
                 activation: str = "silu",
                 names: tuple = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not built; only "
                             f"{' and '.join(self.ACTIVATIONS)}")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.prefix = prefix
        self.activation = activation
        self.names = tuple(names)
        # the fused products that add into the stream belong to the pre-norm block
        if activation != "silu":
            self.adds_to_residual = False
            self.accepts_pending_norm = False
        self.gate_up_weight = self.down_weight = None

    def tensor_specs(self):
        p, h, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + self.names[0], (i, h)),
            TensorSpec(p + self.names[1], (i, h)),
            TensorSpec(p + self.names[2], (h, i)),
        ]

    def load(self, tensors, setup):
        p = self.prefix
        gate = setup.place(tensors[p + self.names[0]])
        up = setup.place(tensors[p + self.names[1]])
        widest = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
        self.gate_up_weight = torch.cat([gate.to(widest), up.to(widest)], dim=0).contiguous()
        self.down_weight = setup.place(tensors[p + self.names[2]])

    def forward(self, x, ctx, residual=None, then_norm=None):
        tokens = x.shape[0]
        act = ctx.buffer("ff_act", tokens, self.intermediate_size)
        if self.activation != "silu":
            ctx.ops.linear_gated(x, self.gate_up_weight, act, ctx, self.activation)
            # float32: the result goes through a norm before it joins the stream
            out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
            ctx.ops.linear(act, self.down_weight, None, out)
            return out
        ctx.ops.linear_swiglu(x, self.gate_up_weight, act, ctx, ahead=self.down_weight)
        if residual is not None:
            return ctx.ops.linear_residual(act, self.down_weight, None, residual, ctx, "ff_out",
                                           then_norm=then_norm)
        out = ctx.buffer("ff_out", tokens, self.hidden_size)
        ctx.ops.linear(act, self.down_weight, None, out)
        return out


register_feed_forward("gated", GatedFeedForward)
