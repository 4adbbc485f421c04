"""Grouped-query attention over the paged cache.

Formulas of mercury/model/qwen2.py:45-69: q, k and v projections (bias on all three when
`qkv_bias`), position encoding on q and k after the bias and before the keys are stored,
keys and values stored before attending (mercury/model/attention.py:127, :154) so that a
portion sees its own keys, softmax(q.k * scale) over the keys j <= p, query head h reading
KV head h // (heads / kv_heads), and an output projection. The three projections are held
as one packed matrix so that one product feeds them.
"""

from __future__ import annotations

import torch

from .base import CacheNeed, Mixer, PartSpec, TensorSpec, build_part, register_mixer


class GroupedQueryAttention(Mixer):
    capturable = True
    accepts_pending_norm = True
    adds_to_residual = True

    def __init__(
        self,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        scale: float,
        prefix: str,
        qkv_bias: bool = True,
        out_bias: bool = False,
        window: int = 0,
        position_encoding: PartSpec | None = None,
    ):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.scale = float(scale)
        self.prefix = prefix
        self.qkv_bias = qkv_bias
        self.out_bias = out_bias
        self.window = int(window)
        self.position = build_part(
            "position_encoding", position_encoding or PartSpec("none", {})
        )
        self.q_size = num_heads * head_dim
        self.kv_size = num_kv_heads * head_dim
        self.qkv_weight = self.qkv_b = self.out_weight = self.out_b = None

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self):
        p, h = self.prefix, self.hidden_size
        specs = [
            TensorSpec(p + "q_proj.weight", (self.q_size, h)),
            TensorSpec(p + "k_proj.weight", (self.kv_size, h)),
            TensorSpec(p + "v_proj.weight", (self.kv_size, h)),
            TensorSpec(p + "o_proj.weight", (h, self.q_size)),
        ]
        if self.qkv_bias:
            specs += [
                TensorSpec(p + "q_proj.bias", (self.q_size,)),
                TensorSpec(p + "k_proj.bias", (self.kv_size,)),
                TensorSpec(p + "v_proj.bias", (self.kv_size,)),
            ]
        if self.out_bias:
            specs.append(TensorSpec(p + "o_proj.bias", (h,)))
        return specs + self.position.tensor_specs()      # a learned encoding owns tensors too

    def load(self, tensors, setup):
        p = self.prefix

        def packed(suffix):
            parts = [setup.place(tensors[p + name + suffix]) for name in ("q_proj", "k_proj", "v_proj")]
            widest = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
            return torch.cat([t.to(widest) for t in parts], dim=0).contiguous()

        self.qkv_weight = packed(".weight")
        self.qkv_b = packed(".bias") if self.qkv_bias else None
        self.out_weight = setup.place(tensors[p + "o_proj.weight"])
        self.out_b = setup.place(tensors[p + "o_proj.bias"]) if self.out_bias else None
        self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state, residual=None, then_norm=None):
        tokens = x.shape[0]
        ops = ctx.ops
        qkv = ctx.buffer("qkv", tokens, self.q_size + 2 * self.kv_size)
        form = self.position.fused_form()
        tables = self.position.rotary_tables() if form == "rotary" else None
        attended = ctx.buffer("attended", tokens, self.q_size)
        fused = getattr(ops, "qkv_attention", None)
        if fused is not None and form is not None:
            # projection, bias, rotation, store into the pages and attention: the kernels
            # choose how to share the work between them
            fused(x, self.qkv_weight, self.qkv_b, qkv, self.num_heads, self.num_kv_heads,
                  self.head_dim, tables, ctx.batch, cache, self.scale, self.window, attended)
            return self._project_out(attended, ctx, residual, then_norm, tokens)
        if form is not None:
            # projection, bias, rotation and the store into the pages, fused where it pays
            ops.qkv_rope_store(x, self.qkv_weight, self.qkv_b, qkv, self.num_heads,
                               self.num_kv_heads, self.head_dim, tables, ctx.batch, cache)
        else:
            if hasattr(x, "materialize"):
                x = x.materialize()
            ops.linear(x, self.qkv_weight, self.qkv_b, qkv)
            self.position.apply(qkv, (self.num_heads, self.num_kv_heads, self.head_dim), ctx)
            ops.rope_cache_write(qkv, self.num_heads, self.num_kv_heads, self.head_dim, None,
                                 ctx.batch, cache)
        ops.paged_attention(
            qkv, self.num_heads, self.num_kv_heads, self.head_dim, ctx.batch, cache,
            self.scale, self.window, attended,
        )
        return self._project_out(attended, ctx, residual, then_norm, tokens)

    def _project_out(self, attended, ctx, residual, then_norm, tokens):
        ops = ctx.ops
        if residual is not None:
            return ops.linear_residual(attended, self.out_weight, self.out_b, residual, ctx,
                                       "mixer_out", then_norm=then_norm)
        out = ctx.buffer("mixer_out", tokens, self.hidden_size)
        ops.linear(attended, self.out_weight, self.out_b, out)
        return out


register_mixer("grouped_query_attention", GroupedQueryAttention)


class MixedHeadAttention(Mixer):
    """Grouped-query attention whose heads exchange their softmax weights, with key and
    value heads of different sizes and an optional blend of the values across layers.

    Per token: q, k, v projections with biases; the position encoding on q and k; the value
    blend; keys and blended values stored in the pages; w_g = softmax(q_g . k * scale) over
    the keys j <= p (and inside `window`, if one is given); when `head_mix` is set the
    weights are mixed before they meet the values, w'_h = sum_g M[h, g] w_g with M a learned
    [heads, heads] matrix, and head h applies w'_h to the values of its own key/value head;
    an output projection with bias.

    `value_blend` = ("source", key): this layer's values of the step's tokens are left in
    `ctx.carry[key]` for later layers. ("blend", key): v <- (1 - c) v + c carry[key], with c
    one learned number (`names["blend"]`); the blended values are what the pages hold.

    `names` maps q, k, v, o (biases: the name + ".b" unless `bias_suffix` says otherwise),
    mix and blend to checkpoint names behind `prefix`.
    """

    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 value_dim: int, scale: float, prefix: str, names: dict | None = None,
                 bias_suffix: str = ".b", head_mix: bool = True,
                 value_blend: tuple | None = None, window: int = 0,
                 position_encoding: PartSpec | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads do not divide into {num_kv_heads} groups")
        self.hidden_size = hidden_size
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.head_dim, self.value_dim = head_dim, value_dim
        self.scale = float(scale)
        self.prefix = prefix
        self.names = {"q": "q", "k": "k", "v": "v", "o": "o", "mix": "talk", "blend": "vmix"}
        self.names.update(names or {})
        self.bias_suffix = bias_suffix
        self.head_mix = bool(head_mix)
        self.value_blend = tuple(value_blend) if value_blend else None
        if self.value_blend and self.value_blend[0] not in ("source", "blend"):
            raise ValueError(f"value_blend role {self.value_blend[0]!r}")
        self.window = int(window)
        self.position = build_part("position_encoding", position_encoding or PartSpec("none", {}))
        if self.position.fused_form() is None:
            raise ValueError("this mixer takes a rotary encoding or none")
        self.q_size = num_heads * head_dim
        self.k_size = num_kv_heads * head_dim
        self.v_size = num_kv_heads * value_dim
        self.qkv_weight = self.qkv_b = self.out_weight = self.out_b = None
        self.mix = self.blend = None

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window, self.value_dim)

    def tensor_specs(self):
        p, h, n, b = self.prefix, self.hidden_size, self.names, self.bias_suffix
        specs = [TensorSpec(p + n["q"], (self.q_size, h)), TensorSpec(p + n["q"] + b, (self.q_size,)),
                 TensorSpec(p + n["k"], (self.k_size, h)), TensorSpec(p + n["k"] + b, (self.k_size,)),
                 TensorSpec(p + n["v"], (self.v_size, h)), TensorSpec(p + n["v"] + b, (self.v_size,)),
                 TensorSpec(p + n["o"], (h, self.num_heads * self.value_dim)),
                 TensorSpec(p + n["o"] + b, (h,))]
        if self.head_mix:
            specs.append(TensorSpec(p + n["mix"], (self.num_heads, self.num_heads),
                                    init="eye_normal", std=0.1))
        if self.value_blend and self.value_blend[0] == "blend":
            specs.append(TensorSpec(p + n["blend"], (), std=0.1, mean=0.4))
        return specs + self.position.tensor_specs()

    def load(self, tensors, setup):
        p, n, b = self.prefix, self.names, self.bias_suffix

        def packed(suffix):
            parts = [setup.place(tensors[p + n[key] + suffix]) for key in ("q", "k", "v")]
            widest = torch.float32 if any(t.dtype == torch.float32 for t in parts) else parts[0].dtype
            return torch.cat([t.to(widest) for t in parts], dim=0).contiguous()

        self.qkv_weight, self.qkv_b = packed(""), packed(b)
        self.out_weight = setup.place(tensors[p + n["o"]])
        self.out_b = setup.place(tensors[p + n["o"] + b])
        # the weights of the softmax are float32, and so is what mixes them
        self.mix = setup.place(tensors[p + n["mix"]]).float().contiguous() if self.head_mix else None
        if self.value_blend and self.value_blend[0] == "blend":
            self.blend = setup.place(tensors[p + n["blend"]]).float().reshape(1).contiguous()
        self.position.load(tensors, setup)

    def forward(self, x, ctx, cache, state):
        tokens = x.shape[0]
        ops = ctx.ops
        qkv = ctx.buffer("qkv_split", tokens, self.q_size + self.k_size + self.v_size)
        ops.linear(x, self.qkv_weight, self.qkv_b, qkv)
        tables = self.position.rotary_tables() if self.position.fused_form() == "rotary" else None
        keep = blend_from = None
        if self.value_blend:
            role, key = self.value_blend
            if role == "source":
                keep = ctx.carry[key] = ctx.buffer("values_" + str(key), tokens, self.v_size)
            else:
                blend_from = ctx.carry.get(key)
                if blend_from is None or blend_from.shape[1] != self.v_size:
                    raise ValueError(f"{self.prefix}: no layer before this one left values of "
                                     f"width {self.v_size} under {key!r}")
        layout = (self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim)
        ops.rope_blend_store(qkv, layout, tables, ctx.batch, cache, blend_from, self.blend, keep)
        attended = ctx.buffer("attended_v", tokens, self.num_heads * self.value_dim)
        ops.mixed_head_attention(qkv, layout, ctx.batch, cache, self.scale, self.window, self.mix,
                                 attended)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(attended, self.out_weight, self.out_b, out)
        return out


class LatentAttention(Mixer):
    """Attention over a cached low-rank latent, without positions, with a softmax sink.

    Per token: q = Wq h (heads x dim); c = rmsnorm(Wdkv h) * w, `rank` numbers, the only
    thing the cache keeps; per head k = Wuk c and v = Wuv c; weights = exp(s_j) / (sum_j'
    exp(s_j') + exp(sink_h)) over the keys j <= p with s = q.k * scale; an output projection.

    The keys and values are never built. Since q.(Wuk_h c) = (Wuk_h^T q).c, a head's query is
    taken into the latent space once per token and the head attends over the cached rows
    themselves, which serve as keys and as values (one shared head of size `rank` for all
    query heads); Wuv_h is applied to the head's weighted sum of rows afterwards.

    `own_latent=False`: the layer has no Wdkv and reads the rows that another layer's call
    stored (its `LayerCall` names that call's cache layer with `writes_cache=False`).
    """

    capturable = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, rank: int,
                 scale: float, eps: float, prefix: str, own_latent: bool = True,
                 names: dict | None = None):
        self.hidden_size, self.num_heads = hidden_size, num_heads
        self.head_dim, self.value_dim, self.rank = head_dim, value_dim, rank
        self.scale, self.eps, self.prefix = float(scale), float(eps), prefix
        self.own_latent = bool(own_latent)
        self.q_size = num_heads * head_dim
        self.names = {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv",
                      "sink": "sink", "o": "o"}
        self.names.update(names or {})

    def cache_need(self):
        return CacheNeed(1, self.rank, 0, shared_values=True)

    def tensor_specs(self):
        p, n, h = self.prefix, self.names, self.hidden_size
        specs = [TensorSpec(p + n["q"], (self.q_size, h))]
        if self.own_latent:
            specs += [TensorSpec(p + n["down"], (self.rank, h)),
                      TensorSpec(p + n["down_norm"], (self.rank,), init="ones_normal", std=0.05)]
        return specs + [TensorSpec(p + n["up_k"], (self.q_size, self.rank)),
                        TensorSpec(p + n["up_v"], (self.num_heads * self.value_dim, self.rank)),
                        TensorSpec(p + n["sink"], (self.num_heads,), std=1.0),
                        TensorSpec(p + n["o"], (h, self.num_heads * self.value_dim))]

    def load(self, tensors, setup):
        p, n = self.prefix, self.names
        mats = [setup.place(tensors[p + n["q"]])]
        if self.own_latent:
            mats.append(setup.place(tensors[p + n["down"]]))
            self.down_norm = setup.place(tensors[p + n["down_norm"]])
        widest = torch.float32 if any(t.dtype == torch.float32 for t in mats) else mats[0].dtype
        self.in_weight = torch.cat([t.to(widest) for t in mats], dim=0).contiguous()   # rows [q; dkv]
        up_k = setup.place(tensors[p + n["up_k"]])
        # both per head and input-major, [heads, in, out]: the key up-projection as stored is the
        # map that takes a query to the latent (its transpose); the value up-projection is turned
        self.absorb = up_k.view(self.num_heads, self.head_dim, self.rank).contiguous()
        self.up_v = (setup.place(tensors[p + n["up_v"]]).view(self.num_heads, self.value_dim, self.rank)
                     .transpose(1, 2).contiguous())
        self.sink = setup.place(tensors[p + n["sink"]]).float().contiguous()
        self.out_weight = setup.place(tensors[p + n["o"]])

    def forward(self, x, ctx, cache, state):
        tokens, ops = x.shape[0], ctx.ops
        if cache.write != self.own_latent:
            raise ValueError(f"{self.prefix}: a layer stores latent rows iff it makes its own")
        pre = ctx.buffer("latent_in", tokens, self.in_weight.shape[0], dtype="float32")
        ops.linear(x, self.in_weight, None, pre)
        if self.own_latent:
            ops.latent_norm_store(pre, self.q_size, self.rank, self.down_norm, self.eps, ctx.batch, cache)
        q = ctx.buffer("latent_q", tokens, self.num_heads * self.rank)
        ops.head_linear(pre, 0, self.absorb, q)
        gathered = ctx.buffer("latent_sum", tokens, self.num_heads * self.rank)
        ops.paged_attention(q, self.num_heads, 1, self.rank, ctx.batch, cache, self.scale, 0,
                            gathered, sinks=self.sink)
        attended = ctx.buffer("attended_v", tokens, self.num_heads * self.value_dim)
        ops.head_linear(gathered, 0, self.up_v, attended)
        out = ctx.buffer("sublayer_out", tokens, self.hidden_size, dtype="float32")
        ops.linear(attended, self.out_weight, None, out)
        return out


register_mixer("mixed_head_attention", MixedHeadAttention)
register_mixer("latent_attention", LatentAttention)
