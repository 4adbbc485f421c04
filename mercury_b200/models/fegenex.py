"""The Fegenex decoder described in parts.

A token's row of the embedding table plus a learned position vector opens the stream.
Every layer is a block with a norm before and behind each sublayer (scalar-gain RMS
norms); its mixer is one of three kinds, chosen per layer by the configuration: attention
whose heads mix their softmax weights (rotary positions over the leading part of each
head, key and value heads of different sizes, values blended with those of the first
blending layer), a minGRU, or a gated linear recurrence behind a short convolution. A layer
may have a gelu-gated feed-forward or none. A scalar-gain norm and an untied head close
the stack. Tensor names: `embed`, `pos`, `l<i>.norm1|norm1b|norm2|norm2b`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down`, `final.norm`, `head`.
"""

from __future__ import annotations

from ..config.model_config import FegenexConfig, register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

VALUE_KEY = "first_values"     # under which the first blending layer leaves its values
DECAY_SCALE = 8.0              # log a = -DECAY_SCALE * r * softplus(lam)


def _mixer(config: FegenexConfig, index: int, layer: dict, blending_seen: bool) -> PartSpec:
    prefix = f"l{index}.mix."
    kind, m = layer["type"], layer["mixer"]
    if kind == "mingru":
        return PartSpec("mingru", {"hidden_size": config.width, "width": int(m["width"]),
                                   "prefix": prefix})
    if kind == "rglru":
        return PartSpec("gated_linear_recurrence", {
            "hidden_size": config.width, "width": int(m["width"]), "blocks": int(m["blocks"]),
            "taps": int(m["conv"]), "prefix": prefix, "decay_scale": DECAY_SCALE})
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    position = None
    if dims:
        position = PartSpec("rotary", {"head_dim": int(m["dim"]), "theta": float(rot["base"]),
                                       "rotary_dim": dims, "table_precision": "float64"})
    blend = None
    if m.get("v_mix"):
        blend = ("blend" if blending_seen else "source", VALUE_KEY)
    return PartSpec("mixed_head_attention", {
        "hidden_size": config.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
        "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]), "scale": float(m["scale"]),
        "prefix": prefix, "head_mix": True, "value_blend": blend,
        "window": int(m.get("window") or 0), "position_encoding": position})


def describe_fegenex(config: FegenexConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("rmsnorm_scalar", {"size": config.width, "eps": config.norm_eps,
                                           "weight_name": name})

    blocks, schedule = [], []
    blending_seen = False
    cache_layers = 0
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        params = {"mixer": _mixer(config, index, layer, blending_seen),
                  "mixer_norm": norm(p + "norm1"), "mixer_post_norm": norm(p + "norm1b")}
        if layer["type"] == "attention" and layer["mixer"].get("v_mix"):
            blending_seen = True
        if layer["mlp"] is not None:
            params["feed_forward"] = PartSpec("gated", {
                "hidden_size": config.width, "intermediate_size": int(layer["mlp"]["ff"]),
                "prefix": p + "mlp.", "activation": "gelu_tanh", "names": ("gate", "up", "down")})
            params["feed_forward_norm"] = norm(p + "norm2")
            params["feed_forward_post_norm"] = norm(p + "norm2b")
        blocks.append(PartSpec("sandwich_norm", params))
        if layer["type"] == "attention":
            schedule.append(LayerCall(block=index, cache=cache_layers))
            cache_layers += 1
        else:
            schedule.append(LayerCall(block=index))
    # a source layer's own blend coefficient is in the checkpoint although nothing reads it
    optional = tuple(f"l{i}.mix.vmix" for i, l in enumerate(config.layers) if l["type"] == "attention")
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=PartSpec("lookup_learned_positions", {
            "vocab_size": config.vocab, "hidden_size": config.width, "weight_name": "embed",
            "position_name": "pos", "max_positions": config.max_positions}),
        blocks=blocks,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": config.vocab, "hidden_size": config.width,
                                 "weight_name": "head"}),
        optional_tensors=optional,
    )


register_architecture("Fegenex", FegenexConfig, describe_fegenex)
