"""The Kinelix decoder described in parts.

A token's row of the embedding table, times a constant, opens the stream. Every layer is a
pre-norm block with a learned scale per feature on each sublayer's output (layer norms with
a weight and no bias); its mixer is one of three kinds, chosen per layer by the
configuration: a Mamba-2 state-space layer, a gated delta rule, or attention over a cached
low-rank latent with a softmax sink and no positions. A latent-attention layer may read the
latent rows that an earlier layer caches instead of making its own. A layer's feed-forward
is a SiLU-gated dense one, a mixture of routed experts, or absent. A layer norm, an untied
head and a soft cap on the logits close the stack. Tensor names: `embed`,
`l<i>.norm1|norm2|ls1|ls2`, `l<i>.mix.*`, `l<i>.mlp.gate|up|down` or
`l<i>.mlp.e<j>.gate|up|down` with `l<i>.mlp.router|correction`, `final.norm`, `head`.
"""

from __future__ import annotations

from ..config.model_config import KinelixConfig, register_architecture
from ..parts.base import PartSpec
from .spec import LayerCall, ModelSpec

UNIT_EPS = 1e-6     # under the root when the delta rule's queries and keys are made unit vectors


def _mixer(config: KinelixConfig, index: int, layer: dict) -> PartSpec:
    prefix = f"l{index}.mix."
    kind, m = layer["type"], layer["mixer"]
    if kind == "mamba2":
        return PartSpec("mamba2", {
            "hidden_size": config.width, "heads": int(m["heads"]), "head_dim": int(m["vdim"]),
            "state_size": int(m["state"]), "groups": int(m["groups"]),
            "norm_groups": int(m["norm_groups"]), "taps": int(m["conv"]), "eps": config.norm_eps,
            "prefix": prefix})
    if kind == "delta":
        return PartSpec("gated_delta_rule", {
            "hidden_size": config.width, "heads": int(m["heads"]), "key_heads": int(m["kv_heads"]),
            "key_dim": int(m["dim"]), "head_dim": int(m["vdim"]), "taps": int(m["conv"]),
            "eps": config.norm_eps, "unit_eps": UNIT_EPS, "prefix": prefix})
    return PartSpec("latent_attention", {
        "hidden_size": config.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]),
        "value_dim": int(m["vdim"]), "rank": int(m["kv_rank"]), "scale": float(m["scale"]),
        "eps": config.norm_eps, "prefix": prefix, "own_latent": m.get("kv_from") is None})


def _feed_forward(config: KinelixConfig, index: int, mlp: dict) -> PartSpec:
    prefix = f"l{index}.mlp."
    if mlp["kind"] == "dense":
        return PartSpec("gated", {
            "hidden_size": config.width, "intermediate_size": int(mlp["ff"]), "prefix": prefix,
            "activation": "silu", "names": ("gate", "up", "down"), "float_out": True})
    router = mlp["router"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    return PartSpec("routed_experts", {
        "hidden_size": config.width, "intermediate_size": int(mlp["expert"]["ff"]),
        "experts": int(router["experts"]), "top": int(router["top"]),
        "route_scale": float(router["scale"]), "group_count": int(groups["count"]),
        "group_keep": int(groups["keep"]), "prefix": prefix})


def describe_kinelix(config: KinelixConfig) -> ModelSpec:
    def norm(name):
        return PartSpec("layernorm", {"size": config.width, "eps": config.norm_eps,
                                      "weight_name": name})

    blocks, schedule = [], []
    cache_of: dict[int, int] = {}      # layer that makes a latent -> its cache layer
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        params = {"hidden_size": config.width, "mixer": _mixer(config, index, layer),
                  "mixer_norm": norm(p + "norm1"), "mixer_scale": p + "ls1"}
        if layer["mlp"] is not None:
            params["feed_forward"] = _feed_forward(config, index, layer["mlp"])
            params["feed_forward_norm"] = norm(p + "norm2")
            params["feed_forward_scale"] = p + "ls2"
        blocks.append(PartSpec("pre_norm_layer_scale", params))
        if layer["type"] != "latent_attention":
            schedule.append(LayerCall(block=index))
            continue
        source = layer["mixer"].get("kv_from")
        if source is None:
            cache_of[index] = len(cache_of)
            schedule.append(LayerCall(block=index, cache=cache_of[index]))
        else:
            schedule.append(LayerCall(block=index, cache=cache_of[int(source)], writes_cache=False))
    return ModelSpec(
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=PartSpec("lookup", {"vocab_size": config.vocab, "hidden_size": config.width,
                                      "weight_name": "embed", "scale": config.embedding_scale}),
        blocks=blocks,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("linear_softcap", {"vocab_size": config.vocab, "hidden_size": config.width,
                                         "weight_name": "head", "cap": config.logit_softcap}),
    )


register_architecture("Kinelix", KinelixConfig, describe_kinelix)
