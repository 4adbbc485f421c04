"""Kinelix through the engine's step function, cache and state manager on the CPU (PyTorch
kernel twins) against the plain implementation: every layer kind alone, whole prompts,
prompts cut into portions down to two tokens, decoding token by token, mixed batches with
pages and state slots used again, and greedy generation through the engine."""

from __future__ import annotations

import pytest
import torch

import plain_kinelix
import replay_cases
from kernel_twins import TorchOps
from kinelix_cases import RAW, kinelix_model, make_runner, replay_and_compare, requests_for

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 100, 41), "odd": (50, 7, 121, 33),
           "wide": (40, 90)}


@pytest.mark.parametrize("name", ["only_mamba2", "only_delta", "only_latent", "only_moe"])
def test_each_layer_kind_alone(name):
    lengths = (1, 2, 50)
    requests = requests_for(name, lengths)
    for builder in (replay_cases.whole, replay_cases.portions):
        steps, rows = builder(requests)
        replay_and_compare(make_runner(name, TorchOps(), "cpu", torch.float32), name, lengths,
                           steps, rows, 3e-5)


@pytest.mark.parametrize("name", ["mix", "ones", "odd", "wide"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 320, seed=5) if mode == "mixed" else builder(requests)
    replay_and_compare(make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=320),
                       name, lengths, steps, rows, 3e-5)


def test_config_round_trip_and_refusals():
    from mercury_b200.config import ConfigError, config_from_dict

    entry, config = config_from_dict(RAW["mix"])
    assert entry.name == "Kinelix" and config.to_dict() == RAW["mix"]
    assert config_from_dict(config.to_dict())[1] == config

    def broken(change):
        raw = config.to_dict()
        change(raw)
        with pytest.raises(ConfigError):
            config_from_dict(raw)

    broken(lambda r: r["layers"][2]["mixer"].update(kv_heads=3))           # 4 heads over 3
    broken(lambda r: r["layers"][0].update(type="lstm"))
    broken(lambda r: r["layers"][3]["mixer"].update(kv_from=2))            # not a latent layer
    broken(lambda r: r["layers"][3]["mixer"].update(kv_from=5))            # a later layer
    broken(lambda r: r["layers"][6]["mixer"].update(kv_from=3))            # a reader, no latent of its own
    broken(lambda r: r["layers"][3]["mixer"].update(kv_rank=16))           # another rank than its source
    broken(lambda r: r["layers"][0]["mlp"]["router"].update(top=5))        # more than the kept groups hold
    broken(lambda r: r["layers"][0]["mixer"].update(norm_groups=3))
    broken(lambda r: r["layers"][4]["mlp"].update(kind="sparse"))


def test_a_reader_has_no_down_projection_and_shares_the_cache_layer():
    from mercury_b200.config import architecture_named
    from mercury_b200.models.model import Model

    _raw, config, _tensors = kinelix_model("mix")
    spec = architecture_named("Kinelix").describe(config)
    model = Model(spec)
    names = {s.name for s in model.tensor_specs()}
    assert "l1.mix.dkv" in names and "l3.mix.dkv" not in names and "l3.mix.uk" in names
    assert "l5.mix.dkv.norm" in names and "l6.mix.dkv.norm" not in names
    assert spec.schedule[3].cache == spec.schedule[1].cache and not spec.schedule[3].writes_cache
    assert spec.schedule[6].cache == spec.schedule[5].cache != spec.schedule[1].cache
    assert len(model.cache_layers) == 2           # two latents are cached, four layers read them
    assert all(l.need.shared_values and l.need.num_kv_heads == 1 for l in model.cache_layers.values())
    assert not model.skips_cached_prefix          # recurrent state: every token has to be run


def greedy(raw, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits = plain_kinelix.forward(raw, tensors, tokens)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]


def test_greedy_generation_through_the_engine():
    from mercury_b200 import Engine, EngineConfig, SamplingParams

    name = "mix"
    raw, config, tensors = kinelix_model(name)
    runner = make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=256, poison=False)
    cfg = EngineConfig(model="(memory)", device="cpu", dtype="float32", block_size=16, num_blocks=16,
                       max_running=4, max_batched_tokens=256, prefill_chunk=24, max_model_len=256,
                       debug_invariants=True)
    engine = Engine(cfg, runner=runner)
    prompts = [requests_for(name, (37, 70, 20))[f"r{i}"] for i in range(3)]
    outs = engine.generate(prompts, SamplingParams(), 6)
    for prompt, out in zip(prompts, outs):
        assert out == greedy(raw, tensors, prompt, 6)
    assert engine.leaked_pages() == 0


def test_preempted_requests_start_again_from_an_empty_state():
    """A pool too small for all requests at once: the newest is put back (its pages and its
    state slot given up) and recomputed later in a slot that another request has used; the
    tokens stay the plain implementation's."""
    from mercury_b200 import Engine, EngineConfig, SamplingParams

    name = "ones"
    raw, config, tensors = kinelix_model(name)
    runner = make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=160, poison=True)
    cfg = EngineConfig(model="(memory)", device="cpu", dtype="float32", block_size=16, num_blocks=10,
                       max_running=4, max_batched_tokens=160, prefill_chunk=32, max_model_len=160,
                       debug_invariants=True)
    engine = Engine(cfg, runner=runner)
    prompts = [requests_for(name, (33, 64, 41, 50))[f"r{i}"] for i in range(4)]
    outs = engine.generate(prompts, SamplingParams(), 12)
    for prompt, out in zip(prompts, outs):
        assert out == greedy(raw, tensors, prompt, 12)
    assert engine.snapshot()["scheduler"]["preemptions"] > 0
    assert engine.leaked_pages() == 0
