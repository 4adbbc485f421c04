"""Fegenex through the engine's step function, cache and state manager on the CPU (PyTorch
kernel twins) against the plain implementation: every layer kind alone, whole prompts,
prompts cut into portions down to two tokens, decoding token by token, mixed batches with
pages and state slots used again, and greedy generation through the engine."""

from __future__ import annotations

import pytest
import torch

import replay_cases
from fegenex_cases import RAW, fegenex_model, make_runner, replay_and_compare, requests_for
from kernel_twins import TorchOps
from plain_fegenex import plain_fegenex

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 150, 41, 90), "wide": (40, 70), "odd": (50, 7, 121, 33)}


@pytest.mark.parametrize("name", ["only_mingru", "only_rglru", "only_attention", "only_ff"])
def test_each_layer_kind_alone(name):
    lengths = (1, 2, 50)
    requests = requests_for(name, lengths)
    for builder in (replay_cases.whole, replay_cases.portions):
        steps, rows = builder(requests)
        replay_and_compare(make_runner(name, TorchOps(), "cpu", torch.float32), name, lengths,
                           steps, rows, 3e-5)


@pytest.mark.parametrize("name", ["mix", "ones", "wide", "odd"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 320, seed=3) if mode == "mixed" else builder(requests)
    replay_and_compare(make_runner(name, TorchOps(), "cpu", torch.float32, num_tokens=320),
                       name, lengths, steps, rows, 3e-5)


def test_config_round_trip_and_refusals():
    from mercury_b200.config import ConfigError, config_from_dict

    entry, config = config_from_dict(RAW["mix"])
    assert entry.name == "Fegenex" and config.to_dict() == RAW["mix"]
    assert config_from_dict(config.to_dict())[1] == config
    broken = config.to_dict()
    broken["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(ConfigError):
        config_from_dict(broken)
    broken = config.to_dict()
    broken["layers"][2]["type"] = "lstm"
    with pytest.raises(ConfigError):
        config_from_dict(broken)


def test_blend_source_must_come_first_and_match():
    """The first blending layer is the source: its own coefficient is not read, and the
    checkpoint may carry it or leave it out."""
    from mercury_b200.models.model import Model
    from mercury_b200.config import architecture_named

    _raw, config, tensors = fegenex_model("mix")
    model = Model(architecture_named("Fegenex").describe(config))
    names = {s.name for s in model.tensor_specs()}
    assert "l1.mix.vmix" not in names and "l3.mix.vmix" in names and "l5.mix.vmix" in names
    assert "l4.mix.vmix" not in names and "l1.mix.vmix" in model.optional_tensors()


def greedy(raw, tensors, prompt, count):
    tokens = list(prompt)
    for _ in range(count):
        logits, _ = plain_fegenex(raw, tensors, tokens)
        tokens.append(int(torch.argmax(logits[-1])))
    return tokens[len(prompt):]


def test_greedy_generation_through_the_engine():
    from mercury_b200 import Engine, EngineConfig, SamplingParams

    name = "mix"
    raw, config, tensors = fegenex_model(name)
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
    raw, config, tensors = fegenex_model(name)
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
