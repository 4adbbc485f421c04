"""Small Fegenex configurations for the tests, their random weights, and the comparison of
a replayed trace with the plain implementation."""

from __future__ import annotations

import json
import tempfile
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

from mercury_b200.config import config_from_dict
from mercury_b200.trace_run import replay
from mercury_b200.weights import random_tensors
from plain_fegenex import plain_fegenex


def _attention(heads, kv_heads, dim, vdim, rot=None, v_mix=False, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
             "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix}
    if rot is not None:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    return mixer


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _model(width, vocab, layers, positions=1024, eps=1e-6):
    return {"architecture": "Fegenex", "width": width, "vocab": vocab, "max_positions": positions,
            "norm": {"eps": eps}, "layers": layers}


RAW = {
    # every kind of layer, in an order that starts with a recurrence; grouped heads, value
    # heads narrower and wider than key heads, rotation over part of a head, the whole head
    # and none; three blending layers; recurrent widths other than the model's
    "mix": _model(64, 131, [
        _layer("mingru", {"width": 96}, ff=112),
        _layer("attention", _attention(4, 2, 32, 16, rot=(16, 10000.0), v_mix=True, scale=0.3)),
        _layer("rglru", {"width": 48, "blocks": 3, "conv": 4}),
        _layer("attention", _attention(4, 2, 32, 16, rot=(32, 500.0), v_mix=True), ff=80),
        _layer("attention", _attention(6, 1, 16, 40, v_mix=False)),
        _layer("attention", _attention(2, 2, 48, 16, rot=(2, 77.0), v_mix=True), ff=40),
    ], positions=700, eps=1e-5),
    # one block, one tap, one key/value head; a single blending layer (a source only)
    "ones": _model(96, 77, [
        _layer("rglru", {"width": 96, "blocks": 1, "conv": 1}, ff=64),
        _layer("attention", _attention(3, 1, 24, 24, rot=(8, 1000000.0), v_mix=True)),
        _layer("mingru", {"width": 32}),
        _layer("rglru", {"width": 64, "blocks": 4, "conv": 2}),
    ], positions=640),
    "only_mingru": _model(48, 50, [_layer("mingru", {"width": 80})], positions=300),
    "only_rglru": _model(48, 50, [_layer("rglru", {"width": 64, "blocks": 2, "conv": 3})], positions=300),
    "only_attention": _model(48, 50, [_layer("attention", _attention(5, 5, 20, 12, rot=(12, 300.0)))],
                             positions=300),
    "only_ff": _model(48, 50, [_layer("mingru", {"width": 16}, ff=200)], positions=300),
    # many heads over few groups and wide heads (several row tiles per sequence)
    "wide": _model(128, 200, [
        _layer("attention", _attention(16, 4, 64, 80, rot=(32, 10000.0), v_mix=True), ff=256),
        _layer("attention", _attention(16, 4, 64, 80, rot=(64, 10000.0), v_mix=True)),
    ], positions=1200),
    # nothing a multiple of 8: width, vocabulary, head sizes, feed-forward, recurrent widths
    "odd": _model(100, 101, [
        _layer("rglru", {"width": 60, "blocks": 3, "conv": 2}),
        _layer("attention", _attention(3, 3, 20, 12, rot=(6, 123.0), v_mix=True), ff=130),
        _layer("mingru", {"width": 52}, ff=34),
        _layer("attention", _attention(6, 3, 20, 12, rot=(20, 9000.0), v_mix=True)),
    ], positions=333, eps=1e-4),
    # the layer sizes of a half-billion-parameter model (few layers, a small vocabulary)
    "real": _model(896, 1000, [
        _layer("attention", _attention(14, 2, 64, 64, rot=(32, 10000.0), v_mix=True), ff=4864),
        _layer("mingru", {"width": 896}),
        _layer("rglru", {"width": 896, "blocks": 7, "conv": 4}),
        _layer("attention", _attention(14, 2, 64, 64, rot=(32, 10000.0), v_mix=True), ff=4864),
    ], positions=1024),
}
SEED = {name: 11 + i for i, name in enumerate(RAW)}
SHARPEN = 3.0     # q and k projections are scaled so that attention is far from uniform


@lru_cache(maxsize=None)
def fegenex_model(name: str):
    """(raw config dictionary, typed config, {name: bfloat16 tensor})."""
    raw = RAW[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, SEED[name], torch.bfloat16, std=0.03 if name == "real" else 0.08)
    for key in tensors:
        if key.endswith(".mix.q") or key.endswith(".mix.k"):
            tensors[key] = (tensors[key].float() * SHARPEN).to(torch.bfloat16)
    return raw, config, tensors


def random_tokens(count: int, vocab: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=gen).tolist()


@lru_cache(maxsize=None)
def requests_for(name: str, lengths: tuple) -> dict:
    return {f"r{i}": random_tokens(n, RAW[name]["vocab"], 300 + i) for i, n in enumerate(lengths)}


@lru_cache(maxsize=None)
def oracle(name: str, lengths: tuple) -> dict:
    raw, _config, tensors = fegenex_model(name)
    return {rid: plain_fegenex(raw, tensors, tokens)[0].numpy()
            for rid, tokens in requests_for(name, lengths).items()}


def make_runner(name, ops, device, dtype, page=16, num_tokens=512, poison=True, **more):
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = fegenex_model(name)
    return ModelRunner(config=config, tensors=tensors, dtype=dtype, device=device, page_size=page,
                       num_pages=num_tokens // page, max_seqs=4, max_step_tokens=num_tokens,
                       max_model_len=min(num_tokens, RAW[name]["max_positions"]), ops=ops,
                       poison_pages=poison, **more)


def replay_and_compare(runner, name, lengths, steps, rows, tolerance) -> float:
    """Replays `steps`; every written row against the plain implementation's logits of the
    whole request. The error of a row is its largest difference over the request's largest
    logit. Returns the worst."""
    want = oracle(name, lengths)
    vocab = RAW[name]["vocab"]
    scale = {rid: float(np.abs(w).max()) for rid, w in want.items()}
    worst = 0.0
    with tempfile.TemporaryDirectory() as tmp:
        done = []
        replay(runner, [json.dumps(s) for s in steps], Path(tmp), done.append)
        assert done == [f"done {s['step']}" for s in steps]
        for step, expected in rows.items():
            if not expected:
                continue
            got = np.fromfile(Path(tmp) / f"{step}.f32", dtype="<f4").reshape(len(expected), vocab)
            for row, (rid, pos) in enumerate(expected):
                assert np.isfinite(got[row]).all(), f"step {step} {rid}@{pos}: non-finite logits"
                err = float(np.abs(got[row].astype(np.float64) - want[rid][pos]).max() / scale[rid])
                assert err <= tolerance, (f"step {step}: request {rid} position {pos}: relative "
                                          f"error {err:.3e} exceeds {tolerance:.0e}")
                worst = max(worst, err)
    assert not runner.cache.live
    runner.cache.check_invariants()
    assert runner.cache.leaked_pages() == 0
    return worst


@lru_cache(maxsize=None)
def bfloat16_bound(name: str, lengths: tuple) -> float:
    """What the bfloat16 engine may be off by on this model: twice what a bfloat16 twin of
    the plain implementation itself is off by (the PyTorch twins of the kernels, float32
    arithmetic, bfloat16 storage between them, whole prompts), and at least 1.5e-2."""
    import replay_cases
    from kernel_twins import TorchOps

    steps, rows = replay_cases.whole(requests_for(name, lengths))
    runner = make_runner(name, TorchOps(), "cpu", torch.bfloat16, poison=False)
    return max(1.5e-2, 2.0 * replay_and_compare(runner, name, lengths, steps, rows, 1.0))


def tolerance_for(dtype, name: str, lengths: tuple) -> float:
    return 3e-5 if dtype == torch.float32 else bfloat16_bound(name, lengths)
