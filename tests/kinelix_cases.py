"""Small Kinelix configurations for the tests, their random weights, and the comparison of a
replayed trace with the plain implementation."""

from __future__ import annotations

import json
import tempfile
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

import plain_kinelix
from mercury_b200.config import config_from_dict
from mercury_b200.trace_run import replay
from mercury_b200.weights import random_tensors


def _mamba(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
            "norm_groups": norm_groups, "conv": conv}


def _delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _latent(heads, dim, vdim, rank, scale=None, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank,
             "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return mixer


def _moe(ff, experts, top, count=1, keep=1, scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "scale": scale,
                       "groups": {"count": count, "keep": keep}}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def _model(width, vocab, layers, eps=1e-6, scale=1.0, cap=0.0):
    return {"architecture": "Kinelix", "width": width, "vocab": vocab, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "logit_softcap": cap, "layers": layers}


RAW = {
    # every kind of layer and feed-forward, starting with a recurrence; a latent shared by a
    # later layer with other head sizes, a second latent of another rank behind it; groups of
    # three experts of which two groups are kept
    "mix": _model(64, 131, [
        _layer("mamba2", _mamba(4, 16, 24, 2, 2, 4), _moe(40, 6, 2, count=3, keep=2, scale=2.5)),
        _layer("latent_attention", _latent(4, 16, 24, 32, scale=0.4), _dense(80)),
        _layer("delta", _delta(4, 2, 24, 16, 3)),
        _layer("latent_attention", _latent(2, 32, 8, 32, scale=0.25, kv_from=1), _moe(24, 4, 3, scale=0.7)),
        _layer("mamba2", _mamba(2, 40, 16, 1, 4, 2), _dense(48)),
        _layer("latent_attention", _latent(3, 8, 16, 48)),
        _layer("latent_attention", _latent(5, 16, 8, 48, kv_from=5), _dense(32)),
    ], eps=1e-5, scale=2.0, cap=12.0),
    # values that may hide a fault when equal or 1: one head, one group, one norm group, one
    # tap, query/key heads as many as value heads, one expert of one, no cap, no scale
    "ones": _model(96, 77, [
        _layer("delta", _delta(3, 3, 16, 32, 1), _moe(64, 1, 1)),
        _layer("mamba2", _mamba(1, 32, 8, 1, 1, 1)),
        _layer("latent_attention", _latent(1, 24, 24, 24), _moe(16, 5, 5, count=5, keep=5)),
        _layer("delta", _delta(1, 1, 8, 8, 2), _dense(64)),
    ]),
    "only_mamba2": _model(48, 50, [_layer("mamba2", _mamba(6, 8, 20, 3, 3, 3))], cap=5.0),
    "only_delta": _model(48, 50, [_layer("delta", _delta(6, 2, 12, 20, 4))], scale=1.5),
    "only_latent": _model(48, 50, [_layer("latent_attention", _latent(5, 12, 20, 40, scale=0.5))]),
    "only_moe": _model(48, 50, [_layer("mamba2", _mamba(2, 8, 8, 1, 1, 2),
                                       _moe(56, 12, 4, count=4, keep=2, scale=1.7))]),
    # nothing a multiple of 8 (or of 4, where the design allows it)
    "odd": _model(100, 101, [
        _layer("latent_attention", _latent(3, 20, 12, 36, scale=0.3), _moe(34, 9, 2, count=3, keep=1)),
        _layer("mamba2", _mamba(6, 10, 18, 3, 5, 2), _dense(130)),
        _layer("delta", _delta(6, 3, 20, 12, 5)),
        _layer("latent_attention", _latent(7, 12, 20, 36, kv_from=0)),
    ], eps=1e-4, scale=0.5, cap=30.0),
    # sizes at the edges of what the kernels choose between: more heads than a decode tile
    # holds and exactly as many, a latent rank the tensor-core kernels refuse beside one they
    # take, matrices of 256 and of 192 rows, many experts in many groups, three experts in one
    "wide": _model(192, 300, [
        _layer("latent_attention", _latent(20, 16, 24, 64, scale=0.3), _moe(48, 64, 8, count=8, keep=4, scale=0.5)),
        _layer("mamba2", _mamba(4, 48, 256, 4, 4, 2), _dense(200)),
        _layer("delta", _delta(4, 2, 192, 48, 2)),
        _layer("latent_attention", _latent(3, 40, 8, 96)),
        _layer("latent_attention", _latent(20, 8, 8, 96, kv_from=3), _moe(40, 3, 2)),
        _layer("latent_attention", _latent(16, 16, 16, 64, kv_from=0)),
    ], scale=1.5, cap=25.0),
    # layer sizes of the order a real model has (few layers, a small vocabulary)
    "real": _model(512, 1000, [
        _layer("mamba2", _mamba(16, 64, 128, 2, 2, 4), _moe(256, 16, 4, count=4, keep=2, scale=2.0)),
        _layer("latent_attention", _latent(8, 64, 64, 128), _dense(1408)),
        _layer("delta", _delta(8, 4, 128, 128, 4), _moe(256, 16, 4, count=4, keep=2, scale=2.0)),
        _layer("latent_attention", _latent(8, 64, 64, 128, kv_from=1)),
    ], scale=4.0, cap=20.0),
}
SEED = {name: 41 + i for i, name in enumerate(RAW)}
SHARPEN = 3.0     # query-side projections are scaled so that attention is far from uniform


@lru_cache(maxsize=None)
def kinelix_model(name: str):
    """(raw config dictionary, typed config, {name: bfloat16 tensor})."""
    raw = RAW[name]
    _entry, config = config_from_dict(raw)
    tensors = random_tensors(config, SEED[name], torch.bfloat16, std=0.03 if name == "real" else 0.08)
    for key in tensors:
        if key.endswith(".mix.q") or key.endswith(".mix.uk"):
            tensors[key] = (tensors[key].float() * SHARPEN).to(torch.bfloat16)
    return raw, config, tensors


def random_tokens(count: int, vocab: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (count,), generator=gen).tolist()


@lru_cache(maxsize=None)
def requests_for(name: str, lengths: tuple) -> dict:
    return {f"r{i}": random_tokens(n, RAW[name]["vocab"], 500 + i) for i, n in enumerate(lengths)}


@lru_cache(maxsize=None)
def oracle(name: str, lengths: tuple) -> dict:
    raw, _config, tensors = kinelix_model(name)
    return {rid: plain_kinelix.forward(raw, tensors, tokens).numpy()
            for rid, tokens in requests_for(name, lengths).items()}


def make_runner(name, ops, device, dtype, page=16, num_tokens=512, poison=True, **more):
    from mercury_b200.engine.runner import ModelRunner

    _raw, config, tensors = kinelix_model(name)
    return ModelRunner(config=config, tensors=tensors, dtype=dtype, device=device, page_size=page,
                       num_pages=num_tokens // page, max_seqs=4, max_step_tokens=num_tokens,
                       max_model_len=num_tokens, ops=ops, poison_pages=poison, **more)


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
