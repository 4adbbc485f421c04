"""Fegenex on the CUDA kernels: every new kernel against its PyTorch twin, and the model
through the engine's step function, cache and state manager against the plain
implementation, in float32 and bfloat16."""

from __future__ import annotations

import json
import subprocess
import sys
from types import SimpleNamespace

import pytest
import torch

import replay_cases
from fegenex_cases import (RAW, fegenex_model, make_runner, replay_and_compare, requests_for,
                           tolerance_for)
from kernel_twins import TorchOps
from mercury_b200.parts.base import LayerCache

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]
IDS = ["f32", "bf16"]


@pytest.fixture(scope="module")
def ops():
    from mercury_b200.kernels.ops import CudaOps

    return CudaOps("cuda")


@pytest.fixture(scope="module")
def twin():
    return TorchOps(exact=True)


def rand(shape, dtype, seed, scale=1.0):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=gen) * scale).to(dtype).cuda()


def close(got, want, dtype, what="", tol32=3e-6, tol16=5e-3):
    tol = tol32 if dtype == torch.float32 else tol16
    scale = max(float(want.double().abs().max()), 1e-6)
    err = float((got.double() - want.double()).abs().max()) / scale
    assert torch.isfinite(got.float()).all(), f"{what}: non-finite"
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.0e}"


def ragged(q_lens, slots=None, pad=0):
    """A batch of sequences of `q_lens` new tokens (an empty one is allowed), `pad` padding
    rows behind them."""
    starts, seq_of = [0], []
    for s, n in enumerate(q_lens):
        starts.append(starts[-1] + n)
        seq_of += [s] * n
    seq_of += [-1] * pad
    dev = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return SimpleNamespace(num_seqs=len(q_lens), num_tokens=len(seq_of), q_start=dev(starts),
                           slots=dev(slots if slots is not None else list(range(len(q_lens)))),
                           seq_of_token=dev(seq_of), max_q_len=max(q_lens))


# ------------------------------------------------------------------------------ small kernels

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embed_with_positions(ops, twin, dtype):
    table, pos_table = rand((300, 136), dtype, 0), rand((50, 136), dtype, 1)
    ids = torch.randint(0, 300, (41,), dtype=torch.int32).cuda()
    positions = torch.randint(0, 50, (41,), dtype=torch.int32).cuda()
    got = torch.empty((41, 136), dtype=torch.float32, device="cuda")
    want = torch.empty_like(got)
    ops.embed(ids, table, got, positions=positions, position_table=pos_table)
    twin.embed(ids, table, want, positions=positions, position_table=pos_table)
    close(got, want, torch.float32, "embedding")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("delta_dtype", DTYPES, ids=["d32", "d16"])
@pytest.mark.parametrize("rows,cols,follow", [(1, 320, True), (9, 100, False), (300, 2048, True),
                                              (17, 4100, True)])
def test_rmsnorm_add(ops, twin, dtype, delta_dtype, rows, cols, follow):
    h = rand((rows, cols), torch.float32, 2)
    delta = rand((rows, cols), delta_dtype, 3, 5.0)
    w = (rand((1,), dtype, 4) + 1).expand(cols).contiguous()
    w2 = rand((cols,), dtype, 5) + 1 if follow else None
    h_want = h.clone()
    got = torch.empty((rows, cols), dtype=dtype, device="cuda") if follow else None
    want = torch.empty_like(got) if follow else None
    ops.rmsnorm_add(h, delta, w, 1e-5, w2, 1e-6, got)
    twin.rmsnorm_add(h_want, delta, w, 1e-5, w2, 1e-6, want)
    close(h, h_want, torch.float32, "stream")
    if follow:
        close(got, want, dtype, "next norm")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_gelu_gate(ops, dtype):
    from plain_fegenex import plain_gelu_tanh

    gate_up = rand((33, 2 * 72), dtype, 6, 2.0)
    got = torch.empty((33, 72), dtype=dtype, device="cuda")
    ops.gated_act(gate_up, got, 1)
    want = plain_gelu_tanh(gate_up[:, :72].double()) * gate_up[:, 72:].double()
    close(got, want, dtype, "gelu gate")


# ------------------------------------------------------------------------------ recurrences

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_mingru_scan_over_steps(ops, twin, dtype):
    """Three sequences in scattered slots over three steps of unequal portions (one of them
    absent from a step), padding rows behind; the state carries over."""
    width = 200
    state = rand((6, width), torch.float32, 7)
    state_want = state.clone()
    for step, q_lens in enumerate([(5, 1, 70), (1, 0, 2), (33, 2, 1)]):
        batch = ragged(q_lens, slots=[4, 0, 2], pad=3)
        pre = rand((batch.num_tokens, 3 * width), torch.float32, 10 + step, 2.0)
        got = torch.zeros((batch.num_tokens, width), dtype=dtype, device="cuda")
        want = torch.zeros_like(got)
        ops.mingru_scan(pre, state, batch, got)
        twin.mingru_scan(pre, state_want, batch, want)
        close(got, want, dtype, f"step {step}")
        close(state, state_want, torch.float32, f"state after step {step}")
    assert torch.equal(state[1], state_want[1]) and torch.equal(state[5], state_want[5])


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("width,blocks,taps", [(192, 3, 4), (96, 1, 1), (320, 2, 2), (130, 5, 7)])
def test_gated_recurrence_over_steps(ops, twin, dtype, width, blocks, taps):
    """Convolution, block gates and scan over steps whose portions are shorter and longer
    than the convolution's reach."""
    size = width // blocks
    state = torch.zeros((5, taps, width), dtype=torch.float32, device="cuda")
    state_want = state.clone()
    conv_w, conv_b = rand((width, taps), torch.float32, 20, 0.5), rand((width,), torch.float32, 21)
    gate_w = rand((2, blocks, size, size), torch.float32, 22, 0.2)
    gate_b = rand((2, blocks, size), torch.float32, 23)
    softplus_lam = torch.nn.functional.softplus(rand((width,), torch.float32, 24))
    for step, q_lens in enumerate([(1, 9), (2, 1), (1, 1), (40, 3), (1, 0)]):
        batch = ragged(q_lens, slots=[3, 1], pad=2)
        tokens = batch.num_tokens
        pre = rand((tokens, 2 * width), torch.float32, 30 + step)
        outs = []
        for which, st in ((ops, state), (twin, state_want)):
            u = torch.zeros((tokens, width), dtype=torch.float32, device="cuda")
            gates = torch.zeros((tokens, 2 * width), dtype=torch.float32, device="cuda")
            out = torch.zeros((tokens, width), dtype=dtype, device="cuda")
            which.causal_conv(pre, width, width, conv_w, conv_b, st, batch, u)
            which.block_gates(u, gate_w, gate_b, gates)
            which.gated_recurrence_scan(pre, u, gates, softplus_lam, 8.0, st, batch, out)
            outs.append((u, gates, out))
        live = batch.seq_of_token >= 0
        close(outs[0][0][live], outs[1][0][live], torch.float32, f"convolution, step {step}")
        close(outs[0][1][live], outs[1][1][live], torch.float32, f"gates, step {step}", 1e-5)
        close(outs[0][2][live], outs[1][2][live], dtype, f"output, step {step}", 2e-5)
        close(state, state_want, torch.float32, f"state after step {step}", 2e-5)


# ------------------------------------------------------------------------------ attention

MIXED_CASES = [
    # heads, kv heads, dim, vdim, rot, page, q_lens, kv_lens, window, mix
    (10, 5, 80, 40, 20, 16, (5, 1, 33), (5, 40, 33), 0, True),
    (4, 2, 32, 16, 16, 8, (1, 1, 1, 1), (1, 9, 24, 40), 0, True),
    (6, 1, 16, 40, 0, 16, (1, 17, 1), (300, 17, 64), 0, True),
    (3, 3, 24, 24, 8, 32, (40, 1, 2), (100, 77, 50), 24, True),
    (16, 4, 64, 80, 32, 16, (70, 2), (200, 66), 0, True),
    (5, 5, 20, 12, 12, 64, (31, 1), (31, 32), 0, False),
    (2, 1, 128, 256, 128, 16, (3, 1), (130, 257), 0, True),
    (12, 3, 48, 100, 2, 16, (1, 1), (1000, 513), 0, True),
    (64, 8, 16, 16, 4, 16, (3, 1), (20, 40), 0, True),
    (14, 2, 64, 64, 32, 16, (130, 1, 9), (130, 515, 300), 0, True),
    (12, 2, 128, 128, 64, 16, (70, 2), (200, 66), 50, True),
    (32, 4, 32, 32, 16, 8, (20, 1), (90, 33), 0, True),
    (7, 7, 16, 8, 0, 16, (17, 1, 1), (17, 100, 1), 0, False),
    # the remaining ways the tensor-core kernel divides heads over warps
    (24, 8, 32, 64, 16, 16, (33, 1), (70, 300), 0, True),
    (8, 2, 48, 48, 48, 16, (20, 2), (150, 66), 0, True),
    (6, 2, 32, 96, 8, 32, (18, 1), (100, 45), 30, True),
    (12, 4, 16, 24, 0, 16, (5, 40), (64, 40), 0, True),
]


def fill_pages(table, kv_lens, q_lens, n_kv, d, vd, page, num_pages, dtype, seed):
    k = torch.full((num_pages, n_kv, page, d), float("nan"), dtype=dtype, device="cuda")
    v = torch.full((num_pages, n_kv, page, vd), float("nan"), dtype=dtype, device="cuda")
    gen = torch.Generator().manual_seed(seed)
    for s, (q, kv) in enumerate(zip(q_lens, kv_lens)):
        for pos in range(kv - q):
            p = int(table[s, pos // page])
            if p >= 0:
                k[p, :, pos % page] = torch.randn((n_kv, d), generator=gen).to(dtype).cuda()
                v[p, :, pos % page] = torch.randn((n_kv, vd), generator=gen).to(dtype).cuda()
    return k, v


KERNELS = [("simt", torch.float32), ("simt", torch.bfloat16), ("mma", torch.bfloat16)]
KERNEL_IDS = ["f32", "bf16", "bf16-mma"]


def mma_takes(ops, heads, kv_heads, d, vd, width):
    return width % 8 == 0 and bool(ops.lib.mb_mixed_head_mma_supports(heads, kv_heads, d, vd))


@pytest.mark.parametrize("kernel,dtype", KERNELS, ids=KERNEL_IDS)
@pytest.mark.parametrize("splits", [1, 3, 7])
@pytest.mark.parametrize("case", range(len(MIXED_CASES)), ids=lambda i: f"case{i}")
def test_rotate_blend_store_and_attend(twin, kernel, dtype, splits, case):
    """`splits`: the keys of a row tile divided over that many blocks (some of them with no
    key at all when the sequence is short), merged afterwards."""
    from mercury_b200.kernels.ops import CudaOps
    from test_kernels_gpu import make_batch

    ops = CudaOps("cuda", decode_splits=splits)

    heads, kv_heads, d, vd, rot, page, q_lens, kv_lens, window, use_mix = MIXED_CASES[case]
    if kernel == "mma" and not mma_takes(ops, heads, kv_heads, d, vd, heads * d + kv_heads * (d + vd)):
        pytest.skip("sizes left to the CUDA-core kernel")
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 3
    batch, table = make_batch(q_lens, kv_lens, page, num_pages, pad_tokens=2, seed=case)
    k, v = fill_pages(table, kv_lens, q_lens, kv_heads, d, vd, page, num_pages, dtype, 40 + case)
    tokens = batch.num_tokens
    width = heads * d + kv_heads * d + kv_heads * vd
    qkv = rand((tokens, width), dtype, 50 + case)
    tables = None
    if rot:
        angle = torch.outer(torch.arange(max(kv_lens) + 1).double(),
                            10000.0 ** (-torch.arange(0, rot, 2).double() / rot))
        tables = (angle.cos().float().cuda(), angle.sin().float().cuda())
    first = rand((tokens, kv_heads * vd), dtype, 60 + case)
    c = torch.tensor([0.37], dtype=torch.float32, device="cuda")
    mix = (torch.eye(heads) + 0.3 * torch.randn(heads, heads)).float().cuda() if use_mix else None
    layout = (heads, kv_heads, d, vd)
    results = []
    for which in (ops, twin):
        rows, kk, vv = qkv.clone(), k.clone(), v.clone()
        keep = torch.zeros((tokens, kv_heads * vd), dtype=dtype, device="cuda")
        cache = LayerCache(kk, vv, page, table, True)
        which.rope_blend_store(rows, layout, tables, batch, cache, first, c, keep)
        out = torch.zeros((tokens, heads * vd), dtype=dtype, device="cuda")
        if which is ops:
            which.mixed_head_attention(rows, layout, batch, cache, d ** -0.5, window, mix, out,
                                       kernel=kernel)
        else:
            which.mixed_head_attention(rows, layout, batch, cache, d ** -0.5, window, mix, out)
        results.append((rows, kk, vv, keep, out))
    live = batch.seq_of_token >= 0
    got, want = results
    close(got[0][live], want[0][live], dtype, "rotated rows")
    for name, a, b in (("key pages", got[1], want[1]), ("value pages", got[2], want[2])):
        assert torch.equal(torch.isnan(a), torch.isnan(b)), f"{name}: other slots were written"
        close(torch.nan_to_num(a), torch.nan_to_num(b), dtype, name)
    assert torch.equal(got[3][live], qkv[live][:, -kv_heads * vd:]), "the kept values are the unblended ones"
    # the tensor-core kernel sums in another order: its bfloat16 result may land on the
    # neighbouring bfloat16 number (2^-7 of a value next to the largest)
    close(got[4][live], want[4][live], dtype, "attention", 2e-5, 8e-3 if kernel == "mma" else 5e-3)


@pytest.mark.parametrize("kernel,dtype", KERNELS, ids=KERNEL_IDS)
@pytest.mark.parametrize("far,kv_len,q_len", [(0, 700, 1), (3, 700, 5), (15, 321, 1), (16, 321, 2),
                                              (255, 700, 1), (256, 700, 40), (31, 33, 2)])
def test_one_far_key_stands_out(ops, kernel, dtype, far, kv_len, q_len):
    """One key far back (the first of the sequence, the last or first of a page or of a key
    tile) matches the queries of one head overwhelmingly: that head's own weights sit on it,
    and every head receives its share through the mixing matrix."""
    from test_kernels_gpu import make_batch

    heads, kv_heads, d, vd, page = 4, 2, 32, 16, 16
    num_pages = -(-kv_len // page) + 2
    batch, table = make_batch((q_len,), (kv_len,), page, num_pages, seed=far)
    k = rand((num_pages, kv_heads, page, d), dtype, 70, 0.1)
    v = rand((num_pages, kv_heads, page, vd), dtype, 71)
    qkv = rand((q_len, heads * d + kv_heads * (d + vd)), dtype, 72, 0.1)
    spike = torch.zeros(d, dtype=dtype, device="cuda")
    spike[5] = 30.0
    sharp_head = 1                       # reads key/value head 0
    k[int(table[0, far // page]), 0, far % page] = spike
    qkv[:, sharp_head * d:(sharp_head + 1) * d] = spike
    mix = torch.tensor([[1.0, 0.5, 0, 0], [0, 1.0, 0, 0], [0, -0.25, 1.0, 0], [0, 2.0, 0, 1.0]]).cuda()
    cache = LayerCache(k, v, page, table, False)
    out = torch.zeros((q_len, heads * vd), dtype=dtype, device="cuda")
    plain = torch.zeros_like(out)
    layout = (heads, kv_heads, d, vd)
    ops.mixed_head_attention(qkv, layout, batch, cache, 1.0, 0, mix, out, kernel=kernel)
    ops.mixed_head_attention(qkv, layout, batch, cache, 1.0, 0, None, plain, kernel=kernel)
    out, plain = out.float().view(q_len, heads, vd), plain.float().view(q_len, heads, vd)
    v_far = v[int(table[0, far // page]), :, far % page].float()          # [kv heads, vd]
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert (plain[:, sharp_head] - v_far[0]).abs().max() < tol
    for head in range(heads):
        want = mix[head, sharp_head] * v_far[head // 2] + \
            sum(mix[head, g] * plain[:, g] for g in range(heads) if g != sharp_head and g // 2 == head // 2)
        others = [g for g in range(heads) if g != sharp_head and g // 2 != head // 2 and mix[head, g] != 0]
        assert not others
        assert (out[:, head] - want).abs().max() < tol * 4, f"head {head}"


# ------------------------------------------------------------------------------ the model

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 150, 41, 90), "wide": (40, 300), "odd": (50, 7, 121, 33)}


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["only_mingru", "only_rglru", "only_attention", "only_ff"])
def test_each_layer_kind_alone(ops, dtype, name):
    lengths = (1, 2, 50)
    requests = requests_for(name, lengths)
    for builder in (replay_cases.whole, replay_cases.portions):
        steps, rows = builder(requests)
        replay_and_compare(make_runner(name, ops, "cuda", dtype), name, lengths, steps, rows,
                           tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["mix", "ones", "wide", "odd"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(ops, dtype, name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 512, seed=3) if mode == "mixed" else builder(requests)
    page = {"mix": 16, "ones": 8, "wide": 32, "odd": 4}[name]
    replay_and_compare(make_runner(name, ops, "cuda", dtype, page=page), name, lengths, steps, rows,
                       tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("mode", ["whole", "mixed"])
def test_real_layer_sizes(ops, dtype, mode):
    """Width 896, 14 heads over 2 groups of 64, feed-forward 4864, recurrences of 896 channels:
    the shapes at which the few-token, library and tensor-core kernels are chosen."""
    name, lengths = "real", (150, 40, 300, 17)
    requests = requests_for(name, lengths)
    steps, rows = (replay_cases.whole(requests) if mode == "whole"
                   else replay_cases.mixed(requests, 640, seed=5))
    replay_and_compare(make_runner(name, ops, "cuda", dtype, num_tokens=640), name, lengths, steps,
                       rows, tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_long_decoding_through_graphs(ops, dtype):
    """A short prompt and then 200 tokens one by one (replayed CUDA graphs in bfloat16 and
    float32 alike), over page borders and key tiles, logits wanted everywhere."""
    name, lengths = "mix", (230,)
    requests = requests_for(name, lengths)
    steps, rows = replay_cases.decode_tail(requests, tail=200)
    runner = make_runner(name, ops, "cuda", dtype, poison=False)
    replay_and_compare(runner, name, lengths, steps, rows, tolerance_for(dtype, name, lengths))
    assert runner.graph_replays > 100


def test_cut_does_not_change_float32_logits(ops):
    """The same request whole and in portions of two tokens: beyond rounding nothing moves."""
    import numpy as np
    from mercury_b200.engine.batch import StepEntry

    name = "mix"
    tokens = requests_for(name, (90,))["r0"]
    got = []
    for cut in (90, 2):
        runner = make_runner(name, ops, "cuda", torch.float32, poison=False, cuda_graphs=False)
        seq = runner.open("a")
        rows = []
        for at in range(0, 90, cut):
            part = tokens[at:at + cut]
            rows.append(runner.step([StepEntry(seq, part, list(range(len(part))))]).clone())
        got.append(torch.cat(rows).cpu().numpy())
    assert np.abs(got[0] - got[1]).max() <= 2e-5 * np.abs(got[0]).max()


def test_greedy_generation_through_the_engine_and_cli(ops, tmp_path):
    from mercury_b200 import Engine, EngineConfig, SamplingParams
    from mercury_b200.weights import write_random_model
    from test_fegenex_cpu import greedy

    name = "mix"
    raw, config, tensors = fegenex_model(name)
    runner = make_runner(name, ops, "cuda", torch.float32, num_tokens=256, poison=False)
    cfg = EngineConfig(model="(memory)", device="cuda", dtype="float32", block_size=16, num_blocks=16,
                       max_running=4, max_batched_tokens=256, prefill_chunk=24, max_model_len=256,
                       debug_invariants=True)
    engine = Engine(cfg, runner=runner)
    prompts = [requests_for(name, (37, 70, 20))[f"r{i}"] for i in range(3)]
    outs = engine.generate(prompts, SamplingParams(), 8)
    for prompt, out in zip(prompts, outs):
        assert out == greedy(raw, tensors, prompt, 8)
    # the command line on a model folder written by the random-weights mode
    folder = write_random_model(tmp_path / "model", config, seed=3)
    from safetensors.torch import load_file
    stored = load_file(str(folder / "model.safetensors"))
    done = subprocess.run(
        [sys.executable, "-m", "mercury_b200.generate", "--model", str(folder), "--dtype", "float32",
         "--prompt-ids", ",".join(map(str, prompts[2])), "--max-tokens", "5", "--num-blocks", "32",
         "--max-model-len", "128", "--max-running", "2", "--max-batched-tokens", "128"],
        capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert json.loads(done.stdout.strip().splitlines()[-1])["output_ids"] == greedy(raw, stored, prompts[2], 5)
