"""Kinelix on the CUDA kernels: every new kernel against its PyTorch twin, and the model
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
from kernel_twins import TorchOps
from kinelix_cases import (RAW, kinelix_model, make_runner, replay_and_compare, requests_for,
                           tolerance_for)
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


# ------------------------------------------------------------------------------ stream and logits

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_embed_with_a_scale(ops, twin, dtype):
    table = rand((300, 136), dtype, 0)
    ids = torch.randint(0, 300, (41,), dtype=torch.int32).cuda()
    got = torch.empty((41, 136), dtype=torch.float32, device="cuda")
    want = torch.empty_like(got)
    ops.embed(ids, table, got, scale=2.5)
    twin.embed(ids, table, want, scale=2.5)
    close(got, want, torch.float32, "embedding")


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("delta_dtype", DTYPES, ids=["d32", "d16"])
@pytest.mark.parametrize("center", [True, False], ids=["layer", "rms"])
@pytest.mark.parametrize("rows,cols,scaled,follow", [(1, 320, True, True), (9, 100, False, True),
                                                     (300, 2048, True, True), (17, 4100, True, False),
                                                     (5, 64, True, True)])
def test_scaled_add_norm(ops, twin, dtype, delta_dtype, center, rows, cols, scaled, follow):
    """A large common offset in the rows: a variance taken as E[x^2] - mean^2 would lose it."""
    h = rand((rows, cols), torch.float32, 2) + 40.0
    delta = rand((rows, cols), delta_dtype, 3, 5.0)
    scale = rand((cols,), dtype, 4) + 1 if scaled else None
    w = rand((cols,), dtype, 5) + 1 if follow else None
    h_want = h.clone()
    got = torch.empty((rows, cols), dtype=dtype, device="cuda") if follow else None
    want = torch.empty_like(got) if follow else None
    ops.scaled_add_norm(h, delta, scale, w, 1e-5, center, got)
    twin.scaled_add_norm(h_want, delta, scale, w, 1e-5, center, want)
    close(h, h_want, torch.float32, "stream")
    if follow:
        close(got, want, dtype, "norm", 2e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
def test_norm_of_picked_rows_leaves_the_stream(ops, twin, dtype):
    h = rand((40, 200), torch.float32, 6) * 3 - 7.0
    before = h.clone()
    rows = torch.tensor([39, 0, 17, 17, 5], dtype=torch.int32).cuda()
    w = rand((200,), dtype, 7) + 1
    got = torch.empty((5, 200), dtype=dtype, device="cuda")
    want = torch.empty_like(got)
    ops.scaled_add_norm(h, None, None, w, 1e-6, True, got, rows)
    twin.scaled_add_norm(before.clone(), None, None, w, 1e-6, True, want, rows)
    assert torch.equal(h, before)
    close(got, want, dtype, "picked rows", 2e-5)


def test_softcap(ops, twin):
    logits = rand((7, 333), torch.float32, 8, 20.0)
    want = logits.clone()
    ops.softcap(logits, 12.5)
    twin.softcap(want, 12.5)
    close(logits, want, torch.float32, "soft cap")
    assert float(logits.abs().max()) <= 12.5


# ------------------------------------------------------------------------------ state-space layers

STEPS = [(1, 9), (2, 1), (1, 1), (40, 3), (1, 0), (3, 70)]


@pytest.mark.parametrize("precise", [False, True], ids=["float", "double"])
@pytest.mark.parametrize("heads,vdim,n,groups,taps", [(4, 16, 24, 2, 4), (1, 32, 8, 1, 1), (6, 10, 18, 3, 2),
                                                      (3, 72, 130, 1, 5), (8, 64, 128, 2, 4)])
def test_convolution_and_mamba2_over_steps(ops, twin, precise, heads, vdim, n, groups, taps):
    """Steps whose portions are shorter and longer than the convolution's reach and than the
    scan's token tile, two sequences in scattered slots (one absent from a step), padding rows
    behind; matrices and convolution inputs carry over."""
    inner = heads * vdim
    channels = inner + 2 * groups * n
    proj = 2 * inner + 2 * groups * n + heads
    cells = heads * n * vdim
    state = torch.zeros((5, cells + (taps - 1) * channels), dtype=torch.float32, device="cuda")
    state_want = state.clone()
    conv_w, conv_b = rand((channels, taps), torch.float32, 20, 0.5), rand((channels,), torch.float32, 21)
    dt_bias, rate = rand((heads,), torch.float32, 22) - 1.0, -torch.exp(rand((heads,), torch.float32, 23, 0.5))
    skip = rand((heads,), torch.float32, 24) + 1
    for step, q_lens in enumerate(STEPS):
        batch = ragged(q_lens, slots=[3, 1], pad=2)
        tokens = batch.num_tokens
        pre = rand((tokens, proj), torch.float32, 30 + step)
        outs = []
        for which, st in ((ops, state), (twin, state_want)):
            xbc = torch.zeros((tokens, channels), dtype=torch.float32, device="cuda")
            y = torch.zeros((tokens, inner), dtype=torch.float32, device="cuda")
            which.conv_act(pre, inner, conv_w, conv_b, st[:, cells:], batch, xbc, "silu")
            which.conv_tail_update(pre, inner, channels, taps, st[:, cells:], batch)
            which.mamba2_scan(xbc, pre, proj - heads, dt_bias, rate, skip, (heads, vdim, n, groups),
                              st[:, :cells], batch, y, precise=precise)
            outs.append((xbc, y))
        live = batch.seq_of_token >= 0
        close(outs[0][0][live], outs[1][0][live], torch.float32, f"convolution, step {step}")
        close(outs[0][1][live], outs[1][1][live], torch.float32, f"output, step {step}", 1e-5)
        close(state, state_want, torch.float32, f"state after step {step}", 1e-5)
    assert not state[0].any() and not state[2].any() and not state[4].any()


@pytest.mark.parametrize("heads,vdim,n,groups", [(4, 16, 24, 2), (6, 64, 128, 3), (2, 40, 16, 1)])
def test_mamba2_long_portions_in_runs(ops, twin, heads, vdim, n, groups):
    """Portions long enough to be cut into runs that blocks walk side by side (a run that is
    full, one that is not, a sequence shorter than a run beside them), from a state that an
    earlier step left, against the sequential walk and the twin."""
    inner = heads * vdim
    channels = inner + 2 * groups * n
    proj = 2 * inner + 2 * groups * n + heads
    cells = heads * n * vdim
    dt_bias, rate = rand((heads,), torch.float32, 22) - 3.0, -torch.exp(rand((heads,), torch.float32, 23, 0.5))
    skip = rand((heads,), torch.float32, 24) + 1
    states = [rand((4, cells), torch.float32, 25, 0.5) for _ in range(3)]
    outs = []
    for step, q_lens in enumerate([(700, 3, 129), (1, 513, 2)]):
        batch = ragged(q_lens, slots=[2, 0, 3], pad=1)
        tokens = batch.num_tokens
        pre = rand((tokens, proj), torch.float32, 30 + step)
        xbc = rand((tokens, channels), torch.float32, 40 + step, 0.5)
        row = []
        for which, st, runs in ((ops, states[0], True), (ops, states[1], False), (twin, states[2], None)):
            if runs is not None:
                ops.scan_runs = runs
            y = torch.zeros((tokens, inner), dtype=torch.float32, device="cuda")
            which.mamba2_scan(xbc, pre, proj - heads, dt_bias, rate, skip, (heads, vdim, n, groups), st,
                              batch, y)
            row.append(y)
        ops.scan_runs = True
        live = batch.seq_of_token >= 0
        close(row[0][live], row[2][live], torch.float32, f"in runs, step {step}", 2e-5)
        close(row[1][live], row[2][live], torch.float32, f"sequential, step {step}", 2e-5)
        close(states[0], states[2], torch.float32, f"state in runs, step {step}", 2e-5)
        close(states[1], states[2], torch.float32, f"state, step {step}", 2e-5)


@pytest.mark.parametrize("precise", [False, True], ids=["float", "double"])
@pytest.mark.parametrize("heads,key_heads,dim,vdim,taps", [(4, 2, 24, 16, 3), (3, 3, 16, 32, 1), (6, 3, 20, 12, 5),
                                                           (2, 1, 130, 72, 2), (8, 4, 128, 128, 4),
                                                           (2, 2, 256, 20, 3), (1, 1, 100, 5, 2)])
def test_convolution_and_delta_rule_over_steps(ops, twin, precise, heads, key_heads, dim, vdim, taps):
    qk, inner = key_heads * dim, heads * vdim
    channels = 2 * qk + inner
    proj = channels + inner + 2 * heads
    cells = heads * dim * vdim
    state = torch.zeros((5, cells + (taps - 1) * channels), dtype=torch.float32, device="cuda")
    state_want = state.clone()
    conv_w = rand((channels, taps), torch.float32, 40, 0.5)
    dt_bias, rate = rand((heads,), torch.float32, 41) - 1.0, -torch.exp(rand((heads,), torch.float32, 42, 0.5))
    for step, q_lens in enumerate(STEPS):
        batch = ragged(q_lens, slots=[4, 0], pad=1)
        tokens = batch.num_tokens
        pre = rand((tokens, proj), torch.float32, 50 + step, 2.0)
        outs = []
        for which, st in ((ops, state), (twin, state_want)):
            qkv = torch.zeros((tokens, channels), dtype=torch.float32, device="cuda")
            o = torch.zeros((tokens, inner), dtype=torch.float32, device="cuda")
            which.conv_act(pre, 0, conv_w, None, st[:, cells:], batch, qkv, "silu")
            which.conv_tail_update(pre, 0, channels, taps, st[:, cells:], batch)
            which.delta_rule_scan(qkv, pre, channels + inner, channels + inner + heads, dt_bias, rate,
                                  (heads, key_heads, dim, vdim), 1e-6, st[:, :cells], batch, o,
                                  precise=precise)
            outs.append((qkv, o))
        live = batch.seq_of_token >= 0
        close(outs[0][0][live], outs[1][0][live], torch.float32, f"convolution, step {step}")
        close(outs[0][1][live], outs[1][1][live], torch.float32, f"output, step {step}", 2e-5)
        close(state, state_want, torch.float32, f"state after step {step}", 2e-5)


def test_the_read_out_sees_the_tokens_own_write(ops):
    """One head, beta = 1, no decay, an empty matrix: o = (k . q) v."""
    dim, vdim = 16, 8
    batch = ragged((1,))
    q, k, v = rand((dim,), torch.float32, 60), rand((dim,), torch.float32, 61), rand((vdim,), torch.float32, 62)
    qkv = torch.cat([q, k, v])[None].contiguous()
    pre = torch.tensor([[50.0, -50.0]], device="cuda")          # beta -> 1, softplus -> 0: g = 1
    state = torch.zeros((1, dim * vdim), dtype=torch.float32, device="cuda")
    o = torch.zeros((1, vdim), dtype=torch.float32, device="cuda")
    ops.delta_rule_scan(qkv, pre, 0, 1, torch.zeros(1, device="cuda"), -torch.ones(1, device="cuda"),
                        (1, 1, dim, vdim), 1e-6, state, batch, o)
    qn, kn = q / q.norm() * dim ** -0.5, k / k.norm()
    close(o[0], (kn @ qn) * v, torch.float32, "read-out", 1e-5)
    close(state.view(dim, vdim), torch.outer(kn, v), torch.float32, "matrix", 1e-5)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("groups,size,shared,first", [(2, 96, False, True), (6, 32, True, False),
                                                      (1, 40, False, True), (5, 12, True, False),
                                                      (3, 200, False, False), (2, 300, False, True),
                                                      (4, 256, True, False)])
def test_gated_group_norm(ops, twin, dtype, groups, size, shared, first):
    width = groups * size
    y = rand((19, width), torch.float32, 70, 3.0)
    pre = rand((19, width + 11), torch.float32, 71)
    w = rand((size if shared else width,), torch.float32, 72) + 1
    got = torch.empty((19, width), dtype=dtype, device="cuda")
    want = torch.empty_like(got)
    ops.gated_group_norm(y, pre, 7, w, groups, 1e-5, first, got)
    twin.gated_group_norm(y, pre, 7, w, groups, 1e-5, first, want)
    close(got, want, dtype, "gated group norm", 1e-5)


# ------------------------------------------------------------------------------ latent attention

LATENT_CASES = [
    # heads, rank, page, q_lens, kv_lens
    (4, 32, 16, (5, 1, 33), (5, 40, 33)),
    (6, 64, 16, (1, 1, 1, 1), (1, 9, 24, 700)),
    (3, 36, 4, (40, 1, 2), (100, 77, 50)),
    (16, 128, 32, (70, 2), (200, 66)),
    (1, 24, 8, (1, 17), (300, 17)),
    (5, 48, 16, (31, 1), (31, 32)),
    (8, 256, 16, (3, 1), (130, 257)),
    (2, 384, 16, (20, 1), (70, 90)),
    # sizes the tensor-core kernels take in bfloat16: decode-like rows (key ranges as a
    # cluster), prompt portions on tensor memory, portions in between, more heads than a
    # decode tile holds
    (8, 64, 16, (40, 3), (200, 66)),
    (4, 128, 16, (3, 1), (130, 257)),
    (20, 64, 16, (1, 1), (300, 90)),
    (4, 64, 8, (5, 2), (77, 300)),
    (14, 128, 16, (1, 1, 1), (515, 1, 64)),
]


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("splits", [1, 3, 7])
@pytest.mark.parametrize("case", range(len(LATENT_CASES)), ids=lambda i: f"case{i}")
def test_latent_store_and_attention_with_sinks(twin, dtype, splits, case):
    """The step's latent rows are normalised and stored (nothing else is written: the other
    slots hold NaN), then all heads attend over the one shared row per token, with a sink per
    head; key ranges with no key at all when the sequence is short."""
    from mercury_b200.kernels.ops import CudaOps
    from test_kernels_gpu import make_batch

    ops = CudaOps("cuda", decode_splits=splits)
    heads, rank, page, q_lens, kv_lens = LATENT_CASES[case]
    num_pages = sum(-(-kv // page) for kv in kv_lens) + 3
    batch, table = make_batch(q_lens, kv_lens, page, num_pages, pad_tokens=2, seed=case)
    pages = torch.full((num_pages, 1, page, rank), float("nan"), dtype=dtype, device="cuda")
    gen = torch.Generator().manual_seed(80 + case)
    for s, (q, kv) in enumerate(zip(q_lens, kv_lens)):
        for pos in range(kv - q):
            pages[int(table[s, pos // page]), 0, pos % page] = torch.randn(rank, generator=gen).to(dtype).cuda()
    tokens = batch.num_tokens
    pre = rand((tokens, 13 + rank), torch.float32, 90 + case, 2.0)
    w = rand((rank,), dtype, 91) + 1
    q = rand((tokens, heads * rank), dtype, 92 + case, 0.3)
    sinks = rand((heads,), torch.float32, 93, 2.0)
    results = []
    for which in (ops, twin):
        held = pages.clone()
        cache = LayerCache(held, held, page, table, True)
        which.latent_norm_store(pre, 13, rank, w, 1e-5, batch, cache)
        out = torch.zeros((tokens, heads * rank), dtype=dtype, device="cuda")
        which.paged_attention(q, heads, 1, rank, batch, cache, 0.2, 0, out, sinks=sinks)
        results.append((held, out))
    live = batch.seq_of_token >= 0
    (got_pages, got), (want_pages, want) = results
    assert torch.equal(torch.isnan(got_pages), torch.isnan(want_pages)), "other slots were written"
    close(torch.nan_to_num(got_pages), torch.nan_to_num(want_pages), dtype, "latent rows", 1e-5)
    # the tensor-core kernels sum in another order: a bfloat16 result may land on the
    # neighbouring bfloat16 number
    close(got[live], want[live], dtype, "attention", 2e-5, 8e-3)


@pytest.mark.parametrize("rank", [32, 64])
@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("far,kv_len,q_len", [(0, 700, 1), (3, 700, 5), (15, 321, 1), (16, 321, 2),
                                              (31, 700, 1), (32, 700, 40), (31, 33, 2), (255, 257, 1)])
def test_one_far_key_stands_out_and_a_sink_takes_its_share(ops, dtype, far, kv_len, q_len, rank):
    """One row far back (the first of the sequence, the last or first of a page or of a key
    tile) matches one head's queries overwhelmingly: without a sink that head returns the row
    itself; with a sink as large as the row's score it returns half of it."""
    from test_kernels_gpu import make_batch

    heads, page = 4, 16
    num_pages = -(-kv_len // page) + 2
    batch, table = make_batch((q_len,), (kv_len,), page, num_pages, seed=far)
    rows = rand((num_pages, 1, page, rank), dtype, 100, 0.1)
    q = rand((q_len, heads * rank), dtype, 101, 0.1)
    spike = torch.zeros(rank, dtype=dtype, device="cuda")
    spike[5] = 8.0
    rows[int(table[0, far // page]), 0, far % page] = spike
    q[:, rank:2 * rank] = spike                                   # head 1
    cache = LayerCache(rows, rows, page, table, False)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for sink, share in ((-1e4, 1.0), (32.0, 0.5)):
        sinks = torch.tensor([-1e4, sink, -1e4, 0.0], device="cuda")
        out = torch.zeros((q_len, heads * rank), dtype=dtype, device="cuda")
        ops.paged_attention(q, heads, 1, rank, batch, cache, 0.5, 0, out, sinks=sinks)
        got = out.float().view(q_len, heads, rank)[:, 1]
        assert (got - share * spike.float()).abs().max() < tol * 8.0, f"sink {sink}"


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("tokens,heads,cols,outs", [(1, 4, 16, 32), (7, 3, 20, 36), (33, 8, 64, 128),
                                                    (300, 2, 130, 9), (9, 16, 128, 200),
                                                    (300, 6, 64, 128), (515, 14, 128, 64)])
def test_head_linear(ops, twin, dtype, tokens, heads, cols, outs):
    x32 = rand((tokens, 8 + heads * cols), torch.float32, 110)
    w = rand((heads, cols, outs), dtype, 111, 0.2)
    for x, offset in ((x32, 8), (x32[:, 8:].to(dtype).contiguous(), 0)):
        got = torch.empty((tokens, heads * outs), dtype=dtype, device="cuda")
        want = torch.empty_like(got)
        ops.head_linear(x, offset, w, got)
        # from 256 tokens on the bfloat16 engine hands the rows to the library in bfloat16
        seen = x.to(dtype).to(x.dtype) if (dtype == torch.bfloat16 and tokens >= 256) else x
        twin.head_linear(seen, offset, w, want)
        close(got, want, dtype, "per-head product", 1e-5)


# ------------------------------------------------------------------------------ routed experts

@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("tokens,hidden,experts,top,count,keep", [(1, 64, 8, 2, 1, 1), (37, 100, 12, 4, 4, 2),
                                                                  (300, 256, 64, 6, 8, 3), (9, 48, 5, 5, 5, 5),
                                                                  (20, 40, 9, 2, 3, 1), (5, 32, 1, 1, 1, 1)])
def test_router(ops, twin, dtype, tokens, hidden, experts, top, count, keep):
    x = rand((tokens, hidden), dtype, 120)
    router = rand((experts, hidden), torch.float32, 121, 0.3)
    correction = rand((experts,), torch.float32, 122, 0.5)
    got_i = torch.zeros((tokens, top), dtype=torch.int32, device="cuda")
    got_w = torch.zeros((tokens, top), dtype=torch.float32, device="cuda")
    want_i, want_w = torch.zeros_like(got_i), torch.zeros_like(got_w)
    ops.route_experts(x, router, correction, count, keep, 1.7, got_i, got_w)
    twin.route_experts(x, router, correction, count, keep, 1.7, want_i, want_w)
    assert torch.equal(got_i, want_i)
    close(got_w, want_w, torch.float32, "weights", 1e-5)
    # the weight is the score without the correction; the chosen lie in at most `keep` groups
    s = torch.sigmoid(x.double() @ router.double().T)
    close(got_w, 1.7 * s.gather(1, got_i.long()), torch.float32, "weights are sigmoid * scale", 1e-5)
    groups_used = (got_i // (experts // count)).cpu()
    assert all(len(set(row.tolist())) <= keep for row in groups_used)


def test_the_correction_steers_the_choice_only(ops):
    """Two experts with equal router rows: the one with the larger correction is chosen, and
    its weight is the uncorrected score. A group whose single best expert beats everything
    loses to a group with two good ones."""
    x = rand((6, 32), torch.float32, 130)
    row = rand((32,), torch.float32, 131, 0.3)
    router = torch.stack([row, row, -row, -row]).contiguous()
    correction = torch.tensor([0.0, 0.01, 5.0, -5.0], device="cuda")
    chosen = torch.zeros((6, 1), dtype=torch.int32, device="cuda")
    weights = torch.zeros((6, 1), dtype=torch.float32, device="cuda")
    ops.route_experts(x, router, correction, 2, 1, 1.0, chosen, weights)
    s = torch.sigmoid(x @ row)
    # group 0 scores 2 s + 0.01, group 1 scores 2 (1 - s): group 1's best expert (choice
    # 1 - s + 5) would win everywhere if groups did not count
    for t in range(6):
        if 2 * float(s[t]) + 0.01 > 2 * (1 - float(s[t])):
            assert int(chosen[t, 0]) == 1 and abs(float(weights[t, 0]) - float(s[t])) < 1e-6
        else:
            assert int(chosen[t, 0]) == 2 and abs(float(weights[t, 0]) - (1 - float(s[t]))) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("tokens,hidden,ff,experts,top", [(1, 64, 40, 8, 2), (37, 100, 34, 6, 3),
                                                          (300, 256, 96, 16, 4), (70, 48, 130, 2, 2),
                                                          (9, 136, 64, 5, 1), (700, 128, 72, 12, 3)])
def test_expert_products(ops, twin, dtype, tokens, hidden, ff, experts, top):
    """Experts that get many rows, one row and none; sizes that fill no tile."""
    x = rand((tokens, hidden), dtype, 140)
    gate_up = rand((experts, 2 * ff, hidden), dtype, 141, 0.1)
    down = rand((experts, hidden, ff), dtype, 142, 0.1)
    gen = torch.Generator().manual_seed(143)
    chosen = torch.stack([torch.randperm(experts, generator=gen)[:top] for _ in range(tokens)])
    if experts > 2:
        chosen[chosen == 1] = 0 if top == 1 else chosen[chosen == 1]      # top 1: expert 1 gets nothing
    chosen = chosen.to(torch.int32).cuda()
    weights = rand((tokens, top), torch.float32, 144).abs()
    ctx = SimpleNamespace(buffer=lambda name, rows, cols, dtype=None: torch.empty(
        (rows, cols), device="cuda",
        dtype=(x.dtype if dtype is None else torch.float32 if dtype == "float32" else dtype)))
    got = torch.empty((tokens, hidden), dtype=torch.float32, device="cuda")
    want = torch.empty_like(got)
    ops.expert_feed_forward(x, chosen, weights, gate_up, down, got, ctx)
    twin.expert_feed_forward(x, chosen, weights, gate_up, down, want, ctx)
    close(got, want, dtype, "experts", 1e-5, 1e-2)


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("tokens", [40, 700])
def test_experts_that_get_no_row(ops, twin, dtype, tokens):
    """Only three of ten experts are ever chosen (the first, one in the middle, the last), in
    a step of few pairs and in one of many (where the bfloat16 engine takes the grouped
    product of the library): the others' empty ranges change nothing."""
    hidden, ff, experts, top = 64, 48, 10, 2
    x = rand((tokens, hidden), dtype, 150)
    gate_up = rand((experts, 2 * ff, hidden), dtype, 151, 0.1)
    down = rand((experts, hidden, ff), dtype, 152, 0.1)
    gen = torch.Generator().manual_seed(153)
    used = torch.tensor([0, 4, 9])
    chosen = torch.stack([used[torch.randperm(3, generator=gen)[:top]] for _ in range(tokens)])
    chosen = chosen.to(torch.int32).cuda()
    weights = rand((tokens, top), torch.float32, 154).abs()
    ctx = SimpleNamespace(buffer=lambda name, rows, cols, dtype=None: torch.empty(
        (rows, cols), device="cuda",
        dtype=(x.dtype if dtype is None else torch.float32 if dtype == "float32" else dtype)))
    got = torch.empty((tokens, hidden), dtype=torch.float32, device="cuda")
    want = torch.empty_like(got)
    ops.expert_feed_forward(x, chosen, weights, gate_up, down, got, ctx)
    twin.expert_feed_forward(x, chosen, weights, gate_up, down, want, ctx)
    close(got, want, dtype, "experts", 1e-5, 1e-2)


# ------------------------------------------------------------------------------ the model

LENGTHS = {"mix": (37, 70, 129, 45, 3, 66), "ones": (33, 64, 150, 41, 90), "odd": (50, 7, 121, 33),
           "wide": (40, 300, 17)}


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["only_mamba2", "only_delta", "only_latent", "only_moe"])
def test_each_layer_kind_alone(ops, dtype, name):
    lengths = (1, 2, 50)
    requests = requests_for(name, lengths)
    for builder in (replay_cases.whole, replay_cases.portions):
        steps, rows = builder(requests)
        replay_and_compare(make_runner(name, ops, "cuda", dtype), name, lengths, steps, rows,
                           tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("name", ["mix", "ones", "odd", "wide"])
@pytest.mark.parametrize("mode", ["whole", "decode_tail", "portions", "mixed"])
def test_replay(ops, dtype, name, mode):
    lengths = LENGTHS[name]
    requests = requests_for(name, lengths)
    builder = getattr(replay_cases, mode)
    steps, rows = builder(requests, 512, seed=3) if mode == "mixed" else builder(requests)
    page = {"mix": 16, "ones": 8, "odd": 4, "wide": 16}[name]
    replay_and_compare(make_runner(name, ops, "cuda", dtype, page=page), name, lengths, steps, rows,
                       tolerance_for(dtype, name, lengths))


@pytest.mark.parametrize("dtype", DTYPES, ids=IDS)
@pytest.mark.parametrize("mode", ["whole", "mixed"])
def test_real_layer_sizes(ops, dtype, mode):
    """Width 512, matrices of 128 x 64 per head, latents of 128, sixteen experts: the shapes
    at which the few-token, library and tensor-core kernels are chosen."""
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
    from test_kinelix_cpu import greedy

    name = "mix"
    raw, config, tensors = kinelix_model(name)
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
