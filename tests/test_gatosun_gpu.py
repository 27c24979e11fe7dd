"""The Gatosun design on a GPU: each new kernel and kernel option against its plain reference, the model against the plain
implementation (tests/plain_gatosun.py) whole, decoded, cut into portions, in unequal batches, in slots, pages and state
rows used before, and through the engine's own entry point with greedy generation. The tests make their own small
configurations (tests/helpers_gatosun.py) and weights; where random weights would hide a fault (a key at the window's edge,
a key far back, a correction that reorders the experts), weights or inputs are made so that it shows."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import kernel_refs as refs
from tests import plain_gatosun as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_gatosun import CONFIGS, GAT_FAST, GAT_ODD, GAT_ONES, attention, config, dense, gla, layer, make_model_dir, moe, parallel

pytestmark = pytest.mark.gpu
DEV = "cuda"
BOTH = [torch.float32, torch.bfloat16]


def close(got, want, dtype, what="", f32=3e-5, bf16=3e-2):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max()) + 1e-9
    bound = (f32 if dtype == torch.float32 else bf16) * scale
    err = float((got - want).abs().max())
    assert err <= bound, f"{what}: max |diff| {err:.3e} exceeds {bound:.3e}"


def expect(cfg, weights, tokens, margin=0.02):
    """The plain implementation's logits, and which rows' routers chose by a clear margin in every layer: in bfloat16 a router
    whose two candidates (experts or groups) are closer than the rounding of its input may choose the other one, and such a
    row says nothing about the kernels."""
    margins = []
    logits = plain.forward(cfg, weights, tokens, margins=margins)
    sure = torch.ones(len(tokens), dtype=torch.bool)
    for m in margins:
        sure &= m >= margin
    return logits, sure


def logits_close(got, want, dtype, what=""):
    """The difference with its mean taken off, root mean square over the vocabulary, against the spread of the logits.
    `want`: logits, or (logits, rows whose routers chose by a clear margin)."""
    want, sure = want if isinstance(want, tuple) else (want, torch.ones(want.shape[0], dtype=torch.bool))
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = d.square().mean(-1).sqrt() / want.std(-1)
    if dtype == torch.float32:
        assert float(err.max()) <= 1e-4, f"{what}: worst row {float(err.max()):.3e} exceeds 1e-4"
    else:   # the typical row within rounding, and no row lost: a wrong key, a mask one position off or a lost state moves
        # every later row by about its whole spread, which the median sees; among the rows whose routers were sure hardly
        # one may stand out (a token before it whose router was not sure reaches it through keys and states)
        assert int(sure.sum()) >= max(1, len(sure) // 2), f"{what}: too few rows with a sure router to judge by"
        far = float((err[sure] > 0.4).double().mean())
        assert float(err.median()) <= 0.05 and far <= 0.015 and float(err.max()) <= 1.5, \
            f"{what}: median {float(err.median()):.3e}, {far:.1%} of the sure rows over 0.4, worst {float(err.max()):.3e}"


def rand(g, *shape, dtype=torch.float32, spread=1.0):
    return (spread * torch.randn(*shape, generator=g)).to(dtype).to(DEV)


def ints(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


class Batch:
    """The integers of a step of sequences with the given slots and (start, length) spans."""

    def __init__(self, slots, spans):
        self.slots, self.n_seqs = ints(slots), len(slots)
        cu, seq, pos = [0], [], []
        for s, (start, length) in enumerate(spans):
            cu.append(cu[-1] + length)
            seq += [s] * length
            pos += list(range(start, start + length))
        self.cu_q, self.tok_seq, self.tok_pos, self.n_tokens = ints(cu), ints(seq), ints(pos), cu[-1]


# ------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("width", [45, 384, 1500])
def test_outputs_enter_the_stream_under_a_factor_each(dtype, width):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(width)
    hidden = rand(g, 19, width, spread=3.0)
    a, b, w = rand(g, 19, width, dtype=dtype), rand(g, 19, width, dtype=dtype), (1 + 0.1 * torch.randn(width, generator=g)).to(dtype).to(DEV)
    for second in (b, None):
        h_ref, h_got = hidden.clone().cpu(), hidden.clone()
        out_ref, out = torch.empty(19, width, dtype=dtype), torch.empty(19, width, dtype=dtype, device=DEV)
        refs.add_rms_norm_scaled(h_ref, a.cpu(), 0.7, None if second is None else second.cpu(), -1.3, w.cpu(), 1e-5, out_ref)
        ops.add_rms_norm_scaled(h_got, a, 0.7, second, -1.3, w, 1e-5, out)
        close(h_got, h_ref, torch.float32, "stream")
        close(out, out_ref, dtype, "normed", bf16=1e-2)
        h_got2 = hidden.clone()
        ops.residual_add_scaled(h_got2, a, 0.7, second, -1.3)
        assert torch.equal(h_got2, h_got)   # the same order of operations with and without the norm


@pytest.mark.parametrize("dtype", BOTH)
def test_norms_over_runs_of_columns_and_rows_drawn_towards_other_rows(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(3)
    x = rand(g, 23, 100, dtype=dtype, spread=2.0)
    wq, wk = rand(g, 42, dtype=dtype), rand(g, 18, dtype=dtype)
    x[:, 30:42] = 0   # columns of padding inside the first run: they hold zeros and do not count
    want = x.clone().cpu()
    refs.rms_norm_cols(want, ((0, 42, 30, wq.cpu()), (42, 18, 18, wk.cpu())), 1e-5)
    ops.rms_norm_cols(x, ((0, 42, 30, wq), (42, 18, 18, wk)), 1e-5)
    close(x, want, dtype, "runs", bf16=1e-2)
    assert torch.equal(x[:, 60:].cpu(), want[:, 60:])
    other = rand(g, 23, 50, dtype=dtype)
    mine, want = x[:, 60:96], x[:, 60:96].clone().cpu()
    refs.mix_rows(want, other.cpu()[:, 5:45], 3, 7, 12, 10, 0.3)
    ops.mix_rows(mine, other[:, 5:45], 3, 7, 12, 10, 0.3)
    close(mine, want, dtype, "mixed", bf16=1e-2)


@pytest.mark.parametrize("dtype", BOTH)
def test_biases_row_norms_and_value_mixing_in_one_launch(dtype):
    """The one kernel behind a q | k | v product against the steps it stands for; heads of q and k padded beyond their size."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(4)
    n, q_w, kv_w = 21, 48, 24                      # 4 heads of 12 (10 used), 2 kv heads of 12 (values: 7 used)
    x = rand(g, n, q_w + 2 * kv_w + 5, dtype=dtype, spread=2.0)
    pad = torch.zeros(q_w + 2 * kv_w, dtype=torch.bool)
    for h in range(6):
        pad[h * 12 + 10:h * 12 + 12] = True
    for h in range(2):
        pad[q_w + kv_w + h * 12 + 7:q_w + kv_w + (h + 1) * 12] = True
    x[:, :q_w + 2 * kv_w][:, pad.to(DEV)] = 0
    bias = rand(g, q_w + 2 * kv_w, dtype=dtype)
    bias[pad.to(DEV)] = 0
    wq, wk, other = rand(g, q_w, dtype=dtype), rand(g, kv_w, dtype=dtype), rand(g, n, 30, dtype=dtype)
    for with_bias in (True, False):
        for mix in (None, (2, other[:, 3:], 7, 12, 9, 0.35)):
            b = (lambda lo, hi: bias[lo:hi]) if with_bias else (lambda lo, hi: None)
            cpu = lambda t: None if t is None else t.cpu()
            runs = [(0, q_w, 40, b(0, q_w), wq), (q_w, kv_w, 20, b(q_w, q_w + kv_w), wk), (q_w + kv_w, kv_w, 0, b(q_w + kv_w, q_w + 2 * kv_w), None)]
            got, want = x.clone(), x.clone().cpu()
            ops.rows_prepare(got, runs, 1e-5, mix)
            refs.rows_prepare(want, [(c, w, k, cpu(bb), cpu(ww)) for c, w, k, bb, ww in runs], 1e-5,
                              None if mix is None else (mix[0], mix[1].cpu(), *mix[2:]))
            close(got, want, dtype, f"bias {with_bias} mix {mix is not None}", bf16=1.6e-2)
            assert torch.equal(got[:, q_w + 2 * kv_w:], x[:, q_w + 2 * kv_w:])


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("k,n", [(44, 14), (128, 64)])
def test_activation_in_the_experts_first_product(dtype, k, n):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(k)
    x, router, weight = rand(g, 50, k, dtype=dtype), rand(g, 6, k, dtype=dtype), rand(g, 6, n, k, dtype=dtype, spread=k ** -0.5)
    plan = ops.moe_plan(None, 2, x=x, router=router)
    plain_out, out = torch.empty(100, n, dtype=dtype, device=DEV), torch.empty(100, n, dtype=dtype, device=DEV)
    ops.expert_linear(x, weight, plan, plain_out, gather=True)
    ops.expert_linear(x, weight, plan, out, gather=True, activation="relu2")
    want = torch.relu(plain_out.float()) ** 2
    close(out, want, dtype, "relu2 behind the product", f32=1e-6, bf16=1e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("inter", [30, 256])
def test_gated_activation_with_biases(dtype, inter):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(inter)
    gu, bias = rand(g, 17, 2 * inter, dtype=dtype, spread=2.0), rand(g, 2 * inter, dtype=dtype)
    for kind in ("gelu_tanh", "silu", "relu2"):
        for b in (bias, None):
            out, want = torch.empty(17, inter, dtype=dtype, device=DEV), torch.empty(17, inter, dtype=dtype)
            ops.bias_glu(gu, b, kind, out)
            refs.bias_glu(gu.cpu(), None if b is None else b.cpu(), kind, want)
            close(out, want, dtype, kind, bf16=1e-2)
    low, want = torch.empty(17, 2 * inter, dtype=dtype, device=DEV), torch.empty(17, 2 * inter, dtype=dtype)
    ops.bias_act(gu, None, "tanh", low)
    refs.bias_act(gu.cpu(), None, "tanh", want)
    close(low, want, dtype, "tanh", bf16=1e-2)


@pytest.mark.parametrize("dtype", BOTH)
def test_token_shift_into_several_mixes_keeps_the_last_row(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(5)
    width, n_mixes = 44, 5
    mu = torch.rand(n_mixes, width, generator=g).to(DEV)
    state, state_ref = torch.zeros(4, 10 + width, device=DEV), torch.zeros(4, 10 + width)
    state[2, 10:] = state_ref[2, 10:] = 1.5   # a slot that a sequence has used before this step
    # a step of portions (one sequence without a slot), then a step of single tokens in the same slots
    for spans, slots, single in (([(0, 7), (3, 1), (0, 12)], [1, 2, -1], False), ([(7, 1), (4, 1)], [1, 2], True)):
        b = Batch(slots, spans)
        h = rand(g, b.n_tokens, width, dtype=dtype)
        out, want = torch.empty(b.n_tokens, n_mixes * width, dtype=dtype, device=DEV), torch.empty(b.n_tokens, n_mixes * width, dtype=dtype)
        ops.shift_mix(h, mu, b.cu_q, b.tok_seq, b.slots, state, 10, out, single=single)
        refs.shift_mix(h.cpu(), mu.cpu(), b.cu_q.cpu(), b.tok_seq.cpu(), b.slots.cpu(), state_ref, 10, want, single=single)
        close(out, want, dtype, f"mixes {spans}", bf16=1e-2)
        assert torch.equal(state.cpu(), state_ref)


def test_decays_per_channel():
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(6)
    pre, bias = rand(g, 33, 50, spread=3.0), rand(g, 50)
    for kind, tau in (("double_exp", 1.0), ("sigmoid_root", 16.0), ("sigmoid_root", 1.0)):
        out, want = torch.empty(33, 50, device=DEV), torch.empty(33, 50)
        ops.channel_decay(pre[:, :50], bias, kind, out, tau=tau)
        refs.channel_decay(pre.cpu(), bias.cpu(), kind, want, tau=tau)
        assert max_err(out, want) < 1e-6, kind


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,dim,vdim", [(3, 10, 6), (2, 32, 64), (2, 64, 64), (1, 130, 20), (2, 8, 8)])
@pytest.mark.parametrize("bonus", [False, True])
def test_scan_with_a_decay_per_state_row(dtype, heads, dim, vdim, bonus):
    """Portions, single tokens and a sequence without a slot in one step; the state rows of a slot used before; the cut
    changes no bit of the output."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(dim)
    size = heads * dim * vdim
    u = rand(g, heads, dim) if bonus else None

    def step(state, batch, q, k, v, w, on_gpu):
        y = torch.empty(q.shape[0], heads * vdim, device=q.device)
        fn = ops.outer_state_scan_rows if on_gpu else refs.outer_state_scan_rows
        fn(q, k, v, w, batch.cu_q if on_gpu else batch.cu_q.cpu(), batch.slots if on_gpu else batch.slots.cpu(), state, 5, heads, dim,
           vdim, 0.5, y, bonus=u if on_gpu or u is None else u.cpu())
        return y

    n = 75
    q, k, v = (rand(g, n, heads * d, dtype=dtype) for d in (dim, dim, vdim))
    w = torch.rand(n, heads * dim, generator=g).pow(0.2).to(DEV)
    state, state_ref = torch.zeros(3, 5 + size + 3, device=DEV), torch.zeros(3, 5 + size + 3)
    whole = Batch([1], [(0, n)])
    y = step(state, whole, q, k, v, w, True)
    y_ref = step(state_ref, whole, q.cpu(), k.cpu(), v.cpu(), w.cpu(), False)
    close(y, y_ref, torch.float32, "whole", f32=2e-5)
    close(state, state_ref, torch.float32, "state", f32=2e-5)
    assert float(state[:, :5].abs().max()) == 0 and float(state[:, 5 + size:].abs().max()) == 0
    # the same sequence in portions and single tokens, in a slot used before (zeroed as the cache does), beside another sequence
    state2 = state.clone()
    state2[2].zero_()
    at, pieces = 0, []
    for length in (33, 1, 1, 38, 2):
        both = Batch([2, -1], [(at, length), (0, 3)])
        rows = list(range(at, at + length)) + [0, 1, 2]
        pieces.append(step(state2, both, q[rows], k[rows], v[rows], w[rows], True)[:length])
        at += length
    assert torch.equal(torch.cat(pieces), y)
    assert torch.equal(state2[2], state[1]) and torch.equal(state2[1], state[1])


@pytest.mark.parametrize("dtype", BOTH)
def test_choice_among_groups_under_a_correction(dtype):
    """The correction reorders the experts without touching the weights; the best expert of a group that is not kept cannot
    be chosen although its score is the largest; choice scores below zero stay above an expert that is shut out."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(8)
    n, experts, top, width = 40, 12, 3, 32
    x, router = rand(g, n, width, dtype=dtype), rand(g, experts, width, dtype=dtype, spread=0.5)
    correction = torch.tensor([-3.0, -2.5, -2.8, -2.6, 0.1, 0.0, 0.2, -0.1, 0.6, -4.0, -4.0, -4.0], device=DEV)
    for groups in ((3, 2), (4, 1), (1, 1), (12, 3), None):
        logits = (x.float() @ router.float().T)
        want = refs.moe_plan(logits.cpu(), top, correction=correction.cpu(), groups=groups)
        for fused in (True, False):
            plan = ops.moe_plan(None if fused else logits, top, x=x if fused else None, router=router if fused else None,
                                correction=correction, groups=groups)
            for t in range(n):
                rows_got, rows_want = plan.dest[t * top:(t + 1) * top].long().cpu(), want.dest[t * top:(t + 1) * top].long()
                offsets = plan.offsets.cpu()
                experts_got = sorted(int(torch.searchsorted(offsets, r, right=True)) - 1 for r in rows_got)
                assert experts_got == sorted(want.row_expert[rows_want].tolist()), (groups, fused, t)
                assert max_err(plan.sorted_weight.cpu()[rows_got].sort().values, want.sorted_weight[rows_want].sort().values) < 1e-5
    # the first group holds the largest scores; its correction pushes all its choice scores below zero, and with two of
    # three groups kept none of its experts is chosen
    logits = torch.zeros(1, experts)
    logits[0, :4] = 4.0
    plan = ops.moe_plan(logits.to(DEV), top, correction=correction, groups=(3, 2))
    assert int(plan.offsets.cpu()[4]) == 0


# ------------------------------------------------------------------ the model
def build(cfg, folder, dtype, seed=0, weights=None):
    """The model on the GPU and the weights it holds: in bfloat16 the plain implementation gets the rounded weights, so
    that the comparison sees the arithmetic and not the rounding of the file."""
    from qwenforge_b200.engine import Model
    weights = plain.random_weights(cfg, seed) if weights is None else weights
    if dtype == torch.bfloat16:
        weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    folder, weights = make_model_dir(cfg, seed, folder, weights=weights)
    return Model.from_dir(folder, dtype, DEV), weights, folder


def run(model, cache, tokens, cuts):
    """One sequence fed in portions of the given sizes (the rest one by one); the logits of every position."""
    slot, at, got = cache.open(), 0, []
    for size in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        got.append(model.step(cache, [(slot, tokens[at:at + size])], want=[list(range(size))]))
        at += size
    cache.close(slot)
    model.raise_on_kernel_error()
    return torch.cat(got)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_and_portions_agree_with_the_plain_implementation(dtype, name, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, dtype)
    cache = model.new_cache(64 * 12, 3)
    tokens = random_tokens(cfg["vocab"], 300, 7)
    want = expect(cfg, weights, tokens)
    for cuts in ([300], [260], [2, 61, 2, 130, 65, 3, 2], [129, 128]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"{name} cuts {cuts[:3]}")
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


GAT_LONG = config(1000, 320, 1e-6, 0.5, [
    layer(parallel(10, 2, 64, 64, 300, 64, 5, 64, 0.9, 0.8, 300000.0, 0.125, rank=24), dense(640)),
    layer(attention(10, 2, 80, 48, 80, 150000.0, v_mix=True), moe(12, 3, 96, groups=(4, 2), shared=160)),
    layer(gla(5, 64, 128, tau=16.0, rank=16), moe(20, 4, 48, groups=(5, 3))),
    layer(attention(8, 2, 128, 48, 64, 10000.0, v_mix=True), moe(12, 3, 96, shared=160)),
    layer(parallel(4, 4, 128, 128, 520, 128, 2, 128, 1.1, 0.6, 1000.0, 0.09, rank=8), None),
])


@pytest.mark.parametrize("dtype", BOTH)
def test_long_prompts_at_larger_sizes(dtype, tmp_path):
    """Steps of more than a thousand tokens: whole, with the last tokens decoded, and cut where the later portions reach back
    over many pages."""
    cfg, n = GAT_LONG, 1400
    model, weights, _ = build(cfg, tmp_path, dtype, seed=11)
    cache = model.new_cache(64 * 40, 3)
    tokens = random_tokens(cfg["vocab"], n, 5)
    want = expect(cfg, weights, tokens)
    for cuts in ([n], [n - 40], [1100, 200, 33]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"cuts {cuts}")
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_the_residual_stream_after_every_layer(tmp_path):
    model, weights, _ = build(GAT_ODD, tmp_path, torch.float32)
    cache = model.new_cache(256, 2)
    tokens = random_tokens(GAT_ODD["vocab"], 50, 1)
    seen = {}
    model.observer = lambda i, hidden, delta: seen.__setitem__(i, (hidden if delta is None else hidden + delta.float()).clone())
    run(model, cache, tokens, [50])
    model.observer = None
    streams = []
    plain.forward(GAT_ODD, weights, tokens, streams)
    assert len(streams) == 5
    for i, stream in enumerate(streams):
        assert max_err(seen[i + 1], stream) < 2e-4 * (1 + float(stream.abs().max())), f"after layer {i}"


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", ["odd", "fast"])
def test_unequal_batches_in_slots_used_before(dtype, name, tmp_path):
    """Requests of unequal lengths start together, are decoded together and end one by one; the second round runs in slots,
    pages and state rows that the first has used. Each request's logits equal those of the plain implementation alone."""
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, dtype, seed=2)
    cache = model.new_cache(64 * 10, 3)
    seqs = [random_tokens(cfg["vocab"], n, 30 + n) for n in (150, 3, 66, 1, 91)]
    want = [expect(cfg, weights, s) for s in seqs]
    for round_ in range(2):
        for batch in ([0, 1, 2], [3, 4]):
            slots = {i: cache.open() for i in batch}
            heads = {i: max(1, len(seqs[i]) - 20) for i in batch}
            logits = model.step(cache, [(slots[i], seqs[i][:heads[i]]) for i in batch], want=[list(range(heads[i])) for i in batch])
            got, o = {i: [] for i in batch}, 0
            for i in batch:
                got[i].append(logits[o:o + heads[i]])
                o += heads[i]
            fed = dict(heads)
            live = [i for i in batch if fed[i] < len(seqs[i])]
            while live:
                logits = model.step(cache, [(slots[i], [seqs[i][fed[i]]]) for i in live])
                for row, i in enumerate(live):
                    got[i].append(logits[row:row + 1])
                    fed[i] += 1
                live = [i for i in live if fed[i] < len(seqs[i])]
            for i in batch:
                cache.close(slots[i])
                logits_close(torch.cat(got[i]), want[i], dtype, f"round {round_} request {i}")
    model.raise_on_kernel_error()


def peaked(cfg, weights, factor=6.0):
    """Weights under which one score stands out: the q projections of every attention grown (the windowed one norms q and k
    to unit length, so its scale does the same)."""
    w = {k: v.clone() for k, v in weights.items()}
    for i, entry in enumerate(cfg["layers"]):
        if entry["type"] == "attention":
            w[f"l{i}.mix.q.norm"] *= factor
    return w


@pytest.mark.parametrize("dtype", BOTH)
def test_keys_at_the_edges_of_windows_and_pages_and_keys_far_back(dtype, tmp_path):
    """Windows of 65, 64 and 1 positions over pages of 64 with sharp scores (a scale that lets one key take the weight), and
    a causal attention with sharp scores over 460 positions: prompts that end just inside and just outside a window or a
    page, decoding across the edges, against the plain implementation. A window one position off moves a sharp row by its
    whole spread."""
    cfg = config(120, 48, 1e-6, 0.7, [
        layer(parallel(4, 2, 16, 16, 65, 8, 3, 16, 1.0, 0.5, 40000.0, 1.5), dense(64)),
        layer(attention(4, 2, 16, 24, 8, 40000.0, 0.25, v_mix=True), None),
        layer(parallel(2, 2, 16, 24, 64, 16, 2, 8, 1.0, 0.5, 900.0, 2.0), moe(4, 2, 16, groups=(2, 1), shared=16)),
        layer(parallel(2, 1, 16, 16, 1, 0, 2, 8, 1.0, 0.5, 900.0, 1.0), None),
        layer(attention(2, 2, 16, 24, 16, 900.0, 0.25, v_mix=True), dense(32))])
    weights = peaked(cfg, plain.random_weights(cfg, 11))
    tokens = random_tokens(cfg["vocab"], 460, 5)
    model, used, _ = build(cfg, tmp_path, dtype, weights=weights)
    cache = model.new_cache(64 * 16, 2)
    want = expect(cfg, used, tokens)
    for cuts in ([460], [64], [65, 1, 1, 62, 1, 1, 100, 9], [129, 2], [63, 1, 1, 62, 2]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"cuts {cuts}")
    # the mask matters here: the same weights with every window one position longer give other logits
    longer = {**cfg, "layers": [dict(e, mixer={**e["mixer"], "left": {**e["mixer"]["left"], "mask": {"size": e["mixer"]["left"]["mask"]["size"] + 1}}})
                                if e["type"] == "parallel" else e for e in cfg["layers"]]}
    other = plain.forward_logits(longer, used, tokens)
    d = (other - want[0])[100:]
    assert float((d - d.mean(-1, keepdim=True)).square().mean(-1).sqrt().median() / want[0].std()) > 0.2


@pytest.mark.parametrize("dtype", BOTH)
def test_long_decoding_passes_windows(dtype, tmp_path):
    cfg = config(90, 32, 1e-6, 0.9, [layer(parallel(2, 1, 16, 16, 30, 16, 2, 8, rank=2), moe(4, 2, 8, groups=(2, 1))),
                                     layer(gla(2, 8, 8, tau=4.0, rank=2), dense(40)),
                                     layer(attention(4, 2, 8, 8, 4), None)])
    model, weights, _ = build(cfg, tmp_path, dtype, seed=4)
    cache = model.new_cache(64 * 12, 2)
    tokens = random_tokens(cfg["vocab"], 420, 9)
    logits_close(run(model, cache, tokens, [3]), expect(cfg, weights, tokens), dtype)
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_the_rank_of_a_low_rank_pair_comes_from_the_tensors(tmp_path):
    """A configuration that does not name the ranks loads all the same, and computes the same."""
    import json
    folder, weights = make_model_dir(GAT_ODD, 3, tmp_path)
    bare = json.loads(json.dumps(GAT_ODD))
    for entry in bare["layers"]:
        (entry["mixer"].get("right") or entry["mixer"]).pop("rank", None)
    (folder / "config.json").write_text(json.dumps(bare))
    from qwenforge_b200.engine import Model
    model = Model.from_dir(folder, "float32", DEV)
    tokens = random_tokens(GAT_ODD["vocab"], 40, 2)
    logits_close(run(model, model.new_cache(256, 2), tokens, [40]), plain.forward_logits(GAT_ODD, weights, tokens), torch.float32)


def test_greedy_generation_through_the_engine(tmp_path):
    """StudentEngine.generate_ids (the scheduler's batches, CUDA-graph decoding with padding rows, prompt graphs) against
    greedy decoding of the plain implementation, in float32 where ties are the only way to differ."""
    from qwenforge_b200.engine import StudentEngine
    for name, cfg in (("odd", GAT_ODD), ("ones", GAT_ONES)):
        folder, weights = make_model_dir(cfg, 6, tmp_path / name)
        prompts = [random_tokens(cfg["vocab"], n, n) for n in (5, 70, 1, 33, 12)]
        want = [plain.greedy_generate(cfg, weights, p, 12) for p in prompts]
        for graphs in (True, False):
            engine = StudentEngine(str(folder), device=DEV, dtype="float32", cuda_graphs=graphs)
            got = engine.generate_ids(prompts, max_new_tokens=12, batch_size=3, ignore_eos=True)
            assert got == want, (name, graphs)
    folder, _ = make_model_dir(GAT_FAST, 6, tmp_path / "fast")
    engine = StudentEngine(str(folder), device=DEV, dtype="bfloat16")
    prompts = [random_tokens(GAT_FAST["vocab"], n, n) for n in (5, 170, 1, 33, 12)]
    assert all(len(t) == 12 for t in engine.generate_ids(prompts, max_new_tokens=12, batch_size=5, ignore_eos=True))


def test_trace_replay_as_a_subprocess(tmp_path):
    import json
    import numpy as np
    cfg = GAT_ODD
    folder, weights = make_model_dir(cfg, 8, tmp_path / "m", store_dtype=torch.bfloat16)
    weights = {k: v.to(torch.bfloat16).float() for k, v in weights.items()}
    a, b = random_tokens(cfg["vocab"], 80, 1), random_tokens(cfg["vocab"], 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 69]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[70:71], "want": [0]}, {"id": "b", "tokens": b[8:], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 2 + i, "entries": [{"id": "a", "tokens": [a[71 + i]], "want": [0]}], "end": ["a"] if i == 8 else []} for i in range(9)]
    root = Path(__file__).resolve().parent.parent
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(out),
                           "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=900)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(11)]
    wa, wb = plain.forward_logits(cfg, weights, a), plain.forward_logits(cfg, weights, b)
    first = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab"]))
    logits_close(first, torch.stack((wa[0], wa[69], wb[7])), torch.float32)
    second = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, cfg["vocab"]))
    logits_close(second, torch.stack((wa[70], wb[8])), torch.float32)
    last = torch.from_numpy(np.fromfile(out / "10.f32", dtype="<f4").reshape(1, cfg["vocab"]))
    logits_close(last, wa[79:80], torch.float32)
