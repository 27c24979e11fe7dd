"""The Rarevik design on a GPU: each new kernel and kernel option against its plain reference, the model against the plain
implementation (tests/plain_rarevik.py) whole, decoded, cut into portions, in unequal batches, in slots, pages and state
rows used before, and through the engine's own entry point with greedy generation. The tests make their own small
configurations (tests/helpers_rarevik.py) and weights; where random weights would hide a fault (a key at the window's edge,
a block that is just seen or not yet, the sink), weights or inputs are made so that it shows."""
import copy
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import kernel_refs as refs
from tests import plain_rarevik as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_rarevik import CONFIGS, RAR_FAST, RAR_LONG, RAR_ODD, RAR_ONES, config, dense, gated, layer, make_model_dir, moe, pooled

pytestmark = pytest.mark.gpu
DEV = "cuda"
BOTH = [torch.float32, torch.bfloat16]


def close(got, want, dtype, what="", f32=3e-5, bf16=3e-2):
    got, want = got.double().cpu(), want.double().cpu()
    scale = float(want.abs().max()) + 1e-9
    bound = (f32 if dtype == torch.float32 else bf16) * scale
    err = float((got - want).abs().max())
    assert err <= bound, f"{what}: max |diff| {err:.3e} exceeds {bound:.3e}"


def logits_close(got, want, dtype, what=""):
    """The difference with its mean taken off, root mean square over the vocabulary, against the spread of the logits."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    err = d.square().mean(-1).sqrt() / want.std(-1)
    if dtype == torch.float32:
        assert float(err.max()) <= 1e-4, f"{what}: worst row {float(err.max()):.3e} exceeds 1e-4"
    else:   # the typical row within rounding, and no row lost: a wrong key, a mask one position off or a lost state moves
        # every later row by about its whole spread, which the median sees; a row whose router had two candidates closer
        # than the rounding of its input may stand out
        far = float((err > 0.4).double().mean())
        assert float(err.median()) <= 0.05 and far <= 0.02 and float(err.max()) <= 1.0, \
            f"{what}: median {float(err.median()):.3e}, {far:.1%} of the rows over 0.4, worst {float(err.max()):.3e}"


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
        self.max_q_len = max(length for _, length in spans)
        self.max_kv_len = max(start + length for start, length in spans)


# ------------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("width", [45, 384])
def test_dynamic_tanh_adds_two_pending_outputs(dtype, width):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(width)
    a, b, w, s = rand(g, 9, width, dtype=dtype), rand(g, 9, width, dtype=dtype), rand(g, width, dtype=dtype), rand(g, width, dtype=dtype)
    for first, second in ((a, b), (a, None), (None, b), (None, None)):
        hidden = rand(g, 9, width, spread=3.0)
        want_hidden = hidden.clone()
        out, want = torch.empty(9, width, dtype=dtype, device=DEV), torch.empty(9, width, dtype=dtype, device=DEV)
        ops.add_dyt_norm(hidden, first, second, w, s, 0.7, out)
        refs.add_dyt_norm(want_hidden, first, second, w, s, 0.7, want)
        assert max_err(hidden, want_hidden) < 1e-5
        close(out, want, dtype, "dyt", bf16=1e-2)
        ops.residual_add_pair(hidden, first, second)
        refs.residual_add_pair(want_hidden, first, second)
        assert max_err(hidden, want_hidden) < 1e-5
        other = rand(g, 9, width, spread=2.0)
        both, want_both = torch.empty(9, 2 * width, dtype=dtype, device=DEV), torch.empty(9, 2 * width, dtype=dtype, device=DEV)
        ops.stream_pair(hidden, first, second, other, both)
        refs.stream_pair(hidden, first, second, other, want_both)
        close(both, want_both, dtype, "stream pair", bf16=1e-2)


@pytest.mark.parametrize("dtype", BOTH)
def test_exact_gelu_and_the_heads_gate(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = rand(g, 7, 52, dtype=dtype, spread=2.0)
    out, want = torch.empty_like(x), torch.empty_like(x)
    ops.bias_act(x, None, "gelu", out)
    refs.bias_act(x, None, "gelu", want)
    close(out, want, dtype, "gelu", bf16=1e-2)
    tanh_form = torch.empty_like(x)
    refs.bias_act(x, None, "gelu_tanh", tanh_form)
    if dtype == torch.float32:
        assert max_err(want, tanh_form) > 1e-4 and max_err(out, want) < max_err(out, tanh_form)     # it is the erf form
    wide = rand(g, 7, 3 * 12 + 5, dtype=dtype)     # the gates are the last columns of wider rows
    y, want_y = rand(g, 7, 3 * 20, dtype=dtype), None
    want_y = y.clone()
    ops.head_gate(y, wide[:, 36:39], 3)
    refs.head_gate(want_y, wide[:, 36:39], 3)
    close(y, want_y, dtype, "head gate", bf16=1e-2)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("taps,channels", [(2, 33), (1, 20), (4, 70)])
def test_convolution_without_activation(dtype, taps, channels):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(taps)
    weight = rand(g, channels, taps)
    states = [torch.zeros(3, 5 + max(taps - 1, 1) * channels, device=DEV) for _ in range(2)]
    for spans, slots in (([(0, 6), (0, 1), (0, 3)], [2, -1, 0]), ([(6, 1), (3, 2)], [2, 0]), ([(7, 1), (5, 1), (0, 1)], [2, 0, -1]),
                         ([(8, 1), (6, 1)], [2, 0]), ([(9, 1), (7, 1)], [2, 0]), ([(10, 5), (8, 1)], [2, 0]), ([(0, 1)], [1]), ([(1, 1)], [1])):
        batch = Batch(slots, spans)
        wide = rand(g, batch.n_tokens, channels + 3, dtype=dtype)
        outs = []
        for fn, state in ((ops.causal_conv, states[0]), (refs.causal_conv, states[1])):
            out = torch.empty(batch.n_tokens, channels, dtype=dtype, device=DEV)
            # steps of one token per sequence move the kept inputs inside the same kernel
            fn(wide[:, :channels], weight, None, batch.cu_q, batch.tok_seq, batch.slots, state, 5, out, single=batch.max_q_len == 1)
            outs.append(out)
        close(outs[0], outs[1], dtype, "conv", bf16=1e-2)
        assert max_err(states[0], states[1]) < 1e-6


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("taps,channels", [(2, 72), (3, 40), (4, 136)])
def test_long_steps_of_the_convolution_agree_bit_for_bit_with_short_ones(dtype, taps, channels):
    """A long step runs on the kernel that walks runs of tokens with the last inputs in registers; the same tokens in steps too
    short for it run on the kernel of one thread per output. Sequences that begin inside a run, of one and two tokens, with a
    state from an earlier step and without a slot."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(taps * channels)
    weight = rand(g, channels, taps)
    lengths, slots = [13, 1, 2, 41, 7, 30], [2, 0, -1, 1, 3, 4]
    before = rand(g, 5, (taps - 1) * channels)
    per_seq = [rand(g, n, channels, dtype=dtype) for n in lengths]
    whole, whole_state = Batch(slots, [(3, n) for n in lengths]), before.clone()
    out = torch.empty(whole.n_tokens, channels, dtype=dtype, device=DEV)
    ops.causal_conv(torch.cat(per_seq), weight, None, whole.cu_q, whole.tok_seq, whole.slots, whole_state, 0, out)
    want, want_state = torch.empty_like(out), before.clone()
    refs.causal_conv(torch.cat(per_seq), weight, None, whole.cu_q, whole.tok_seq, whole.slots, want_state, 0, want)
    close(out, want, dtype, "conv of a long step", bf16=1e-2)
    assert max_err(whole_state, want_state) < 1e-6
    pieces, piece_state, begin = [], before.clone(), 0
    for s, (n, slot) in enumerate(zip(lengths, slots)):
        for cut in range(0, n, 9):
            part = per_seq[s][cut:cut + 9]
            batch = Batch([slot], [(3 + cut, part.shape[0])])
            got = torch.empty(part.shape[0], channels, dtype=dtype, device=DEV)
            if slot < 0 and cut > 0:     # nothing is kept without a slot: such a sequence cannot be cut
                got = out[begin + cut:begin + cut + part.shape[0]].clone()
            else:
                ops.causal_conv(part, weight, None, batch.cu_q, batch.tok_seq, batch.slots, piece_state, 0, got)
            pieces.append(got)
        begin += n
    assert torch.equal(torch.cat(pieces), out)
    assert torch.equal(piece_state, whole_state)


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("width", [45, 384])
def test_token_shift_inside_the_norm_kernel_is_the_convolution_behind_it(dtype, width):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(width + 1)
    a, b, w, s = rand(g, 4, width, dtype=dtype), rand(g, 4, width, dtype=dtype), rand(g, width, dtype=dtype), rand(g, width, dtype=dtype)
    frac = torch.rand(width, generator=g).to(DEV)
    taps = torch.stack((frac, 1.0 - frac), dim=1).contiguous()
    slots, every = ints([3, -1, 0, 5]), ints([0, 1, 2, 3, 4])
    states = [rand(g, 6, width + 7).clone() for _ in range(2)]
    states[1].copy_(states[0])
    for _ in range(3):     # a few steps in a row: what one leaves the next one reads
        hidden = rand(g, 4, width, spread=3.0)
        twin = hidden.clone()
        out, shifted = torch.empty(4, width, dtype=dtype, device=DEV), torch.empty(4, width, dtype=dtype, device=DEV)
        ops.add_dyt_norm_shift(hidden, a, b, w, s, 0.7, out, taps, slots, states[0], shifted)
        want, want_shifted = torch.empty_like(out), torch.empty_like(out)
        ops.add_dyt_norm(twin, a, b, w, s, 0.7, want)
        ops.causal_conv(want, taps, None, every, every[:-1], slots, states[1], 0, want_shifted, single=True)
        assert torch.equal(hidden, twin) and torch.equal(out, want) and torch.equal(shifted, want_shifted)
        assert torch.equal(states[0], states[1])
        ref_hidden, ref_out, ref_shifted = twin.clone(), torch.empty_like(out), torch.empty_like(out)
    state = rand(g, 6, width)
    ref_state = state.clone()
    hidden = rand(g, 4, width, spread=3.0)
    ref_hidden = hidden.clone()
    ops.add_dyt_norm_shift(hidden, a, None, w, s, 1.3, out, taps, slots, state, shifted)
    refs.add_dyt_norm_shift(ref_hidden, a, None, w, s, 1.3, ref_out, taps, slots, ref_state, ref_shifted)
    close(out, ref_out, dtype, "dyt", bf16=1e-2)
    close(shifted, ref_shifted, dtype, "shifted", bf16=2e-2)
    close(state, ref_state, dtype, "kept", bf16=1e-2)


def two_caches(kv_heads, dim, dtype, pool=0, window=0):
    from qwenforge_b200.cache import BundleNeed, KvNeed, SequenceCache
    need = KvNeed(kv_heads, dim, window, pool=pool)
    if pool:
        need = BundleNeed((("kv", need), ("blocks", KvNeed(kv_heads, dim, every=pool))))
    return [SequenceCache([need], 2048, 3, 1024, dtype, DEV) for _ in range(2)]


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv_heads,dim,norm_dim,rot,interleaved,first", [
    (4, 2, 14, 10, 6, False, True), (3, 3, 64, 64, 64, True, False), (2, 1, 40, 40, 0, False, True), (5, 1, 96, 96, 48, True, False),
    (2, 2, 128, 96, 96, False, True), (2, 1, 20, 20, 20, True, True),
    # whole heads normed and rotated, in sizes that the kernel of eight components per thread takes in long bfloat16 steps
    (14, 2, 64, 64, 64, False, True), (3, 1, 128, 128, 128, False, True), (2, 2, 32, 32, 32, True, True), (5, 5, 16, 16, 16, False, True),
    (4, 2, 256, 256, 256, False, True)])
def test_norm_before_the_rotation_and_neighbours_paired(dtype, heads, kv_heads, dim, norm_dim, rot, interleaved, first):
    """The weighted RMS norm of q and k before the rotation over a head's own components (the rest are padding and stay zero),
    the rotation of halves or of neighbours, queries out and keys and values into the pages, from rows that are wider."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(dim)
    batch = Batch([1, -1, 0], [(60, 9), (0, 3), (5, 70)])
    caches = two_caches(kv_heads, dim, dtype)
    for cache in caches:
        for slot, total in ((cache.open(), 75), (cache.open(), 69)):
            cache.reserve([(slot, total)])
        cache.flush()
    inv_freq = (1.0 / (300.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV) if rot else None
    width = (heads + 2 * kv_heads) * dim
    wide = rand(g, batch.n_tokens, width + 8, dtype=dtype)
    wide[:, :width].view(batch.n_tokens, -1, dim)[:, :, norm_dim:] = 0          # padded heads carry zeros beyond their own size
    qn, kn = rand(g, norm_dim, dtype=dtype) + 1, rand(g, norm_dim, dtype=dtype) + 1
    outs = []
    for fn, cache in ((ops.rope_cache_write, caches[0]), (refs.rope_cache_write, caches[1])):
        site = cache.site(0)
        q = torch.empty(batch.n_tokens, heads * dim, dtype=dtype, device=DEV)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        args = ops.KvSiteArgs(site.storage, site.table, kv_heads, dim) if fn is ops.rope_cache_write else site
        fn(wide[:, :width] if fn is refs.rope_cache_write else wide, batch.tok_seq, batch.tok_pos, batch.slots, inv_freq, rot, heads, q, args,
           True, err, unit_norm_eps=1e-5 if first else None, norm_dim=norm_dim, interleaved=interleaved, norm_first=first,
           q_norm=qn if first else None, k_norm=kn if first else None)
        assert int(err) == 0
        outs.append(q)
    close(outs[0], outs[1], dtype, "queries", bf16=1e-2)
    close(caches[0].site(0).storage, caches[1].site(0).storage, dtype, "pages", bf16=1e-2)
    assert float(caches[0].site(0).storage.abs().max()) > 0


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("heads,kv_heads,dim,window,pool", [(4, 2, 14, 37, 5), (4, 1, 64, 128, 32), (3, 3, 24, 1, 1), (2, 2, 96, 9, 70),
                                                            (6, 2, 128, 40, 16)])
def test_rows_of_whole_blocks_join_the_window_under_a_learned_sink(dtype, heads, kv_heads, dim, window, pool):
    """The kernel that forms the rows of completed blocks and the attention that reads them beside the window's keys, each
    against its reference: prompts, continuations that complete several blocks or none, and single tokens, with queries grown
    so that single keys stand out."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(window)
    caches = two_caches(kv_heads, dim, dtype, pool=pool, window=window)
    sinks = rand(g, heads)
    slots = [[c.open() for _ in range(3)] for c in caches]
    lengths = [0, 0, 0]
    for spans in ([(0, 150), (0, 3), (0, 70)], [(150, 1), (3, 1), (70, 1)], [(151, 69), (4, 140), (71, 2)], [(220, 1), (144, 1), (73, 1)]):
        batch = Batch(slots[0], spans)
        k = rand(g, batch.n_tokens, 2, kv_heads, dim, dtype=dtype)
        q = rand(g, batch.n_tokens, heads * dim, dtype=dtype, spread=3.0)
        outs = []
        for which, cache in enumerate(caches):
            cache.reserve([(slot, start + n) for slot, (start, n) in zip(slots[which], spans)])
            cache.flush()
            kv, rows = cache.site(0)["kv"], cache.site(0)["blocks"]
            for t in range(batch.n_tokens):     # the step's keys and values into the pages
                s, pos = int(batch.tok_seq[t]), int(batch.tok_pos[t])
                page = int(kv.table[slots[which][s], pos // 64])
                kv.storage[page, :, :, pos % 64, :] = k[t]
            err = torch.zeros(1, dtype=torch.int32, device=DEV)
            out = torch.empty(batch.n_tokens, heads * dim, dtype=dtype, device=DEV)
            if which == 0:
                a, b = ops.KvSiteArgs(kv.storage, kv.table, kv_heads, dim), ops.KvSiteArgs(rows.storage, rows.table, kv_heads, dim)
                ops.pool_cache_write(batch.cu_q, batch.tok_pos, batch.slots, a, b, pool, batch.max_q_len, err)
                ops.attention_generic(q, out, batch.cu_q, batch.tok_pos, batch.slots, a, heads, 3, batch.max_q_len, dim ** -0.5, window,
                                      err, sinks=sinks, blocks=b, pool=pool)
            else:
                refs.pool_cache_write(batch.cu_q, batch.tok_pos, batch.slots, kv, rows, pool, batch.max_q_len, err)
                refs.attention_generic(q, out, batch.cu_q, batch.tok_pos, batch.slots, kv, heads, 3, batch.max_q_len, dim ** -0.5, window,
                                       err, sinks=sinks, blocks=rows, pool=pool)
            assert int(err) == 0
            outs.append(out)
            for slot, (start, n) in zip(slots[which], spans):
                cache.advance(slot, n)
        close(caches[0].site(0)["blocks"].storage, caches[1].site(0)["blocks"].storage, dtype, "rows of blocks", bf16=1e-2)
        close(outs[0], outs[1], dtype, f"attention {spans}", f32=1e-4, bf16=2e-2)
    assert float(caches[0].site(0)["blocks"].storage.abs().max()) > 0


@pytest.mark.parametrize("heads,kv_heads,dim,window,pool", [(4, 1, 64, 128, 32), (6, 3, 96, 190, 7), (2, 2, 32, 1, 1), (6, 2, 128, 40, 16),
                                                            (4, 2, 64, 9, 70)])
def test_tensor_core_attention_takes_the_rows_of_whole_blocks(heads, kv_heads, dim, window, pool):
    """The mma.sync kernel of prompts, portions and single tokens against the float32 SIMT kernel on the same pages: rows of
    blocks that fill more than a page, tiles whose rows see different numbers of blocks, a learned sink."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(pool)
    dtype = torch.bfloat16
    cache = two_caches(kv_heads, dim, dtype, pool=pool, window=window)[0]
    sinks = rand(g, heads)
    slots = [cache.open() for _ in range(3)]
    for spans in ([(0, 700), (0, 3), (0, 130)], [(700, 1), (3, 1), (130, 1)], [(701, 69), (4, 200), (131, 2)], [(770, 1), (204, 1), (133, 1)]):
        batch = Batch(slots, spans)
        k = rand(g, batch.n_tokens, 2, kv_heads, dim, dtype=dtype)
        q = rand(g, batch.n_tokens, heads * dim, dtype=dtype, spread=2.0)
        cache.reserve([(slot, start + n) for slot, (start, n) in zip(slots, spans)])
        cache.flush()
        kv, rows = cache.site(0)["kv"], cache.site(0)["blocks"]
        pages = kv.table[batch.slots.long()[batch.tok_seq.long()], (batch.tok_pos // 64).long()].long()
        kv.storage[pages, :, :, (batch.tok_pos % 64).long(), :] = k
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        a, b = ops.KvSiteArgs(kv.storage, kv.table, kv_heads, dim), ops.KvSiteArgs(rows.storage, rows.table, kv_heads, dim)
        ops.pool_cache_write(batch.cu_q, batch.tok_pos, batch.slots, a, b, pool, batch.max_q_len, err)
        out, want = (torch.empty(batch.n_tokens, heads * dim, dtype=dtype, device=DEV) for _ in range(2))
        ops.attention_prefill(q, out, batch.cu_q, batch.tok_pos, batch.slots, a, heads, 3, batch.max_q_len, dim ** -0.5, window, err,
                              max_kv_len=batch.max_kv_len, sinks=sinks, blocks=b, pool=pool)
        ops.attention_generic(q, want, batch.cu_q, batch.tok_pos, batch.slots, a, heads, 3, batch.max_q_len, dim ** -0.5, window, err,
                              sinks=sinks, blocks=b, pool=pool)
        assert int(err) == 0
        close(out, want, dtype, f"{spans}", bf16=2e-2)
        for slot, (start, n) in zip(slots, spans):
            cache.advance(slot, n)


@pytest.mark.parametrize("dtype", BOTH)
def test_router_bias_softmax_over_the_chosen_and_the_shared_expert(dtype):
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(3)
    for tokens, experts, top in ((9, 5, 2), (300, 16, 3), (1200, 8, 1), (4, 3, 3)):
        x, router, bias = rand(g, tokens, 48, dtype=dtype), rand(g, experts, 48, dtype=dtype, spread=0.3), rand(g, experts, spread=2.0)
        logits = ops.linear(x, router, out_dtype=torch.float32)
        for given in (logits, None):
            if given is None and tokens * experts > ops.MOE_FUSED_ROUTER_MAX:
                continue
            plan = ops.moe_plan(given, top, True, True, x=x, router=router, bias=bias)
            want = refs.moe_plan(logits.cpu(), top, True, True, bias=bias.cpu())
            z = (logits + bias).cpu().double()
            ordered = z.sort(-1, descending=True).values
            sure = (ordered[:, top - 1] - ordered[:, top] > 1e-3) if experts > top else torch.ones(tokens, dtype=torch.bool)
            got_experts = plan.pair_expert.cpu().view(tokens, top).sort(-1).values
            want_experts = z.topk(top, -1).indices.sort(-1).values
            assert bool((got_experts == want_experts)[sure].all())
            got_w = torch.zeros(tokens, experts, dtype=torch.float64)
            got_w[plan.sorted_token.cpu().long(), plan.pair_expert.cpu().view(-1)[torch.argsort(plan.dest.cpu())].long()] = plan.sorted_weight.cpu().double()
            want_w = torch.zeros(tokens, experts, dtype=torch.float64).scatter(1, z.topk(top, -1).indices, torch.softmax(z.topk(top, -1).values, -1))
            assert float((got_w - want_w)[sure].abs().max()) < 1e-5
            assert float((got_w.sum(-1) - 1).abs().max()) < 1e-5          # the softmax is over the chosen alone
        y, extra, gate = rand(g, tokens * top, 40, dtype=dtype), rand(g, tokens, 40, dtype=dtype), rand(g, tokens, spread=2.0)
        out, want_out = torch.empty(tokens, 40, dtype=dtype, device=DEV), torch.empty(tokens, 40, dtype=dtype, device=DEV)
        for e, lg in ((extra, gate), (extra, None), (None, None)):
            ops.moe_combine(y, plan, out, True, e, lg)
            refs.moe_combine(y, plan, want_out, True, e, lg)
            close(out, want_out, dtype, "combine", bf16=1e-2)
        gate_weight = rand(g, 48, dtype=dtype, spread=0.3)      # the gate's logit formed inside the kernel
        ops.moe_combine(y, plan, out, True, extra, None, x, gate_weight)
        refs.moe_combine(y, plan, want_out, True, extra, None, x, gate_weight)
        close(out, want_out, dtype, "combine with its own gate", bf16=1e-2)


def test_clamped_gate_in_the_grouped_tensor_core_product():
    """A step long enough for tiles of 128 rows: the experts' first product with the clamped gate in its epilogue against
    the reference, with limits that most sums exceed and limits that none does."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(5)
    tokens, experts, top, width, inter = 1500, 4, 2, 128, 96
    x, router = rand(g, tokens, width, dtype=torch.bfloat16), rand(g, experts, width, dtype=torch.bfloat16, spread=0.3)
    weight = rand(g, experts, 2 * inter, width, dtype=torch.bfloat16, spread=0.2)
    plan = ops.moe_plan(ops.linear(x, router, out_dtype=torch.float32), top, True, True, 128)
    rows = torch.empty(tokens * top, width, dtype=torch.bfloat16, device=DEV)
    ops.moe_gather(x, plan, rows, False)
    assert ops.tc_gemm_grouped_takes(rows, weight, plan, ops.TC_SWIGLU)
    experts_of = torch.empty(tokens * top, dtype=torch.long, device=DEV)
    experts_of[plan.dest.long()] = plan.pair_expert.long()
    class Routing:
        row_expert = experts_of
    for limit in (0.5, 50.0):
        out, want = (torch.empty(tokens * top, inter, dtype=torch.bfloat16, device=DEV) for _ in range(2))
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        ops.tc_gemm_grouped(ops.TC_SWIGLU, rows, weight, plan, out, None, err, clamp=(limit, 1.702))
        refs.tc_gemm_grouped(1, rows, weight, Routing, want, clamp=(limit, 1.702))
        assert int(err) == 0
        close(out, want, torch.bfloat16, f"limit {limit}", bf16=2e-2)


def test_clamped_gate_in_the_small_grouped_product():
    """Short steps: the experts' first product through the plan's row map, tiles of 64 rows, the clamped gate on its float32
    sums; experts without a row, rows that do not fill a tile, an expert size that is no multiple of the tile's columns."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(6)
    for tokens, experts, top, width, inter in ((8, 8, 2, 128, 40), (70, 3, 3, 64, 112)):
        x, router = rand(g, tokens, width, dtype=torch.bfloat16), rand(g, experts, width, dtype=torch.bfloat16, spread=0.3)
        weight = rand(g, experts, 2 * inter, width, dtype=torch.bfloat16, spread=0.2)
        plan = ops.moe_plan(ops.linear(x, router, out_dtype=torch.float32), top, True, True, 64)
        assert ops.expert_gate_takes(x, weight, plan)
        rows = torch.empty(tokens * top, width, dtype=torch.bfloat16, device=DEV)
        ops.moe_gather(x, plan, rows, False)
        experts_of = torch.empty(tokens * top, dtype=torch.long, device=DEV)
        experts_of[plan.dest.long()] = plan.pair_expert.long()
        class Routing:
            row_expert = experts_of
        for limit in (0.5, 50.0):
            out, want = (torch.empty(tokens * top, inter, dtype=torch.bfloat16, device=DEV) for _ in range(2))
            ops.expert_gate_up(x, weight, plan, out, None, gather=True, clamp=(limit, 1.702))
            refs.tc_gemm_grouped(1, rows, weight, Routing, want, clamp=(limit, 1.702))
            close(out, want, torch.bfloat16, f"limit {limit}", bf16=2e-2)


def test_clamped_gate_in_the_product_of_few_rows():
    """The shared expert's first product in steps of few rows: the weight streamer with the clamped gate on its float32 sums,
    against the product and the gate as two steps."""
    from qwenforge_b200 import ops
    g = torch.Generator().manual_seed(8)
    ran = 0
    for rows, width, inter in ((1, 256, 96), (8, 896, 608), (16, 512, 1024)):
        x = rand(g, rows, width, dtype=torch.bfloat16)
        weight = rand(g, 2 * inter, width, dtype=torch.bfloat16, spread=0.1)
        for limit in (0.7, 40.0):
            out, want = (torch.zeros(rows, inter, dtype=torch.bfloat16, device=DEV) for _ in range(2))
            if not ops.gated_rows(x, weight, out, clamp=(limit, 1.702)):
                continue
            ran += 1
            refs.clamped_glu(refs.linear(x, weight, out_dtype=torch.float32), limit, 1.702, want)
            close(out, want, torch.bfloat16, f"rows {rows}, limit {limit}", bf16=2e-2)
        plain_out, plain_want = torch.zeros_like(out), torch.zeros_like(out)
        if ops.gated_rows(x, weight, plain_out):
            refs.swiglu(refs.linear(x, weight, out_dtype=torch.float32), plain_want)
            close(plain_out, plain_want, torch.bfloat16, f"rows {rows}, silu", bf16=2e-2)
    assert ran > 0


# ------------------------------------------------------------------------------------------------ the model
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
    want = plain.forward_logits(cfg, weights, tokens)
    for cuts in ([300], [260], [2, 61, 2, 130, 65, 3, 2], [129, 128]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"{name} cuts {cuts[:3]}")
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


@pytest.mark.parametrize("dtype", BOTH)
def test_long_prompts_at_larger_sizes(dtype, tmp_path):
    """Steps of more than a thousand tokens: whole, with the last tokens decoded, and cut where the later portions reach back
    over many pages."""
    cfg, n = RAR_LONG, 1400
    model, weights, _ = build(cfg, tmp_path, dtype, seed=11)
    cache = model.new_cache(64 * 40, 3)
    tokens = random_tokens(cfg["vocab"], n, 5)
    want = plain.forward_logits(cfg, weights, tokens)
    for cuts in ([n], [n - 40], [1100, 200, 33]):
        logits_close(run(model, cache, tokens, cuts), want, dtype, f"cuts {cuts}")
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_the_residual_stream_after_every_layer_run(tmp_path):
    model, weights, _ = build(RAR_ODD, tmp_path, torch.float32)
    cache = model.new_cache(256, 2)
    tokens = random_tokens(RAR_ODD["vocab"], 50, 1)
    seen = {}
    model.observer = lambda i, hidden, delta: seen.__setitem__(i, (hidden if delta is None else hidden + delta.float()).clone())
    run(model, cache, tokens, [50])
    model.observer = None
    streams = []
    plain.forward(RAR_ODD, weights, tokens, streams)
    assert len(streams) == 7
    for i, stream in enumerate(streams):
        assert max_err(seen[i + 1], stream) < 2e-4 * (1 + float(stream.abs().max())), f"after run {i}"


@pytest.mark.parametrize("dtype", BOTH)
@pytest.mark.parametrize("name", ["odd", "fast"])
def test_unequal_batches_in_slots_used_before(dtype, name, tmp_path):
    """Requests of unequal lengths start together, are decoded together and end one by one; the second round runs in slots,
    pages and state rows that the first has used. Each request's logits equal those of the plain implementation alone.
    (Odd sizes run on the kernels of one element per thread, the other configuration on those of 16 bytes per thread, where
    a sequence may begin in the middle of a thread's run of tokens.)"""
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, dtype, seed=2)
    cache = model.new_cache(64 * 10, 3)
    seqs = [random_tokens(cfg["vocab"], n, 30 + n) for n in (150, 3, 66, 1, 91)]
    want = [plain.forward_logits(cfg, weights, s) for s in seqs]
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


def peaked(cfg, weights):
    """Weights under which one score stands out and the sink matters only where every score is low: the q projections grown."""
    w = {k: v.clone() for k, v in weights.items()}
    for i in range(len(cfg["layers"])):
        w[f"l{i}.mix.q"] *= 4.0
    return w


@pytest.mark.parametrize("dtype", BOTH)
def test_keys_at_the_edges_of_windows_blocks_and_pages(dtype, tmp_path):
    """A window of 150 positions over blocks of 40 over pages of 64, and a gated window of 65: prompts that end just inside and
    just outside, decoding across the edges, with sharpened scores, against the plain implementation; a sink far above and
    far below the scores."""
    cfg = config(120, 48, 1e-6, [
        layer(pooled(4, 2, 16, 16, 150, 40, 3, 8, 40000.0, 1.0), dense(64)),
        layer(gated(4, 2, 16, 16, 65, 8, 40000.0, 1.0, (4.0, 1.0, 4.0, 128)), None),
        layer(pooled(2, 2, 16, 24, 63, 64, 2, 16, 900.0, 1.0), moe(4, 2, 16, 1.0, (16, 1.0)))], loop=(1, 3, 2))
    weights = peaked(cfg, plain.random_weights(cfg, 11))
    tokens = random_tokens(cfg["vocab"], 460, 5)
    for sink in (None, 12.0, -30.0):
        if sink is not None:
            weights["l0.mix.sink"] = torch.full_like(weights["l0.mix.sink"], sink)
        model, used, _ = build(cfg, tmp_path / str(sink), dtype, weights=weights)
        cache = model.new_cache(64 * 16, 2)
        want = plain.forward_logits(cfg, used, tokens)
        for cuts in ([460], [149], [150, 1, 1, 38, 1, 1, 100, 9], [189, 2], [63, 1, 1, 62, 2]):
            logits_close(run(model, cache, tokens, cuts), want, dtype, f"sink {sink} cuts {cuts}")


@pytest.mark.parametrize("dtype", BOTH)
def test_long_decoding_passes_windows_and_blocks(dtype, tmp_path):
    cfg = config(90, 32, 1e-6, [layer(pooled(2, 1, 16, 16, 30, 8, 4, 16), moe(4, 2, 8, 2.0)), layer(gated(4, 2, 8, 8, 50, 4), dense(40))],
                 loop=(0, 1, 2))
    model, weights, _ = build(cfg, tmp_path, dtype, seed=4)
    cache = model.new_cache(64 * 12, 2)
    tokens = random_tokens(cfg["vocab"], 420, 9)
    logits_close(run(model, cache, tokens, [3]), plain.forward_logits(cfg, weights, tokens), dtype)
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_greedy_generation_through_the_engine(tmp_path):
    """StudentEngine.generate_ids (the scheduler's batches, CUDA-graph decoding with padding rows, prompt graphs) against
    greedy decoding of the plain implementation, in float32 where ties are the only way to differ."""
    from qwenforge_b200.engine import StudentEngine
    for name, cfg in (("odd", RAR_ODD), ("ones", RAR_ONES)):
        folder, weights = make_model_dir(cfg, 6, tmp_path / name)
        prompts = [random_tokens(cfg["vocab"], n, n) for n in (5, 70, 1, 33, 12)]
        want = [plain.greedy_generate(cfg, weights, p, 12) for p in prompts]
        for graphs in (True, False):
            engine = StudentEngine(str(folder), device=DEV, dtype="float32", cuda_graphs=graphs)
            got = engine.generate_ids(prompts, max_new_tokens=12, batch_size=3, ignore_eos=True)
            assert got == want, (name, graphs)
    folder, _ = make_model_dir(RAR_FAST, 6, tmp_path / "fast")
    engine = StudentEngine(str(folder), device=DEV, dtype="bfloat16")
    prompts = [random_tokens(RAR_FAST["vocab"], n, n) for n in (5, 170, 1, 33, 12)]
    assert all(len(t) == 12 for t in engine.generate_ids(prompts, max_new_tokens=12, batch_size=5, ignore_eos=True))


def test_trace_replay_as_a_subprocess(tmp_path):
    import json
    import numpy as np
    cfg = RAR_ODD
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
