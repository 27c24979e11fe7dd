"""The Gatosun design through the package's own configuration, loader, cache, state and step function on the CPU, with
every CUDA kernel replaced by its plain reference (the `reference_kernels` fixture), against the plain implementation of
tests/plain_gatosun.py. This checks the host side: names and shapes, the order of the parts, padded heads, what every kind of
layer keeps per sequence, the chain of layers that share values, the factors under which outputs enter the stream, pages
given back as a window passes. The kernels themselves are checked on a GPU."""
import json

import pytest
import torch

from tests import plain_gatosun as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_gatosun import CONFIGS, GAT_FAST, GAT_ODD, GAT_ONES, attention, config, dense, gla, layer, make_model_dir, moe, parallel


def build(cfg, tmp_path, seed=0):
    from qwenforge_b200.engine import Model
    folder, weights = make_model_dir(cfg, seed, tmp_path)
    return Model.from_dir(folder, "float32", "cpu"), weights, folder


def run(model, cache, tokens, cuts):
    slot, at, got = cache.open(), 0, []
    for size in list(cuts) + [1] * (len(tokens) - sum(cuts)):
        got.append(model.step(cache, [(slot, tokens[at:at + size])], want=[list(range(size))]))
        at += size
    cache.close(slot)
    return torch.cat(got)


def test_configuration_names_every_tensor():
    from qwenforge_b200.config import GatosunConfig, config_from_dict
    from qwenforge_b200.engine import Model
    for cfg in CONFIGS.values():
        cfg_obj = config_from_dict(cfg)
        assert isinstance(cfg_obj, GatosunConfig)
        spec = cfg_obj.model_spec()
        wanted = {t.name: tuple(t.shape) for t in Model.tensor_specs_of(spec)}
        shapes = plain.tensor_shapes(cfg)
        unread = set(spec.ignored_tensors)
        assert wanted == {k: v for k, v in shapes.items() if k not in unread}
        assert config_from_dict(cfg_obj.to_dict()).model_spec() == spec
        assert [e.layer for e in spec.schedule] == list(range(len(cfg["layers"])))
    # the first layer with shared values does not read its mixing weight; a layer without a feed-forward has no second norm
    spec = config_from_dict(GAT_ODD).model_spec()
    assert "l1.mix.vmix" in spec.ignored_tensors and "l2.norm2" in spec.ignored_tensors
    roles = [layer_.parts["mixer"].params.get("value_mix") for layer_ in spec.layers]
    assert [r and r["role"] for r in roles] == [None, "source", None, "mix", "mix"]
    with pytest.raises(ValueError, match="not supported"):
        config_from_dict(config(50, 16, 1e-6, 1.0, [dict(type="other", mixer={}, mlp=None)]))
    with pytest.raises(ValueError, match="top"):
        config_from_dict(config(50, 16, 1e-6, 1.0, [layer(gla(1, 8, 8), moe(2, 3, 4))]))
    with pytest.raises(ValueError, match="groups"):
        config_from_dict(config(50, 16, 1e-6, 1.0, [layer(gla(1, 8, 8), moe(6, 3, 4, groups=(3, 1)))]))
    with pytest.raises(ValueError, match="v_mix"):
        config_from_dict(config(50, 16, 1e-6, 1.0, [layer(attention(2, 2, 8, 8, 8, v_mix=True), None), layer(attention(2, 1, 8, 8, 8, v_mix=True), None)]))
    with pytest.raises(ValueError, match="residual_mult"):
        config_from_dict({k: v for k, v in GAT_ONES.items() if k != "residual_mult"})


def test_what_a_layer_keeps(reference_kernels, tmp_path):
    from qwenforge_b200.cache import BundleNeed, KvNeed, StateNeed
    model, _, _ = build(GAT_ODD, tmp_path)
    needs = model.cache_needs()
    assert needs[0] == StateNeed((3 * 10 * 6,))                       # the gated linear attention: S alone
    assert needs[1] == KvNeed(2, 10, 0) and needs[3] == KvNeed(2, 14, 0) and needs[4] == KvNeed(2, 10, 0)   # heads padded to the wider side
    assert isinstance(needs[2], BundleNeed)
    both = dict(needs[2].items)
    assert both["left"] == KvNeed(2, 10, 7) and both["right"] == StateNeed((3 * 6 * 6 + 44,))   # S and the last token's input
    cache = model.new_cache(512, 2)
    assert cache.site(2)["right"].storage.shape[1] == 3 * 6 * 6 + 44


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_agrees_with_the_plain_implementation(reference_kernels, name, tmp_path):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, seed=1)
    tokens = random_tokens(cfg["vocab"], 90, 3)
    want = plain.forward_logits(cfg, weights, tokens)
    cache = model.new_cache(512, 2)
    for cuts in ([90], [37, 2, 20], [], [64, 2], [1, 65]):
        got = run(model, cache, tokens, cuts)
        assert max_err(got, want) < 2e-4, (name, cuts)
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_pages_leave_as_the_window_passes_and_slots_come_back_clean(reference_kernels, tmp_path):
    cfg = config(40, 16, 1e-5, 0.8, [layer(parallel(2, 1, 8, 8, 10, 4, 2, 4, rank=2), None), layer(gla(2, 4, 4, rank=2), dense(8))])
    model, weights, _ = build(cfg, tmp_path, seed=5)
    cache = model.new_cache(64 * 6, 2)
    windowed = [g for g in cache.kv_groups if g.need.window == 10][0]
    tokens = random_tokens(40, 200, 4)
    want = plain.forward_logits(cfg, weights, tokens)
    slot = cache.open()
    got = [model.step(cache, [(slot, tokens[:70])], want=[list(range(70))])]
    for t in range(70, 200):
        got.append(model.step(cache, [(slot, [tokens[t]])]))
        assert windowed.pages_held(slot) <= 2
    assert max_err(torch.cat(got), want) < 2e-4
    cache.close(slot)
    # the slot and its state rows again, for another sequence: nothing of the first one is left
    other = random_tokens(40, 30, 8)
    assert max_err(run(model, cache, other, [30]), plain.forward_logits(cfg, weights, other)) < 2e-4
    assert max_err(run(model, cache, other, [12]), plain.forward_logits(cfg, weights, other)) < 2e-4


def test_unequal_batches_against_each_request_alone(reference_kernels, tmp_path):
    model, weights, _ = build(GAT_ODD, tmp_path, seed=2)
    cache = model.new_cache(64 * 8, 3)
    seqs = [random_tokens(GAT_ODD["vocab"], n, 30 + n) for n in (40, 3, 17)]
    want = [plain.forward_logits(GAT_ODD, weights, s) for s in seqs]
    for _ in range(2):
        slots = [cache.open() for _ in seqs]
        heads = [max(1, len(s) - 5) for s in seqs]
        logits = model.step(cache, [(slots[i], seqs[i][:heads[i]]) for i in range(3)], want=[list(range(h)) for h in heads])
        got, o = [[] for _ in seqs], 0
        for i, h in enumerate(heads):
            got[i].append(logits[o:o + h])
            o += h
        fed = list(heads)
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        while live:
            logits = model.step(cache, [(slots[i], [seqs[i][fed[i]]]) for i in live])
            for row, i in enumerate(live):
                got[i].append(logits[row:row + 1])
                fed[i] += 1
            live = [i for i in live if fed[i] < len(seqs[i])]
        for i in range(3):
            cache.close(slots[i])
            assert max_err(torch.cat(got[i]), want[i]) < 2e-4


def test_the_router_of_the_plain_implementation_on_a_made_case():
    """Scores, correction, groups and the weights, on numbers chosen by hand."""
    cfg = config(10, 4, 1e-5, 1.0, [layer(gla(1, 4, 4), moe(6, 2, 4, groups=(3, 2)))])
    mlp = cfg["layers"][0]["mlp"]
    weights = {"r.router": torch.eye(6, 4), "r.correction": torch.tensor([0.0, 0.0, -2.0, -2.0, 0.3, 0.3])}
    h = torch.tensor([[4.0, 3.0, 0.0, 0.0]], dtype=torch.float64)
    chosen, weight, _ = plain.router(weights, "r.", mlp, h)
    # scores: .982 .953 .5 .5 .5 .5; choice scores: .982 .953 -1.5 -1.5 .8 .8; groups (0,1) (2,3) (4,5) score 1.93, -3, 1.6:
    # the second group is shut out, and the best two of the others are experts 0 and 1, weighted by their scores alone
    assert chosen.tolist() == [[0, 1]]
    assert max_err(weight, torch.sigmoid(torch.tensor([[4.0, 3.0]], dtype=torch.float64))) < 1e-12
    weights["r.correction"] = torch.tensor([0.0, -3.0, 0.4, 0.4, 0.3, 0.3])
    chosen, weight, _ = plain.router(weights, "r.", mlp, h)
    # group scores now .982 - 2.05 < 0, 1.8, 1.6: the expert with the largest score of all cannot be chosen
    assert sorted(chosen.tolist()[0]) == [2, 3] and max_err(weight, torch.full((1, 2), 0.5, dtype=torch.float64)) < 1e-12


def test_generation_loop_on_the_cpu(reference_kernels, tmp_path):
    from qwenforge_b200.engine import StudentEngine
    folder, weights = make_model_dir(GAT_ONES, 6, tmp_path)
    prompts = [random_tokens(GAT_ONES["vocab"], n, n) for n in (5, 20, 1)]
    want = [plain.greedy_generate(GAT_ONES, weights, p, 6) for p in prompts]
    engine = StudentEngine(str(folder), device="cpu", dtype="float32", cuda_graphs=False)
    assert engine.generate_ids(prompts, max_new_tokens=6, batch_size=2, ignore_eos=True) == want
