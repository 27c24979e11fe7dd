"""The Rarevik design through the package's own configuration, loader, cache, state and step function on the CPU, with
every CUDA kernel replaced by its plain reference (the `reference_kernels` fixture), against the plain implementation of
tests/plain_rarevik.py. This checks the host side: names and shapes, the schedule of a repeated run, the order of the parts,
padded heads, the several things one layer keeps (keys and values, rows of whole blocks, a convolution's last inputs, the
token shift's last input), pages given back as the window and the blocks pass. The kernels themselves are checked on a GPU."""
import pytest
import torch

from tests import plain_rarevik as plain
from tests.helpers import max_err, random_tokens
from tests.helpers_rarevik import CONFIGS, RAR_FAST, RAR_ODD, RAR_ONES, config, dense, gated, layer, make_model_dir, pooled


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


def test_configuration_names_every_tensor_and_lays_out_the_passes():
    from qwenforge_b200.config import RarevikConfig, config_from_dict
    from qwenforge_b200.engine import Model
    for cfg in CONFIGS.values():
        cfg_obj = config_from_dict(cfg)
        assert isinstance(cfg_obj, RarevikConfig)
        spec = cfg_obj.model_spec()
        wanted = {t.name: tuple(t.shape) for t in Model.tensor_specs_of(spec)}
        assert wanted == plain.tensor_shapes(cfg)
        assert config_from_dict(cfg_obj.to_dict()).model_spec() == spec
        runs = plain.schedule(cfg)
        assert [(e.layer, e.enter is not None) for e in spec.schedule] == runs
    assert len(config_from_dict(RAR_ODD).model_spec().schedule) == 7 and len(config_from_dict(RAR_ONES).model_spec().stream_parts) == 0
    with pytest.raises(ValueError, match="loop"):
        config_from_dict(config(50, 16, 1e-6, [layer(gated(2, 1, 8, 8, 16, 8), None)], loop=(0, 2, 1)))
    with pytest.raises(ValueError, match="pool"):
        bad = layer(pooled(2, 1, 8, 8, 16, 4, 2, 8), None)
        del bad["mixer"]["mask"]["pool"]
        config_from_dict(config(50, 16, 1e-6, [bad]))
    with pytest.raises(ValueError, match="not supported"):
        config_from_dict(config(50, 16, 1e-6, [dict(type="other", mixer={}, mlp=None)]))
    with pytest.raises(ValueError, match="top"):
        config_from_dict(config(50, 16, 1e-6, [layer(gated(2, 1, 8, 8, 16, 8), dict(kind="moe", router=dict(experts=2, top=3), expert=dict(ff=4, limit=1.0)))]))


def test_what_a_layer_keeps(reference_kernels, tmp_path):
    from qwenforge_b200.cache import BundleNeed, KvNeed, StateNeed
    model, _, _ = build(RAR_ODD, tmp_path)
    needs = model.cache_needs()
    assert len(needs) == 7 and needs[0] == needs[2] == needs[4] and needs[1] == needs[3]
    first = dict(needs[0].items)
    assert first["input"] == StateNeed((52,)) and isinstance(first["mixer"], BundleNeed)
    mixer = dict(first["mixer"].items)
    # heads padded to the wider of keys and values; the positions stay until their block of 5 is complete
    assert mixer["kv"] == KvNeed(2, 14, 37, pool=5) and mixer["blocks"] == KvNeed(2, 14, every=5)
    assert mixer["conv"] == StateNeed(((4 + 2 + 2) * 14,))
    assert dict(needs[1].items)["mixer"] == KvNeed(3, 12, 23)
    last = dict(dict(needs[6].items)["mixer"].items)
    assert last["kv"] == KvNeed(1, 18, 9, pool=70) and last["conv"] == StateNeed((3 * 4 * 18,))
    # every pass has a cache and state of its own: seven sites, no two the same storage
    cache = model.new_cache(512, 2)
    shifts = {cache.site(i)["input"].storage.data_ptr() for i in range(7)}
    pages = {cache.site(i)["mixer"]["kv"].storage.data_ptr() for i in (0, 2, 4)}
    assert len(shifts) == 7 and len(pages) == 3


def test_first_kept_and_rows():
    from qwenforge_b200.cache import KvNeed
    need = KvNeed(1, 8, 9, pool=70)
    assert [need.first_kept(n) for n in (0, 5, 69, 70, 75, 139, 140, 150)] == [0, 0, 0, 62, 67, 70, 132, 140]
    assert KvNeed(1, 8, 37, pool=5).first_kept(100) == 64 and KvNeed(1, 8, 37).first_kept(100) == 64
    rows = KvNeed(1, 8, every=5)
    assert [rows.rows(n) for n in (0, 4, 5, 9, 10, 324)] == [0, 0, 1, 1, 2, 64]


def test_pages_leave_as_the_window_and_the_blocks_pass(reference_kernels, tmp_path):
    cfg = config(60, 16, 1e-6, [layer(pooled(2, 1, 8, 8, 20, 100, 2, 8), None), layer(gated(2, 1, 8, 8, 70, 8), None)])
    model, weights, _ = build(cfg, tmp_path)
    cache = model.new_cache(64 * 12, 2)
    kv = next(g for g in cache.kv_groups if g.need.pool == 100)
    rows = next(g for g in cache.kv_groups if g.need.every == 100)
    window = next(g for g in cache.kv_groups if g.need.window == 70)
    tokens = random_tokens(60, 330, 3)
    want = plain.forward_logits(cfg, weights, tokens)
    slot, got = cache.open(), []
    for at, size in ((0, 190), (190, 9), (199, 1), (200, 1), (201, 99), (300, 30)):
        got.append(model.step(cache, [(slot, tokens[at:at + size])], want=[list(range(size))]))
        n = at + size
        # positions stay for the window of 20 and until their block of 100 is complete
        assert kv.pages_held(slot) == (n - 1) // 64 - min(max(0, n - 19), n // 100 * 100) // 64 + 1, n
        assert rows.pages_held(slot) == (1 if n >= 100 else 0)
        assert window.pages_held(slot) == (n - 1) // 64 - max(0, n - 69) // 64 + 1
    assert max_err(torch.cat(got), want) < 1e-4
    cache.close(slot)
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_agrees_with_the_plain_implementation(reference_kernels, tmp_path, name):
    cfg = CONFIGS[name]
    model, weights, _ = build(cfg, tmp_path, seed=3)
    cache = model.new_cache(64 * 8, 2)
    tokens = random_tokens(cfg["vocab"], 150, 11)
    want = plain.forward_logits(cfg, weights, tokens)
    for cuts in ([150], [140], [2, 61, 2, 70, 3, 2], [75, 74]):
        assert max_err(run(model, cache, tokens, cuts), want) < 2e-4 * (1 + float(want.abs().max())), (name, cuts)
    assert all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_batches_in_slots_and_state_rows_used_before(reference_kernels, tmp_path):
    cfg = RAR_ODD
    model, weights, _ = build(cfg, tmp_path, seed=5)
    cache = model.new_cache(64 * 8, 3)
    seqs = [random_tokens(cfg["vocab"], n, 40 + n) for n in (90, 3, 41)]
    want = [plain.forward_logits(cfg, weights, s) for s in seqs]
    for round_ in range(2):
        slots = [cache.open() for _ in seqs]
        heads = [max(1, len(s) - 6) for s in seqs]
        logits = model.step(cache, [(slot, s[:h]) for slot, s, h in zip(slots, seqs, heads)], want=[[h - 1] for h in heads])
        for row, (s, h) in enumerate(zip(seqs, heads)):
            assert max_err(logits[row], want[row][h - 1]) < 1e-3, (round_, row)
        fed = list(heads)
        live = [i for i in range(3) if fed[i] < len(seqs[i])]
        while live:
            logits = model.step(cache, [(slots[i], [seqs[i][fed[i]]]) for i in live])
            for row, i in enumerate(live):
                assert max_err(logits[row], want[i][fed[i]]) < 1e-3, (round_, i, fed[i])
                fed[i] += 1
            live = [i for i in live if fed[i] < len(seqs[i])]
        for slot in slots:
            cache.close(slot)


def test_the_plain_window_and_blocks_end_where_they_should():
    """The plain implementation itself: a window one position longer, or blocks seen one position earlier, change the logits
    exactly from the position where the two masks part, under weights that make single keys stand out."""
    import copy
    cfg = config(70, 24, 1e-6, [layer(pooled(2, 1, 8, 8, 11, 4, 2, 8, 100.0, 2.0), None)])
    weights = plain.random_weights(cfg, 2)
    weights["l0.mix.q"] *= 3.0
    tokens = random_tokens(70, 40, 1)
    base = plain.forward_logits(cfg, weights, tokens)
    wider = copy.deepcopy(cfg)
    wider["layers"][0]["mixer"]["mask"]["size"] = 12
    d = (plain.forward_logits(wider, weights, tokens) - base).abs().max(-1).values
    assert float(d[:11].max()) < 1e-12 and float(d[11]) > 1e-4          # position 11 is the first that loses position 0
    # blocks of 4 behind a window of 11: block 0 (positions 0..3) is seen from position 14 on; tokens 0..2 are unseen at 11..13
    pool_off = copy.deepcopy(cfg)
    pool_off["layers"][0]["mixer"]["mask"]["pool"] = 3
    d = (plain.forward_logits(pool_off, weights, tokens) - base).abs().max(-1).values
    assert float(d[:13].max()) < 1e-12 and float(d[13]) > 1e-6          # blocks of 3: block 0 is seen from position 13 on


def test_greedy_generation_loop_on_the_cpu(reference_kernels, tmp_path):
    """The scheduler's batches through the package's generation loop (stepping, no graphs) against the plain greedy decoding."""
    from qwenforge_b200.engine import StudentEngine
    cfg = RAR_ONES
    folder, weights = make_model_dir(cfg, 6, tmp_path)
    prompts = [random_tokens(cfg["vocab"], n, n) for n in (5, 20, 1)]
    want = [plain.greedy_generate(cfg, weights, p, 6) for p in prompts]
    engine = StudentEngine(str(folder), device="cpu", dtype="float32", cuda_graphs=False)
    assert engine.generate_ids(prompts, max_new_tokens=6, batch_size=2, ignore_eos=True) == want
