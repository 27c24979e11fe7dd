"""Small Rarevik configurations for the tests, none with the sizes of any published model: they differ from one another in
every size, in the order of their layers and in which run of layers repeats."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from tests import plain_rarevik as plain


def pooled(heads, kv_heads, dim, vdim, size, pool, conv, rot_dims, base=10000.0, scale=None):
    return "attention", dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv, mask=dict(size=size, pool=pool),
                             rot=dict(dims=rot_dims, base=base), scale=scale if scale is not None else dim ** -0.5)


def gated(heads, kv_heads, dim, vdim, size, rot_dims, base=10000.0, scale=None, scaling=None):
    rot = dict(dims=rot_dims, base=base)
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return "attention_2", dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=size), rot=rot,
                               scale=scale if scale is not None else dim ** -0.5)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, limit, shared=None):
    m = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))
    if shared is not None:
        m["shared"] = dict(ff=shared[0], limit=shared[1])
    return m


def layer(mix, mlp):
    return dict(type=mix[0], mixer=mix[1], mlp=mlp)


def config(vocab, width, eps, layers, loop=None):
    cfg = dict(architecture="Rarevik", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# odd sizes everywhere; values wider than keys; a window shorter than its blocks and blocks longer than a page; the first
# layers repeat three times; a layer without a feed-forward
RAR_ODD = config(211, 52, 1e-5, [
    layer(pooled(4, 2, 10, 14, 37, 5, 2, 6, 5000.0, 0.9), moe(5, 2, 12, 2.0, (20, 1.5))),
    layer(gated(3, 3, 12, 8, 23, 8, 3000.0, 0.7, (8.0, 1.0, 4.0, 64)), dense(70)),
    layer(pooled(2, 1, 18, 6, 9, 70, 4, 18, 200.0, 0.5), None),
], loop=(0, 2, 3))
# sizes the vector and tensor-core kernels take; the middle layer repeats twice
RAR_FAST = config(384, 128, 1e-6, [
    layer(gated(4, 1, 64, 64, 100, 64, 100000.0, None, (4.0, 1.0, 2.0, 256)), dense(192)),
    layer(pooled(4, 1, 64, 64, 128, 32, 3, 64, 50000.0), moe(8, 2, 64, 1.0, (64, 1.0))),
    layer(gated(2, 2, 128, 128, 200, 32, 1000.0), moe(4, 1, 32, 3.0)),
], loop=(1, 2, 2))
# what other configurations make larger than 1 or unequal: one expert of one chosen, as many experts as are chosen, one query
# head per key head, blocks of one position behind a window of one, one tap, no rotation, no repeated run, no shared expert
RAR_ONES = config(97, 40, 1e-6, [
    layer(pooled(3, 3, 16, 8, 1, 1, 1, 0, 10000.0, 0.6), moe(1, 1, 24, 0.5)),
    layer(gated(2, 2, 8, 12, 1, 8, 300.0, 1.1), moe(3, 3, 10, 1.0, (8, 2.0))),
    layer(pooled(1, 1, 20, 20, 2, 3, 2, 4, 50.0, 0.4), dense(24)),
    layer(gated(5, 1, 8, 8, 7, 0), None),
])
# heads padded up to a size the tensor-core kernels take (keys of 96 beside values of 128, and the other way round), a window of
# several pages over blocks of one page, seven taps, one pass over the last layers (the mixing-in alone)
RAR_WIDE = config(150, 72, 1e-5, [
    layer(pooled(2, 2, 96, 128, 200, 64, 7, 48, 20000.0, 0.2), dense(80)),
    layer(gated(4, 2, 32, 16, 150, 16, 7000.0, 0.3, (2.0, 2.0, 16.0, 100)), moe(6, 3, 16, 1.5, (12, 0.7))),
    layer(pooled(6, 2, 128, 96, 70, 16, 3, 128, 100000.0, 0.1), None),
], loop=(1, 3, 1))

# larger sizes for long prompts: steps of more than a thousand tokens (the routing plan of long steps, windows over many pages,
# twenty experts of which four are chosen), three passes over the middle layers, heads padded from 80 and 48 to 80
RAR_LONG = config(1000, 320, 1e-6, [
    layer(gated(10, 2, 64, 64, 300, 64, 300000.0, None, (8.0, 1.0, 4.0, 1024)), dense(640)),
    layer(pooled(10, 2, 80, 48, 100, 32, 4, 80, 150000.0), moe(12, 3, 96, 1.25, (160, 2.0))),
    layer(pooled(5, 5, 64, 64, 130, 16, 2, 64, 10000.0), moe(12, 3, 96, 1.25, (160, 2.0))),
    layer(gated(8, 4, 128, 128, 520, 128, 300000.0), moe(20, 4, 48, 7.0)),
    layer(gated(10, 2, 64, 64, 300, 32, 1000.0), None),
], loop=(1, 4, 3))

CONFIGS = {"odd": RAR_ODD, "fast": RAR_FAST, "ones": RAR_ONES, "wide": RAR_WIDE}


def make_model_dir(cfg: dict, seed: int, folder=None, store_dtype=torch.float32, weights=None):
    """config.json + model.safetensors with the tests' own random weights; returns the folder and the float32 weights."""
    from qwenforge_b200.weights import save_safetensors

    folder = Path(folder or tempfile.mkdtemp(prefix="rar_model_"))
    folder.mkdir(parents=True, exist_ok=True)
    weights = plain.random_weights(cfg, seed) if weights is None else weights
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors(folder / "model.safetensors", {k: v.to(store_dtype) for k, v in weights.items()})
    return folder, weights
