"""Small Gatosun configurations and model folders for the tests (random weights of the tests' own making)."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import torch

from tests import plain_gatosun as plain


def attention(heads, kv_heads, dim, vdim, rot_dims, base=10000.0, scale=None, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=dict(dims=rot_dims, base=base), scale=scale or dim ** -0.5)
    if v_mix:
        m["v_mix"] = True
    return "attention", m


def parallel(heads, kv_heads, dim, vdim, size, rot_dims, r_heads, r_dim, left_scale=0.7, right_scale=1.2, base=10000.0, scale=None, rank=4):
    left = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, mask=dict(size=size), rot=dict(dims=rot_dims, base=base),
                scale=scale or 1.0)
    return "parallel", dict(left=left, left_scale=left_scale, right=dict(heads=r_heads, dim=r_dim, rank=rank), right_scale=right_scale)


def gla(heads, dim, vdim, tau=8.0, rank=4):
    return "gla", dict(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    out = dict(kind="moe", router=router, expert=dict(ff=ff))
    if shared:
        out["shared"] = dict(ff=shared)
    return out


def layer(mix, mlp):
    return dict(type=mix[0], mixer=mix[1], mlp=mlp)


def config(vocab, width, eps, mult, layers):
    return dict(architecture="Gatosun", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult, layers=layers)


# sizes that are multiples of nothing: padded heads both ways, odd widths, a window shorter than a page
GAT_ODD = config(53, 44, 1e-5, 0.6, [
    layer(gla(3, 10, 6, tau=5.0, rank=3), moe(6, 2, 14, groups=(3, 2), shared=10)),
    layer(attention(4, 2, 6, 10, 4, v_mix=True), dense(30)),
    layer(parallel(4, 2, 10, 6, 7, 6, 3, 6, rank=5), None),
    layer(attention(2, 2, 14, 10, 0, v_mix=True), moe(5, 5, 12)),
    layer(attention(6, 2, 8, 10, 8, scale=0.3, v_mix=True), moe(4, 1, 9, groups=(4, 1))),
])
# sizes that the tensor-core kernels and 16-byte paths take
GAT_FAST = config(320, 128, 1e-6, 0.8, [
    layer(parallel(4, 2, 64, 64, 48, 16, 4, 32, rank=8), dense(256)),
    layer(gla(4, 32, 64, tau=8.0, rank=8), moe(6, 2, 64, groups=(3, 1), shared=64)),
    layer(attention(8, 2, 64, 32, 32, v_mix=True), moe(8, 4, 64, groups=(4, 2))),
    layer(parallel(2, 2, 32, 32, 70, 32, 2, 64, rank=16), moe(8, 2, 64, shared=128)),
    layer(attention(8, 2, 32, 32, 16, v_mix=True), dense(128)),
])
# values that a given model may happen to make equal or 1
GAT_ONES = config(31, 32, 1e-5, 1.0, [
    layer(attention(1, 1, 16, 16, 16), moe(1, 1, 8)),
    layer(parallel(1, 1, 8, 8, 1, 0, 1, 8, left_scale=1.0, right_scale=1.0, rank=1), dense(8)),
    layer(gla(1, 8, 8, tau=1.0, rank=1), moe(2, 2, 8, groups=(1, 1))),
])

CONFIGS = {"odd": GAT_ODD, "fast": GAT_FAST, "ones": GAT_ONES}


def make_model_dir(cfg: dict, seed: int, folder=None, store_dtype=torch.float32, weights=None):
    """config.json + model.safetensors with the tests' own random weights; returns the folder and the float32 weights."""
    from qwenforge_b200.weights import save_safetensors

    folder = Path(folder or tempfile.mkdtemp(prefix="gat_model_"))
    folder.mkdir(parents=True, exist_ok=True)
    weights = plain.random_weights(cfg, seed) if weights is None else weights
    (folder / "config.json").write_text(json.dumps(cfg))
    save_safetensors(folder / "model.safetensors", {k: v.to(store_dtype) for k, v in weights.items()})
    return folder, weights
