"""A plain, slow implementation of the Rarevik decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the package: the tests compare the package's kernels, cache, state and step function with it.
Every function works on ONE whole sequence from its position 0 (no cache, no state: earlier tokens are simply there).

The design, in this file's notation (t: a token at position p_t counted from 0; x: the stream; e: the embedding output):

  stream      x_t = E[token_t];  e = x as the embedding leaves it
  schedule    layers 0 .. start-1, then layers start .. stop-1 `times` times over (same weights), then stop .. L-1;
              before the first layer of every pass:  x <- M [x ; e]   (M: [W, 2W], x's half first)
  layer       h = dyt(x; n1);  x <- x + (mixer(shift(h)) + ff(h))     (both sublayers read the one norm)
  dyt(v; n)   tanh(alpha v) * w + b   (no mean, no variance)
  shift(h)_t  h_t + (h_t-1 - h_t) * s   element by element, h_-1 = 0
  conv(u)_t   sum_j c[:, j] u_(t - taps + 1 + j), zeros before the start, per channel
  rms(v; w)   v / sqrt(mean(v^2) + eps) * w
  attention   q, k, v = conv(Wq h), conv(Wk h), conv(Wv h) in heads;  q <- rms(q; wq), k <- rms(k; wk) per head;
              the first `rot.dims` components of q and k turn by p_t, component i with i + dims/2, angle p * base^(-2i/dims);
              s_ij = scale q_i . k_j for 0 <= i - j < size;  and one pooled key and value per block b of P positions with
              bP + P - 1 <= i - size: the means of the block's keys (as kept: normed and turned) and of its values;
              weights = exp(s) / (exp(sink_head) + sum over visible tokens and blocks of exp(s));  out = Wo concat_heads
  attention_2 q, k, v = Wq h, Wk h, Wv h in heads; q and k turn by p_t, component 2i with 2i + 1, with frequencies rescaled
              by wavelength (below);  s_ij = scale q_i . k_j for 0 <= i - j < size; an ordinary softmax;
              head's output * sigmoid(Wg h)_head;  out = Wo concat_heads
  dense ff    Wd gelu(Wu h), the erf form
  expert(h)   g = min(Wg h, limit), u = clamp(Wu h, -limit, limit);  Wd (g * sigmoid(1.702 g) * (u + 1))
  moe         z = R h + r;  the `top` largest z are chosen, their weights the softmax over the chosen z alone;
              out = sum of weight * expert_e(h)  +  sigmoid(Wsg h) * shared(h)     (shared: one more expert with its own sizes)
  logits      E dyt(x; nf)
"""
from __future__ import annotations

import math

import torch

F = torch.float64
EXPERT_GATE_SLOPE = 1.702


# ------------------------------------------------------------------ small pieces
def dyt(v, weights, name):
    return torch.tanh(weights[name + ".alpha"].to(F) * v) * weights[name].to(F) + weights[name + ".b"].to(F)


def token_shift(h, s):
    before = torch.cat((torch.zeros_like(h[:1]), h[:-1]), dim=0)
    return h + (before - h) * s.to(F)


def short_conv(u, c):
    """u [T, C], c [C, taps]:  y_t = sum_j c[:, j] * u_(t - taps + 1 + j)."""
    taps = c.shape[1]
    padded = torch.cat((torch.zeros((taps - 1, u.shape[1]), dtype=F), u), dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + c[:, j].to(F) * padded[j:j + u.shape[0]]
    return y


def rms(v, w, eps):
    return v / torch.sqrt((v * v).mean(dim=-1, keepdim=True) + eps) * w.to(F)


def frequencies(rot):
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        factor, low, high, original = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for fi in f:
            wavelength = 2.0 * math.pi / fi
            if wavelength < original / high:
                out.append(fi)
            elif wavelength > original / low:
                out.append(fi / factor)
            else:
                s = (original / wavelength - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F)


def rotate(x, positions, rot, interleaved):
    """x [T, heads, dim]; the first rot.dims components of every head turn by the token's position."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    angle = positions.to(F)[:, None, None] * frequencies(rot)
    cos, sin = angle.cos(), angle.sin()
    if interleaved:
        u, w = x[..., 0:dims:2], x[..., 1:dims:2]
        turned = torch.stack((u * cos - w * sin, w * cos + u * sin), dim=-1).flatten(-2)
    else:
        u, w = x[..., :dims // 2], x[..., dims // 2:dims]
        turned = torch.cat((u * cos - w * sin, w * cos + u * sin), dim=-1)
    return torch.cat((turned, x[..., dims:]), dim=-1)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


# ------------------------------------------------------------------ mixers
def pooled_window_attention(weights, p, m, h, eps):
    """The mixer 'attention' on a whole sequence h [T, W] (already shifted)."""
    t, heads, g, dim, vdim = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    size, pool = int(m["mask"]["size"]), int(m["mask"]["pool"])
    positions = torch.arange(t)
    q = short_conv(h @ weights[p + "q"].to(F).T, weights[p + "q.conv"]).view(t, heads, dim)
    k = short_conv(h @ weights[p + "k"].to(F).T, weights[p + "k.conv"]).view(t, g, dim)
    v = short_conv(h @ weights[p + "v"].to(F).T, weights[p + "v.conv"]).view(t, g, vdim)
    q = rotate(rms(q, weights[p + "q.norm"], eps), positions, m["rot"], False)
    k = rotate(rms(k, weights[p + "k.norm"], eps), positions, m["rot"], False)
    n_blocks = t // pool
    pooled_k = k[:n_blocks * pool].view(n_blocks, pool, g, dim).mean(dim=1)
    pooled_v = v[:n_blocks * pool].view(n_blocks, pool, g, vdim).mean(dim=1)
    sink = weights[p + "sink"].to(F)
    out = torch.zeros((t, heads, vdim), dtype=F)
    per = heads // g
    for i in range(t):
        first = max(0, i - size + 1)
        seen = max(0, (i - size + 1) // pool)          # blocks b with b * pool + pool - 1 <= i - size
        keys = torch.cat((pooled_k[:seen], k[first:i + 1]), dim=0).repeat_interleave(per, dim=1)      # [n, heads, dim]
        values = torch.cat((pooled_v[:seen], v[first:i + 1]), dim=0).repeat_interleave(per, dim=1)
        s = torch.einsum("nhd,hd->hn", keys, q[i]) * float(m["scale"])
        top = torch.maximum(s.max(dim=1).values, sink)
        e = torch.exp(s - top[:, None])
        out[i] = torch.einsum("hn,nhd->hd", e, values) / (e.sum(dim=1) + torch.exp(sink - top))[:, None]
    return out.reshape(t, heads * vdim) @ weights[p + "o"].to(F).T


def gated_window_attention(weights, p, m, h):
    """The mixer 'attention_2' on a whole sequence h [T, W] (already shifted)."""
    t, heads, g, dim, vdim = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    size = int(m["mask"]["size"])
    positions = torch.arange(t)
    q = rotate((h @ weights[p + "q"].to(F).T).view(t, heads, dim), positions, m["rot"], True)
    k = rotate((h @ weights[p + "k"].to(F).T).view(t, g, dim), positions, m["rot"], True)
    v = (h @ weights[p + "v"].to(F).T).view(t, g, vdim)
    gate = torch.sigmoid(h @ weights[p + "g"].to(F).T)     # [T, heads]
    out = torch.zeros((t, heads, vdim), dtype=F)
    per = heads // g
    for i in range(t):
        first = max(0, i - size + 1)
        s = torch.einsum("nhd,hd->hn", k[first:i + 1].repeat_interleave(per, dim=1), q[i]) * float(m["scale"])
        out[i] = torch.einsum("hn,nhd->hd", torch.softmax(s, dim=1), v[first:i + 1].repeat_interleave(per, dim=1)) * gate[i][:, None]
    return out.reshape(t, heads * vdim) @ weights[p + "o"].to(F).T


# ------------------------------------------------------------------ feed-forwards
def dense_ff(weights, p, h):
    return gelu_erf(h @ weights[p + "up"].to(F).T) @ weights[p + "down"].to(F).T


def expert(weights, p, h, limit):
    g = torch.clamp(h @ weights[p + "gate"].to(F).T, max=limit)
    u = torch.clamp(h @ weights[p + "up"].to(F).T, min=-limit, max=limit)
    return (g * torch.sigmoid(EXPERT_GATE_SLOPE * g) * (u + 1.0)) @ weights[p + "down"].to(F).T


def router(weights, p, h, top):
    """Chosen experts [T, top] and their weights; also the margin between the last chosen and the first left out."""
    z = h @ weights[p + "router"].to(F).T + weights[p + "router.b"].to(F)
    ordered, index = torch.sort(z, dim=-1, descending=True, stable=True)
    chosen, logits = index[:, :top], ordered[:, :top]
    margin = ordered[:, top - 1] - ordered[:, top] if z.shape[1] > top else torch.full((z.shape[0],), float("inf"), dtype=F)
    return chosen, torch.softmax(logits, dim=-1), margin


def moe_ff(weights, p, mlp, h, margins=None):
    top, limit = int(mlp["router"]["top"]), float(mlp["expert"]["limit"])
    chosen, weight, margin = router(weights, p, h, top)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros((h.shape[0], weights[p + "e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        for k in range(top):
            out[t] += weight[t, k] * expert(weights, f"{p}e{int(chosen[t, k])}.", h[t:t + 1], limit)[0]
    shared = mlp.get("shared")
    if shared:
        gate = torch.sigmoid(h @ weights[p + "shared.sg"].to(F).T)     # [T, 1]
        out = out + gate * expert(weights, p + "shared.", h, float(shared["limit"]))
    return out


# ------------------------------------------------------------------ the model
def schedule(cfg):
    """Layer indices in the order they run, and which runs are the first of a pass."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for _ in range(times):
        runs += [(i, i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def layer_forward(cfg, weights, index, x, margins=None):
    layer, p = cfg["layers"][index], f"l{index}."
    h = dyt(x, weights, p + "norm1")
    shifted = token_shift(h, weights[p + "shift"])
    if layer["type"] == "attention":
        mixed = pooled_window_attention(weights, p + "mix.", layer["mixer"], shifted, float(cfg["norm"]["eps"]))
    elif layer["type"] == "attention_2":
        mixed = gated_window_attention(weights, p + "mix.", layer["mixer"], shifted)
    else:
        raise ValueError(layer["type"])
    mlp = layer.get("mlp")
    if mlp is None:
        return x + mixed
    ff = dense_ff(weights, p + "mlp.", h) if mlp["kind"] == "dense" else moe_ff(weights, p + "mlp.", mlp, h, margins)
    return x + (mixed + ff)


def forward(cfg, weights, tokens, streams=None, margins=None):
    """Logits [T, vocab] of one whole sequence; `streams` collects the stream after every layer run."""
    table = weights["embed"].to(F)
    x = table[torch.as_tensor(tokens, dtype=torch.long)]
    e = x
    for index, first_of_pass in schedule(cfg):
        if first_of_pass:
            x = torch.cat((x, e), dim=-1) @ weights["loop.in"].to(F).T
        x = layer_forward(cfg, weights, index, x, margins)
        if streams is not None:
            streams.append(x)
    return dyt(x, weights, "final.norm") @ table.T


def forward_logits(cfg, weights, tokens):
    return forward(cfg, weights, tokens)


def greedy_generate(cfg, weights, prompt, n_new):
    tokens, out = list(prompt), []
    for _ in range(n_new):
        out.append(int(forward(cfg, weights, tokens)[-1].argmax()))
        tokens.append(out[-1])
    return out


# ------------------------------------------------------------------ random weights for the tests
def tensor_shapes(cfg):
    w = int(cfg["width"])
    shapes = {"embed": (int(cfg["vocab"]), w), "final.norm": (w,), "final.norm.b": (w,), "final.norm.alpha": ()}
    if cfg.get("loop"):
        shapes["loop.in"] = (w, 2 * w)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        heads, g, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
        shapes.update({p + "norm1": (w,), p + "norm1.b": (w,), p + "norm1.alpha": (), p + "shift": (w,),
                       p + "mix.q": (heads * dim, w), p + "mix.k": (g * dim, w), p + "mix.v": (g * vdim, w),
                       p + "mix.o": (w, heads * vdim)})
        if layer["type"] == "attention":
            taps = int(m["conv"])
            shapes.update({p + "mix.q.norm": (dim,), p + "mix.k.norm": (dim,), p + "mix.sink": (heads,),
                           p + "mix.q.conv": (heads * dim, taps), p + "mix.k.conv": (g * dim, taps),
                           p + "mix.v.conv": (g * vdim, taps)})
        else:
            shapes[p + "mix.g"] = (heads, w)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (int(mlp["ff"]), w), p + "mlp.down": (w, int(mlp["ff"]))})
            continue
        experts, ff = int(mlp["router"]["experts"]), int(mlp["expert"]["ff"])
        shapes.update({p + "mlp.router": (experts, w), p + "mlp.router.b": (experts,)})
        for e in range(experts):
            shapes.update({f"{p}mlp.e{e}.gate": (ff, w), f"{p}mlp.e{e}.up": (ff, w), f"{p}mlp.e{e}.down": (w, ff)})
        if mlp.get("shared"):
            sf = int(mlp["shared"]["ff"])
            shapes.update({p + "mlp.shared.gate": (sf, w), p + "mlp.shared.up": (sf, w), p + "mlp.shared.down": (w, sf),
                           p + "mlp.shared.sg": (1, w)})
    return shapes


def random_weights(cfg, seed):
    """Weights that keep the stream and every branch alive: matrices of variance 1 / inputs, norms near 1, shifts in
    (0, 1), taps of about equal weight, sinks and router biases of order 1. All are bfloat16 numbers kept as float32."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            value = torch.tensor(0.6) + 0.2 * torch.rand((), generator=gen)
        elif name.endswith("norm1") or name.endswith("final.norm") or name.endswith(".norm"):
            value = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif last == "b" and "router" not in name:
            value = 0.1 * torch.randn(shape, generator=gen)
        elif last == "b":
            value = 0.5 * torch.randn(shape, generator=gen)
        elif last == "shift":
            value = torch.rand(shape, generator=gen)
        elif last == "conv":
            value = (1.0 + 0.5 * torch.randn(shape, generator=gen)) / shape[1] ** 0.5
        elif last == "sink":
            value = torch.randn(shape, generator=gen)
        elif name == "embed":
            value = torch.randn(shape, generator=gen)
        elif name == "loop.in":
            value = torch.randn(shape, generator=gen) / (shape[1] / 2) ** 0.5
        elif last == "router":
            value = 2.0 * torch.randn(shape, generator=gen) / shape[1] ** 0.5
        else:
            value = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        out[name] = value.to(torch.bfloat16).to(torch.float32)
    return out
