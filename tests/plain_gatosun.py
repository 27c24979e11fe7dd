"""A plain, slow implementation of the Gatosun decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the package: the tests compare the package's kernels, cache, state and step function with it.
Every function works on ONE whole sequence from its position 0 (no cache, no state: earlier tokens are simply there).

The design, in this file's notation (t: a token at position p_t counted from 0; x: the stream; m: residual_mult):

  stream      x_t = E[token_t]
  layer       x <- x + m * mixer(rms(x; n1));  x <- x + m * ff(rms(x; n2))   (a layer may have no feed-forward)
  rms(v; w)   v / sqrt(mean(v^2) + eps) * w
  turn        the first `rot.dims` components of a head turn by p_t, component i with i + dims/2, angle p * base^(-2i/dims)
  attention   q, k, v = Wq h + bq, Wk h + bk, Wv h + bv;  q <- rms(q; wq), k <- rms(k; wk) over the WHOLE rows (all heads at
              once), then turned;  in every layer with v_mix but the first such:  v <- (1 - l) v + l v_first  (v_first: the
              first such layer's v of the same token, l a learned number);  s_ij = scale q_i . k_j for j <= i;  softmax;
              out = Wo concat_heads + bo
  parallel    a_left * left(h) + a_right * right(h), both reading the same h
    left      q, k, v = Wq h, Wk h, Wv h in heads;  q, k turned, then divided by their root mean square per head;
              s_ij = scale q_i . k_j for 0 <= i - j < size;  softmax;  out = Wo concat_heads
    right     with h' the token before (zeros at the start) each of r, k, v, g, w reads  h + (h' - h) mu_s;
              r, k, v = Wr., Wk., Wv. in heads of `dim`;  gate = silu(Wg .);  w = exp(-exp(W2 tanh(W1 .) + w0)) per head and channel;
              o_t = (S + diag(u) k_t v_t^T)^T r_t with S the state BEFORE this token;  S <- diag(w_t) S + k_t v_t^T;
              out = Wo ((o / rms_per_head(o)) * n * gate)
  gla         q = Wq h / sqrt(dim), k = Wk h, v = Wv h in heads;  a = sigmoid(A2 (A1 h) + b)^(1 / tau) per head and key channel;
              S <- diag(a_t) S + k_t v_t^T;  o_t = S^T q_t (the state AFTER this token);
              out = Wo (rms(o; n) per head over vdim, the weight shared by the heads, * silu(Wg h))
  dense ff    Wd (gelu_tanh(Wg h + bg) * (Wu h + bu)) + bd
  moe         z = R h;  s = sigmoid(z);  c = s + correction;  experts in `count` equal groups of neighbours, a group's score the
              sum of its two largest c;  only experts of the `keep` best groups may be chosen;  the `top` largest c among them;
              out = sum over the chosen of s_e * Wd_e relu(Wu_e h)^2  +  Wd_s relu(Wu_s h)^2   (the shared expert)
  logits      H rms(x; nf)
"""
from __future__ import annotations

import math

import torch

F = torch.float64


# ------------------------------------------------------------------ small pieces
def rms(v, w, eps):
    out = v / torch.sqrt(v.square().mean(-1, keepdim=True) + eps)
    return out if w is None else out * w.to(F)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def turn(x, positions, rot):
    """x [T, heads, dim]: the first rot.dims components of every head turned by the token's position."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat((u * cos - v * sin, v * cos + u * sin, x[..., dims:]), dim=-1)


def masked_softmax_attention(q, k, v, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, V]; query head h reads key/value head h // (H / G); window 0: every j <= i."""
    t, heads, _ = q.shape
    groups = k.shape[1]
    i, j = torch.arange(t)[:, None], torch.arange(t)[None, :]
    visible = (j <= i) if window <= 0 else ((j <= i) & (i - j < window))
    out = torch.zeros((t, heads, v.shape[-1]), dtype=F)
    for h in range(heads):
        g = h // (heads // groups)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


# ------------------------------------------------------------------ mixers
def full_attention(weights, p, m, h, eps, shared):
    """`shared`: what the layers with v_mix hand on within one forward pass (the first such layer's values)."""
    t = h.shape[0]
    heads, groups, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    w = lambda name: weights[p + name].to(F)
    q = h @ w("q").T + w("q.b")
    k = h @ w("k").T + w("k.b")
    v = h @ w("v").T + w("v.b")
    q, k = rms(q, w("q.norm"), eps), rms(k, w("k.norm"), eps)
    positions = torch.arange(t)
    q = turn(q.view(t, heads, dim), positions, m["rot"])
    k = turn(k.view(t, groups, dim), positions, m["rot"])
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = w("vmix")
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    o = masked_softmax_attention(q, k, v.view(t, groups, vdim), float(m["scale"]), 0)
    return o.reshape(t, heads * vdim) @ w("o").T + w("o.b")


def window_attention(weights, p, m, h, eps):
    t = h.shape[0]
    heads, groups, dim, vdim = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    w = lambda name: weights[p + name].to(F)
    positions = torch.arange(t)
    q = turn((h @ w("q").T).view(t, heads, dim), positions, m["rot"])
    k = turn((h @ w("k").T).view(t, groups, dim), positions, m["rot"])
    q, k = rms(q, None, eps), rms(k, None, eps)
    v = (h @ w("v").T).view(t, groups, vdim)
    o = masked_softmax_attention(q, k, v, float(m["scale"]), int(m["mask"]["size"]))
    return o.reshape(t, heads * vdim) @ w("o").T


def time_mix(weights, p, m, h, eps):
    t, width = h.shape
    heads, dim = int(m["heads"]), int(m["dim"])
    w = lambda name: weights[p + name].to(F)
    before = torch.cat((torch.zeros((1, width), dtype=F), h[:-1]), dim=0)
    mix = lambda s: h + (before - h) * w("mu." + s)
    r = (mix("r") @ w("r").T).view(t, heads, dim)
    k = (mix("k") @ w("k").T).view(t, heads, dim)
    v = (mix("v") @ w("v").T).view(t, heads, dim)
    gate = silu(mix("g") @ w("g").T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w("w1").T) @ w("w2").T + w("w0"))).view(t, heads, dim)
    u = w("u")                                               # [heads, dim]
    state = torch.zeros((heads, dim, dim), dtype=F)          # [head, key channel, value channel]
    out = torch.zeros((t, heads, dim), dtype=F)
    for i in range(t):
        kv = k[i][:, :, None] * v[i][:, None, :]
        out[i] = torch.einsum("hkv,hk->hv", state + u[:, :, None] * kv, r[i])
        state = decay[i][:, :, None] * state + kv
    out = rms(out, None, eps).reshape(t, heads * dim) * w("norm") * gate
    return out @ w("o").T


def gated_linear_attention(weights, p, m, h, eps):
    t = h.shape[0]
    heads, dim, vdim, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    w = lambda name: weights[p + name].to(F)
    q = (h @ w("q").T).view(t, heads, dim) * dim ** -0.5
    k = (h @ w("k").T).view(t, heads, dim)
    v = (h @ w("v").T).view(t, heads, vdim)
    z = (h @ w("a1").T) @ w("a2").T + w("a2.b")
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(t, heads, dim)
    state = torch.zeros((heads, dim, vdim), dtype=F)
    out = torch.zeros((t, heads, vdim), dtype=F)
    for i in range(t):
        state = alpha[i][:, :, None] * state + k[i][:, :, None] * v[i][:, None, :]
        out[i] = torch.einsum("hkv,hk->hv", state, q[i])
    out = rms(out, w("norm"), eps).reshape(t, heads * vdim) * silu(h @ w("g").T)
    return out @ w("o").T


def parallel_mixer(weights, p, m, h, eps):
    return float(m["left_scale"]) * window_attention(weights, p + "left.", m["left"], h, eps) \
        + float(m["right_scale"]) * time_mix(weights, p + "right.", m["right"], h, eps)


# ------------------------------------------------------------------ feed-forwards
def dense_ff(weights, p, h):
    w = lambda name: weights[p + name].to(F)
    return (gelu_tanh(h @ w("gate").T + w("gate.b")) * (h @ w("up").T + w("up.b"))) @ w("down").T + w("down.b")


def expert(weights, p, h):
    return torch.relu(h @ weights[p + "up"].to(F).T).square() @ weights[p + "down"].to(F).T


def router(weights, p, mlp, h):
    """Per token: the chosen experts (in falling order of their choice scores), their weights, and the margin between the
    last choice and the best one left out (among those that may be chosen, and between the groups)."""
    r = mlp["router"]
    experts, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    count, keep = int(groups["count"]), int(groups["keep"])
    size = experts // count
    s = torch.sigmoid(h @ weights[p + "router"].to(F).T)
    c = s + weights[p + "correction"].to(F)
    chosen, weight, margin = [], [], []
    for t in range(h.shape[0]):
        grouped = c[t].view(count, size)
        score = grouped.topk(min(2, size), dim=-1).values.sum(-1)
        order = torch.argsort(score, descending=True, stable=True)
        kept = order[:keep]
        gap = float(score[order[keep - 1]] - score[order[keep]]) if keep < count else float("inf")
        allowed = torch.full((experts,), float("-inf"), dtype=F)
        for g in kept.tolist():
            allowed[g * size:(g + 1) * size] = c[t, g * size:(g + 1) * size]
        ranked = torch.argsort(allowed, descending=True, stable=True)
        pick = ranked[:top]
        if top < keep * size:
            gap = min(gap, float(allowed[ranked[top - 1]] - allowed[ranked[top]]))
        chosen.append(pick)
        weight.append(s[t, pick])
        margin.append(gap)
    return torch.stack(chosen), torch.stack(weight), torch.tensor(margin, dtype=F)


def moe_ff(weights, p, mlp, h, margins=None):
    chosen, weight, margin = router(weights, p, mlp, h)
    if margins is not None:
        margins.append(margin)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t].tolist(), weight[t]):
            out[t] += w * expert(weights, f"{p}e{e}.", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + expert(weights, p + "shared.", h)
    return out


# ------------------------------------------------------------------ the model
def layer_forward(cfg, weights, index, x, shared, margins=None):
    layer = cfg["layers"][index]
    p, eps, mult = f"l{index}.", float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    h = rms(x, weights[p + "norm1"], eps)
    kind, m = layer["type"], layer["mixer"]
    if kind == "attention":
        y = full_attention(weights, p + "mix.", m, h, eps, shared)
    elif kind == "parallel":
        y = parallel_mixer(weights, p + "mix.", m, h, eps)
    elif kind == "gla":
        y = gated_linear_attention(weights, p + "mix.", m, h, eps)
    else:
        raise ValueError(kind)
    x = x + mult * y
    mlp = layer.get("mlp")
    if mlp is not None:
        h = rms(x, weights[p + "norm2"], eps)
        y = dense_ff(weights, p + "mlp.", h) if mlp["kind"] == "dense" else moe_ff(weights, p + "mlp.", mlp, h, margins)
        x = x + mult * y
    return x


def forward(cfg, weights, tokens, streams=None, margins=None):
    """Logits [T, vocab] of one whole sequence; `streams` collects the stream after every layer."""
    x = weights["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    shared = {}
    for index in range(len(cfg["layers"])):
        x = layer_forward(cfg, weights, index, x, shared, margins)
        if streams is not None:
            streams.append(x.clone())
    return rms(x, weights["final.norm"], float(cfg["norm"]["eps"])) @ weights["head"].to(F).T


def forward_logits(cfg, weights, tokens):
    return forward(cfg, weights, tokens)


def greedy_generate(cfg, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


# ------------------------------------------------------------------ shapes and random weights
def tensor_shapes(cfg):
    width, vocab = int(cfg["width"]), int(cfg["vocab"])
    shapes = {"embed": (vocab, width), "final.norm": (width,), "head": (vocab, width)}
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
        shapes[p + "norm1"] = (width,)
        if kind == "attention":
            hd, gd, gv, hv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"], m["heads"] * m["vdim"]
            shapes.update({p + "mix.q": (hd, width), p + "mix.q.b": (hd,), p + "mix.k": (gd, width), p + "mix.k.b": (gd,),
                           p + "mix.v": (gv, width), p + "mix.v.b": (gv,), p + "mix.q.norm": (hd,), p + "mix.k.norm": (gd,),
                           p + "mix.o": (width, hv), p + "mix.o.b": (width,)})
            if m.get("v_mix"):
                shapes[p + "mix.vmix"] = ()
        elif kind == "parallel":
            a, b = m["left"], m["right"]
            q = p + "mix.left."
            shapes.update({q + "q": (a["heads"] * a["dim"], width), q + "k": (a["kv_heads"] * a["dim"], width),
                           q + "v": (a["kv_heads"] * a["vdim"], width), q + "o": (width, a["heads"] * a["vdim"])})
            q, inner = p + "mix.right.", b["heads"] * b["dim"]
            rank = int(b["rank"])
            for s in "rkvgw":
                shapes[q + "mu." + s] = (width,)
            for s in "rkvg":
                shapes[q + s] = (inner, width)
            shapes.update({q + "w1": (rank, width), q + "w2": (inner, rank), q + "w0": (inner,), q + "u": (b["heads"], b["dim"]),
                           q + "norm": (inner,), q + "o": (width, inner)})
        else:
            hd, hv, rank = m["heads"] * m["dim"], m["heads"] * m["vdim"], int(m["rank"])
            q = p + "mix."
            shapes.update({q + "q": (hd, width), q + "k": (hd, width), q + "v": (hv, width), q + "g": (hv, width), q + "o": (width, hv),
                           q + "norm": (m["vdim"],), q + "a1": (rank, width), q + "a2": (hd, rank), q + "a2.b": (hd,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (width,)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            shapes.update({q + "gate": (ff, width), q + "gate.b": (ff,), q + "up": (ff, width), q + "up.b": (ff,),
                           q + "down": (width, ff), q + "down.b": (width,)})
        else:
            ff, n = mlp["expert"]["ff"], mlp["router"]["experts"]
            for e in range(n):
                shapes.update({f"{q}e{e}.up": (ff, width), f"{q}e{e}.down": (width, ff)})
            shapes.update({q + "router": (n, width), q + "correction": (n,)})
            if mlp.get("shared"):
                shapes.update({q + "shared.up": (mlp["shared"]["ff"], width), q + "shared.down": (width, mlp["shared"]["ff"])})
    return shapes


def random_weights(cfg, seed):
    """Weights that keep every mechanism alive: norms around one, decays spread over (0, 1), a correction that reorders."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        normal = lambda std, mean=0.0: (torch.randn(shape, generator=gen) * std + mean)
        if last in ("norm1", "norm2") or name.endswith(".norm") or name == "final.norm":
            t = normal(0.1, 1.0)
        elif ".mu." in name or last == "vmix":
            t = torch.rand(shape, generator=gen)
        elif last == "w0":
            t = normal(1.0, -1.0)
        elif last in ("w2", "a2"):
            t = normal(0.5)
        elif last == "u":
            t = normal(0.5)
        elif last == "correction":
            t = normal(0.3)
        elif last == "b":
            t = normal(1.0) if name.endswith("a2.b") else normal(0.1)
        elif last == "router":
            t = normal(0.3)
        elif name in ("embed",):
            t = normal(1.0)
        else:
            t = normal(shape[-1] ** -0.5)
        out[name] = t.to(torch.bfloat16).to(torch.float32)   # exact in both storage precisions
    return out
