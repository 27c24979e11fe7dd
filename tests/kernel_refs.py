"""Plain PyTorch references of every CUDA kernel, with the kernels' own signatures.

Each function states in tensor operations what its kernel computes; the `-m gpu` tests compare the
two on the same inputs. The functions work on any device, so the CPU tests can also put them in
the kernels' place (`conftest.reference_kernels`) to exercise the step function, the cache and the
generation loop without a GPU. They are test code: the package never imports them.
"""
from __future__ import annotations

import torch

from tests import plain_qwen2 as plain

PAGE = 64


def _f(t):
    return t.to(torch.float64)


def embed_gather(ids, table, out, err):
    out.copy_(table[ids.long()].to(torch.float32))


def gather_rows(hidden, delta, rows, out, err):
    picked = hidden[rows.long()]
    if delta is not None:
        picked = picked + delta[rows.long()].to(torch.float32)
    out.copy_(picked)


def gather_rows_norm(hidden, delta, rows, weight, eps, out, err):
    picked = hidden[rows.long()]
    if delta is not None:
        picked = picked + delta[rows.long()].to(torch.float32)
    x = _f(picked)
    out.copy_((x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)).to(out.dtype))


def add_rms_norm(hidden, delta, weight, eps, out):
    if delta is not None:
        hidden += delta.to(torch.float32)
    x = _f(hidden)
    normed = x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)
    out.copy_(normed.to(out.dtype))


def gemm_f32(x, weight, bias, out):
    y = _f(x) @ _f(weight).T
    if bias is not None:
        y = y + _f(bias)
    out.copy_(y.to(out.dtype))


def linear(x, weight, bias=None, out=None, out_dtype=None):
    y = _f(x) @ _f(weight).T
    if bias is not None:
        y = y + _f(bias)
    y = y.to(out_dtype or x.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def _kv_rows(site, slot, positions, head, which):
    """storage rows of `positions` (list) for one head: returns (page ids, offsets)."""
    pages = site.table[slot, torch.as_tensor(positions, device=site.table.device) // PAGE].long()
    offs = torch.as_tensor(positions, device=site.table.device) % PAGE
    return pages, offs


def rope_cache_write(qkv, tok_seq, tok_pos, slots, inv_freq, rot_dim, n_heads, q_out, site, write_cache, err, bias=None,
                     unit_norm_eps=None, norm_dim=0, has_kv=True, interleaved=False, norm_first=False, q_norm=None, k_norm=None):
    n = qkv.shape[0]
    d, kvh = site.head_dim, site.kv_heads
    x = _f(qkv)[:, :(n_heads + (2 * kvh if has_kv else 0)) * d]
    if bias is not None:
        x = x + _f(bias)
    q = x[:, :n_heads * d].reshape(n, n_heads, d).clone()
    if has_kv:
        k = x[:, n_heads * d:(n_heads + kvh) * d].reshape(n, kvh, d).clone()
        v = x[:, (n_heads + kvh) * d:].reshape(n, kvh, d)
    else:
        k, v = q[:, :0].clone(), None
    if unit_norm_eps is not None and norm_first:
        over = norm_dim or d
        for t, w in ((q, q_norm), (k, k_norm)):
            t[..., :over] = t[..., :over] / torch.sqrt(t[..., :over].square().mean(-1, keepdim=True) + unit_norm_eps) \
                * (1.0 if w is None else _f(w))
    if inv_freq is not None and rot_dim > 0 and interleaved:
        angle = (tok_pos.to(torch.float32).unsqueeze(-1) * inv_freq.to(torch.float32)).to(torch.float64)
        cos, sin = angle.cos().unsqueeze(1), angle.sin().unsqueeze(1)
        for t in (q, k):
            x1, x2 = t[..., 0:rot_dim:2].clone(), t[..., 1:rot_dim:2].clone()
            t[..., 0:rot_dim:2] = x1 * cos - x2 * sin
            t[..., 1:rot_dim:2] = x2 * cos + x1 * sin
    elif inv_freq is not None and rot_dim > 0:
        angle = (tok_pos.to(torch.float32).unsqueeze(-1) * inv_freq.to(torch.float32)).to(torch.float64)
        cos, sin = angle.cos().unsqueeze(1), angle.sin().unsqueeze(1)
        half = rot_dim // 2
        for t in (q, k):
            x1, x2 = t[..., :half].clone(), t[..., half:rot_dim].clone()
            t[..., :half] = x1 * cos - x2 * sin
            t[..., half:rot_dim] = x2 * cos + x1 * sin
    if unit_norm_eps is not None and not norm_first:
        over = norm_dim or d
        for t in (q, k):
            t /= torch.sqrt(t[..., :over].square().mean(-1, keepdim=True) + unit_norm_eps)
    q_out.copy_(q.reshape(n, n_heads * d).to(q_out.dtype))
    if not write_cache:
        return
    for t in range(n):
        slot = int(slots[int(tok_seq[t])])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        page = int(site.table[slot, pos // PAGE])
        assert page >= 0, "reference: write to a page that is not held"
        site.storage[page, 0, :, pos % PAGE, :] = k[t].to(site.storage.dtype)
        site.storage[page, 1, :, pos % PAGE, :] = v[t].to(site.storage.dtype)


def gather_kv(site, slot, lo, hi):
    """Keys and values of positions lo..hi-1 of `slot`: two [kv_heads, hi-lo, head_dim] float64 tensors."""
    pos = torch.arange(lo, hi, device=site.table.device)
    pages = site.table[slot, pos // PAGE].long()
    assert bool((pages >= 0).all()), "reference: read of a page that is not held"
    k = site.storage[pages, 0, :, pos % PAGE, :]  # [n, kvh, d]
    v = site.storage[pages, 1, :, pos % PAGE, :]
    return _f(k).transpose(0, 1), _f(v).transpose(0, 1)


def gather_keys(site, slot, lo, hi):
    """Rows lo..hi-1 of a one-plane cache: [kv_heads, hi-lo, head_dim] float64."""
    pos = torch.arange(lo, hi, device=site.table.device)
    pages = site.table[slot, pos // PAGE].long()
    assert bool((pages >= 0).all()), "reference: read of a page that is not held"
    return _f(site.storage[pages, 0, :, pos % PAGE, :]).transpose(0, 1)


def attention_generic(q, out, cu_q, tok_pos, slots, site, n_heads, n_seqs, max_q_len, scale, window, err, scratch=None, max_kv_len=None,
                      sinks=None, shared_values=False, chunk=0, softcap=0.0, blocks=None, pool=0):
    d, kvh = site.head_dim, site.kv_heads
    groups = n_heads // kvh
    for s in range(n_seqs):
        b, e = int(cu_q[s]), int(cu_q[s + 1])
        slot = int(slots[s])
        if slot < 0:
            out[b:e] = 0
            continue
        for t in range(b, e):
            p = int(tok_pos[t])
            lo = max(0, p - window + 1) if window > 0 else 0
            if chunk > 0:
                lo = max(lo, p // chunk * chunk)
            if shared_values:
                k = v = gather_keys(site, slot, lo, p + 1)
            else:
                k, v = gather_kv(site, slot, lo, p + 1)
            if pool > 0 and p - window + 1 >= pool:   # the rows of the blocks that lie wholly before the window
                bk, bv = gather_kv(blocks, slot, 0, (p - window + 1) // pool)
                k, v = torch.cat((bk, k), dim=1), torch.cat((bv, v), dim=1)
            qt = _f(q[t]).view(n_heads, d)
            k = k.repeat_interleave(groups, dim=0)
            v = v.repeat_interleave(groups, dim=0)
            scores = torch.einsum("hd,hjd->hj", qt, k) * scale
            if softcap > 0:
                scores = softcap * torch.tanh(scores / softcap)
            if sinks is not None:   # one more term in the denominator, with no value
                weights = torch.softmax(torch.cat((scores, _f(sinks)[:, None]), dim=-1), -1)[:, :-1]
            else:
                weights = torch.softmax(scores, -1)
            ctx = torch.einsum("hj,hjd->hd", weights, v)
            out[t] = ctx.reshape(-1).to(out.dtype)


def swiglu(gate_up, out):
    inter = gate_up.shape[1] // 2
    g, u = _f(gate_up[:, :inter]), _f(gate_up[:, inter:])
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def sample(logits, temperature, seed, seq_ids, steps, out, scratch=None):
    for r in range(logits.shape[0]):
        token, _ = plain.sample_token(logits[r].cpu(), temperature, seed,
                                      int(seq_ids[r]) if seq_ids is not None else 0,
                                      int(steps[r]) if steps is not None else 0)
        out[r] = token


def _rms(x, weight, eps):
    x = _f(x)
    return x * torch.rsqrt(x.square().mean(-1, keepdim=True) + eps) * _f(weight)


def embed_positions(ids, tok_pos, table, positions, out, err):
    out.copy_((_f(table[ids.long()]) + _f(positions[tok_pos.long()])).to(torch.float32))


def sandwich_norm(hidden, y, post_weight, post_eps, next_weight=None, next_eps=0.0, out=None, dest=None, top=1, row_weight=None):
    if dest is not None:
        y = _f(y) if row_weight is None else _f(y) * _f(row_weight)[:, None]
        y = y[dest.long()].view(-1, top, y.shape[1]).sum(1)
    hidden += _rms(y, post_weight, post_eps).to(torch.float32)
    if next_weight is not None:
        out.copy_(_rms(hidden, next_weight, next_eps).to(out.dtype))


def clamped_glu(gate_up, limit, alpha, out):
    inter = gate_up.shape[1] // 2
    g = _f(gate_up[:, :inter]).clamp(max=limit)
    u = _f(gate_up[:, inter:]).clamp(min=-limit, max=limit)
    out.copy_((g * torch.sigmoid(alpha * g) * (u + 1)).to(out.dtype))


def latent_norm_cache(down, q_rank, q_norm, kv_norm, eps, tok_seq, tok_pos, slots, q_latent, site, write_cache, err, latent_out=None):
    if q_rank:
        q_latent.copy_(_rms(down[:, :q_rank], q_norm, eps).to(q_latent.dtype))
    c = _rms(down[:, q_rank:], kv_norm, eps)
    if latent_out is not None:
        latent_out.copy_(c.to(latent_out.dtype))
    if not write_cache:
        return
    for t in range(down.shape[0]):
        slot = int(slots[int(tok_seq[t])])
        if slot < 0:
            continue
        pos = int(tok_pos[t])
        page = int(site.table[slot, pos // PAGE])
        assert page >= 0, "reference: write to a page that is not held"
        site.storage[page, 0, 0, pos % PAGE, :] = c[t].to(site.storage.dtype)


def head_linear(x, weight, out):
    groups, n, k = weight.shape
    y = torch.einsum("tgk,gnk->tgn", _f(x).view(x.shape[0], groups, k), _f(weight))
    out.copy_(y.reshape(x.shape[0], groups * n).to(out.dtype))


class _Routing:
    pass


def linear_rows(x, weight, out_dtype=None):
    return linear(x, weight, None, out_dtype=out_dtype)


def moe_tile_rows(n_tokens, n_experts, top, weight):
    return 64


def expert_gate_takes(x, weight, plan):
    return False


def tc_gemm_grouped(epilogue, x, weight, plan, out, row_scale=None, err=None, clamp=None):
    y = torch.einsum("rk,rnk->rn", _f(x), _f(weight)[plan.row_expert])
    if epilogue == 1:   # gate rows then up rows, a scale on both before the gate
        inter = y.shape[1] // 2
        s = _f(row_scale)[:, None] if row_scale is not None else 1.0
        g, u = y[:, :inter] * s, y[:, inter:] * s
        if clamp is not None:
            g, u = g.clamp(max=clamp[0]), u.clamp(min=-clamp[0], max=clamp[0]) + 1
            y = g * torch.sigmoid(clamp[1] * g) * u
        else:
            y = g * torch.sigmoid(g) * u
    out.copy_(y.to(out.dtype))


def scaled_swiglu(gate_up, row_scale, out):
    inter = gate_up.shape[1] // 2
    g, u = _f(gate_up[:, :inter]) * _f(row_scale)[:, None], _f(gate_up[:, inter:]) * _f(row_scale)[:, None]
    out.copy_((g * torch.sigmoid(g) * u).to(out.dtype))


def moe_plan(logits, top, softmax_scores=False, renormalize=False, tile_rows=64, x=None, router=None, bias=None, correction=None,
             groups=None):
    if logits is None:
        logits = (_f(x) @ _f(router).T)
    z = logits.to(torch.float32)
    if bias is not None:
        z = z + bias.to(torch.float32)
    scores = torch.softmax(z, -1) if softmax_scores else torch.sigmoid(z)
    if correction is not None or groups is not None:
        choice = scores if correction is None else scores + correction.to(torch.float32)
        count, keep = groups if groups is not None else (1, 1)
        if keep < count:
            grouped = choice.view(z.shape[0], count, -1)
            group_score = grouped.topk(min(2, grouped.shape[-1]), dim=-1).values.sum(-1)
            kept = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, group_score.topk(keep, dim=-1).indices, True)
            choice = grouped.masked_fill(~kept[:, :, None], float("-inf")).reshape(z.shape)
        picked = torch.topk(choice, top, dim=-1).indices
        chosen = torch.return_types.topk((scores.gather(1, picked), picked))
    else:
        chosen = torch.topk(scores, top, dim=-1)
    weights = chosen.values / chosen.values.sum(-1, keepdim=True) if renormalize else chosen.values
    plan = _Routing()
    plan.n_tokens, plan.n_experts, plan.top, plan.pairs = z.shape[0], z.shape[1], top, z.shape[0] * top
    experts = chosen.indices.reshape(-1)
    order = torch.sort(experts, stable=True).indices                    # rows: pairs sorted by expert
    plan.sorted_token = (order // top).to(torch.int32)
    plan.sorted_weight = weights.reshape(-1)[order].to(torch.float32)
    plan.row_expert = experts[order]
    plan.dest = torch.empty(plan.pairs, dtype=torch.int32)
    plan.dest[order] = torch.arange(plan.pairs, dtype=torch.int32)
    return plan


def moe_gather(x, plan, out, scale_input):
    rows = _f(x)[plan.sorted_token.long()]
    if scale_input:
        rows = rows * _f(plan.sorted_weight)[:, None]
    out.copy_(rows.to(out.dtype))


def moe_combine(y, plan, out, scale_output, extra=None, extra_gate=None, gate_input=None, gate_weight=None):
    if gate_weight is not None:
        extra_gate = _f(gate_input) @ _f(gate_weight)
    rows = _f(y)
    if scale_output:
        rows = rows * _f(plan.sorted_weight)[:, None]
    total = rows[plan.dest.long()].view(plan.n_tokens, plan.top, -1).sum(1)
    if extra is not None:
        total = total + _f(extra) * (1.0 if extra_gate is None else torch.sigmoid(_f(extra_gate)).view(-1, 1))
    out.copy_(total.to(out.dtype))


def expert_linear(x, weight, plan, out, gather=False, activation=None):
    rows = _f(x)[plan.sorted_token.long()] if gather else _f(x)
    y = torch.einsum("rk,rnk->rn", rows, _f(weight)[plan.row_expert])
    out.copy_((y if activation is None else _act(y, activation)).to(out.dtype))


def bias_act(x, bias, kind, out):
    z = _f(x) if bias is None else _f(x) + _f(bias)
    if kind == "relu2":
        y = torch.relu(z) ** 2
    elif kind == "gelu_tanh":
        y = 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    elif kind == "silu":
        y = z * torch.sigmoid(z)
    elif kind == "gelu":
        y = 0.5 * z * (1 + torch.erf(z / 2 ** 0.5))
    elif kind == "tanh":
        y = torch.tanh(z)
    else:
        y = torch.relu(z)
    out.copy_(y.to(out.dtype))


def _act(z, kind):
    out = torch.empty_like(z)
    bias_act(z, None, kind, out)
    return out


def bias_glu(gate_up, bias, kind, out):
    inter = out.shape[1]
    z = _f(gate_up) if bias is None else _f(gate_up) + _f(bias)
    out.copy_((_act(z[:, :inter], kind) * z[:, inter:]).to(out.dtype))


def add_rms_norm_scaled(hidden, a, scale_a, b, scale_b, weight, eps, out):
    residual_add_scaled(hidden, a, scale_a, b, scale_b)
    out.copy_(_rms(hidden, weight, eps).to(out.dtype))


def residual_add_scaled(hidden, a, scale_a, b=None, scale_b=0.0):
    t = scale_a * _f(a)
    if b is not None:
        t = t + scale_b * _f(b)
    hidden.add_(t.to(torch.float32))


def rms_norm_cols(x, runs, eps):
    for col0, width, count, weight in runs:
        v = _f(x[:, col0:col0 + width])
        x[:, col0:col0 + width] = (v / torch.sqrt(v.square().sum(-1, keepdim=True) / count + eps) * _f(weight)).to(x.dtype)


def mix_rows(x, other, heads, size, x_head, other_head, weight):
    for h in range(heads):
        mine, theirs = x[:, h * x_head:h * x_head + size], other[:, h * other_head:h * other_head + size]
        mine.copy_(((1.0 - weight) * _f(mine) + weight * _f(theirs)).to(x.dtype))


def rows_prepare(x, runs, eps, mix=None):
    for index, (col0, width, count, bias, weight) in enumerate(runs):
        view = x[:, col0:col0 + width]
        if bias is not None:
            view.copy_((_f(view) + _f(bias)).to(x.dtype))
        if mix is not None and mix[0] == index:
            _, other, size, x_head, other_head, lam = mix
            mix_rows(view, other, -(-width // x_head), size, x_head, other_head, lam)
        if count > 0:
            rms_norm_cols(x, ((col0, width, count, weight),), eps)


def shift_mix(h, mu, cu_q, tok_seq, slots, state, offset, out, single=False):
    width = h.shape[1]
    for s in range(cu_q.numel() - 1):
        begin, end, slot = int(cu_q[s]), int(cu_q[s + 1]), int(slots[s])
        if end <= begin:
            continue
        first = _f(state[slot, offset:offset + width]) if slot >= 0 else torch.zeros(width, dtype=torch.float64, device=h.device)
        mine = _f(h[begin:end])
        before = torch.cat((first[None], mine[:-1]), dim=0)
        for i in range(mu.shape[0]):
            out[begin:end, i * width:(i + 1) * width] = (mine + (before - mine) * _f(mu[i])).to(out.dtype)
        if slot >= 0:
            state[slot, offset:offset + width] = mine[-1].float()


def channel_decay(pre, bias, kind, out, tau=1.0):
    z = _f(pre) if bias is None else _f(pre) + _f(bias)
    w = torch.exp(-torch.exp(z)) if kind == "double_exp" else torch.exp(torch.nn.functional.logsigmoid(z) / tau)
    out.copy_(w.float())


def outer_state_scan_rows(q, k, v, decay, cu_q, slots, state, s_offset, n_heads, dim, vdim, q_scale, y, bonus=None, decay_from=None):
    size = n_heads * dim * vdim
    if decay_from is not None:
        made = torch.empty_like(decay)
        channel_decay(decay, decay_from[1], decay_from[0], made, tau=decay_from[2])
        decay = made
    for s in range(cu_q.numel() - 1):
        slot = int(slots[s])
        S = torch.zeros(n_heads, dim, vdim, dtype=torch.float64, device=q.device)
        if slot >= 0:
            S = _f(state[slot, s_offset:s_offset + size]).view(n_heads, dim, vdim).clone()
        for t in range(int(cu_q[s]), int(cu_q[s + 1])):
            qt, kt, vt = (_f(q[t]) * q_scale).view(n_heads, dim), _f(k[t]).view(n_heads, dim), _f(v[t]).view(n_heads, vdim)
            kv = kt[:, :, None] * vt[:, None, :]
            if bonus is not None:
                y[t] = torch.einsum("hdv,hd->hv", S + _f(bonus).view(n_heads, dim)[:, :, None] * kv, qt).reshape(-1).float()
            S = _f(decay[t]).view(n_heads, dim)[:, :, None] * S + kv
            if bonus is None:
                y[t] = torch.einsum("hdv,hd->hv", S, qt).reshape(-1).float()
        if slot >= 0:
            state[slot, s_offset:s_offset + size] = S.reshape(-1).float()


def softcap_(x, cap):
    x.copy_((cap * torch.tanh(_f(x) / cap)).to(x.dtype))


def stabilized_gates(pre, bias, cap, cu_q, slots, state, m_offset, n_heads, decay, take, floor):
    z = _f(pre) + _f(bias)
    a = cap * torch.tanh(z[:, :n_heads] / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh(z[:, n_heads:] / cap))
    for s in range(cu_q.numel() - 1):
        slot = int(slots[s])
        m = _f(state[slot, m_offset:m_offset + n_heads]) if slot >= 0 else torch.zeros(n_heads, dtype=torch.float64, device=pre.device)
        for t in range(int(cu_q[s]), int(cu_q[s + 1])):
            m_new = torch.maximum(f[t] + m, a[t])
            decay[t] = torch.exp(f[t] + m - m_new).float()
            take[t] = torch.exp(a[t] - m_new).float()
            floor[t] = torch.exp(-m_new).float()
            m = m_new
        if slot >= 0:
            state[slot, m_offset:m_offset + n_heads] = m.float()


def decay_gates(dt_pre, dt_bias, rate_log, decay, take):
    dt = torch.nn.functional.softplus(_f(dt_pre) + _f(dt_bias))
    decay.copy_(torch.exp(-torch.exp(_f(rate_log)) * dt).float())
    take.copy_(dt.float())


def outer_state_scan(q, k, v, decay, take, cu_q, slots, state, s_offset, n_offset, n_heads, n_groups, dim, vdim, q_scale, y, nq):
    per = n_heads // n_groups
    for s in range(cu_q.numel() - 1):
        slot = int(slots[s])
        S = torch.zeros(n_heads, dim, vdim, dtype=torch.float64, device=q.device)
        nv = torch.zeros(n_heads, dim, dtype=torch.float64, device=q.device)
        if slot >= 0:
            S = _f(state[slot, s_offset:s_offset + n_heads * dim * vdim]).view(n_heads, dim, vdim).clone()
            if nq is not None:
                nv = _f(state[slot, n_offset:n_offset + n_heads * dim]).view(n_heads, dim).clone()
        for t in range(int(cu_q[s]), int(cu_q[s + 1])):
            qt = (_f(q[t]) * q_scale).view(n_groups, dim).repeat_interleave(per, dim=0)
            kt = _f(k[t]).view(n_groups, dim).repeat_interleave(per, dim=0)
            vt = _f(v[t]).view(n_heads, vdim)
            d, g = _f(decay[t])[:, None], _f(take[t])[:, None]
            S = d[:, :, None] * S + g[:, :, None] * kt[:, :, None] * vt[:, None, :]
            y[t] = torch.einsum("hdv,hd->hv", S, qt).reshape(-1).float()
            if nq is not None:
                nv = d * nv + g * kt
                nq[t] = (nv * qt).sum(-1).float()
        if slot >= 0:
            state[slot, s_offset:s_offset + n_heads * dim * vdim] = S.reshape(-1).float()
            if nq is not None:
                state[slot, n_offset:n_offset + n_heads * dim] = nv.reshape(-1).float()


def gated_group_norm(y, gate, weight, eps, out, n_parts, n_heads, gate_kind, gate_first, nq=None, floor=None, floor_add=0.0,
                     skip=None, skip_x=None):
    n, c = y.shape
    z = _f(y).view(n, n_heads, c // n_heads)
    if nq is not None:
        z = z / (torch.maximum(_f(nq).abs(), _f(floor)) + floor_add)[:, :, None]
    if skip is not None:
        z = z + _f(skip)[None, :, None] * _f(skip_x).view(n, n_heads, -1)
    z = z.reshape(n, c)
    g = _f(gate)
    g = torch.sigmoid(g) if gate_kind == "sigmoid" else g * torch.sigmoid(g)
    if gate_first:
        z = z * g
    z = z.view(n, n_parts, c // n_parts)
    z = (z / torch.sqrt(z.square().mean(-1, keepdim=True) + eps)).reshape(n, c) * _f(weight)
    if not gate_first:
        z = z * g
    out.copy_(z.to(out.dtype))


def causal_conv_silu(x, weight, bias, cu_q, tok_seq, slots, state, offset, out, activation="silu", single=False):
    n, c = x.shape
    taps = weight.shape[1]
    for s in range(cu_q.numel() - 1):
        b, e = int(cu_q[s]), int(cu_q[s + 1])
        slot = int(slots[s])
        before = torch.zeros(taps - 1, c, dtype=torch.float64, device=x.device)
        if slot >= 0:
            before = _f(state[slot, offset:offset + (taps - 1) * c]).view(taps - 1, c)
        padded = torch.cat((before, _f(x[b:e])))
        z = sum(padded[j:j + e - b] * _f(weight)[:, j] for j in range(taps))
        if bias is not None:
            z = z + _f(bias)
        out[b:e] = (z * torch.sigmoid(z) if activation == "silu" else z).to(out.dtype)
        if slot >= 0 and taps > 1:
            state[slot, offset:offset + (taps - 1) * c] = padded[padded.shape[0] - (taps - 1):].reshape(-1).float()


def causal_conv(x, weight, bias, cu_q, tok_seq, slots, state, offset, out, single=False):
    causal_conv_silu(x, weight, bias, cu_q, tok_seq, slots, state, offset, out, activation="none")


def add_dyt_norm(hidden, a, b, weight, bias, alpha, out):
    if a is not None or b is not None:
        hidden += ((0 if a is None else _f(a)) + (0 if b is None else _f(b))).to(hidden.dtype)
    out.copy_((torch.tanh(alpha * _f(hidden)) * _f(weight) + _f(bias)).to(out.dtype))


def add_dyt_norm_shift(hidden, a, b, weight, bias, alpha, out, taps, slots, state, shifted):
    add_dyt_norm(hidden, a, b, weight, bias, alpha, out)
    rows = out.shape[0]
    every = torch.arange(rows + 1, dtype=torch.int32, device=out.device)
    causal_conv(out, taps, None, every, every[:-1], slots, state, 0, shifted, single=True)


def gated_rows(x, weight, out, clamp=None):
    return False     # the product and the gate as two steps


def residual_add_pair(hidden, a, b):
    if a is not None or b is not None:
        hidden += ((0 if a is None else _f(a)) + (0 if b is None else _f(b))).to(hidden.dtype)


def stream_pair(hidden, a, b, other, out):
    x = _f(hidden) + (0 if a is None else _f(a)) + (0 if b is None else _f(b))
    out.copy_(torch.cat((x, _f(other)), dim=-1).to(out.dtype))


def head_gate(x, gate, n_heads):
    rows = x.shape[0]
    x.copy_((_f(x).view(rows, n_heads, -1) * torch.sigmoid(_f(gate))[:, :, None]).view(rows, -1).to(x.dtype))


def pool_cache_write(cu_q, tok_pos, slots, site, blocks, pool, max_q_len, err):
    for s in range(slots.numel()):
        slot, b, e = int(slots[s]), int(cu_q[s]), int(cu_q[s + 1])
        if slot < 0 or e <= b:
            continue
        start = int(tok_pos[b])
        for block in range(start // pool, (start + e - b) // pool):
            k, v = gather_kv(site, slot, block * pool, block * pool + pool)      # [kvh, pool, d]
            page = int(blocks.table[slot, block // PAGE])
            assert page >= 0, "reference: write to a page of block rows that is not held"
            blocks.storage[page, 0, :, block % PAGE, :] = k.mean(1).to(blocks.storage.dtype)
            blocks.storage[page, 1, :, block % PAGE, :] = v.mean(1).to(blocks.storage.dtype)


ALL = dict(rows_prepare=rows_prepare, bias_glu=bias_glu, add_rms_norm_scaled=add_rms_norm_scaled, residual_add_scaled=residual_add_scaled, rms_norm_cols=rms_norm_cols,
           mix_rows=mix_rows, shift_mix=shift_mix, channel_decay=channel_decay, outer_state_scan_rows=outer_state_scan_rows,
           gated_rows=gated_rows, causal_conv=causal_conv, add_dyt_norm=add_dyt_norm, add_dyt_norm_shift=add_dyt_norm_shift, residual_add_pair=residual_add_pair, stream_pair=stream_pair,
           head_gate=head_gate, pool_cache_write=pool_cache_write, bias_act=bias_act, softcap_=softcap_, stabilized_gates=stabilized_gates, decay_gates=decay_gates,
           outer_state_scan=outer_state_scan, gated_group_norm=gated_group_norm, causal_conv_silu=causal_conv_silu,
           expert_gate_takes=expert_gate_takes, linear_rows=linear_rows, moe_tile_rows=moe_tile_rows, scaled_swiglu=scaled_swiglu, embed_positions=embed_positions, sandwich_norm=sandwich_norm, clamped_glu=clamped_glu, latent_norm_cache=latent_norm_cache,
           head_linear=head_linear, moe_plan=moe_plan, moe_gather=moe_gather, moe_combine=moe_combine, expert_linear=expert_linear,
           embed_gather=embed_gather, gather_rows=gather_rows, gather_rows_norm=gather_rows_norm, add_rms_norm=add_rms_norm, gemm_f32=gemm_f32,
           linear=linear, rope_cache_write=rope_cache_write, attention_generic=attention_generic, swiglu=swiglu,
           sample=sample)
