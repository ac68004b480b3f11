"""Plain PyTorch statements of the engine's kernels, one function per kernel,
with the signatures of ``einf_b200.ops``.

Two uses.  The ``-m gpu`` tests run each kernel alone against its function here.
And :func:`emulate_kernels` swaps them in for the kernels, which lets the
engine's host logic (batch packing, cache, replay, scheduler and executor) be
tested on a machine without a GPU; the product itself has no such path.

Arithmetic is 32-bit (or 64-bit with ``HIGH_PRECISION``); results are rounded
once into the output's dtype, as the kernels do.
"""
from __future__ import annotations

import contextlib

import torch

_MASK64 = (1 << 64) - 1


def embed(tokens, table, residual, status, positions=None, position_table=None, scale=1.0):
    residual.copy_(table[tokens.long()].float() * scale)
    if position_table is not None:
        residual.add_(position_table[positions.long()].float())


def add_rmsnorm(x, residual, weight, eps, out, rows=None, status=None):
    total = residual.float()
    if x is not None:
        xf = x.float()
        if xf.dim() == 3:
            xf = xf.sum(0)
        total = total + xf
    source = total if rows is None else total[rows.long()]
    variance = source.pow(2).mean(-1, keepdim=True)
    out.copy_((weight * (source * torch.rsqrt(variance + eps))).to(out.dtype))
    if rows is None and x is not None:
        residual.copy_(total)


def rope_kv_write(qkv, bias, positions, inv_freq, slots, q_out, k_cache, v_cache,
                  num_heads, num_kv_heads, head_size, status):
    values = qkv.float()
    if values.dim() == 3:
        values = values.sum(0)
    tokens = values.shape[0]
    if bias is not None:
        values = values + bias
    q, k, v = values.split([num_heads * head_size, num_kv_heads * head_size, num_kv_heads * head_size], dim=-1)
    q = q.reshape(tokens, num_heads, head_size)
    k = k.reshape(tokens, num_kv_heads, head_size)
    v = v.reshape(tokens, num_kv_heads, head_size)
    half = inv_freq.shape[0]
    if half:
        angles = positions.float()[:, None] * inv_freq[None, :]
        cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]

        def rotate(x):
            a, b, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)

        q, k = rotate(q), rotate(k)
    q_out.copy_(q.reshape(q_out.shape).to(q_out.dtype))
    if slots is not None:
        page_size = k_cache.shape[2]
        keep = slots >= 0
        page = (slots[keep] // page_size).long()
        offset = (slots[keep] % page_size).long()
        k_cache[page, :, offset, :] = k[keep].to(k_cache.dtype)
        v_cache[page, :, offset, :] = v[keep].to(v_cache.dtype)


def silu_mul(gate_up, out):
    inter = out.shape[-1]
    gate_up = gate_up.float()
    if gate_up.dim() == 3:
        gate_up = gate_up.sum(0)
    g, u = gate_up[:, :inter], gate_up[:, inter:]
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))


def linear(x, weight, bias, out):
    result = x.float() @ weight.float().T
    if bias is not None:
        result = result + bias
    out.copy_(result.to(out.dtype))


def gemm_simt(x, weight, bias, out):
    linear(x, weight, bias, out)


def project(x, weight, status, out_dtype=None, allow_partial=True):
    out = torch.empty((x.shape[0], weight.shape[0]), dtype=out_dtype or x.dtype, device=x.device)
    linear(x, weight, None, out)
    return out


def paged_attention_generic(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window, status,
                            chunk=None, softcap=None, keep_first=0, values_in_keys=None, sink=None):
    tokens, num_heads, head_size = q.shape
    _, num_kv_heads, page_size, _ = k_cache.shape
    groups = num_heads // num_kv_heads
    for t in range(tokens):
        r = int(seq_of_token[t])
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        if chunk:
            lo = max(lo, pos // chunk * chunk)
        keys = torch.arange(lo, pos + 1, device=q.device)
        if window and keep_first:
            keys = torch.cat([torch.arange(0, min(keep_first, lo), device=q.device), keys])
        pages = block_table[r, (keys // page_size).long()].long()
        offsets = (keys % page_size).long()
        k = k_cache[pages, :, offsets, :].float()      # [n, kv_heads, D]
        v = k[..., :values_in_keys] if values_in_keys else v_cache[pages, :, offsets, :].float()
        k = k.repeat_interleave(groups, dim=1)
        v = v.repeat_interleave(groups, dim=1)
        scores = torch.einsum("hd,nhd->hn", q[t].float(), k) * scale
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        if sink is not None:        # one more column in the denominator, with no value
            scores = torch.cat([scores, sink.float()[:, None]], dim=1)
        probabilities = torch.softmax(scores, dim=-1)[:, :keys.shape[0]]
        out[t] = torch.einsum("hn,nhd->hd", probabilities, v).to(out.dtype)


def latent_decode_attention(q, cache, block_table, seq_of_token, positions, out, scale, splits, status):
    paged_attention_generic(q, cache, None, block_table, seq_of_token, positions, out, scale, None, status,
                            values_in_keys=out.shape[2])


def latent_decode_splits(num_tokens, num_heads, max_context):
    return 1


def _summed(x):
    x = x.float()
    return x.sum(0) if x.dim() == 3 else x


def activation(x, out, kind):
    z = _summed(x)
    if kind == "relu2":
        y = torch.clamp(z, min=0) ** 2
    elif kind == "gelu_tanh":
        y = 0.5 * z * (1 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
    elif kind == "silu":
        y = z / (1 + torch.exp(-z))
    elif kind == "relu":
        y = torch.clamp(z, min=0)
    else:
        raise ValueError(kind)
    out.copy_(y.to(out.dtype))


def _rotate(x, positions, inv_freq, interleaved):
    """x [T, heads, D]: rotate the first 2n dims, pair i = (i, i + n) or (2i, 2i + 1)."""
    n = inv_freq.shape[0]
    if not n:
        return x
    angles = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    index = torch.arange(n, device=x.device)
    first, second = (2 * index, 2 * index + 1) if interleaved else (index, index + n)
    u, v = x[..., first], x[..., second]
    out = x.clone()
    out[..., first] = u * cos - v * sin
    out[..., second] = v * cos + u * sin
    return out


def qkv_norm_store(qkv, bias, slots, q_out, k_cache, v_cache, num_heads, num_kv_heads, key_size, value_size,
                   unit_eps, status, positions=None, inv_freq=None, interleaved=False, value_mix=None,
                   shared_values=None, mix=None, q_norm_weight=None, k_norm_weight=None, norm_rows=False,
                   values_from_keys=False):
    values = _summed(qkv)
    tokens = values.shape[0]
    if bias is not None:
        values = values + bias
    if values_from_keys:
        q, k = values.split([num_heads * key_size, num_kv_heads * key_size], dim=-1)
        v = k
    else:
        q, k, v = values.split([num_heads * key_size, num_kv_heads * key_size, num_kv_heads * value_size], dim=-1)
    v = v.reshape(tokens, num_kv_heads, value_size)
    if unit_eps is not None and norm_rows:          # one root mean square for all heads of a row
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + unit_eps)
        if num_kv_heads:
            k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + unit_eps)
        if q_norm_weight is not None:
            q = q * q_norm_weight
        if k_norm_weight is not None and num_kv_heads:
            k = k * k_norm_weight
    q = q.reshape(tokens, num_heads, key_size)
    k = k.reshape(tokens, num_kv_heads, key_size)
    if unit_eps is not None and not norm_rows:
        q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + unit_eps)
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + unit_eps)
        if q_norm_weight is not None:
            q = q * q_norm_weight
        if k_norm_weight is not None:
            k = k * k_norm_weight
    if inv_freq is not None and inv_freq.shape[0]:
        q = _rotate(q, positions, inv_freq, interleaved)
        k = _rotate(k, positions, inv_freq, interleaved)
    if value_mix == "source":
        shared_values.copy_(v.reshape(shared_values.shape))
    elif value_mix == "blend":
        m = mix.float().reshape(())
        v = (1 - m) * v + m * shared_values.reshape(v.shape)
    q_out.copy_(q.reshape(q_out.shape).to(q_out.dtype))
    if slots is not None and num_kv_heads:
        page_size = k_cache.shape[2]
        keep = slots >= 0
        page = (slots[keep] // page_size).long()
        offset = (slots[keep] % page_size).long()
        k_cache[page, :, offset, :] = k[keep].to(k_cache.dtype)
        v_cache[page, :, offset, :] = v[keep].to(v_cache.dtype)


def latent_down_store(down, q_rank, kv_rank, rot_dim, q_norm_weight, kv_norm_weight, eps, positions, inv_freq,
                      interleaved, slots, q_latent_out, cache, status):
    values = _summed(down)
    q_latent, latent, part = values.split([q_rank, kv_rank, rot_dim], dim=-1)
    if q_rank:
        q_latent = q_latent * torch.rsqrt(q_latent.pow(2).mean(-1, keepdim=True) + eps) * q_norm_weight
        q_latent_out.copy_(q_latent.to(q_latent_out.dtype))
    latent = latent * torch.rsqrt(latent.pow(2).mean(-1, keepdim=True) + eps) * kv_norm_weight
    part = _rotate(part[:, None, :], positions, inv_freq, interleaved)[:, 0]
    if slots is not None:
        page_size = cache.shape[2]
        keep = slots >= 0
        page = (slots[keep] // page_size).long()
        offset = (slots[keep] % page_size).long()
        cache[page, 0, offset, :] = torch.cat([latent, part], dim=-1)[keep].to(cache.dtype)


def latent_q_store(q, positions, inv_freq, interleaved, q_plain, q_full):
    tokens, heads, dim = q_plain.shape
    rot_dim = 2 * inv_freq.shape[0]
    values = _summed(q).reshape(tokens, heads, dim + rot_dim)
    q_plain.copy_(values[..., :dim].to(q_plain.dtype))
    q_full[..., q_full.shape[2] - rot_dim:] = _rotate(values[..., dim:], positions, inv_freq, interleaved).to(q_full.dtype)


def per_head_project(x, weight, out):
    out.copy_(torch.einsum("thi,hoi->tho", x.float(), weight.float()).to(out.dtype))


def router_topk(logits, top_k, score, renormalise, expert_ids, weights, num_experts=None, correction=None,
                groups=None):
    z = _summed(logits)
    if num_experts is not None:
        z = z[:, :num_experts]
    scores = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, dim=-1)
    # without a correction the choice goes by the logits themselves (the scores are monotone in them)
    choice = z if correction is None else scores + correction
    if groups is not None:
        count, keep = groups
        tokens, experts = choice.shape
        best = choice.reshape(tokens, count, experts // count).max(dim=-1).values
        kept = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
        allowed = torch.zeros(tokens, count, dtype=torch.bool, device=z.device)
        allowed.scatter_(1, kept, True)
        allowed = allowed.repeat_interleave(experts // count, dim=1)
        choice = torch.where(allowed, choice, torch.full_like(choice, -torch.inf))
    order = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top_k]
    chosen = torch.gather(scores, 1, order)
    if renormalise:
        chosen = chosen / chosen.sum(-1, keepdim=True)
    expert_ids.copy_(order.to(expert_ids.dtype))
    weights.copy_(chosen)


def moe_dispatch(x, expert_ids, weights, num_experts, scale_rows, work, place, sorted_x):
    tokens, top_k = expert_ids.shape
    flat = expert_ids.reshape(-1).long()
    order = torch.sort(flat, stable=True).indices          # sorted row -> pair; ids beyond the experts come last
    counts = torch.bincount(flat, minlength=num_experts)[:num_experts]
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32, device=x.device)
    offsets[1:] = counts.cumsum(0).to(torch.int32)
    work[2 * num_experts:] = offsets
    rows = torch.empty_like(flat)
    rows[order] = torch.arange(flat.shape[0], device=x.device)
    place.copy_(rows.reshape(tokens, top_k).to(place.dtype))
    source = x.float()[(order // top_k)]
    if scale_rows:
        source = source * weights.reshape(-1)[order][:, None]
    sorted_x.copy_(source.to(sorted_x.dtype))
    return work[2 * num_experts:]


def moe_gemm(x, weight, offsets, out, status=None):
    if out.dim() == 3:          # partial sums: everything in the first, zeros in the others
        out.zero_()
        out = out[0]
    for e in range(weight.shape[0]):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi > lo:
            out[lo:hi] = (x[lo:hi].float() @ weight[e].float().T).to(out.dtype)


def moe_gemm_on_tensor_cores(x, weight):
    return False


def moe_gemm_splits(rows, experts, n, k):
    return 1


def moe_combine(y, expert_ids, place, weights, scale_outputs, addend, out, num_experts, identity_input=None,
                num_identity=0, addend_gate=None):
    total = torch.zeros_like(out) if addend is None else _summed(addend).clone()
    if addend_gate is not None:
        gate, column = addend_gate
        total = total * torch.sigmoid(_summed(gate)[:, column])[:, None]
    y = _summed(y)
    for j in range(expert_ids.shape[1]):
        e = expert_ids[:, j]
        term = y[place[:, j].long()]
        term = weights[:, j, None] * term if scale_outputs else term
        term = torch.where((e < num_experts)[:, None], term, torch.zeros_like(term))
        if num_identity:
            through = (e >= num_experts) & (e < num_experts + num_identity)
            term = term + torch.where(through[:, None], weights[:, j, None] * identity_input.float(), torch.zeros_like(term))
        total = total + term
    out.copy_(total)


def softcap(values, cap, scale=1.0):
    values.copy_(cap * torch.tanh(values * scale / cap) if cap else values * scale)


def conv_silu(x, weight, bias, conv_state, seq_of_token, q_start, state_slots, out, dt_raw=None, dt_bias=None,
              a_log=None, dt_out=None, decay_out=None, activation=True, input_bias=None):
    taps = weight.shape[1]
    xf = x.float()
    if input_bias is not None:
        xf = xf + input_bias
    for r in range(state_slots.shape[0]):
        first, last = int(q_start[r]), int(q_start[r + 1])
        slot = int(state_slots[r])
        if last <= first:
            continue
        history = conv_state[slot].clone() if slot >= 0 else torch.zeros(taps - 1, x.shape[1], device=x.device)
        line = torch.cat([history, xf[first:last]], dim=0)            # [taps - 1 + n, channels]
        for i in range(last - first):
            acc = (line[i:i + taps].T * weight).sum(dim=1)
            if bias is not None:
                acc = acc + bias
            out[first + i] = ((acc / (1 + torch.exp(-acc))) if activation else acc).to(out.dtype)
        if slot >= 0 and taps > 1:
            conv_state[slot] = line[-(taps - 1):]
    if dt_raw is not None:
        dt = torch.nn.functional.softplus(dt_raw.float() + dt_bias)
        dt_out.copy_(dt)
        decay_out.copy_(torch.exp(-torch.exp(a_log) * dt))


def linear_recurrence(q, k, v, state, q_start, state_slots, y, heads, groups, dim, vdim, head_decay=None,
                      token_decay=None, token_scale=None, skip=None, silu_inputs=False, max_q_len=None, rows=0,
                      segment_len=None, columns=0):
    def act(t):
        t = t.float()
        return t / (1 + torch.exp(-t)) if silu_inputs else t

    tokens = v.shape[0]
    if y.dim() == 3:            # parts of several CTAs: everything in the first, zeros in the others
        y.zero_()
        y = y[0]
    qf, kf = act(q).reshape(tokens, groups, dim), act(k).reshape(tokens, groups, dim)
    vf = act(v).reshape(tokens, heads, vdim)
    per_group = heads // groups
    for r in range(state_slots.shape[0]):
        first, last = int(q_start[r]), int(q_start[r + 1])
        slot = int(state_slots[r])
        for h in range(heads):
            S = state[slot, h].clone() if slot >= 0 else torch.zeros(dim, vdim, device=v.device)
            g = h // per_group
            for t in range(first, last):
                a = head_decay[h] if head_decay is not None else token_decay[t, h]
                s = token_scale[t, h] if token_scale is not None else 1.0
                S = a * S + torch.outer(kf[t, g], s * vf[t, h])
                row = S.T @ qf[t, g]
                if skip is not None:
                    row = row + skip[h] * vf[t, h]
                y[t, h * vdim:(h + 1) * vdim] = row
            if slot >= 0 and last > first:
                state[slot, h] = S


def gated_norm(y, gate, weight, out, parts, eps, gate_first, gate_kind):
    g = gate.float()
    g = g / (1 + torch.exp(-g)) if gate_kind == "silu" else torch.sigmoid(g)
    u = y * g if gate_first else y
    tokens, width = y.shape
    cut = u.reshape(tokens, parts, width // parts)
    cut = cut * torch.rsqrt(cut.pow(2).mean(-1, keepdim=True) + eps)
    result = cut.reshape(tokens, width) * weight
    if not gate_first:
        result = result * g
    out.copy_(result.to(out.dtype))


def memory_value_columns(vdim):
    return (vdim + 1 + 3) // 4 * 4


def recurrence_step_splits(num_requests, heads, dim, vdim, state):
    return 1


def memory_gates(gates, bias, cap, v, top_state, q_start, state_slots, decay, scale, floor, v_wide, heads, vdim,
                 max_q_len=None):
    z = _summed(gates) + bias
    tokens = z.shape[0]
    log_in = cap * torch.tanh(z[:, :heads] / cap)
    log_keep = torch.nn.functional.logsigmoid(cap * torch.tanh(z[:, heads:] / cap))
    for r in range(state_slots.shape[0]):
        first, last = int(q_start[r]), int(q_start[r + 1])
        slot = int(state_slots[r])
        top = top_state[slot].clone() if slot >= 0 else torch.zeros(heads, device=z.device)
        for t in range(first, last):
            new_top = torch.maximum(log_keep[t] + top, log_in[t])
            decay[t] = torch.exp(log_keep[t] + top - new_top)
            scale[t] = torch.exp(log_in[t] - new_top)
            floor[t] = torch.exp(-new_top)
            top = new_top
        if slot >= 0 and last > first:
            top_state[slot] = top
    columns = v_wide.shape[1] // heads
    wide = torch.zeros(tokens, heads, columns, dtype=torch.float32, device=v.device)
    wide[:, :, :vdim] = v.float().reshape(tokens, heads, vdim)
    wide[:, :, vdim] = 1.0
    v_wide.copy_(wide.reshape(tokens, heads * columns).to(v_wide.dtype))


def memory_output(y, floor, gate, weight, out, heads, vdim, query_scale, eps, denominator_eps):
    y = _summed(y)
    tokens = y.shape[0]
    wide = y.reshape(tokens, heads, -1)
    below = torch.maximum((query_scale * wide[:, :, vdim]).abs(), floor) + denominator_eps
    o = query_scale * wide[:, :, :vdim] / below[:, :, None]
    o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)
    out.copy_((o.reshape(tokens, heads * vdim) * weight * torch.sigmoid(gate.float())).to(out.dtype))


def norm_join(terms, weights, eps, out, scale=1.0):
    total = torch.zeros_like(out)
    for term, weight in zip(terms, weights):
        t = _summed(term)
        total = total + weight * (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps))
    out.copy_(scale * total)


def _gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))


def act_mul(gate_up, out, kind):
    g = _summed(gate_up)
    inter = out.shape[1]
    gate, up = g[:, :inter], g[:, inter:]
    act = {"silu": lambda z: z / (1 + torch.exp(-z)), "gelu_tanh": _gelu_tanh}[kind]
    out.copy_((act(gate) * up).to(out.dtype))


def _add_pending(residual, pending, scale):
    terms = [t for t in (pending or []) if t is not None]
    if terms:
        total = _summed(terms[0])
        for t in terms[1:]:
            total = total + _summed(t)
        residual.add_(scale * total)


def norm_conv(pending, pending_scale, residual, norm_weight, eps, conv_weight, conv_state, seq_of_token, q_start,
              state_slots, out, single_tokens=False):
    _add_pending(residual, pending, pending_scale)
    h = residual * torch.rsqrt(residual.pow(2).mean(-1, keepdim=True) + eps) * norm_weight
    if conv_weight is None:
        out.copy_(h.to(out.dtype))
        return
    taps = conv_weight.shape[1]
    for r in range(state_slots.shape[0]):
        first, last = int(q_start[r]), int(q_start[r + 1])
        slot = int(state_slots[r])
        if last <= first:
            continue
        history = conv_state[slot].clone() if (slot >= 0 and taps > 1) else torch.zeros(taps - 1, h.shape[1])
        line = torch.cat([history, h[first:last]], dim=0)
        for i in range(last - first):
            out[first + i] = (h[first + i] + (line[i:i + taps].T * conv_weight).sum(dim=1)).to(out.dtype)
        if slot >= 0 and taps > 1:
            conv_state[slot] = line[-(taps - 1):]


def stream_tail(residual, pending, pending_scale, token_ids, side, depth):
    _add_pending(residual, pending, pending_scale)
    if side is not None:
        table, gate, proj_t, norm, eps = side
        g = _gelu_tanh(residual @ gate.float().T) * table[token_ids.long()].float()
        y = g @ proj_t.float()
        residual.add_(pending_scale * y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * norm)
    if depth is not None:
        history, index, weight = depth
        history[index + 1] = residual
        residual.copy_((weight[:, None, None] * history[:index + 2]).sum(0))


def paged_attention_mixed(q, k_cache, v_cache, block_table, seq_of_token, positions, out, scale, window, slopes, talk,
                          sink, out_scale, status, q_tiles=None, single_tokens=None, num_singles=0, max_context=0):
    tokens, num_heads, _ = q.shape
    _, num_kv_heads, page_size, _ = k_cache.shape
    groups = num_heads // num_kv_heads
    for t in range(tokens):
        r = int(seq_of_token[t])
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        keys = torch.arange(lo, pos + 1)
        pages = block_table[r, (keys // page_size).long()].long()
        offsets = (keys % page_size).long()
        k = k_cache[pages, :, offsets, :].float().repeat_interleave(groups, dim=1)
        v = v_cache[pages, :, offsets, :].float().repeat_interleave(groups, dim=1)
        scores = torch.einsum("hd,nhd->hn", q[t].float(), k) * scale
        if slopes is not None:
            scores = scores - slopes[:, None] * (pos - keys).float()[None, :]
        if talk is not None:
            scores = talk @ scores
        if sink is not None:
            scores = torch.cat([scores, sink[:, None]], dim=1)
        probabilities = torch.softmax(scores, dim=-1)[:, :keys.shape[0]]
        out[t] = (out_scale * torch.einsum("hn,nhd->hd", probabilities, v)).to(out.dtype)


def gated_scan(gates, gate_bias, u, y_raw, y_bias, rate, state, q_start, state_slots, out, out_scale, max_q_len=None):
    tokens, blocks, twice = gates.shape
    part = twice // 2
    raw = gates + gate_bias.view(1, blocks, twice)
    r = torch.sigmoid(raw[:, :, :part]).reshape(tokens, -1)
    i = torch.sigmoid(raw[:, :, part:]).reshape(tokens, -1)
    a = torch.exp(rate * r)
    b = torch.sqrt(1.0 - a * a) * i * u.float()
    y = _gelu_tanh(y_raw.float() + y_bias)
    for request in range(state_slots.shape[0]):
        first, last = int(q_start[request]), int(q_start[request + 1])
        slot = int(state_slots[request])
        s = state[slot].clone() if slot >= 0 else torch.zeros(u.shape[1])
        for t in range(first, last):
            s = a[t] * s + b[t]
            out[t] = (out_scale * s * y[t]).to(out.dtype)
        if slot >= 0 and last > first:
            state[slot] = s


def argmax(logits, tokens):
    tokens[: logits.shape[0]] = torch.argmax(logits, dim=-1).to(torch.int32)


def keyed_uniform(seed, index):
    def mix(z):
        z = (z + 0x9E3779B97F4A7C15) & _MASK64
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        return z ^ (z >> 31)

    z = mix(int(seed) & _MASK64)
    z = mix(z ^ (int(index) & _MASK64))
    return (z >> 40) / float(1 << 24)


def kept_weights(row, temperature, top_k, top_p, min_p):
    """Unnormalised probabilities of the tokens a row may draw (0 for dropped ones).  Tokens with
    equal scaled logits stay or go together: top-k keeps every token that ties the k-th, top-p
    keeps a token iff the mass of the strictly more probable ones has not passed top_p of the
    mass.  (The reference sorts, so among equal logits it keeps whichever the sort puts first.)"""
    scaled = row.float() / temperature
    weights = torch.exp(scaled - scaled.max())
    keep = torch.ones_like(weights, dtype=torch.bool)
    if top_k and top_k < row.numel():
        kth = torch.topk(scaled, top_k).values[-1]
        keep &= scaled >= kth
    if top_p < 1.0:
        masked = torch.where(keep, weights, torch.zeros_like(weights)).double()
        values, which = torch.unique(scaled, return_inverse=True)               # ascending
        mass_of_value = torch.zeros(values.numel(), dtype=torch.float64).index_add_(0, which, masked)
        above = mass_of_value.flip(0).cumsum(0).flip(0) - mass_of_value         # mass of the strictly larger values
        keep &= (above <= top_p * masked.sum())[which]
    if min_p > 0.0:
        keep &= weights >= min_p
    return torch.where(keep, weights, torch.zeros_like(weights))


def sample(logits, tokens, temperature, top_k, top_p, min_p, seed, sample_index):
    for r in range(logits.shape[0]):
        t = float(temperature[r])
        if t <= 0:
            tokens[r] = int(torch.argmax(logits[r]))
            continue
        weights = kept_weights(logits[r], t, int(top_k[r]), float(top_p[r]), float(min_p[r])).double()
        cumulative = weights.cumsum(0)
        target = keyed_uniform(int(seed[r]), int(sample_index[r])) * float(cumulative[-1])
        index = int(torch.searchsorted(cumulative, torch.tensor(target, dtype=torch.float64), right=True))
        tokens[r] = min(index, logits.shape[1] - 1)


def advance_decode(token_ids, positions, context_lens, sampled, slots, block_tables, page_size):
    n = sampled.shape[0]
    token_ids[:n] = sampled
    positions[:n] += 1
    context_lens[:n] += 1
    for slot, table in zip(slots, block_tables):
        for i in range(n):
            if int(slot[i]) < 0:
                continue
            position = int(positions[i])
            slot[i] = int(table[i, position // page_size]) * page_size + position % page_size


def zero_fresh_state(state, state_slots, q_start, positions):
    for request in range(state_slots.shape[0]):
        slot = int(state_slots[request])
        if 0 <= slot < state.shape[0] and int(positions[int(q_start[request])]) == 0:
            state[slot] = 0


def has_fast_attention(dtype, head_size):
    return False          # the plain statement of attention serves every dtype here


def report(tokens, count, status, host):
    host[:count] = tokens[:count]
    host[count] = status[0]


def ensure_built(names):
    return None


def recurrence_plan(num_requests, max_q_len, heads, dim, vdim, sms=None):
    return 1, max(1, max_q_len or 1)


_NAMES = (
    "embed", "add_rmsnorm", "rope_kv_write", "silu_mul", "linear", "gemm_simt", "project",
    "paged_attention_generic", "argmax", "sample", "ensure_built", "advance_decode", "report",
    "zero_fresh_state", "has_fast_attention", "activation", "qkv_norm_store", "conv_silu", "linear_recurrence",
    "gated_norm", "recurrence_plan", "latent_down_store", "latent_q_store", "per_head_project", "router_topk",
    "moe_dispatch", "moe_gemm", "moe_combine", "softcap", "latent_decode_attention", "latent_decode_splits", "moe_gemm_on_tensor_cores", "moe_gemm_splits",
    "act_mul", "norm_conv", "stream_tail", "paged_attention_mixed", "gated_scan", "memory_gates", "memory_output",
    "norm_join", "memory_value_columns", "recurrence_step_splits",
)


@contextlib.contextmanager
def emulate_kernels():
    """Within the block, ``einf_b200.ops`` computes with the functions above and a
    ``ModelRunner`` accepts the CPU device."""
    from einf_b200 import ops
    from einf_b200.engine.runner import ModelRunner

    saved_ops = {name: getattr(ops, name) for name in _NAMES}
    saved = tuple(ModelRunner.__dict__[n] for n in ("_check_device", "_guard", "synchronize", "_graphable"))
    for name in _NAMES:
        setattr(ops, name, globals()[name])
    ModelRunner._check_device = staticmethod(lambda device: None)
    ModelRunner._guard = lambda self: contextlib.nullcontext()
    ModelRunner.synchronize = lambda self: None
    ModelRunner._graphable = staticmethod(lambda requests: False)   # no CUDA graphs without CUDA
    try:
        yield
    finally:
        for name, function in saved_ops.items():
            setattr(ops, name, function)
        ModelRunner._check_device, ModelRunner._guard, ModelRunner.synchronize, ModelRunner._graphable = saved
