"""Plain PyTorch references of every kernel, with the signatures of ``flexengine_b200.ops``.

Two uses: the ``-m gpu`` tests compare each CUDA kernel with its function here, and the
CPU tests hand this module to the engine as its kernel provider, so that the step
function, cache and scheduler are exercised here without a GPU.  Intermediate math is
float32; results are rounded to the dtype the kernel returns.
"""
from __future__ import annotations

import math

import torch


def embedding(token_ids, table, scale=1.0, streams=None):
    rows = table[token_ids.long()].float() * scale
    return rows if streams is None else rows[None].repeat(streams, 1, 1)


def carry_tokens(token_ids, rows, sources, previous):
    keep = rows >= 0
    token_ids[rows[keep].long()] = previous[sources[keep].long()].to(token_ids.dtype)


def _post_normed(delta, post):
    """What a branch output becomes on its way through a norm of its own: w * (y + bias) / rms(y + bias)."""
    weight, eps, bias = post
    y = delta.float() if bias is None else delta.float() + bias.float()
    return y * torch.rsqrt(y.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.float()


def add_rmsnorm(residual, delta, weight, eps, out_dtype, rows=None, upcoming=None, post=None):
    if post is not None and delta is not None:
        delta = _post_normed(delta if rows is None else delta[rows.long()], post)
        if rows is None:
            residual += delta
            x = residual
        else:
            x = residual[rows.long()] + delta
        variance = x.pow(2).mean(dim=-1, keepdim=True)
        return (x * torch.rsqrt(variance + eps) * weight.float()).to(out_dtype)
    if rows is None:
        if delta is not None:
            residual += delta.float()
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return (x * torch.rsqrt(variance + eps) * weight.float()).to(out_dtype)


def residual_concat(residual, delta, extra, out_dtype, post=None):
    """residual += delta (through its own norm with ``post``), then [residual | extra] in ``out_dtype``."""
    if delta is not None:
        residual += _post_normed(delta, post) if post is not None else delta.float()
    return torch.cat([residual, extra.float()], dim=-1).to(out_dtype)


def scale_softcap(logits, scale, cap):
    logits.mul_(scale)
    if cap > 0.0:
        logits.copy_(cap * torch.tanh(logits / cap))
    return logits


def linear(x, w, bias=None, out_float32=False):
    y = x.float() @ w.float().T
    if bias is not None:
        y = y + bias.float()
    return y if out_float32 else y.to(x.dtype)


def swiglu(gate_up, intermediate):
    g = gate_up[:, :intermediate].float()
    u = gate_up[:, intermediate:].float()
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def linear_swiglu(x, w, intermediate):
    return swiglu(linear(x, w), intermediate)


def gated_activation(gate_up, intermediate, activation, bias=None, out_dtype=None):
    g = gate_up[:, :intermediate].float()
    u = gate_up[:, intermediate:].float()
    if bias is not None:
        g, u = g + bias[:intermediate].float(), u + bias[intermediate:].float()
    if activation == "silu":
        a = g / (1.0 + torch.exp(-g))
    elif activation == "gelu_tanh":
        a = 0.5 * g * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (g + 0.044715 * g * g * g)))
    else:
        raise ValueError(activation)
    return (a * u).to(out_dtype or gate_up.dtype)


def linear_gated(x, w, intermediate, activation):
    return gated_activation(linear(x, w), intermediate, activation)


def qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache,
                        nq, nkv, d, page_size, src=None):
    """``src``: the projection in float32 when it was kept so; else ``qkv`` is rewritten in place."""
    T = qkv.shape[0]
    x = (qkv if src is None else src).float()
    if bias is not None:
        x = x + bias.float()
    x = x.view(T, nq + 2 * nkv, d)
    if inv_freq is not None and rot > 0:
        ang = positions.float()[:, None] * inv_freq.float()[None, :]          # [T, rot/2]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        qk = x[:, :nq + nkv]
        a, b = qk[..., :rot // 2].clone(), qk[..., rot // 2:rot].clone()
        qk[..., :rot // 2] = a * cos - b * sin
        qk[..., rot // 2:rot] = b * cos + a * sin
    out = x.to(qkv.dtype)
    qkv.copy_(out.view(T, -1))
    if slot_mapping is not None:
        slots = slot_mapping.long()
        keep = slots >= 0
        page, off = slots[keep] // page_size, slots[keep] % page_size
        k_cache[page, :, off] = out[keep, nq:nq + nkv]
        v_cache[page, :, off] = out[keep, nq + nkv:]


def qkv_projection(h, w, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size):
    """The product stays float32 until bias and rotation are in: one rounding, whatever the number of rows."""
    product = linear(h, w, out_float32=True)
    qkv = torch.empty(product.shape, dtype=h.dtype, device=h.device)
    qkv_bias_rope_cache(qkv, bias, positions, inv_freq, rot, slot_mapping, k_cache, v_cache, nq, nkv, d, page_size,
                        src=product)
    return qkv


def paged_attention(qkv, k_cache, v_cache, block_table, ctx, nq, nkv, d, page_size, scale, window, upcoming=None, sink=False,
                    weights="softmax", head_bias=None):
    """``window`` > 0: the last ``window`` keys; < 0: the earlier keys of the query's chunk of -window positions.
    ``sink``: 1 is added to the softmax's denominator.  ``weights`` "sigmoid": a visible key weighs
    sigmoid(score + head_bias[head]), not normalised over the keys."""
    T = qkv.shape[0]
    chunk, window = (-window, 0) if window < 0 else (0, window)
    out = torch.zeros(T, nq * d, dtype=qkv.dtype, device=qkv.device)
    q_all = qkv[:, :nq * d].float().view(T, nq, d)
    cu = ctx.cu_q.tolist()
    starts = ctx.q_start.tolist()
    ratio = nq // nkv
    for r in range(len(starts)):
        q = q_all[cu[r]:cu[r + 1]]
        n = q.shape[0]
        length = starts[r] + n
        lo = max(0, starts[r] - window + 1) if window > 0 else (starts[r] // chunk * chunk if chunk else 0)
        lo_page = lo // page_size
        pages = block_table[r, lo_page:-(-length // page_size)].long()
        k = k_cache[pages].float().permute(0, 2, 1, 3).reshape(-1, nkv, d)      # [tokens, nkv, d]
        v = v_cache[pages].float().permute(0, 2, 1, 3).reshape(-1, nkv, d)
        key_pos = torch.arange(lo_page * page_size, lo_page * page_size + k.shape[0], device=q.device)
        q_pos = torch.arange(starts[r], length, device=q.device)
        visible = (key_pos[None, :] <= q_pos[:, None]) & (key_pos[None, :] < length)
        if window > 0:
            visible &= key_pos[None, :] > q_pos[:, None] - window
        if chunk:
            visible &= key_pos[None, :] // chunk == q_pos[:, None] // chunk
        kh = k.repeat_interleave(ratio, dim=1)
        vh = v.repeat_interleave(ratio, dim=1)
        scores = torch.einsum("qhd,thd->hqt", q, kh) * scale
        scores = scores.masked_fill(~visible[None], float("-inf"))
        if weights == "sigmoid":
            w = torch.sigmoid(scores if head_bias is None else scores + head_bias.float()[:, None, None])
        elif sink:
            top = torch.clamp(scores.max(dim=-1, keepdim=True).values, min=0.0)
            e = torch.exp(scores - top)
            w = e / (e.sum(dim=-1, keepdim=True) + torch.exp(-top))
        else:
            w = torch.softmax(scores, dim=-1)
        w = torch.where(visible[None], w, torch.zeros_like(w))
        o = torch.einsum("hqt,thd->qhd", w, vh)
        out[cu[r]:cu[r + 1]] = o.reshape(n, nq * d).to(qkv.dtype)
    return out


# ---- several residual streams, token shift, gated attention, minGRU ---------------------------------------
FUSES_TOKEN_SHIFT = True


def stream_rmsnorm(streams, read, weight, eps, out_dtype, update=None, rows=None, shift=None):
    """u = sum_s read[s] x_s (read None: the plain sum) through an RMSNorm; ``update`` (y, gate, gate_bias, mix, write) is
    put into the streams first: x_t <- sum_s mix[s, t] x_s + write[t] * y * sigmoid(gate + gate_bias).  With ``rows``
    only those rows are read and nothing is written back."""
    x = streams if rows is None else streams[:, rows.long()]
    if update is not None:
        y, gate = update.y.float(), update.gate.float()
        if rows is not None:
            y, gate = y[rows.long()], gate[rows.long()]
        gated = y * torch.sigmoid(gate + update.gate_bias.float())
        x = torch.einsum("st,snd->tnd", update.mix.float(), x) + update.write.float()[:, None, None] * gated[None]
        if rows is None:
            streams.copy_(x)
    u = x.sum(dim=0) if read is None else torch.einsum("s,snd->nd", read.float(), x)
    out = (u * torch.rsqrt(u.pow(2).mean(dim=-1, keepdim=True) + eps) * weight.float()).to(out_dtype)
    if shift is None:
        return out
    # a step of one token a request: row i is request i's; the token shift of the normed rows, on the rows as rounded
    mu, kept, seats = shift
    hf = out.float()
    before = torch.zeros_like(hf)
    for i, seat in enumerate(seats.tolist()):
        if seat >= 0:
            before[i] = kept[seat]
            kept[seat] = hf[i]
    return out, (hf + (before - hf) * mu.float()).to(out_dtype)


def token_shift(h, mu, kept, state_slots, cu_q, token_request):
    """h + (h' - h) * mu with h' the row before (the seat's kept row for a portion's first token, zeros for a seat below
    0); every seat then keeps its request's last row."""
    hf = h.float()
    before = torch.zeros_like(hf)
    cu, seats = cu_q.tolist(), state_slots.tolist()
    for r in range(len(seats)):
        a, b = cu[r], cu[r + 1]
        before[a + 1:b] = hf[a:b - 1]
        if seats[r] >= 0:
            before[a] = kept[seats[r]]
            kept[seats[r]] = hf[b - 1]
    return (hf + (before - hf) * mu.float()).to(h.dtype)


def qkv_conv_rope_norm_cache(projected, conv, history, taps, state_slots, cu_q, token_request, positions, inv_freq, rot_dims,
                             qk_norm, eps, slot_mapping, k_cache, v_cache, heads, kv_heads, dim, vdim, head, page_size,
                             q_weight=None, k_weight=None, temp=None):
    """projected [T, >= channels] holds q | k | v.  A causal convolution of ``taps`` taps over time per channel (``conv``
    [taps, channels]; ``history`` [seats, (taps - 1) channels] holds every request's last taps - 1 projected rows and is
    brought up to date), rotation of the first ``rot_dims`` entries of the query and key heads, their unit norm, keys and
    values into the cache and the queries out, both padded with zeros to ``head`` entries a head."""
    T = projected.shape[0]
    C = (heads + kv_heads) * dim + kv_heads * vdim
    u = projected[:, :C].float()
    if conv is not None:
        y = torch.zeros_like(u)
        cu, seats = cu_q.tolist(), state_slots.tolist()
        back = taps - 1
        for r in range(len(seats)):
            a, b = cu[r], cu[r + 1]
            old = history[seats[r]].view(back, C) if (seats[r] >= 0 and back) else torch.zeros(back, C, device=u.device)
            rows = torch.cat([old, u[a:b]])
            for j in range(taps):
                y[a:b] += conv[j].float() * rows[j:j + (b - a)]
            if seats[r] >= 0 and back:
                history[seats[r]] = rows[rows.shape[0] - back:].reshape(-1)
        u = y
    q = u[:, :heads * dim].reshape(T, heads, dim)
    k = u[:, heads * dim:(heads + kv_heads) * dim].reshape(T, kv_heads, dim)
    v = u[:, (heads + kv_heads) * dim:].reshape(T, kv_heads, vdim)
    if inv_freq is not None and rot_dims > 0:
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        half = rot_dims // 2

        def turn(x):
            a, b = x[..., :half], x[..., half:rot_dims]
            return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot_dims:]], dim=-1)
        q, k = turn(q), turn(k)
    if qk_norm:
        q = q * torch.rsqrt(q.pow(2).mean(dim=-1, keepdim=True) + eps)
        k = k * torch.rsqrt(k.pow(2).mean(dim=-1, keepdim=True) + eps)
    if q_weight is not None:
        q, k = q * q_weight.float(), k * k_weight.float()
    if temp is not None:
        coef, every = temp
        q = q * (1.0 + coef * torch.log(torch.div(positions + 1, every, rounding_mode="floor").float() + 1.0))[:, None, None]
    dt = projected.dtype
    queries = torch.zeros(T, heads, head, dtype=dt, device=u.device)
    queries[..., :dim] = q.to(dt)
    if slot_mapping is not None:
        slots = slot_mapping.long()
        keep = slots >= 0
        page, off = slots[keep] // page_size, slots[keep] % page_size
        kp = torch.zeros(T, kv_heads, head, dtype=dt, device=u.device)
        vp = torch.zeros(T, kv_heads, head, dtype=dt, device=u.device)
        kp[..., :dim] = k.to(dt)
        vp[..., :vdim] = v.to(dt)
        k_cache[page, :, off] = kp[keep]
        v_cache[page, :, off] = vp[keep]
    return queries.view(T, heads * head)


def _turn(x, positions, inv_freq, dims, pairs, sign=1.0):
    """x [T, heads, n]: the first ``dims`` entries of every head turn by sign * position * inv_freq."""
    ang = sign * positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
    y = x.clone()
    if pairs == "interleaved":
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        y[..., 0:dims:2] = a * cos - b * sin
        y[..., 1:dims:2] = b * cos + a * sin
    else:
        half = dims // 2
        a, b = x[..., :half], x[..., half:dims]
        y[..., :half] = a * cos - b * sin
        y[..., half:dims] = b * cos + a * sin
    return y


def qkv_norm_rope_cache(projected, q_weight, k_weight, eps, positions, inv_freq, rot_dims, pairs, value_inv_freq, slot_mapping,
                        k_cache, v_cache, heads, kv_heads, dim, vdim, head, page_size):
    """projected [T, >= channels] holds q | k | v.  One RMS norm over the whole query projection and one over the whole key
    projection (weights of their full widths; None: no norm), then the rotation of the first ``rot_dims`` entries of every
    query and key head, the values turned over all ``vdim`` entries (``value_inv_freq`` None: as they are), keys and values
    into the cache and the queries out, padded with zeros to ``head`` entries a head."""
    T = projected.shape[0]
    qw, kw = heads * dim, kv_heads * dim
    u = projected.float()
    q, k, v = u[:, :qw], u[:, qw:qw + kw], u[:, qw + kw:qw + kw + kv_heads * vdim]
    if q_weight is not None:
        q = q * torch.rsqrt(q.pow(2).mean(dim=-1, keepdim=True) + eps) * q_weight.float()
        k = k * torch.rsqrt(k.pow(2).mean(dim=-1, keepdim=True) + eps) * k_weight.float()
    q, k, v = q.reshape(T, heads, dim), k.reshape(T, kv_heads, dim), v.reshape(T, kv_heads, vdim)
    if inv_freq is not None and rot_dims > 0:
        q, k = _turn(q, positions, inv_freq, rot_dims, pairs), _turn(k, positions, inv_freq, rot_dims, pairs)
    if value_inv_freq is not None:
        v = _turn(v, positions, value_inv_freq, vdim, pairs)
    dt = projected.dtype
    queries = torch.zeros(T, heads, head, dtype=dt, device=u.device)
    queries[..., :dim] = q.to(dt)
    if slot_mapping is not None:
        slots = slot_mapping.long()
        keep = slots >= 0
        page, off = slots[keep] // page_size, slots[keep] % page_size
        kp = torch.zeros(T, kv_heads, head, dtype=dt, device=u.device)
        vp = torch.zeros(T, kv_heads, head, dtype=dt, device=u.device)
        kp[..., :dim] = k.to(dt)
        vp[..., :vdim] = v.to(dt)
        k_cache[page, :, off] = kp[keep]
        v_cache[page, :, off] = vp[keep]
    return queries.view(T, heads * head)


def unrotate_heads(mixed, positions, inv_freq, heads, head, vdim, pairs, scale=1.0, out=None):
    """[T, heads vdim]: the first ``vdim`` entries of every head of ``mixed`` [T, heads head] turned back by the position
    (pair m by -position * inv_freq[m]), times ``scale``."""
    T = mixed.shape[0]
    rows = _turn(mixed.float().view(T, heads, head)[..., :vdim], positions, inv_freq, vdim, pairs, sign=-1.0) * scale
    rows = rows.reshape(T, heads * vdim).to(mixed.dtype)
    if out is None:
        return rows
    out.copy_(rows)
    return out


def head_gate(mixed, projected, offset, heads, head, vdim, per_element=False, scale=1.0, out=None):
    """out[t, h, :vdim] = mixed[t, h, :vdim] * sigmoid(projected[t, offset + h]) * scale; with ``per_element`` the gate of
    entry j of head h is projected[t, offset + h vdim + j]."""
    T = mixed.shape[0]
    if per_element:
        gate = torch.sigmoid(projected[:, offset:offset + heads * vdim].float()).view(T, heads, vdim)
    else:
        gate = torch.sigmoid(projected[:, offset:offset + heads].float())[:, :, None]
    rows = (mixed.view(T, heads, head)[..., :vdim].float() * gate * scale).reshape(T, heads * vdim).to(mixed.dtype)
    if out is None:
        return rows
    out.copy_(rows)
    return out


def rotate_heads(projected, heads, dim, positions, inv_freq, rot_dims, scales):
    """float32 [T, heads dim]: the first ``heads * dim`` columns of ``projected`` as heads of ``dim``, the first ``rot_dims``
    entries of each turned by position * inv_freq (pairs i, i + rot_dims/2); ``scales`` ((count, factor), ...) multiplies
    runs of heads by a factor each."""
    T = projected.shape[0]
    x = projected[:, :heads * dim].float().reshape(T, heads, dim)
    if inv_freq is not None and rot_dims > 0:
        ang = positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        half = rot_dims // 2
        a, b = x[..., :half], x[..., half:rot_dims]
        x = torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot_dims:]], dim=-1)
    factor = torch.cat([torch.full((count,), float(f)) for count, f in scales]).to(x.device)
    return (x * factor[None, :, None]).reshape(T, heads * dim).contiguous()


def retention_scan(qk, values, decay, state, state_slots, cu_q, heads, dim, vdim, max_q_len=0):
    """S <- decay_h S + k_t v_t^T, o_t = S^T q_t per request and head, S [dim, vdim] float32 in ``state[seat]`` (zeros and
    nothing kept for a seat below 0).  qk float32 [T, 2 heads dim] (queries, then keys); values [T, heads vdim]."""
    T = qk.shape[0]
    q = qk[:, :heads * dim].view(T, heads, dim)
    k = qk[:, heads * dim:].view(T, heads, dim)
    v = values.float().reshape(T, heads, vdim)
    out = torch.zeros(T, heads, vdim, dtype=torch.float32, device=qk.device)
    cu, seats = cu_q.tolist(), state_slots.tolist()
    w = decay.float()[:, None, None]
    for r in range(len(seats)):
        seat = seats[r]
        S = state[seat, :heads * dim * vdim].view(heads, dim, vdim).clone() if seat >= 0 else torch.zeros(heads, dim, vdim, device=qk.device)
        for t in range(cu[r], cu[r + 1]):
            S = w * S + k[t][:, :, None] * v[t][:, None, :]
            out[t] = torch.einsum("hdv,hd->hv", S, q[t])
        if seat >= 0:
            state[seat, :heads * dim * vdim] = S.reshape(-1)
    return out.view(T, heads * vdim)


def retention_decode(projected, heads, dim, vdim, positions, inv_freq, rot_dims, key_scale, decay, state, state_slots, eps, out_dtype,
                     scale=1.0, into=None):
    """One token a request: rotation, recurrence, head norm and gate (the three references above, one after the other)."""
    R = projected.shape[0]
    qk = rotate_heads(projected, 2 * heads, dim, positions, inv_freq, rot_dims, ((heads, 1.0), (heads, key_scale)))
    at = 2 * heads * dim
    cu = torch.arange(R + 1, dtype=torch.int32, device=projected.device)
    o = retention_scan(qk, projected[:, at:at + heads * vdim], decay, state, state_slots, cu, heads, dim, vdim)
    return head_rmsnorm_gate(o, None, projected[:, at + heads * vdim:at + 2 * heads * vdim], eps, heads, out_dtype, scale=scale, into=into)


def mingru_scan(zxg, bias, state, state_slots, cu_q, width, out_dtype, max_q_len=0):
    """zxg [T, 3 width] float32 (z | x | g before their biases and activations).  z = sigmoid(. + b_z), u = . + b_x,
    c = u + 1/2 where u >= 0 else sigmoid(u), S <- (1 - z) S + z c from the seat's kept S (zeros for a seat below 0),
    out = S * silu(g)."""
    W = width
    z = torch.sigmoid(zxg[:, :W].float() + bias[:W].float())
    u = zxg[:, W:2 * W].float() + bias[W:].float()
    c = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    g = zxg[:, 2 * W:].float()
    out = torch.zeros(zxg.shape[0], W, dtype=torch.float32, device=zxg.device)
    cu, seats = cu_q.tolist(), state_slots.tolist()
    for r in range(len(seats)):
        S = state[seats[r]].clone() if seats[r] >= 0 else torch.zeros(W, device=zxg.device)
        for t in range(cu[r], cu[r + 1]):
            S = (1.0 - z[t]) * S + z[t] * c[t]
            out[t] = S
        if seats[r] >= 0:
            state[seats[r]] = S
    return (out * (g / (1.0 + torch.exp(-g)))).to(out_dtype)


# ---- hashed pair embedding, grouped norm, depth average ----------------------------------------------
def embedding_hashed_pairs(token_ids, table, pair_table, previous, state_slots, cu_q, q_start, token_request,
                           buckets, mul_prev, mul_cur):
    """table[token] + pair_table[(previous token * mul_prev + token * mul_cur) % buckets], row ``buckets`` at
    position 0; ``previous`` [seats, 1] holds every seat's last token and is brought up to date."""
    out = table[token_ids.long()].float()
    cu, starts, seats = cu_q.tolist(), q_start.tolist(), state_slots.tolist()
    for r in range(len(starts)):
        a, b = cu[r], cu[r + 1]
        tokens = token_ids[a:b].long()
        before = torch.zeros_like(tokens)
        before[1:] = tokens[:-1]
        if starts[r] > 0 and seats[r] >= 0:
            before[0] = previous[seats[r], 0]
        rows = (before * mul_prev + tokens * mul_cur) % buckets
        if starts[r] == 0:
            rows[0] = buckets
        out[a:b] += pair_table[rows].float()
        if seats[r] >= 0:
            previous[seats[r], 0] = tokens[-1].to(previous.dtype)
    return out


def add_group_rmsnorm(residual, delta, weight, eps, groups, out_dtype, rows=None):
    if rows is None:
        if delta is not None:
            residual += delta.float()
        x = residual
    else:
        x = residual[rows.long()]
        if delta is not None:
            x = x + delta[rows.long()].float()
    n, width = x.shape
    parts = x.view(n, groups, width // groups)
    parts = parts * torch.rsqrt(parts.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (parts.reshape(n, width) * weight.float()).to(out_dtype)


def depth_average(history, x, mixed, fed, alpha, depth):
    """history[depth + 1] = x + (mixed + fed); x <- sum_j alpha[j] history[j], j = 0 .. depth + 1 (history[0] = x first
    when depth is 0).  All float32."""
    if depth == 0:
        history[0].copy_(x)
    delta = mixed.float() if fed is None else mixed.float() + fed.float()
    history[depth + 1].copy_(x + delta)
    total = torch.zeros_like(x)
    for j in range(depth + 2):
        total += alpha[j] * history[j]
    x.copy_(total)


# ---- linear-recurrent mixer ---------------------------------------------------------------------------
def token_shift_blend(h, mu, state, offset, state_slots, cu_q, token_request):
    """Five blends h + (h' - h) * mu_s with h' the row before (the seat's kept row for a portion's first token);
    returns ([4, T, D] in h's dtype, [T, D] float32) and keeps every seat's last row in state[seat, offset:]."""
    T, D = h.shape
    hf = h.float()
    before = torch.zeros_like(hf)
    cu, seats = cu_q.tolist(), state_slots.tolist()
    for r in range(len(seats)):
        a, b = cu[r], cu[r + 1]
        before[a + 1:b] = hf[a:b - 1]
        if seats[r] >= 0:
            before[a] = state[seats[r], offset:offset + D]
            state[seats[r], offset:offset + D] = hf[b - 1]
    mus = mu.float().view(5, D)
    blends = hf[None] + (before - hf)[None] * mus[:, None, :]
    return blends[:4].to(h.dtype).contiguous(), blends[4].contiguous()


def activation(x, kind, params=None):
    z = x.float()
    if kind == "tanh":
        y = torch.tanh(z)
    elif kind == "xielu":
        p, q = params.float()
        ap, an = torch.log1p(torch.exp(p)), 0.5 + torch.log1p(torch.exp(q))
        y = torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.exp(torch.clamp(z, max=0.0)) - 1.0 - z) + 0.5 * z)
    elif kind == "relu2":
        y = torch.relu(z) ** 2
    else:
        raise ValueError(kind)
    return y.to(x.dtype)


def linear_activated(x, w, kind):
    return activation(linear(x, w), kind)


def wkv_recurrence(r, k, v, decay_logits, w0, u, state, state_slots, cu_q, heads, dim):
    T = r.shape[0]
    rf, kf, vf = (t.float().view(T, heads, dim) for t in (r, k, v))
    decay = torch.exp(-torch.exp(decay_logits.float() + w0.float())).view(T, heads, dim)
    bonus = u.float().view(heads, dim)
    out = torch.zeros(T, heads, dim, dtype=torch.float32, device=r.device)
    cu, seats = cu_q.tolist(), state_slots.tolist()
    n = heads * dim * dim
    for i in range(len(seats)):
        S = state[seats[i], :n].view(heads, dim, dim).clone() if seats[i] >= 0 else torch.zeros(heads, dim, dim)
        for t in range(cu[i], cu[i + 1]):
            kv = kf[t][:, :, None] * vf[t][:, None, :]
            out[t] = torch.einsum("hi,hij->hj", rf[t], S + bonus[:, :, None] * kv)
            S = decay[t][:, :, None] * S + kv
        if seats[i] >= 0:
            state[seats[i], :n] = S.reshape(-1)
    return out.view(T, heads * dim)


def head_rmsnorm_gate(out, weight, g, eps, heads, out_dtype, scale=1.0, into=None):
    T, inner = out.shape
    x = out.float().view(T, heads, inner // heads)
    x = (x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)).reshape(T, inner)
    if weight is not None:
        x = x * weight.float()
    gf = g.float()
    rows = (x * (gf / (1.0 + torch.exp(-gf))) * scale).to(out_dtype)
    if into is None:
        return rows
    into.copy_(rows)
    return into


# ---- attention over a cached latent -------------------------------------------------------------------
def batched_linear(x, w, token_major=False):
    """x [B, M, K] (any strides) times w [B, N, K]^T -> [B, M, N], or [M, B N] with ``token_major``."""
    y = torch.einsum("bmk,bnk->bmn", x.float(), w.float()).to(x.dtype)
    if token_major:
        return y.transpose(0, 1).reshape(x.shape[1], -1).contiguous()
    return y


def latent_prepare(q, q_latent, down, norm_weight, eps, positions, inv_freq, rot_dims, slot_mapping, rows,
                   heads, dim, rot_dim, rank, row, page_size):
    T = q.shape[0]
    qf = q.float().view(T, heads, dim + rot_dim)
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    cos, sin = ang.cos(), ang.sin()

    def turn(x):                                   # x [..., rot_dim], pairs (2i, 2i + 1) of the first rot_dims
        y = x.clone()
        a, b = x[..., 0:rot_dims:2], x[..., 1:rot_dims:2]
        c, s = (cos, sin) if x.dim() == 2 else (cos[:, None, :], sin[:, None, :])
        y[..., 0:rot_dims:2] = a * c - b * s
        y[..., 1:rot_dims:2] = b * c + a * s
        return y

    queries = torch.zeros(T, heads, row, dtype=torch.float32, device=q.device)
    queries[:, :, :rank] = q_latent.float().transpose(0, 1)
    queries[:, :, rank:rank + rot_dim] = turn(qf[:, :, dim:])
    if down is None:                             # a layer that reads another layer's latents: queries only
        return queries.view(T, heads * row).to(q.dtype)
    latent = down.float()[:, :rank]
    latent = latent * torch.rsqrt(latent.pow(2).mean(dim=-1, keepdim=True) + eps) * norm_weight.float()
    cached = torch.zeros(T, row, dtype=torch.float32, device=q.device)
    cached[:, :rank] = latent
    cached[:, rank:rank + rot_dim] = turn(down.float()[:, rank:])
    if slot_mapping is not None:
        slots = slot_mapping.long()
        keep = slots >= 0
        rows[slots[keep] // page_size, 0, slots[keep] % page_size] = cached[keep].to(rows.dtype)
    return queries.view(T, heads * row).to(q.dtype)


# ---- routed feed-forward ------------------------------------------------------------------------------
def route_top(logits, top, scale, over_chosen=False, correction=None, groups=(1, 1)):
    """``correction`` (float32, one number per router output) is added to the scores for the choice only; ``groups`` =
    (count, keep): only outputs of the ``keep`` groups (of ``count`` equal groups of neighbours) with the largest corrected
    score can be chosen.  Ties go to the lower index."""
    count, keep = groups
    if correction is not None or count > 1:
        scores = torch.softmax(logits.float(), dim=-1)
        choice = scores if correction is None else scores + correction.float()
        T, E = choice.shape
        if count > 1:
            best = choice.view(T, count, E // count).max(dim=-1).values
            order = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
            kept = torch.zeros(T, count, dtype=torch.bool, device=choice.device)
            kept.scatter_(1, order, True)
            choice = choice.masked_fill(~kept.repeat_interleave(E // count, dim=1), float("-inf"))
        picked = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
        return picked.to(torch.int32), (scores.gather(1, picked) * scale).float()
    if over_chosen:
        best = torch.topk(logits.float(), top, dim=-1)
        return best.indices.to(torch.int32), (torch.softmax(best.values, dim=-1) * scale).float()
    scores = torch.softmax(logits.float(), dim=-1)
    best = torch.topk(scores, top, dim=-1)
    return best.indices.to(torch.int32), (best.values * scale).float()


def routed_experts(h, chosen, weights, gate_up, down, shared=None, activation="silu", limit=0.0, identity=0):
    """``activation`` "relu2": ``gate_up`` is [experts, F, H], an expert is down(relu(up h)^2).  ``identity``: choices from
    ``experts`` on stand for experts that return their input."""
    T, D = h.shape
    f = down.shape[2]
    experts = down.shape[0]
    total = torch.zeros(T, D, dtype=torch.float32, device=h.device)
    hf = h.float()
    for slot in range(chosen.shape[1]):                   # a token's experts are added in the order they were chosen
        for e in chosen[:, slot].unique().tolist():
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if e >= experts:
                if e < experts + identity:
                    total[rows] += weights[rows, slot, None] * hf[rows]
                continue
            gu = hf[rows] @ gate_up[e].float().T
            if activation == "relu2":
                act = (torch.relu(gu) ** 2).to(h.dtype).float()
                total[rows] += weights[rows, slot, None] * (act @ down[e].float().T)
                continue
            g, u = gu[:, :f], gu[:, f:]
            if activation == "clamped":
                g, u = torch.clamp(g, max=limit), torch.clamp(u, min=-limit, max=limit)
                act = (g / (1.0 + torch.exp(-1.702 * g)) * (u + 1.0)).to(h.dtype).float()
            else:
                act = (g / (1.0 + torch.exp(-g)) * u).to(h.dtype).float()
            total[rows] += weights[rows, slot, None] * (act @ down[e].float().T)
    if shared is not None:
        total += shared.float()
    return total.to(h.dtype)


# ---- sampling ----------------------------------------------------------------------------------
MASK64 = (1 << 64) - 1


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & MASK64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & MASK64
    return x ^ (x >> 31)


def uniform_from(seed: int, draw: int) -> float:
    """The uniform number in [0, 1) of request seed ``seed`` at its ``draw``-th sampled token."""
    bits = splitmix64((splitmix64(seed & MASK64) + draw) & MASK64)
    return (bits >> 40) * (1.0 / (1 << 24))


def sample(logits, temperature, top_k, seed, draw):
    """Greedy rows (temperature 0): lowest index of the maximum.  Other rows: x = logits / T; keep
    the k largest (ties by lowest index) when 0 < k < V; p = softmax over the kept; the token is
    the first index whose cumulative probability (in index order) exceeds u * total."""
    R, V = logits.shape
    out = torch.zeros(R, dtype=torch.int32)
    for r in range(R):
        row = logits[r].detach().float().cpu()
        t = float(temperature[r])
        if t == 0.0:
            out[r] = int(torch.nonzero(row == row.max())[0])
            continue
        x = row / t
        k = int(top_k[r])
        keep = torch.ones(V, dtype=torch.bool)
        if 0 < k < V:
            order = torch.sort(x, descending=True, stable=True).indices[:k]
            keep = torch.zeros(V, dtype=torch.bool)
            keep[order] = True
        e = torch.where(keep, torch.exp(x - x[keep].max()), torch.zeros_like(x)).double()
        cum = torch.cumsum(e, 0)
        u = uniform_from(int(seed[r]), int(draw[r]))
        target = u * float(cum[-1])
        idx = int(torch.searchsorted(cum, torch.tensor(target, dtype=torch.float64), right=True))
        idx = min(idx, V - 1)
        while not keep[idx]:
            idx -= 1
        out[r] = idx
    return out.to(logits.device)
