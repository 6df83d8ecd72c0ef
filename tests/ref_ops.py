"""Plain PyTorch statement of every kernel the engine launches: the reference each CUDA
kernel is tested against, and a stand-in kernel namespace that lets the engine's batching
and cache logic run on the CPU inside the tests.  Not part of the product path: the package
never imports this file."""
from __future__ import annotations

import torch


class TorchRefOps:
    prefill_tile = 64

    # ---------------------------------------------------------------- elementwise / norms
    def scatter_i32(self, table, idx, val):
        table[idx.long()] = val

    def embedding(self, ids, table):
        return table[ids.long()]

    def add_rmsnorm(self, x, delta, weight, eps, rows=None):
        if rows is None:
            if delta is not None:
                x.copy_((x.float() + delta.float()).to(x.dtype))
            src = x
        else:
            src = x[rows.long()]
            if delta is not None:
                src = (src.float() + delta[rows.long()].float()).to(x.dtype)
        x32 = src.float()
        y = (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
        return (y.float() * weight.float()).to(x.dtype)

    def linear(self, x, w, out_dtype=None, defer=False):
        return (x.float() @ w.float().T).to(out_dtype or x.dtype)

    def gated_linear(self, x, w):
        return self.swiglu(self.linear(x, w))

    def swiglu(self, gate_up):
        g, u = gate_up.float().chunk(2, dim=-1)
        return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)

    # ---------------------------------------------------------------- q/k norm, rotation, cache write
    def qk_norm_rope_cache(self, qkv, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        T = qkv.shape[0]
        dt = qkv.dtype
        q, k, v = qkv.split([H * D, KV * D, KV * D], dim=-1)
        q, k, v = q.reshape(T, H, D), k.reshape(T, KV, D), v.reshape(T, KV, D)

        def norm(t, w):
            if w is None:
                return t
            t32 = t.float()
            y = (t32 * torch.rsqrt(t32.pow(2).mean(-1, keepdim=True) + eps)).to(dt)
            return (y.float() * w.float()).to(dt)

        def rope(t):
            if inv_freq is None:
                return t
            ang = meta.positions.float()[:, None] * inv_freq.float()[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            t32 = t.float()
            a, b = t32[..., :D // 2], t32[..., D // 2:]
            return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(dt)

        q = rope(norm(q, q_weight))
        if k_cache is not None:
            k = rope(norm(k, k_weight))
            page, off = meta.slots.long() // meta.page_size, meta.slots.long() % meta.page_size
            k_cache[page, :, off, :] = k
            v_cache[page, :, off, :] = v
        return q.reshape(T, H * D)

    def qkv_project(self, h, w, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        return self.qk_norm_rope_cache(self.linear(h, w), H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache)

    # ---------------------------------------------------------------- attention over the pages
    def paged_attention(self, q, k_cache, v_cache, meta, H, KV, D, scale, window):
        T = q.shape[0]
        out = torch.empty_like(q)
        q = q.view(T, H, D)
        q_start = meta.seg_q_start.tolist()
        pos0, kv_len = meta.seg_pos0.tolist(), meta.seg_kv_len.tolist()
        ps = meta.page_size
        rows = getattr(meta, "table_rows", None)
        rows = list(range(len(pos0))) if rows is None else rows.tolist()
        for s in range(len(pos0)):
            a, b, L = q_start[s], q_start[s + 1], kv_len[s]
            j = torch.arange(L, device=q.device)
            pages = meta.block_table[rows[s], j // ps].long()
            k = k_cache[pages, :, j % ps, :].float()              # [L, KV, D]
            v = v_cache[pages, :, j % ps, :].float()
            k = k.repeat_interleave(H // KV, dim=1)
            v = v.repeat_interleave(H // KV, dim=1)
            p = pos0[s] + torch.arange(b - a, device=q.device)
            visible = j[None, :] <= p[:, None]
            if window is not None:
                visible &= j[None, :] > p[:, None] - window
            sc = torch.einsum("phd,jhd->hpj", q[a:b].float(), k) * scale
            sc = sc.masked_fill(~visible[None], float("-inf"))
            o = torch.einsum("hpj,jhd->phd", torch.softmax(sc, dim=-1), v)
            out[a:b] = o.reshape(b - a, H * D).to(q.dtype)
        return out

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        return logits.argmax(dim=-1).to(torch.int32)

    def sample(self, logits, temperatures, seeds, counters):
        from tests.ref_sampling import gumbel_sample_reference
        return gumbel_sample_reference(logits, temperatures, seeds, counters)


# ---------------------------------------------------------------- float32 stream, polynomial norm, recurrences, latent attention
def _rms(x, eps):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def _embed_scaled_norm(self, ids, table, g, eps, out_dtype):
    return (_rms(table[ids.long()].float(), eps) * g.float()).to(out_dtype)


def _add_scaled_rmsnorm(self, x, delta, g, eps, rows, pre_add, out_dtype):
    assert x.dtype == torch.float32
    if rows is None:
        if delta is not None:
            x.add_(delta.float())
        if pre_add is not None:
            x.add_(pre_add.float())
        src = x
    else:
        src = x[rows.long()]
        if delta is not None:
            src = src + delta[rows.long()].float()
        if pre_add is not None:
            src = src + pre_add.float()
    return (_rms(src, eps) * g.float()).to(out_dtype)


def _polynorm(self, z, coef, eps):
    z32 = z.float()
    a, b, c, e = coef.float().tolist()
    return (a * _rms(z32, eps) + b * _rms(z32 ** 2, eps) + c * _rms(z32 ** 3, eps) + e).to(z.dtype)


def _segments(batch):
    qs = batch.host["seg_q_start"]
    return [(int(qs[i]), int(qs[i + 1]), int(batch.host["seg_slot"][i])) for i in range(batch.num_segs)]


def _lightning_scan(self, p, H, D, V, decay, state, batch):
    T = p.shape[0]
    silu = torch.nn.functional.silu
    q = silu(p[:, :H * D].float()).view(T, H, D)
    k = silu(p[:, H * D:2 * H * D].float()).view(T, H, D)
    v = silu(p[:, 2 * H * D:2 * H * D + H * V].float()).view(T, H, V)
    o = torch.zeros(T, H * V, dtype=torch.float32, device=p.device)
    for a, b, slot in _segments(batch):
        S = state[slot].view(H, D, V).clone()
        for t in range(a, b):
            S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
        state[slot] = S.reshape(-1)
    return o


def _group_rmsnorm_gate(self, o, weight, gate, eps, groups, gs, out_dtype, act="sigmoid"):
    T = o.shape[0]
    y = _rms(o.view(T, groups, gs), eps).reshape(T, groups * gs)
    if weight is not None:
        y = y * weight.float().repeat(groups * gs // weight.numel())
    g = gate.float()
    return (y * (torch.sigmoid(g) if act == "sigmoid" else g * torch.sigmoid(g))).to(out_dtype)


def _delta_prepare(self, p, a, conv, A_log, dt_bias, H, KV, D, V, taps, unit_eps, state, batch):
    T = p.shape[0]
    C = 2 * KV * D + H * V
    x = p[:, :C].float()
    out = torch.zeros(T, (C + H * D + H + 3) // 4 * 4, dtype=torch.float32, device=p.device)      # q | k | v | g | beta | padding
    base = H * D * V
    for s0, s1, slot in _segments(batch):
        hist = state[slot, base:base + (taps - 1) * C].view(taps - 1, C)
        ext = torch.cat([hist, x[s0:s1]], dim=0)                           # row i: position first - (taps - 1) + i
        y = torch.zeros(s1 - s0, C, device=p.device)
        for j in range(taps):
            y += conv[:, j].float() * ext[j:j + s1 - s0]
        y = torch.nn.functional.silu(y)
        qk = y[:, :2 * KV * D].view(s1 - s0, 2 * KV, D)
        qk = qk / torch.sqrt(qk.pow(2).sum(-1, keepdim=True) + unit_eps)
        qk[:, :KV] *= D ** -0.5
        out[s0:s1, :2 * KV * D] = qk.reshape(s1 - s0, -1)
        out[s0:s1, 2 * KV * D:C] = y[:, 2 * KV * D:]
        if taps > 1:
            state[slot, base:base + (taps - 1) * C] = ext[ext.shape[0] - (taps - 1):].reshape(-1)
    out[:, C + H * D:C + H * D + H] = torch.sigmoid(p[:, C:C + H].float())
    sp = torch.nn.functional.softplus(a.float() + dt_bias.float()).view(T, H, D)
    out[:, C:C + H * D] = torch.exp(-torch.exp(A_log.float())[None, :, None] * sp).reshape(T, H * D)
    return out


def _delta_scan(self, prep, H, KV, D, V, state, batch):
    T = prep.shape[0]
    C = 2 * KV * D + H * V
    q = prep[:, :KV * D].view(T, KV, D).repeat_interleave(H // KV, dim=1)
    k = prep[:, KV * D:2 * KV * D].view(T, KV, D).repeat_interleave(H // KV, dim=1)
    v = prep[:, 2 * KV * D:C].view(T, H, V)
    g, beta = prep[:, C:C + H * D].view(T, H, D), prep[:, C + H * D:C + H * D + H]
    o = torch.zeros(T, H * V, dtype=torch.float32, device=prep.device)
    for s0, s1, slot in _segments(batch):
        S = state[slot, :H * D * V].view(H, D, V).clone()
        for t in range(s0, s1):
            S = g[t][:, :, None] * S
            u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
            S = S + k[t][:, :, None] * u[:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
        state[slot, :H * D * V] = S.reshape(-1)
    return o


def _batched_linear(self, x, col0, head_stride, K, w, side_by_side=False):
    H = w.shape[0]
    if col0 is not None:
        x = torch.stack([x[:, col0 + h * head_stride:col0 + h * head_stride + K] for h in range(H)])
    out = torch.einsum("htk,hnk->htn", x.float(), w.float()).to(x.dtype)
    return out.transpose(0, 1).reshape(out.shape[1], -1).contiguous() if side_by_side else out


def _rotate_pairs(v, positions, inv_freq):
    n = inv_freq.numel()
    ang = positions.float()[:, None] * inv_freq.float()[None, :]
    shape = (v.shape[0],) + (1,) * (v.dim() - 2) + (n,)
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    out = v.clone()
    a, b = v[..., 0:2 * n:2], v[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def _latent_prepare(self, p, q_abs, H, D, R, C, norm_w, eps, inv_freq, meta, cache):
    T, dt = p.shape[0], p.dtype
    qr = p[:, :H * (D + R)].view(T, H, D + R)[:, :, D:].float()
    q = torch.cat([q_abs.transpose(0, 1).float(), _rotate_pairs(qr, meta.positions, inv_freq)], dim=-1).to(dt)
    if cache is not None:
        dkv = p[:, H * (D + R):H * (D + R) + C + R].float()
        row = torch.cat([_rms(dkv[:, :C], eps) * norm_w.float(), _rotate_pairs(dkv[:, C:], meta.positions, inv_freq)], dim=-1)
        page, off = meta.slots.long() // meta.page_size, meta.slots.long() % meta.page_size
        cache[page, 0, off, :] = row.to(cache.dtype)
    return q.contiguous()


def _latent_attention(self, q, cache, meta, H, C, R, scale):
    T = q.shape[0]
    out = torch.zeros(H, T, C, dtype=q.dtype, device=q.device)
    q_start, pos0, kv_len = meta.seg_q_start.tolist(), meta.seg_pos0.tolist(), meta.seg_kv_len.tolist()
    rows = meta.table_rows.tolist()
    ps = meta.page_size
    for s in range(len(pos0)):
        a, b, L = q_start[s], q_start[s + 1], kv_len[s]
        j = torch.arange(L, device=q.device)
        kv = cache[meta.block_table[rows[s], j // ps].long(), 0, j % ps, :].float()         # [L, C + R]
        pq = pos0[s] + torch.arange(b - a, device=q.device)
        sc = torch.einsum("phd,jd->hpj", q[a:b].float(), kv) * scale
        sc = sc.masked_fill(~(j[None, :] <= pq[:, None])[None], float("-inf"))
        out[:, a:b] = torch.einsum("hpj,jc->hpc", torch.softmax(sc, dim=-1), kv[:, :C]).to(q.dtype)
    return out


def _head_gate(self, o, gate, out_dtype):
    H, T, V = o.shape
    return (o.float() * torch.sigmoid(gate.float()).T[:, :, None]).transpose(0, 1).reshape(T, H * V).to(out_dtype)


# ---------------------------------------------------------------- output norms, block-local sink attention, retention, routed experts
def _embed_stream(self, ids, table, rows_dtype):
    x = table[ids.long()].float()
    return x, (x if rows_dtype == torch.float32 else x.to(rows_dtype))


def _cast_rows(self, x, dtype):
    return x.to(dtype)


def _out_rmsnorm_add(self, x, y, weight, scale, mult, eps, rows_dtype):
    n = _rms(y.float(), eps) * weight.float()
    if scale is not None:
        n = n * scale.float()
    x.add_(mult * n)
    return x if rows_dtype == torch.float32 else x.to(rows_dtype)


def _stream_rmsnorm(self, x, delta, weight, eps, rows, out_dtype):
    if rows is None:
        if delta is not None:
            x.add_(delta.float())
        src = x
    else:
        src = x[rows.long()]
        if delta is not None:
            src = src + delta[rows.long()].float()
    return (_rms(src, eps) * weight.float()).to(out_dtype)


def _unit_qk_cache(self, p, H, KV, D, V, eps, lam, source, meta, k_cache, v_cache):
    T, dt = p.shape[0], p.dtype
    q = p[:, :H * D].float().view(T, H, D)
    k = p[:, H * D:(H + KV) * D].float().view(T, KV, D)
    v = p[:, (H + KV) * D:].float().view(T, KV, V)
    if eps is not None:
        q, k = _rms(q, eps), _rms(k, eps)
    if source is not None:
        v = (1.0 - lam.float()) * v + lam.float() * source.float().view(T, KV, V)
    if eps is not None:
        p[:, :H * D] = q.reshape(T, H * D).to(dt)
    if k_cache is not None:
        page, off = meta.slots.long() // meta.page_size, meta.slots.long() % meta.page_size
        k_cache[page, :, off, :] = k.to(dt)
        v_cache[page, :, off, :] = v.to(dt)
    return p[:, :H * D]


def _masked_attention(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink):
    T = q.shape[0]
    out = torch.empty((T, H * V), dtype=q.dtype, device=q.device)
    q_start, pos0, kv_len = meta.seg_q_start.tolist(), meta.seg_pos0.tolist(), meta.seg_kv_len.tolist()
    ps = meta.page_size
    rows = getattr(meta, "table_rows", None)
    rows = list(range(len(pos0))) if rows is None else rows.tolist()
    for s in range(len(pos0)):
        a, b, L = q_start[s], q_start[s + 1], kv_len[s]
        j = torch.arange(L, device=q.device)
        pages = meta.block_table[rows[s], j // ps].long()
        k = k_cache[pages, :, j % ps, :].float().repeat_interleave(H // KV, dim=1)        # [L, H, D]
        v = v_cache[pages, :, j % ps, :].float().repeat_interleave(H // KV, dim=1)        # [L, H, V]
        p = pos0[s] + torch.arange(b - a, device=q.device)
        visible = j[None, :] <= p[:, None]
        if window is not None:
            visible &= j[None, :] > p[:, None] - window
        if block_size is not None:
            visible &= (j[None, :] // block_size) == (p[:, None] // block_size)
        sc = torch.einsum("phd,jhd->hpj", q[a:b].reshape(b - a, H, D).float(), k) * scale
        sc = sc.masked_fill(~visible[None], float("-inf"))
        m = sc.max(-1, keepdim=True).values
        if sink:
            m = m.clamp_min(0.0)
        e = torch.exp(sc - m)
        den = e.sum(-1, keepdim=True) + (torch.exp(-m) if sink else 0.0)
        out[a:b] = torch.einsum("hpj,jhd->phd", e / den, v).reshape(b - a, H * V).to(q.dtype)
    return out


def _retention_scan(self, p, H, D, V, inv_freq, k_scale, decay, state, batch):
    T = p.shape[0]
    q = p[:, :H * D].float().view(T, H, D).clone()
    k = p[:, H * D:2 * H * D].float().view(T, H, D).clone()
    v = p[:, 2 * H * D:2 * H * D + H * V].float().view(T, H, V)
    if inv_freq is not None:
        half = inv_freq.numel()
        ang = batch.positions.float()[:, None] * inv_freq.float()[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        for t in (q, k):
            a, b = t[..., :half].clone(), t[..., half:2 * half].clone()
            t[..., :half] = a * cos - b * sin
            t[..., half:2 * half] = b * cos + a * sin
    k = k * k_scale
    o = torch.zeros(T, H * V, dtype=torch.float32, device=p.device)
    for a, b, slot in _segments(batch):
        S = state[slot].view(H, D, V).clone()
        for t in range(a, b):
            S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, q[t]).reshape(-1)
        state[slot] = S.reshape(-1)
    return o


def _route_topk(self, h, router, correction, top, groups):
    s = torch.softmax(h.float() @ router.float().T, dim=-1)
    choice = s + correction.float()
    if groups:
        count, keep = groups
        best = choice.view(choice.shape[0], count, -1).max(-1).values
        kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, best.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept.repeat_interleave(choice.shape[1] // count, dim=1), float("-inf"))
    idx = choice.topk(top, dim=-1).indices
    return idx.to(torch.int32), s.gather(1, idx)


def _clamped_glu(self, gu, limit, slope):
    g, u = gu.float().chunk(2, dim=-1)
    g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    return (g * torch.sigmoid(slope * g) * (u + 1.0)).to(gu.dtype)


def _expert_ffn(self, h, chosen, weights, w_in, w_out, limit, slope, shared):
    T, top = chosen.shape
    acc = torch.zeros(T, w_out.shape[1], dtype=torch.float32, device=h.device)
    for j in range(top):                                   # in the order of choice
        y = torch.empty(T, w_out.shape[1], dtype=h.dtype, device=h.device)
        for e in chosen[:, j].unique().tolist():
            rows = (chosen[:, j] == e).nonzero().flatten()
            a = _clamped_glu(self, self.linear(h[rows], w_in[e]), limit, slope)
            y[rows] = self.linear(a, w_out[e])
        acc += weights[:, j:j + 1].float() * y.float()
    if shared is not None:
        acc += shared.float()
    return acc.to(h.dtype)


# ---------------------------------------------------------------- hashed pair embedding, filters, gated additions, three more recurrences
def _embed_bigram_stream(self, ids, table, pairs, buckets, mul_prev, mul_cur, state, batch):
    ids_l, pos = ids.long(), batch.positions.long()
    prev = torch.roll(ids_l, 1)
    for a, b, slot in _segments(batch):
        prev[a] = state[slot, 0].long()
        state[slot, 0] = ids[b - 1]
    row = (prev * mul_prev + ids_l * mul_cur) % buckets
    row = torch.where(pos == 0, torch.full_like(row, buckets), row)
    return table[ids_l].float() + pairs[row].float()


_plain_stream_rmsnorm = _stream_rmsnorm


def _stream_rmsnorm_gated(self, x, delta, weight, eps, rows, out_dtype):
    from mini_inference_b200.parts.base import GatedDelta
    if isinstance(delta, GatedDelta):
        y = delta.y.float() if delta.y_bias is None else delta.y.float() + delta.y_bias.float()
        delta = torch.sigmoid(delta.logits.float() + delta.bias.float()) * y
    return _plain_stream_rmsnorm(self, x, delta, weight, eps, rows, out_dtype)


def _short_conv(self, h, weight, bias, taps, state, offset, batch, residual=False, act="none"):
    T, C = h.shape
    out = torch.empty(T, C, dtype=torch.float32, device=h.device)
    x = h.float()
    for a, b, slot in _segments(batch):
        hist = state[slot, offset:offset + (taps - 1) * C].view(taps - 1, C) if taps > 1 else x[:0]
        ext = torch.cat([hist, x[a:b]], dim=0)
        y = torch.zeros(b - a, C, device=h.device)
        for j in range(taps):
            y += weight[:, j].float() * ext[j:j + b - a]
        if bias is not None:
            y = y + bias.float()
        if act == "silu":
            y = torch.nn.functional.silu(y)
        out[a:b] = y + x[a:b] if residual else y
        if taps > 1:
            state[slot, offset:offset + (taps - 1) * C] = ext[ext.shape[0] - (taps - 1):].reshape(-1)
    return out.to(h.dtype)


def _general_delta_prepare(self, p, w2, w0, a_b, H, D, V, rank, decay_scale, unit_eps):
    T, HD = p.shape[0], H * D
    f = p.float()
    r, k, v = f[:, :HD], f[:, HD:2 * HD], f[:, 2 * HD:2 * HD + H * V]
    a = torch.sigmoid(f[:, 2 * HD + H * V:3 * HD + H * V] + a_b.float())
    low = torch.tanh(f[:, 3 * HD + 2 * H * V:3 * HD + 2 * H * V + rank])
    d = torch.exp(-decay_scale * torch.sigmoid(low @ w2.float().T + w0.float()))
    kh = k.view(T, H, D)
    u = (kh / torch.sqrt(kh.pow(2).sum(-1, keepdim=True) + unit_eps)).reshape(T, HD)
    return torch.cat([r, k, u, a * u, d, v], dim=1).contiguous()                   # r | k | u | a u | decay | v


def _general_delta_scan(self, prep, H, D, V, state, batch):
    T, HD = prep.shape[0], H * D
    r, k, u, au, d = (prep[:, i * HD:(i + 1) * HD].view(T, H, D) for i in range(5))
    v = prep[:, 5 * HD:5 * HD + H * V].view(T, H, V)
    o = torch.zeros(T, H * V, dtype=torch.float32, device=prep.device)
    for a, b, slot in _segments(batch):
        S = state[slot, :HD * V].view(H, D, V).clone()
        for t in range(a, b):
            seen = torch.einsum("hd,hdv->hv", u[t], S)
            S = d[t][:, :, None] * S - au[t][:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hdv,hd->hv", S, r[t]).reshape(-1)
        state[slot, :HD * V] = S.reshape(-1)
    return o


def _matrix_memory(self, p, gl, gate_bias, H, D, V, cap, den_eps, norm, gate, eps, state, batch, out_dtype):
    T, HD, W = p.shape[0], H * D, V + 4
    f = p.float()
    q = f[:, :HD].view(T, H, D) * D ** -0.5
    k = f[:, HD:2 * HD].view(T, H, D)
    v = f[:, 2 * HD:2 * HD + H * V].view(T, H, V)
    z = gl.float() + gate_bias.float()
    if cap is not None:
        z = cap * torch.tanh(z / cap)
    ig, fg = z[:, :H], torch.nn.functional.logsigmoid(z[:, H:])
    o = torch.zeros(T, H, V, dtype=torch.float32, device=p.device)
    for a, b, slot in _segments(batch):
        S = state[slot, :HD * W].view(H, D, W).clone()                 # columns 0..V-1 the memory, column V the normaliser
        m = state[slot, HD * W:HD * W + H].clone()
        for t in range(a, b):
            new = torch.maximum(fg[t] + m, ig[t])
            keep, take = torch.exp(fg[t] + m - new), torch.exp(ig[t] - new)
            vv = torch.cat([v[t], torch.ones(H, 1), torch.zeros(H, 3)], dim=1)
            S = keep[:, None, None] * S + (take[:, None] * k[t])[:, :, None] * vv[:, None, :]
            m = new
            full = torch.einsum("hdw,hd->hw", S, q[t])
            den = torch.maximum(full[:, V].abs(), torch.exp(-m)) + den_eps
            o[t] = full[:, :V] / den[:, None]
        state[slot, :HD * W] = S.reshape(-1)
        state[slot, HD * W:HD * W + H] = m
    y = _rms(o, eps).reshape(T, H * V) * norm.float() * torch.sigmoid(gate.float())
    return y.to(out_dtype)


def _selective_scan(self, x, dt, dt_b, A, B, C, Dv, z, state, batch, out_dtype):
    T, I = x.shape
    N = A.shape[1]
    xf, zf, Bf, Cf = x.float(), z.float(), B.float(), C.float()
    step = torch.nn.functional.softplus(dt.float() + dt_b.float())
    y = torch.zeros(T, I, dtype=torch.float32, device=x.device)
    for a, b, slot in _segments(batch):
        S = state[slot, :I * N].view(I, N).clone()
        for t in range(a, b):
            S = torch.exp(step[t][:, None] * A) * S + (step[t] * xf[t])[:, None] * Bf[t][None, :]
            y[t] = S @ Cf[t] + Dv.float() * xf[t]
        state[slot, :I * N] = S.reshape(-1)
    return (y * torch.nn.functional.silu(zf)).to(out_dtype)


_plain_masked_attention = _masked_attention


def _masked_attention_biased(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink, sink_values=None,
                             distance_bias=None, distance_bias_by_head=None):
    if sink_values is None and distance_bias is None:
        return _plain_masked_attention(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink)
    T = q.shape[0]
    out = torch.empty((T, H * V), dtype=q.dtype, device=q.device)
    q_start, pos0, kv_len = meta.seg_q_start.tolist(), meta.seg_pos0.tolist(), meta.seg_kv_len.tolist()
    ps = meta.page_size
    rows = getattr(meta, "table_rows", None)
    rows = list(range(len(pos0))) if rows is None else rows.tolist()
    for s in range(len(pos0)):
        a, b, L = q_start[s], q_start[s + 1], kv_len[s]
        j = torch.arange(L, device=q.device)
        pages = meta.block_table[rows[s], j // ps].long()
        k = k_cache[pages, :, j % ps, :].float().repeat_interleave(H // KV, dim=1)
        v = v_cache[pages, :, j % ps, :].float().repeat_interleave(H // KV, dim=1)
        p = pos0[s] + torch.arange(b - a, device=q.device)
        dist = p[:, None] - j[None, :]
        visible = dist >= 0
        if window is not None:
            visible &= dist < window
        if block_size is not None:
            visible &= (j[None, :] // block_size) == (p[:, None] // block_size)
        sc = torch.einsum("phd,jhd->hpj", q[a:b].reshape(b - a, H, D).float(), k) * scale
        if distance_bias is not None:
            sc = sc + distance_bias[dist.clamp(0, distance_bias.shape[0] - 1)].permute(2, 0, 1)
        sc = sc.masked_fill(~visible[None], float("-inf"))
        m = sc.max(-1, keepdim=True).values
        extra = 0.0
        if sink:
            sv = sink_values.float().view(H, 1, 1) if sink_values is not None else torch.zeros(H, 1, 1)
            m = torch.maximum(m, sv)
            extra = torch.exp(sv - m)
        e = torch.exp(sc - m)
        out[a:b] = torch.einsum("hpj,jhd->phd", e / (e.sum(-1, keepdim=True) + extra), v).reshape(b - a, H * V).to(q.dtype)
    return out


def _dual_rmsnorm_mix(self, a, wa, sa, b, wb, sb, eps):
    return (sa * _rms(a.float(), eps) * wa.float() + sb * _rms(b.float(), eps) * wb.float()).to(a.dtype)


_plain_route_topk = _route_topk


def _route_topk_scored(self, h, router, correction, top, groups, score="softmax", extra_rows=0):
    if score == "softmax" and not extra_rows:
        return _plain_route_topk(self, h, router, correction, top, groups)
    E = router.shape[0] - extra_rows
    logits = h.float() @ router.float().T
    extra = logits[:, E:].contiguous() if extra_rows else None
    s = torch.sigmoid(logits[:, :E]) if score == "sigmoid" else torch.softmax(logits[:, :E], dim=-1)
    choice = s if correction is None else s + correction.float()
    assert not groups
    idx = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    return idx.to(torch.int32), s.gather(1, idx), extra


_plain_expert_ffn = _expert_ffn


def _expert_ffn_general(self, h, chosen, weights, w_in, w_out, limit, slope, shared, up_shift=1.0, weight_on_input=False, shared_gate=None):
    if up_shift == 1.0 and not weight_on_input and shared_gate is None:
        return _plain_expert_ffn(self, h, chosen, weights, w_in, w_out, limit, slope, shared)
    T, top = chosen.shape
    acc = torch.zeros(T, w_out.shape[1], dtype=torch.float32, device=h.device)
    for j in range(top):
        for e in chosen[:, j].unique().tolist():
            rows = (chosen[:, j] == e).nonzero().flatten()
            w = weights[rows, j:j + 1].float()
            g, u = (h[rows].float() @ w_in[e].float().T).chunk(2, dim=-1)
            if weight_on_input:
                g, u = g * w, u * w
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
            act = (g * torch.sigmoid(slope * g) * (u + up_shift)).to(h.dtype)
            y = self.linear(act, w_out[e]).float()
            acc[rows] += y if weight_on_input else w * y
    if shared is not None:
        acc += shared.float() if shared_gate is None else torch.sigmoid(shared_gate.float()) * shared.float()
    return acc.to(h.dtype)


def _bias_act(self, z, bias, act):
    y = z.float() + bias.float()
    if act == "relu2":
        y = torch.relu(y).pow(2)
    return y.to(z.dtype)


def _softcap(self, logits, cap):
    return cap * torch.tanh(logits / cap)



# ---------------------------------------------------------------- scaled embedding with positions, pair additions, row norms, gated bias activation,
# normed q/k with a temperature and keys as values, distance slopes, group-limited sigmoid routing with renormalised weights
def _embed_scaled_stream(self, ids, table, scale, pos_table, positions):
    x = table[ids.long()].float() * scale
    return x if pos_table is None else x + pos_table[positions.long()].float()


def _stream_rmsnorm_pair(self, x, a, b, bias, pre_add, weight, eps, rows, out_dtype):
    add = torch.zeros_like(x)
    for part in (a, b):
        if part is not None:
            add = add + part.float()
    if bias is not None:
        add = add + bias.float()
    if pre_add is not None:
        add = add + pre_add.float()
    if rows is None:
        x.add_(add)
        src = x
    else:
        src = x[rows.long()] + add[rows.long()]
    return (_rms(src, eps) * weight.float()).to(out_dtype)


def _rows_rmsnorm(self, x, weight, eps):
    return (_rms(x.float(), eps) * weight.float()).to(x.dtype).contiguous()


def _bias_glu(self, gu, bias, act):
    y = gu.float() if bias is None else gu.float() + bias.float()
    g, u = y.chunk(2, dim=-1)
    f = {"relu": torch.relu, "silu": torch.nn.functional.silu, "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}[act]
    return (f(g) * u).to(gu.dtype)


def _scale_logits(self, logits, s):
    return logits * s


_latent_prepare_plain = _latent_prepare


def _latent_prepare_general(self, p, q_abs, H, D, R, C, norm_w, eps, inv_freq, meta, cache, q_rows=None, dkv_col=None):
    if q_rows is None and dkv_col is None and R:
        return _latent_prepare_plain(self, p, q_abs, H, D, R, C, norm_w, eps, inv_freq, meta, cache)
    T, dt = p.shape[0], p.dtype
    src = p if q_rows is None else q_rows
    col = H * (D + R) if dkv_col is None else dkv_col
    parts = [q_abs.transpose(0, 1).float()]
    if R:
        parts.append(_rotate_pairs(src[:, :H * (D + R)].view(T, H, D + R)[:, :, D:].float(), meta.positions, inv_freq))
    q = torch.cat(parts, dim=-1).to(dt)
    if cache is not None:
        dkv = p[:, col:col + C + R].float()
        row = _rms(dkv[:, :C], eps) * norm_w.float()
        if R:
            row = torch.cat([row, _rotate_pairs(dkv[:, C:], meta.positions, inv_freq)], dim=-1)
        page, off = meta.slots.long() // meta.page_size, meta.slots.long() % meta.page_size
        cache[page, 0, off, :] = row.to(cache.dtype)
    return q.contiguous()


_head_gate_plain = _head_gate


def _head_gate_optional(self, o, gate, out_dtype):
    if gate is not None:
        return _head_gate_plain(self, o, gate, out_dtype)
    H, T, V = o.shape
    return o.transpose(0, 1).reshape(T, H * V).to(out_dtype)


_unit_qk_cache_plain = _unit_qk_cache


def _unit_qk_cache_general(self, p, H, KV, D, V, eps, lam, source, meta, k_cache, v_cache, q_weight=None, k_weight=None, q_temp=None,
                           values_are_keys=False):
    if q_weight is None and q_temp is None and not values_are_keys:
        return _unit_qk_cache_plain(self, p, H, KV, D, V, eps, lam, source, meta, k_cache, v_cache)
    T, dt = p.shape[0], p.dtype
    q = p[:, :H * D].float().view(T, H, D)
    k_raw = p[:, H * D:(H + KV) * D].float().view(T, KV, D)
    v = k_raw if values_are_keys else p[:, (H + KV) * D:].float().view(T, KV, V)
    k = k_raw
    if eps is not None:
        q, k = _rms(q, eps), _rms(k_raw, eps)
    if q_weight is not None:
        q, k = q * q_weight.float(), k * k_weight.float()
    if q_temp is not None:
        coef, every = q_temp
        pos = meta.positions.long()
        q = q * (1.0 + coef * torch.log(((pos + 1) // every + 1).float()))[:, None, None]
    p[:, :H * D] = q.reshape(T, H * D).to(dt)
    if k_cache is not None:
        page, off = meta.slots.long() // meta.page_size, meta.slots.long() % meta.page_size
        k_cache[page, :, off, :] = k.to(dt)
        v_cache[page, :, off, :] = v.to(dt)
    return p[:, :H * D]


_masked_attention_tables = _masked_attention_biased


def _masked_attention_sloped(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink, sink_values=None,
                             distance_bias=None, distance_bias_by_head=None, distance_slopes=None):
    if distance_slopes is None:
        return _masked_attention_tables(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink, sink_values,
                                        distance_bias, distance_bias_by_head)
    far = int(max(meta.seg_kv_len.tolist()))                       # the slopes as a table of every distance that occurs
    table = -torch.arange(far + 1, dtype=torch.float32)[:, None] * distance_slopes.float()[None, :]
    if distance_bias is not None:
        table = table + distance_bias[torch.arange(far + 1).clamp(max=distance_bias.shape[0] - 1)]
    return _masked_attention_tables(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink, sink_values, table, None)


_route_topk_simple = _route_topk_scored


def _route_topk_grouped(self, h, router, correction, top, groups, score="softmax", extra_rows=0, group_score="max", renormalise=False,
                        weight_eps=0.0, route_scale=1.0, explicit=False):
    if group_score == "max" and not renormalise and route_scale == 1.0 and not explicit:
        if score == "softmax" and not extra_rows:
            return _plain_route_topk(self, h, router, correction, top, groups)
        return _route_topk_simple(self, h, router, correction, top, groups, score, extra_rows)
    E = router.shape[0] - extra_rows
    logits = h.float() @ router.float().T
    extra = logits[:, E:].contiguous() if extra_rows else None
    s = torch.sigmoid(logits[:, :E]) if score == "sigmoid" else torch.softmax(logits[:, :E], dim=-1)
    choice = s if correction is None else s + correction.float()
    if groups:
        count, keep = groups
        per = E // count
        grouped = choice.view(-1, count, per)
        rank = grouped.max(-1).values if group_score == "max" else grouped.topk(min(2, per), dim=-1).values.sum(-1)
        best = torch.sort(rank, dim=-1, descending=True, stable=True).indices[:, :keep]
        allowed = torch.zeros_like(rank, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, dim=1)
        choice = choice.masked_fill(~allowed, float("-inf"))
    idx = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
    w = s.gather(1, idx)
    if renormalise:
        w = w / (w.sum(-1, keepdim=True) + weight_eps)
    return idx.to(torch.int32), w * route_scale, extra


def _route_topk_any(self, h, router, correction, top, groups, score=None, extra_rows=0, **options):
    if score is None and not options:
        return _plain_route_topk(self, h, router, correction, top, groups)
    return _route_topk_grouped(self, h, router, correction, top, groups, score or "softmax", extra_rows, explicit=True, **options)


_stream_rmsnorm, _masked_attention, _route_topk, _expert_ffn = _stream_rmsnorm_gated, _masked_attention_biased, _route_topk_scored, _expert_ffn_general
_latent_prepare, _head_gate, _unit_qk_cache, _masked_attention, _route_topk = _latent_prepare_general, _head_gate_optional, _unit_qk_cache_general, _masked_attention_sloped, _route_topk_any


for _name, _fn in list(globals().items()):
    if _name.startswith("_") and _name[1:] in ("embed_scaled_norm", "add_scaled_rmsnorm", "polynorm", "lightning_scan", "group_rmsnorm_gate",
                                               "delta_prepare", "delta_scan", "batched_linear", "latent_prepare", "latent_attention", "head_gate",
                                               "embed_stream", "cast_rows", "out_rmsnorm_add", "stream_rmsnorm", "unit_qk_cache", "masked_attention",
                                               "retention_scan", "route_topk", "clamped_glu", "expert_ffn",
                                               "embed_bigram_stream", "short_conv", "general_delta_prepare", "general_delta_scan", "matrix_memory",
                                               "selective_scan", "dual_rmsnorm_mix", "bias_act", "softcap",
                                               "embed_scaled_stream", "stream_rmsnorm_pair", "rows_rmsnorm", "bias_glu", "scale_logits"):
        setattr(TorchRefOps, _name[1:], _fn)
