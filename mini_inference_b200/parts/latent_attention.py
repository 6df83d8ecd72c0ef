"""Latent attention: keys and values are up-projections of ONE compressed vector per token,
so only that vector (and a small rotated key part shared by all heads) is cached.

Per token:  q = W_q h, per head [nope_dim unrotated | rot_dim rotated];
            W_dkv h = [kv_rank | rot_dim]: c = rmsnorm(first part) * weight (the latent), kr = rotate(last part);
            head h: key = [W_uk_h c | kr], value = W_uv_h c; score = (q . key) * scale; causal softmax;
            the head's output is multiplied by sigmoid(W_g h)_h, then W_o on the concatenated heads.
The cache holds one row [c | kr] per token in pages of a one-plane pool.  The up-projections are
absorbed into the query and the output:  q_u . (W_uk_h c) = (W_uk_h^T q_u) . c  and
sum_j p_j W_uv_h c_j = W_uv_h (sum_j p_j c_j),  so attention runs as H query heads of size
kv_rank + rot_dim over ONE shared key row per token whose first kv_rank entries are also the value,
for prompt portions and decoded tokens alike; neither keys nor values of a head are ever materialised.

Options: rot_dim=0 (no rotated part: the cached row is the latent alone and positions do not enter); gate=False (no
per-head output gate, no tensor `g`); q_rank=n (the queries pass a latent of their own: c_q = rmsnorm(W_dq h) * w with the
tensor `dq.norm`, q = W_uq c_q; tensors `dq`, `dq.norm`, `uq` instead of `q`).
"""
from __future__ import annotations

import torch

from .attention import paged_attention_step_arrays
from .base import KVCacheNeed, Part, WeightSpec, register_mixer


@register_mixer("latent_attention")
class LatentAttention(Part):
    offers_open = True
    step_arrays_key = "paged_attention"

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H = int(g("hidden_size")), int(g("num_heads"))
        self.D, self.R, self.V, self.C = int(g("nope_dim")), int(g("rot_dim")), int(g("value_dim")), int(g("kv_rank"))
        self.scale, self.eps = float(g("scale")), float(g("latent_norm_eps"))
        self.gate = bool(g("gate", True))
        self.q_rank = int(g("q_rank")) if g("q_rank") else None
        self.proj = self.uk_t = self.uv = self.o = self.latent_norm = self.uq = self.q_norm = None

    def weight_specs(self):
        H, D, R, V, C, hid = self.H, self.D, self.R, self.V, self.C, self.hidden
        if self.q_rank:
            specs = [WeightSpec("dq", (self.q_rank, hid)), WeightSpec("dq.norm", (self.q_rank,), kind="vector", init="norm"),
                     WeightSpec("uq", (H * (D + R), self.q_rank))]
        else:
            specs = [WeightSpec("q", (H * (D + R), hid))]
        specs += [WeightSpec("dkv", (C + R, hid)), WeightSpec("dkv.norm", (C,), kind="vector", init="norm"),
                  WeightSpec("uk", (H * D, C)), WeightSpec("uv", (H * V, C))]
        if self.gate:
            specs.append(WeightSpec("g", (H, hid)))
        return specs + [WeightSpec("o", (hid, H * V))]

    def cache_need(self):
        return KVCacheNeed(1, self.C + self.R, None, planes=1)

    def load(self, tensors, dtype, device):
        H, D, V, C = self.H, self.D, self.V, self.C
        first = [tensors.pop("dq")] if self.q_rank else [tensors.pop("q")]                                     # q (or its latent) | c, kr | gate
        self.proj = torch.cat(first + [tensors.pop("dkv")] + ([tensors.pop("g")] if self.gate else []), dim=0).contiguous()
        if self.q_rank:
            self.uq, self.q_norm = tensors.pop("uq"), tensors.pop("dq.norm").float().contiguous()
        self.uk_t = tensors.pop("uk").view(H, D, C).transpose(1, 2).contiguous()       # [H, C, D]: q_abs_h = uk_t_h q_u
        self.uv = tensors.pop("uv").view(H, V, C).contiguous()                         # [H, V, C]: o_h = uv_h o_lat_h
        self.latent_norm = tensors.pop("dkv.norm").float().contiguous()
        self.o = tensors.pop("o")

    step_arrays = staticmethod(paged_attention_step_arrays)

    @property
    def open_weight(self):
        return self.o

    @property
    def first_weight(self):
        return self.proj

    def step_flops(self, rows, pairs):
        H, D, R, V, C = self.H, self.D, self.R, self.V, self.C
        return 2 * H * (2 * C + R) * pairs + 2 * rows * H * C * (D + V)      # scores and weighted sums in the latent space; the two absorbed projections

    def forward(self, h, ctx, cache, position, owns_cache=True):
        rows, w = self.forward_open(h, ctx, cache, position, owns_cache)
        return ctx.ops.linear(rows, w)

    def forward_open(self, h, ctx, cache, position, owns_cache=True):
        ops, H, D, R, V, C = ctx.ops, self.H, self.D, self.R, self.V, self.C
        meta = ctx.batch.group_view(cache.group, self.step_arrays_key)
        p = ops.linear(h, self.proj)                                               # [T, H (D + R) + C + R + H]
        if self.q_rank:                                                            # p = c_q as projected | c, kr | gate
            qp = ops.linear(ops.rows_rmsnorm(p[:, :self.q_rank], self.q_norm, self.eps), self.uq)
            q_abs = ops.batched_linear(qp, 0, D + R, D, self.uk_t)
            q = ops.latent_prepare(p, q_abs, H, D, R, C, self.latent_norm, self.eps, position.rotary_inv_freq(), meta,
                                   cache.k if owns_cache else None, q_rows=qp, dkv_col=self.q_rank)
            gate_col = self.q_rank + C + R
        else:
            q_abs = ops.batched_linear(p, 0, D + R, D, self.uk_t)                  # [H, T, C]
            q = ops.latent_prepare(p, q_abs, H, D, R, C, self.latent_norm, self.eps, position.rotary_inv_freq(), meta,
                                   cache.k if owns_cache else None)                # [T, H, C + R]; [c | kr] -> the pages
            gate_col = H * (D + R) + C + R
        o_lat = ops.latent_attention(q, cache.k, meta, H, C, R, self.scale)        # [H, T, C]
        if not self.gate:                                                          # no gate: the products write the heads side by side
            return ops.batched_linear(o_lat, None, None, C, self.uv, side_by_side=True), self.o
        o = ops.batched_linear(o_lat, None, None, C, self.uv)                      # [H, T, V]
        rows = ops.head_gate(o, p[:, gate_col:], ctx.dtype)                        # [T, H V]
        return rows, self.o
