"""Mixers that keep a fixed-size matrix state per request instead of keys and values.

Both keep, per head, a float32 state S [key_dim, value_dim] in the request's state slot and
walk the tokens of a step's entry in order from the state that earlier steps left; prompt
portions and single decoded tokens go through the same kernels.  The columns of S never mix
(every update is "row factors times S plus key times a row vector"), so a kernel gives every
column to a few lanes that hold its rows in registers.

lightning       q, k, v = silu(W h);  S <- decay_h S + k v^T;  o = S^T q
                rows: rmsnorm over all heads' outputs together * weight, * sigmoid(W_g h)
channel_delta   q, k, v = silu(causal_conv(W h)); q, k unit vectors per head (q also * key_dim^-1/2);
                beta = sigmoid(W_b h); per head and key channel g = exp(-exp(A_log) softplus(W_a2 W_a1 h + dt_bias));
                S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                rows: per head o / rms(o) * weight [value_dim], * sigmoid(W_g2 W_g1 h)
                The last conv_taps - 1 projected inputs are part of the state (behind S in the slot).
"""
from __future__ import annotations

import torch

from .base import Part, StateNeed, WeightSpec, register_mixer


@register_mixer("lightning")
class LightningAttention(Part):
    offers_open = True

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.D, self.V = int(g("hidden_size")), int(g("num_heads")), int(g("key_dim")), int(g("value_dim"))
        self.decay_values = tuple(float(v) for v in g("decay"))
        self.eps = float(g("out_norm_eps"))
        if len(self.decay_values) != self.H:
            raise ValueError(f"{len(self.decay_values)} decay constants for {self.H} heads")
        self.proj = self.o = self.norm = self.decay = None

    def weight_specs(self):
        H, D, V, hid = self.H, self.D, self.V, self.hidden
        return [WeightSpec("q", (H * D, hid)), WeightSpec("k", (H * D, hid)), WeightSpec("v", (H * V, hid)),
                WeightSpec("g", (H * V, hid)), WeightSpec("o", (hid, H * V)),
                WeightSpec("norm", (H * V,), kind="vector", init="norm")]

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V,), "float32")

    def load(self, tensors, dtype, device):
        self.proj = torch.cat([tensors.pop(n) for n in ("q", "k", "v", "g")], dim=0).contiguous()     # one product for all four
        self.o = tensors.pop("o")
        self.norm = tensors.pop("norm").float().contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    @property
    def open_weight(self):
        return self.o

    @property
    def first_weight(self):
        return self.proj

    def step_flops(self, rows, pairs):
        return 4 * self.H * self.D * self.V * rows                 # state update and read-out, a multiply and an add each

    def forward(self, h, ctx, cache, position, owns_cache=True):
        rows, w = self.forward_open(h, ctx, cache, position, owns_cache)
        return ctx.ops.linear(rows, w)

    def forward_open(self, h, ctx, cache, position, owns_cache=True):
        ops, H, D, V = ctx.ops, self.H, self.D, self.V
        p = ops.linear(h, self.proj)                                # [T, 2 H D + 2 H V]: q | k | v | gate
        o = ops.lightning_scan(p, H, D, V, self.decay, cache.state, ctx.batch)          # float32 [T, H V]
        rows = ops.group_rmsnorm_gate(o, self.norm, p[:, 2 * H * D + H * V:], self.eps, 1, H * V, ctx.dtype)
        return rows, self.o


@register_mixer("channel_delta")
class ChannelDeltaRule(Part):
    offers_open = True

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.KV = int(g("hidden_size")), int(g("num_heads")), int(g("num_kv_heads"))
        self.D, self.V, self.taps = int(g("key_dim")), int(g("value_dim")), int(g("conv_taps"))
        self.eps, self.unit_eps = float(g("out_norm_eps")), float(g("unit_eps"))
        if self.H % self.KV:
            raise ValueError(f"{self.H} heads are not a multiple of {self.KV} key heads")
        # the low ranks of the decay and gate projections are the checkpoint's business (-1: any); a configuration
        # that is to be filled with random weights names them
        self.a_rank, self.g_rank = int(g("decay_rank", -1)), int(g("gate_rank", -1))
        self.C = 2 * self.KV * self.D + self.H * self.V             # channels that pass the short convolution
        self.proj = self.ag2 = self.o = self.conv = self.A_log = self.dt_bias = self.norm = None

    def weight_specs(self):
        H, KV, D, V, hid, taps = self.H, self.KV, self.D, self.V, self.hidden, self.taps
        return [WeightSpec("q", (KV * D, hid)), WeightSpec("k", (KV * D, hid)), WeightSpec("v", (H * V, hid)),
                WeightSpec("q.conv", (KV * D, taps), kind="vector"), WeightSpec("k.conv", (KV * D, taps), kind="vector"),
                WeightSpec("v.conv", (H * V, taps), kind="vector"),
                WeightSpec("b", (H, hid)), WeightSpec("A_log", (H,), kind="vector", init="zeros"),
                WeightSpec("norm", (V,), kind="vector", init="norm"),
                WeightSpec("a1", (self.a_rank, hid)), WeightSpec("a2", (H * D, self.a_rank)),
                WeightSpec("dt_bias", (H * D,), kind="vector", init="zeros"),
                WeightSpec("g1", (self.g_rank, hid)), WeightSpec("g2", (H * V, self.g_rank)), WeightSpec("o", (hid, H * V))]

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V + (self.taps - 1) * self.C,), "float32")

    def load(self, tensors, dtype, device):
        a1, g1 = tensors.pop("a1"), tensors.pop("g1")
        a2, g2 = tensors.pop("a2"), tensors.pop("g2")
        self.a_rank, self.g_rank = a1.shape[0], g1.shape[0]
        if a2.shape[1] != self.a_rank or g2.shape[1] != self.g_rank:
            raise ValueError("the two halves of a low-rank projection disagree about its rank")
        # the second halves of both low-rank projections as ONE product: [a2 0; 0 g2] on the neighbouring columns a1 | g1
        # of the first product (the zero blocks add nothing to any sum)
        self.ag2 = torch.block_diag(a2, g2).contiguous()
        # one product for everything that reads the mixer's input: q | k | v | b | a1 | g1
        self.proj = torch.cat([tensors.pop("q"), tensors.pop("k"), tensors.pop("v"), tensors.pop("b"), a1, g1], dim=0).contiguous()
        self.conv = torch.cat([tensors.pop("q.conv"), tensors.pop("k.conv"), tensors.pop("v.conv")], dim=0).float().contiguous()
        self.A_log, self.dt_bias = tensors.pop("A_log").float().contiguous(), tensors.pop("dt_bias").float().contiguous()
        self.norm = tensors.pop("norm").float().contiguous()
        self.o = tensors.pop("o")

    @property
    def open_weight(self):
        return self.o

    @property
    def first_weight(self):
        return self.proj

    def step_flops(self, rows, pairs):
        return 8 * self.H * self.D * self.V * rows                 # decay, S^T k, rank-one update, read-out

    def forward(self, h, ctx, cache, position, owns_cache=True):
        rows, w = self.forward_open(h, ctx, cache, position, owns_cache)
        return ctx.ops.linear(rows, w)

    def forward_open(self, h, ctx, cache, position, owns_cache=True):
        ops, H, KV, D, V, C = ctx.ops, self.H, self.KV, self.D, self.V, self.C
        p = ops.linear(h, self.proj)
        ag = ops.linear(p[:, C + H:], self.ag2)                     # [T, H D + H V]: decay logits | gate logits
        a, gate = ag[:, :H * D], ag[:, H * D:]
        prep = ops.delta_prepare(p, a, self.conv, self.A_log, self.dt_bias, H, KV, D, V, self.taps, self.unit_eps,
                                 cache.state, ctx.batch)            # float32 q | k | v | beta | g per token; conv tail -> state
        o = ops.delta_scan(prep, H, KV, D, V, cache.state, ctx.batch)                   # float32 [T, H V]
        rows = ops.group_rmsnorm_gate(o, self.norm, gate, self.eps, H, V, ctx.dtype)
        return rows, self.o


@register_mixer("retention")
class Retention(Part):
    """q, k = rotate(W h) (the position part's rotate-half frequencies on the first coordinates of each head; none: no
    rotation), k also * key_dim^-1/2 after the rotation;  S <- decay_h S + k v^T;  o = S^T q;
    rows: per head o / rms(o) (no weight), * silu(W_g h).  What enters the recurrence is float32."""

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.D, self.V = int(g("hidden_size")), int(g("num_heads")), int(g("key_dim")), int(g("value_dim"))
        self.decay_values = tuple(float(v) for v in g("decay"))
        self.eps = float(g("out_norm_eps"))
        if len(self.decay_values) != self.H:
            raise ValueError(f"{len(self.decay_values)} decay constants for {self.H} heads")
        self.proj = self.o = self.decay = None

    def weight_specs(self):
        H, D, V, hid = self.H, self.D, self.V, self.hidden
        return [WeightSpec("q", (H * D, hid)), WeightSpec("k", (H * D, hid)), WeightSpec("v", (H * V, hid)),
                WeightSpec("g", (H * V, hid)), WeightSpec("o", (hid, H * V))]

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V,), "float32")

    def load(self, tensors, dtype, device):
        self.proj = torch.cat([tensors.pop(n) for n in ("q", "k", "v", "g")], dim=0).contiguous()     # one product for all four
        self.o = tensors.pop("o")
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=device)

    @property
    def first_weight(self):
        return self.proj

    def step_flops(self, rows, pairs):
        return 4 * self.H * self.D * self.V * rows

    def forward(self, h, ctx, cache, position, owns_cache=True):
        ops, H, D, V = ctx.ops, self.H, self.D, self.V
        p = ops.linear(h, self.proj)                                # [T, 2 H D + 2 H V]: q | k | v | gate
        o = ops.retention_scan(p, H, D, V, position.rotary_inv_freq(), float(D) ** -0.5, self.decay, cache.state, ctx.batch)
        rows = ops.group_rmsnorm_gate(o, None, p[:, 2 * H * D + H * V:], self.eps, H, V, ctx.dtype, act="silu")
        return ops.linear(rows, self.o)


@register_mixer("general_delta")
class GeneralDeltaRule(Part):
    """A delta rule whose decay and removal act per head and key channel, both reading the OLD state:
        d = exp(-decay_scale * sigmoid(W_w2 tanh(W_w1 h) + w0)),  a = sigmoid(W_a h + a_b),  u = k / sqrt(sum k^2 + unit_eps);
        S <- diag(d) S - (a * u) (u^T S) + k v^T;   o = S^T r.
    rows: per head o / rms(o), * weight [all heads], * sigmoid(W_g h).  Everything that enters the recurrence is made in float32 by
    one prologue kernel (the second half of the low-rank decay projection included); the state is float32 [H, key_dim, value_dim]."""

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.D = int(g("hidden_size")), int(g("num_heads")), int(g("key_dim"))
        self.V = int(g("value_dim", self.D))
        self.eps, self.unit_eps, self.decay_scale = float(g("out_norm_eps")), float(g("unit_eps")), float(g("decay_scale"))
        self.rank = int(g("decay_rank", -1))                         # the checkpoint's business; a configuration for random weights names it
        self.proj = self.w2 = self.w0 = self.a_b = self.norm = self.o = None

    def weight_specs(self):
        H, D, V, hid = self.H, self.D, self.V, self.hidden
        return [WeightSpec("r", (H * D, hid)), WeightSpec("k", (H * D, hid)), WeightSpec("v", (H * V, hid)),
                WeightSpec("g", (H * V, hid)), WeightSpec("a", (H * D, hid)), WeightSpec("a.b", (H * D,), kind="vector", init="zeros"),
                WeightSpec("w1", (self.rank, hid)), WeightSpec("w2", (H * D, self.rank)), WeightSpec("w0", (H * D,), kind="vector", init="zeros"),
                WeightSpec("norm", (H * V,), kind="vector", init="norm"), WeightSpec("o", (hid, H * V))]

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V,), "float32")

    def load(self, tensors, dtype, device):
        w1 = tensors.pop("w1")
        self.rank = w1.shape[0]
        self.w2 = tensors.pop("w2").contiguous()
        if self.w2.shape[1] != self.rank:
            raise ValueError("the two halves of the low-rank decay projection disagree about its rank")
        # one product for everything that reads the mixer's input: r | k | v | a | g | w1
        self.proj = torch.cat([tensors.pop("r"), tensors.pop("k"), tensors.pop("v"), tensors.pop("a"), tensors.pop("g"), w1], dim=0).contiguous()
        self.w0, self.a_b = tensors.pop("w0").float().contiguous(), tensors.pop("a.b").float().contiguous()
        self.norm = tensors.pop("norm").float().contiguous()
        self.o = tensors.pop("o")

    @property
    def first_weight(self):
        return self.proj

    def step_flops(self, rows, pairs):
        return 8 * self.H * self.D * self.V * rows                 # u^T S, decay, two rank-one updates, read-out

    def forward(self, h, ctx, cache, position, owns_cache=True):
        ops, H, D, V = ctx.ops, self.H, self.D, self.V
        p = ops.linear(h, self.proj)
        prep = ops.general_delta_prepare(p, self.w2, self.w0, self.a_b, H, D, V, self.rank, self.decay_scale, self.unit_eps)
        o = ops.general_delta_scan(prep, H, D, V, cache.state, ctx.batch)                  # float32 [T, H V]
        gate = p[:, 3 * H * D + H * V:3 * H * D + 2 * H * V]
        rows = ops.group_rmsnorm_gate(o, self.norm, gate, self.eps, H, V, ctx.dtype)
        return ops.linear(rows, self.o)


@register_mixer("matrix_memory")
class MatrixMemory(Part):
    """An exponentially gated matrix memory with a running maximum m that keeps the exponentials bounded:
        i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))   (one of each per head; cap None: no cap)
        m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n <- e^(f + m - m') n + e^(i - m') k;  m <- m'
        o = S^T q / (max(|n . q|, e^(-m)) + den_eps),  q = W_q h * key_dim^-1/2;
    rows: per head o / rms(o), * weight [all heads], * sigmoid(W_g h).  m starts at 0 with S and n.  The gates' products are made
    in float32; n rides in the scan as one more value column (a value that is always 1), so the state slot holds per head
    [key_dim, value_dim + 4] floats (the column of n and three unused ones keep 16-byte pieces), then the H running maxima."""

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.D, self.V = int(g("hidden_size")), int(g("num_heads")), int(g("key_dim")), int(g("value_dim"))
        self.cap = g("gate_cap")
        self.eps, self.den_eps = float(g("out_norm_eps")), float(g("den_eps"))
        self.proj = self.gates = self.gate_bias = self.norm = self.o = None

    def weight_specs(self):
        H, D, V, hid = self.H, self.D, self.V, self.hidden
        return [WeightSpec("q", (H * D, hid)), WeightSpec("k", (H * D, hid)), WeightSpec("v", (H * V, hid)), WeightSpec("g", (H * V, hid)),
                WeightSpec("i", (H, hid)), WeightSpec("i.b", (H,), kind="vector", init="zeros"),
                WeightSpec("f", (H, hid)), WeightSpec("f.b", (H,), kind="vector", init="zeros"),
                WeightSpec("norm", (H * V,), kind="vector", init="norm"), WeightSpec("o", (hid, H * V))]

    @property
    def state_floats(self):
        return self.H * self.D * (self.V + 4) + self.H

    def cache_need(self):
        return StateNeed((self.state_floats,), "float32")

    def load(self, tensors, dtype, device):
        self.proj = torch.cat([tensors.pop(n) for n in ("q", "k", "v", "g")], dim=0).contiguous()     # one product for all four
        self.gates = torch.cat([tensors.pop("i"), tensors.pop("f")], dim=0).contiguous()              # [2 H, hidden]: its product is float32
        self.gate_bias = torch.cat([tensors.pop("i.b").float(), tensors.pop("f.b").float()]).contiguous()
        self.norm = tensors.pop("norm").float().contiguous()
        self.o = tensors.pop("o")

    @property
    def first_weight(self):
        return self.proj

    def step_flops(self, rows, pairs):
        return 4 * self.H * self.D * (self.V + 1) * rows

    def forward(self, h, ctx, cache, position, owns_cache=True):
        ops, H, D, V = ctx.ops, self.H, self.D, self.V
        p = ops.linear(h, self.proj)                                # [T, 2 H D + 2 H V]: q | k | v | gate
        gl = ops.linear(h, self.gates, out_dtype=torch.float32)     # [T, 2 H]: input-gate and forget-gate logits
        rows = ops.matrix_memory(p, gl, self.gate_bias, H, D, V, self.cap, self.den_eps, self.norm, p[:, 2 * H * D + H * V:],
                                 self.eps, cache.state, ctx.batch, ctx.dtype)
        return ops.linear(rows, self.o)


@register_mixer("selective_scan")
class SelectiveScan(Part):
    """A selective state-space scan over `inner` channels with `state` numbers each:
        x, z = W_in h;  x <- silu(conv(x) + b) (causal, per channel, conv_taps taps);  dt_low, B, C = W_x x;
        dt = softplus(W_dt dt_low + b_dt) per channel;  A = -exp(A_log) [inner, state];
        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;   y_c = sum_n S[c, n] C_n + D_c x_c;   out = W_o (y * silu(z)).
    The state slot holds S (float32 [inner, state]) and behind it the convolution's last conv_taps - 1 inputs."""

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.I, self.N, self.R, self.taps = int(g("hidden_size")), int(g("inner")), int(g("state")), int(g("dt_rank")), int(g("conv_taps"))
        self.w_in = self.conv = self.conv_b = self.w_x = self.w_dt = self.dt_b = self.A = self.Dv = self.o = None

    def weight_specs(self):
        I, N, R, hid = self.I, self.N, self.R, self.hidden
        return [WeightSpec("in", (2 * I, hid)), WeightSpec("conv", (I, self.taps), kind="vector"), WeightSpec("conv.b", (I,), kind="vector", init="zeros"),
                WeightSpec("x", (R + 2 * N, I)), WeightSpec("dt", (I, R)), WeightSpec("dt.b", (I,), kind="vector", init="zeros"),
                WeightSpec("A_log", (I, N), kind="vector", init="zeros"), WeightSpec("D", (I,), kind="vector", init="norm"), WeightSpec("o", (hid, I))]

    def cache_need(self):
        return StateNeed((self.I * self.N + (self.taps - 1) * self.I,), "float32")

    def load(self, tensors, dtype, device):
        self.w_in, self.w_x, self.w_dt, self.o = tensors.pop("in"), tensors.pop("x"), tensors.pop("dt"), tensors.pop("o")
        self.conv, self.conv_b = tensors.pop("conv").float().contiguous(), tensors.pop("conv.b").float().contiguous()
        self.dt_b, self.Dv = tensors.pop("dt.b").float().contiguous(), tensors.pop("D").float().contiguous()
        self.A = (-torch.exp(tensors.pop("A_log").float())).contiguous()

    @property
    def first_weight(self):
        return self.w_in

    def step_flops(self, rows, pairs):
        return 6 * self.I * self.N * rows

    def forward(self, h, ctx, cache, position, owns_cache=True):
        ops, I, N, R = ctx.ops, self.I, self.N, self.R
        xz = ops.linear(h, self.w_in)                               # [T, 2 I]: x | z
        x = ops.short_conv(xz[:, :I], self.conv, self.conv_b, self.taps, cache.state, I * N, ctx.batch, residual=False, act="silu")
        p = ops.linear(x, self.w_x)                                 # [T, R + 2 N]: dt_low | B | C
        dt = ops.linear(p[:, :R], self.w_dt, out_dtype=torch.float32)    # [T, I] float32, before bias and softplus
        y = ops.selective_scan(x, dt, self.dt_b, self.A, p[:, R:R + N], p[:, R + N:], self.Dv, xz[:, I:], cache.state, ctx.batch, ctx.dtype)
        return ops.linear(y, self.o)
