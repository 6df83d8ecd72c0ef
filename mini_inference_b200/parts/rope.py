"""Rotary position encoding, rotate-half layout (engine/core/model_runner.py:6-8,151-152).
inv_freq_i = 1 / theta^(2i/D) is made once on the host in float32; the angle pos * inv_freq
and its cos/sin are computed in float32 inside the kernel that rotates q and k."""
from __future__ import annotations

import torch

from .base import Part, WeightSpec, register_position


@register_position("rotary")
class RotaryEncoding(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.head_dim = int(spec.get("head_dim"))
        self.theta = float(spec.get("theta"))
        self._inv_freq = None

    def load(self, tensors, dtype, device):
        D = self.head_dim
        inv = 1.0 / (self.theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
        self._inv_freq = inv.to(device)

    def rotary_inv_freq(self):
        return self._inv_freq

    def on_embedding(self, x, ctx):
        return x


@register_position("none")
class NoPosition(Part):
    def rotary_inv_freq(self):
        return None

    def on_embedding(self, x, ctx):
        return x


@register_position("rotary_interleaved")
class InterleavedRotary(Part):
    """Rotary encoding in the interleaved layout: coordinate 2i is paired with 2i+1, i < dims/2, and the pair
    (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * theta^(-2i/dims).  A mixer
    rotates the first `dims` coordinates of the vectors it declares as rotated and passes the rest unchanged.
    The frequencies are made on the host in float64 and rounded once to float32; angle, cos and sin are
    float32 inside the kernel."""
    interleaved = True

    def __init__(self, spec):
        super().__init__(spec)
        self.dims = int(spec.get("dims"))
        self.theta = float(spec.get("theta"))
        self._inv_freq = None

    def load(self, tensors, dtype, device):
        i = torch.arange(0, self.dims // 2, dtype=torch.float64)
        self._inv_freq = (self.theta ** (-2.0 * i / self.dims)).to(torch.float32).to(device)

    def rotary_inv_freq(self):
        return self._inv_freq

    def on_embedding(self, x, ctx):
        return x


@register_position("rotary_half")
class HalfRotary(Part):
    """Rotary encoding of the first `dims` coordinates of a vector in the rotate-half layout: coordinate i is paired with
    i + dims/2, and the pair (u, v) at position p becomes (u cos a - v sin a, v cos a + u sin a), a = p * theta^(-2i/dims);
    coordinates from `dims` on pass unchanged.  The frequencies are made on the host in float64 and rounded once to
    float32; angle, cos and sin are float32 inside the kernel."""

    def __init__(self, spec):
        super().__init__(spec)
        self.dims = int(spec.get("dims"))
        self.theta = float(spec.get("theta"))
        self._inv_freq = None

    def load(self, tensors, dtype, device):
        i = torch.arange(0, self.dims // 2, dtype=torch.float64)
        self._inv_freq = (self.theta ** (-2.0 * i / self.dims)).to(torch.float32).to(device)

    def rotary_inv_freq(self):
        return self._inv_freq

    def on_embedding(self, x, ctx):
        return x


@register_position("learned_absolute")
class LearnedAbsolute(Part):
    """A learned vector per position, added to the embedded token (after the embedding's own scale, itself unscaled):
    x_t = embed[token_t] * scale + table[p_t].  The table is handed to the kernel that starts the float32 stream
    (Part.absolute_table), which adds it in the same pass; mixers of such a model rotate nothing."""
    adds_to_embedding = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size, self.rows = int(spec.get("size")), int(spec.get("rows"))
        self.table = None

    def weight_specs(self):
        return [WeightSpec("table", (self.rows, self.size))]

    def load(self, tensors, dtype, device):
        if "table" in tensors:
            self.table = tensors["table"]

    @property
    def absolute_table(self):
        return self.table

    def rotary_inv_freq(self):
        return None

    def on_embedding(self, x, ctx):
        return x
