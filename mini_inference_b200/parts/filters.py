"""What stands between a norm and the sublayer that reads it, and between a sublayer and the residual stream.

causal_conv (input filter)     h <- h + conv(h): a causal convolution over time on every channel, weight [size, taps], no bias,
                               conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) with zeros before a sequence's first position.  The last
                               taps - 1 inputs of a request are state (float32 [taps - 1, size] in its slot), so a portion of a
                               prompt or a single decoded token continues where the step before stopped.
sigmoid_gate (residual gate)   the sublayer's output is multiplied, element by element, by sigmoid(W h + b), h being the rows the
                               norm handed out (before any input filter).  The part only makes the logits W h; the multiplication
                               happens where the output joins the stream, in float32 (GatedDelta, parts/base.py)."""
from __future__ import annotations

from .base import Part, StateNeed, WeightSpec, register_input_filter, register_residual_gate


@register_input_filter("causal_conv")
class CausalConvFilter(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.size, self.taps = int(spec.get("size")), int(spec.get("taps"))
        if self.taps < 1:
            raise ValueError("causal_conv needs at least one tap")
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.size, self.taps), kind="vector")]

    def cache_need(self):
        return StateNeed(((self.taps - 1) * self.size,), "float32") if self.taps > 1 else None

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].float().contiguous()

    def forward(self, h, ctx, state):
        return ctx.ops.short_conv(h, self.weight, None, self.taps, state, 0, ctx.batch, residual=True, act="none")


@register_residual_gate("sigmoid_gate")
class SigmoidGate(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec.get("size"))
        self.weight = self.bias = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.size, self.size)), WeightSpec("bias", (self.size,), kind="vector", init="zeros")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"]
        self.bias = tensors["bias"].float().contiguous()

    @property
    def first_weight(self):
        return self.weight

    def forward(self, h, ctx):
        return ctx.ops.linear(h, self.weight), self.bias
