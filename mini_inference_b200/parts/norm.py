"""RMSNorm: y = w * cast(x32 * rsqrt(mean(x32^2) + eps)), statistics in float32.  The
reference calls the loaded model's norm modules (engine/core/model_runner.py:120-121,133);
here the residual addition that precedes a norm is fused into the same kernel."""
from __future__ import annotations

import torch

from .base import PairDelta, Part, WeightSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Part):
    accepts_deferred = True      # delta goes to the kernel namespace untouched
    takes_next_weight = True     # and so does the hint about the weight that is read next

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec.get("size"))
        self.eps = float(spec.get("eps"))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.size,), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"]

    def forward(self, x, delta, ctx, rows=None, next_weight=None):
        if next_weight is not None and ctx.hints_ok:
            return ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, rows, next_weight=next_weight)
        return ctx.ops.add_rmsnorm(x, delta, self.weight, self.eps, rows)


@register_norm("scalar_rmsnorm")
class ScalarRMSNorm(Part):
    """y = g * x / sqrt(mean(x^2) + eps) with ONE learned number g for all coordinates.  The stream x is float32
    whatever the run's dtype: the kernel adds the pending delta (and a pass vector, if one is due) to it in
    float32, stores it back in float32 and hands out the normed rows in the run's dtype."""
    keeps_float32_stream = True

    def __init__(self, spec):
        super().__init__(spec)
        self.eps = float(spec.get("eps"))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].float().reshape(1).contiguous()

    def embed(self, ids, table, ctx, float32=True):
        return ctx.ops.embed_scaled_norm(ids, table, self.weight, self.eps, torch.float32 if float32 else ctx.dtype)

    def forward(self, x, delta, ctx, rows=None, pre_add=None):
        return ctx.ops.add_scaled_rmsnorm(x, delta, self.weight, self.eps, rows, pre_add, ctx.dtype)


@register_norm("stream_rmsnorm")
class StreamRMSNorm(Part):
    """y = w * x / sqrt(mean(x^2) + eps) on a float32 residual stream, rows handed out in the run's dtype
    (a pending delta, if any, is added to the stream first, in float32; a GatedDelta is gated in the same kernel)."""
    keeps_float32_stream = True
    takes_gated_delta = True
    takes_pair_delta = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size, self.eps = int(spec.get("size")), float(spec.get("eps"))
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.size,), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].float().contiguous()

    def forward(self, x, delta, ctx, rows=None, pre_add=None):
        """pre_add: float32 [hidden] (a vector for every row) or [T, hidden] (row by row), added to the stream with the delta."""
        if pre_add is not None or isinstance(delta, PairDelta):
            pair = delta if isinstance(delta, PairDelta) else PairDelta(delta)
            return ctx.ops.stream_rmsnorm_pair(x, pair.a, pair.b, pair.bias, pre_add, self.weight, self.eps, rows, ctx.dtype)
        return ctx.ops.stream_rmsnorm(x, delta, self.weight, self.eps, rows, ctx.dtype)


@register_norm("out_rmsnorm")
class OutputRMSNorm(Part):
    """The norm of an arrangement that norms what a sublayer RETURNS: x <- x + mult * scale * (w * y / rms(y)), with w the
    norm's weight, scale a layer-scale vector (layer_scale=False: none) and mult one number.  x is the float32 stream;
    one kernel norms y, adds to x in float32 and writes x's rows in the run's dtype for the next reader of the stream."""
    keeps_float32_stream = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size, self.eps, self.mult = int(spec.get("size")), float(spec.get("eps")), float(spec.get("mult", 1.0))
        self.layer_scale = bool(spec.get("layer_scale", False))
        self.weight = self.scale = None

    def weight_specs(self):
        specs = [WeightSpec("weight", (self.size,), kind="vector", init="norm")]
        if self.layer_scale:
            specs.append(WeightSpec("scale", (self.size,), kind="vector", init="norm"))
        return specs

    def load(self, tensors, dtype, device):
        self.weight = tensors["weight"].float().contiguous()
        self.scale = tensors["scale"].float().contiguous() if self.layer_scale else None

    def add_normed(self, x, y, ctx):
        """Adds the normed y to the stream x (in place) and returns x's rows in the run's dtype."""
        rows = ctx.ops.out_rmsnorm_add(x, y, self.weight, self.scale, self.mult, self.eps, ctx.dtype)
        ctx.note_rows(x, rows)
        return rows

    def forward(self, x, delta, ctx, rows=None, pre_add=None):
        raise TypeError("out_rmsnorm norms a sublayer's output (add_normed); it is not a norm of the stream")
