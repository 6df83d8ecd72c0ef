"""SwiGLU feed-forward: down(silu(gate(h)) * up(h)) (engine/core/model_runner.py:124-131).
gate and up are stored as one [2*inter, hidden] matrix so that one product serves both, as
the reference does with FUSED_PROJ (engine/core/fused_linear.py:173-177,196)."""
from __future__ import annotations

import torch

from .base import Part, WeightSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(Part):
    offers_open = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.get("hidden_size"))
        self.inter = int(spec.get("intermediate_size"))
        self.gate_up = self.down = None

    def weight_specs(self):
        return [WeightSpec("gate_proj", (self.inter, self.hidden)),
                WeightSpec("up_proj", (self.inter, self.hidden)),
                WeightSpec("down_proj", (self.hidden, self.inter))]

    def load(self, tensors, dtype, device):
        self.gate_up = torch.cat([tensors.pop("gate_proj"), tensors.pop("up_proj")], dim=0).contiguous()
        self.down = tensors.pop("down_proj")

    @property
    def open_weight(self):
        return self.down

    @property
    def first_weight(self):
        return self.gate_up

    @property
    def gated_weight(self):
        return self.gate_up

    def first_product_probe(self, ops, rows):
        x = torch.randn(rows, self.hidden, device=self.gate_up.device, dtype=self.gate_up.dtype)
        return lambda w: ops.gated_linear(x, w)

    def forward(self, h, ctx):
        rows, w = self.forward_open(h, ctx)
        return ctx.ops.linear(rows, w)

    def forward_open(self, h, ctx):
        """Everything but the last product: (silu(gate) * up, down weight)."""
        return ctx.ops.gated_linear(h, self.gate_up), self.down


@register_feed_forward("polynorm_mlp")
class PolyNormMLP(Part):
    """down(act(up(h))) with the polynomial-norm activation
        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,   N(y) = y / sqrt(mean(y^2) + eps) over a token's row,
    powers taken element by element; a, b, c, e are the four learned numbers of the tensor `act`.
    The three statistics are float32 sums over the row, made in one pass by one kernel."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec.get("hidden_size"))
        self.inter = int(spec.get("intermediate_size"))
        self.eps = float(spec.get("eps"))
        self.up = self.down = self.coef = None

    def weight_specs(self):
        return [WeightSpec("up", (self.inter, self.hidden)), WeightSpec("down", (self.hidden, self.inter)),
                WeightSpec("act", (4,), kind="vector", init="norm")]

    def load(self, tensors, dtype, device):
        self.up, self.down = tensors.pop("up"), tensors.pop("down")
        self.coef = tensors.pop("act").float().contiguous()

    @property
    def first_weight(self):
        return self.up

    def forward(self, h, ctx):
        ops = ctx.ops
        return ops.linear(ops.polynorm(ops.linear(h, self.up), self.coef, self.eps), self.down)


@register_feed_forward("routed_experts")
class RoutedExperts(Part):
    """A mixture of small gated feed-forwards of which each token uses `top`, plus an optional expert that every token uses.

    Router (float32): s = softmax(W_r h) over all experts; the CHOICE is made on s + correction, confined to the `keep`
    groups (of `count` equal groups of neighbouring experts) whose best choice score is largest; the chosen experts'
    weights are their plain s, not renormalised.  Expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit),
    y = g * sigmoid(gate_slope * g) * (u + 1), output W_down y.  The token's output is the weighted sum over its experts
    (added in the order of choice, in float32) plus the shared expert's output.

    Options that other designs set: score="sigmoid" (s = sigmoid(W_r h) per expert instead of the softmax); correction=False (no
    correction tensor: the choice is made on s itself); act="silu" (an expert is W_down(silu(W_gate h) * W_up h), no clamps);
    weight_on="input" (a chosen expert's score multiplies its INPUT, out = sum expert(s * h), instead of its output);
    shared_gate=True (the shared expert's output is multiplied by sigmoid(w_sg . h), one number per token, tensor `shared.sg`;
    its logit is made in float32 beside the router's); group_score="top2_sum" (a group is ranked by the sum of its two largest
    choice scores instead of its largest; a group of one expert by that expert's); renormalise=True (the chosen experts' scores are
    divided by their sum + weight_eps); route_scale (the weights are multiplied by it, after the division if there is one)."""

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.E, self.top, self.F = int(g("hidden_size")), int(g("num_experts")), int(g("top")), int(g("expert_size"))
        self.groups = tuple(g("groups")) if g("groups") else None
        self.score, self.act, self.weight_on = g("score", "softmax"), g("act", "clamped"), g("weight_on", "output")
        if self.score not in ("softmax", "sigmoid") or self.act not in ("clamped", "silu") or self.weight_on not in ("output", "input"):
            raise ValueError("routed_experts: score is softmax or sigmoid, act clamped or silu, weight_on output or input")
        self.has_correction, self.shared_gate = bool(g("correction", True)), bool(g("shared_gate", False))
        self.group_score, self.renormalise = g("group_score", "max"), bool(g("renormalise", False))
        self.weight_eps, self.route_scale = float(g("weight_eps", 0.0)), float(g("route_scale", 1.0))
        if self.group_score not in ("max", "top2_sum"):
            raise ValueError("routed_experts: group_score is max or top2_sum")
        self.plain_weights = self.group_score == "max" and not self.renormalise and self.route_scale == 1.0
        self.limit = float(g("limit")) if self.act == "clamped" else float("inf")
        self.slope = float(g("gate_slope", 1.702)) if self.act == "clamped" else 1.0
        self.up_shift = 1.0 if self.act == "clamped" else 0.0
        self.shared_size = g("shared_size")
        self.shared_limit = float(g("shared_limit")) if self.shared_size and self.act == "clamped" else None
        if self.shared_gate and not self.shared_size:
            raise ValueError("routed_experts: a shared gate needs a shared expert")
        self.router = self.correction = self.w_in = self.w_out = self.shared_in = self.shared_out = None

    def weight_specs(self):
        hid, F = self.hidden, self.F
        specs = [WeightSpec("router", (self.E, hid))]
        if self.has_correction:
            specs.append(WeightSpec("correction", (self.E,), kind="vector", init="zeros"))
        for e in range(self.E):
            specs += [WeightSpec(f"e{e}.gate", (F, hid)), WeightSpec(f"e{e}.up", (F, hid)), WeightSpec(f"e{e}.down", (hid, F))]
        if self.shared_size:
            S = int(self.shared_size)
            specs += [WeightSpec("shared.gate", (S, hid)), WeightSpec("shared.up", (S, hid)), WeightSpec("shared.down", (hid, S))]
            if self.shared_gate:
                specs.append(WeightSpec("shared.sg", (1, hid)))
        return specs

    def load(self, tensors, dtype, device):
        self.router = tensors.pop("router").contiguous()                   # stored values as they are; products and sums are float32
        if self.shared_gate:                                               # the shared gate's row rides behind the experts' rows
            self.router = torch.cat([self.router, tensors.pop("shared.sg").reshape(1, -1)], dim=0).contiguous()
        self.correction = tensors.pop("correction").float().contiguous() if self.has_correction else None
        # per expert [gate rows | up rows] and the down matrix, stacked: one grouped product each
        self.w_in = torch.stack([torch.cat([tensors.pop(f"e{e}.gate"), tensors.pop(f"e{e}.up")], dim=0) for e in range(self.E)]).contiguous()
        self.w_out = torch.stack([tensors.pop(f"e{e}.down") for e in range(self.E)]).contiguous()
        if self.shared_size:
            self.shared_in = torch.cat([tensors.pop("shared.gate"), tensors.pop("shared.up")], dim=0).contiguous()
            self.shared_out = tensors.pop("shared.down")

    @property
    def first_weight(self):
        return self.shared_in if self.shared_size else None

    def step_flops(self, rows, pairs):
        return 2 * rows * self.top * 3 * self.F * self.hidden      # the chosen experts' three products (the stacked tensors are not matrices)

    def forward(self, h, ctx):
        ops = ctx.ops
        if not self.plain_weights:
            chosen, weights, extra = ops.route_topk(h, self.router, self.correction, self.top, self.groups, score=self.score,
                                                    extra_rows=int(self.shared_gate), group_score=self.group_score,
                                                    renormalise=self.renormalise, weight_eps=self.weight_eps, route_scale=self.route_scale)
        elif self.score == "softmax" and not self.shared_gate:
            chosen, weights = ops.route_topk(h, self.router, self.correction, self.top, self.groups)
            extra = None
        else:
            chosen, weights, extra = ops.route_topk(h, self.router, self.correction, self.top, self.groups, score=self.score,
                                                    extra_rows=int(self.shared_gate))
        shared = None
        if self.shared_size and self.act == "clamped":
            shared = ops.linear(ops.clamped_glu(ops.linear(h, self.shared_in), self.shared_limit, self.slope), self.shared_out)
        elif self.shared_size:
            shared = ops.linear(ops.gated_linear(h, self.shared_in), self.shared_out)
        if self.act == "clamped" and self.weight_on == "output" and extra is None:
            return ops.expert_ffn(h, chosen, weights, self.w_in, self.w_out, self.limit, self.slope, shared)
        return ops.expert_ffn(h, chosen, weights, self.w_in, self.w_out, self.limit, self.slope, shared, up_shift=self.up_shift,
                              weight_on_input=self.weight_on == "input", shared_gate=extra)


@register_feed_forward("relu2_mlp")
class SquaredReluMLP(Part):
    """W_down (relu(W_up h + b_up))^2 + b_down.  The first bias and the activation are one kernel; the second bias is left to
    whoever adds the output to the stream (forward_unbiased), or added here."""
    offers_unbiased = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.inter = int(spec.get("hidden_size")), int(spec.get("intermediate_size"))
        self.up = self.down = self.up_b = self.down_b = None

    def weight_specs(self):
        return [WeightSpec("up", (self.inter, self.hidden)), WeightSpec("up.b", (self.inter,), kind="vector", init="zeros"),
                WeightSpec("down", (self.hidden, self.inter)), WeightSpec("down.b", (self.hidden,), kind="vector", init="zeros")]

    def load(self, tensors, dtype, device):
        self.up, self.down = tensors.pop("up"), tensors.pop("down")
        self.up_b, self.down_b = tensors.pop("up.b").float().contiguous(), tensors.pop("down.b").float().contiguous()

    @property
    def first_weight(self):
        return self.up

    def forward_unbiased(self, h, ctx):
        ops = ctx.ops
        return ops.linear(ops.bias_act(ops.linear(h, self.up), self.up_b, "relu2"), self.down), self.down_b

    def forward(self, h, ctx):
        y, b = self.forward_unbiased(h, ctx)
        return ctx.ops.bias_act(y, b, "none")


@register_feed_forward("gated_mlp")
class GatedMLP(Part):
    """W_down (act(W_gate h + b_gate) * (W_up h + b_up)) + b_down with act one of relu, silu, gelu_tanh; biases=False: no bias
    anywhere.  gate and up are one [2 I, hidden] product; the first biases, the activation and the product of the two halves are
    one kernel (float32 arithmetic on the product's values); the last bias is left to whoever adds the output to the stream
    (forward_unbiased), or added here."""

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden, self.inter = int(spec.get("hidden_size")), int(spec.get("intermediate_size"))
        self.act, self.biases = spec.get("act", "silu"), bool(spec.get("biases", False))
        if self.act not in ("relu", "silu", "gelu_tanh"):
            raise ValueError("gated_mlp: act is relu, silu or gelu_tanh")
        self.offers_unbiased = self.biases
        self.gate_up = self.down = self.gate_up_b = self.down_b = None

    def weight_specs(self):
        specs = [WeightSpec("gate", (self.inter, self.hidden)), WeightSpec("up", (self.inter, self.hidden)),
                 WeightSpec("down", (self.hidden, self.inter))]
        if self.biases:
            specs += [WeightSpec("gate.b", (self.inter,), kind="vector", init="zeros"), WeightSpec("up.b", (self.inter,), kind="vector", init="zeros"),
                      WeightSpec("down.b", (self.hidden,), kind="vector", init="zeros")]
        return specs

    def load(self, tensors, dtype, device):
        self.gate_up = torch.cat([tensors.pop("gate"), tensors.pop("up")], dim=0).contiguous()
        self.down = tensors.pop("down")
        if self.biases:
            self.gate_up_b = torch.cat([tensors.pop("gate.b").float(), tensors.pop("up.b").float()]).contiguous()
            self.down_b = tensors.pop("down.b").float().contiguous()

    @property
    def first_weight(self):
        return self.gate_up

    def forward_unbiased(self, h, ctx):
        ops = ctx.ops
        return ops.linear(ops.bias_glu(ops.linear(h, self.gate_up), self.gate_up_b, self.act), self.down), self.down_b

    def forward(self, h, ctx):
        y, b = self.forward_unbiased(h, ctx)
        return y if b is None else ctx.ops.bias_act(y, b, "none")
