"""A mixer made of two mixers that read the same input side by side.

parallel_pair   y = left_share * (w_left * N(left(h))) + right_share * (w_right * N(right(h))),  N(y) = y / sqrt(mean(y^2) + eps) over
                the model width, w_left and w_right learned vectors (`left.out`, `right.out`).  `left` and `right` are PartSpecs of
                registered mixers; their tensors are named `left.<name>` and `right.<name>`.  The pair's cache need is the two
                needs side by side (pages of one, a state of the other, two states, ...); each branch gets its own piece of the
                step's cache.  One kernel norms both outputs and adds them."""
from __future__ import annotations

from .base import KVCacheNeed, Part, StateNeed, WeightSpec, build_part, flatten_needs, register_mixer


@register_mixer("parallel_pair")
class ParallelPair(Part):
    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.eps = int(g("hidden_size")), float(g("eps"))
        self.shares = (float(g("left_share", 0.5)), float(g("right_share", 0.5)))
        self.left, self.right = build_part("mixer", g("left")), build_part("mixer", g("right"))
        self.step_arrays_key = self.left.step_arrays_key or self.right.step_arrays_key
        if self.left.step_arrays_key and self.right.step_arrays_key and self.left.step_arrays_key != self.right.step_arrays_key:
            raise ValueError("the two branches ask for per-step arrays under different keys")
        needs = [flatten_needs(self.left.cache_need()), flatten_needs(self.right.cache_need())]
        self._pages = [any(isinstance(n, KVCacheNeed) for n in ns) for ns in needs]
        counts = [sum(isinstance(n, StateNeed) for n in ns) for ns in needs]
        self._states = [slice(0, counts[0]), slice(counts[0], counts[0] + counts[1])]
        self._need = needs[0] + needs[1]
        self.w_left = self.w_right = None

    def subparts(self):
        return [self.left, self.right] + self.left.subparts() + self.right.subparts()

    def step_arrays(self, facts):
        return (self.left if self.left.step_arrays_key else self.right).step_arrays(facts)

    def weight_specs(self):
        specs = [WeightSpec("left." + ws.name, ws.shape, ws.kind, ws.init, ws.optional) for ws in self.left.weight_specs()]
        specs += [WeightSpec("right." + ws.name, ws.shape, ws.kind, ws.init, ws.optional) for ws in self.right.weight_specs()]
        return specs + [WeightSpec("left.out", (self.hidden,), kind="vector", init="norm"),
                        WeightSpec("right.out", (self.hidden,), kind="vector", init="norm")]

    def cache_need(self):
        return flatten_needs(self._need) or None

    def load(self, tensors, dtype, device):
        self.w_left, self.w_right = tensors.pop("left.out").float().contiguous(), tensors.pop("right.out").float().contiguous()
        self.left.load({k[5:]: v for k, v in tensors.items() if k.startswith("left.")}, dtype, device)
        self.right.load({k[6:]: v for k, v in tensors.items() if k.startswith("right.")}, dtype, device)

    @property
    def first_weight(self):
        return self.left.first_weight

    def forward(self, h, ctx, cache, position, owns_cache=True):
        a = self.left.forward(h, ctx, cache.only(self._pages[0], self._states[0]), position, owns_cache)
        b = self.right.forward(h, ctx, cache.only(self._pages[1], self._states[1]), position, owns_cache)
        return ctx.ops.dual_rmsnorm_mix(a, self.w_left, self.shares[0], b, self.w_right, self.shares[1], self.eps)
