"""Pre-norm residual arrangement (engine/core/model_runner.py:120-131):
x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).  Each addition is carried as a
pending delta into the next norm's kernel, which adds it to the residual stream (in float32,
stored back in the stream's dtype) and normalises in one pass.

What the parts offer of the optional protocol (parts/base.py) is read once at construction:
a mixer or feed-forward that can stop before its last product lets the block make that product
with defer=True when every norm of the model accepts deferred sums; a norm that takes the hint is
told which weight the following part streams first."""
from __future__ import annotations

from .base import GatedDelta, PairDelta, Part, StateNeed, flatten_needs, register_block


@register_block("prenorm")
class PreNormBlock(Part):
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm", "position": "position"}

    def __init__(self, spec, parts):
        super().__init__(spec)
        self.parts = dict(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts.get("feed_forward")
        self.norm1, self.norm2, self.position = parts["norm1"], parts.get("norm2"), parts["position"]
        self.open_mixer = bool(self.mixer.offers_open)
        self.open_ffn = bool(self.feed_forward is not None and self.feed_forward.offers_open)
        self.hint1 = bool(self.norm1.takes_next_weight)
        self.hint2 = bool(self.norm2 is not None and self.norm2.takes_next_weight)

    def norms(self):
        return [n for n in (self.norm1, self.norm2) if n is not None]

    def forward(self, x, delta, ctx, cache, owns_cache=True, pre_add=None):
        """pre_add: a vector added to every row of the stream before this layer (the first norm's kernel adds it
        together with the pending delta); only norms that declare keeps_float32_stream take it."""
        ops = ctx.ops
        w1 = self.mixer.first_weight if self.hint1 else None
        if pre_add is not None:
            h = self.norm1.forward(x, delta, ctx, pre_add=pre_add)
        else:
            h = self.norm1.forward(x, delta, ctx, next_weight=w1) if w1 is not None else self.norm1.forward(x, delta, ctx)
        defer = ctx.defer_ok                   # the readers of `a` and of the returned delta are norms that accept it
        if self.open_mixer:
            rows, w_out = self.mixer.forward_open(h, ctx, cache, self.position, owns_cache)
            a = ops.linear(rows, w_out, defer=True) if defer else ops.linear(rows, w_out)
        else:
            a = self.mixer.forward(h, ctx, cache, self.position, owns_cache)
        if self.feed_forward is None:
            return x, a
        w2 = self.feed_forward.first_weight if self.hint2 else None
        h = self.norm2.forward(x, a, ctx, next_weight=w2) if w2 is not None else self.norm2.forward(x, a, ctx)
        if self.open_ffn and defer:
            rows, w_out = self.feed_forward.forward_open(h, ctx)
            return x, ops.linear(rows, w_out, defer=True)
        return x, self.feed_forward.forward(h, ctx)


@register_block("prenorm_mixer")
class PreNormMixerOnly(PreNormBlock):
    """A layer without feed-forward: x = x + mixer(norm1(x))."""
    roles = {"mixer": "mixer", "norm1": "norm", "position": "position"}


@register_block("outnorm")
class OutputNormBlock(Part):
    """Sublayers read the stream itself and their OUTPUT is normed before it joins the stream:
    x <- x + norm1(mixer(x)); x <- x + norm2(feed_forward(x)), the norms being of the kind that offers add_normed
    (they own the multiplier and the layer scale).  The stream is float32; the sublayers get its rows in the run's
    dtype, which the norm kernel that last wrote the stream has left in the step context."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm", "position": "position"}

    def __init__(self, spec, parts):
        super().__init__(spec)
        self.parts = dict(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts.get("feed_forward")
        self.norm1, self.norm2, self.position = parts["norm1"], parts.get("norm2"), parts["position"]

    def forward(self, x, delta, ctx, cache, owns_cache=True, pre_add=None):
        if delta is not None or pre_add is not None:
            raise ValueError("the output-norm arrangement carries no pending addition and takes no pass vector")
        h = ctx.rows_of(x)
        h = self.norm1.add_normed(x, self.mixer.forward(h, ctx, cache, self.position, owns_cache), ctx)
        if self.feed_forward is not None:
            self.norm2.add_normed(x, self.feed_forward.forward(h, ctx), ctx)
        return x, None


@register_block("outnorm_mixer")
class OutputNormMixerOnly(OutputNormBlock):
    """A layer without feed-forward: x <- x + norm1(mixer(x))."""
    roles = {"mixer": "mixer", "norm1": "norm", "position": "position"}


@register_block("gated_prenorm")
class GatedPreNormBlock(Part):
    """Pre-norm arrangement whose sublayers read a FILTERED copy of the normed rows and whose outputs are GATED by the
    unfiltered rows before they join the stream:
        n = norm1(x);  x <- x + gate1(n) * mixer(filter1(n));   n = norm2(x);  x <- x + gate2(n) * feed_forward(filter2(n)).
    The stream is float32.  Each gated output travels as a GatedDelta to the next norm, whose kernel applies the gate and adds
    to the stream in float32.  The filters may keep state of their own: the block declares the step's whole cache need, the
    mixer's first and the filters' behind it, and hands each part its own piece of the step's LayerCache."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "norm2": "norm", "position": "position",
             "filter1": "input_filter", "filter2": "input_filter", "gate1": "residual_gate", "gate2": "residual_gate"}
    owns_state = True

    def __init__(self, spec, parts):
        super().__init__(spec)
        self.parts = dict(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts.get("feed_forward")
        self.norm1, self.norm2, self.position = parts["norm1"], parts.get("norm2"), parts["position"]
        self.filter1, self.filter2 = parts["filter1"], parts.get("filter2")
        self.gate1, self.gate2 = parts["gate1"], parts.get("gate2")
        for n in self.norms():
            if not n.takes_gated_delta:
                raise ValueError("the gated arrangement needs norms that apply a gated addition (takes_gated_delta)")
        mixer_needs = flatten_needs(self.mixer.cache_need())
        self._mixer_states = sum(isinstance(n, StateNeed) for n in mixer_needs)
        self._needs, at = list(mixer_needs), self._mixer_states
        self._filter_state = {}
        for name in ("filter1", "filter2"):
            f = parts.get(name)
            if f is not None and f.cache_need() is not None:
                self._needs.append(f.cache_need())
                self._filter_state[name] = at
                at += 1

    def norms(self):
        return [n for n in (self.norm1, self.norm2) if n is not None]

    def cache_need(self):
        return tuple(self._needs)

    def _state(self, cache, name):
        return cache.states[self._filter_state[name]] if name in self._filter_state else None

    def forward(self, x, delta, ctx, cache, owns_cache=True, pre_add=None):
        if pre_add is not None:
            raise ValueError("the gated arrangement takes no pass vector")
        n = self.norm1.forward(x, delta, ctx)
        logits, bias = self.gate1.forward(n, ctx)
        y = self.mixer.forward(self.filter1.forward(n, ctx, self._state(cache, "filter1")), ctx,
                               cache.only(True, slice(0, self._mixer_states)), self.position, owns_cache)
        a = GatedDelta(y, logits, bias)
        if self.feed_forward is None:
            return x, a
        n = self.norm2.forward(x, a, ctx)
        logits, bias = self.gate2.forward(n, ctx)
        h = self.filter2.forward(n, ctx, self._state(cache, "filter2"))
        if self.feed_forward.offers_unbiased:
            y, y_bias = self.feed_forward.forward_unbiased(h, ctx)
            return x, GatedDelta(y, logits, bias, y_bias)
        return x, GatedDelta(self.feed_forward.forward(h, ctx), logits, bias)


@register_block("gated_prenorm_mixer")
class GatedPreNormMixerOnly(GatedPreNormBlock):
    """A layer without feed-forward: x <- x + gate1(n) * mixer(filter1(n))."""
    roles = {"mixer": "mixer", "norm1": "norm", "position": "position", "filter1": "input_filter", "gate1": "residual_gate"}


@register_block("parallel_prenorm")
class ParallelPreNormBlock(Part):
    """ONE norm whose rows both sublayers read; their sum joins the stream:  n = norm1(x);  x <- x + (mixer(n) + feed_forward(n)).
    The two outputs travel as a PairDelta to the next norm, whose kernel adds them (and the feed-forward's last bias, when the
    feed-forward leaves it to the adder) to the stream in float32.  pre_add: what is added to the stream before this layer
    (a vector, or a tensor row by row), in the same kernel as the pending addition."""
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "norm1": "norm", "position": "position"}

    def __init__(self, spec, parts):
        super().__init__(spec)
        self.parts = dict(parts)
        self.mixer, self.feed_forward = parts["mixer"], parts.get("feed_forward")
        self.norm1, self.position = parts["norm1"], parts["position"]
        if not self.norm1.takes_pair_delta:
            raise ValueError("the parallel arrangement needs a norm that adds a pair of outputs (takes_pair_delta)")

    def norms(self):
        return [self.norm1]

    def forward(self, x, delta, ctx, cache, owns_cache=True, pre_add=None):
        n = self.norm1.forward(x, delta, ctx, pre_add=pre_add)
        a = self.mixer.forward(n, ctx, cache, self.position, owns_cache)
        if self.feed_forward is None:
            return x, PairDelta(a)
        if self.feed_forward.offers_unbiased:
            f, bias = self.feed_forward.forward_unbiased(n, ctx)
            return x, PairDelta(a, f, bias)
        return x, PairDelta(a, self.feed_forward.forward(n, ctx))


@register_block("parallel_prenorm_mixer")
class ParallelPreNormMixerOnly(ParallelPreNormBlock):
    """A layer without feed-forward: x <- x + mixer(norm1(x)), in the same float32 arithmetic."""
    roles = {"mixer": "mixer", "norm1": "norm", "position": "position"}
