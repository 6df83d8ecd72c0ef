"""Softmax attention over the paged cache whose mask, softmax and inputs are chosen by constants:

  unit norm    q and k are divided by their root mean square per head (no weight) instead of being rotated;
               positions do not enter the scores
  block_size   B: position i sees j <= i only inside its own block of B positions, floor(i / B) = floor(j / B),
               blocks counted from position 0 of the sequence (None: every j <= i); window: the last W keys (None: all)
  sink         the softmax has one more term whose score is 0 and which carries no value:
               p_j = exp(s_j) / (1 + sum_j exp(s_j))
  value_mix    "source": this layer's values are left in the step context for later layers;
               "blend": v <- (1 - lambda) v + lambda v_source with lambda the tensor `vmix` and v_source the source
               layer's values of the same tokens; the blended v is what is cached
               sink="learned": the term is exp(sink_h) with one learned number per head (the tensor `sink`) instead of 1
  distance_bias  (rows, far): a learned table `rel` [rows, heads] is added to the scaled scores by the distance n = i - j >= 0:
               row n for n < rows / 2, else min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far / (rows/2)) * (rows - rows/2)))
               (one row per distance near by, logarithmic steps that reach the last row at `far`).  The table is spread out
               once, when the weights are loaded, into one float32 row per distance 0 .. far, which the kernels index directly
  key and value rows may differ in size (key_dim, value_dim); the value pool is then a tensor of its own.
  norm_weights True: the per-head norm of q and k multiplies by a learned weight of key_dim entries that all heads share (tensors
               `q.norm`, `k.norm`) after the division by the root mean square (needs unit_norm_eps)
  values       "keys": there is no value projection; a key head's values are its keys AS PROJECTED, before the norm (value_dim = key_dim)
  q_temp       (coef, every): the normed q at position p is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1)
  slope_exponent  e: slope_h * (i - j) is taken off the scaled score of head h = 0 .. H-1, slope_h = 2^(-e (h + 1) / H)

q, k, v come from one product; one kernel norms q and k, blends v and writes k and v into the step's pages
before attention runs, so a portion attends to itself through the cache.  Scores, softmax weights and the weighted
sum are float32."""
from __future__ import annotations

import math

import torch

from .attention import paged_attention_step_arrays
from .base import KVCacheNeed, Part, WeightSpec, register_mixer


@register_mixer("sink_attention")
class SinkAttention(Part):
    step_arrays_key = "paged_attention"

    def __init__(self, spec):
        super().__init__(spec)
        g = spec.get
        self.hidden, self.H, self.KV = int(g("hidden_size")), int(g("num_heads")), int(g("num_kv_heads"))
        self.D, self.V, self.scale = int(g("key_dim")), int(g("value_dim")), float(g("scale"))
        self.eps = g("unit_norm_eps")                       # None: q and k are used as projected
        self.block_size, self.window, self.sink = g("block_size"), g("window"), bool(g("sink", False))
        self.learned_sink = g("sink", False) == "learned"
        self.distance_bias = tuple(g("distance_bias")) if g("distance_bias") else None          # (rows, far)
        # rows = -1: the checkpoint's table says how many rows there are
        if self.distance_bias and self.distance_bias[0] >= 0 and not 0 < self.distance_bias[0] // 2 < self.distance_bias[1]:
            raise ValueError("distance_bias needs at least two rows and a far distance beyond half of them")
        self.value_mix = g("value_mix")
        self.mix_key = g("value_mix_key", "values")
        self.norm_weights, self.values_are_keys = bool(g("norm_weights", False)), g("values", "projected") == "keys"
        self.q_temp = tuple(g("q_temp")) if g("q_temp") else None                               # (coef, every)
        self.slope_exponent = float(g("slope_exponent")) if g("slope_exponent") is not None else None
        if g("values", "projected") not in ("projected", "keys"):
            raise ValueError("values is one of projected, keys")
        if self.norm_weights and self.eps is None:
            raise ValueError("norm_weights needs unit_norm_eps")
        if self.values_are_keys and (self.V != self.D or self.value_mix):
            raise ValueError("values that are the keys have the keys' size and are not blended")
        self.q_norm = self.k_norm = self.slopes = None
        if self.H % self.KV:
            raise ValueError(f"{self.H} query heads are not a multiple of {self.KV} kv heads")
        if self.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix '{self.value_mix}' is not one of source, blend")
        self.qkv = self.o = self.lam = self.sink_values = self.bias_by_distance = self.bias_by_head = None

    def weight_specs(self):
        H, KV, D, V, hid = self.H, self.KV, self.D, self.V, self.hidden
        specs = [WeightSpec("q", (H * D, hid)), WeightSpec("k", (KV * D, hid))]
        if not self.values_are_keys:
            specs.append(WeightSpec("v", (KV * V, hid)))
        specs.append(WeightSpec("o", (hid, H * V)))
        if self.norm_weights:
            specs += [WeightSpec("q.norm", (D,), kind="vector", init="norm"), WeightSpec("k.norm", (D,), kind="vector", init="norm")]
        if self.value_mix:                                  # a source layer's checkpoint holds the number too; it is not used
            specs.append(WeightSpec("vmix", (), kind="vector", init="norm"))
        if self.learned_sink:
            specs.append(WeightSpec("sink", (H,), kind="vector"))
        if self.distance_bias:
            specs.append(WeightSpec("rel", (self.distance_bias[0], H), kind="vector"))
        return specs

    @staticmethod
    def distance_row(n: int, rows: int, far: int) -> int:
        half = rows // 2
        if n < half:
            return n
        return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))

    def cache_need(self):
        return KVCacheNeed(self.KV, self.D, self.window, value_dim=None if self.V == self.D else self.V)

    def load(self, tensors, dtype, device):
        self.qkv = torch.cat([tensors.pop("q"), tensors.pop("k")] + ([] if self.values_are_keys else [tensors.pop("v")]), dim=0).contiguous()
        self.o = tensors.pop("o")
        if self.norm_weights:
            self.q_norm, self.k_norm = tensors.pop("q.norm").float().contiguous(), tensors.pop("k.norm").float().contiguous()
        if self.slope_exponent is not None:
            self.slopes = torch.tensor([2.0 ** (-self.slope_exponent * (h + 1) / self.H) for h in range(self.H)], dtype=torch.float32, device=device)
        if self.value_mix == "blend":
            self.lam = tensors["vmix"].float().reshape(1).contiguous()
        if self.learned_sink:
            self.sink_values = tensors["sink"].float().contiguous()
        if self.distance_bias:
            rows, far = tensors["rel"].shape[0], int(self.distance_bias[1])
            if not 0 < rows // 2 < far:
                raise ValueError("distance_bias needs at least two rows and a far distance beyond half of them")
            index = torch.tensor([self.distance_row(n, rows, far) for n in range(far + 1)], dtype=torch.long, device=device)
            self.bias_by_distance = tensors["rel"].float()[index].contiguous()          # [far + 1, H]; distances beyond far read the last row
            self.bias_by_head = self.bias_by_distance.t().contiguous()                  # [H, far + 1]: the same, read along the distance

    step_arrays = staticmethod(paged_attention_step_arrays)

    @property
    def first_weight(self):
        return self.qkv

    def step_flops(self, rows, pairs):
        return 2 * self.H * (self.D + self.V) * pairs

    def forward(self, h, ctx, cache, position, owns_cache=True):
        ops, H, KV, D, V = ctx.ops, self.H, self.KV, self.D, self.V
        meta = ctx.batch.group_view(cache.group, self.step_arrays_key)
        p = ops.linear(h, self.qkv)                                        # [T, H D + KV D + KV V]
        source = None
        if self.value_mix == "blend":
            source = ctx.shared.get(("value_mix", self.mix_key))
            if source is None or source.shape[1] != KV * V:
                raise ValueError("a layer that blends values in runs before the layer that lends them, or their sizes differ")
        elif self.value_mix == "source":
            ctx.shared[("value_mix", self.mix_key)] = p[:, (H + KV) * D:]      # a view: the kernel below leaves these columns alone
        if self.norm_weights or self.values_are_keys or self.q_temp:
            q = ops.unit_qk_cache(p, H, KV, D, V, self.eps, self.lam, source, meta, cache.k if owns_cache else None,
                                  cache.v if owns_cache else None, q_weight=self.q_norm, k_weight=self.k_norm, q_temp=self.q_temp,
                                  values_are_keys=self.values_are_keys)
        else:
            q = ops.unit_qk_cache(p, H, KV, D, V, self.eps, self.lam, source, meta,
                                  cache.k if owns_cache else None, cache.v if owns_cache else None)
        if self.slopes is not None:
            o = ops.masked_attention(q, cache.k, cache.v, meta, H, KV, D, V, self.scale, self.block_size, self.window, self.sink,
                                     sink_values=self.sink_values, distance_bias=self.bias_by_distance,
                                     distance_bias_by_head=self.bias_by_head, distance_slopes=self.slopes)
        elif self.learned_sink or self.distance_bias:
            o = ops.masked_attention(q, cache.k, cache.v, meta, H, KV, D, V, self.scale, self.block_size, self.window, self.sink,
                                     sink_values=self.sink_values, distance_bias=self.bias_by_distance,
                                     distance_bias_by_head=self.bias_by_head)
        else:
            o = ops.masked_attention(q, cache.k, cache.v, meta, H, KV, D, V, self.scale, self.block_size, self.window, self.sink)
        return ops.linear(o, self.o)
