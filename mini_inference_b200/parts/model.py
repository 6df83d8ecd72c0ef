"""The generic decoder: embedding, the layers of a ModelSpec run in the spec's order, final
norm on the rows whose logits are wanted, and the head (engine/core/model_runner.py:112-135).
It is built from the spec alone; which family the spec came from is unknown here."""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.spec import ModelSpec, PartSpec
from .base import Part, WeightSpec, build_part, lookup


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self._positions: Dict = {}
        self.blocks = []
        self._owned: List[Tuple[str, WeightSpec, Part]] = []      # (checkpoint name, spec, owner)
        for li, layer in enumerate(spec.layers):
            names = dict(layer.weight_names)
            block_cls = lookup("block", layer.block)
            given = dict(layer.parts)
            if set(given) != set(block_cls.roles):
                raise KeyError(f"layer {li}: block '{layer.block}' arranges the roles {sorted(block_cls.roles)}, "
                               f"the layer gives {sorted(given)}")
            parts = {}
            for role, family in block_cls.roles.items():
                pspec = given[role]
                if family == "position":               # one position part per distinct spec, shared by its layers;
                    part = self._positions.get(pspec)  # its tensors (if any) are named by the first layer that uses it
                    if part is not None:
                        parts[role] = part
                        continue
                    part = self._positions[pspec] = build_part(family, pspec)
                else:
                    part = build_part(family, pspec)
                parts[role] = part
                for ws in part.weight_specs():
                    key = f"{role}.{ws.name}"
                    if key not in names:
                        raise KeyError(f"layer {li}: weight_names has no entry for '{key}'")
                    self._owned.append((names[key], ws, part))
            self.blocks.append(block_cls(PartSpec.of(layer.block), parts))
        self.final_norm = build_part("norm", spec.final_norm)
        self.embedding_norm = build_part("norm", spec.embedding_norm) if spec.embedding_norm is not None else None
        self.embedder = None
        if spec.embedding_part is not None:
            if spec.embedding_norm is not None or spec.residual != "float32":
                raise ValueError("an embedding part starts a float32 stream and takes the place of an embedding norm")
            self.embedder = build_part("embedding", spec.embedding_part)
            names = dict(spec.embedding_part_names)
            for ws in self.embedder.weight_specs():
                if ws.name not in names:
                    raise KeyError(f"embedding_part_names has no entry for '{ws.name}'")
                self._owned.append((names[ws.name], ws, self.embedder))
        norms = [p for b in self.blocks for role, p in b.parts.items() if b.roles[role] == "norm"] + [self.final_norm]
        if self.embedding_norm is not None:
            norms.append(self.embedding_norm)
            for ws in self.embedding_norm.weight_specs():
                self._owned.append((spec.embedding_norm_name, ws, self.embedding_norm))
        if spec.residual == "float32" and not all(n.keeps_float32_stream for n in norms):
            raise ValueError("the spec keeps the residual stream in float32, but one of its norms does not offer that")
        self._norms_accept_deferred = all(n.accepts_deferred for n in norms)
        absolute = [p for p in self._positions.values() if p.adds_to_embedding]
        self._absolute = absolute[0] if absolute else None
        if len(absolute) > 1 or ((absolute or spec.embedding_scale != 1.0) and
                                 (spec.residual != "float32" or spec.embedding_norm is not None or spec.embedding_part is not None)):
            raise ValueError("a position table and an embedding scale belong to the plain start of a float32 stream, one table at most")
        self._adds_embedding = any(step.add_embedding for step in spec.order)
        for ws in self.final_norm.weight_specs():
            self._owned.append((spec.final_norm_name, ws, self.final_norm))
        self.embedding = None
        self.lm_head = None
        self.pass_vectors = None
        self.dtype = None
        self.device = None

    def _parts_of(self, block):
        """The block's parts and, behind each, the parts it is composed of."""
        for part in block.parts.values():
            yield part
            yield from part.subparts()

    # ---------------------------------------------------------------- weights
    def weight_table(self) -> List[Tuple[str, WeightSpec]]:
        """Every tensor the checkpoint must hold: (checkpoint name, spec)."""
        table = [(self.spec.embedding_name, WeightSpec("embedding", (self.spec.vocab_size, self.spec.hidden_size)))]
        table += [(name, ws) for name, ws, _ in self._owned]
        if self.spec.pass_vectors_name is not None:
            table.append((self.spec.pass_vectors_name, WeightSpec("pass_vectors", (self.spec.pass_vectors_rows, self.spec.hidden_size),
                                                                  kind="vector")))
        if self.spec.lm_head_name is not None:
            table.append((self.spec.lm_head_name, WeightSpec("lm_head", (self.spec.vocab_size, self.spec.hidden_size))))
        return table

    def ignorable_names(self):
        """Tensors a checkpoint may hold that the model does not read (a tied head's copy)."""
        return {"lm_head.weight"} if self.spec.lm_head_name is None else set()

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device) -> None:
        """tensors: checkpoint name -> tensor already on the device in its runtime dtype."""
        self.dtype, self.device = dtype, torch.device(device)
        per_part: Dict[int, Dict[str, torch.Tensor]] = {}
        for name, ws, part in self._owned:
            per_part.setdefault(id(part), {})[ws.name] = tensors[name]
        seen = set()
        for _, _, part in self._owned:
            if id(part) not in seen:
                seen.add(id(part))
                part.load(per_part[id(part)], dtype, self.device)
        for position in self._positions.values():
            if id(position) not in seen:
                position.load({}, dtype, self.device)
        self.embedding = tensors[self.spec.embedding_name]
        if self.spec.pass_vectors_name is not None:            # added to a float32 stream or to one of the run's dtype
            pv = tensors[self.spec.pass_vectors_name]
            self.pass_vectors = (pv.float() if self.spec.residual == "float32" else pv.to(dtype)).contiguous()
        self.lm_head = self.embedding if self.spec.lm_head_name is None else tensors[self.spec.lm_head_name]

    def matrix_weights(self):
        """The matrices the model multiplies by (after the parts fused what they fuse)."""
        out = []
        for block in self.blocks:
            for part in self._parts_of(block):
                out += [v for v in vars(part).values() if isinstance(v, torch.Tensor) and v.dim() == 2 and v.is_floating_point()]
        out.append(self.lm_head)
        return out

    def deferrable_shapes(self):
        """(N, K) of the products whose only reader is a norm (the last product of a mixer or feed-forward that offers
        forward_open), when every norm accepts deferred sums: the kernel namespace may time them accordingly."""
        if not self._norms_accept_deferred:
            return frozenset()
        shapes = set()
        for block in self.blocks:
            for part in self._parts_of(block):
                w = part.open_weight
                if part.offers_open and isinstance(w, torch.Tensor) and w.dim() == 2:
                    shapes.add((w.shape[0], w.shape[1]))
        return frozenset(shapes)

    def gated_shapes(self):
        """(N, K) of the matrices that go through ctx.ops.gated_linear."""
        shapes = set()
        for block in self.blocks:
            for part in self._parts_of(block):
                w = part.gated_weight
                if isinstance(w, torch.Tensor) and w.dim() == 2:
                    shapes.add((w.shape[0], w.shape[1]))
        return frozenset(shapes)

    def first_product_probes(self, ops):
        """{(N, K) of a part's first weight: probe(rows) -> run(weight)} for the parts that offer one (see Part)."""
        probes = {}
        for block in self.blocks:
            for part in self._parts_of(block):
                w = part.first_weight
                if isinstance(w, torch.Tensor) and w.dim() == 2 and (w.shape[0], w.shape[1]) not in probes:
                    if part.first_product_probe(ops, 1) is not None:
                        probes[(w.shape[0], w.shape[1])] = (lambda rows, part=part: part.first_product_probe(ops, rows))
        return probes

    def step_flops(self, rows: int, pairs: int, logit_rows: int) -> int:
        """Floating-point operations of a step that feeds `rows` tokens which see `pairs` (query, key) pairs in all and
        wants logits for `logit_rows` of them: 2 per weight element and row, plus what the mixers report."""
        total = 2 * logit_rows * self.lm_head.numel()
        for step in self.spec.order:
            for part in self._parts_of(self.blocks[step.layer]):
                total += 2 * rows * sum(v.numel() for v in vars(part).values()
                                        if isinstance(v, torch.Tensor) and v.dim() == 2 and v.is_floating_point())
                total += part.step_flops(rows, pairs)
        return total

    def step_array_hooks(self):
        """{key: part.step_arrays} of the parts that ask for per-step arrays of their own, one per key."""
        hooks = {}
        for block in self.blocks:
            for part in self._parts_of(block):
                if part.step_arrays_key is not None:
                    hooks.setdefault(part.step_arrays_key, part.step_arrays)
        return hooks

    # ---------------------------------------------------------------- cache needs
    def cache_needs(self):
        """Per execution step: the mixer's need (the block's, when its own parts keep state too), or None when the step
        reads another's cache.  An embedding part that keeps state adds one more entry behind the steps'."""
        needs = []
        for step in self.spec.order:
            block = self.blocks[step.layer]
            if step.cache_from is not None:
                needs.append(None)
            else:
                needs.append(block.cache_need() if block.owns_state else block.mixer.cache_need())
        if self.embedder is not None and self.embedder.cache_need() is not None:
            needs.append(self.embedder.cache_need())
        return needs

    # ---------------------------------------------------------------- one step
    def forward(self, ctx, caches):
        """caches[i]: LayerCache of execution step i.  Returns float32 logits for
        ctx.batch.logit_rows, or None when no row wants logits."""
        b, ops = ctx.batch, ctx.ops
        ctx.defer_ok = self._norms_accept_deferred and getattr(ops, "deferred", False)
        ctx.hints_ok = getattr(ops, "takes_hints", False)
        if self.embedder is not None:                          # its cache entry, if it keeps state, lies behind the steps'
            x = self.embedder.forward(b.token_ids, self.embedding, ctx, caches[len(self.spec.order)] if len(caches) > len(self.spec.order) else None)
        elif self.embedding_norm is not None:                  # gather and norm in one kernel; the stream starts normed
            x = self.embedding_norm.embed(b.token_ids, self.embedding, ctx, float32=self.spec.residual == "float32")
        elif self._absolute is not None or self.spec.embedding_scale != 1.0:      # embed[token] * scale + table[position], one kernel
            x = ops.embed_scaled_stream(b.token_ids, self.embedding, float(self.spec.embedding_scale),
                                        None if self._absolute is None else self._absolute.absolute_table, b.positions)
        elif self.spec.residual == "float32":                  # the stream in float32 and, beside it, its rows in the run's dtype
            x, rows = ops.embed_stream(b.token_ids, self.embedding, ctx.dtype)
            ctx.note_rows(x, rows)
        else:
            x = ops.embedding(b.token_ids, self.embedding)
        for position in self._positions.values():
            x = position.on_embedding(x, ctx)
        delta = None
        entered = x.clone() if self._adds_embedding else None  # the stream is rewritten in place; the passes add what entered it
        for i, step in enumerate(self.spec.order):
            src = i if step.cache_from is None else step.cache_from
            block = self.blocks[step.layer]
            if step.add_embedding:
                x, delta = block.forward(x, delta, ctx, caches[src], step.cache_from is None, pre_add=entered)
            elif step.add_row is None:
                x, delta = block.forward(x, delta, ctx, caches[src], step.cache_from is None)
            else:
                x, delta = block.forward(x, delta, ctx, caches[src], step.cache_from is None,
                                         pre_add=self.pass_vectors[step.add_row])
        if b.num_logit_rows == 0:
            return None
        h = self.final_norm.forward(x, delta, ctx, rows=b.logit_rows)
        logits = ops.linear(h, self.lm_head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0:
            logits = ops.scale_logits(logits, float(self.spec.logit_scale))
        if self.spec.logit_softcap is not None:
            logits = ops.softcap(logits, float(self.spec.logit_softcap))
        return logits
