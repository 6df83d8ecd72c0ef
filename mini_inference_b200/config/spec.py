"""Architecture-neutral description of a decoder: which parts make each layer, with which
constants, and in which order the layers run.

A model family (models/qwen3.py) turns its typed configuration into a ModelSpec; the
generic decoder (parts/model.py) builds itself from the spec alone.  Nothing in a spec
names a model family, and no part receives more than its own PartSpec.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple


def _freeze(value):
    if isinstance(value, Mapping):
        return tuple(sorted((k, _freeze(v)) for k, v in value.items()))
    if isinstance(value, (list, tuple)):
        return tuple(_freeze(v) for v in value)
    return value


@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name from its registry, with its sizes and constants."""
    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, **params) -> "PartSpec":
        return PartSpec(kind, _freeze(params))

    def get(self, key, default=None):
        return dict(self.params).get(key, default)

    def as_dict(self) -> dict:
        return dict(self.params)


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (block) and the parts it arranges, by ROLE.  Which roles exist
    is the block's business: the pre-norm block takes "mixer", "feed_forward", "norm1", "norm2"
    and "position"; a block with one shared norm, or with four, names its own.  weight_names
    maps each part's tensor names, prefixed by its role ("mixer.q_proj", "norm1.weight", ...),
    to the checkpoint's names, so that no part knows a checkpoint's naming."""
    block: str
    parts: Tuple[Tuple[str, PartSpec], ...]
    weight_names: Tuple[Tuple[str, str], ...]

    @staticmethod
    def of(block: str, weight_names, **parts: PartSpec) -> "LayerSpec":
        names = weight_names.items() if isinstance(weight_names, Mapping) else weight_names
        return LayerSpec(block, tuple(parts.items()), tuple(sorted(names)))

    def part(self, role: str) -> PartSpec:
        return dict(self.parts)[role]

    def checkpoint_name(self, part_tensor: str) -> str:
        return dict(self.weight_names)[part_tensor]


@dataclass(frozen=True)
class ExecStep:
    """One entry of the execution order.  layer indexes ModelSpec.layers (a layer may be named
    by several steps: shared weights, separate caches).  cache_from names an EARLIER step whose
    cache this step's mixer reads instead of owning one.  add_row names a row of the model's
    table of pass vectors (ModelSpec.pass_vectors_name) that is added to the residual stream
    right before this step's layer runs (a model that repeats a span of layers marks each
    repetition this way).  add_embedding: the embedded tokens, as they entered the stream before the first
    layer, are added to the stream right before this step's layer runs (row by row, in the stream's precision)."""
    layer: int
    cache_from: Optional[int] = None
    add_row: Optional[int] = None
    add_embedding: bool = False


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: Tuple[LayerSpec, ...]
    order: Tuple[ExecStep, ...]
    final_norm: PartSpec
    embedding_name: str
    final_norm_name: str
    lm_head_name: Optional[str]          # None: the head is the embedding matrix (tied)
    max_position: int
    eos_token_ids: Tuple[int, ...] = ()
    extra: Tuple[Tuple[str, Any], ...] = field(default=())
    # a norm applied to the embedded tokens before the first layer (None: the embedding enters the stream as it is)
    embedding_norm: Optional[PartSpec] = None
    embedding_norm_name: Optional[str] = None
    # a [rows, hidden] tensor whose rows ExecStep.add_row names
    pass_vectors_name: Optional[str] = None
    pass_vectors_rows: int = 0
    # "compute": the residual stream has the run's dtype; "float32": it is kept in 32 bits whatever the run's dtype
    # (the norms of such a model read and write a float32 stream and hand rows of the run's dtype to the parts)
    residual: str = "compute"
    # a part of the "embedding" family that turns token ids into the first rows of the stream (None: a plain lookup in the
    # embedding table); its tensors are named by embedding_part_names ((part tensor, checkpoint name) pairs); it may keep state
    embedding_part: Optional[PartSpec] = None
    embedding_part_names: Tuple[Tuple[str, str], ...] = ()
    # logits <- cap * tanh(logits / cap) (None: the head's product as it is)
    logit_softcap: Optional[float] = None
    # the embedded token is multiplied by embedding_scale as it enters a float32 stream; the head's product by logit_scale
    embedding_scale: float = 1.0
    logit_scale: float = 1.0

    def __post_init__(self):
        for i, step in enumerate(self.order):
            if not 0 <= step.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {step.layer}; the model has {len(self.layers)}")
            if step.cache_from is not None:
                if not 0 <= step.cache_from < i:
                    raise ValueError(f"order[{i}] reads the cache of step {step.cache_from}, which does not run before it")
                if self.order[step.cache_from].cache_from is not None:
                    raise ValueError(f"order[{i}] reads the cache of step {step.cache_from}, which owns none")
            if step.add_row is not None and not 0 <= step.add_row < self.pass_vectors_rows:
                raise ValueError(f"order[{i}] adds pass vector {step.add_row}; the model has {self.pass_vectors_rows}")
            if step.add_row is not None and step.add_embedding:
                raise ValueError(f"order[{i}] adds both a pass vector and the embedded tokens")
        if self.residual not in ("compute", "float32"):
            raise ValueError(f"residual '{self.residual}' is not one of compute, float32")
