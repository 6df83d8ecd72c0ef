"""Interfaces and registries of the parts a decoder layer is assembled from.

A part (mixer, feed-forward, norm, position encoding, block arrangement) is a class
registered under a name in the registry of its family.  It is built from its own PartSpec
(sizes and constants), names the tensors it needs in its own terms, and computes through the
kernel namespace handed to it in the StepContext.  It never sees the model's configuration
or its neighbours' specs.

Interfaces
  every part   __init__(spec)            sizes/constants from spec only
               weight_specs()            -> [WeightSpec] (part-local names)
               load(tensors, dtype, device)   takes its tensors (part-local names), may fuse them
  Norm         forward(x, delta, ctx, rows=None) -> y
                   delta is added to x first (in place when rows is None); rows selects
                   the rows to normalise (then x is left untouched)
  Position     rotary_inv_freq() -> float32 [D/2] tensor or None
               on_embedding(x, ctx) -> x       (absolute encodings add here; default: identity)
                   may own tensors like any part (weight names under "position.<name>" of the first layer using it)
  FeedForward  forward(h, ctx) -> [T, hidden]
  Mixer        cache_need() -> KVCacheNeed | StateNeed | None
               forward(h, ctx, cache, position, owns_cache) -> [T, hidden]
                   cache is the LayerCache of the execution step (or of the step it reads)
  Embedding    cache_need() -> StateNeed | None
               forward(ids, table, ctx, cache) -> float32 stream [T, hidden] (the model's embedding table is handed in)
  InputFilter  cache_need() -> StateNeed | None;  forward(h, ctx, state) -> rows of the same shape
  ResidualGate forward(h, ctx) -> (logits [T, hidden], bias [hidden]): the sublayer's output is multiplied by sigmoid(logits + bias)
  Block        roles = {role: family}    the parts it arranges; the model builds one part per role from
                                         LayerSpec.parts and hands them over as a dict
               __init__(spec, parts)
               mixer                     the part whose cache_need() the cache manager serves
               cache_need()              (optional) the step's whole need when parts other than the mixer keep state too:
                                         a tuple of needs; the step's LayerCache then carries the slot tensors in that order
               forward(x, delta, ctx, cache, owns_cache) -> (x, delta)
                   x is the residual stream, delta an addition not yet applied to it

Per-step arrays of a part's own (any part may offer this; the step builder calls it once per step and key):
  step_arrays_key = "name"               parts that share a key share the arrays (all attention layers: one work list)
  step_arrays(facts) -> {name: int32 numpy array}
                   facts: StepFacts (lens, pos0, kv_len, q_start, slots of the entries; tile size of the kernels).
                   The arrays travel to the device in the step's one metadata buffer; the part finds them as
                   ctx.batch.extras[key][name] (device) and ctx.batch.extras_host[key][name] (numpy).  For a given
                   list of entry lengths the arrays must always have the same sizes (decode steps are replayed
                   as graphs over fixed buffers).

Optional fast-path protocol.  Every name below is declared on Part with a default that means "not offered";
a block reads the attributes, it never probes with hasattr:
  offers_open = True       Mixer: forward_open(h, ctx, cache, position, owns_cache) -> (rows, out_weight)
                           FeedForward: forward_open(h, ctx) -> (rows, out_weight)
                               forward() without its last product: forward == linear(rows, out_weight)
  open_weight              the tensor forward_open returns as out_weight (after load)
  first_weight             the tensor that forward() streams first (after load)
  gated_weight             FeedForward: a [2 I, hidden] tensor that forward() hands to ctx.ops.gated_linear (its product is
                               read by the activation only, so the start-up timing of kernels times the pair)
  first_product_probe(ops, rows)
                           -> run(weight), or None.  run does what forward() does with its first weight (the product and
                               whatever this part lets the kernel namespace fuse with it) for `rows` rows of made-up input;
                               the start-up timing of many-row kernels then times that instead of the bare product
  accepts_deferred = True  Norm: forward hands `delta` to ctx.ops.add_rmsnorm untouched, so the block may give it the
                               result of ctx.ops.linear(..., defer=True) (possibly partial sums the kernel adds up)
  keeps_float32_stream = True
                           Norm: forward takes a float32 stream x (and keeps it float32), returns rows of the run's dtype, and
                               accepts pre_add=<float32 [hidden]> (a vector added to every row of the stream before the norm);
                               embed(ids, table, ctx, float32) gathers and norms embedded tokens into a new stream.  A spec
                               with residual="float32" needs it of all its norms
  takes_pair_delta = True  Norm: forward accepts a PairDelta as `delta` (two sublayers' outputs and a bias vector, added to the
                               stream in float32 inside the norm's kernel) and pre_add=<float32 [T, hidden]> (added row by row)
  absolute_table           Position: a learned [rows, hidden] table; the kernel that starts a float32 stream adds row p to the token
                               at position p (on_embedding then has nothing left to do)
  takes_next_weight = True Norm: forward accepts next_weight=<tensor> and passes it to ctx.ops.add_rmsnorm: the block
                               names the first weight of the part that follows, and the kernel may request it into L2
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

from ..config.spec import PartSpec


@dataclass(frozen=True)
class WeightSpec:
    name: str                       # part-local name, e.g. "q_proj"
    shape: Tuple[int, ...]          # a size of -1 is taken from the checkpoint (random-weights mode cannot draw such a tensor)
    kind: str = "matrix"            # "matrix" (GEMM operand) | "vector" | "table" (integers)
    init: str = "normal"            # random-weights mode: "normal" | "norm" | "zeros"
    optional: bool = False


@dataclass(frozen=True)
class KVCacheNeed:
    """Keys and values in pages; window=None keeps every key, W keeps the last W.  planes: 2 = a key and a value
    pool; 1 = one pool of rows per token (a mixer that caches one compressed vector per token and derives both
    keys and values from it); the LayerCache then has no v.  value_dim: the size of a value row when it differs from a
    key row's (head_dim); the value pool is then a tensor of its own."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    planes: int = 2
    value_dim: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state, one slot per live request, zeroed when claimed."""
    shape: Tuple[int, ...]
    dtype: str = "float32"          # "float32", "int32" or "compute"


def flatten_needs(need):
    """A cache need may be None, one need, or a tuple of needs (a mixer that keeps pages AND a state; a block whose own
    parts keep state beside the mixer's): the needs in order, at most one of them a KVCacheNeed."""
    if need is None:
        return ()
    if isinstance(need, (tuple, list)):
        out = tuple(n for part in need for n in flatten_needs(part))
        if sum(isinstance(n, KVCacheNeed) for n in out) > 1:
            raise ValueError("an execution step can own the pages of one cache group only")
        return out
    return (need,)


class GatedDelta:
    """An addition to the residual stream that is still to be gated: the stream receives sigmoid(logits + bias) * (y + y_bias),
    element by element (y_bias: a vector added to every row of y first, or None).  Only norms that declare
    takes_gated_delta understand it; a block hands it to the next norm, whose kernel applies it in float32."""
    __slots__ = ("y", "logits", "bias", "y_bias")

    def __init__(self, y, logits, bias, y_bias=None):
        self.y, self.logits, self.bias, self.y_bias = y, logits, bias, y_bias


class PairDelta:
    """An addition to the residual stream made of two sublayers' outputs that read the same normed rows: the stream receives
    a + b (+ bias, a float32 vector added to every row; None: none), summed in float32.  b may be None (a layer with one
    sublayer).  Only norms that declare takes_pair_delta understand it; a block hands it to the next norm, whose kernel adds it."""
    __slots__ = ("a", "b", "bias")

    def __init__(self, a, b=None, bias=None):
        self.a, self.b, self.bias = a, b, bias


class LayerCache:
    """What one execution step's mixer gets from the cache manager: for pages, the step's key
    and value pools [pages, kv_heads, page_size, head_dim] and the index of the cache group
    whose block tables (ctx.batch.group_view(group, ...)) address them; for state, the slot tensor."""
    def __init__(self, group: int, k=None, v=None, state=None, states=None):
        self.group, self.k, self.v = group, k, v
        # a step that declared several StateNeeds finds their slot tensors in `states`, in the order it declared them
        self.states = tuple(states) if states is not None else (() if state is None else (state,))
        self.state = state if state is not None else (self.states[0] if self.states else None)

    def only(self, pages: bool, states):
        """The view a sub-part gets: the pages (or none) and the given slice of the state tensors."""
        return LayerCache(self.group if pages else -1, self.k if pages else None, self.v if pages else None, states=self.states[states])


class StepContext:
    """What a part sees of the step being run."""
    def __init__(self, ops, batch, dtype, device):
        self.ops, self.batch, self.dtype, self.device = ops, batch, dtype, device
        self.defer_ok = False        # set by the model when every reader of a block's outputs accepts deferred sums
        self.hints_ok = False        # the kernel namespace's add_rmsnorm takes next_weight=
        self.shared = {}             # what a part leaves for later parts of the SAME step, by a key the parts agree on
        self._rows = (None, None)    # (stream, its rows in the run's dtype): see note_rows

    def note_rows(self, stream, rows):
        """A kernel that wrote the float32 stream also wrote its rows in the run's dtype: whoever reads the stream next
        (a block whose sublayers read the stream itself) takes them instead of converting again."""
        self._rows = (stream, rows)

    def rows_of(self, stream):
        """The stream's rows in the run's dtype."""
        if self._rows[0] is stream:
            return self._rows[1]
        return stream if stream.dtype == self.dtype else self.ops.cast_rows(stream, self.dtype)


class Part:
    # the optional protocol, declared (see the module text); a subclass overrides what it offers
    offers_open = False
    open_weight = None
    first_weight = None
    gated_weight = None
    accepts_deferred = False
    takes_next_weight = False
    keeps_float32_stream = False     # Norm: reads and writes a float32 residual stream whatever the run's dtype, takes pre_add=
    takes_gated_delta = False        # Norm: `delta` may be a GatedDelta, applied to the stream in the norm's kernel
    takes_pair_delta = False         # Norm: `delta` may be a PairDelta; pre_add may be a [T, hidden] float32 tensor added row by row
    adds_to_embedding = False        # Position: owns an absolute_table (known before the weights are loaded)
    absolute_table = None            # Position: a [rows, hidden] table whose row p the embedding kernel adds to the token at position p
    owns_state = False               # Block: cache_need() gives the step's whole need (its own parts' state beside the mixer's)
    offers_unbiased = False          # FeedForward: forward_unbiased(h, ctx) -> (y, bias): forward == y + bias, the addition left to the caller
    step_arrays_key: Optional[str] = None

    def first_product_probe(self, ops, rows):
        return None

    def __init__(self, spec: PartSpec):
        self.spec = spec

    def weight_specs(self):
        return []

    def load(self, tensors, dtype, device):
        pass

    def step_arrays(self, facts):
        return {}

    def subparts(self):
        """Parts this part is composed of (a mixer made of two mixers): the model looks through them for weights to time,
        work to count and per-step arrays, as it does through the block's own parts."""
        return []

    def step_flops(self, rows: int, pairs: int) -> int:
        """Floating-point operations beyond the part's matrix products, for `rows` tokens that see `pairs`
        (query, key) pairs (an attention mixer: scores and weighted sum)."""
        return 0


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    "mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {},
    # embedding: how token ids become the first rows of the stream (beyond a plain table lookup);
    # input_filter: what a sublayer's input passes before the sublayer reads it; residual_gate: what a sublayer's output is multiplied by
    "embedding": {}, "input_filter": {}, "residual_gate": {}}


def _register(family: str, name: str):
    def deco(cls):
        _REGISTRIES[family][name] = cls
        return cls
    return deco


def register_mixer(name): return _register("mixer", name)
def register_feed_forward(name): return _register("feed_forward", name)
def register_norm(name): return _register("norm", name)
def register_position(name): return _register("position", name)
def register_block(name): return _register("block", name)
def register_embedding(name): return _register("embedding", name)
def register_input_filter(name): return _register("input_filter", name)
def register_residual_gate(name): return _register("residual_gate", name)


def lookup(family: str, name: str):
    if family not in _REGISTRIES:
        raise KeyError(f"no family of parts named '{family}' (known: {', '.join(sorted(_REGISTRIES))})")
    table = _REGISTRIES[family]
    if name not in table:
        raise KeyError(f"no {family} part named '{name}' is registered (known: {', '.join(sorted(table)) or 'none'})")
    return table[name]


def build_part(family: str, spec: PartSpec, *args):
    return lookup(family, spec.kind)(spec, *args)
