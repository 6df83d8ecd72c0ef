"""Megovik: configuration -> ModelSpec.

A decoder whose layers are chosen one by one from three softmax-attention mixers without rotation (latent attention whose
keys and values are up-projections of one cached vector per token; the same with queries that pass a normed latent of their
own; grouped attention whose values are the keys as projected, with normed queries and keys, a query temperature that grows
with the position and a slope per head times the distance taken off the scores).  A layer has ONE norm; the mixer and the
feed-forward (dense with biases and a relu gate, routed with sigmoid scores and a choice confined to the best groups, or
none) both read it and their sum joins the stream.  Tokens enter as embed[token] * scale + pos[position]; a span of layers
may run several times with the same weights, each pass with caches of its own and the embedded tokens added before it; the
stream is float32.
Tensor names are the checkpoint's own: embed, pos, l<i>.norm1, l<i>.mix.*, l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

from ..config.megovik_config import MegovikConfig
from ..config.registry import register_architecture
from ..config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec

# constants the design fixes
SLOPE_EXPONENT = 8.0                # head h of H takes 2^(-SLOPE_EXPONENT (h + 1) / H) per position of distance off its scores
ROUTE_WEIGHT_EPS = 1e-20            # added to the sum the chosen experts' scores are divided by

_MIXER_TENSORS = {
    "latent_attention": ("q", "dkv", "dkv.norm", "uk", "uv", "o"),
    "latent_attention_2": ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "o"),
    "attention": ("q", "k", "q.norm", "k.norm", "o"),
}


def execution_order(num_layers: int, loop):
    """Layers before the repeated span once, the span `times` times (the first layer of every pass but the first is
    marked: the embedded tokens are added before it), the rest once."""
    if loop is None:
        return tuple(ExecStep(i) for i in range(num_layers))
    start, stop, times = loop
    order = [ExecStep(i) for i in range(start)]
    for t in range(times):
        order += [ExecStep(i, add_embedding=t > 0 and i == start) for i in range(start, stop)]
    return tuple(order + [ExecStep(i) for i in range(stop, num_layers)])


def _mixer(cfg: MegovikConfig, kind: str, m: dict) -> PartSpec:
    if kind == "attention":
        t = m.get("q_temp")
        return PartSpec.of("sink_attention", hidden_size=cfg.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], key_dim=m["dim"],
                           value_dim=m["vdim"], scale=m["scale"], unit_norm_eps=cfg.norm_eps, norm_weights=True, values="keys",
                           q_temp=(t["coef"], t["every"]) if t else None, slope_exponent=SLOPE_EXPONENT)
    return PartSpec.of("latent_attention", hidden_size=cfg.width, num_heads=m["heads"], nope_dim=m["dim"], rot_dim=0,
                       value_dim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], latent_norm_eps=cfg.norm_eps, gate=False,
                       q_rank=m["q_rank"] if kind == "latent_attention_2" else None)


def build_spec(cfg: MegovikConfig) -> ModelSpec:
    norm = PartSpec.of("stream_rmsnorm", size=cfg.width, eps=cfg.norm_eps)
    position = PartSpec.of("learned_absolute", size=cfg.width, rows=cfg.max_position)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        names = {"norm1.weight": p + "norm1"}
        names.update({f"mixer.{t}": p + "mix." + t for t in _MIXER_TENSORS[layer.type]})
        if i == 0:
            names["position.table"] = "pos"
        parts = dict(mixer=_mixer(cfg, layer.type, layer.mixer_dict()), norm1=norm, position=position)
        block, mlp = "parallel_prenorm_mixer", layer.mlp
        if mlp is not None:
            block = "parallel_prenorm"
            if mlp.kind == "dense":
                parts["feed_forward"] = PartSpec.of("gated_mlp", hidden_size=cfg.width, intermediate_size=mlp.ff, act="relu", biases=True)
                names.update({f"feed_forward.{t}": p + "mlp." + t for t in ("gate", "gate.b", "up", "up.b", "down", "down.b")})
            else:
                parts["feed_forward"] = PartSpec.of(
                    "routed_experts", hidden_size=cfg.width, num_experts=mlp.experts, top=mlp.top, groups=mlp.groups, expert_size=mlp.ff,
                    score="sigmoid", act="silu", correction=False, group_score="top2_sum", renormalise=True, weight_eps=ROUTE_WEIGHT_EPS,
                    route_scale=mlp.route_scale)
                names["feed_forward.router"] = p + "mlp.router"
                for e in range(mlp.experts):
                    names.update({f"feed_forward.e{e}.{t}": f"{p}mlp.e{e}.{t}" for t in ("gate", "up", "down")})
        layers.append(LayerSpec.of(block, names, **parts))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers), order=execution_order(len(layers), cfg.loop),
        final_norm=norm, embedding_name="embed", final_norm_name="final.norm", lm_head_name="head", max_position=cfg.max_position,
        residual="float32", embedding_scale=cfg.embedding_scale, logit_scale=cfg.logit_scale)


register_architecture("Megovik", "Megovik (latent / query-latent / distance-biased attention layers, one norm for mixer and feed-forward, "
                      "looped span, learned positions, float32 stream)", MegovikConfig, build_spec)
