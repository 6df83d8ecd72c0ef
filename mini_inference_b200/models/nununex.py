"""Nununex: configuration -> ModelSpec.

A decoder whose layers are chosen one by one from three mixers (a delta rule with decay and removal per key channel;
a selective state-space scan; a pair of mixers side by side: windowed softmax attention with a learned distance bias and a
learned sink, and an exponentially gated matrix memory), each followed by a dense feed-forward with a squared relu, a routed
one whose scores multiply the experts' inputs, or none.  Every sublayer reads the normed stream through a short causal
convolution and its output is gated by the normed stream before it is added; the embedding adds a hashed table of token
pairs; the logits pass a soft cap.  The stream is float32.
Tensor names are the checkpoint's own: embed, bigram, l<i>.norm1, l<i>.canon1, l<i>.rg1(.b), l<i>.mix.*, l<i>.norm2, l<i>.canon2,
l<i>.rg2(.b), l<i>.mlp.*, final.norm, head.
"""
from __future__ import annotations

import math

from ..config.nununex_config import NununexConfig
from ..config.registry import register_architecture
from ..config.spec import ExecStep, LayerSpec, ModelSpec, PartSpec

# constants the design fixes
DECAY_SCALE = math.exp(-0.5)        # the delta rule's decay is exp(-DECAY_SCALE * sigmoid(.))
UNIT_KEY_EPS = 1e-6                 # inside the root of the delta rule's unit key
MEMORY_DEN_EPS = 1e-6               # added to the matrix memory's denominator


def _mixer(cfg: NununexConfig, kind: str, m: dict, p: str):
    """(PartSpec of the mixer, {part tensor: checkpoint name})."""
    if kind == "general_delta":
        spec = PartSpec.of("general_delta", hidden_size=cfg.width, num_heads=m["heads"], key_dim=m["dim"], out_norm_eps=cfg.norm_eps,
                           unit_eps=UNIT_KEY_EPS, decay_scale=DECAY_SCALE, decay_rank=m.get("decay_rank", -1))
        tensors = ("r", "k", "v", "g", "a", "a.b", "w1", "w2", "w0", "norm", "o")
    elif kind == "mamba1":
        spec = PartSpec.of("selective_scan", hidden_size=cfg.width, inner=m["inner"], state=m["state"], dt_rank=m["dt_rank"],
                           conv_taps=m["conv"])
        tensors = ("in", "conv", "conv.b", "x", "dt", "dt.b", "A_log", "D", "o")
    else:
        lt, rt = m["left"], m["right"]
        left = PartSpec.of("sink_attention", hidden_size=cfg.width, num_heads=lt["heads"], num_kv_heads=lt["kv_heads"], key_dim=lt["dim"],
                           value_dim=lt["vdim"], scale=lt["scale"], unit_norm_eps=None, window=(lt.get("mask") or {}).get("size"),
                           sink="learned", distance_bias=(lt.get("bias_rows", -1), lt["bias_max"]))
        right = PartSpec.of("matrix_memory", hidden_size=cfg.width, num_heads=rt["heads"], key_dim=rt["dim"], value_dim=rt["vdim"],
                            gate_cap=rt["gate_cap"], out_norm_eps=cfg.norm_eps, den_eps=MEMORY_DEN_EPS)
        spec = PartSpec.of("parallel_pair", hidden_size=cfg.width, eps=cfg.norm_eps, left=left, right=right, left_share=0.5, right_share=0.5)
        tensors = tuple("left." + t for t in ("q", "k", "v", "o", "sink", "rel", "out")) + \
            tuple("right." + t for t in ("q", "k", "v", "g", "i", "i.b", "f", "f.b", "norm", "o", "out"))
    return spec, {f"mixer.{t}": p + "mix." + t for t in tensors}


def build_spec(cfg: NununexConfig) -> ModelSpec:
    none = PartSpec.of("none")
    norm = PartSpec.of("stream_rmsnorm", size=cfg.width, eps=cfg.norm_eps)
    conv = PartSpec.of("causal_conv", size=cfg.width, taps=cfg.canon_taps)
    gate = PartSpec.of("sigmoid_gate", size=cfg.width)
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        mixer, names = _mixer(cfg, layer.type, layer.mixer_dict(), p)
        names.update({"norm1.weight": p + "norm1", "filter1.weight": p + "canon1", "gate1.weight": p + "rg1", "gate1.bias": p + "rg1.b"})
        parts = dict(mixer=mixer, norm1=norm, position=none, filter1=conv, gate1=gate)
        block = "gated_prenorm_mixer"
        if layer.mlp is not None:
            block = "gated_prenorm"
            names.update({"norm2.weight": p + "norm2", "filter2.weight": p + "canon2", "gate2.weight": p + "rg2", "gate2.bias": p + "rg2.b"})
            mlp = layer.mlp
            if mlp.kind == "dense":
                ff = PartSpec.of("relu2_mlp", hidden_size=cfg.width, intermediate_size=mlp.ff)
                names.update({f"feed_forward.{t}": p + "mlp." + t for t in ("up", "up.b", "down", "down.b")})
            else:
                ff = PartSpec.of("routed_experts", hidden_size=cfg.width, num_experts=mlp.experts, top=mlp.top, groups=None,
                                 expert_size=mlp.ff, score="sigmoid", act="silu", weight_on="input", correction=False,
                                 shared_size=mlp.shared, shared_gate=mlp.shared is not None)
                names["feed_forward.router"] = p + "mlp.router"
                for e in range(mlp.experts):
                    names.update({f"feed_forward.e{e}.{t}": f"{p}mlp.e{e}.{t}" for t in ("gate", "up", "down")})
                if mlp.shared is not None:
                    names.update({f"feed_forward.shared.{t}": f"{p}mlp.shared.{t}" for t in ("gate", "up", "down", "sg")})
            parts.update(norm2=norm, filter2=conv, gate2=gate, feed_forward=ff)
        layers.append(LayerSpec.of(block, names, **parts))
    buckets, mul_prev, mul_cur = cfg.bigram
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, layers=tuple(layers), order=tuple(ExecStep(i) for i in range(len(layers))),
        final_norm=norm, embedding_name="embed", final_norm_name="final.norm", lm_head_name="head", max_position=cfg.max_position,
        residual="float32",
        embedding_part=PartSpec.of("hashed_bigram", hidden_size=cfg.width, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur),
        embedding_part_names=(("pairs", "bigram"),), logit_softcap=cfg.logit_softcap)


register_architecture("Nununex", "Nununex (delta-rule / selective-scan / attention-beside-matrix-memory layers, filtered inputs, gated residuals, float32 stream)",
                      NununexConfig, build_spec)
