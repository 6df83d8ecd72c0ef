"""Typed configuration of the Nununex design, read from its own config.json keys.

config.json names every size and every constant that differs between models of the design:
  architecture        "Nununex"
  vocab, width        vocabulary and width of the residual stream
  norm.eps            the one epsilon of all root-mean-square norms
  canon.taps          taps of the causal convolution that every sublayer's input passes
  embedding.bigram    {buckets, mul_prev, mul_cur}: the hashed table of token pairs added to the embedding
  logit_softcap       logits <- cap * tanh(logits / cap) (absent or null: none)
  layers[i]           type ("general_delta" | "mamba1" | "parallel"), mixer {sizes and constants of that mixer}, and
                      mlp: null (no feed-forward), {"kind": "dense", "ff": n}, or {"kind": "moe", "router": {experts, top},
                      "expert": {ff}, "shared": {ff} (optional)}
    general_delta     heads, dim
    mamba1            inner, state, dt_rank, conv
    parallel          left {heads, kv_heads, dim, vdim, scale, bias_max, mask {size} (optional)}, right {heads, dim, vdim, gate_cap}
A missing key is an error that names it.  Sizes that config.json does not give (the rank of the decay projection, the rows of
the distance table) are read from the checkpoint's tensors; a configuration that is to be filled with random weights names
them (mixer.decay_rank, mixer.left.bias_rows).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError

MIXER_KEYS = {
    "general_delta": ("heads", "dim"),
    "mamba1": ("inner", "state", "dt_rank", "conv"),
    "parallel": ("left", "right"),
}
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max")
RIGHT_KEYS = ("heads", "dim", "vdim", "gate_cap")


def _need(d, keys, where: str):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if d.get(k) is None]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {', '.join(missing)}")


def _frozen(value):
    if isinstance(value, dict):
        return tuple(sorted((k, _frozen(v)) for k, v in value.items()))
    if isinstance(value, list):
        return tuple(_frozen(v) for v in value)
    return value


def _thawed(value):
    if isinstance(value, tuple) and all(isinstance(v, tuple) and len(v) == 2 and isinstance(v[0], str) for v in value):
        return {k: _thawed(v) for k, v in value}
    return value


@dataclass(frozen=True)
class NununexMLP:
    kind: str                                     # "dense" | "moe"
    ff: int                                       # dense: the intermediate size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared: Optional[int] = None                  # intermediate size of the expert that every token uses

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        out = {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff}}
        if self.shared is not None:
            out["shared"] = {"ff": self.shared}
        return out


@dataclass(frozen=True)
class NununexLayer:
    type: str
    mixer: tuple                                  # nested objects as sorted (key, value) pairs
    mlp: Optional[NununexMLP]

    def mixer_dict(self) -> dict:
        return _thawed(self.mixer)


def _read_mlp(mlp, where: str) -> Optional[NununexMLP]:
    if mlp is None:
        return None
    _need(mlp, ("kind",), where)
    if mlp["kind"] == "dense":
        _need(mlp, ("ff",), where)
        return NununexMLP("dense", int(mlp["ff"]))
    if mlp["kind"] != "moe":
        raise ConfigError(f"config.json: {where}.kind '{mlp['kind']}' is not one of dense, moe")
    _need(mlp, ("router", "expert"), where)
    _need(mlp["router"], ("experts", "top"), f"{where}.router")
    _need(mlp["expert"], ("ff",), f"{where}.expert")
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    if not 1 <= top <= experts:
        raise ConfigError(f"config.json: {where}.router.top is {top}; {experts} experts can be chosen")
    shared = mlp.get("shared")
    if shared is not None:
        _need(shared, ("ff",), f"{where}.shared")
        shared = int(shared["ff"])
    return NununexMLP("moe", int(mlp["expert"]["ff"]), experts, top, shared)


@dataclass(frozen=True)
class NununexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int
    bigram: Tuple[int, int, int]                  # buckets, mul_prev, mul_cur
    logit_softcap: Optional[float]
    layers: Tuple[NununexLayer, ...]
    max_position: int = 1 << 20                   # the design tabulates no positions: an engine limit only

    @classmethod
    def from_dict(cls, raw: dict) -> "NununexConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "canon", "embedding"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
        _need(raw["canon"], ("taps",), "'canon'")
        _need(raw["embedding"], ("bigram",), "'embedding'")
        _need(raw["embedding"]["bigram"], ("buckets", "mul_prev", "mul_cur"), "'embedding.bigram'")
        if int(raw["canon"]["taps"]) < 1:
            raise ConfigError("config.json: canon.taps must be at least 1")
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(entry, ("type", "mixer"), where)
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: {where} has type '{kind}' (known: {', '.join(sorted(MIXER_KEYS))})")
            mx = dict(entry["mixer"])
            _need(mx, MIXER_KEYS[kind], f"{where}.mixer")
            if kind == "parallel":
                left, right = dict(mx["left"]), dict(mx["right"])
                _need(left, LEFT_KEYS, f"{where}.mixer.left")
                _need(right, RIGHT_KEYS, f"{where}.mixer.right")
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ConfigError(f"config.json: {where}: {left['heads']} heads are not a multiple of {left['kv_heads']} kv_heads")
                if left.get("mask") is not None:
                    _need(left["mask"], ("size",), f"{where}.mixer.left.mask")
                    if int(left["mask"]["size"]) < 1:
                        raise ConfigError(f"config.json: {where}.mixer.left.mask.size must be at least 1")
                else:
                    left.pop("mask", None)
                mx["left"], mx["right"] = left, right
            if kind == "mamba1" and int(mx["conv"]) < 1:
                raise ConfigError(f"config.json: {where}.mixer.conv must be at least 1")
            layers.append(NununexLayer(kind, _frozen(mx), _read_mlp(entry.get("mlp"), f"{where}.mlp")))
        b = raw["embedding"]["bigram"]
        cap = raw.get("logit_softcap")
        return cls(architecture=raw.get("architecture") or (raw.get("architectures") or ["Nununex"])[0],
                   vocab=int(raw["vocab"]), width=int(raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   canon_taps=int(raw["canon"]["taps"]), bigram=(int(b["buckets"]), int(b["mul_prev"]), int(b["mul_cur"])),
                   logit_softcap=float(cap) if cap else None, layers=tuple(layers),
                   max_position=int(raw.get("max_position", 1 << 20)))

    def to_dict(self) -> dict:
        layers = [{"type": layer.type, "mixer": layer.mixer_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict()}
                  for layer in self.layers]
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "canon": {"taps": self.canon_taps},
               "embedding": {"bigram": {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}},
               "layers": layers}
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out

    def describe(self) -> dict:
        return {"architecture": self.architecture,
                "layers": [f"{layer.type}+{layer.mlp.kind if layer.mlp else 'none'}" for layer in self.layers]}
