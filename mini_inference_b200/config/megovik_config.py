"""Typed configuration of the Megovik design, read from its own config.json keys.

config.json names every size and every constant that differs between models of the design:
  architecture        "Megovik"
  vocab, width        vocabulary and width of the residual stream
  max_positions       rows of the learned position table
  norm.eps            the one epsilon of all root-mean-square norms
  embedding.scale     the embedded token is multiplied by it before the position vector is added
  logit_scale         the head's product is multiplied by it (absent: 1)
  loop                {start, stop, times}: layers start .. stop-1 run `times` times in a row (absent or null: every layer once)
  layers[i]           type ("latent_attention" | "latent_attention_2" | "attention"), mixer {sizes and constants of that mixer}, and
                      mlp: null (no feed-forward), {"kind": "dense", "ff": n}, or {"kind": "moe", "expert": {ff},
                      "router": {experts, top, scale, groups {count, keep} (optional)}}
    latent_attention    heads, dim, vdim, kv_rank, scale
    latent_attention_2  the same and q_rank
    attention           heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (optional)
A missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .model_config import ConfigError

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "vdim", "kv_rank", "scale"),
    "latent_attention_2": ("heads", "dim", "vdim", "kv_rank", "q_rank", "scale"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
}


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
class MegovikMLP:
    kind: str                                     # "dense" | "moe"
    ff: int                                       # dense: the intermediate size; moe: an expert's
    experts: int = 0
    top: int = 0
    route_scale: float = 1.0
    groups: Optional[Tuple[int, int]] = None      # (count, keep)

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top, "scale": self.route_scale}
        if self.groups is not None:
            router["groups"] = {"count": self.groups[0], "keep": self.groups[1]}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": router}


@dataclass(frozen=True)
class MegovikLayer:
    type: str
    mixer: tuple                                  # nested objects as sorted (key, value) pairs
    mlp: Optional[MegovikMLP]

    def mixer_dict(self) -> dict:
        return _thawed(self.mixer)


def _read_mlp(mlp, where: str) -> Optional[MegovikMLP]:
    if mlp is None:
        return None
    _need(mlp, ("kind",), where)
    if mlp["kind"] == "dense":
        _need(mlp, ("ff",), where)
        return MegovikMLP("dense", int(mlp["ff"]))
    if mlp["kind"] != "moe":
        raise ConfigError(f"config.json: {where}.kind '{mlp['kind']}' is not one of dense, moe")
    _need(mlp, ("router", "expert"), where)
    _need(mlp["router"], ("experts", "top"), f"{where}.router")
    _need(mlp["expert"], ("ff",), f"{where}.expert")
    r = mlp["router"]
    experts, top = int(r["experts"]), int(r["top"])
    if not 1 <= top <= experts:
        raise ConfigError(f"config.json: {where}.router.top is {top}; {experts} experts can be chosen")
    groups = None
    if r.get("groups") is not None:
        _need(r["groups"], ("count", "keep"), f"{where}.router.groups")
        count, keep = int(r["groups"]["count"]), int(r["groups"]["keep"])
        if count < 1 or experts % count or not 1 <= keep <= count:
            raise ConfigError(f"config.json: {where}.router.groups: {experts} experts in {count} groups of which {keep} are kept")
        if keep * (experts // count) < top:
            raise ConfigError(f"config.json: {where}.router: {keep} groups of {experts // count} experts cannot give {top} choices")
        groups = (count, keep)
    return MegovikMLP("moe", int(mlp["expert"]["ff"]), experts, top, float(r.get("scale", 1.0)), groups)


@dataclass(frozen=True)
class MegovikConfig:
    architecture: str
    vocab: int
    width: int
    max_position: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    loop: Optional[Tuple[int, int, int]]          # start, stop, times
    layers: Tuple[MegovikLayer, ...]

    @classmethod
    def from_dict(cls, raw: dict) -> "MegovikConfig":
        _need(raw, ("vocab", "width", "layers", "norm", "max_positions"), "the top level")
        _need(raw["norm"], ("eps",), "'norm'")
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
            if kind == "attention":
                if int(mx["heads"]) % int(mx["kv_heads"]):
                    raise ConfigError(f"config.json: {where}: {mx['heads']} heads are not a multiple of {mx['kv_heads']} kv_heads")
                if int(mx["vdim"]) != int(mx["dim"]):
                    raise ConfigError(f"config.json: {where}: the values are the keys, so vdim ({mx['vdim']}) must equal dim ({mx['dim']})")
                if mx.get("q_temp") is not None:
                    _need(mx["q_temp"], ("coef", "every"), f"{where}.mixer.q_temp")
                    if int(mx["q_temp"]["every"]) < 1:
                        raise ConfigError(f"config.json: {where}.mixer.q_temp.every must be at least 1")
                else:
                    mx.pop("q_temp", None)
            layers.append(MegovikLayer(kind, _frozen(mx), _read_mlp(entry.get("mlp"), f"{where}.mlp")))
        loop = raw.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "'loop'")
            loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
            if not (0 <= loop[0] <= loop[1] <= len(layers)) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {loop} does not fit {len(layers)} layers")
            if loop[0] == loop[1] or loop[2] == 1:
                loop = None
        return cls(architecture=raw.get("architecture") or (raw.get("architectures") or ["Megovik"])[0],
                   vocab=int(raw["vocab"]), width=int(raw["width"]), max_position=int(raw["max_positions"]),
                   norm_eps=float(raw["norm"]["eps"]), embedding_scale=float((raw.get("embedding") or {}).get("scale", 1.0)),
                   logit_scale=float(raw.get("logit_scale", 1.0) if raw.get("logit_scale") is not None else 1.0),
                   loop=loop, layers=tuple(layers))

    def to_dict(self) -> dict:
        layers = [{"type": layer.type, "mixer": layer.mixer_dict(), "mlp": None if layer.mlp is None else layer.mlp.to_dict()}
                  for layer in self.layers]
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_position,
               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
               "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    def describe(self) -> dict:
        return {"architecture": self.architecture, "loop": self.loop,
                "layers": [f"{layer.type}+{layer.mlp.kind if layer.mlp else 'none'}" for layer in self.layers]}
