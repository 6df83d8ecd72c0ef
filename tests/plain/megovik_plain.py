"""Plain, slow statement of the Megovik design: one function per mechanism, whole sequences, no cache.
It shares no code with the package; the tests compare the engine with it.

Notation: h is a sublayer's input [T, width]; weights are [out, in]; positions count from 0 in a sequence;
N(y) = y / sqrt(mean(y^2) + eps) over the last axis.
A layer:   n = N(x) * norm1;   x <- x + (mixer(n) + ff(n))          (one norm, both sublayers read it)
The model: x0 = embed[token] * s + pos[p]; layers in order, a span [start, stop) run `times` times in a row with the
same weights, x0 added to x before every pass but the first; logits = head (N(x) * final.norm) * logit_scale.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch
import torch.nn.functional as F


def rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


# ------------------------------------------------------------------ mixers
def causal_softmax_heads(q, k, v, scale, bias=None):
    """q [T, H, D], k [T, H, D], v [T, H, V] (one key/value head per query head); bias [H, T, T] added to the scaled
    scores (None: none).  Position i sees j <= i."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    if bias is not None:
        s = s + bias
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("hij,jhv->ihv", torch.softmax(s, dim=-1), v)


def latent_attention(h, w, pre, m, eps):
    """Keys and values are up-projections of one normed latent per token; queries come straight from h, or through a
    normed latent of their own when the mixer has a `dq` tensor."""
    T, H, D, V = h.shape[0], m["heads"], m["dim"], m["vdim"]
    if pre + "dq" in w:
        q = (rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]) @ w[pre + "uq"].T
    else:
        q = h @ w[pre + "q"].T
    c = rms(h @ w[pre + "dkv"].T, eps) * w[pre + "dkv.norm"]
    k = (c @ w[pre + "uk"].T).view(T, H, D)
    v = (c @ w[pre + "uv"].T).view(T, H, V)
    o = causal_softmax_heads(q.view(T, H, D), k, v, m["scale"])
    return o.reshape(T, H * V) @ w[pre + "o"].T


def head_slopes(H):
    return torch.tensor([2.0 ** (-8.0 * (hd + 1) / H) for hd in range(H)], dtype=torch.float64)


def query_temperature(T, coef, every):
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=torch.float64)


def biased_attention(h, w, pre, m, eps):
    """Grouped attention whose values are the keys as projected; q and k normed per head with one weight for all heads;
    q scaled by a temperature that grows with the position; slope_head * distance taken off the scaled scores."""
    T, H, G, D = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[pre + "q"].T).view(T, H, D)
    kv = (h @ w[pre + "k"].T).view(T, G, D)
    q = rms(q, eps) * w[pre + "q.norm"]
    k = rms(kv, eps) * w[pre + "k.norm"]
    t = m.get("q_temp")
    if t:
        q = q * query_temperature(T, t["coef"], t["every"]).to(h.dtype)[:, None, None]
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), kv.repeat_interleave(rep, dim=1)
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)                       # i - j
    bias = -head_slopes(H).to(h.dtype)[:, None, None] * dist[None]
    o = causal_softmax_heads(q, k, v, m["scale"], bias)
    return o.reshape(T, H * D) @ w[pre + "o"].T


# ------------------------------------------------------------------ feed-forwards
def dense_ff(h, w, pre):
    g = h @ w[pre + "gate"].T + w[pre + "gate.b"]
    u = h @ w[pre + "up"].T + w[pre + "up.b"]
    return (F.relu(g) * u) @ w[pre + "down"].T + w[pre + "down.b"]


def gated_expert(h, w, pre):
    return (F.silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, r):
    """(chosen experts [T, top], their weights [T, top]).  Scores are sigmoids; a group's score is the sum of its two
    largest scores; only experts of the `keep` best groups can be chosen; ties go to the lower index."""
    s = torch.sigmoid(h.float() @ w[pre + "router"].float().T).to(h.dtype)
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        count, keep = groups["count"], groups["keep"]
        per = E // count
        gs = s.view(T, count, per).topk(min(2, per), dim=-1).values.sum(-1)
        best = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep]
        allowed = torch.zeros(T, count, dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, dim=1)
    masked = torch.where(allowed, s, torch.full_like(s, -1.0))
    idx = torch.sort(masked, dim=-1, descending=True, stable=True).indices[:, :r["top"]]
    chosen = s.gather(1, idx)
    return idx, chosen / (chosen.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def routed_ff(h, w, pre, mlp, choice=None):
    idx, wt = choice if choice is not None else route(h, w, pre, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(idx.shape[1]):
            out[t] += wt[t, j] * gated_expert(h[t:t + 1], w, f"{pre}e{int(idx[t, j])}.")[0]
    return out


# ------------------------------------------------------------------ the model
def load_model_dir(model_dir, dtype=torch.float64):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    with open(os.path.join(model_dir, "model.safetensors"), "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}
    w = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[info["dtype"]]).reshape(info["shape"]) if b > a else \
            torch.zeros(info["shape"], dtype=kinds[info["dtype"]])
        w[name] = t.to(dtype) if t.is_floating_point() else t
    return cfg, w


def layer_runs(cfg):
    """The layers' indices in the order they run, with a mark on the first layer of every pass but the first."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop or loop["times"] <= 1 or loop["stop"] <= loop["start"]:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def mixer_of(layer, h, w, pre, eps):
    if layer["type"] in ("latent_attention", "latent_attention_2"):
        return latent_attention(h, w, pre, layer["mixer"], eps)
    if layer["type"] == "attention":
        return biased_attention(h, w, pre, layer["mixer"], eps)
    raise ValueError(layer["type"])


def forward(cfg, w, tokens, trace=None, choices=None):
    """Logits [T, vocab] of one sequence fed whole.  trace: a list that receives the stream after every layer run.
    choices: {run index: (experts, weights)} to impose a routing instead of computing it."""
    eps = cfg["norm"]["eps"]
    tokens = list(tokens)
    x0 = w["embed"][tokens] * cfg["embedding"]["scale"] + w["pos"][:len(tokens)]
    x = x0
    for run, (i, again) in enumerate(layer_runs(cfg)):
        layer, p = cfg["layers"][i], f"l{i}."
        if again:
            x = x + x0
        n = rms(x, eps) * w[p + "norm1"]
        y = mixer_of(layer, n, w, p + "mix.", eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ff(n, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(n, w, p + "mlp.", mlp, (choices or {}).get(run)))
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T * cfg.get("logit_scale", 1.0)


def forward_logits(cfg, w, tokens):
    return forward(cfg, w, tokens)
