"""Plain, slow statement of the Nununex design: one function per mechanism, token by token where the
design is a recurrence, whole-sequence where it is attention.  It shares no code with the package; the
tests compare the engine with it.

Notation: h is a sublayer's input [T, width]; weights are [out, in]; positions count from 0 in a sequence.
A layer:   n = N(x) * norm1;   x <- x + sigmoid(R1 n + r1) * mixer(n + C1(n));
           n = N(x) * norm2;   x <- x + sigmoid(R2 n + r2) * ff(n + C2(n))
with N(y) = y / sqrt(mean(y^2) + eps) and C a causal per-channel convolution over time (zeros before position 0).
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ small pieces
def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def causal_conv(x, w, bias=None):
    """x [T, C], w [C, taps]: y_t = sum_j w[:, j] x_(t - taps + 1 + j); the last column multiplies the current token."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * x[s]
    return y if bias is None else y + bias


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def distance_bucket(n, rows, far):
    """Row of the distance table for a distance n >= 0: the first half of the rows one by one, the second half in
    logarithmic steps that reach the last row at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


# ------------------------------------------------------------------ embedding
def embed_with_bigram(tokens, w, e):
    """embed[token] + bigram[(prev * mul_prev + token * mul_cur) mod buckets]; a sequence's first token takes row `buckets`."""
    b = e["bigram"]
    rows = []
    for i, t in enumerate(tokens):
        r = b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
        rows.append(w["embed"][t] + w["bigram"][r])
    return torch.stack(rows)


# ------------------------------------------------------------------ mixers
def general_delta(h, w, pre, m, eps):
    """S_t = diag(d_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,  o_t = S_t^T r_t, per head; u the unit key."""
    T, H, D = h.shape[0], m["heads"], m["dim"]
    r = (h @ w[pre + "r"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, H, D)
    v = (h @ w[pre + "v"].T).view(T, H, D)
    d = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ w[pre + "w1"].T) @ w[pre + "w2"].T + w[pre + "w0"])).view(T, H, D)
    a = torch.sigmoid(h @ w[pre + "a"].T + w[pre + "a.b"]).view(T, H, D)
    u = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, D, D, dtype=h.dtype)
    o = torch.zeros(T, H, D, dtype=h.dtype)
    for t in range(T):
        seen = torch.einsum("hd,hde->he", u[t], S)                                 # u^T S_(t-1)
        S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * seen[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hde,hd->he", S, r[t])
    y = rms(o, eps).reshape(T, H * D) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


def window_attention(h, w, pre, m):
    """Grouped softmax attention over the last mask.size positions, a learned bias per distance bucket and head added to
    the scaled scores, and one more term exp(sink_head) in the denominator that has no value."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, D)
    k = (h @ w[pre + "k"].T).view(T, G, D)
    v = (h @ w[pre + "v"].T).view(T, G, V)
    rel, sink = w[pre + "rel"], w[pre + "sink"]
    size = (m.get("mask") or {}).get("size")
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for i in range(T):
        lo = 0 if not size else max(0, i - size + 1)
        rows = [distance_bucket(i - j, rel.shape[0], m["bias_max"]) for j in range(lo, i + 1)]
        for hd in range(H):
            g = hd // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hd]) * m["scale"] + rel[rows, hd]
            top = max(s.max().item(), sink[hd].item())
            e = torch.exp(s - top)
            out[i, hd] = (e[:, None] * v[lo:i + 1, g]).sum(0) / (e.sum() + math.exp(sink[hd].item() - top))
    return out.reshape(T, H * V) @ w[pre + "o"].T


def matrix_memory(h, w, pre, m, eps):
    """Exponentially gated matrix memory with a running maximum that keeps the exponentials small:
    m_t = max(f_t + m_(t-1), i_t);  S_t = e^(f_t + m_(t-1) - m_t) S_(t-1) + e^(i_t - m_t) k_t v_t^T;  n_t alike with k_t alone;
    o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6).  m starts at 0."""
    T, H, D, V, cap = h.shape[0], m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[pre + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[pre + "k"].T).view(T, H, D)
    v = (h @ w[pre + "v"].T).view(T, H, V)
    ig = cap * torch.tanh((h @ w[pre + "i"].T + w[pre + "i.b"]) / cap)
    fg = F.logsigmoid(cap * torch.tanh((h @ w[pre + "f"].T + w[pre + "f.b"]) / cap))
    S = torch.zeros(H, D, V, dtype=h.dtype)
    n = torch.zeros(H, D, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    o = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        new = torch.maximum(fg[t] + mx, ig[t])
        keep, take = torch.exp(fg[t] + mx - new), torch.exp(ig[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    y = rms(o, eps).reshape(T, H * V) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].T)
    return y @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    """Half the sum of the two branches, each normed over the model width with its own weight."""
    left = window_attention(h, w, pre + "left.", m["left"])
    right = matrix_memory(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms(left, eps) * w[pre + "left.out"] + rms(right, eps) * w[pre + "right.out"])


def selective_scan(h, w, pre, m):
    """x, z = W_in h; x = silu(conv(x) + b); dt, B, C = W_x x; dt = softplus(W_dt dt + b) per channel; A = -exp(A_log);
    S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;  out = W_o (y * silu(z))."""
    T, I, N, R = h.shape[0], m["inner"], m["state"], m["dt_rank"]
    xz = h @ w[pre + "in"].T
    x, z = xz[:, :I], xz[:, I:]
    x = F.silu(causal_conv(x, w[pre + "conv"], w[pre + "conv.b"]))
    p = x @ w[pre + "x"].T
    dt = F.softplus(p[:, :R] @ w[pre + "dt"].T + w[pre + "dt.b"])
    Bm, Cm = p[:, R:R + N], p[:, R + N:R + 2 * N]
    A = -torch.exp(w[pre + "A_log"])
    S = torch.zeros(I, N, dtype=h.dtype)
    y = torch.zeros(T, I, dtype=h.dtype)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * Bm[t][None, :]
        y[t] = S @ Cm[t] + w[pre + "D"] * x[t]
    return (y * F.silu(z)) @ w[pre + "o"].T


# ------------------------------------------------------------------ feed-forwards
def dense_ff(h, w, pre):
    return F.relu(h @ w[pre + "up"].T + w[pre + "up.b"]).pow(2) @ w[pre + "down"].T + w[pre + "down.b"]


def gated_expert(h, w, pre):
    return (F.silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, mlp):
    """(chosen experts [T, top], their sigmoid scores [T, top]); the largest scores win, ties to the lower index."""
    s = torch.sigmoid(h @ w[pre + "router"].T)
    idx = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :mlp["router"]["top"]]
    return idx, s.gather(1, idx)


def routed_ff(h, w, pre, mlp, choice=None):
    """sum over a token's chosen experts of expert(score * h), plus sigmoid(W_sg h) * shared(h)."""
    T = h.shape[0]
    idx, s = choice if choice is not None else route(h, w, pre, mlp)
    out = torch.zeros_like(h)
    for t in range(T):
        for j in range(idx.shape[1]):
            out[t] += gated_expert(s[t, j] * h[t:t + 1], w, f"{pre}e{int(idx[t, j])}.")[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[pre + "shared.sg"].T) * gated_expert(h, w, pre + "shared.")
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


def mixer_of(layer, h, w, pre, eps):
    kind, m = layer["type"], layer["mixer"]
    if kind == "general_delta":
        return general_delta(h, w, pre, m, eps)
    if kind == "parallel":
        return parallel_mixer(h, w, pre, m, eps)
    if kind == "mamba1":
        return selective_scan(h, w, pre, m)
    raise ValueError(kind)


def forward(cfg, w, tokens, trace=None, choices=None):
    """Logits [T, vocab] of one sequence fed whole.  trace: a list that receives the stream after every layer.
    choices: {layer: (experts, scores)} to impose a routing instead of computing it."""
    eps = cfg["norm"]["eps"]
    x = embed_with_bigram(list(tokens), w, cfg["embedding"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        n = rms(x, eps) * w[p + "norm1"]
        gate = torch.sigmoid(n @ w[p + "rg1"].T + w[p + "rg1.b"])
        x = x + gate * mixer_of(layer, n + causal_conv(n, w[p + "canon1"]), w, p + "mix.", eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            n = rms(x, eps) * w[p + "norm2"]
            gate = torch.sigmoid(n @ w[p + "rg2"].T + w[p + "rg2.b"])
            inp = n + causal_conv(n, w[p + "canon2"])
            y = dense_ff(inp, w, p + "mlp.") if mlp["kind"] == "dense" else routed_ff(inp, w, p + "mlp.", mlp, (choices or {}).get(i))
            x = x + gate * y
        if trace is not None:
            trace.append(x.clone())
    logits = (rms(x, eps) * w["final.norm"]) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


def forward_logits(cfg, w, tokens):
    return forward(cfg, w, tokens)
