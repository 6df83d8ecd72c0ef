"""Nununex in the engine against the plain implementation (tests/plain/nununex_plain.py).

Without a GPU the engine runs on the stand-in kernel namespace (tests/ref_ops.py), which exercises configuration,
weights, spec, parts, the cache and state manager, the batch builder, the scheduler and the entry point.  With a GPU
(-m gpu) the same checks run on the CUDA kernels in float32 and bfloat16, plus each kernel alone against the plain
statement of its op."""
import io
import json
import math
import os
import random
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from mini_inference_b200 import LLM, SamplingParams
from mini_inference_b200.config import ConfigError, load_config, resolve
from mini_inference_b200.config.nununex_config import NununexConfig
from mini_inference_b200.engine.batch import StepEntry
from mini_inference_b200.engine.factory import load_model, make_runner
from mini_inference_b200.weights import write_random_model
from mini_inference_b200.weights.safetensors_io import write_safetensors
from tests.plain import nununex_plain as plain
from tests.ref_ops import TorchRefOps

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
gpu = pytest.mark.gpu


def delta(heads, dim, rank, mlp=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp}


def scan(inner, state, dt_rank, conv, mlp=None):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}, "mlp": mlp}


def pair(heads, kv, dim, vdim, scale, rows, far, window, r_heads, r_dim, r_vdim, cap, mlp=None):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far, "bias_rows": rows}
    if window:
        left["mask"] = {"size": window}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "gate_cap": cap}}, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def config(width, vocab, layers, taps=3, eps=1e-5, cap=25.0, bigram=(89, 13, 5)):
    return {"architecture": "Nununex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "logit_softcap": cap,
            "embedding": {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}, "layers": layers}


# Small configurations that differ from one another in every size; none makes two sizes equal by accident.
CONFIGS = {
    # all three mixers, every kind of feed-forward, a window of 7 positions (edges inside every page and portion), two and three
    # experts per token, filters of four taps beside a scan convolution of two, a layer without feed-forward
    "mix": (config(48, 131, [delta(3, 8, 5, dense(40)), scan(40, 6, 3, 2, moe(6, 2, 10, shared=14)),
                             pair(6, 2, 8, 12, 0.3, 10, 40, 7, 2, 12, 8, 9.0, moe(5, 3, 12)), delta(2, 12, 4)], taps=4), 4),
    # one head everywhere, one expert of one, no window, a single tap (no filter state at all), no soft cap, one bucket of pairs
    "ones": (config(40, 97, [pair(1, 1, 24, 8, 0.2, 4, 9, None, 1, 16, 20, 2.0, moe(3, 1, 8)), scan(24, 1, 1, 1, dense(56)),
                             delta(1, 16, 1, moe(2, 2, 6, shared=5))], taps=1, eps=1e-6, cap=None, bigram=(1, 3, 2)), 8),
    # a window equal to the page size, one of twice the page size and one longer than any request; a distance table that ends inside
    # the window (far < window) and one that is never exhausted; five taps
    "pages": (config(64, 150, [pair(4, 1, 16, 16, 0.25, 8, 12, 16, 4, 8, 16, 15.0, dense(72)), scan(48, 5, 4, 4, moe(8, 2, 8, shared=24)),
                               pair(8, 4, 8, 4, 0.35, 6, 500, 32, 2, 8, 12, 30.0, moe(4, 4, 16)),
                               pair(2, 2, 8, 8, 0.3, 16, 64, 400, 1, 4, 4, 5.0), delta(4, 8, 3, dense(36))], taps=5, bigram=(1021, 65537, 99991)), 16),
}
STD = 0.25


def _perturb(d, seed=7):
    """The random-weights writer leaves biases and offsets at zero; give every one of them values, so that leaving one out shows."""
    cfg, w = plain.load_model_dir(d, dtype=torch.bfloat16)         # the checkpoint's own type
    g = torch.Generator().manual_seed(seed)
    for name in w:
        if name.endswith((".b", ".w0", ".A_log", ".sink")):
            scale = 1.0 if name.endswith((".sink", ".f.b", ".i.b")) else 0.4
            w[name] = (torch.randn(w[name].shape, generator=g) * scale).to(torch.bfloat16)
    write_safetensors(os.path.join(d, "model.safetensors"), [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in w.items()])
    _PLAIN.pop(d, None)
    return d


@pytest.fixture(scope="module")
def dirs(tmp_path_factory):
    out = {}
    for i, (name, (cfg, page)) in enumerate(CONFIGS.items()):
        d = str(tmp_path_factory.mktemp("nununex_" + name))
        write_random_model(cfg, d, seed=30 + i, std=STD, norm_init="uniform")
        out[name] = (_perturb(d), cfg, page)
    return out


def tokens(vocab, n, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


_PLAIN = {}


def plain_logits(d, ids):
    if d not in _PLAIN:
        _PLAIN[d] = plain.load_model_dir(d)
    cfg, w = _PLAIN[d]
    return plain.forward_logits(cfg, w, ids).float()


def err(got, want):
    return ((got - want).abs().max() / want.abs().max()).item()


def assert_close(got, want, tol, what=""):
    """float32 (tol < 1e-2): every position within tol.  bfloat16: the rows that reach a router carry 8 mantissa bits, so where two
    experts' scores nearly tie the choice can fall the other way than in the plain implementation, and that token (and, through
    the states, some later ones) then differs by more than rounding.  So: the median position within tol / 3 and at most one in
    six beyond tol; what the mechanisms compute is pinned by the float32 runs and the kernels' own tests."""
    if tol < 1e-2:
        assert err(got, want) < tol, (what, err(got, want))
        return
    per = (got - want).abs().amax(-1) / want.abs().max()
    assert per.median().item() < tol / 3 and (per > tol).float().mean().item() <= 1 / 6, (what, per.median().item(), per.max().item())


def engine(d, page, pages, dtype="float32", device="cpu", max_seqs=4):
    _, model, _ = load_model(d, dtype, device)
    return make_runner(model, page, pages, max_seqs, ops=TorchRefOps() if device == "cpu" else None)


def feed(runner, key, ids, cuts):
    seq = runner.cache.admit(key)
    out, at = [], 0
    for n in cuts:
        out.append(runner.step([StepEntry(seq, ids[at:at + n], range(n))]).float().cpu())
        at += n
    assert at == len(ids)
    runner.cache.free(seq)
    return torch.cat(out)


def portions(n, rng, smallest=2, largest=9):
    cuts = []
    while n > 0:
        c = min(n, rng.randint(smallest, largest))
        if n - c == 1:
            c += 1
        cuts.append(c)
        n -= c
    return cuts


def check_cuts(runner, d, vocab, tol, n=61):
    """Whole prompt; most of it then the last 24 one by one; portions of 2..9 tokens; portions of two; from the first token one by
    one (long decoding: every state and cache row is written one token at a time, every window edge is crossed)."""
    ids = tokens(vocab, n, seed=3)
    want = plain_logits(d, ids)
    free = runner.cache.free_pages()
    assert_close(feed(runner, "w", ids, [n]), want, tol, "whole")
    assert_close(feed(runner, "d", ids, [n - 24] + [1] * 24), want, tol, "decode")
    assert_close(feed(runner, "p", ids, portions(n, random.Random(1))), want, tol, "portions")
    assert_close(feed(runner, "2", ids[:20], [2] * 10), want[:20], tol, "twos")
    assert_close(feed(runner, "1", ids, [1] * n), want, tol, "ones")
    runner.cache.check_invariants()
    assert runner.cache.free_pages() == free


def check_mixed(make, d, vocab, page, tol, lens=(23, 9, 31, 17, 40, 12, 27, 36, 20, 33), seed=7):
    """Up to four live requests, portions of some beside single tokens of others, some left out of a step; the pool holds four of
    the longest requests and there are four state slots, so pages and slots are used again (both counted)."""
    rng = random.Random(seed)
    reqs = {f"r{i}": tokens(vocab, n, seed=100 + i) for i, n in enumerate(lens)}
    want = {k: plain_logits(d, v) for k, v in reqs.items()}
    pages = 4 * -(-max(lens) // page)
    runner = make(pages)
    takes, slot_uses = {}, {}
    for g in runner.cache.kv_groups:
        inner = g.pool.take
        def counted(inner=inner, gi=id(g)):
            pg = inner()
            takes[(gi, pg)] = takes.get((gi, pg), 0) + 1
            return pg
        g.pool.take = counted
    pending, live, got = list(reqs), {}, {k: [] for k in reqs}
    while pending or live:
        while pending and len(live) < 4:
            k = pending.pop(0)
            live[k] = [runner.cache.admit(k), 0]
            slot_uses[live[k][0].slot] = slot_uses.get(live[k][0].slot, 0) + 1
        entries, owners = [], []
        for k, (seq, at) in live.items():
            if rng.random() < 0.2 and len(live) > 1:
                continue
            left = len(reqs[k]) - at
            n = 1 if (at > 0 and rng.random() < 0.5) else min(left, rng.randint(2, 8))
            if left - n == 1:
                n = left
            entries.append(StepEntry(seq, reqs[k][at:at + n], range(n)))
            owners.append((k, n))
        if not entries:
            continue
        logits = runner.step(entries).float().cpu()
        row = 0
        for k, n in owners:
            got[k].append(logits[row:row + n])
            row += n
            live[k][1] += n
        for k in [k for k, (seq, at) in live.items() if at == len(reqs[k])]:
            runner.cache.free(live.pop(k)[0])
        runner.cache.check_invariants()
    if tol < 1e-2:
        for k in reqs:
            assert_close(torch.cat(got[k]), want[k], tol, k)
    else:                                                        # bfloat16: the positions of all requests judged together (see assert_close)
        assert_close(torch.cat([torch.cat(got[k]) for k in reqs]), torch.cat([want[k] for k in reqs]), tol, "all requests")
    assert runner.cache.free_pages() == pages
    assert len(slot_uses) <= 4 and max(slot_uses.values()) >= 2, "no state slot was used again"
    assert sum(n - 1 for n in takes.values()) * 3 >= sum(takes.values()), "too few pages were used again"


# ---------------------------------------------------------------- configuration, registry, spec, cache needs
def test_config_reads_every_key_and_refuses_what_is_missing():
    raw = CONFIGS["mix"][0]
    assert resolve(raw).name == "Nununex" and resolve({"architectures": ["Nununex"]}).name == "Nununex"
    cfg = NununexConfig.from_dict(raw)
    assert NununexConfig.from_dict(cfg.to_dict()) == cfg and cfg.canon_taps == 4 and cfg.bigram == (89, 13, 5) and cfg.logit_softcap == 25.0
    assert cfg.layers[1].mlp.shared == 14 and cfg.layers[1].mlp.top == 2 and cfg.layers[3].mlp is None
    assert cfg.layers[2].mixer_dict()["left"]["mask"] == {"size": 7} and cfg.layers[2].mixer_dict()["right"]["gate_cap"] == 9.0
    assert NununexConfig.from_dict(CONFIGS["ones"][0]).logit_softcap is None
    for path, msg in ((("norm",), "norm"), (("canon",), "canon"), (("embedding", "bigram", "mul_prev"), "mul_prev"), (("vocab",), "vocab"),
                      (("layers", 0, "mixer", "dim"), "dim"), (("layers", 1, "mixer", "dt_rank"), "dt_rank"),
                      (("layers", 2, "mixer", "left", "scale"), "scale"), (("layers", 2, "mixer", "left", "bias_max"), "bias_max"),
                      (("layers", 2, "mixer", "right", "gate_cap"), "gate_cap"), (("layers", 1, "mlp", "expert"), "expert"),
                      (("layers", 1, "mlp", "router", "top"), "top")):
        broken = json.loads(json.dumps(raw))
        node = broken
        for p in path[:-1]:
            node = node[p]
        del node[path[-1]]
        with pytest.raises(ConfigError, match=msg):
            NununexConfig.from_dict(broken)
    for edit, msg in ((lambda c: c["layers"][0].update(type="retention"), "retention"),
                      (lambda c: c["layers"][1]["mlp"]["router"].update(top=7), "top"),
                      (lambda c: c["layers"][2]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
                      (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "conv"), (lambda c: c["canon"].update(taps=0), "taps")):
        bad = json.loads(json.dumps(raw))
        edit(bad)
        with pytest.raises(ConfigError, match=msg):
            NununexConfig.from_dict(bad)


def test_spec_and_cache_needs(dirs):
    d, cfg, page = dirs["mix"]
    _, spec = load_config(d)
    assert spec.residual == "float32" and spec.embedding_part.kind == "hashed_bigram" and spec.logit_softcap == 25.0
    assert [spec.layers[i].part("mixer").kind for i in range(4)] == ["general_delta", "selective_scan", "parallel_pair", "general_delta"]
    assert spec.layers[3].block == "gated_prenorm_mixer" and spec.layers[0].part("feed_forward").kind == "relu2_mlp"
    runner = engine(d, page, 8)
    caches = runner.cache.layer_caches
    hid, taps = 48, 4
    filt = (taps - 1) * hid
    # layer 0: the delta rule's state, then the two filters'; layer 1: scan state + its own convolution's inputs, then the filters'
    assert [s.shape[1] for s in caches[0].states] == [3 * 8 * 8, filt, filt]
    assert [s.shape[1] for s in caches[1].states] == [40 * 6 + (2 - 1) * 40, filt, filt]
    # layer 2: pages (key rows of 8, value rows of 12: a pool each) and the matrix memory's state with its normaliser column and maxima
    assert caches[2].k.shape[-1] == 8 and caches[2].v.shape[-1] == 12 and caches[2].group >= 0 and caches[0].group == -1
    assert [s.shape[1] for s in caches[2].states] == [2 * 12 * (8 + 4) + 2, filt, filt]
    assert [s.shape[1] for s in caches[3].states] == [2 * 12 * 12, filt]                 # no feed-forward: one filter
    assert caches[4].state.dtype == torch.int32 and caches[4].state.shape[1] == 1        # the embedding's previous token
    d, cfg, page = dirs["ones"]
    runner = engine(d, page, 8)
    assert [s.shape[1] for s in runner.cache.layer_caches[1].states] == [24 * 1]         # one tap everywhere: no filter state, no convolution inputs


# ---------------------------------------------------------------- the plain functions on inputs whose answer is known
def test_plain_mechanisms_by_hand():
    f64 = torch.float64
    assert torch.allclose(plain.rms(torch.tensor([[3.0, 4.0]], dtype=f64), 0.0), torch.tensor([[3.0, 4.0]], dtype=f64) / 12.5 ** 0.5)
    # the filter: the LAST column multiplies the current token
    x = torch.tensor([[1.0], [10.0], [100.0]], dtype=f64)
    assert plain.causal_conv(x, torch.tensor([[2.0, 3.0]], dtype=f64)).flatten().tolist() == [3.0, 32.0, 320.0]
    # distance rows: 8 rows, far 32: 0..3 one by one, then 4 + floor(log(n / 4) / log(8) * 4)
    assert [plain.distance_bucket(n, 8, 32) for n in (0, 3, 4, 6, 7, 11, 12, 19, 20, 31, 32, 1000)] == [0, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    # pair embedding: first token takes the last row
    w = {"embed": torch.zeros(5, 1, dtype=f64), "bigram": torch.arange(8, dtype=f64).view(8, 1)}
    e = {"bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 2}}
    assert plain.embed_with_bigram([4, 1, 3], w, e).flatten().tolist() == [7.0, (4 * 3 + 1 * 2) % 7, (1 * 3 + 3 * 2) % 7]
    # one key of score s beside the sink: weight e^s / (e^s + e^sink)
    eye = torch.eye(2, dtype=f64)
    w = {"q": eye, "k": eye, "v": eye, "o": eye, "rel": torch.tensor([[0.5], [-1.0]], dtype=f64), "sink": torch.tensor([0.7], dtype=f64)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 0.5, "bias_max": 4, "mask": {"size": 1}}
    h = torch.tensor([[1.0, 1.0], [2.0, 0.0]], dtype=f64)
    out = plain.window_attention(h, w, "", m)
    s0, s1 = 0.5 * 2.0 + 0.5, 0.5 * 4.0 + 0.5
    assert torch.allclose(out[0], h[0] * math.exp(s0) / (math.exp(s0) + math.exp(0.7)))
    assert torch.allclose(out[1], h[1] * math.exp(s1) / (math.exp(s1) + math.exp(0.7)))          # a window of one: itself only
    # the delta rule with removal 1 and no decay forgets what it held along the new key's direction
    S = torch.zeros(1, 2, 2, dtype=f64)
    k1, v1 = torch.tensor([2.0, 0.0], dtype=f64), torch.tensor([1.0, 3.0], dtype=f64)
    S = S + k1[:, None] * v1[None, :]
    u = k1 / k1.norm()
    S2 = S - u[:, None] * (u @ S[0])[None, :] + k1[:, None] * v1[None, :]
    assert torch.allclose(S2, S)                                                                 # written twice, held once
    # router: sigmoid scores, the two largest, in order; the weight multiplies the INPUT
    wr = {"router": torch.tensor([[0.0], [2.0], [1.0]], dtype=f64)}
    idx, wt = plain.route(torch.ones(1, 1, dtype=f64), wr, "", {"router": {"top": 2}})
    assert idx.tolist() == [[1, 2]] and torch.allclose(wt[0], torch.sigmoid(torch.tensor([2.0, 1.0], dtype=f64)))
    we = {"e0.gate": torch.tensor([[1.0]], dtype=f64), "e0.up": torch.tensor([[1.0]], dtype=f64), "e0.down": torch.tensor([[1.0]], dtype=f64)}
    y = plain.routed_ff(torch.ones(1, 1, dtype=f64), we, "", {"router": {"top": 1}}, choice=(torch.tensor([[0]]), torch.tensor([[0.5]], dtype=f64)))
    assert torch.allclose(y, torch.tensor([[0.5 / (1 + math.exp(-0.5)) * 0.5]], dtype=f64))      # silu(0.5) * 0.5, not 0.5 * silu(1) * 1


# ---------------------------------------------------------------- each mechanism alone (one layer)
SINGLE = {
    "delta": config(36, 67, [delta(3, 8, 4)]),
    "delta_one_head_rank_one": config(36, 67, [delta(1, 20, 1)], taps=2),
    "delta_odd": config(27, 53, [delta(3, 5, 2)], taps=1),
    "scan": config(32, 61, [scan(24, 5, 3, 3)]),
    "scan_long_filter": config(32, 61, [scan(20, 9, 2, 5)], taps=2),
    "scan_no_filter": config(27, 53, [scan(11, 3, 1, 1)], taps=1),
    "pair_window": config(32, 61, [pair(4, 2, 8, 6, 0.3, 6, 10, 5, 2, 8, 6, 6.0)]),
    "pair_whole": config(32, 61, [pair(3, 3, 8, 10, 0.4, 8, 20, None, 3, 4, 8, 3.0)], taps=2),
    "pair_far_inside_window": config(32, 61, [pair(2, 1, 16, 6, 0.25, 4, 5, 30, 1, 6, 10, 50.0)]),
    "pair_odd": config(27, 53, [pair(3, 1, 7, 5, 0.3, 5, 9, 4, 3, 5, 7, 4.0)]),
    "pair_rows64": config(48, 61, [pair(4, 2, 64, 64, 0.125, 12, 30, 20, 2, 16, 16, 8.0)]),
    "dense": config(40, 71, [delta(1, 4, 1, dense(52))]),
    "experts_shared": config(40, 71, [delta(1, 4, 1, moe(12, 3, 7, shared=9))]),
    "experts_plain": config(40, 71, [delta(1, 4, 1, moe(5, 2, 11))], taps=1),
    "experts_all": config(27, 53, [delta(1, 3, 1, moe(3, 3, 5, shared=3))]),
}


def single_dir(tmp_path, name):
    return _perturb(write_random_model(SINGLE[name], str(tmp_path), seed=3, std=0.3, norm_init="uniform"), seed=11)


@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone(tmp_path, name):
    cfg = SINGLE[name]
    d = single_dir(tmp_path, name)
    ids = tokens(cfg["vocab"], 37, seed=1)
    want = plain_logits(d, ids)
    runner = engine(d, 4, 16)
    assert err(feed(runner, "w", ids, [37]), want) < 2e-5
    assert err(feed(runner, "d", ids, [20] + [1] * 17), want) < 2e-5
    assert err(feed(runner, "p", ids, [2, 3, 2, 9, 2, 7, 5, 2, 5]), want) < 2e-5


def test_every_part_of_a_layer_matters(dirs):
    """Zeroing any one tensor of the model changes the logits: nothing that the checkpoint holds is left unused."""
    d, cfg, page = dirs["mix"]
    c0, w = plain.load_model_dir(d)
    ids = tokens(cfg["vocab"], 30, seed=2)
    want = plain.forward_logits(c0, w, ids)
    for name in w:
        if name.startswith("l") and ".mlp.e" in name and not name.startswith("l1.mlp.e0"):
            continue                                                # an expert that no token of this prompt chose changes nothing
        broken = dict(w)
        broken[name] = torch.zeros_like(w[name])
        got = plain.forward_logits(c0, broken, ids)
        if name.startswith("l1.mlp.e0"):
            continue
        assert (got - want).abs().max() > 1e-6, name


# ---------------------------------------------------------------- the engine on the stand-in kernels (CPU)
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_on_cpu(dirs, name):
    d, cfg, page = dirs[name]
    check_cuts(engine(d, page, 32), d, cfg["vocab"], 2e-5)


@pytest.mark.parametrize("name", ["mix", "pages"])
def test_mixed_batches_on_cpu(dirs, name):
    d, cfg, page = dirs[name]
    check_mixed(lambda pages: engine(d, page, pages), d, cfg["vocab"], page, 2e-5)


def test_a_batch_does_not_change_its_members(dirs):
    d, cfg, page = dirs["mix"]
    runner = engine(d, page, 64)
    a, b, c = (tokens(cfg["vocab"], n, seed=n) for n in (19, 7, 30))
    alone = [feed(runner, i, ids, [len(ids)]) for i, ids in enumerate((a, b, c))]
    seqs = [runner.cache.admit(k) for k in "abc"]
    first = runner.step([StepEntry(seqs[0], a[:10], range(10)), StepEntry(seqs[1], b, range(7)), StepEntry(seqs[2], c[:1], [0])])
    second = runner.step([StepEntry(seqs[2], c[1:], range(29)), StepEntry(seqs[0], a[10:11], [0])])
    third = runner.step([StepEntry(seqs[0], a[11:], range(8))])
    got_a = torch.cat([first[:10], second[29:30], third])
    got_c = torch.cat([first[17:18], second[:29]])
    assert err(got_a, alone[0]) < 1e-5 and err(first[10:17], alone[1]) < 1e-5 and err(got_c, alone[2]) < 1e-5


def test_a_freed_slot_starts_from_zero(dirs):
    """A request that takes the slot (and pages) another one just gave back must not see what that one left: not its states,
    not its filters' inputs, not its last token."""
    d, cfg, page = dirs["mix"]
    runner = engine(d, page, 16, max_seqs=1)
    a, b = tokens(cfg["vocab"], 26, seed=1), tokens(cfg["vocab"], 11, seed=2)
    feed(runner, "a", a, [26])
    assert err(feed(runner, "b", b, [4, 1, 1, 5]), plain_logits(d, b)) < 2e-5


def test_the_first_tokens_of_a_sequence(dirs):
    """Positions 0 .. taps: the filters and the scan's convolution see zeros before the start, the pair table gives its last row,
    the matrix memory's maximum starts at 0 and the states at zero; fed one by one and in twos."""
    for name in ("mix", "pages"):
        d, cfg, page = dirs[name]
        runner = engine(d, page, 16)
        ids = tokens(cfg["vocab"], 8, seed=9)
        want = plain_logits(d, ids)
        assert err(feed(runner, "a", ids, [1] * 8), want) < 2e-5
        assert err(feed(runner, "b", ids, [2] * 4), want) < 2e-5
        assert err(feed(runner, "c", ids[:1], [1]), want[:1]) < 2e-5


def llm_cpu(d, **kw):
    kw.setdefault("kv_cache_tokens", 512)
    return LLM(d, dtype="float32", device="cpu", ops=TorchRefOps(), **kw)


def plain_greedy(d, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(plain_logits(d, ids)[-1].argmax()))
    return ids[len(prompt):]


@pytest.mark.parametrize("chunked", [False, True])
def test_generate_through_the_entry_point_on_cpu(dirs, chunked):
    d, cfg, page = dirs["mix"]
    prompts = [tokens(cfg["vocab"], n, seed=40 + n) for n in (5, 13, 22, 9, 3)]
    want = [plain_greedy(d, p, 6) for p in prompts]
    llm = llm_cpu(d, kv_block_size=page, max_num_seqs=3, chunked_prefill=chunked, max_batched_tokens=16 if chunked else 64)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=6, ignore_eos=True))
    assert got == want
    assert llm.cache.free_pages() == llm.cache.num_pages and llm.cache.slots.num_free == 3


def test_preemption_recomputes_state(dirs):
    d, cfg, page = dirs["pages"]                                 # one of its layers sees every key: requests keep all their pages
    prompts = [tokens(cfg["vocab"], n, seed=60 + n) for n in (14, 15, 13)]
    want = [plain_greedy(d, p, 8) for p in prompts]
    llm = llm_cpu(d, kv_block_size=page, kv_cache_tokens=64, max_num_seqs=3, kv_watermark=0.0)
    assert llm.generate(prompts, SamplingParams(max_new_tokens=8, ignore_eos=True)) == want
    assert llm.scheduler.preemptions > 0


def test_trace_replay_in_process(dirs, tmp_path, monkeypatch, capsys):
    from mini_inference_b200.cli import trace_run
    d, cfg, page = dirs["pages"]
    a, b = tokens(cfg["vocab"], 9, seed=1), tokens(cfg["vocab"], 6, seed=2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:5], "want": [4]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [0, 3]}, {"id": "a", "tokens": a[5:6], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[6:], "want": [2]}], "end": ["a"]}]
    monkeypatch.setattr(sys, "stdin", io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"))
    monkeypatch.setattr("mini_inference_b200.engine.factory.make_runner",
                        lambda model, *a_, **k: make_runner(model, *a_, **{**k, "ops": TorchRefOps()}))
    assert trace_run.main(["--model", d, "--dtype", "float32", "--out", str(tmp_path), "--max-tokens", "128", "--device", "cpu",
                           "--page-size", str(page)]) == 0
    assert [line for line in capsys.readouterr().out.split("\n") if line.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = plain_logits(d, a), plain_logits(d, b)
    g0 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "0.f32"), dtype="<f4").reshape(1, -1))
    g1 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "1.f32"), dtype="<f4").reshape(3, -1))
    g2 = torch.from_numpy(np.fromfile(os.path.join(tmp_path, "2.f32"), dtype="<f4").reshape(1, -1))
    assert err(g0, wa[4:5]) < 2e-5 and err(g1, torch.stack([wb[2], wb[5], wa[5]])) < 2e-5 and err(g2, wa[8:9]) < 2e-5


# ---------------------------------------------------------------- inputs made so that a fault shows
def _i32(v, device):
    return torch.tensor(v, dtype=torch.int32, device=device)


def biased_key_case(ops, device, dtype, L, hot, window, page, rows=1, H=4, KV=2, D=24, V=16, table_rows=8, far=40):
    """L cached keys over shuffled pages; the entry feeds the last `rows` positions and the LAST query is looked at.  Every key
    is orthogonal to the query except key `hot`, whose scaled score stands out by 30.  A key that the query may see wins the
    softmax against the distance table and the sink; if `hot` lies outside the window, the visible scores are the distance
    table's entries alone and the output is sum_j e^{b_j} v_j / (sum_j e^{b_j} + e^{sink})."""
    g = torch.Generator().manual_seed(L * 1000 + hot)
    keys, vals = torch.randn(L, KV, D, generator=g) * 0.3, torch.randn(L, KV, V, generator=g)
    target = torch.randn(D, generator=g)
    target = target / target.norm()
    keys -= (keys @ target)[..., None] * target
    keys[hot] += 6.0 * target
    rel, sink = torch.randn(table_rows, H, generator=g), torch.randn(H, generator=g)
    by_distance = torch.stack([rel[plain.distance_bucket(n, table_rows, far)] for n in range(far + 1)])
    pages = -(-L // page)
    order = torch.randperm(pages, generator=g) + 1               # page 0 is the null page
    kc, vc = torch.zeros(pages + 1, KV, page, D), torch.zeros(pages + 1, KV, page, V)
    for j in range(L):
        kc[order[j // page], :, j % page], vc[order[j // page], :, j % page] = keys[j], vals[j]
    table = torch.zeros(2, pages, dtype=torch.int32)
    table[1] = order.to(torch.int32)
    tiles = [(0, r) for r in range(0, rows, 64)] if rows > 1 else []
    meta = SimpleNamespace(seg_q_start=_i32([0, rows], device), seg_pos0=_i32([L - rows], device), seg_kv_len=_i32([L], device),
                           table_rows=_i32([1], device), block_table=table.to(device), max_pages=pages, page_size=page,
                           decode_segs=_i32([0] if rows == 1 else [], device), prefill_tiles=_i32(tiles, device).view(-1, 2), tile=64, max_kv_len=L)
    q = torch.randn(rows, H, D, generator=g)
    q[-1] = 10.0 * target                                        # times the scale of 0.5: 5, times the key's 6: a score of 30
    out = ops.masked_attention(q.reshape(rows, H * D).to(device, dtype), kc.to(device, dtype), vc.to(device, dtype), meta, H, KV, D, V, 0.5,
                               None, window, True, sink_values=sink.to(device), distance_bias=by_distance.to(device)).float().cpu()[-1].view(H, V)
    p = L - 1
    lo = 0 if not window else max(0, p - window + 1)
    kvh = torch.arange(H) // (H // KV)
    if hot >= lo:
        return out, vals[hot][kvh], 2e-3                         # what is left for the others: e^{-30 + a few}
    b = torch.stack([rel[plain.distance_bucket(p - j, table_rows, far)] for j in range(lo, L)])      # [n, H]
    e = torch.exp(b)
    want = torch.einsum("jh,jhv->hv", e, vals[lo:][:, kvh]) / (e.sum(0) + torch.exp(sink))[:, None]
    return out, want, 1e-4


# (keys, the hot key, window): the first and last key inside the window and the one just outside, in the middle of a page and at a
# page's border; windows of one page, of two, of one key; no window with the key far back and at the very start; short sequences
BIASED = [(300, 0, None), (300, 299, None), (200, 104, 96), (200, 103, 96), (129, 113, 16), (129, 112, 16), (128, 96, 32), (128, 95, 32),
          (77, 76, 1), (77, 75, 1), (50, 3, 47), (50, 2, 47), (5, 0, 9), (3, 1, 2), (3, 0, 2), (1, 0, 4)]


@pytest.mark.parametrize("L,hot,window", BIASED)
@pytest.mark.parametrize("rows", [1, 3])
def test_keys_at_window_edges_with_distance_rows_and_sink_on_cpu(L, hot, window, rows):
    out, want, tol = biased_key_case(TorchRefOps(), "cpu", torch.float32, L, hot, window, page=16, rows=min(rows, L))
    assert (out - want).abs().max() < tol * want.abs().max() + 1e-6


def test_the_learned_sink_counts_once_and_unscaled():
    """One visible key with score s beside a sink of value c: the weight is e^s / (e^s + e^c) whatever the scale."""
    ops = TorchRefOps()
    k, v = torch.zeros(2, 1, 4, 2), torch.zeros(2, 1, 4, 3)
    k[1, 0, 0], v[1, 0, 0] = torch.tensor([1.0, 0.0]), torch.tensor([1.0, 2.0, 3.0])
    meta = SimpleNamespace(seg_q_start=_i32([0, 1], "cpu"), seg_pos0=_i32([0], "cpu"), seg_kv_len=_i32([1], "cpu"), table_rows=_i32([0], "cpu"),
                           block_table=_i32([[1]], "cpu"), max_pages=1, page_size=4, decode_segs=_i32([0], "cpu"),
                           prefill_tiles=_i32([], "cpu").view(-1, 2), tile=64, max_kv_len=1)
    for scale in (1.0, 0.25):
        out = ops.masked_attention(torch.tensor([[2.0, 5.0]]), k, v, meta, 1, 1, 2, 3, scale, None, None, True,
                                   sink_values=torch.tensor([0.7]), distance_bias=torch.tensor([[0.3], [9.0]]))
        s = 2.0 * scale + 0.3
        assert torch.allclose(out[0], v[1, 0, 0] * math.exp(s) / (math.exp(s) + math.exp(0.7)), rtol=1e-5)


def _segs(device, cuts_at, n, slot=1):
    return SimpleNamespace(host={"seg_q_start": [0, n], "seg_slot": [slot]}, num_segs=1, seg_q_start=_i32([0, n], device), seg_slot=_i32([slot], device),
                           positions=_i32(list(range(cuts_at, cuts_at + n)), device), token_seg=_i32([0] * n, device))


CUTS = ([401], [400, 1], [200, 150, 50, 1], [1] * 3 + [398])


def far_delta_case(ops, device):
    """Head 0 decays by 0.999 a token and must still hold a write from 400 tokens back (0.999^400 = 0.67); head 1 decays by 0.5
    and must not.  Head 2 holds it without decay until token 200 removes the key's direction with rate 1, head 3 until a removal
    along ANOTHER direction, which must leave it alone.  Whole, with the reader decoded alone, in portions, and after single tokens."""
    H, D, V, T = 4, 4, 5, 401
    HD = H * D
    prep = torch.zeros(T, 5 * HD + H * V)
    r, k, u, au, d = (prep[:, i * HD:(i + 1) * HD].view(T, H, D) for i in range(5))
    v = prep[:, 5 * HD:].view(T, H, V)
    d[:] = 1.0
    d[:, 0], d[:, 1] = 0.999, 0.5
    k[0, :, 0], v[0] = 2.0, 3.0                                   # token 0 writes key 2 e_0 with value 3
    u[200, 2, 0] = au[200, 2, 0] = 1.0                            # head 2: u = e_0, removal 1
    u[200, 3, 1] = au[200, 3, 1] = 1.0                            # head 3: u = e_1
    r[T - 1, :, 0] = 1.0                                          # the last token reads along e_0
    want = torch.tensor([6.0 * 0.999 ** 400, 0.0, 0.0, 6.0])
    for cuts in CUTS:
        state = torch.zeros(2, HD * V, device=device)
        outs, at = [], 0
        for n in cuts:
            outs.append(ops.general_delta_scan(prep[at:at + n].contiguous().to(device), H, D, V, state, _segs(device, at, n)).cpu())
            at += n
        o = torch.cat(outs)[T - 1].view(H, V)
        assert torch.allclose(o, want[:, None].expand(H, V), rtol=2e-4, atol=1e-30), (cuts, o[:, 0])


def far_memory_case(ops, device, dtype=torch.float32):
    """The matrix memory: token 0 writes with an open input gate (+cap), every later token with a closed one (-cap), and the
    forget gate stays open (log sigmoid(cap) = -e^{-cap}); 400 tokens later the read-out along the first key is still the first
    value's direction, which the per-head norm turns into v / rms(v).  Head 1's forget gate is closed (-cap): it holds only the
    latest writes, so its read-out is the LAST value's direction."""
    H, D, V, T, cap = 2, 4, 6, 401, 8.0
    g = torch.Generator().manual_seed(5)
    p = torch.zeros(T, 2 * H * D + H * V)
    q, k, v = p[:, :H * D].view(T, H, D), p[:, H * D:2 * H * D].view(T, H, D), p[:, 2 * H * D:].view(T, H, V)
    v[:] = torch.randn(T, H, V, generator=g)
    k[:, :, 1] = 1.0                                              # later tokens write along e_1 ...
    k[0], k[0, :, 0] = 0.0, 1.0                                   # ... the first along e_0
    k[T - 1, 1], k[T - 1, 1, 0] = 0.0, 1.0                        # head 1's last token writes along e_0 too and reads it back
    q[T - 1, :, 0] = 2.0
    gl = torch.zeros(T, 2 * H)
    gl[:, :H] = -100.0                                            # input gates: -cap after the soft cap ...
    gl[0, :H] = 100.0                                             # ... +cap at the first token
    gl[T - 1, 1] = 100.0
    gl[:, H], gl[:, H + 1] = 100.0, -100.0                        # forget gates: head 0 open, head 1 closed
    want = torch.stack([v[0, 0] / v[0, 0].pow(2).mean().sqrt(), v[T - 1, 1] / v[T - 1, 1].pow(2).mean().sqrt()])
    norm, gate = torch.ones(H * V), torch.full((T, H * V), 30.0)
    for cuts in CUTS:
        state = torch.zeros(2, H * D * (V + 4) + H, device=device)
        outs, at = [], 0
        for n in cuts:
            outs.append(ops.matrix_memory(p[at:at + n].contiguous().to(device, dtype), gl[at:at + n].contiguous().to(device), torch.zeros(2 * H, device=device),
                                          H, D, V, cap, 1e-6, norm.to(device), gate[at:at + n].contiguous().to(device, dtype), 0.0, state,
                                          _segs(device, at, n), dtype).float().cpu())
            at += n
        o = torch.cat(outs)[T - 1].view(H, V)
        assert torch.allclose(o, want, rtol=1e-3 if dtype == torch.float32 else 2e-2, atol=1e-3 if dtype == torch.float32 else 2e-2), (cuts, o, want)


def far_scan_case(ops, device):
    """Selective scan: channel 0 (A = -0.001) must still hold a write from 400 tokens back, channel 1 (A = -1) must not; the
    read-out is step x B C e^{400 step A} silu(z) with step = softplus(dt + bias)."""
    I, N, T = 2, 3, 401
    x, B, C = torch.zeros(T, I), torch.zeros(T, N), torch.zeros(T, N)
    x[0], B[0, 2], C[T - 1, 2] = 1.5, 2.0, 0.5
    dt, dt_b, z = torch.full((T, I), 0.2), torch.tensor([0.1, 0.1]), torch.ones(T, I)
    A, Dv = torch.tensor([[-0.001] * N, [-1.0] * N]), torch.tensor([7.0, 7.0])
    step = math.log1p(math.exp(0.3))
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    want = torch.tensor([step * 1.5 * 2.0 * 0.5 * math.exp(-0.001 * step * 400) * silu1, 0.0])
    for cuts in CUTS:
        state = torch.zeros(2, I * N, device=device)
        outs, at = [], 0
        for n in cuts:
            sl = slice(at, at + n)
            outs.append(ops.selective_scan(x[sl].contiguous().to(device), dt[sl].contiguous().to(device), dt_b.to(device), A.to(device), B[sl].contiguous().to(device),
                                           C[sl].contiguous().to(device), Dv.to(device), z[sl].contiguous().to(device), state, _segs(device, at, n),
                                           torch.float32).cpu())
            at += n
        o = torch.cat(outs)
        assert torch.allclose(o[T - 1], want, rtol=2e-4, atol=1e-30), (cuts, o[T - 1])
        assert torch.allclose(o[0], torch.tensor([(step * 1.5 * 0 + 7.0 * 1.5) * silu1] * 2), rtol=1e-5)      # C is zero there: the skip term alone


def test_recurrences_remember_a_far_token_on_cpu():
    far_delta_case(TorchRefOps(), "cpu")
    far_memory_case(TorchRefOps(), "cpu")
    far_scan_case(TorchRefOps(), "cpu")


def test_the_pair_table_reads_across_a_portions_start():
    """The row of the pair table depends on the token BEFORE a portion's first one: two prompts that differ only there must differ
    at the next position and the filters must carry the difference taps - 1 positions further, also when the portion starts there."""
    ops = TorchRefOps()
    table, pairs = torch.zeros(10, 1), torch.arange(8.0).view(8, 1)
    state = torch.zeros(3, 1, dtype=torch.int32)
    first = ops.embed_bigram_stream(_i32([4, 1], "cpu"), table, pairs, 7, 3, 2, state, _segs("cpu", 0, 2, slot=2))
    nxt = ops.embed_bigram_stream(_i32([3], "cpu"), table, pairs, 7, 3, 2, state, _segs("cpu", 2, 1, slot=2))
    assert first.flatten().tolist() == [7.0, (4 * 3 + 1 * 2) % 7] and nxt.item() == (1 * 3 + 3 * 2) % 7 and state[2, 0].item() == 3
    # large multipliers and ids: the row is computed in 64 bits
    big = ops.embed_bigram_stream(_i32([9, 9], "cpu"), table, torch.arange(1022.0).view(1022, 1), 1021, 2 ** 31 - 1, 2 ** 30 + 7, state, _segs("cpu", 5, 2, slot=1))
    assert big.flatten().tolist() == [float((0 * (2 ** 31 - 1) + 9 * (2 ** 30 + 7)) % 1021), float((9 * (2 ** 31 - 1) + 9 * (2 ** 30 + 7)) % 1021)]


# ================================================================ on the GPU
TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def cuda_ops():
    from mini_inference_b200.ops import get_ops
    return get_ops("cuda:0")


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cuts_on_gpu(dirs, name, dtype):
    d, cfg, page = dirs[name]
    check_cuts(engine(d, page, 32, dtype, "cuda:0"), d, cfg["vocab"], TOL[dtype])
    cuda_ops().check_errors()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mix", "pages"])
def test_mixed_batches_on_gpu(dirs, name, dtype):
    d, cfg, page = dirs[name]
    check_mixed(lambda pages: engine(d, page, pages, dtype, "cuda:0"), d, cfg["vocab"], page, TOL[dtype])
    cuda_ops().check_errors()


@gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_each_mechanism_alone_on_gpu(tmp_path, name, dtype):
    cfg = SINGLE[name]
    d = single_dir(tmp_path, name)
    ids = tokens(cfg["vocab"], 150, seed=1)
    want = plain_logits(d, ids)
    runner = engine(d, 16, 16, dtype, "cuda:0")
    assert_close(feed(runner, "w", ids, [150]), want, TOL[dtype], "whole")
    assert_close(feed(runner, "d", ids, [110] + [1] * 40), want, TOL[dtype], "decode")
    assert_close(feed(runner, "p", ids, [2, 64, 3, 17, 2, 33, 29]), want, TOL[dtype], "portions")
    cuda_ops().check_errors()


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("L,hot,window", BIASED + [(1500, 7, None), (1500, 476, 1024), (1500, 475, 1024), (1100, 1030, 70), (1100, 1029, 70)])
def test_keys_at_window_edges_with_distance_rows_and_sink_on_gpu(L, hot, window, dtype):
    ops = cuda_ops()
    for D, V in ((24, 16), (64, 64), (40, 72), (128, 128)):
        for rows in (1, 3, 70):
            for splits in (None, 3):
                ops.force_splits = splits
                try:
                    out, want, tol = biased_key_case(ops, "cuda:0", dtype, L, hot, window, page=16, rows=min(rows, L), D=D, V=V)
                finally:
                    ops.force_splits = None
                assert (out - want).abs().max() < (tol if dtype == torch.float32 else 2e-2) * want.abs().max() + 1e-6, (D, V, rows, splits)
    ops.check_errors()


@gpu
def test_recurrences_remember_a_far_token_on_gpu():
    far_delta_case(cuda_ops(), "cuda:0")
    far_memory_case(cuda_ops(), "cuda:0")
    far_memory_case(cuda_ops(), "cuda:0", torch.bfloat16)
    far_scan_case(cuda_ops(), "cuda:0")
    cuda_ops().check_errors()


@gpu
@pytest.mark.parametrize("lens,slots,starts", [([1, 23, 6, 2], [3, 1, 4, 2], [40, 0, 100, 0]), ([1000, 1, 59], [2, 4, 1], [0, 7, 300]),
                                               ([1, 1, 1], [2, 4, 1], [5, 0, 9])])        # single tokens only: the step kernels
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_kernels_against_the_stand_ins(dtype, lens, slots, starts):
    """Every kernel of the design alone, at sizes no model above has (odd ones too), several entries of unequal length in one
    launch, states that start non-zero and slots out of order, against the plain PyTorch statement of the same op."""
    from mini_inference_b200.parts.base import GatedDelta
    ops, ref, dev = cuda_ops(), TorchRefOps(), "cuda:0"
    g = torch.Generator().manual_seed(0)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype)      # noqa: E731
    f32 = lambda *s: torch.randn(*s, generator=g)                # noqa: E731
    close = lambda a, b, t=tol: (a.float().cpu() - b.float().cpu()).abs().max() <= t * max(1.0, b.float().abs().max().item())  # noqa: E731
    qs, T, n = [0] + list(np.cumsum(lens)), sum(lens), len(lens)
    qs = [int(v) for v in qs]
    pos = [p0 + i for p0, ln in zip(starts, lens) for i in range(ln)]
    seg = [i for i, ln in enumerate(lens) for _ in range(ln)]
    batch = SimpleNamespace(host={"seg_q_start": qs, "seg_slot": slots}, num_segs=n, positions=_i32(pos, "cpu"), token_seg=_i32(seg, "cpu"),
                            seg_q_start=_i32(qs, "cpu"), seg_slot=_i32(slots, "cpu"))
    dbatch = SimpleNamespace(num_segs=n, positions=_i32(pos, dev), token_seg=_i32(seg, dev), seg_q_start=_i32(qs, dev), seg_slot=_i32(slots, dev))
    # pair embedding: the previous token of an entry comes from its slot; position 0 takes the last row
    for hid, buckets, mp, mc in ((77, 13, 5, 3), (192, 1, 7, 2), (40, 509, 2 ** 31 - 1, 2 ** 29 + 3)):
        ids, table, pairs = torch.randint(0, 50, (T,), generator=g, dtype=torch.int32), rnd(50, hid), rnd(buckets + 1, hid)
        st = torch.randint(0, 50, (5, 1), generator=g, dtype=torch.int32)
        sa, sb = st.clone().to(dev), st.clone()
        xa = ops.embed_bigram_stream(ids.to(dev), table.to(dev), pairs.to(dev), buckets, mp, mc, sa, dbatch)
        assert close(xa, ref.embed_bigram_stream(ids, table, pairs, buckets, mp, mc, sb, batch), 1e-6) and torch.equal(sa.cpu(), sb)
    # gated addition + norm in one kernel, with and without the addend's bias, on chosen rows too
    for hid in (77, 192, 1030):
        x, y, lg, b, yb, w = f32(T, hid), rnd(T, hid), rnd(T, hid), f32(hid), f32(hid), f32(hid)
        for y_bias in (None, yb):
            xa, xb = x.clone().to(dev), x.clone()
            ra = ops.stream_rmsnorm(xa, GatedDelta(y.to(dev), lg.to(dev), b.to(dev), None if y_bias is None else y_bias.to(dev)), w.to(dev), 1e-5, None, dtype)
            rb = ref.stream_rmsnorm(xb, GatedDelta(y, lg, b, y_bias), w, 1e-5, None, dtype)
            assert close(xa, xb, 2e-6) and close(ra, rb)
        a, b2, wa, wb = rnd(T, hid), rnd(T, hid), f32(hid), f32(hid)
        assert close(ops.dual_rmsnorm_mix(a.to(dev), wa.to(dev), 0.5, b2.to(dev), wb.to(dev), 0.25, 1e-5),
                     ref.dual_rmsnorm_mix(a, wa, 0.5, b2, wb, 0.25, 1e-5))
        z = rnd(T, hid)
        for act in ("none", "relu2"):
            assert close(ops.bias_act(z.to(dev), b.to(dev), act), ref.bias_act(z, b, act))
    lo = f32(7, 131) * 40
    assert close(ops.softcap(lo.clone().to(dev), 25.0), ref.softcap(lo, 25.0), 1e-6)
    # the filter: one to five taps, a strided view as input, the state behind an offset, with and without bias, activation, residual
    # (rows that start on a 16-byte boundary with channels in eights take the kernel that moves eight channels a thread)
    for C, taps, off, lead, more in ((48, 4, 0, 4, 9), (48, 4, 0, 8, 8), (77, 2, 5, 4, 9), (192, 3, 192 * 7, 4, 9), (192, 3, 192 * 7, 16, 16), (33, 5, 1, 4, 9),
                                     (20, 1, 0, 4, 9), (2048, 2, 8, 0, 0), (40, 1, 0, 8, 8), (64, 5, 4, 0, 8)):
        wide, w, b = rnd(T, C + more), f32(C, taps), f32(C)
        st = f32(5, off + (taps - 1) * C + (4 if lead % 8 == 0 else 3))
        for bias, residual, act in ((None, True, "none"), (b, False, "silu"), (b, True, "none")):
            sa, sb = st.clone().to(dev), st.clone()
            ya = ops.short_conv(wide.to(dev)[:, lead:lead + C], w.to(dev), None if bias is None else bias.to(dev), taps, sa, off, dbatch, residual, act)
            yb = ref.short_conv(wide[:, lead:lead + C], w, bias, taps, sb, off, batch, residual, act)
            assert close(ya, yb) and close(sa, sb, 1e-6), (C, taps, lead)
    # the general delta rule
    for H, D, V, rank in ((3, 8, 8, 5), (1, 20, 20, 1), (2, 64, 64, 16), (3, 5, 5, 2), (2, 33, 33, 7), (1, 128, 128, 32)):
        HD = H * D
        p, w2, w0, ab = rnd(T, 3 * HD + 2 * H * V + rank + 5), rnd(HD, rank), f32(HD), f32(HD)
        pa = ops.general_delta_prepare(p.to(dev), w2.to(dev), w0.to(dev), ab.to(dev), H, D, V, rank, 0.6, 1e-6)
        pb = ref.general_delta_prepare(p, w2, w0, ab, H, D, V, rank, 0.6, 1e-6)
        assert close(pa[:, :pb.shape[1]], pb, 1e-5 if dtype == torch.float32 else tol)
        st = f32(5, HD * V + 2) * 0.3
        sa, sb = st.clone().to(dev), st.clone()
        oa = ops.general_delta_scan(pa, H, D, V, sa, dbatch)
        ob = ref.general_delta_scan(pa.cpu()[:, :pb.shape[1]], H, D, V, sb, batch)
        assert close(oa, ob, 1e-4) and close(sa, sb, 1e-4), (H, D)
    # the matrix memory, with and without the gates' cap
    for H, D, V, cap in ((2, 12, 8, 9.0), (1, 16, 20, 2.0), (4, 48, 48, 12.0), (3, 5, 7, None), (2, 64, 128, 15.0), (1, 128, 64, 30.0)):
        p, gl, gb = rnd(T, 2 * H * D + H * V + 3), f32(T, 2 * H) * 3, f32(2 * H)
        norm, gate = f32(H * V), rnd(T, H * V + 6)
        st = torch.zeros(5, H * D * (V + 4) + H)
        st[:, :H * D * (V + 4)] = f32(5, H * D * (V + 4)) * 0.2
        st[:, H * D * (V + 4):] = torch.rand(5, H, generator=g) * 2
        sa, sb = st.clone().to(dev), st.clone()
        ya = ops.matrix_memory(p.to(dev), gl.to(dev), gb.to(dev), H, D, V, cap, 1e-6, norm.to(dev), gate.to(dev)[:, 3:3 + H * V], 1e-5, sa, dbatch, dtype)
        yb = ref.matrix_memory(p, gl, gb, H, D, V, cap, 1e-6, norm, gate[:, 3:3 + H * V], 1e-5, sb, batch, dtype)
        W = V + 4
        keep = torch.zeros(H, D, W, dtype=torch.bool)
        keep[:, :, :V + 1] = True                               # the three unused columns of a row are not compared
        keep = torch.cat([keep.flatten(), torch.ones(H, dtype=torch.bool)])
        assert close(ya, yb, 2e-4 if dtype == torch.float32 else 3e-2) and close(sa.cpu()[:, keep], sb[:, keep], 1e-4), (H, D, V)
    # the selective scan
    for I, N in ((40, 6), (24, 1), (256, 24), (11, 3), (300, 16), (64, 33)):
        x, dt, dtb, A = rnd(T, I), f32(T, I), f32(I), -torch.rand(I, N, generator=g) * 2
        BC, Dv, z = rnd(T, 2 * N + 5), f32(I), rnd(T, I + 3)
        st = f32(5, I * N + 4) * 0.3
        sa, sb = st.clone().to(dev), st.clone()
        ya = ops.selective_scan(x.to(dev), dt.to(dev), dtb.to(dev), A.to(dev), BC.to(dev)[:, 2:2 + N], BC.to(dev)[:, 2 + N:2 + 2 * N], Dv.to(dev),
                                z.to(dev)[:, 3:], sa, dbatch, dtype)
        yb = ref.selective_scan(x, dt, dtb, A, BC[:, 2:2 + N], BC[:, 2 + N:2 + 2 * N], Dv, z[:, 3:], sb, batch, dtype)
        assert close(ya, yb, 1e-4 if dtype == torch.float32 else tol) and close(sa, sb, 1e-4), (I, N)
    # sigmoid router with rider rows; experts weighted on their input, the shared expert gated
    for T2, hid, E, top, F, extra in ((13, 44, 6, 2, 10, 1), (70, 128, 16, 5, 64, 0), (5, 33, 7, 7, 9, 1), (40, 64, 8, 1, 64, 1), (900, 192, 8, 1, 128, 1)):
        h, router = rnd(T2, hid), rnd(E + extra, hid) * 0.5
        ca, wa, ea = ops.route_topk(h.to(dev), router.to(dev), None, top, None, score="sigmoid", extra_rows=extra)
        cb, wb, eb = ref.route_topk(h, router, None, top, None, score="sigmoid", extra_rows=extra)
        assert torch.equal(ca.cpu(), cb) and close(wa, wb, 1e-5) and (extra == 0 or close(ea, eb, 1e-4))
        w_in, w_out, shared = rnd(E, 2 * F, hid) * 0.3, rnd(E, hid, F) * 0.3, rnd(T2, hid)
        for sh, sg in ((None, None), (shared, None), (shared, eb)):
            if sh is not None and sg is None and extra:
                continue
            for tc, tc5 in (((False, False), (True, False), (True, True)) if dtype == torch.bfloat16 else ((False, False),)):
                keep = (ops.moe_tc, ops.moe_tcgen05)
                ops.moe_tc, ops.moe_tcgen05 = tc and keep[0], tc5 and keep[1]
                try:
                    got = ops.expert_ffn(h.to(dev), ca, wa, w_in.to(dev), w_out.to(dev), 1e30, 1.0, None if sh is None else sh.to(dev), up_shift=0.0,
                                         weight_on_input=True, shared_gate=None if sg is None else ea)
                finally:
                    ops.moe_tc, ops.moe_tcgen05 = keep
                assert close(got, ref.expert_ffn(h, cb, wb, w_in, w_out, 1e30, 1.0, sh, up_shift=0.0, weight_on_input=True, shared_gate=sg)), (T2, tc, tc5)
    ops.check_errors()


def plain_judged(d, prompts, got):
    """Generated tokens judged by the plain logits: each is within a rounding's reach of the largest, but for the one in six
    that a router's near tie may send through another expert than the plain implementation's (see assert_close)."""
    far, total = 0, 0
    for p, out in zip(prompts, got):
        logits = plain_logits(d, p + out)
        for i, tok in enumerate(out):
            row = logits[len(p) + i - 1]
            far += int(row[tok] < row.max() - 0.12 * row.abs().max())
            total += 1
    assert far * 6 <= total, (far, total)


@gpu
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generate_through_the_entry_point_on_gpu(dirs, dtype, graphs):
    d, cfg, page = dirs["mix"]
    prompts = [tokens(cfg["vocab"], n, seed=40 + n) for n in (5, 13, 22, 9, 3, 30)]
    llm = LLM(d, dtype=dtype, kv_block_size=page, kv_cache_tokens=1024, max_num_seqs=4, cuda_graphs=graphs)
    got = llm.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    assert llm.cache.free_pages() == llm.cache.num_pages
    if graphs:
        assert llm.graphs.replays > 0
    if dtype == "float32":
        assert got == [plain_greedy(d, p, 12) for p in prompts]
    else:
        plain_judged(d, prompts, got)


@gpu
def test_long_decoding_on_gpu(dirs):
    """300 tokens generated one by one after a short prompt, through the scheduler: every window slides past the prompt, pages
    fill and new ones are taken, and the plain implementation agrees on the whole sequence at the end."""
    d, cfg, page = dirs["pages"]
    prompt = tokens(cfg["vocab"], 11, seed=77)
    llm = LLM(d, dtype="float32", kv_block_size=page, kv_cache_tokens=512, max_num_seqs=2)
    out = llm.generate([prompt], SamplingParams(max_new_tokens=300, ignore_eos=True))[0]
    logits = plain_logits(d, prompt + out)
    picks = logits[len(prompt) - 1:-1].argmax(-1).tolist()
    assert sum(a == b for a, b in zip(picks, out)) >= 297          # a near tie may fall the other way; it does not derail the rest


@gpu
def test_trace_run_program_on_gpu(dirs, tmp_path):
    d, cfg, page = dirs["pages"]
    a = tokens(cfg["vocab"], 70, seed=5)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:64], "want": [0, 63]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[64:], "want": [5]}], "end": ["a"]}]
    for dtype in ("float32", "bfloat16"):
        out = tmp_path / dtype
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", str(out), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        want = plain_logits(d, a)
        g0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
        g1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1))
        assert_close(torch.cat([g0, g1]), want[[0, 63, 69]], TOL[dtype])
