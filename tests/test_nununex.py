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
    for k in reqs:
        assert_close(torch.cat(got[k]), want[k], tol, k)
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
