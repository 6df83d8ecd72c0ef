"""Microbenchmarks of the decode step's bandwidth-bound kernels, in the manner of the
reference's bench/micro/bench_gemm.py (:35-170: every linear of a model at a few row counts,
ms, GB/s and share of peak, rotating weight copies to defeat the L2) and
bench/micro/bench_attention.py (:61-167: paged decode attention over batch x context).

    python -m mini_inference_b200.cli.microbench gemm      [--rows 1,8,64] [--size 4b]
    python -m mini_inference_b200.cli.microbench attention [--batch 1,8,64] [--ctx 4096]
    python -m mini_inference_b200.cli.microbench prefill   [--tokens 2048] [--ctx-before 0]
    python -m mini_inference_b200.cli.microbench design    [--design-size 2k|4k]   (the Naditar kernels beside Qwen3's)
    python -m mini_inference_b200.cli.microbench namesun   [--design-size 2k|4k]   (the Namesun kernels beside Qwen3's)

Each line: kernel, shape, microseconds (CUDA events, after warm-up), GB/s of the bytes the
kernel has to read, and that as a share of the measured copy bandwidth."""
from __future__ import annotations

import argparse
import json
import os
import sys
import types

import torch

from .run_engine import SIZES


def peak_gbs():
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(here, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f)["hbm_gbs"], "measured"
    return 6650.0, "fallback"


def timed(fn, iters, warmup=3):
    """Microseconds per call.  The calls are recorded into one CUDA graph (fn(i) for i in
    range(iters), each on different operands) and the graph is replayed, so the figure is the
    kernels' time on the device, not the host's launch cost."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for i in range(warmup):
            fn(i)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fn(i)
    graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e3 / iters


def bench_gemm(args, ops, peak):
    cfg = SIZES[args.size]
    h, H, KV, D, I, V = (cfg["hidden_size"], cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"],
                         cfg["intermediate_size"], cfg["vocab_size"])
    shapes = [("qkv", (H + 2 * KV) * D, h), ("o", h, H * D), ("gate_up", 2 * I, h), ("down", h, I), ("lm_head", V, h)]
    for name, N, K in shapes:
        if args.only and name not in args.only:
            continue
        copies = max(2, -(-args.rotate_mb * 2 ** 20 // (N * K * 2)))      # rotate >= rotate_mb of weights
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        for M in args.rows:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            od = torch.float32 if name == "lm_head" else None
            ops.skinny_max_rows, ops.skinny_max_cols = 64, 1 << 30
            for label, stream, skinny, tc in (("stream", True, False, False), ("skinny", False, True, False),
                                              ("tcgen05 x2", False, False, True), ("library", False, False, False)):
                ops.stream_gemm, ops.skinny_gemm, ops.tc_gemm = stream, skinny, tc
                if (stream and M > 32) or (skinny and M > 64) or (tc and (M < 128 or od is not None)):
                    continue
                us = timed(lambda i: ops.linear(x, ws[i % copies], out_dtype=od), args.iters)
                gbs = N * K * 2 / us / 1e3
                tf = 2.0 * M * N * K / us / 1e6
                print(f"gemm {name:8s} M={M:<4d} N={N:<6d} K={K:<5d} {label:10s} {us:9.2f} us {gbs:8.1f} GB/s "
                      f"{100 * gbs / peak:5.1f} % of peak bandwidth {tf:8.1f} TFLOP/s", flush=True)
            ops.stream_gemm = ops.skinny_gemm = True
            ops.tc_gemm = False
        del ws


def bench_attention(args, ops, peak):
    cfg = SIZES[args.size]
    H, KV, D, ps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], args.page_size
    for B in args.batch:
        pages_per_seq = -(-args.ctx // ps)
        layers = max(2, -(-args.rotate_mb * 2 ** 20 // (B * pages_per_seq * ps * KV * D * 4)))
        num_pages = B * pages_per_seq
        kv = torch.randn(layers, 2, num_pages + 1, KV, ps, D, device="cuda", dtype=torch.bfloat16)
        perm = torch.randperm(num_pages, device="cuda").to(torch.int32) + 1
        table = perm.view(B, pages_per_seq).contiguous()
        ar = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        meta = types.SimpleNamespace(
            page_size=ps, tile=64, block_table=table, max_pages=pages_per_seq, seg_q_start=ar,
            seg_pos0=torch.full((B,), args.ctx - 1, dtype=torch.int32, device="cuda"),
            seg_kv_len=torch.full((B,), args.ctx, dtype=torch.int32, device="cuda"), decode_segs=ar[:B],
            table_rows=None, prefill_tiles=torch.zeros((0, 2), dtype=torch.int32, device="cuda"), prefill_tiles2=None,
            max_kv_len=args.ctx, num_tokens=B)
        q = torch.randn(B, H * D, device="cuda", dtype=torch.bfloat16)
        for label, flag in (("tensor-core", True), ("generic", False)):
            for splits in (args.splits or [None]):
                if splits and not flag:
                    continue
                ops.fast_attention, ops.force_splits = flag, splits
                us = timed(lambda i: ops.paged_attention(q, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D,
                                                         D ** -0.5, None), args.iters)
                gbs = B * args.ctx * KV * D * 4 / us / 1e3
                print(f"decode attention B={B:<3d} ctx={args.ctx} heads {H}/{KV} D={D} {label:12s} "
                      f"{'splits ' + str(splits) if splits else 'splits chosen'} {us:9.2f} us {gbs:8.1f} GB/s {100 * gbs / peak:5.1f} % of peak",
                      flush=True)
        ops.fast_attention, ops.force_splits = True, None
        del kv


def bench_prefill_attention(args, ops, peak):
    """Prompt attention over the pages: one request of --tokens tokens whose first token is at position --ctx-before
    (a later portion of a long prompt when that is not 0), causal; TFLOP/s of the scores and weighted sums that count."""
    import numpy as np
    cfg = SIZES[args.size]
    H, KV, D, ps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], args.page_size
    T, p0 = args.tokens, args.ctx_before
    pages_per_seq = -(-(p0 + T) // ps)
    layers = max(2, -(-args.rotate_mb * 2 ** 20 // (pages_per_seq * ps * KV * D * 4)))
    kv = torch.randn(layers, 2, pages_per_seq + 1, KV, ps, D, device="cuda", dtype=torch.bfloat16)
    table = (torch.randperm(pages_per_seq, device="cuda").to(torch.int32) + 1).view(1, pages_per_seq).contiguous()
    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device="cuda")
    meta = types.SimpleNamespace(
        page_size=ps, tile=64, block_table=table, table_rows=None, max_pages=pages_per_seq, seg_q_start=t([0, T]), seg_pos0=t([p0]),
        seg_kv_len=t([p0 + T]), decode_segs=t([]), prefill_tiles=t([(0, r) for r in range(0, T, 64)]).view(-1, 2),
        prefill_tiles2=t([(0, r) for r in range(0, T, 128)]).view(-1, 2), max_kv_len=p0 + T, num_tokens=T)
    q = torch.randn(T, H * D, device="cuda", dtype=torch.bfloat16)
    flops = 4.0 * H * D * (T * p0 + T * (T + 1) / 2)
    for label, tc, fast in (("tcgen05", True, True), ("mma.sync", False, True)):
        ops.tc_attention, ops.fast_attention = tc, fast
        us = timed(lambda i: ops.paged_attention(q, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D, D ** -0.5, None), args.iters)
        print(f"prompt attention T={T} from position {p0} heads {H}/{KV} D={D} page {ps} {label:9s} {us:9.2f} us "
              f"{flops / us / 1e6:8.1f} TFLOP/s", flush=True)
        if tc and hasattr(ops.lib, "mi_attn_tc_timing"):
            # a library built with MI_NVCC_EXTRA=-DMI_ATT_TIMING counts clocks of one softmax thread per block and key tile
            import ctypes
            ticks = (ctypes.c_ulonglong * 16)()
            ops.lib.mi_attn_tc_timing(ticks, 1)
            ops.paged_attention(q, kv[0, 0], kv[0, 1], meta, H, KV, D, D ** -0.5, None)
            torch.cuda.synchronize()
            ops.lib.mi_attn_tc_timing(ticks, 1)
            n = max(1, ticks[3])
            print(f"  softmax thread, clocks per 64-key tile over {n} tiles: wait for scores {ticks[0] / n:.0f}, "
                  f"maximum + exponentials + P store {ticks[1] / n:.0f}, wait for the previous PV + hand-over {ticks[2] / n:.0f}", flush=True)
            print(f"  MMA thread, clocks per tile: wait for the next keys + issue of their scores {ticks[4] / n:.0f}, wait for P {ticks[5] / n:.0f}, "
                  f"wait for the values {ticks[6] / n:.0f}", flush=True)
            print(f"  of the middle part: score load {ticks[8] / n:.0f}, mask + maximum {ticks[9] / n:.0f}, exponentials + sums + packing {ticks[10] / n:.0f}, "
                  f"P store {ticks[11] / n:.0f}", flush=True)
    ops.tc_attention = ops.fast_attention = True
    ops.check_errors()


# ---------------------------------------------------------------- the kernels of the Naditar design beside their Qwen3 counterparts
NADITAR_SIZES = {
    # width, feed-forward, heads and head sizes in the range of 1-3 B and 7-8 B parameter models; the latent rows have 128 entries
    "2k": dict(width=2048, ff=8192, heads=16, kv_heads=8, dim=128, vdim=128, conv=4, rank=64, l_heads=16, l_dim=64, l_rot=32, l_rank=96, l_vdim=64),
    "4k": dict(width=4096, ff=12288, heads=32, kv_heads=16, dim=128, vdim=128, conv=4, rank=128, l_heads=16, l_dim=128, l_rot=32, l_rank=96, l_vdim=128),
}


def naditar_config(size, layers, vocab=65536):
    z = NADITAR_SIZES[size]
    ff = {"kind": "dense", "ff": z["ff"]}
    delta = {"type": "channel_delta", "mlp": ff, "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                                                           "conv": z["conv"], "decay_rank": z["rank"], "gate_rank": z["rank"]}}
    light = {"type": "lightning", "mlp": ff, "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"],
                                                       "decay": [1.0 - 2.0 ** -(2 + 6 * h / z["heads"]) for h in range(z["heads"])]}}
    lat = {"type": "latent_attention", "mlp": ff,
           "mixer": {"heads": z["l_heads"], "dim": z["l_dim"], "rot_dim": z["l_rot"], "vdim": z["l_vdim"], "kv_rank": z["l_rank"],
                     "scale": (z["l_dim"] + z["l_rot"]) ** -0.5, "rot": {"base": 1e6, "dims": z["l_rot"]}}}
    pattern = [delta, delta, lat, light]
    return {"architecture": "Naditar", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6},
            "layers": [pattern[i % 4] for i in range(layers)]}


def qwen3_config_like(size, layers, vocab=65536):
    """Qwen3 dense of the same width, depth and vocabulary; its three feed-forward matrices hold what Naditar's two do."""
    z = NADITAR_SIZES[size]
    return {"architectures": ["Qwen3ForCausalLM"], "hidden_size": z["width"], "num_hidden_layers": layers, "num_attention_heads": z["heads"],
            "num_key_value_heads": z["kv_heads"], "head_dim": 128, "intermediate_size": z["ff"] * 2 // 3 // 128 * 128, "vocab_size": vocab,
            "rope_theta": 1e6, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 40960}


def bench_design(args, ops, peak, out=print):
    """Each new kernel at the layer sizes of --design-size, with the bytes or operations it cannot avoid and that as a share
    of the bound it is up against: the measured copy bandwidth, the measured bf16 tensor peak, or (float32 recurrences and
    float32 attention weights, which the design prescribes) the float32 FMA rate of the CUDA cores, SMs x 128 x 2 x clock."""
    import numpy as np
    z = NADITAR_SIZES[args.design_size]
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    bf16_peak = 1590.0
    if os.path.isfile(os.path.join(here, "MEASURED_PEAKS.json")):
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            bf16_peak = json.load(f)["bf16_tflops"]
    props = torch.cuda.get_device_properties(0)
    fma_peak = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12             # TFLOP/s at the maximum SM clock
    rows = []

    def line(kernel, shape, us, amount, bound):
        if bound == "hbm":
            got, top, unit = amount / us / 1e3, peak, "GB/s"
        elif bound == "bf16":
            got, top, unit = amount / us / 1e6, bf16_peak, "TFLOP/s"
        else:
            got, top, unit = amount / us / 1e6, fma_peak, "TFLOP/s (fp32 FMA)"
        rows.append({"kernel": kernel, "shape": shape, "us": round(us, 2), "achieved": round(got, 1), "unit": unit, "frac": round(got / top, 3)})
        out(f"{kernel:34s} {shape:38s} {us:9.2f} us {got:9.1f} {unit:20s} {100 * got / top:5.1f} % of bound", flush=True)

    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device="cuda")       # noqa: E731
    bf = torch.bfloat16
    W, FF, H, KV, D, V, taps = z["width"], z["ff"], z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["conv"]
    T, it = args.tokens, args.iters
    # ---- stream kernels (prompt step of T tokens)
    x = torch.randn(4, T, W, device="cuda")
    dl = torch.randn(4, T, W, device="cuda", dtype=bf)
    g1 = torch.ones(1, device="cuda")
    us = timed(lambda i: ops.add_scaled_rmsnorm(x[i % 4], dl[i % 4], g1, 1e-6, None, None, bf), it)
    line("add + scalar rmsnorm (f32 stream)", f"T={T} width={W}", us, T * W * 12.0, "hbm")
    xb, wn = torch.randn(4, T, W, device="cuda", dtype=bf), torch.ones(W, device="cuda", dtype=bf)
    us = timed(lambda i: ops.add_rmsnorm(xb[i % 4], dl[i % 4], wn, 1e-6), it)
    line("  Qwen3: add + rmsnorm (bf16 stream)", f"T={T} width={W}", us, T * W * 8.0, "hbm")
    zz, coef = torch.randn(4, T, FF, device="cuda", dtype=bf), torch.tensor([0.5, 0.3, 0.2, 0.1], device="cuda")
    us = timed(lambda i: ops.polynorm(zz[i % 4], coef, 1e-6), it)
    line("polynorm activation", f"T={T} ff={FF}", us, T * FF * 4.0, "hbm")
    inter = FF * 2 // 3 // 128 * 128
    gu = torch.randn(4, T, 2 * inter, device="cuda", dtype=bf)
    us = timed(lambda i: ops.swiglu(gu[i % 4]), it)
    line("  Qwen3: swiglu", f"T={T} inter={inter}", us, T * inter * 6.0, "hbm")
    # ---- recurrences: one prompt of T tokens; decode steps of B requests
    for B, n in ((1, T), (8, 1), (64, 1)):
        rows_n = B * n
        batch = types.SimpleNamespace(seg_q_start=t(np.arange(B + 1) * n), seg_slot=t(np.arange(B) + 1), num_segs=B,
                                      token_seg=t(np.repeat(np.arange(B), n)))
        kind = "prompt" if n > 1 else "decode"
        shape = f"{kind} B={B} T={n} heads={H} {D}x{V}"
        reps = 4 if n > 1 else max(2, (256 << 20) // (B * H * D * V * 4) + 1)      # decode: rotate through more states than the L2 holds
        p = torch.randn(rows_n, 2 * H * D + 2 * H * V, device="cuda", dtype=bf)
        decay = torch.full((H,), 0.99, device="cuda")
        st = torch.zeros(reps, B + 1, H * D * V, device="cuda")
        us = timed(lambda i: ops.lightning_scan(p, H, D, V, decay, st[i % reps], batch), it)
        if n > 1:
            line("lightning scan", shape, us, 4.0 * H * D * V * rows_n, "fma")
        else:
            line("lightning scan", shape, us, 8.0 * B * H * D * V, "hbm")
        C = 2 * KV * D + H * V
        pd, a = torch.randn(rows_n, C + H + 2 * z["rank"], device="cuda", dtype=bf), torch.randn(rows_n, H * D, device="cuda", dtype=bf)
        conv, A_log, dtb = torch.randn(C, taps, device="cuda") * 0.3, torch.zeros(H, device="cuda"), torch.zeros(H * D, device="cuda")
        st2 = torch.zeros(reps, B + 1, H * D * V + (taps - 1) * C, device="cuda")
        prep = ops.delta_prepare(pd, a, conv, A_log, dtb, H, KV, D, V, taps, 1e-6, st2[0], batch)
        us = timed(lambda i: ops.delta_prepare(pd, a, conv, A_log, dtb, H, KV, D, V, taps, 1e-6, st2[i % reps], batch), it)
        line("delta rule: conv, norms, decay", shape, us, rows_n * (2.0 * (C + H + H * D) + 4.0 * (C + H + H * D)), "hbm")
        us = timed(lambda i: ops.delta_scan(prep, H, KV, D, V, st2[i % reps], batch), it)
        if n > 1:
            line("delta rule scan", shape, us, 8.0 * H * D * V * rows_n, "fma")
        else:
            line("delta rule scan", shape, us, 8.0 * B * H * D * V, "hbm")
        del st, st2
    # ---- latent attention beside grouped-query attention
    LH, C, R, ps = z["l_heads"], z["l_rank"], z["l_rot"], 16
    pages = -(-T // ps)
    table = (torch.randperm(pages, device="cuda").to(torch.int32) + 1).view(1, pages).contiguous()
    tiles = dict(prefill_tiles=t([(0, r) for r in range(0, T, 64)]).view(-1, 2), prefill_tiles2=t([(0, r) for r in range(0, T, 128)]).view(-1, 2))
    meta = types.SimpleNamespace(page_size=ps, tile=64, block_table=table, table_rows=t([0]), max_pages=pages, seg_q_start=t([0, T]), seg_pos0=t([0]),
                                 seg_kv_len=t([T]), decode_segs=t([]), max_kv_len=T, num_tokens=T, **tiles)
    cache = torch.randn(4, pages + 1, 1, ps, C + R, device="cuda", dtype=bf)
    q = torch.randn(T, LH, C + R, device="cuda", dtype=bf)
    pairs = T * (T + 1) / 2
    # default: mma.sync kernels with every softmax weight as two bfloat16 numbers; MI_LATENT_TC=1: tcgen05 / mma kernels, bfloat16 weights;
    # the float32 kernels of csrc/attention_latent.cu (any row size) are timed on a shorter prompt
    for label, tc, fast in (("split weights", False, True), ("bf16 weights", True, True), ("float32 kernel", False, False)):
        ops.latent_tc, ops.fast_attention = tc, fast
        us = timed(lambda i: ops.latent_attention(q, cache[i % 4], meta, LH, C, R, 0.1), it if fast else 3)
        line(f"latent attention, {label}", f"prompt T={T} heads={LH} rows {C}+{R}", us, 2.0 * LH * (2 * C + R) * pairs, "bf16" if fast else "fma")
    ops.fast_attention = True
    kv = torch.randn(4, 2, pages + 1, KV, ps, 128, device="cuda", dtype=bf)
    qq = torch.randn(T, H * 128, device="cuda", dtype=bf)
    meta.table_rows = None
    us = timed(lambda i: ops.paged_attention(qq, kv[i % 4, 0], kv[i % 4, 1], meta, H, KV, 128, 0.1, None), it)
    line("  Qwen3: attention", f"prompt T={T} heads={H}/{KV} D=128", us, 4.0 * H * 128 * pairs, "bf16")
    ctx = args.ctx
    pages = -(-ctx // ps)
    for B in (8, 64):
        layers = max(2, (512 << 20) // (B * pages * ps * (C + R) * 2) + 1)
        table = (torch.stack([torch.randperm(pages, device="cuda") for _ in range(B)]) + 1 + (torch.arange(B, device="cuda") * pages)[:, None]).to(torch.int32)
        ar = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        meta = types.SimpleNamespace(page_size=ps, tile=64, block_table=table.contiguous(), table_rows=ar[:B].contiguous(), max_pages=pages, seg_q_start=ar,
                                     seg_pos0=torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda"),
                                     seg_kv_len=torch.full((B,), ctx, dtype=torch.int32, device="cuda"), decode_segs=ar[:B].contiguous(),
                                     prefill_tiles=torch.zeros((0, 2), dtype=torch.int32, device="cuda"), prefill_tiles2=None, max_kv_len=ctx, num_tokens=B)
        cache = torch.randn(layers, B * pages + 1, 1, ps, C + R, device="cuda", dtype=bf)
        q = torch.randn(B, LH, C + R, device="cuda", dtype=bf)
        for label, tc, fast in (("split weights", False, True), ("bf16 weights", True, True), ("float32 kernel", False, False)):
            ops.latent_tc, ops.fast_attention = tc, fast
            us = timed(lambda i: ops.latent_attention(q, cache[i % layers], meta, LH, C, R, 0.1), it if fast else 3)
            line(f"latent attention, {label}", f"decode B={B} ctx={ctx} heads={LH} rows {C}+{R}", us, B * ctx * (C + R) * 2.0, "hbm")
        ops.fast_attention = True
        del cache
        layers = max(2, (512 << 20) // (B * pages * ps * KV * 128 * 4) + 1)
        kv = torch.randn(layers, 2, B * pages + 1, KV, ps, 128, device="cuda", dtype=bf)
        qq = torch.randn(B, H * 128, device="cuda", dtype=bf)
        meta.table_rows = None
        us = timed(lambda i: ops.paged_attention(qq, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, 128, 0.1, None), it)
        line("  Qwen3: attention", f"decode B={B} ctx={ctx} heads={H}/{KV} D=128", us, B * ctx * KV * 128 * 4.0, "hbm")
        del kv
    ops.latent_tc, ops.fast_attention = False, True
    ops.check_errors()
    return rows


NAMESUN_SIZES = {
    # width, heads, head sizes and active feed-forward parameters per token in the range of 1-3 B and 7-8 B active-parameter models
    "2k": dict(width=2048, ff=8192, heads=16, kv_heads=8, dim=128, vdim=128, block=1024, experts=32, top=4, eff=1024, shared=2048, groups=(8, 4)),
    "4k": dict(width=4096, ff=12288, heads=32, kv_heads=8, dim=128, vdim=128, block=1024, experts=64, top=6, eff=1536, shared=3072, groups=(8, 4)),
}


def namesun_config(size, layers, vocab=65536):
    z = NAMESUN_SIZES[size]
    experts = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}},
               "expert": {"ff": z["eff"], "limit": 7.0}, "shared": {"ff": z["shared"], "limit": 7.0}}
    ret = {"type": "retention", "mixer": {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "rot": {"dims": z["dim"], "base": 1e6},
                                          "decay": [1.0 - 2.0 ** -(2 + 6 * h / z["heads"]) for h in range(z["heads"])]}}
    att = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5 * 8,
                                          "mask": {"size": z["block"]}, "v_mix": True}}
    pattern = [dict(ret, mlp={"kind": "dense", "ff": z["ff"]}), dict(ret, mlp=experts), dict(att, mlp=experts), dict(ret, mlp=experts)]
    return {"architecture": "Namesun", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.3,
            "layers": [pattern[i % 4] if i else pattern[0] for i in range(layers)]}


def qwen3_config_like_namesun(size, layers, vocab=65536):
    """Qwen3 dense of the same width, depth, vocabulary and heads; its feed-forward holds what a Namesun token uses (top experts + shared)."""
    z = NAMESUN_SIZES[size]
    return {"architectures": ["Qwen3ForCausalLM"], "hidden_size": z["width"], "num_hidden_layers": layers, "num_attention_heads": z["heads"],
            "num_key_value_heads": z["kv_heads"], "head_dim": 128, "intermediate_size": z["top"] * z["eff"] + z["shared"], "vocab_size": vocab,
            "rope_theta": 1e6, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 40960}


def bench_namesun(args, ops, peak, out=print):
    """Each kernel of the Namesun design at the layer sizes of --design-size beside the like kernel of Qwen3 dense, with the bytes
    or operations it cannot avoid as a share of its bound (measured copy bandwidth, measured bf16 tensor peak, or, for the
    float32 recurrence, the float32 FMA rate of the CUDA cores)."""
    import numpy as np
    z = NAMESUN_SIZES[args.design_size]
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    bf16_peak = 1590.0
    if os.path.isfile(os.path.join(here, "MEASURED_PEAKS.json")):
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            bf16_peak = json.load(f)["bf16_tflops"]
    props = torch.cuda.get_device_properties(0)
    fma_peak = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    rows = []

    def line(kernel, shape, us, amount, bound):
        got, top, unit = {"hbm": (amount / us / 1e3, peak, "GB/s"), "bf16": (amount / us / 1e6, bf16_peak, "TFLOP/s"),
                          "fma": (amount / us / 1e6, fma_peak, "TFLOP/s (fp32 FMA)")}[bound]
        rows.append({"kernel": kernel, "shape": shape, "us": round(us, 2), "achieved": round(got, 1), "unit": unit, "frac": round(got / top, 3)})
        out(f"{kernel:40s} {shape:44s} {us:9.2f} us {got:9.1f} {unit:20s} {100 * got / top:5.1f} % of bound", flush=True)

    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device="cuda")       # noqa: E731
    bf = torch.bfloat16
    W, H, KV, D, V = z["width"], z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    E, top, F, SH = z["experts"], z["top"], z["eff"], z["shared"]
    T, it = args.tokens, args.iters
    # ---- stream kernels
    x, y = torch.randn(4, T, W, device="cuda"), torch.randn(4, T, W, device="cuda", dtype=bf)
    wn = torch.ones(W, device="cuda")
    us = timed(lambda i: ops.out_rmsnorm_add(x[i % 4], y[i % 4], wn, wn, 0.3, 1e-6, bf), it)
    line("output norm + add (f32 stream)", f"T={T} width={W}", us, T * W * 12.0, "hbm")
    xb, wb = torch.randn(4, T, W, device="cuda", dtype=bf), torch.ones(W, device="cuda", dtype=bf)
    us = timed(lambda i: ops.add_rmsnorm(xb[i % 4], y[i % 4], wb, 1e-6), it)
    line("  Qwen3: add + rmsnorm (bf16 stream)", f"T={T} width={W}", us, T * W * 8.0, "hbm")
    gu = torch.randn(4, T, 2 * SH, device="cuda", dtype=bf)
    us = timed(lambda i: ops.clamped_glu(gu[i % 4], 7.0, 1.702), it)
    line("clamped gated activation", f"T={T} inter={SH}", us, T * SH * 6.0, "hbm")
    us = timed(lambda i: ops.swiglu(gu[i % 4]), it)
    line("  Qwen3: swiglu", f"T={T} inter={SH}", us, T * SH * 6.0, "hbm")
    # ---- routed experts beside the dense feed-forward of equal active size
    for rows_n in (T, 64, 8):
        h = torch.randn(rows_n, W, device="cuda", dtype=bf)
        router, corr = (torch.randn(E, W, device="cuda") * 0.05).to(bf), torch.zeros(E, device="cuda")
        reps = 4 if rows_n > 64 else max(2, (300 << 20) // (E * 3 * F * W * 2) + 1)
        w_in = torch.randn(reps, E, 2 * F, W, device="cuda", dtype=bf) * 0.02
        w_out = torch.randn(reps, E, W, F, device="cuda", dtype=bf) * 0.02
        us = timed(lambda i: ops.route_topk(h, router, corr, top, z["groups"]), it)
        line("router: logits, softmax, grouped top-k", f"rows={rows_n} experts={E} top={top}", us, rows_n * W * 2.0 + E * W * 2.0, "hbm")
        chosen, wts = ops.route_topk(h, router, corr, top, z["groups"])
        us = timed(lambda i: ops.expert_ffn(h, chosen, wts, w_in[i % reps], w_out[i % reps], 7.0, 1.702, None), it)
        flops = 2.0 * rows_n * top * 3 * F * W
        hit = min(E, rows_n * top)                                   # experts that can be hit at all
        if rows_n > 64:
            line("experts: sort, 2 grouped products, sum", f"rows={rows_n} experts={E} top={top} ff={F}", us, flops, "bf16")
        else:
            line("experts: sort, 2 grouped products, sum", f"rows={rows_n} experts={E} top={top} ff={F}", us, hit * 3.0 * F * W * 2, "hbm")
        inter = top * F
        wg, wd = torch.randn(reps, 2 * inter, W, device="cuda", dtype=bf) * 0.02, torch.randn(reps, W, inter, device="cuda", dtype=bf) * 0.02
        us = timed(lambda i: ops.linear(ops.gated_linear(h, wg[i % reps]), wd[i % reps]), it)
        if rows_n > 64:
            line("  Qwen3: gate/up + swiglu + down", f"rows={rows_n} inter={inter}", us, flops, "bf16")
        else:
            line("  Qwen3: gate/up + swiglu + down", f"rows={rows_n} inter={inter}", us, 3.0 * inter * W * 2, "hbm")
        del w_in, w_out, wg, wd
    # ---- retention: one prompt of T tokens; decode steps of B requests
    inv = (1e6 ** (-torch.arange(0, D, 2, dtype=torch.float64) / D)).float().cuda()
    for B, n in ((1, T), (8, 1), (64, 1)):
        rows_n = B * n
        batch = types.SimpleNamespace(seg_q_start=t(np.arange(B + 1) * n), seg_slot=t(np.arange(B) + 1), num_segs=B,
                                      positions=t(np.tile(np.arange(n), B) if n > 1 else np.full(B, 4095)))
        shape = f"{'prompt' if n > 1 else 'decode'} B={B} T={n} heads={H} {D}x{V}"
        reps = 4 if n > 1 else max(2, (256 << 20) // (B * H * D * V * 4) + 1)
        p = torch.randn(rows_n, 2 * H * D + 2 * H * V, device="cuda", dtype=bf)
        decay = torch.full((H,), 0.99, device="cuda")
        st = torch.zeros(reps, B + 1, H * D * V, device="cuda")
        us = timed(lambda i: ops.retention_scan(p, H, D, V, inv, D ** -0.5, decay, st[i % reps], batch), it)
        line("retention: rotation + scan", shape, us, 4.0 * H * D * V * rows_n if n > 1 else 8.0 * B * H * D * V, "fma" if n > 1 else "hbm")
        del st
    # ---- attention inside blocks beside causal attention
    ps, blk = 16, z["block"]
    pages = -(-T // ps)
    table = (torch.randperm(pages, device="cuda").to(torch.int32) + 1).view(1, pages).contiguous()
    tiles = dict(prefill_tiles=t([(0, r) for r in range(0, T, 64)]).view(-1, 2), prefill_tiles2=t([(0, r) for r in range(0, T, 128)]).view(-1, 2))
    meta = types.SimpleNamespace(page_size=ps, tile=64, block_table=table, table_rows=t([0]), max_pages=pages, seg_q_start=t([0, T]), seg_pos0=t([0]),
                                 seg_kv_len=t([T]), decode_segs=t([]), max_kv_len=T, num_tokens=T, positions=t(np.arange(T)),
                                 slots=t(np.arange(T) + ps), **tiles)
    kv = torch.randn(4, 2, pages + 1, KV, ps, D, device="cuda", dtype=bf)
    qq = torch.randn(T, H * D, device="cuda", dtype=bf)
    pairs_blk = sum((p % blk) + 1 for p in range(T))
    pairs = T * (T + 1) / 2
    us = timed(lambda i: ops.masked_attention(qq, kv[i % 4, 0], kv[i % 4, 1], meta, H, KV, D, V, 0.7, blk, None, True), it)
    line("attention in blocks, sink (split weights)", f"prompt T={T} heads={H}/{KV} D={D} block={blk}", us, 2.0 * H * (D + V) * pairs_blk, "bf16")
    ops.fast_attention = False
    us = timed(lambda i: ops.masked_attention(qq, kv[i % 4, 0], kv[i % 4, 1], meta, H, KV, D, V, 0.7, blk, None, True), 3)
    line("attention in blocks, sink (float32 kernel)", f"prompt T={T} heads={H}/{KV} D={D} block={blk}", us, 2.0 * H * (D + V) * pairs_blk, "fma")
    ops.fast_attention = True
    meta.table_rows = None
    us = timed(lambda i: ops.paged_attention(qq, kv[i % 4, 0], kv[i % 4, 1], meta, H, KV, 128, 0.1, None), it)
    line("  Qwen3: attention", f"prompt T={T} heads={H}/{KV} D=128", us, 4.0 * H * 128 * pairs, "bf16")
    p3 = torch.randn(4, T, (H + 2 * KV) * D, device="cuda", dtype=bf)
    lam = torch.tensor([0.3], device="cuda")
    us = timed(lambda i: ops.unit_qk_cache(p3[i % 4], H, KV, D, V, 1e-6, lam, p3[(i + 1) % 4][:, (H + KV) * D:], meta, kv[i % 4, 0], kv[i % 4, 1]), it)
    line("unit norms, value blend, cache write", f"T={T} heads={H}/{KV}", us, T * ((H + 2 * KV) * D * 2.0 * 2 + KV * V * 2.0), "hbm")
    nw, invf = torch.ones(D, device="cuda", dtype=bf), torch.full((D // 2,), 0.01, device="cuda")
    us = timed(lambda i: ops.qk_norm_rope_cache(p3[i % 4], H, KV, D, nw, nw, 1e-6, invf, meta, kv[i % 4, 0], kv[i % 4, 1]), it)
    line("  Qwen3: q/k norm, rotation, cache write", f"T={T} heads={H}/{KV}", us, T * (H + 2 * KV) * D * 2.0 * 2, "hbm")
    ctx = args.ctx
    pages = -(-ctx // ps)
    for B in (8, 64):
        layers = max(2, (512 << 20) // (B * pages * ps * KV * D * 4) + 1)
        table = (torch.stack([torch.randperm(pages, device="cuda") for _ in range(B)]) + 1 + (torch.arange(B, device="cuda") * pages)[:, None]).to(torch.int32)
        ar = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        meta = types.SimpleNamespace(page_size=ps, tile=64, block_table=table.contiguous(), table_rows=ar[:B].contiguous(), max_pages=pages, seg_q_start=ar,
                                     seg_pos0=torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda"),
                                     seg_kv_len=torch.full((B,), ctx, dtype=torch.int32, device="cuda"), decode_segs=ar[:B].contiguous(),
                                     prefill_tiles=torch.zeros((0, 2), dtype=torch.int32, device="cuda"), prefill_tiles2=None, max_kv_len=ctx, num_tokens=B)
        kv = torch.randn(layers, 2, B * pages + 1, KV, ps, D, device="cuda", dtype=bf)
        qq = torch.randn(B, H * D, device="cuda", dtype=bf)
        seen = (ctx - 1) % blk + 1
        us = timed(lambda i: ops.masked_attention(qq, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D, V, 0.7, blk, None, True), it)
        line("attention in blocks, sink", f"decode B={B} ctx={ctx} sees {seen} heads={H}/{KV}", us, B * seen * KV * (D + V) * 2.0, "hbm")
        meta.table_rows = None
        us = timed(lambda i: ops.paged_attention(qq, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, 128, 0.1, None), it)
        line("  Qwen3: attention", f"decode B={B} ctx={ctx} heads={H}/{KV} D=128", us, B * ctx * KV * 128 * 4.0, "hbm")
        del kv
    ops.check_errors()
    return rows


NUNUNEX_SIZES = {
    # the widths, experts and attention heads of the Namesun sizes; delta-rule heads of 64 x 64, a scan of twice the width with 16
    # states a channel, a matrix memory of 8 heads whose values are twice as wide as its keys
    "2k": dict(width=2048, ff=8192, d_heads=32, d_dim=64, rank=64, inner=4096, state=16, dt_rank=128, conv=4, heads=16, kv_heads=8, dim=128, vdim=128,
               window=1024, rows=32, far=4096, m_heads=8, m_dim=128, m_vdim=256, experts=32, top=4, eff=1024, shared=2048, taps=4),
    "4k": dict(width=4096, ff=12288, d_heads=64, d_dim=64, rank=128, inner=8192, state=16, dt_rank=256, conv=4, heads=32, kv_heads=8, dim=128, vdim=128,
               window=1024, rows=32, far=4096, m_heads=8, m_dim=256, m_vdim=512, experts=64, top=6, eff=1536, shared=3072, taps=4),
}


def nununex_config(size, layers, vocab=65536):
    z = NUNUNEX_SIZES[size]
    experts = {"kind": "moe", "router": {"experts": z["experts"], "top": z["top"]}, "expert": {"ff": z["eff"]}, "shared": {"ff": z["shared"]}}
    dense = {"kind": "dense", "ff": z["ff"]}
    delta = {"type": "general_delta", "mixer": {"heads": z["d_heads"], "dim": z["d_dim"], "decay_rank": z["rank"]}}
    scan = {"type": "mamba1", "mixer": {"inner": z["inner"], "state": z["state"], "dt_rank": z["dt_rank"], "conv": z["conv"]}}
    pair = {"type": "parallel", "mixer": {
        "left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5, "bias_max": z["far"],
                 "bias_rows": z["rows"], "mask": {"size": z["window"]}},
        "right": {"heads": z["m_heads"], "dim": z["m_dim"], "vdim": z["m_vdim"], "gate_cap": 15.0}}}
    pattern = [dict(delta, mlp=dense), dict(scan, mlp=experts), dict(delta, mlp=dense), dict(pair, mlp=experts)]
    return {"architecture": "Nununex", "vocab": vocab, "width": z["width"], "norm": {"eps": 1e-6}, "canon": {"taps": z["taps"]}, "logit_softcap": 30.0,
            "embedding": {"bigram": {"buckets": 1000003, "mul_prev": 1000033, "mul_cur": 7919}}, "layers": [pattern[i % 4] for i in range(layers)]}


def namesun_config_like_nununex(size, layers, vocab=65536):
    """Namesun (float32 stream, retention and windowed attention with a sink, routed experts) of the same width, depth, vocabulary,
    attention heads and experts: the closest design the engine already serves."""
    return namesun_config(size, layers, vocab)


def bench_nununex(args, ops, peak, out=print):
    """Each kernel of the Nununex design at the layer sizes of --design-size beside the like kernel of Namesun, with the bytes or
    operations it cannot avoid as a share of its bound: the measured copy bandwidth, the float32 FMA rate of the CUDA cores, the
    rate of the special-function units (one exponential per state element of the selective scan), or the measured bf16 peak."""
    import numpy as np
    from ..parts.base import GatedDelta
    z = NUNUNEX_SIZES[args.design_size]
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    bf16_peak = 1590.0
    if os.path.isfile(os.path.join(here, "MEASURED_PEAKS.json")):
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            bf16_peak = json.load(f)["bf16_tflops"]
    props = torch.cuda.get_device_properties(0)
    fma_peak = props.multi_processor_count * 128 * 2 * 1.965e9 / 1e12
    sfu_peak = props.multi_processor_count * 16 * 1.965e9 / 1e12
    rows = []

    def line(kernel, shape, us, amount, bound):
        got, top, unit = {"hbm": (amount / us / 1e3, peak, "GB/s"), "bf16": (amount / us / 1e6, bf16_peak, "TFLOP/s"),
                          "fma": (amount / us / 1e6, fma_peak, "TFLOP/s (fp32 FMA)"), "sfu": (amount / us / 1e6, sfu_peak, "Texp/s (SFU)")}[bound]
        rows.append({"kernel": kernel, "shape": shape, "us": round(us, 2), "achieved": round(got, 2), "unit": unit, "frac": round(got / top, 3)})
        out(f"{kernel:44s} {shape:46s} {us:9.2f} us {got:9.2f} {unit:20s} {100 * got / top:5.1f} % of bound", flush=True)

    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device="cuda")       # noqa: E731
    bf = torch.bfloat16
    W, T, it = z["width"], args.tokens, args.iters
    rb = lambda *s: torch.randn(*s, device="cuda", dtype=bf)                       # noqa: E731
    rf = lambda *s: torch.randn(*s, device="cuda")                                 # noqa: E731

    def entries(B, n, pos0=0):
        return types.SimpleNamespace(seg_q_start=t(np.arange(B + 1) * n), seg_slot=t(np.arange(B) + 1), num_segs=B,
                                     token_seg=t(np.repeat(np.arange(B), n)), positions=t(np.tile(np.arange(n), B) + pos0))

    # ---- stream kernels
    x, y, lg = rf(4, T, W), rb(4, T, W), rb(4, T, W)
    wn, gb = torch.ones(W, device="cuda"), torch.zeros(W, device="cuda")
    us = timed(lambda i: ops.stream_rmsnorm(x[i % 4], GatedDelta(y[i % 4], lg[i % 4], gb), wn, 1e-6, None, bf), it)
    line("gated addition + norm (f32 stream)", f"T={T} width={W}", us, T * W * 14.0, "hbm")
    us = timed(lambda i: ops.out_rmsnorm_add(x[i % 4], y[i % 4], wn, wn, 0.3, 1e-6, bf), it)
    line("  Namesun: output norm + add (f32 stream)", f"T={T} width={W}", us, T * W * 12.0, "hbm")
    us = timed(lambda i: ops.dual_rmsnorm_mix(y[i % 4], wn, 0.5, lg[i % 4], wn, 0.5, 1e-6), it)
    line("norm and mix of two mixers' outputs", f"T={T} width={W}", us, T * W * 6.0, "hbm")
    ids = torch.randint(0, 65536, (T,), device="cuda", dtype=torch.int32)
    table, pairs, prev = rb(65536, W), rb(1000004, W), torch.zeros(2, 1, dtype=torch.int32, device="cuda")
    e1 = entries(1, T)
    us = timed(lambda i: ops.embed_bigram_stream(ids, table, pairs, 1000003, 1000033, 7919, prev, e1), it)
    line("embedding + hashed pair row", f"T={T} width={W}", us, T * W * 8.0, "hbm")
    us = timed(lambda i: ops.embed_stream(ids, table, bf), it)
    line("  Namesun: embedding", f"T={T} width={W}", us, T * W * 8.0, "hbm")
    del table, pairs
    cw = rf(W, z["taps"])
    for B, n in ((1, T), (64, 1)):
        st = torch.zeros(B + 1, (z["taps"] - 1) * W, device="cuda")
        hh, e = rb(4, B * n, W), entries(B, n)
        us = timed(lambda i: ops.short_conv(hh[i % 4], cw, None, z["taps"], st, 0, e, residual=True), it)
        line("input filter (causal convolution + input)", f"B={B} T={n} width={W} taps={z['taps']}", us,
             B * n * W * 4.0 + (B * (z["taps"] - 1) * W * 8.0 if n == 1 else 0), "hbm")
    F = z["ff"]
    zz, fb = rb(4, T, F), torch.zeros(F, device="cuda")
    us = timed(lambda i: ops.bias_act(zz[i % 4], fb, "relu2"), it)
    line("bias + squared relu", f"T={T} ff={F}", us, T * F * 4.0, "hbm")
    gu = rb(4, T, 2 * z["shared"])
    us = timed(lambda i: ops.clamped_glu(gu[i % 4], 7.0, 1.702), it)
    line("  Namesun: clamped gated activation", f"T={T} inter={z['shared']}", us, T * z["shared"] * 6.0, "hbm")
    del zz, gu
    # ---- the three recurrences beside Namesun's retention: one prompt of T tokens; decode steps of B requests
    H, D, R = z["d_heads"], z["d_dim"], z["rank"]
    w2, w0, ab = rb(H * D, R) * 0.1, torch.zeros(H * D, device="cuda"), torch.zeros(H * D, device="cuda")
    for B, n in ((1, T), (8, 1), (64, 1)):
        rows_n, e = B * n, entries(B, n, 0 if n > 1 else 4095)
        kind = "prompt" if n > 1 else "decode"
        reps = 4 if n > 1 else max(2, (256 << 20) // (B * H * D * D * 4) + 1)
        p = rb(rows_n, 5 * H * D + R)
        st = torch.zeros(reps, B + 1, H * D * D, device="cuda")
        us = timed(lambda i: ops.general_delta_prepare(p, w2, w0, ab, H, D, D, R, 0.6, 1e-6), it)
        line("delta rule: unit key, decay, removal", f"{kind} B={B} T={n} heads={H} {D}x{D}", us, rows_n * ((5 * H * D + R) * 2.0 + 6 * H * D * 4.0), "hbm")
        prep = ops.general_delta_prepare(p, w2, w0, ab, H, D, D, R, 0.6, 1e-6)
        us = timed(lambda i: ops.general_delta_scan(prep, H, D, D, st[i % reps], e), it)
        line("delta rule: scan", f"{kind} B={B} T={n} heads={H} {D}x{D}", us, 10.0 * H * D * D * rows_n if n > 1 else 8.0 * B * H * D * D, "fma" if n > 1 else "hbm")
        del st
        H2, D2, V2 = z["heads"], z["dim"], z["vdim"]
        reps = 4 if n > 1 else max(2, (256 << 20) // (B * H2 * D2 * V2 * 4) + 1)
        p2, decay = rb(rows_n, 2 * H2 * D2 + 2 * H2 * V2), torch.full((H2,), 0.99, device="cuda")
        inv = (1e6 ** (-torch.arange(0, D2, 2, dtype=torch.float64) / D2)).float().cuda()
        st = torch.zeros(reps, B + 1, H2 * D2 * V2, device="cuda")
        us = timed(lambda i: ops.retention_scan(p2, H2, D2, V2, inv, D2 ** -0.5, decay, st[i % reps], e), it)
        line("  Namesun: retention (rotation + scan)", f"{kind} B={B} T={n} heads={H2} {D2}x{V2}", us,
             4.0 * H2 * D2 * V2 * rows_n if n > 1 else 8.0 * B * H2 * D2 * V2, "fma" if n > 1 else "hbm")
        del st
        H3, D3, V3 = z["m_heads"], z["m_dim"], z["m_vdim"]
        Wd = V3 + 4
        reps = 4 if n > 1 else max(2, (256 << 20) // (B * H3 * D3 * Wd * 4) + 1)
        p3, gl, gbias = rb(rows_n, 2 * H3 * D3 + 2 * H3 * V3), rf(rows_n, 2 * H3), torch.zeros(2 * H3, device="cuda")
        norm3 = torch.ones(H3 * V3, device="cuda")
        st = torch.zeros(reps, B + 1, H3 * D3 * Wd + H3, device="cuda")
        us = timed(lambda i: ops.matrix_memory(p3, gl, gbias, H3, D3, V3, 15.0, 1e-6, norm3, p3[:, 2 * H3 * D3 + H3 * V3:], 1e-6, st[i % reps], e, bf), it)
        line("matrix memory: gates, scan, norm, gate", f"{kind} B={B} T={n} heads={H3} {D3}x{V3}", us,
             4.0 * H3 * D3 * Wd * rows_n if n > 1 else 8.0 * B * H3 * D3 * Wd, "fma" if n > 1 else "hbm")
        del st
        I, N = z["inner"], z["state"]
        reps = 4 if n > 1 else max(2, (256 << 20) // (B * I * N * 4) + 1)
        xs, dt, bc, zs = rb(rows_n, I), rf(rows_n, I), rb(rows_n, 2 * N), rb(rows_n, I)
        A, dtb, Dv = -torch.rand(I, N, device="cuda"), torch.zeros(I, device="cuda"), torch.ones(I, device="cuda")
        st = torch.zeros(reps, B + 1, I * N, device="cuda")
        us = timed(lambda i: ops.selective_scan(xs, dt, dtb, A, bc[:, :N], bc[:, N:], Dv, zs, st[i % reps], e, bf), it)
        line("selective scan", f"{kind} B={B} T={n} inner={I} state={N}", us, 1.0 * I * N * rows_n if n > 1 else 8.0 * B * I * N, "sfu" if n > 1 else "hbm")
        del st
    # ---- windowed attention with distance rows and a learned sink beside Namesun's attention in blocks
    H, KV, D, V = z["heads"], z["kv_heads"], z["dim"], z["vdim"]
    ps, win = 16, z["window"]
    pages = -(-T // ps)
    table = (torch.randperm(pages, device="cuda").to(torch.int32) + 1).view(1, pages).contiguous()
    meta = types.SimpleNamespace(page_size=ps, tile=64, block_table=table, table_rows=t([0]), max_pages=pages, seg_q_start=t([0, T]), seg_pos0=t([0]),
                                 seg_kv_len=t([T]), decode_segs=t([]), max_kv_len=T, num_tokens=T, positions=t(np.arange(T)), slots=t(np.arange(T) + ps),
                                 prefill_tiles=t([(0, r) for r in range(0, T, 64)]).view(-1, 2), prefill_tiles2=t([(0, r) for r in range(0, T, 128)]).view(-1, 2))
    kv = rb(4, 2, pages + 1, KV, ps, D)
    qq = rb(T, H * D)
    sinks, bias = rf(H), rf(z["far"] + 1, H) * 0.1
    bias_h = bias.t().contiguous()
    pairs_win = sum(min(p + 1, win) for p in range(T))
    us = timed(lambda i: ops.masked_attention(qq, kv[i % 4, 0], kv[i % 4, 1], meta, H, KV, D, V, D ** -0.5, None, win, True, sink_values=sinks, distance_bias=bias,
                                              distance_bias_by_head=bias_h), it)
    bound = "bf16" if getattr(ops, "biased_attention_tc", False) else "fma"
    line("attention: window, distance rows, learned sink", f"prompt T={T} heads={H}/{KV} D={D} window={win}", us, 2.0 * H * (D + V) * pairs_win, bound)
    us = timed(lambda i: ops.masked_attention(qq, kv[i % 4, 0], kv[i % 4, 1], meta, H, KV, D, V, 0.7, win, None, True), it)
    line("  Namesun: attention in blocks, sink (split weights)", f"prompt T={T} heads={H}/{KV} D={D} block={win}", us,
         2.0 * H * (D + V) * sum((p % win) + 1 for p in range(T)), "bf16")
    ctx = args.ctx
    pages = -(-ctx // ps)
    for B in (8, 64):
        layers = max(2, (512 << 20) // (B * pages * ps * KV * D * 4) + 1)
        table = (torch.stack([torch.randperm(pages, device="cuda") for _ in range(B)]) + 1 + (torch.arange(B, device="cuda") * pages)[:, None]).to(torch.int32)
        ar = torch.arange(B + 1, dtype=torch.int32, device="cuda")
        meta = types.SimpleNamespace(page_size=ps, tile=64, block_table=table.contiguous(), table_rows=ar[:B].contiguous(), max_pages=pages, seg_q_start=ar,
                                     seg_pos0=torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda"),
                                     seg_kv_len=torch.full((B,), ctx, dtype=torch.int32, device="cuda"), decode_segs=ar[:B].contiguous(),
                                     prefill_tiles=torch.zeros((0, 2), dtype=torch.int32, device="cuda"), prefill_tiles2=None, max_kv_len=ctx, num_tokens=B)
        kv = rb(layers, 2, B * pages + 1, KV, ps, D)
        qq = rb(B, H * D)
        seen = min(ctx, win)
        us = timed(lambda i: ops.masked_attention(qq, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D, V, D ** -0.5, None, win, True, sink_values=sinks,
                                                  distance_bias=bias, distance_bias_by_head=bias_h), it)
        line("attention: window, distance rows, learned sink", f"decode B={B} ctx={ctx} sees {seen} heads={H}/{KV}", us, B * seen * KV * (D + V) * 2.0, "hbm")
        us = timed(lambda i: ops.masked_attention(qq, kv[i % layers, 0], kv[i % layers, 1], meta, H, KV, D, V, 0.7, win, None, True), it)
        line("  Namesun: attention in blocks, sink", f"decode B={B} ctx={ctx} sees {(ctx - 1) % win + 1} heads={H}/{KV}", us,
             B * ((ctx - 1) % win + 1) * KV * (D + V) * 2.0, "hbm")
        del kv
    # ---- sigmoid router with the shared gate's row; experts weighted on their input beside experts weighted on their output
    E, top, F = z["experts"], z["top"], z["eff"]
    for rows_n in (T, 64, 8):
        h = rb(rows_n, W)
        router, corr = rb(E + 1, W) * 0.05, torch.zeros(E, device="cuda")
        reps = 4 if rows_n > 64 else max(2, (300 << 20) // (E * 3 * F * W * 2) + 1)
        w_in, w_out = rb(reps, E, 2 * F, W) * 0.02, rb(reps, E, W, F) * 0.02
        us = timed(lambda i: ops.route_topk(h, router, None, top, None, score="sigmoid", extra_rows=1), it)
        line("router: logits, sigmoid, top-k, gate row", f"rows={rows_n} experts={E} top={top}", us, rows_n * W * 2.0 + (E + 1) * W * 2.0, "hbm")
        us = timed(lambda i: ops.route_topk(h, router[:E].contiguous(), corr, top, None), it)
        line("  Namesun: router (softmax, top-k)", f"rows={rows_n} experts={E} top={top}", us, rows_n * W * 2.0 + E * W * 2.0, "hbm")
        chosen, wts, gate_row = ops.route_topk(h, router, None, top, None, score="sigmoid", extra_rows=1)
        shared = rb(rows_n, W)
        flops, hit = 2.0 * rows_n * top * 3 * F * W, min(E, rows_n * top)
        amount, bound = (flops, "bf16") if rows_n > 64 else (hit * 3.0 * F * W * 2, "hbm")
        us = timed(lambda i: ops.expert_ffn(h, chosen, wts, w_in[i % reps], w_out[i % reps], float("inf"), 1.0, shared, up_shift=0.0, weight_on_input=True,
                                            shared_gate=gate_row), it)
        line("experts weighted on their input, gated shared", f"rows={rows_n} experts={E} top={top} ff={F}", us, amount, bound)
        us = timed(lambda i: ops.expert_ffn(h, chosen, wts, w_in[i % reps], w_out[i % reps], 7.0, 1.702, shared), it)
        line("  Namesun: experts weighted on their output", f"rows={rows_n} experts={E} top={top} ff={F}", us, amount, bound)
        del w_in, w_out
    lo = rf(64, 65536)
    us = timed(lambda i: ops.softcap(lo, 30.0), it)
    line("soft cap of the logits", "rows=64 vocab=65536", us, 64 * 65536 * 8.0, "hbm")
    ops.check_errors()
    return rows


MEGOVIK_SIZES = {
    # the widths, heads, experts and active feed-forward parameters of NAMESUN_SIZES; latent rows of 128 entries, a query latent of 3/8 of the width
    "2k": dict(width=2048, ff=8192, heads=16, kv_heads=8, dim=128, l_heads=16, l_dim=64, l_vdim=64, rank=128, q_rank=768, experts=32, top=4, eff=1024, groups=(8, 4)),
    "4k": dict(width=4096, ff=12288, heads=32, kv_heads=8, dim=128, l_heads=32, l_dim=64, l_vdim=64, rank=128, q_rank=1536, experts=64, top=6, eff=1536, groups=(8, 4)),
}


def megovik_config(size, layers, vocab=65536):
    z = MEGOVIK_SIZES[size]
    experts = {"kind": "moe", "expert": {"ff": z["eff"]},
               "router": {"experts": z["experts"], "top": z["top"], "scale": 2.5, "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    dense = {"kind": "dense", "ff": z["ff"]}
    lat = {"heads": z["l_heads"], "dim": z["l_dim"], "vdim": z["l_vdim"], "kv_rank": z["rank"], "scale": z["l_dim"] ** -0.5}
    att = {"type": "attention", "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "scale": z["dim"] ** -0.5,
                                          "q_temp": {"coef": 0.1, "every": 1024}}}
    pattern = [dict(type="latent_attention", mixer=lat, mlp=dense), dict(type="latent_attention", mixer=lat, mlp=experts), dict(att, mlp=experts),
               dict(type="latent_attention_2", mixer=dict(lat, q_rank=z["q_rank"]), mlp=experts)]
    return {"architecture": "Megovik", "vocab": vocab, "width": z["width"], "max_positions": 8192, "norm": {"eps": 1e-6}, "embedding": {"scale": z["width"] ** 0.5},
            "logit_scale": 0.5, "layers": [pattern[i % 4] for i in range(layers)]}


def namesun_config_like_megovik(size, layers, vocab=65536):
    """Namesun (float32 stream, attention with a mask chosen by constants, routed experts with groups) of the same width, depth, vocabulary,
    attention heads and experts: the closest design the engine already serves."""
    return namesun_config(size, layers, vocab)


def bench_megovik(args, ops, peak, out=print):
    """Each kernel that the Megovik design added or widened, at the layer sizes of --design-size, beside the like kernel of Namesun (of Naditar
    for latent attention), with the bytes or operations it cannot avoid as a share of its bound: the measured copy bandwidth or the measured
    bf16 peak."""
    import numpy as np
    z = MEGOVIK_SIZES[args.design_size]
    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    bf16_peak = 1590.0
    if os.path.isfile(os.path.join(here, "MEASURED_PEAKS.json")):
        with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
            bf16_peak = json.load(f)["bf16_tflops"]
    rows = []

    def line(kernel, shape, us, amount, bound):
        got, top, unit = {"hbm": (amount / us / 1e3, peak, "GB/s"), "bf16": (amount / us / 1e6, bf16_peak, "TFLOP/s")}[bound]
        rows.append({"kernel": kernel, "shape": shape, "us": round(us, 2), "achieved": round(got, 2), "unit": unit, "frac": round(got / top, 3)})
        out(f"{kernel:52s} {shape:46s} {us:9.2f} us {got:9.2f} {unit:10s} {100 * got / top:5.1f} % of bound", flush=True)

    t = lambda a: torch.tensor(np.asarray(a, dtype=np.int32), device="cuda")       # noqa: E731
    bf = torch.bfloat16
    W, T, it = z["width"], args.tokens, args.iters
    rb = lambda *s: torch.randn(*s, device="cuda", dtype=bf)                       # noqa: E731
    rf = lambda *s: torch.randn(*s, device="cuda")                                 # noqa: E731
    # ---- stream kernels
    x, a, b = rf(4, T, W), rb(4, T, W), rb(4, T, W)
    wn, bias, pre = torch.ones(W, device="cuda"), rf(W), rf(T, W)
    us = timed(lambda i: ops.stream_rmsnorm_pair(x[i % 4], a[i % 4], b[i % 4], bias, None, wn, 1e-6, None, bf), it)
    line("pair addition + norm (f32 stream)", f"T={T} width={W}", us, T * W * 14.0, "hbm")
    us = timed(lambda i: ops.stream_rmsnorm_pair(x[i % 4], a[i % 4], b[i % 4], bias, pre, wn, 1e-6, None, bf), it)
    line("pair addition + embedded tokens + norm", f"T={T} width={W}", us, T * W * 18.0, "hbm")
    us = timed(lambda i: ops.out_rmsnorm_add(x[i % 4], a[i % 4], wn, wn, 0.3, 1e-6, bf), it)
    line("  Namesun: output norm + add (f32 stream)", f"T={T} width={W}", us, T * W * 12.0, "hbm")
    ids = torch.randint(0, 65536, (T,), device="cuda", dtype=torch.int32)
    table, ptab, pos = rb(65536, W), rb(8192, W), t(np.arange(T) % 8192)
    us = timed(lambda i: ops.embed_scaled_stream(ids, table, 45.0, ptab, pos), it)
    line("embedding * scale + position row", f"T={T} width={W}", us, T * W * 8.0, "hbm")
    us = timed(lambda i: ops.embed_stream(ids, table, bf), it)
    line("  Namesun: embedding", f"T={T} width={W}", us, T * W * 8.0, "hbm")
    del table, ptab
    F = z["ff"]
    gu, gb = rb(2, T, 2 * F), rf(2 * F)
    us = timed(lambda i: ops.bias_glu(gu[i % 2], gb, "relu"), it)
    line("biases + relu gate", f"T={T} ff={F}", us, T * F * 6.0, "hbm")
    us = timed(lambda i: ops.clamped_glu(gu[i % 2], 7.0, 1.702), it)
    line("  Namesun: clamped gate", f"T={T} ff={F}", us, T * F * 6.0, "hbm")
    del gu
    cq, wq = rb(T, z["q_rank"] + z["rank"]), torch.ones(z["q_rank"], device="cuda")
    us = timed(lambda i: ops.rows_rmsnorm(cq[:, :z["q_rank"]], wq, 1e-6), it)
    line("norm of the query latent", f"T={T} q_rank={z['q_rank']}", us, T * z["q_rank"] * 4.0, "hbm")
    # ---- attention with weighted norms, a temperature, keys as values and distance slopes, beside Namesun's masked attention
    H, KV, D, page = z["heads"], z["kv_heads"], z["dim"], args.page_size if hasattr(args, "page_size") else 16
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], device="cuda")
    qw = torch.ones(D, device="cuda")
    for B, n, ctx in ((1, T, T), (8, 1, args.ctx), (64, 1, args.ctx)):
        pages_per = -(-ctx // page)
        n_pages = B * pages_per + 1
        kc, vc = rb(n_pages, KV, page, D), rb(n_pages, KV, page, D)
        table = t(np.arange(1, n_pages).reshape(B, pages_per))
        tiles = [(s, r) for s in range(B) for r in range(0, n, 64)] if n > 1 else []
        meta = types.SimpleNamespace(seg_q_start=t(np.arange(B + 1) * n), seg_pos0=t([ctx - n] * B), seg_kv_len=t([ctx] * B), table_rows=t(np.arange(B)),
                                     block_table=table, max_pages=pages_per, page_size=page, decode_segs=t(np.arange(B) if n == 1 else []),
                                     prefill_tiles=t(tiles).view(-1, 2), tile=64, max_kv_len=ctx,
                                     slots=t((np.arange(B)[:, None] * pages_per * page + page + ctx - n + np.arange(n)[None, :]).reshape(-1)),
                                     positions=t(np.tile(np.arange(ctx - n, ctx), B)))
        Tn = B * n
        p2, p3 = rb(Tn, (H + KV) * D), rb(Tn, (H + 2 * KV) * D)
        us = timed(lambda i: ops.unit_qk_cache(p2, H, KV, D, D, 1e-6, None, None, meta, kc, vc, q_weight=qw, k_weight=qw, q_temp=(0.1, 1024), values_are_keys=True), it)
        line("q/k norm * weight, temperature, k -> both pools", f"rows={Tn} H={H} KV={KV} D={D}", us, Tn * ((2 * H + 3 * KV) * D) * 2.0, "hbm")
        us = timed(lambda i: ops.unit_qk_cache(p3, H, KV, D, D, 1e-6, None, None, meta, kc, vc), it)
        line("  Namesun: unit q/k, k and v -> pools", f"rows={Tn} H={H} KV={KV} D={D}", us, Tn * ((2 * H + 4 * KV) * D) * 2.0, "hbm")
        q = p2[:, :H * D]
        if n > 1:
            amount, bound = 4.0 * H * D * (n * (n + 1) / 2) * B, "bf16"
        else:
            amount, bound = B * ctx * KV * D * 2 * 2.0, "hbm"
        us = timed(lambda i: ops.masked_attention(q, kc, vc, meta, H, KV, D, D, D ** -0.5, None, None, False, distance_slopes=slopes), it)
        line("attention with distance slopes", f"B={B} rows={n} keys={ctx} H={H} KV={KV} D={D}", us, amount, bound)
        us = timed(lambda i: ops.masked_attention(q, kc, vc, meta, H, KV, D, D, D ** -0.5, None, None, True), it)
        line("  Namesun: attention with a sink (no block)", f"B={B} rows={n} keys={ctx} H={H} KV={KV} D={D}", us, amount, bound)
        # latent attention without a rotated part: the cached row is key and value of every head
        LH, C = z["l_heads"], z["rank"]
        lc = rb(n_pages, 1, page, C)
        ql = rb(Tn, LH, C)
        if n > 1:
            amount, bound = 4.0 * LH * C * (n * (n + 1) / 2) * B, "bf16"
        else:
            amount, bound = B * ctx * C * 2.0, "hbm"
        us = timed(lambda i: ops.latent_attention(ql, lc, meta, LH, C, 0, 0.125), it)
        line("latent attention (row = key = value)", f"B={B} rows={n} keys={ctx} H={LH} C={C}", us, amount, bound)
        del kc, vc, lc
    # ---- routed feed-forward: sigmoid router with groups ranked by two scores and renormalised weights; experts weighted on their output
    E, top, Fe, groups = z["experts"], z["top"], z["eff"], z["groups"]
    for rows_n in (T, 64, 8):
        h = rb(rows_n, W)
        router, corr = rb(E, W) * 0.05, torch.zeros(E, device="cuda")
        reps = 4 if rows_n > 64 else max(2, (300 << 20) // (E * 3 * Fe * W * 2) + 1)
        w_in, w_out = rb(reps, E, 2 * Fe, W) * 0.02, rb(reps, E, W, Fe) * 0.02
        us = timed(lambda i: ops.route_topk(h, router, None, top, groups, score="sigmoid", group_score="top2_sum", renormalise=True, weight_eps=1e-20,
                                            route_scale=2.5), it)
        line("router: sigmoid, groups by two scores, renormalised", f"rows={rows_n} experts={E} top={top}", us, rows_n * W * 2.0 + E * W * 2.0, "hbm")
        us = timed(lambda i: ops.route_topk(h, router, corr, top, groups), it)
        line("  Namesun: router (softmax, groups by one score)", f"rows={rows_n} experts={E} top={top}", us, rows_n * W * 2.0 + E * W * 2.0, "hbm")
        chosen, wts, _ = ops.route_topk(h, router, None, top, groups, score="sigmoid", group_score="top2_sum", renormalise=True, weight_eps=1e-20, route_scale=2.5)
        flops, hit = 2.0 * rows_n * top * 3 * Fe * W, min(E, rows_n * top)
        amount, bound = (flops, "bf16") if rows_n > 64 else (hit * 3.0 * Fe * W * 2, "hbm")
        us = timed(lambda i: ops.expert_ffn(h, chosen, wts, w_in[i % reps], w_out[i % reps], float("inf"), 1.0, None, up_shift=0.0), it)
        line("experts (silu gate), weighted on their output", f"rows={rows_n} experts={E} top={top} ff={Fe}", us, amount, bound)
        us = timed(lambda i: ops.expert_ffn(h, chosen, wts, w_in[i % reps], w_out[i % reps], 7.0, 1.702, None), it)
        line("  Namesun: experts (clamped gate)", f"rows={rows_n} experts={E} top={top} ff={Fe}", us, amount, bound)
        del w_in, w_out
    lo = rf(64, 65536)
    us = timed(lambda i: ops.scale_logits(lo, 0.5), it)
    line("scale of the logits", "rows=64 vocab=65536", us, 64 * 65536 * 8.0, "hbm")
    ops.check_errors()
    return rows


DESIGNS = {"naditar": (naditar_config, qwen3_config_like, bench_design), "namesun": (namesun_config, qwen3_config_like_namesun, bench_namesun),
           "nununex": (nununex_config, namesun_config_like_nununex, bench_nununex),
           "megovik": (megovik_config, namesun_config_like_megovik, bench_megovik)}
BESIDE = {"nununex": "namesun", "megovik": "namesun"}            # the design an entry of DESIGNS is set beside (default: qwen3)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("what", choices=["gemm", "attention", "prefill", "design", "namesun", "nununex", "megovik"])
    ap.add_argument("--design-size", default="2k", choices=sorted(NADITAR_SIZES), help="design: layer sizes of the Naditar kernels")
    ap.add_argument("--size", default="4b", choices=sorted(SIZES))
    ap.add_argument("--rows", default="1,8,64", type=lambda s: [int(v) for v in s.split(",")])
    ap.add_argument("--batch", default="1,8,64", type=lambda s: [int(v) for v in s.split(",")])
    ap.add_argument("--ctx", type=int, default=4096)
    ap.add_argument("--tokens", type=int, default=2048, help="prefill: tokens of the portion")
    ap.add_argument("--ctx-before", type=int, default=0, help="prefill: tokens of the request already in the cache")
    ap.add_argument("--only", default=None, type=lambda s: s.split(","), help="gemm: only these (qkv,o,gate_up,down,lm_head)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--splits", default=None, type=lambda s: [int(v) for v in s.split(",")],
                    help="attention: time these numbers of key splits instead of the chosen one")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--rotate-mb", type=int, default=512, help="rotate through at least this many MB of operands")
    args = ap.parse_args(argv)
    from ..ops import get_ops
    ops = get_ops("cuda:0")
    peak, src = peak_gbs()
    print(f"# peak {peak} GB/s ({src})")
    {"gemm": bench_gemm, "attention": bench_attention, "prefill": bench_prefill_attention, "design": bench_design, "namesun": bench_namesun, "nununex": bench_nununex, "megovik": bench_megovik}[args.what](args, ops, peak)
    return 0


if __name__ == "__main__":
    sys.exit(main())
