"""Kernel namespace of the engine: thin Python entry points over the hand-written sm_100a
kernels in csrc/ (built into _kernels.so, called through its C interface).

There is no CPU path and no silent fall-back: get_ops() raises when there is no CUDA device
or the library cannot be built or loaded.  Matrix products of the bfloat16 path go to the
library GEMM, as the reference's do (engine/core/fused_linear.py:29-34); the float32 path
uses this package's own float32 GEMM kernel, which never uses a reduced-precision mode.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from ..parts.base import GatedDelta

_LIB = None
_c = ctypes


def load_library():
    global _LIB
    if _LIB is None:
        from .build import build
        path = build()
        _LIB = ctypes.CDLL(path)
    return _LIB


_CODES = {torch.float32: 0, torch.bfloat16: 1}


def _code(dtype):
    try:
        return _CODES[dtype]
    except KeyError:
        raise TypeError(f"dtype {dtype} is not supported by the kernels (float32, bfloat16)") from None


def _raw_stream(device_index):
    getter = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if getter is not None:
        return getter(device_index)
    return torch.cuda.current_stream(device_index).cuda_stream


def _p(t):
    return _c.c_void_p(0 if t is None else t.data_ptr())


def _check(err, what):
    if err != 0:
        if err == -1:
            raise TypeError(f"{what}: unsupported combination of dtypes")
        if err == -2:
            raise ValueError(f"{what}: size not supported by this kernel")
        raise RuntimeError(f"{what}: CUDA error {err} at launch")


class DeferredSum:
    """A product [M, N] that the few-row GEMM left as partial sums (csrc/gemm_stream.cu, deferred mode).  Only
    add_rmsnorm (as its `delta`) and CudaOps.materialize understand it; a part that gets one must pass it on untouched."""
    __slots__ = ("ws", "M", "N", "K", "grid", "max_contrib", "tok", "device")

    def __init__(self, ws, M, N, K, grid, max_contrib, tok):
        self.ws, self.M, self.N, self.K, self.grid, self.max_contrib, self.tok = ws, M, N, K, grid, max_contrib, tok
        self.device = ws.device

    @property
    def shape(self):
        return (self.M, self.N)


class CudaOps:
    prefill_tile = 64
    deferred = True                          # linear(..., defer=True) may answer with a DeferredSum
    takes_hints = True                       # add_rmsnorm(..., next_weight=) is understood
    MAX_ROWS = 4096                          # decode rows x kv heads that the attention merge counters cover

    def __init__(self, device):
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise RuntimeError("mini_inference_b200 runs on a CUDA device only (no CPU path); "
                               f"device '{device}' is not one")
        self.lib = load_library()
        self._device_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.NUM_SMS = torch.cuda.get_device_properties(self._device_index).multi_processor_count
        self.force_splits = None             # tests set this to exercise the split merge on short contexts
        # many-row bfloat16 products on this package's two-block tcgen05 kernel (csrc/gemm_tc2.cu) instead of the library GEMM:
        # MI_TC_GEMM=1 all of them, 0 none; otherwise ("auto") those that tune_many_rows found faster on this model's weights
        self.tc_mode = os.environ.get("MI_TC_GEMM", "auto")
        self.tc_gemm = self.tc_mode == "1"
        self._many_choice = {}               # {(row bucket, N, K): "tc2"} from tune_many_rows; anything else: library
        self.tc_min_rows = 128
        # scratch of the own GEMM for the tiles it cuts along K (the shares of a last, partly filled wave of tiles)
        self._tc2_ws = torch.empty(20 << 20, dtype=torch.uint8, device=self.device)
        self._tc2_counters = torch.zeros(512, dtype=torch.int32, device=self.device)
        self.tc_attention = os.environ.get("MI_TC_ATTENTION", "1") == "1"    # prompt attention on the tcgen05 kernel
        self.stream_gemm = True              # few-row products on the persistent TMA weight-streaming kernel
        self.stream_max_cols = int(os.environ.get("MI_STREAM_MAX_COLS", 1 << 30))
        self._sample_slots = torch.zeros(4096, dtype=torch.int64, device=self.device)
        self._sample_arrivals = torch.zeros(4096, dtype=torch.int32, device=self.device)
        # decode attention stages K/V through shared memory with swizzled TMA tiles and per-warp mbarrier rings (31 vs
        # 33 us at batch 8, 168 vs 202 us at batch 64, context 4096, against streaming them into registers);
        # MI_BULK_DECODE=0 selects the register-streaming variant
        self.bulk_decode = os.environ.get("MI_BULK_DECODE", "1") == "1"
        self.fused_merge = True              # the last split block to finish merges the splits (no merge launch)
        # 2..8 splits of a (request, kv head): one thread-block cluster, merged through distributed shared memory
        self.cluster_merge = os.environ.get("MI_CLUSTER_MERGE", "1") == "1"
        self._cluster_fit = {}
        self._linear_choice = None           # {(row bucket, N, K): "library" | "stream" | "skinny"} from tune_linear
        self._stream_plans = {}
        # Scratch that kernels address directly and that captured graphs keep the address of: allocated here, once, at
        # fixed sizes; a call that needs more raises instead of moving them.
        self._merge_counters = torch.zeros(self.MAX_ROWS * 8, dtype=torch.int32, device=self.device)
        self._stream_counters = torch.zeros(4096, dtype=torch.int32, device=self.device)
        self._stream_error = torch.zeros(1, dtype=torch.int32, device=self.device)
        # a few-row product whose only reader is the next residual-add + norm is left as partial sums for that kernel
        # to add up (no fix-up tail in the GEMM); MI_DEFER_SUMS=0 turns it off
        self.defer_sums = os.environ.get("MI_DEFER_SUMS", "1") == "1"
        # few rows: the residual-add + norm kernel's idle blocks request the first bytes of the weight that the next
        # product streams into L2 (MI_L2_AHEAD_MB=0 turns it off)
        self.l2_ahead_bytes = int(float(os.environ.get("MI_L2_AHEAD_MB", "32")) * (1 << 20))
        self.l2_ahead_max_rows = 64
        self.skinny_gemm = True              # few-row products on this package's weight-streaming kernel ...
        self.skinny_max_rows, self.skinny_max_cols = 16, 4096    # ... where it is at least as fast as the library's
        self.fast_attention = True           # tests clear this to run the generic attention kernels in bfloat16
        self.biased_attention_tc = True      # prompts of attention with a distance table or a learned sink on the tensor cores (bfloat16)
        self._zero_bias = {}
        # Latent attention whose cached rows have 64 or 128 entries can run on the tensor-core paged attention kernels.  Those
        # round the softmax weights to bfloat16 before the weighted sum; a design that asks for float32 weights gets the
        # float32 kernels of csrc/attention_latent.cu unless MI_LATENT_TC=1 (or this flag) says otherwise.
        self.latent_tc = os.environ.get("MI_LATENT_TC", "0") == "1"
        # the grouped products of routed experts on mma.sync tensor-core tiles (bfloat16); MI_MOE_TC=0: the CUDA-core form
        self.moe_tc = os.environ.get("MI_MOE_TC", "1") == "1" and hasattr(self.lib, "mi_moe_gemm_tc")
        # ... and, where an expert gets many rows, on tcgen05 tiles of 128 sorted rows (csrc/moe_grouped_tc.cu); MI_MOE_TCGEN05=0: never
        self.moe_tcgen05 = os.environ.get("MI_MOE_TCGEN05", "1") == "1"
        self.launches = 0                    # kernels of this package launched so far

    def _stream(self):
        # the raw handle of torch's current stream on this device: one C call (torch.cuda.current_stream builds a
        # Stream object every time, which at ~10 launches per layer was a fifth of an eager decode step's host time)
        return _c.c_void_p(_raw_stream(self._device_index))

    # ---------------------------------------------------------------- elementwise / norms
    def scatter_i32(self, table, idx, val):
        """table[idx[i]] = val[i]: the block-table entries that changed since the last step (cache/manager.py)."""
        n = idx.shape[0]
        if n:
            _check(self.lib.mi_scatter_i32(_p(table), _p(idx), _p(val), n, _c.c_longlong(table.numel()), self._stream()),
                   "scatter_i32")
            self.launches += 1

    def embedding(self, ids, table):
        T, hidden = ids.shape[0], table.shape[1]
        out = torch.empty((T, hidden), dtype=table.dtype, device=table.device)
        _check(self.lib.mi_embedding(_p(ids), _p(table), _p(out), T, hidden, table.shape[0], _code(table.dtype),
                                     self._stream()), "embedding")
        self.launches += 1
        return out

    def add_rmsnorm(self, x, delta, weight, eps, rows=None, next_weight=None):
        """x += delta (if any), y = rmsnorm(x) * weight.  next_weight: the tensor that the caller's next kernel streams; at
        few rows the kernel's idle blocks ask for its first bytes to be brought into L2 (a hint, never needed)."""
        hidden = x.shape[-1]
        ahead, ahead_bytes = None, 0
        if next_weight is not None and self.l2_ahead_bytes and x.shape[0] <= self.l2_ahead_max_rows and next_weight.is_contiguous():
            ahead, ahead_bytes = next_weight, min(next_weight.numel() * next_weight.element_size(), self.l2_ahead_bytes)
        if isinstance(delta, DeferredSum):
            if rows is None and x.dtype == torch.bfloat16 and x.is_contiguous() and hidden % 4 == 0 and delta.shape == tuple(x.shape):
                y = torch.empty_like(x)
                rc = self.lib.mi_deferred_add_rmsnorm(_p(x), _p(delta.ws), _p(weight), _p(y), delta.M, delta.N, delta.K, delta.grid,
                                                      delta.max_contrib, delta.tok, _c.c_float(eps), _code(weight.dtype),
                                                      _p(ahead), _c.c_longlong(ahead_bytes), self._stream())
                if rc == 0:
                    self.launches += 1
                    return y
                if rc != -2:
                    _check(rc, "deferred_add_rmsnorm")
            delta = self.materialize(delta)
        assert x.is_contiguous() and (delta is None or delta.is_contiguous())
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, hidden), dtype=x.dtype, device=x.device)
        _check(self.lib.mi_add_rmsnorm_ahead(_p(x), _p(delta), _p(weight), _p(y), _p(rows), n, hidden, _c.c_float(eps),
                                             _code(x.dtype), _code(weight.dtype), _p(ahead), _c.c_longlong(ahead_bytes),
                                             self._stream()), "add_rmsnorm")
        self.launches += 1
        return y

    def gated_linear(self, x, w):
        """silu(g) * u with [g | u] = x @ w.T (w = [gate rows | up rows]).  Many rows with the own tcgen05 GEMM chosen for this shape:
        one kernel whose epilogue applies the activation (csrc/gemm_tc2.cu), so the [M, 2 I] product is never written;
        otherwise product, then swiglu (or, for a few rows, the activation kernel that adds the product's partial sums)."""
        M, K = x.shape
        inter = w.shape[0] // 2
        if (self._use_tc(M, w.shape[0], K) and K % 64 == 0 and inter % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            act = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
            rc = self.lib.mi_gemm_tc2_swiglu(_p(x), x.stride(0), _p(w), _p(act), M, inter, K, *self._tc2_scratch(), _p(self._stream_error), self._stream())
            if rc == 0:
                self.launches += 1
                return act
            if rc != -2:
                _check(rc, "gemm_tc2_swiglu")
        gu = self.linear(x, w, defer=True)
        if isinstance(gu, DeferredSum):          # the few-row product left its partial sums: the activation kernel adds them
            act = torch.empty((M, inter), dtype=torch.bfloat16, device=x.device)
            rc = self.lib.mi_deferred_swiglu(_p(gu.ws), _p(act), M, inter, gu.K, gu.grid, gu.max_contrib, gu.tok, self._stream())
            if rc == 0:
                self.launches += 1
                return act
            if rc != -2:
                _check(rc, "deferred_swiglu")
            gu = self.materialize(gu)
        return self.swiglu(gu)

    def materialize(self, value):
        """The bfloat16 tensor behind a DeferredSum (anything else is returned as it is)."""
        if not isinstance(value, DeferredSum):
            return value
        out = torch.empty((value.M, value.N), dtype=torch.bfloat16, device=value.device)
        _check(self.lib.mi_deferred_reduce(_p(value.ws), _p(out), value.M, value.N, value.K, value.grid, value.max_contrib,
                                           value.tok, self._stream()), "deferred_reduce")
        self.launches += 1
        return out

    def swiglu(self, gate_up):
        rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
        assert gate_up.is_contiguous()
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
        _check(self.lib.mi_swiglu(_p(gate_up), _p(out), rows, inter, _code(gate_up.dtype), self._stream()), "swiglu")
        self.launches += 1
        return out

    # ---------------------------------------------------------------- matrix products
    def linear(self, x, w, out_dtype=None, defer=False):
        """x [M, K] (rows may be strided), w [N, K] -> [M, N].  defer=True: the caller will use the result only as the
        `delta` of add_rmsnorm (or pass it through materialize); the answer may then be a DeferredSum."""
        if x.dtype == torch.float32:
            M, K = x.shape
            N = w.shape[0]
            assert x.stride(1) == 1 and w.is_contiguous() and w.dtype == torch.float32
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
            _check(self.lib.mi_gemm_f32_nt(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, self._stream()), "gemm_f32")
            self.launches += 1
            return out
        M, K = x.shape
        if (self._use_tc(M, w.shape[0], K) and K % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            out = self._gemm_tc(x, w, out_dtype or x.dtype)
            if out is not None:
                return out
        choice = self._linear_choice.get((self._row_bucket(M), w.shape[0], K)) if self._linear_choice else None
        if choice == "library":
            return self._library_linear(x, w, out_dtype)
        if (self.stream_gemm and choice in (None, "stream") and M <= 32 and w.shape[0] <= self.stream_max_cols and K % 64 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            out = self._gemm_stream(x, w, out_dtype or x.dtype, defer=defer and self.defer_sums and choice == "stream"
                                    and out_dtype in (None, torch.bfloat16) and w.shape[0] % 4 == 0)
            if out is not None:
                return out
        if (self.skinny_gemm and (choice == "skinny" or (choice is None and M <= self.skinny_max_rows
                                                         and w.shape[0] <= self.skinny_max_cols)) and M <= 64 and K % 32 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and w.is_contiguous() and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
            N = w.shape[0]
            od = out_dtype or x.dtype
            out = torch.empty((M, N), dtype=od, device=x.device)
            err = self.lib.mi_gemm_skinny(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, _code(od), self._stream())
            if err == 0:
                self.launches += 1
                return out
            if err != -2:
                _check(err, "gemm_skinny")
        return self._library_linear(x, w, out_dtype)

    @staticmethod
    def _library_linear(x, w, out_dtype):
        if out_dtype is not None and out_dtype != x.dtype:
            try:
                return torch.mm(x, w.t(), out_dtype=out_dtype)
            except TypeError:
                return torch.mm(x, w.t()).to(out_dtype)
        return torch.mm(x, w.t())

    ROW_BUCKETS = (1, 2, 4, 8, 16, 32)
    MANY_BUCKETS = (256, 512, 1024, 2048, 4096)

    def _many_bucket(self, M):
        for b in self.MANY_BUCKETS:
            if M <= b:
                return b
        return self.MANY_BUCKETS[-1]

    def _use_tc(self, M, N, K):
        if M < self.tc_min_rows:
            return False
        return self.tc_gemm or self._many_choice.get((self._many_bucket(M), N, K)) == "tc2"

    def tune_many_rows(self, weights, probes=None, iters=6, min_bytes=64 << 20):
        """Per weight shape and bucket of many rows (prompt steps), time the own two-block tcgen05 GEMM against the library
        GEMM on the model's own weights and remember where the own kernel wins.  probes: {(N, K): probe(rows) -> run(weight)}
        for products that run together with what follows them (gate/up with its activation, q/k/v with norm, rotation and
        cache write: own kernel with that in its epilogue against library product + separate kernel).  Shapes of less than
        min_bytes in all are left to the library (tiny models).  Returns the timings in microseconds."""
        probes = probes or {}
        report = {}
        if self.tc_mode != "auto":
            return report
        groups = {}
        for w in weights:
            if w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous() and w.shape[1] % 64 == 0 and w.shape[0] % 8 == 0:
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        saved, table = self.tc_gemm, {}
        try:
            self._many_choice = {}
            for (N, K), ws in groups.items():
                if len(ws) * N * K * 2 < min_bytes:
                    continue
                for M in self.MANY_BUCKETS:
                    if M * N * 2 > 512 << 20:              # a vocabulary-wide product never has this many rows
                        continue
                    x = torch.randn(M, K, device=ws[0].device, dtype=torch.bfloat16)
                    times = {}
                    for name in ("library", "tc2"):
                        self.tc_gemm = name == "tc2"
                        if (N, K) in probes:
                            probe = probes[(N, K)](M)
                            run = lambda i: probe(ws[i % len(ws)])
                        else:
                            run = lambda i: self.linear(x, ws[i % len(ws)])
                        times[name] = min(self._time_in_graph(run, iters) for _ in range(2))
                    if times["tc2"] < 0.97 * times["library"]:
                        table[(M, N, K)] = "tc2"
                    report[f"{N}x{K} M<={M}"] = {k: round(v, 1) for k, v in times.items()} | {"best": table.get((M, N, K), "library")}
        finally:
            self.tc_gemm = saved
        self._many_choice = table
        self.check_errors()
        return report

    def _row_bucket(self, M):
        for b in self.ROW_BUCKETS:
            if M <= b:
                return b
        return 0

    def tune_linear(self, weights, out_dtypes=None, iters=16, min_bytes=256 << 20, deferrable=(), gated=()):
        """Per weight shape and row-count bucket, time this package's few-row kernels against the
        library GEMM on the model's own weights and remember the fastest.  The reference does the
        same kind of start-up timing to choose a weight layout per shape
        (engine/core/fused_linear.py:51-94); rotating over the layers' real weights keeps the L2
        from flattering anyone.  weights: bfloat16 [N, K] tensors; out_dtypes: {(N, K): dtype}."""
        groups = {}
        for w in weights:
            if w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous():
                groups.setdefault((w.shape[0], w.shape[1]), []).append(w)
        saved = (self.stream_gemm, self.skinny_gemm, self.skinny_max_rows, self.skinny_max_cols, self.stream_max_cols)
        table, report = {}, {}
        try:
            self._linear_choice = None
            for (N, K), ws in groups.items():
                od = (out_dtypes or {}).get((N, K))
                # one weight cannot defeat the L2 by rotation; leave such shapes to the default rule
                if len(ws) * N * K * 2 < min_bytes:
                    continue
                for M in self.ROW_BUCKETS:
                    x = torch.randn(M, K, device=ws[0].device, dtype=torch.bfloat16)
                    times = {}
                    for name in ("library", "stream", "skinny"):
                        if name == "stream" and K % 64:
                            continue
                        if name == "skinny" and K % 32:
                            continue
                        self.stream_gemm, self.skinny_gemm = name == "stream", name == "skinny"
                        self.skinny_max_rows, self.skinny_max_cols, self.stream_max_cols = 64, 1 << 30, 1 << 30
                        run = lambda i: self.linear(x, ws[i % len(ws)], out_dtype=od)
                        if (N, K) in gated:
                            # a gate/up product is read by the activation only: the pair is timed, as it runs in a step
                            self._linear_choice = {(M, N, K): name}
                            run = lambda i: self.gated_linear(x, ws[i % len(ws)])
                        elif name == "stream" and (N, K) in deferrable and self.defer_sums and od in (None, torch.bfloat16):
                            # these products are read by a norm kernel that adds the partial sums itself
                            run = lambda i: self._gemm_stream(x, ws[i % len(ws)], torch.bfloat16, defer=True)
                        times[name] = min(self._time_in_graph(run, iters) for _ in range(2))
                        self._linear_choice = None
                    best = min(times, key=times.get)
                    if times[best] > 0.95 * times["library"]:      # an own kernel has to win clearly
                        best = "library"
                    table[(M, N, K)] = best
                    report[f"{N}x{K} M<={M}"] = {k: round(v, 2) for k, v in times.items()} | {"best": best}
        finally:
            self.stream_gemm, self.skinny_gemm, self.skinny_max_rows, self.skinny_max_cols, self.stream_max_cols = saved
        self._linear_choice = table
        self.check_errors()
        return report

    def _time_in_graph(self, fn, iters):
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            fn(0)
            fn(1)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(i)
        graph.replay()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(self.device)
        start.record()
        graph.replay()
        stop.record()
        torch.cuda.synchronize(self.device)
        return start.elapsed_time(stop) * 1e3 / iters

    def _gemm_stream(self, x, w, od, defer=False):
        """Persistent TMA weight-streaming product (csrc/gemm_stream.cu); None if the shape is not taken."""
        M, K = x.shape
        N = w.shape[0]
        plan = self._stream_plans.get((M, N, K))
        if plan is None:
            g, rt, mc = _c.c_int(), _c.c_int(), _c.c_int()
            rc = self.lib.mi_gemm_stream_plan(M, N, K, _c.byref(g), _c.byref(rt), _c.byref(mc))
            plan = self._stream_plans[(M, N, K)] = None if rc else (g.value, rt.value, mc.value)
        if not plan:
            return None
        grid, row_tiles, max_contrib = plan
        if row_tiles > self._stream_counters.numel():
            return None                      # more row tiles than the fixed counters cover: another kernel takes it
        tok = 8 if M <= 8 else 16 if M <= 16 else 32
        workspace = torch.empty(row_tiles * max_contrib * 128 * tok, dtype=torch.float32, device=x.device)
        if defer:
            rc = self.lib.mi_gemm_stream_deferred(_p(x), x.stride(0), _p(w), M, N, K, _p(workspace), _p(self._stream_error),
                                                  self._stream())
            if rc == 0:
                self.launches += 1
                return DeferredSum(workspace, M, N, K, grid, max_contrib, tok)
            if rc != -2:
                _check(rc, "gemm_stream_deferred")
        out = torch.empty((M, N), dtype=od, device=x.device)
        rc = self.lib.mi_gemm_stream(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, _code(od), _p(workspace),
                                     _p(self._stream_counters), _p(self._stream_error), self._stream())
        if rc == -2:
            return None
        _check(rc, "gemm_stream")
        self.launches += 1
        return out

    def _gemm_tc(self, x, w, od):
        """Two-block tcgen05 + TMA product for many rows (csrc/gemm_tc2.cu), bfloat16 result; None if the shape or the
        result type is not taken."""
        M, K = x.shape
        N = w.shape[0]
        if od != torch.bfloat16 or N % 8:
            return None
        out = torch.empty((M, N), dtype=od, device=x.device)
        rc = self.lib.mi_gemm_tc2(_p(x), x.stride(0), _p(w), _p(out), N, M, N, K, *self._tc2_scratch(), _p(self._stream_error), self._stream())
        if rc == -2:
            return None
        _check(rc, "gemm_tc2")
        self.launches += 1
        return out

    def _tc2_scratch(self):
        return (_p(self._tc2_ws), _c.c_longlong(self._tc2_ws.numel()), _p(self._tc2_counters), self._tc2_counters.numel())

    def check_errors(self):
        """Raises if a bounded wait inside a kernel ran out (synchronises the device)."""
        code = int(self._stream_error.item())
        if code != 0:
            self._stream_error.zero_()
            self._tc2_counters.zero_()
            raise RuntimeError(f"a pipeline wait inside a kernel ran out (code {code}: 1-2 gemm_stream, 21+ attention, 51-55 gemm_tc2, 61-63 grouped expert product)")

    # ---------------------------------------------------------------- q/k norm, rotation, cache write
    def qk_norm_rope_cache(self, qkv, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        T = qkv.shape[0]
        assert qkv.is_contiguous() and qkv.shape[1] == (H + 2 * KV) * D
        w_dtype = q_weight.dtype if q_weight is not None else qkv.dtype
        _check(self.lib.mi_qk_norm_rope_cache(
            _p(qkv), _p(q_weight), _p(k_weight), _p(inv_freq), _p(meta.positions), _p(meta.slots),
            _p(k_cache), _p(v_cache), T, H, KV, D, meta.page_size, _c.c_float(eps), _code(qkv.dtype),
            _code(w_dtype), self._stream()), "qk_norm_rope_cache")
        self.launches += 1
        return qkv[:, :H * D]

    # ---------------------------------------------------------------- attention over the pages
    def _cluster_fits(self, D, S, clusters):
        """Whether `clusters` clusters of S blocks of the staged decode kernel are resident at once, with the margin the
        kernel itself asks for (clusters are placed whole inside a GPC; a second wave costs more than the merge saves)."""
        key = (D, S)
        if key not in self._cluster_fit:
            self._cluster_fit[key] = int(self.lib.mi_attn_decode_cluster_fit(D, S))
        return clusters * 100 <= self._cluster_fit[key] * 92

    def choose_splits(self, ctas, max_kv_len, per_sm=2, cluster=False, head_dim=128):
        """Enough blocks to fill the GPU about twice, never more splits than the longest
        request has 256-key pieces (kernels/paged_attention/decode_triton.py:114-120).
        cluster: up to 8 splits can merge through distributed shared memory, which is worth more
        than finer splits while a split stays within ~1,000 keys (12.5 vs 14.8 us at batch 1, context 4096)."""
        if self.force_splits:
            return self.force_splits
        slots = per_sm * self.NUM_SMS                      # blocks resident at once
        most = max(1, min(math.ceil(max_kv_len / 256), 32))
        if ctas * most <= slots:
            return 8 if cluster and most > 8 and max_kv_len <= 8 * 1024 and self._cluster_fits(head_dim, 8, ctas) else most
        # more blocks than fit at once: take the fewest splits whose last wave is at least 85 % full
        best, best_eff = 1, 0.0
        for S in range(1, most + 1):
            total = ctas * S
            eff = total / (math.ceil(total / slots) * slots)
            if eff >= 0.85:
                # one split fewer if that lets the splits merge as clusters
                if cluster and 2 < S <= 8 and not self._cluster_fits(head_dim, S, ctas) and self._cluster_fits(head_dim, S - 1, ctas):
                    return S - 1
                return S
            if eff > best_eff:
                best, best_eff = S, eff
        return best

    def qkv_project(self, h, w, H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache):
        """q [T, H D] (a strided view is allowed) = rotated(normed(h @ w_q.T)); rotated(normed(k)) and v go to the rows' slots
        of the caches (None: this layer writes none).  The product, then the norm / rotation / cache-write kernel; one entry,
        so that the start-up timing of kernels sees the pair (a version with all of it in the GEMM's epilogue was measured
        and dropped: 76-92 us against 59 us for the pair at 2,048 rows)."""
        return self.qk_norm_rope_cache(self.linear(h, w), H, KV, D, q_weight, k_weight, eps, inv_freq, meta, k_cache, v_cache)

    def paged_attention(self, q, k_cache, v_cache, meta, H, KV, D, scale, window, split_weights=False):
        """split_weights: the tensor-core kernels take every softmax weight into the P V product as TWO bfloat16 numbers (its
        rounding and the rest: 16 mantissa bits, float32 sums) instead of one; the tcgen05 prompt kernel, which has no such
        form, is left out.  The float32 kernels behind them compute the weights in float32 anyway.
        meta: the step's arrays for this cache group.  seg_q_start, seg_pos0, seg_kv_len per entry; decode_segs (entries
        that feed one token), prefill_tiles / prefill_tiles2 ((entry, first row) per tile of meta.tile / 2 * meta.tile query
        rows); block_table [rows, max_pages] with entry i reading row table_rows[i] (row i when table_rows is None)."""
        T = q.shape[0]
        assert q.stride(1) == 1
        out = torch.empty((T, H * D), dtype=q.dtype, device=q.device)
        code, win = _code(q.dtype), int(window or 0)
        rows = getattr(meta, "table_rows", None)
        num_decode, num_tiles = meta.decode_segs.shape[0], meta.prefill_tiles.shape[0]
        tiles2 = getattr(meta, "prefill_tiles2", None)
        num_tiles2 = 0 if tiles2 is None else tiles2.shape[0]
        fast = (self.fast_attention and q.dtype == torch.bfloat16 and D in (64, 128) and q.stride(0) % 8 == 0
                and q.data_ptr() % 16 == 0)
        tc = (fast and self.tc_attention and num_tiles and meta.tile == 64 and meta.page_size % 8 == 0
              and 64 % meta.page_size == 0 and num_tiles2 and not split_weights)
        if tc:
            rc = self.lib.mi_attn_prefill_tc(
                _p(q), q.stride(0), T, _p(k_cache), _p(v_cache), _c.c_longlong(k_cache.shape[0] * KV * meta.page_size),
                _p(out), _p(tiles2), num_tiles2, _p(meta.seg_q_start), _p(meta.seg_pos0),
                _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, meta.page_size, 128, _c.c_float(scale), win,
                _p(self._stream_error), self._stream())
            _check(rc, "attn_prefill_tc")
            self.launches += 1
        elif num_tiles and fast and meta.tile == 64:
            _check((self.lib.mi_attn_prefill_mma_split if split_weights else self.lib.mi_attn_prefill_mma)(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles,
                _p(meta.seg_q_start), _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D,
                meta.page_size, meta.tile, _c.c_float(scale), win, self._stream()), "attn_prefill_mma")
            self.launches += 1
        elif num_tiles:
            _check(self.lib.mi_attn_prefill_generic(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles,
                _p(meta.seg_q_start), _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D,
                meta.page_size, meta.tile, _c.c_float(scale), win, code, self._stream()), "attn_prefill")
            self.launches += 1
        if not num_decode:
            return out
        fast_decode = fast and H // KV <= 16 and meta.page_size % 16 == 0
        S = self.choose_splits(num_decode * (KV if fast_decode else math.ceil(H / 4)), meta.max_kv_len,
                               (2 if self.bulk_decode else 3) if fast_decode else 2,
                               cluster=fast_decode and self.bulk_decode and self.cluster_merge, head_dim=D)
        o_part = lse = None
        if S > 1:
            o_part = torch.empty((num_decode, H, S, D), dtype=torch.float32, device=q.device)
            lse = torch.empty((num_decode, H, S), dtype=torch.float32, device=q.device)
        if fast_decode:
            counters = None
            if S > 1 and self.fused_merge:
                if num_decode * KV > self._merge_counters.numel():
                    raise ValueError(f"attn_decode: {num_decode} rows x {KV} kv heads exceed the {self._merge_counters.numel()} "
                                     "merge counters allocated at start-up")
                counters = self._merge_counters
            # without counters the splits stay in o_part / lse for the merge launch below: the cluster merge must be off too
            cluster = int(self.cluster_merge and counters is not None)
            _check((self.lib.mi_attn_decode_mma_rows_split if split_weights else self.lib.mi_attn_decode_mma_rows)(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(o_part), _p(lse), _p(meta.decode_segs),
                num_decode, _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(rows), meta.max_pages,
                H, KV, D, meta.page_size, S, _c.c_float(scale), win, _p(counters),
                _p(self._stream_error if self.bulk_decode else None), k_cache.shape[0], cluster, self._stream()),
                "attn_decode_mma")
            self.launches += 1
            if S > 1 and counters is None:
                _check(self.lib.mi_attn_decode_merge(_p(o_part), _p(lse), _p(out), _p(meta.decode_segs), num_decode,
                                                     _p(meta.seg_q_start), H, D, S, code, self._stream()), "attn_merge")
                self.launches += 1
        else:
            _check(self.lib.mi_attn_decode_generic(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(o_part), _p(lse), _p(meta.decode_segs),
                num_decode, _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(rows), meta.max_pages,
                H, KV, D, meta.page_size, S, _c.c_float(scale), win, code, self._stream()), "attn_decode")
            self.launches += 2 if S > 1 else 1
        return out

    # ---------------------------------------------------------------- float32 stream, scalar norms, polynomial norm
    def embed_scaled_norm(self, ids, table, g, eps, out_dtype):
        """x = g * e / rms(e), e = table[ids]: the start of a residual stream (float32 [T, hidden] when out_dtype says so)."""
        T, hidden = ids.shape[0], table.shape[1]
        x = torch.empty((T, hidden), dtype=out_dtype, device=table.device)
        _check(self.lib.mi_embed_scaled_norm(_p(ids), _p(table), _p(g), _p(x), T, hidden, table.shape[0], _c.c_float(eps),
                                             _code(table.dtype), _code(out_dtype), self._stream()), "embed_scaled_norm")
        self.launches += 1
        return x

    def add_scaled_rmsnorm(self, x, delta, g, eps, rows, pre_add, out_dtype):
        """x (float32 stream) += delta (+ pre_add, a float32 [hidden] vector); y = g * x / rms(x) in out_dtype.
        rows: normalise only these rows and leave the stream untouched."""
        assert x.dtype == torch.float32 and x.is_contiguous() and (delta is None or delta.is_contiguous())
        hidden = x.shape[-1]
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
        _check(self.lib.mi_add_scaled_rmsnorm(_p(x), _p(delta), _p(pre_add), _p(g), _p(y), _p(rows), n, hidden, _c.c_float(eps),
                                              _code(delta.dtype if delta is not None else out_dtype), _code(out_dtype),
                                              self._stream()), "add_scaled_rmsnorm")
        self.launches += 1
        return y

    def polynorm(self, z, coef, eps):
        """a N(z) + b N(z^2) + c N(z^3) + e per row, N(y) = y / rms(y); coef = float32 (a, b, c, e) on the device."""
        assert z.is_contiguous()
        out = torch.empty_like(z)
        _check(self.lib.mi_polynorm(_p(z), _p(coef), _p(out), z.shape[0], z.shape[1], _c.c_float(eps), _code(z.dtype), self._stream()),
               "polynorm")
        self.launches += 1
        return out

    def group_rmsnorm_gate(self, o, weight, gate, eps, groups, gs, out_dtype, act="sigmoid"):
        """o float32 [T, groups * gs] -> o / rms(o over each group) * weight * act(gate) in out_dtype.  weight has
        groups * gs entries (one vector for the row), gs (shared by the groups) or is None (no weight); gate [T, groups * gs]
        may be a strided view; act: "sigmoid" or "silu"."""
        T = o.shape[0]
        assert o.dtype == torch.float32 and o.is_contiguous() and gate.stride(1) == 1 and gate.dtype == out_dtype
        y = torch.empty((T, groups * gs), dtype=out_dtype, device=o.device)
        _check(self.lib.mi_group_rmsnorm_gate(_p(o), _p(weight), 1 if weight is None else weight.numel(), _p(gate), gate.stride(0), _p(y),
                                              T, groups, gs, _c.c_float(eps), _code(out_dtype), {"sigmoid": 0, "silu": 1}[act],
                                              self._stream()), "group_rmsnorm_gate")
        self.launches += 1
        return y

    def head_gate(self, o, gate, out_dtype):
        """o [H, T, V], gate [T, H] (a strided view is allowed) -> rows [T, H V] = o * sigmoid(gate) per head; gate None: the
        heads laid side by side as they are."""
        H, T, V = o.shape
        assert o.is_contiguous() and o.dtype == out_dtype and (gate is None or (gate.stride(1) == 1 and gate.dtype == out_dtype))
        y = torch.empty((T, H * V), dtype=out_dtype, device=o.device)
        _check(self.lib.mi_head_gate(_p(o), _p(gate), 0 if gate is None else gate.stride(0), _p(y), T, H, V, _code(out_dtype), self._stream()), "head_gate")
        self.launches += 1
        return y

    # ---------------------------------------------------------------- matrix-state recurrences
    def lightning_scan(self, p, H, D, V, decay, state, batch):
        """p [T, >= 2 H D + H V] = q | k | v before silu; state float32 [slots, H D V] (an entry continues from its slot's
        state and leaves the new one there).  Returns float32 [T, H V]."""
        T = p.shape[0]
        assert p.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
        out = torch.empty((T, H * V), dtype=torch.float32, device=p.device)
        prep = torch.empty((T, 2 * H * D + H * V), dtype=torch.float32, device=p.device)      # silu(q | k | v), what the scan stages
        _check(self.lib.mi_lightning_scan(_p(p), p.stride(0), _p(prep), _p(decay), _p(state), _c.c_longlong(state.stride(0)), _p(out),
                                          _p(batch.seg_q_start), _p(batch.seg_slot), T, batch.num_segs, H, D, V, _code(p.dtype),
                                          self._stream()), "lightning_scan")
        self.launches += 2
        return out

    def delta_prepare(self, p, a, conv, A_log, dt_bias, H, KV, D, V, taps, unit_eps, state, batch):
        """What enters the gated delta rule, in float32 per token: q | k (after convolution, silu, unit norm; q also
        * D^-1/2) | v (convolution, silu) | g = exp(-exp(A_log) softplus(a + dt_bias)) | beta = sigmoid (rows padded to a
        multiple of four floats, so that the scan can fetch them in 16-byte pieces).  The
        convolutions read the inputs before an entry's first token from the slot (behind the H D V state entries)
        and leave their last taps - 1 inputs there."""
        T = p.shape[0]
        C = 2 * KV * D + H * V
        assert p.stride(1) == 1 and a.stride(1) == 1 and a.dtype == p.dtype and state.is_contiguous()
        out = torch.empty((T, (C + H * D + H + 3) // 4 * 4), dtype=torch.float32, device=p.device)
        _check(self.lib.mi_delta_prepare(_p(p), p.stride(0), _p(a), a.stride(0), _p(conv), _p(A_log), _p(dt_bias), _p(state),
                                         _c.c_longlong(state.stride(0)), _c.c_longlong(H * D * V), _p(out), out.stride(0),
                                         _p(batch.token_seg), _p(batch.seg_q_start), _p(batch.seg_slot), T, batch.num_segs,
                                         H, KV, D, V, taps, _c.c_float(unit_eps), _code(p.dtype), self._stream()), "delta_prepare")
        self.launches += 2 if taps > 1 and not (T == batch.num_segs and T < 256) else 1
        return out

    def delta_scan(self, prep, H, KV, D, V, state, batch):
        """S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q per head, token by token.  float32 [T, H V]."""
        T = prep.shape[0]
        out = torch.empty((T, H * V), dtype=torch.float32, device=prep.device)
        _check(self.lib.mi_delta_scan(_p(prep), prep.stride(0), _p(state), _c.c_longlong(state.stride(0)), _p(out),
                                      _p(batch.seg_q_start), _p(batch.seg_slot), T, batch.num_segs, H, KV, D, V, self._stream()),
               "delta_scan")
        self.launches += 1
        return out

    # ---------------------------------------------------------------- latent attention
    def batched_linear(self, x, col0, head_stride, K, w, side_by_side=False):
        """One product per head: w [H, N, K]; x is [T, ...] with head h's K inputs at columns col0 + h * head_stride
        (col0 given), or [H, T, K].  Returns [H, T, N], or with side_by_side [T, H N] (the heads' outputs laid side by side in
        each token's row, written there by the products themselves).  bfloat16: the library's batched product; float32: this
        package's float32 product, head by head (no reduced-precision mode)."""
        H, N, _ = w.shape
        if col0 is not None:
            T = x.shape[0]
            xs = torch.as_strided(x, (H, T, K), (head_stride, x.stride(0), 1), x.storage_offset() + col0)
        else:
            T, xs = x.shape[1], x
        if side_by_side:
            rows = torch.empty((T, H * N), dtype=x.dtype, device=x.device)
            out = rows.view(T, H, N).transpose(0, 1)                     # [H, T, N] with a row stride of H N
        if x.dtype != torch.float32:
            if side_by_side:
                torch.bmm(xs, w.transpose(1, 2), out=out)
                return rows
            return torch.bmm(xs, w.transpose(1, 2))
        if not side_by_side:
            out = torch.empty((H, T, N), dtype=torch.float32, device=x.device)
        for h in range(H):
            _check(self.lib.mi_gemm_f32_nt(_p(xs[h]), xs.stride(1), _p(w[h]), _p(out[h]), out.stride(1), T, N, K, self._stream()), "gemm_f32")
        self.launches += H
        return rows if side_by_side else out

    def latent_prepare(self, p, q_abs, H, D, R, C, norm_w, eps, inv_freq, meta, cache, q_rows=None, dkv_col=None):
        """p [T, ..] = q heads [H, D + R] | dkv [C + R] | ..; q_abs [H, T, C].  Returns q [T, H, C + R] = [q_abs | rotated
        q part]; writes the token's cache row [rmsnorm(dkv[:C]) * norm_w | rotated dkv[C:]] at its slot (cache None: no write).
        q_rows [T, H (D + R)]: the query heads lie in a tensor of their own; dkv_col: the column of p at which dkv starts."""
        T = p.shape[0]
        assert p.stride(1) == 1 and q_abs.is_contiguous() and (q_rows is None or (q_rows.stride(1) == 1 and q_rows.dtype == p.dtype))
        q = torch.empty((T, H, C + R), dtype=p.dtype, device=p.device)
        nf = 0 if inv_freq is None else inv_freq.numel()
        _check(self.lib.mi_latent_prepare(_p(p), p.stride(0), _p(q_rows), 0 if q_rows is None else q_rows.stride(0),
                                          -1 if dkv_col is None else int(dkv_col), _p(q_abs), _p(q), _p(cache), _p(norm_w), _p(inv_freq), nf,
                                          _p(meta.positions), _p(meta.slots), T, H, D, R, C, _c.c_float(eps), _code(p.dtype),
                                          self._stream()), "latent_prepare")
        self.launches += 1
        return q

    def latent_attention(self, q, cache, meta, H, C, R, scale):
        """q [T, H, C + R] over the cached rows [c | kr] (cache [pages, 1, page, C + R]); causal softmax; the weighted
        sum is over the rows' first C entries.  Returns [H, T, C]."""
        T = q.shape[0]
        if self.latent_tc and q.dtype == torch.bfloat16 and (C + R) in (64, 128) and meta.page_size % 16 == 0:
            # one shared key head of size C + R whose rows are also the values: the paged attention kernels on the tensor cores
            # take it as it is (the pool given as keys AND values); the last R columns of each head's output are dropped
            o = self.paged_attention(q.view(T, H * (C + R)), cache, cache, meta, H, 1, C + R, scale, None)
            return o.view(T, H, C + R)[:, :, :C].permute(1, 0, 2)
        num_decode, num_tiles = meta.decode_segs.shape[0], meta.prefill_tiles.shape[0]
        code, Dk = _code(q.dtype), C + R
        # Cached rows of 64 or 128 entries, bfloat16: the paged tensor-core kernels (mma.sync forms) with the pool as keys AND values
        # of one shared kv head and every softmax weight split into two bfloat16 numbers for the P V product, which keeps the
        # weights' precision where the design wants it; their output has C + R columns per head, of which the first C count.
        if (q.dtype == torch.bfloat16 and Dk in (64, 128) and meta.tile == 64 and self.fast_attention and meta.page_size % 16 == 0
                and q.data_ptr() % 16 == 0):
            if H <= 16 or not num_decode:
                o = self.paged_attention(q.view(T, H * Dk), cache, cache, meta, H, 1, Dk, scale, None, split_weights=True)
            else:
                # the decode kernel takes up to 16 query heads per key head as the rows of its tile: more heads go in groups of 16
                # (each group reads the cached rows once; the rows are small next to what the heads' weights cost)
                qv = q.view(T, H * Dk)
                o = torch.cat([self.paged_attention(qv[:, h0 * Dk:min(h0 + 16, H) * Dk], cache, cache, meta, min(16, H - h0), 1, Dk, scale, None,
                                                    split_weights=True) for h0 in range(0, H, 16)], dim=1)
            return o.view(T, H, Dk)[:, :, :C].permute(1, 0, 2)
        out = torch.empty((H, T, C), dtype=q.dtype, device=q.device)
        buf, hs, ts = out, T * C, C
        if num_tiles:
            _check(self.lib.mi_latent_prefill(_p(q), _p(cache), _p(buf), _p(meta.prefill_tiles), num_tiles, _p(meta.seg_q_start),
                                              _p(meta.seg_pos0), _p(meta.block_table), _p(meta.table_rows), meta.max_pages,
                                              _c.c_longlong(hs), _c.c_longlong(ts), H, C, R, meta.page_size, meta.tile,
                                              _c.c_float(scale), code, self._stream()), "latent_prefill")
            self.launches += 1
        if num_decode:
            S = self.choose_splits(num_decode * math.ceil(H / 4), meta.max_kv_len, 2)
            o_part = lse = None
            if S > 1:
                o_part = torch.empty((num_decode, H, S, C), dtype=torch.float32, device=q.device)
                lse = torch.empty((num_decode, H, S), dtype=torch.float32, device=q.device)
            _check(self.lib.mi_latent_decode(_p(q), _p(cache), _p(buf), _p(o_part), _p(lse), _p(meta.decode_segs), num_decode,
                                             _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(meta.table_rows),
                                             meta.max_pages, _c.c_longlong(hs), _c.c_longlong(ts), H, C, R, meta.page_size, S,
                                             _c.c_float(scale), code, self._stream()), "latent_decode")
            self.launches += 2 if S > 1 else 1
        return out

    # ---------------------------------------------------------------- float32 stream with norms on the sublayers' outputs
    def embed_stream(self, ids, table, rows_dtype):
        """(x, rows): x float32 [T, hidden] = table[ids], the start of a float32 residual stream, and the same rows in the
        run's dtype (x itself in a float32 run)."""
        T, hidden = ids.shape[0], table.shape[1]
        x = torch.empty((T, hidden), dtype=torch.float32, device=table.device)
        rows = None if rows_dtype == torch.float32 else torch.empty((T, hidden), dtype=table.dtype, device=table.device)
        assert table.dtype == rows_dtype
        _check(self.lib.mi_embed_stream(_p(ids), _p(table), _p(x), _p(rows), T, hidden, table.shape[0], _code(table.dtype),
                                        self._stream()), "embed_stream")
        self.launches += 1
        return x, (x if rows is None else rows)

    def cast_rows(self, x, dtype):
        assert x.dtype == torch.float32 and x.is_contiguous()
        y = torch.empty(x.shape, dtype=dtype, device=x.device)
        _check(self.lib.mi_cast_rows(_p(x), _p(y), _c.c_longlong(x.numel()), _code(dtype), self._stream()), "cast_rows")
        self.launches += 1
        return y

    def out_rmsnorm_add(self, x, y, weight, scale, mult, eps, rows_dtype):
        """x (float32 stream, in place) += mult * scale * (weight * y / rms(y)); scale None: no layer scale.  Returns x's rows in
        rows_dtype (x itself when that is float32)."""
        assert x.dtype == torch.float32 and x.is_contiguous() and y.is_contiguous() and y.shape == x.shape
        rows = None if rows_dtype == torch.float32 else torch.empty(x.shape, dtype=rows_dtype, device=x.device)
        _check(self.lib.mi_out_rmsnorm_add(_p(x), _p(y), _p(weight), _p(scale), _c.c_float(mult), _p(rows), x.shape[0], x.shape[1],
                                           _c.c_float(eps), _code(y.dtype), self._stream()), "out_rmsnorm_add")
        self.launches += 1
        return x if rows is None else rows

    def stream_rmsnorm(self, x, delta, weight, eps, rows, out_dtype):
        """x (float32 stream) += delta if given; y = weight * x / rms(x) in out_dtype.  rows: only these rows, stream untouched.
        A GatedDelta adds sigmoid(logits + bias) * (y + y_bias) instead, gate and sum in float32, in the same kernel."""
        hidden = x.shape[-1]
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
        if isinstance(delta, GatedDelta):
            d = delta
            assert x.dtype == torch.float32 and x.is_contiguous() and d.y.is_contiguous() and d.logits.is_contiguous() and d.y.dtype == d.logits.dtype
            assert d.y.shape == x.shape and d.logits.shape == x.shape and d.bias.dtype == torch.float32
            _check(self.lib.mi_stream_rmsnorm_gated(_p(x), _p(d.y), _p(d.logits), _p(d.bias), _p(d.y_bias), _p(weight), _p(y), _p(rows), n, hidden,
                                                    _c.c_float(eps), _code(d.y.dtype), _code(out_dtype), self._stream()), "stream_rmsnorm_gated")
            self.launches += 1
            return y
        assert x.dtype == torch.float32 and x.is_contiguous() and (delta is None or delta.is_contiguous())
        _check(self.lib.mi_stream_rmsnorm(_p(x), _p(delta), _p(weight), _p(y), _p(rows), n, hidden, _c.c_float(eps),
                                          _code(delta.dtype if delta is not None else out_dtype), _code(out_dtype), self._stream()),
               "stream_rmsnorm")
        self.launches += 1
        return y

    # ---------------------------------------------------------------- attention with a block mask, a sink and unit-norm q, k
    def unit_qk_cache(self, p, H, KV, D, V, eps, lam, source, meta, k_cache, v_cache, q_weight=None, k_weight=None, q_temp=None,
                      values_are_keys=False):
        """p [T, H D + KV D + KV V] = q | k | v.  q and k are divided by their root mean square per head (eps None: left as they
        are), q in place; v becomes (1 - lam) v + lam source when source [T, KV V] (another layer's values, a view is allowed) is
        given; k and v go to the rows' slots of the caches (None: this layer writes none).  Returns the q view.
        q_weight, k_weight float32 [D]: multiplied in after the division (shared by all heads); q_temp (coef, every): q at position p
        is multiplied by 1 + coef * ln(floor((p + 1) / every) + 1); values_are_keys: p has no v columns and the cached values are
        the keys as projected, before the norm."""
        T = p.shape[0]
        assert p.is_contiguous() and p.shape[1] == (H + KV) * D + (0 if values_are_keys else KV * V)
        assert source is None or (source.stride(1) == 1 and source.dtype == p.dtype and lam is not None)
        assert q_weight is None or (q_weight.dtype == k_weight.dtype == torch.float32 and q_weight.numel() == k_weight.numel() == D)
        coef, every = q_temp if q_temp else (0.0, 0)
        _check(self.lib.mi_normed_qk_cache(_p(p), p.stride(0), _p(source), 0 if source is None else source.stride(0), _p(lam if source is not None else None),
                                           _p(meta.slots), _p(k_cache), _p(v_cache), T, H, KV, D, V, meta.page_size,
                                           _c.c_float(eps or 0.0), int(eps is not None), _p(q_weight), _p(k_weight), _p(meta.positions if q_temp else None),
                                           _c.c_float(coef), int(every), int(bool(values_are_keys)), _code(p.dtype), self._stream()), "unit_qk_cache")
        self.launches += 1
        return p[:, :H * D]

    def masked_attention(self, q, k_cache, v_cache, meta, H, KV, D, V, scale, block_size, window, sink, sink_values=None, distance_bias=None,
                         distance_bias_by_head=None, distance_slopes=None):
        """q [T, H D] (a strided view is allowed) over the pages; keys of D and values of V entries; block_size / window / sink as
        csrc/attention_masked.cu states them.  sink_values float32 [H]: the sink's score per head (None: 0); distance_bias float32
        [far + 1, H]: added to the scaled score by the distance i - j (beyond far: the last row); distance_bias_by_head: the same
        table as float32 [H, far + 1], for the kernels that read it along the distance.  distance_slopes float32 [H]: slope_h * (i - j)
        is taken off the scaled score of head h.  Scores, weights and sums are float32.  Returns [T, H V]."""
        T = q.shape[0]
        assert q.stride(1) == 1
        out = torch.empty((T, H * V), dtype=q.dtype, device=q.device)
        code, blk, win = _code(q.dtype), int(block_size or 0), int(window or 0)
        rows = getattr(meta, "table_rows", None)
        num_decode, num_tiles = meta.decode_segs.shape[0], meta.prefill_tiles.shape[0]
        slopes = distance_slopes
        plain = sink_values is None and distance_bias is None and slopes is None
        if not plain:
            assert slopes is None or (slopes.dtype == torch.float32 and slopes.is_contiguous() and slopes.numel() == H)
            assert sink_values is None or (sink and sink_values.dtype == torch.float32 and sink_values.numel() == H)
            assert distance_bias is None or (distance_bias.dtype == torch.float32 and distance_bias.is_contiguous() and distance_bias.shape[1] == H)
        bias_last = 0 if distance_bias is None else distance_bias.shape[0] - 1
        if (num_tiles and plain and self.fast_attention and q.dtype == torch.bfloat16 and D == V and D in (64, 128) and meta.tile == 64
                and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
            # key and value rows of 64 or 128 entries: the mma.sync prompt kernel, every softmax weight entering P V as two
            # bfloat16 numbers (float32 scores and softmax, 16 mantissa bits of each weight, float32 sums)
            _check(self.lib.mi_attn_prefill_mma_masked(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles, _p(meta.seg_q_start),
                _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, meta.page_size, meta.tile,
                _c.c_float(scale), win, blk, int(bool(sink)), self._stream()), "attn_prefill_mma_masked")
            self.launches += 1
        elif (num_tiles and self.fast_attention and self.biased_attention_tc and q.dtype == torch.bfloat16 and D == V and D in (64, 128)
                and meta.tile == 64 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
            # the same kernel with the learned sink's score and the distance table (one row per head) in its softmax
            no_table = slopes is not None and distance_bias is None and distance_bias_by_head is None        # slopes alone: the kernel reads no table
            bias_t = None if no_table else self._bias_rows_by_head(distance_bias, distance_bias_by_head, H, q.device)
            args = (_p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles, _p(meta.seg_q_start),
                    _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, meta.page_size, meta.tile,
                    _c.c_float(scale), win, blk, int(bool(sink)), _p(sink_values), _p(bias_t), 0 if no_table else bias_t.shape[1] - 1)
            if slopes is None:
                _check(self.lib.mi_attn_prefill_mma_biased(*args, self._stream()), "attn_prefill_mma_biased")
            else:                                          # a slope per head times the distance, beside (or instead of) the table
                _check(self.lib.mi_attn_prefill_mma_sloped(*args, _p(slopes), self._stream()), "attn_prefill_mma_sloped")
            self.launches += 1
        elif num_tiles:
            _check(self.lib.mi_masked_prefill(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(meta.prefill_tiles), num_tiles, _p(meta.seg_q_start),
                _p(meta.seg_pos0), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, V, meta.page_size, meta.tile,
                _c.c_float(scale), blk, win, int(bool(sink)), _p(sink_values), _p(distance_bias), bias_last, _p(slopes), code, self._stream()), "masked_prefill")
            self.launches += 1
        if not num_decode:
            return out
        reach = meta.max_kv_len if not blk else min(meta.max_kv_len, blk)              # the most keys a decoded token can see
        reach = reach if not win else min(reach, win)
        if ((plain or self.biased_attention_tc) and self.fast_attention and q.dtype == torch.bfloat16 and D == V and D in (64, 128) and H // KV <= 16
                and meta.page_size % 16 == 0 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0):
            # the tensor-core decode kernel (the G query heads of a kv head are the rows of one tile), split weights
            S = self.choose_splits(num_decode * KV, reach, 2 if self.bulk_decode else 3, cluster=self.bulk_decode and self.cluster_merge, head_dim=D)
            o_part = lse = counters = None
            if S > 1:
                o_part = torch.empty((num_decode, H, S, D), dtype=torch.float32, device=q.device)
                lse = torch.empty((num_decode, H, S), dtype=torch.float32, device=q.device)
                if self.fused_merge:
                    if num_decode * KV > self._merge_counters.numel():
                        raise ValueError(f"attn_decode: {num_decode} rows x {KV} kv heads exceed the {self._merge_counters.numel()} "
                                         "merge counters allocated at start-up")
                    counters = self._merge_counters
            args = (_p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(o_part), _p(lse), _p(meta.decode_segs), num_decode,
                    _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, meta.page_size, S,
                    _c.c_float(scale), win, _p(counters), _p(self._stream_error if self.bulk_decode else None), k_cache.shape[0],
                    int(self.cluster_merge and counters is not None), blk, int(bool(sink)))
            if plain:
                _check(self.lib.mi_attn_decode_mma_rows_masked(*args, self._stream()), "attn_decode_mma_masked")
            else:                                          # the learned sink's score and the distance table (one row per head) in the softmax
                if slopes is None:
                    bias_t = self._bias_rows_by_head(distance_bias, distance_bias_by_head, H, q.device)
                    _check(self.lib.mi_attn_decode_mma_rows_biased(*args, _p(sink_values), _p(bias_t), bias_t.shape[1] - 1, self._stream()),
                           "attn_decode_mma_biased")
                elif distance_bias is None and distance_bias_by_head is None:                 # slopes alone: the kernel reads no table
                    _check(self.lib.mi_attn_decode_mma_rows_sloped(*args, _p(sink_values), _p(None), 0, _p(slopes), self._stream()), "attn_decode_mma_sloped")
                else:
                    bias_t = self._bias_rows_by_head(distance_bias, distance_bias_by_head, H, q.device)
                    _check(self.lib.mi_attn_decode_mma_rows_sloped(*args, _p(sink_values), _p(bias_t), bias_t.shape[1] - 1, _p(slopes), self._stream()),
                           "attn_decode_mma_sloped")
            self.launches += 1
            if S > 1 and counters is None:
                _check(self.lib.mi_attn_decode_merge(_p(o_part), _p(lse), _p(out), _p(meta.decode_segs), num_decode,
                                                     _p(meta.seg_q_start), H, D, S, code, self._stream()), "attn_merge")
                self.launches += 1
            return out
        if num_decode:
            S = self.choose_splits(num_decode * math.ceil(H / 4), reach, 2)
            o_part = lse = None
            if S > 1:
                o_part = torch.empty((num_decode, H, S, V), dtype=torch.float32, device=q.device)
                lse = torch.empty((num_decode, H, S), dtype=torch.float32, device=q.device)
            _check(self.lib.mi_masked_decode(
                _p(q), q.stride(0), _p(k_cache), _p(v_cache), _p(out), _p(o_part), _p(lse), _p(meta.decode_segs), num_decode,
                _p(meta.seg_q_start), _p(meta.seg_kv_len), _p(meta.block_table), _p(rows), meta.max_pages, H, KV, D, V,
                meta.page_size, S, _c.c_float(scale), blk, win, int(bool(sink)), _p(sink_values), _p(distance_bias), bias_last, _p(slopes), code,
                self._stream()), "masked_decode")
            self.launches += 2 if S > 1 else 1
        return out

    def _bias_rows_by_head(self, distance_bias, by_head, H, device):
        """The distance table [far + 1, H] one row per head, [H, far + 1]: the caller's own copy if it keeps one, else made here;
        no table at all (a learned sink alone): one zero a head."""
        if by_head is not None:
            assert by_head.dtype == torch.float32 and by_head.is_contiguous() and by_head.shape[0] == H
            return by_head
        if distance_bias is not None:
            return distance_bias.t().contiguous()
        zero = self._zero_bias.get(H)
        if zero is None:
            zero = self._zero_bias[H] = torch.zeros((H, 1), dtype=torch.float32, device=device)
        return zero

    # ---------------------------------------------------------------- retention
    def retention_scan(self, p, H, D, V, inv_freq, k_scale, decay, state, batch):
        """p [T, >= 2 H D + H V] = q | k | v as projected.  q and k are rotated (rotate-half over the first 2 * len(inv_freq)
        coordinates of each head; inv_freq None: not at all), k is multiplied by k_scale, all in float32; then
        S <- decay_h S + k v^T, o = S^T q from the slot's state, which receives the new one.  Returns float32 [T, H V]."""
        T = p.shape[0]
        assert p.stride(1) == 1 and state.dtype == torch.float32 and state.is_contiguous()
        out = torch.empty((T, H * V), dtype=torch.float32, device=p.device)
        prep = torch.empty((T, 2 * H * D + H * V), dtype=torch.float32, device=p.device)
        half = 0 if inv_freq is None else inv_freq.numel()
        _check(self.lib.mi_retention_scan(_p(p), p.stride(0), _p(prep), _p(batch.positions), _p(inv_freq), half, _c.c_float(k_scale),
                                          _p(decay), _p(state), _c.c_longlong(state.stride(0)), _p(out), _p(batch.seg_q_start),
                                          _p(batch.seg_slot), T, batch.num_segs, H, D, V, _code(p.dtype), self._stream()),
               "retention_scan")
        self.launches += 2
        return out

    # ---------------------------------------------------------------- routed experts
    def route_topk(self, h, router, correction, top, groups, score=None, extra_rows=0, group_score="max", renormalise=False, weight_eps=0.0,
                   route_scale=1.0):
        """(chosen int32 [T, top], weights float32 [T, top]).  router [E, hidden] in the dtype of h, correction float32 [E] or None;
        groups None or (count, keep).  Products, sums, scores and the choice are float32 (csrc/moe.cu).  Called with `score`
        ("softmax" or "sigmoid") it answers (chosen, weights, extra): the router matrix then has extra_rows more rows behind the
        experts' and extra float32 [T, extra_rows] holds their logits (None without extra rows).  group_score "top2_sum": a group is
        ranked by the sum of its two largest choice scores; renormalise: the weights are divided by their sum + weight_eps; route_scale
        multiplies them last."""
        T, E = h.shape[0], router.shape[0] - extra_rows
        assert h.stride(1) == 1 and router.dtype == h.dtype and router.is_contiguous() and (correction is None or correction.dtype == torch.float32)
        chosen = torch.empty((T, top), dtype=torch.int32, device=h.device)
        weights = torch.empty((T, top), dtype=torch.float32, device=h.device)
        extra = torch.empty((T, extra_rows), dtype=torch.float32, device=h.device) if extra_rows else None
        count, keep = groups if groups else (0, 0)
        _check(self.lib.mi_route_topk(_p(h), h.stride(0), _p(router), _p(correction), _p(chosen), _p(weights), T, h.shape[1], E, top,
                                      count, keep, int(score == "sigmoid"), extra_rows, _p(extra), int(group_score == "top2_sum"),
                                      int(bool(renormalise)), _c.c_float(weight_eps), _c.c_float(route_scale), _code(h.dtype), self._stream()),
               "route_topk")
        self.launches += 1
        return (chosen, weights) if score is None else (chosen, weights, extra)

    def clamped_glu(self, gu, limit, slope):
        """[g | u] -> min(g, limit) * sigmoid(slope * min(g, limit)) * (clamp(u, -limit, limit) + 1)."""
        rows, inter = gu.shape[0], gu.shape[1] // 2
        assert gu.is_contiguous()
        out = torch.empty((rows, inter), dtype=gu.dtype, device=gu.device)
        _check(self.lib.mi_clamped_glu(_p(gu), _p(out), rows, inter, _c.c_float(limit), _c.c_float(slope), _c.c_float(1.0), _code(gu.dtype),
                                       self._stream()), "clamped_glu")
        self.launches += 1
        return out

    def expert_ffn(self, h, chosen, weights, w_in, w_out, limit, slope, shared, up_shift=1.0, weight_on_input=False, shared_gate=None):
        """sum_j weights[t, j] * expert_{chosen[t, j]}(h[t]) (+ shared[t]).  w_in [E, 2 F, hidden] (gate rows | up rows),
        w_out [E, hidden, F].  The (token, choice) pairs are sorted by expert on the device; two grouped products run over the
        sorted rows, the first with the gated activation min(g, limit) sigmoid(slope g) (clamp(u) + up_shift) in its epilogue;
        nothing returns to the host.  weight_on_input: sum_j expert(weights[t, j] * h[t]) instead (the rows are scaled where they
        are gathered, the sum is unweighted).  shared_gate float32 [T, 1]: shared[t] is multiplied by sigmoid of it."""
        T, top = chosen.shape
        sh = _c.c_float(up_shift)
        sum_weights = None if weight_on_input else weights
        sg = None if shared_gate is None else shared_gate.reshape(-1)
        assert sg is None or (sg.dtype == torch.float32 and sg.is_contiguous() and sg.numel() == T and shared is not None)
        E, F2, K = w_in.shape
        F, hidden = F2 // 2, w_out.shape[1]
        assert h.stride(1) == 1 and w_in.is_contiguous() and w_out.is_contiguous() and K == h.shape[1] and w_in.dtype == h.dtype
        P, code, dev = T * top, _code(h.dtype), h.device
        if (h.dtype == torch.bfloat16 and self.moe_tcgen05 and P > 48 * E and K % 64 == 0 and F % 64 == 0 and hidden % 8 == 0
                and h.stride(0) % 8 == 0 and h.data_ptr() % 16 == 0):
            # many rows per expert: tiles of 128 sorted rows on the tcgen05 tensor cores (csrc/moe_grouped_tc.cu)
            cap_tiles = (P + 127) // 128 + min(E, P)
            cap_pos = cap_tiles * 128
            sorted_pair = torch.empty(cap_pos, dtype=torch.int32, device=dev)
            tile_expert = torch.empty(cap_tiles, dtype=torch.int32, device=dev)
            _check(self.lib.mi_moe_align(_p(chosen), P, E, 128, _p(sorted_pair), cap_pos, _p(tile_expert), cap_tiles, self._stream()), "moe_align")
            a = torch.empty((cap_pos, K), dtype=h.dtype, device=dev)
            _check(self.lib.mi_moe_gather_rows(_p(h), h.stride(0), _p(sorted_pair), top, _p(a), cap_pos, K, _p(weights if weight_on_input else None), self._stream()), "moe_gather_rows")
            y = torch.empty((cap_pos, F), dtype=h.dtype, device=dev)
            rows = torch.empty((P, hidden), dtype=h.dtype, device=dev)
            _check(self.lib.mi_moe_gemm_tcgen05(_p(a), _p(w_in), E, _p(y), F, _p(sorted_pair), _p(tile_expert), cap_tiles, F, K,
                                                _c.c_float(limit), _c.c_float(slope), sh, 0, _p(self._stream_error), self._stream()), "moe_gemm_tcgen05 (in)")
            _check(self.lib.mi_moe_gemm_tcgen05(_p(y), _p(w_out), E, _p(rows), hidden, _p(sorted_pair), _p(tile_expert), cap_tiles, hidden, F,
                                                _c.c_float(limit), _c.c_float(slope), sh, 1, _p(self._stream_error), self._stream()), "moe_gemm_tcgen05 (out)")
            out = torch.empty((T, hidden), dtype=h.dtype, device=dev)
            assert shared is None or (shared.is_contiguous() and shared.shape == out.shape)
            _check(self.lib.mi_moe_combine(_p(rows), _p(sum_weights), _p(shared), _p(sg), _p(out), T, hidden, top, code, self._stream()), "moe_combine")
            self.launches += 5
            return out
        src, src_top = h, top
        if weight_on_input:                                # row p = weights[p] * h[p // top]; the products then see one choice per row
            src = torch.empty((P, K), dtype=h.dtype, device=dev)
            _check(self.lib.mi_moe_scale_rows(_p(h), h.stride(0), _p(weights), top, _p(src), P, K, code, self._stream()), "moe_scale_rows")
            src_top = 1
            self.launches += 1
        tc = h.dtype == torch.bfloat16 and self.moe_tc and K % 64 == 0 and F % 64 == 0 and hidden % 2 == 0 and src.stride(0) % 8 == 0
        BM = int(self.lib.mi_moe_tile_rows_tc(P, E) if tc else self.lib.mi_moe_tile_rows_simt())
        cap_tiles = (P + BM - 1) // BM + min(E, P)
        cap_pos = cap_tiles * BM
        sorted_pair = torch.empty(cap_pos, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(cap_tiles, dtype=torch.int32, device=dev)
        _check(self.lib.mi_moe_align(_p(chosen), P, E, BM, _p(sorted_pair), cap_pos, _p(tile_expert), cap_tiles, self._stream()), "moe_align")
        y = torch.empty((cap_pos, F), dtype=h.dtype, device=dev)
        rows = torch.empty((P, hidden), dtype=h.dtype, device=dev)
        gemm = self.lib.mi_moe_gemm_tc if tc else self.lib.mi_moe_gemm_simt
        extra = (BM,) if tc else ()
        _check(gemm(_p(src), src.stride(0), _p(w_in), _p(y), F, _p(sorted_pair), _p(tile_expert), cap_tiles, src_top, F, K,
                    _c.c_float(limit), _c.c_float(slope), sh, 0, *extra, code, self._stream()), "moe_gemm (in)")
        _check(gemm(_p(y), F, _p(w_out), _p(rows), hidden, _p(sorted_pair), _p(tile_expert), cap_tiles, src_top, hidden, F,
                    _c.c_float(limit), _c.c_float(slope), sh, 1, *extra, code, self._stream()), "moe_gemm (out)")
        out = torch.empty((T, hidden), dtype=h.dtype, device=dev)
        assert shared is None or (shared.is_contiguous() and shared.shape == out.shape)
        _check(self.lib.mi_moe_combine(_p(rows), _p(sum_weights), _p(shared), _p(sg), _p(out), T, hidden, top, code, self._stream()), "moe_combine")
        self.launches += 4
        return out

    # ---------------------------------------------------------------- hashed pair embedding, input filter, bias + activation, soft cap
    def embed_bigram_stream(self, ids, table, pairs, buckets, mul_prev, mul_cur, state, batch):
        """x float32 [T, hidden] = table[id] + pairs[(prev * mul_prev + id * mul_cur) mod buckets]; a token at position 0 takes row
        `buckets`.  prev of an entry's first token is what its slot of state (int32 [slots, 1]) remembers; the entry's last token is
        left there."""
        T, hidden = ids.shape[0], table.shape[1]
        assert state.dtype == torch.int32 and state.is_contiguous() and pairs.dtype == table.dtype and pairs.shape == (buckets + 1, hidden)
        x = torch.empty((T, hidden), dtype=torch.float32, device=table.device)
        _check(self.lib.mi_embed_pair_stream(_p(ids), _p(table), _p(pairs), _p(x), _p(state), _c.c_longlong(state.stride(0)), _p(batch.positions),
                                             _p(batch.token_seg), _p(batch.seg_q_start), _p(batch.seg_slot), T, hidden, table.shape[0],
                                             _c.c_longlong(buckets), _c.c_longlong(mul_prev), _c.c_longlong(mul_cur), _code(table.dtype),
                                             self._stream()), "embed_bigram_stream")
        self.launches += 1
        return x

    def short_conv(self, h, weight, bias, taps, state, offset, batch, residual=False, act="none"):
        """Causal convolution over time on every channel: out[t] = act(sum_j weight[:, j] h[t - taps + 1 + j] + bias) (+ h[t] when
        residual).  h [T, C] may be a strided view; weight float32 [C, taps]; the inputs before an entry's first token are read from
        state[slot, offset : offset + (taps - 1) C] (float32), which then receives the entry's last taps - 1 inputs."""
        T, C = h.shape
        assert h.stride(1) == 1 and weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape == (C, taps)
        assert state is None or (state.dtype == torch.float32 and state.is_contiguous())
        assert taps == 1 or state is not None
        out = torch.empty((T, C), dtype=h.dtype, device=h.device)
        _check(self.lib.mi_short_conv(_p(h), h.stride(0), _p(weight), _p(bias), _p(state), _c.c_longlong(state.stride(0) if state is not None else 0),
                                      _c.c_longlong(offset), _p(out), _p(batch.token_seg), _p(batch.seg_q_start), _p(batch.seg_slot), T,
                                      batch.num_segs, C, taps, int(residual), {"none": 0, "silu": 1}[act], _code(h.dtype), self._stream()),
               "short_conv")
        self.launches += 2 if taps > 1 else 1
        return out

    def bias_act(self, z, bias, act):
        """z + bias (float32 [cols]), then act: "none" or "relu2" (the square of relu)."""
        assert z.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == z.shape[-1]
        out = torch.empty_like(z)
        _check(self.lib.mi_bias_act(_p(z), _p(bias), _p(out), _c.c_longlong(z.numel() // z.shape[-1]), z.shape[-1], {"none": 0, "relu2": 1}[act],
                                    _code(z.dtype), self._stream()), "bias_act")
        self.launches += 1
        return out

    def embed_scaled_stream(self, ids, table, scale, pos_table, positions):
        """x float32 [T, hidden] = table[id] * scale + pos_table[position] (pos_table None: no positions): the start of a float32 stream."""
        T, hidden = ids.shape[0], table.shape[1]
        assert table.is_contiguous() and (pos_table is None or (pos_table.is_contiguous() and pos_table.dtype == table.dtype and pos_table.shape[1] == hidden))
        x = torch.empty((T, hidden), dtype=torch.float32, device=table.device)
        _check(self.lib.mi_embed_scaled_stream(_p(ids), _p(table), _c.c_float(scale), _p(pos_table), _p(positions), _p(x), T, hidden, table.shape[0],
                                               0 if pos_table is None else pos_table.shape[0], _code(table.dtype), self._stream()), "embed_scaled_stream")
        self.launches += 1
        return x

    def stream_rmsnorm_pair(self, x, a, b, bias, pre_add, weight, eps, rows, out_dtype):
        """x (float32 stream) += a + b + bias + pre_add, each of which may be None: a, b [T, hidden] outputs of two sublayers (one
        dtype), bias float32 [hidden], pre_add float32 [hidden] or [T, hidden]; y = weight * x / rms(x) in out_dtype.  rows: only these
        rows are normed and the stream is left as it is.  All sums are float32, in one kernel."""
        hidden = x.shape[-1]
        n = x.shape[0] if rows is None else rows.shape[0]
        y = torch.empty((n, hidden), dtype=out_dtype, device=x.device)
        assert x.dtype == torch.float32 and x.is_contiguous()
        for d in (a, b):
            assert d is None or (d.is_contiguous() and d.shape == x.shape)
        assert a is None or b is None or a.dtype == b.dtype
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == hidden)
        stride = 0
        if pre_add is not None:
            assert pre_add.dtype == torch.float32 and pre_add.is_contiguous() and pre_add.numel() in (hidden, x.numel())
            stride = hidden if pre_add.dim() == 2 else 0
        first = a if a is not None else b
        _check(self.lib.mi_stream_rmsnorm_pair(_p(x), _p(a), _p(b), _p(bias), _p(pre_add), _c.c_longlong(stride), _p(weight), _p(y), _p(rows), n, hidden,
                                               _c.c_float(eps), _code(first.dtype if first is not None else out_dtype), _code(out_dtype), self._stream()),
               "stream_rmsnorm_pair")
        self.launches += 1
        return y

    def rows_rmsnorm(self, x, weight, eps):
        """y = weight * x / rms(x) over the rows of x [T, n] (a strided view is allowed); y contiguous, in x's dtype; float32 statistics."""
        assert x.stride(1) == 1 and weight.dtype == torch.float32 and weight.numel() == x.shape[1]
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        _check(self.lib.mi_rows_rmsnorm(_p(x), _c.c_longlong(x.stride(0)), _p(weight), _p(y), x.shape[0], x.shape[1], _c.c_float(eps), _code(x.dtype),
                                        self._stream()), "rows_rmsnorm")
        self.launches += 1
        return y

    def bias_glu(self, gu, bias, act):
        """[g | u] (+ bias float32 [2 I], or None) -> act(g) * u, act one of relu, silu, gelu_tanh; float32 arithmetic."""
        rows, inter = gu.shape[0], gu.shape[1] // 2
        assert gu.is_contiguous() and (bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * inter))
        out = torch.empty((rows, inter), dtype=gu.dtype, device=gu.device)
        _check(self.lib.mi_bias_glu(_p(gu), _p(bias), _p(out), rows, inter, {"relu": 0, "silu": 1, "gelu_tanh": 2}[act], _code(gu.dtype),
                                    self._stream()), "bias_glu")
        self.launches += 1
        return out

    def scale_logits(self, logits, s):
        """logits <- logits * s, in place (float32)."""
        assert logits.dtype == torch.float32 and logits.is_contiguous()
        _check(self.lib.mi_scale_f32(_p(logits), _c.c_longlong(logits.numel()), _c.c_float(s), self._stream()), "scale_logits")
        self.launches += 1
        return logits

    def softcap(self, logits, cap):
        """logits <- cap * tanh(logits / cap), in place (float32)."""
        assert logits.dtype == torch.float32 and logits.is_contiguous()
        _check(self.lib.mi_softcap(_p(logits), _c.c_longlong(logits.numel()), _c.c_float(cap), self._stream()), "softcap")
        self.launches += 1
        return logits

    def dual_rmsnorm_mix(self, a, wa, sa, b, wb, sb, eps):
        """sa * wa * a / rms(a) + sb * wb * b / rms(b) over the rows of a and b (same shape and dtype), float32 statistics."""
        assert a.is_contiguous() and b.is_contiguous() and a.shape == b.shape and a.dtype == b.dtype
        out = torch.empty_like(a)
        _check(self.lib.mi_dual_rmsnorm_mix(_p(a), _p(wa), _c.c_float(sa), _p(b), _p(wb), _c.c_float(sb), _p(out), a.shape[0], a.shape[1],
                                            _c.c_float(eps), _code(a.dtype), self._stream()), "dual_rmsnorm_mix")
        self.launches += 1
        return out

    # ---------------------------------------------------------------- three more recurrences
    def general_delta_prepare(self, p, w2, w0, a_b, H, D, V, rank, decay_scale, unit_eps):
        """p [T, 3 H D + 2 H V + rank] = r | k | v | a | g | low.  Returns float32 [T, 5 H D + H V (padded to four)] =
        r | k | u | a u | decay | v with u = k / sqrt(sum k^2 + unit_eps) per head, a = sigmoid(. + a_b),
        decay = exp(-decay_scale * sigmoid(w2 tanh(low) + w0))."""
        T = p.shape[0]
        assert p.stride(1) == 1 and w2.is_contiguous() and w2.dtype == p.dtype and w2.shape == (H * D, rank)
        out = torch.empty((T, (5 * H * D + H * V + 3) // 4 * 4), dtype=torch.float32, device=p.device)
        _check(self.lib.mi_general_delta_prepare(_p(p), p.stride(0), _p(w2), _p(w0), _p(a_b), _p(out), out.stride(0), T, H, D, V, rank,
                                                 _c.c_float(decay_scale), _c.c_float(unit_eps), _code(p.dtype), self._stream()),
               "general_delta_prepare")
        self.launches += 1
        return out

    def general_delta_scan(self, prep, H, D, V, state, batch):
        """S <- diag(decay) S - (a u)(u^T S) + k v^T, both terms reading the old S; o = S^T r.  float32 [T, H V]."""
        T = prep.shape[0]
        assert prep.dtype == torch.float32 and state.dtype == torch.float32 and state.is_contiguous()
        out = torch.empty((T, H * V), dtype=torch.float32, device=prep.device)
        _check(self.lib.mi_general_delta_scan(_p(prep), prep.stride(0), _p(state), _c.c_longlong(state.stride(0)), _p(out), _p(batch.seg_q_start),
                                              _p(batch.seg_slot), T, batch.num_segs, H, D, V, self._stream()), "general_delta_scan")
        self.launches += 1
        return out

    def matrix_memory(self, p, gl, gate_bias, H, D, V, cap, den_eps, norm, gate, eps, state, batch, out_dtype):
        """p [T, >= 2 H D + H V] = q | k | v; gl float32 [T, 2 H] = logits of the input and forget gates; the slot holds per head
        [D, V + 4] floats (memory, normaliser column, three unused) and behind them the H running maxima.  Returns the rows
        o / rms(o) * norm * sigmoid(gate) per head in out_dtype (gate [T, H V] may be a strided view)."""
        T = p.shape[0]
        W = V + 4
        assert p.stride(1) == 1 and gate.stride(1) == 1 and gate.dtype == p.dtype == out_dtype and gl.dtype == torch.float32 and gl.is_contiguous()
        assert state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] >= H * D * W + H
        dev = p.device
        lg = torch.empty((T, 2 * H), dtype=torch.float32, device=dev)
        mneg = torch.empty((T, H), dtype=torch.float32, device=dev)
        prep = torch.empty((T, (2 * H * D + H * W + H + 3) // 4 * 4), dtype=torch.float32, device=dev)
        full = torch.empty((T, H * W), dtype=torch.float32, device=dev)
        y = torch.empty((T, H * V), dtype=out_dtype, device=dev)
        _check(self.lib.mi_matrix_memory(_p(p), p.stride(0), _p(gl), _p(gate_bias), _c.c_float(cap or 0.0), int(cap is not None), _c.c_float(den_eps),
                                         _p(norm), _p(gate), gate.stride(0), _c.c_float(eps), _p(lg), _p(mneg), _p(prep), prep.stride(0), _p(full),
                                         _p(y), _p(state), _c.c_longlong(state.stride(0)), _p(batch.seg_q_start), _p(batch.seg_slot), T,
                                         batch.num_segs, H, D, V, _code(p.dtype), self._stream()), "matrix_memory")
        self.launches += 3 if T == batch.num_segs else 5
        return y

    def selective_scan(self, x, dt, dt_b, A, B, C, Dv, z, state, batch, out_dtype):
        """S[c, n] <- exp(step_c A[c, n]) S[c, n] + step_c x_c B_n, step = softplus(dt + dt_b); y_c = sum_n S[c, n] C_n + Dv_c x_c;
        returns y * silu(z) in out_dtype.  x [T, I] contiguous; dt [T, I] in the run's dtype or float32; B, C [T, N] and z [T, I] may be
        strided views; A float32 [I, N]; the slot's first I N floats are S."""
        T, I = x.shape
        N = A.shape[1]
        assert x.is_contiguous() and x.dtype == out_dtype and B.stride(1) == 1 and C.stride(1) == 1 and z.stride(1) == 1
        assert A.dtype == torch.float32 and A.is_contiguous() and state.dtype == torch.float32 and state.is_contiguous()
        if dt.dtype != torch.float32:
            dt = dt.float()
        assert dt.is_contiguous()
        out = torch.empty((T, I), dtype=out_dtype, device=x.device)
        _check(self.lib.mi_selective_scan(_p(x), _p(dt), _p(dt_b), _p(A), _p(B), B.stride(0), _p(C), C.stride(0), _p(Dv), _p(z), z.stride(0),
                                          _p(state), _c.c_longlong(state.stride(0)), _p(out), _p(batch.seg_q_start), _p(batch.seg_slot), T,
                                          batch.num_segs, I, N, _code(x.dtype), self._stream()), "selective_scan")
        self.launches += 1
        return out

    # ---------------------------------------------------------------- sampling
    def argmax(self, logits):
        return self.sample(logits, None, None, None)

    def sample(self, logits, temperatures, seeds, counters):
        """logits float32 [R, V]; temperatures float32 [R] (0 = greedy); seeds, counters: int32
        tensors read as unsigned.  Returns int32 [R]."""
        assert logits.dtype == torch.float32 and logits.stride(1) == 1
        R, V = logits.shape
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
        if V >= 16384 and R <= 4096:                     # several blocks per row
            _check(self.lib.mi_sample_split(_p(logits), logits.stride(0), R, V, _p(temperatures), _p(seeds), _p(counters),
                                            _p(out), _p(self._sample_slots), _p(self._sample_arrivals), self._stream()),
                   "sample")
            self.launches += 1
            return out
        _check(self.lib.mi_sample(_p(logits), logits.stride(0), R, V, _p(temperatures), _p(seeds), _p(counters),
                                  _p(out), self._stream()), "sample")
        self.launches += 1
        return out


_OPS = {}


def get_ops(device) -> CudaOps:
    device = torch.device(device)
    key = (device.type, device.index)
    if key not in _OPS:
        _OPS[key] = CudaOps(device)
    return _OPS[key]
