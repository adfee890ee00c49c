#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B shape with random bfloat16 weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--impl ours|reference]

A "step" is one decode step of a batch of 8 requests whose contexts start at 2,048 tokens (the
context length of the benchmark is 4,096). `value` is decoded tokens per second with the steps
enqueued back to back (sampled tokens fed back on the device) and timed with CUDA events; `e2e` is the
same through the Python entry point (`Engine.submit` / `Engine.step`), every step taking its inputs
from pinned host memory and handing its tokens back to the host. One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B layer sizes: the third configuration the baseline names.
QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
    tie_word_embeddings=False, max_position_embeddings=40960, hidden_act="silu", attention_bias=False, torch_dtype="bfloat16")
# The two larger shapes the baseline names (same architecture; --shape 14b / 32b): not the default run.
SHAPES = {
    "8b": QWEN3_8B,
    "14b": dict(QWEN3_8B, hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
    "32b": dict(QWEN3_8B, hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
    # the one size the reference published numbers for (on other hardware)
    "0.6b": dict(QWEN3_8B, hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
}
CONTEXT = 4096          # benchmark context length
PROMPT = 2048           # prefill length, and the context each decode request starts from
PAGE = 16           # keys per cache page of the benchmark configuration
PAGE_ENGINE = 64    # the engine's own default (one TMA box of 64 rows per page, plane and half head): measured too, as extra points
SETTLE_MS = 250     # idle time between building the requests' contexts (prefill at full power) and a decode measurement's warm-up steps:
                    # the power limiter's clock reduction after the prefill would otherwise be charged to the decode steps
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            return json.load(f), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows: list[list[str]] = []      # each with the time it arrived at
        self.proc = None
        self.begin = self.end = None         # the timed region, by time.perf_counter()

    def mark_begin(self):
        self.begin = time.perf_counter()

    def mark_end(self):
        self.end = time.perf_counter()

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")] + [time.perf_counter()])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        rows = [r for r in self.rows if len(r) >= 8]
        if self.begin is not None:   # the samples of the timed region; if it was too short to catch one, the first ones after its start
            inside = [r for r in rows if self.begin <= r[-1] <= (self.end or float("inf")) + 0.03]
            rows = inside or [r for r in rows if r[-1] >= self.begin][:3]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        num = lambda s: float(s) if s.replace(".", "", 1).isdigit() else None
        sm = [num(r[0]) for r in rows if num(r[0]) is not None]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": num(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def weight_bytes(cfg: dict, layers: int) -> int:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * H + H * q + 2 * I * H + H * I
    return 2 * (layers * per_layer + V * H)      # bfloat16; the lm_head is read once per step, the embedding rows are negligible


def kv_bytes_per_token(cfg: dict, layers: int) -> int:
    return 2 * 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * layers


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2.0 * T * layers * ((q + 2 * kv) * H + H * q + 2 * I * H + H * I)
    attention = layers * 4.0 * (T * (T + 1) / 2) * q     # QK^T and PV over the causal half
    return linear + attention + 2.0 * V * H


def _prompt(seed: int, n: int, vocab: int) -> list[int]:
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def measure_prefill(engine, steps: int, warmup: int, after: int = 0) -> float:
    """Milliseconds for one step that prefills a PROMPT-token prompt portion and returns its last logits; with
    `after`, the portion follows that many tokens of the same request already in the cache (not timed)."""
    import torch
    from inference_bench_b200.engine.step import StepEntry
    vocab = engine.decoder.plan.vocab_size
    times = []
    for i in range(warmup + steps):
        rid = ("prefill", i)
        toks = _prompt(1000 + i, PROMPT, vocab)
        engine.cache.admit(rid)
        for a in range(0, after, PROMPT):
            engine.runner.step([StepEntry(rid, _prompt(2000 + i + a, min(PROMPT, after - a), vocab), [])], check=False)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.runner.step([StepEntry(rid, toks, [PROMPT - 1])], check=False)
        e1.record()
        torch.cuda.synchronize()
        engine.cache.release(rid)
        if i >= warmup:
            times.append(e0.elapsed_time(e1))
    engine.rt.check_status()
    return statistics.median(times)


def measure_decode_device(engine, batch: int, steps: int, warmup: int, clocks=None, start: int = PROMPT) -> tuple[float, int]:
    """Milliseconds per decode step of `batch` requests whose contexts start at PROMPT tokens, steps
    enqueued back to back with tokens fed back on the device; and kernel launches per step."""
    import torch
    from inference_bench_b200.engine.executor import RUN_AHEAD_MAX
    from inference_bench_b200.engine.step import StepEntry
    from inference_bench_b200.sampling.params import GREEDY
    vocab = engine.decoder.plan.vocab_size
    ids = [("decode", batch, i) for i in range(batch)]
    last = []
    for i, rid in enumerate(ids):
        engine.cache.admit(rid)
        toks = _prompt(2000 + i, start, vocab)
        for a in range(0, start, PROMPT):   # the context, in portions of the benchmark's prefill length
            part = toks[a:a + PROMPT]
            logits = engine.runner.step([StepEntry(rid, part, [len(part) - 1] if a + PROMPT >= start else [])], check=False)
        last.append(int(engine.executor.sampler.sample(logits, [GREEDY], [0]).item()))
    generated = 1
    torch.cuda.synchronize()
    time.sleep(SETTLE_MS / 1e3)

    def run(n):
        nonlocal last, generated
        done = 0
        while done < n:
            k = min(RUN_AHEAD_MAX, n - done)
            entries = [StepEntry(rid, [tok], [0]) for rid, tok in zip(ids, last)]
            hist = engine.executor.decode_ahead(entries, [(GREEDY, generated)] * batch, k)
            last = hist[-1]
            generated += k
            done += k

    run(max(warmup, 1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.mark_begin()
    e0.record()
    run(steps)
    e1.record()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.mark_end()
    ms = e0.elapsed_time(e1) / steps
    launches = engine.executor.graph_for(batch).launches
    for rid in ids:
        engine.cache.release(rid)
    engine.rt.check_status()
    return ms, launches


LEAVE_OUT = {   # kinds of kernel by the library entry points that launch them
    "attention": ["ib_attention_decode", "ib_attention_decode_stream", "ib_attention_decode_fused", "ib_attention_prefill_ws", "ib_attention_prefill_tc"],
    "head": ["ib_embed", "ib_sample_rows"],
    "qkv": ["ib_gemm_qkv_tcgen05_2cta"],
    "norm": ["ib_add_rmsnorm"], "silu_mul": ["ib_silu_mul"], "qk": ["ib_qk_norm_rope_kv"], "sampling": ["ib_sample_rows"],
    "gemm": ["ib_gemm_tcgen05", "ib_gemm_swiglu_tcgen05", "ib_gemm_swiglu_tcgen05_2cta", "ib_gemm_tcgen05_2cta", "ib_gemm_tcgen05_2cta_add"],
    "small": ["ib_add_rmsnorm", "ib_silu_mul", "ib_qk_norm_rope_kv", "ib_rope_table", "ib_sample_rows", "ib_embed"],
}


def leave_out_costs(engine, batch: int, steps: int, warmup: int, kinds: str) -> dict:
    """Milliseconds per decode step with one kind of kernel left out of the captured step at a time (the results of such a
    step are void; only its time means something). The difference from the whole step is what that kind costs inside
    the graph, where kernels overlap their neighbours' tails: the figure a launch list cannot give."""
    from inference_bench_b200.kernels import lib as L
    real, out = L.call, {}
    try:
        for kind in kinds.split(","):
            names = set(sum((LEAVE_OUT[k] for k in kind.split("+")), []))
            L.call = lambda name, *a, _n=names: None if name in _n else real(name, *a)
            engine.executor._graphs.clear()
            out[kind] = measure_decode_device(engine, batch, steps, warmup)[0]
    finally:
        L.call = real
        engine.executor._graphs.clear()
    return out


def measure_mixed_step(engine, steps: int, cfg: dict, layers: int) -> tuple[float, int, float, float]:
    """Milliseconds for one step that holds 8 prompt portions of 512 tokens (starting 0, 512, ... 3,584 tokens into
    their prompts) beside 56 decoded tokens of requests at contexts drawn uniformly from 1,024 to 4,096: the
    mixed batch the baseline names for the 14B shape. Returns (median ms, rows in the step, the step's FLOPs, the
    bytes it has to read: every weight once and the cache of the live requests)."""
    import numpy as np
    import torch
    from inference_bench_b200.engine.step import StepEntry
    vocab = engine.decoder.plan.vocab_size
    rng = np.random.default_rng(0)
    contexts = rng.integers(1024, CONTEXT + 1, 56).tolist()

    def fill(rid, n):   # bring a request to n tokens in the cache
        engine.cache.admit(rid)
        toks = _prompt(abs(hash(rid)) % 1000, n, vocab)
        for a in range(0, n, PROMPT):
            engine.runner.step([StepEntry(rid, toks[a:a + PROMPT], [])], check=False)

    for i, c in enumerate(contexts):
        fill(("mixed-d", i), c - 1)
    for i in range(8):
        fill(("mixed-p", i), 512 * i)
    entries = [StepEntry(("mixed-d", i), [int(rng.integers(0, vocab))], [0]) for i in range(56)]
    entries += [StepEntry(("mixed-p", i), _prompt(50 + i, 512, vocab), [511]) for i in range(8)]
    times = []
    for _ in range(steps + 2):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.runner.step(entries, check=False)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
        for e in entries:   # the same work again: forget the step's tokens
            engine.cache.commit(e.request, engine.cache.length(e.request) - len(e.tokens))
    for e in entries:
        engine.cache.release(e.request)
    engine.rt.check_status()
    rows = sum(len(e.tokens) for e in entries)
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    keys_seen = sum(contexts) + sum(512 * (512 * i) + 512 * 513 // 2 for i in range(8))       # (query, key) pairs of the step
    flops = 2.0 * rows * layers * ((q + 2 * kv) * H + H * q + 3 * I * H) + layers * 4.0 * keys_seen * q + 2.0 * 64 * V * H
    cached = sum(contexts) + sum(512 * (i + 1) for i in range(8))
    return statistics.median(times[2:]), rows, flops, weight_bytes(cfg, layers) + cached * kv_bytes_per_token(cfg, layers)


def measure_decode_e2e(engine, batch: int, steps: int, warmup: int) -> tuple[float, float, float]:
    """Milliseconds per decode step through Engine.submit / Engine.step: host token ids in (pinned
    staging, copied every step) and sampled token ids back on the host every step."""
    import torch
    vocab = engine.decoder.plan.vocab_size
    for i in range(batch):
        engine.submit(_prompt(3000 + i, PROMPT, vocab), max_tokens=warmup + steps + 8)
    while engine.scheduler.waiting or any(not s.decoding for s in engine.scheduler.running):
        engine.step()
    torch.cuda.synchronize()
    time.sleep(SETTLE_MS / 1e3)
    for _ in range(max(warmup, 1)):
        engine.step()
    ex = engine.executor
    h0, d0 = ex.h2d_bytes, ex.d2h_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    emitted = 0
    for _ in range(steps):
        emitted += len(engine.step().emitted)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    assert emitted == batch * steps, f"{emitted} tokens emitted in {steps} steps of {batch} requests"
    h2d, d2h = (ex.h2d_bytes - h0) / steps, (ex.d2h_bytes - d0) / steps
    for s in list(engine.scheduler.running):
        engine.cancel(s.req.id)
    engine.rt.check_status()
    return (t1 - t0) * 1e3 / steps, h2d, d2h


def make_engine(cfg: dict, page: int, big: int, ctx: int = CONTEXT):
    from inference_bench_b200 import Engine
    return Engine(cfg, dtype="bfloat16", max_ctx=ctx, page_size=page, num_pages=big * (ctx // page) + 64, max_num_seqs=big,
                  max_batched_tokens=8192, prefill_chunk=PROMPT, random_weights_seed=0)


def run_ours(args) -> dict:
    import gc

    import torch
    pk, pk_src = peaks()
    cfg = dict(SHAPES[args.shape])
    full_layers = cfg["num_hidden_layers"]
    cfg["num_hidden_layers"] = layers = args.layers or full_layers
    big = max(args.batch, 64)
    page = args.page_size
    start = args.context_start
    after = args.prefill_after if args.only == "prefill" else 0
    if after:   # a portion deep in a long context: a cache for one such request
        engine = make_engine(cfg, page, 1, after + PROMPT)
    elif args.only == "decode" and start != PROMPT:   # another context length: a cache for just these requests
        engine = make_engine(cfg, page, max(args.batch, 8), start + CONTEXT - PROMPT)
    else:
        engine = make_engine(cfg, page, big)
    steps, warmup = args.steps, max(args.warmup, 3)
    if args.only == "prefill":   # one part alone, for profiling: a short report, not the benchmark line
        warm = 1 if after else 2
        report = {"only": "prefill", "layers": layers, "page_size": page, **({"after": after} if after else {}),
                  "ms": measure_prefill(engine, args.steps, warm, after)}
        if args.leave_out:
            from inference_bench_b200.kernels import lib as L
            real, report["without"] = L.call, {}
            try:
                for kind in args.leave_out.split(","):
                    names = set(sum((LEAVE_OUT[k] for k in kind.split("+")), []))
                    L.call = lambda name, *a, _n=names: None if name in _n else real(name, *a)
                    report["without"][kind] = measure_prefill(engine, args.steps, warm, after)
            finally:
                L.call = real
        return report
    if args.only == "mixed":
        clocks = ClockSampler()
        clocks.start()
        ms, rows, flops, step_bytes = measure_mixed_step(engine, max(args.steps, 3) if args.steps < 16 else 5, cfg, layers)
        return {"only": "mixed", "shape": args.shape, "layers": layers, "layers_full": full_layers, "page_size": page, "rows": rows, "ms": ms,
                "tok_s": rows * 1e3 / ms, "prefill": {"tokens": 8 * 512, "frac": flops / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "peak_tflops": pk["bf16_tflops"]},
                "roofline": {"bound": "hbm", "achieved": step_bytes / (ms * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                             "frac": step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}, "peaks": pk_src, "clocks": clocks.stop()}
    if args.only == "decode":
        ms, launches = measure_decode_device(engine, args.batch, steps, warmup, start=start)
        step_bytes = weight_bytes(cfg, layers) + args.batch * (start + 1 + warmup + steps / 2) * kv_bytes_per_token(cfg, layers)
        report = {"only": "decode", "shape": args.shape, "layers": layers, "batch": args.batch, "context_start": start, "page_size": page, "ms_per_step": ms,
                  "tok_s": args.batch * 1e3 / ms, "launches_per_step": launches, "hbm_frac": step_bytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
        if args.leave_out:
            report["without"] = leave_out_costs(engine, args.batch, steps, warmup, args.leave_out)
        return report

    # the headline first (device-timed, then through the entry point), then the other points
    clocks = ClockSampler()
    clocks.start()      # nvidia-smi takes a while to start reporting: it runs from here on, and the samples of the timed region are kept
    ms, launches = measure_decode_device(engine, args.batch, steps, warmup, clocks)
    clock_report = clocks.stop()
    e2e_ms, h2d, d2h = measure_decode_e2e(engine, args.batch, steps, warmup)
    b1_ms, _ = measure_decode_device(engine, 1, steps, warmup)
    b64_ms, _ = measure_decode_device(engine, 64, min(steps, 64), warmup)
    prefill_ms = measure_prefill(engine, 5, 3)
    extra = {}
    if page != PAGE_ENGINE:   # the same measurements at the engine's default page size
        del engine
        gc.collect()   # the engine's parts refer to one another: without this its weights outlive the name
        torch.cuda.empty_cache()
        engine = make_engine(cfg, PAGE_ENGINE, big)
        tag = f"_page{PAGE_ENGINE}"
        extra["prefill" + tag] = PROMPT * 1e3 / measure_prefill(engine, 5, 3)
        extra["decode_b1" + tag] = 1e3 / measure_decode_device(engine, 1, steps, warmup)[0]
        extra["decode_b64" + tag] = 64e3 / measure_decode_device(engine, 64, min(steps, 64), warmup)[0]
        extra[f"decode_b{args.batch}" + tag] = args.batch * 1e3 / measure_decode_device(engine, args.batch, steps, warmup)[0]

    B = args.batch
    avg_ctx = PROMPT + 1 + warmup + steps / 2
    step_bytes = weight_bytes(cfg, layers) + B * avg_ctx * kv_bytes_per_token(cfg, layers)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    flops = prefill_flops(cfg, layers, PROMPT)
    return {
        "metric": f"decode tok/s at batch {B} (Qwen3-{args.shape.upper()} shape, random bf16 weights, context 2048 growing toward 4096)",
        "value": B * 1e3 / ms, "unit": "tok/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": B, "seq_len": CONTEXT, "decode_context_start": PROMPT, "prefill_tokens": PROMPT,
                   "page_size": page, "weights": "random N(0,0.02) bf16 seed 0", "parallelism": "single_gpu",
                   "l2": "inputs larger than L2 (weights read every step)", "peaks": pk_src, "settle_ms": SETTLE_MS},
        "e2e": {"value": B * 1e3 / e2e_ms, "unit": "tok/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches * steps,
        "prefill": {"value": PROMPT * 1e3 / prefill_ms, "tokens": PROMPT, "ms": prefill_ms, "frac": flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"]},
        "points": {"decode_b1": 1e3 / b1_ms, "decode_b64": 64e3 / b64_ms, **extra},
        "clocks": clock_report,
    }


# ---------------------------------------------------------------------------------------------- another design beside the closest Qwen3
# Layer sizes that resemble published latent-attention models with routed experts (a 16-head one with 64 experts, and a small one),
# and the Qwen3 shape of equal width, heads and active feed-forward size. Layers alternate: one that keeps its own latent, one that
# reads the layer before's; the first feed-forward is dense, the rest are routed.
DESIGN_SIZES = {
    "small": dict(width=1024, heads=8, dim=64, rot=32, vdim=64, rank=256, dense_ff=4096, experts=16, top=2, expert_ff=1024, shared_ff=1024, groups=(4, 2), vocab=32768),
    "lite": dict(width=2048, heads=16, dim=128, rot=64, vdim=128, rank=512, dense_ff=10944, experts=64, top=6, expert_ff=1408, shared_ff=2816, groups=(8, 4), vocab=32768),
}
DESIGN_KINDS = {   # kinds of kernel by the library entry points that launch them
    "zabonex": {"attention": ["ib_latent_attention", "ib_latent_attention_mma"], "experts": ["ib_gemm_grouped", "ib_gemm_grouped_mma", "ib_gemm_grouped_tcgen05", "ib_gemm_grouped_swiglu_tcgen05", "ib_gather_rows"],
                "heads": ["ib_gemm_heads", "ib_gemm_heads_mma"], "route": ["ib_moe_route", "ib_moe_sort", "ib_moe_combine"],
                "norm": ["ib_norm_residual", "ib_latent_prepare", "ib_cast_rows"], "gemm": LEAVE_OUT["gemm"]},
    "qwen3": {"attention": LEAVE_OUT["attention"], "norm": LEAVE_OUT["norm"] + LEAVE_OUT["qk"], "gemm": LEAVE_OUT["gemm"] + LEAVE_OUT["qkv"]},
    "busadra": {"attention": ["ib_attention_generic", "ib_attention_decode_capped", "ib_attention_decode_stream_capped", "ib_attention_prefill_ws_capped"],
                "recurrence": ["ib_gated_recurrence", "ib_recurrence_chunks_finish", "ib_head_rmsnorm"],
                "experts": ["ib_gemm_grouped", "ib_gemm_grouped_mma", "ib_gemm_grouped_tcgen05", "ib_gemm_grouped_swiglu_tcgen05", "ib_scatter_scaled_rows"],
                "route": ["ib_moe_route", "ib_moe_sort", "ib_moe_combine"],
                "norm": ["ib_add_layernorm", "ib_causal_conv_rows", "ib_add_layernorm_conv_single", "ib_depth_average", "ib_qk_norm_rope_kv"], "gemm": LEAVE_OUT["gemm"]},
    "lulenex": {"attention": ["ib_attention_generic", "ib_attention_decode_capped", "ib_attention_decode_stream_capped", "ib_attention_prefill_ws_capped"],
                "recurrence": ["ib_gated_recurrence", "ib_recurrence_chunks_finish", "ib_gated_rmsnorm"],
                "scan": ["ib_conv_silu", "ib_selective_scan"],
                "norm": ["ib_add_rmsnorm", "ib_add_rmsnorm_ext", "ib_token_shift_rows", "ib_qk_norm_rope_kv", "ib_loop_pack", "ib_xielu_rows", "ib_add_bias_rows"],
                "gemm": LEAVE_OUT["gemm"] + ["ib_gemm_xielu_tcgen05"]},
}
# Ditalorn at the sizes above (the same width, heads, latent and experts as the Zabonex shape it stands beside): layers alternate between windowed
# latent attention with a query latent and grouped attention with sigmoid weights behind a convolution of four taps; every feed-forward is routed.
DITALORN_SIZES = {
    "small": dict(DESIGN_SIZES["small"], q_rank=384, window=1024, att_heads=8, att_kv_heads=2, att_dim=128, att_vdim=128, conv=4),
    "lite": dict(DESIGN_SIZES["lite"], q_rank=768, window=1024, att_heads=16, att_kv_heads=4, att_dim=128, att_vdim=128, conv=4),
}
DESIGN_KINDS["ditalorn"] = {
    "attention": ["ib_latent_attention", "ib_latent_attention_mma"], "sigmoid": ["ib_sigmoid_attention", "ib_sigmoid_attention_mma"],
    "experts": ["ib_gemm_grouped", "ib_gemm_grouped_mma", "ib_gemm_grouped_tcgen05", "ib_gemm_grouped_swiglu_tcgen05", "ib_gather_rows"],
    "heads": ["ib_gemm_heads", "ib_gemm_heads_mma"], "route": ["ib_moe_route", "ib_moe_sort", "ib_moe_combine"],
    "norm": ["ib_add_rmsnorm", "ib_post_norm", "ib_latent_down", "ib_latent_prepare", "ib_qkv_conv", "ib_embed_pos"], "gemm": LEAVE_OUT["gemm"]}


def ditalorn_config(z: dict, layers: int) -> dict:
    lat = {"heads": z["heads"], "dim": z["dim"], "vdim": z["vdim"], "kv_rank": z["rank"], "q_rank": z["q_rank"], "scale": z["dim"] ** -0.5, "mask": {"size": z["window"]}}
    att = {"heads": z["att_heads"], "kv_heads": z["att_kv_heads"], "dim": z["att_dim"], "vdim": z["att_vdim"], "scale": z["att_dim"] ** -0.5, "conv": z["conv"],
           "q_temp": {"coef": 0.5, "every": 128}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"], "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    ls = [{"type": "attention" if i % 2 else "latent_attention", "mixer": att if i % 2 else lat, "mlp": moe} for i in range(layers)]
    return {"architecture": "Ditalorn", "vocab": z["vocab"], "width": z["width"], "max_positions": CONTEXT, "embedding": {"scale": z["width"] ** 0.5}, "norm": {"eps": 1e-6},
            "layers": ls}


def ditalorn_work(z: dict, layers: int, T: int, ctx: int, batch: int) -> tuple:
    """Algorithmic FLOPs and bytes of the design's kinds of kernel for a prefill of T tokens and for a decode step of `batch` requests at `ctx`
    tokens of context (per step, all layers), and the single-matrix products' weights (elements)."""
    n_att = layers // 2
    n_lat = layers - n_att
    W, H, r, win = z["width"], z["heads"], z["rank"], z["window"]
    AH, AG, AD, AV = z["att_heads"], z["att_kv_heads"], z["att_dim"], z["att_vdim"]
    pairs_w = sum(min(t + 1, win) for t in range(T))
    pairs = T * (T + 1) / 2
    seen = min(ctx, win)
    R = (AH + AG) * AD + AG * AV
    norm_row = layers * W * (4.0 * 4 + 2 + 4 + 4 + 2) + n_lat * (4.0 * (z["q_rank"] + r) + 2 * (z["q_rank"] + r) + 6.0 * H * z["dim"]) + n_att * R * (4.0 * z["conv"] + 2)
    lin = n_lat * ((z["q_rank"] + r + H) * W + H * z["dim"] * z["q_rank"] + H * z["vdim"] * W) + n_att * (R * W + AH * AV * W) + layers * z["experts"] * W + z["vocab"] * W
    work = {
        "prefill": {"attention": {"flops": n_lat * 4.0 * H * pairs_w * r}, "sigmoid": {"flops": n_att * 2.0 * AH * pairs * (AD + AV)},
                    "experts": {"flops": layers * 2.0 * T * z["top"] * 3 * z["expert_ff"] * W},
                    "heads": {"flops": n_lat * 2.0 * T * H * r * (z["dim"] + z["vdim"])}, "norm": {"flops": 0.0, "bytes": T * norm_row}},
        "decode": {"attention": {"flops": n_lat * 4.0 * H * batch * seen * r, "bytes": n_lat * 2.0 * batch * seen * r},
                   "sigmoid": {"flops": n_att * 2.0 * AH * batch * ctx * (AD + AV), "bytes": n_att * 2.0 * batch * ctx * AG * (AD + AV)},
                   "experts": {"flops": layers * 2.0 * batch * z["top"] * 3 * z["expert_ff"] * W, "bytes": layers * 2.0 * min(batch * z["top"], z["experts"]) * 3 * z["expert_ff"] * W},
                   "heads": {"flops": n_lat * 2.0 * batch * H * r * (z["dim"] + z["vdim"]), "bytes": n_lat * 2.0 * H * r * (z["dim"] + z["vdim"])},
                   "norm": {"flops": 0.0, "bytes": batch * norm_row}},
    }
    return work, lin


# Busadra at layer sizes that resemble small hybrid models: windowed grouped-query attention with heads of 128, a gated linear recurrence
# whose heads hold a 128 x 128 state, and routed experts; layers in the order attention, recurrence, recurrence, attention (repeated).
BUSADRA_SIZES = {
    "small": dict(width=1024, heads=8, kv_heads=2, dim=128, window=1024, rec_heads=8, rec_dim=128, rec_vdim=128, experts=16, top=2, expert_ff=1024, vocab=32768),
    "mid": dict(width=2048, heads=16, kv_heads=4, dim=128, window=2048, rec_heads=16, rec_dim=128, rec_vdim=128, experts=64, top=6, expert_ff=1408, vocab=32768),
}


def busadra_config(z: dict, layers: int) -> dict:
    att = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "mask": {"size": z["window"]}, "scale": z["dim"] ** -0.5, "softcap": 30.0,
           "rot": {"base": 500000.0, "dims": z["dim"], "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    rec = {"heads": z["rec_heads"], "dim": z["rec_dim"], "vdim": z["rec_vdim"]}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "router": {"experts": z["experts"], "top": z["top"]}}
    ls = [{"type": "attention", "mixer": att, "mlp": moe} if i % 4 in (0, 3) else {"type": "hgrn2", "mixer": rec, "mlp": moe} for i in range(layers)]
    return {"architecture": "Busadra", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "canon": {"taps": 4}, "logit_scale": 1.0, "layers": ls}


def qwen3_like_busadra(z: dict, layers: int) -> dict:
    """The Qwen3 shape of equal width, heads, kv heads, head size and active feed-forward size, every layer windowed like the design's attention."""
    return dict(QWEN3_8B, vocab_size=z["vocab"], hidden_size=z["width"], num_hidden_layers=layers, num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
                head_dim=z["dim"], intermediate_size=z["top"] * z["expert_ff"], use_sliding_window=True, sliding_window=z["window"], max_window_layers=0,
                layer_types=["sliding_attention"] * layers)


def busadra_work(z: dict, layers: int, T: int, ctx: int, batch: int) -> dict:
    """Algorithmic FLOPs and bytes of the design's own kinds of kernel, for a prefill of T tokens and for a decode step of `batch` requests
    at `ctx` tokens of context (per step, all layers). The recurrence's products are float32 FMAs, not tensor-core work: its floor is
    given in bytes only (the projections it reads and, per decoded token, the state's trip from memory and back)."""
    n_att = sum(1 for i in range(layers) if i % 4 in (0, 3))
    n_rec = layers - n_att
    H, G, D, W = z["heads"], z["kv_heads"], z["dim"], z["window"]
    pairs = sum(min(t + 1, W) for t in range(T))
    seen = min(ctx, W)
    rh, rd, rv = z["rec_heads"], z["rec_dim"], z["rec_vdim"]
    width = z["width"]
    norm_bytes = lambda rows: layers * rows * width * (2 * (4 + 4 + 4 + 4 + 4 + 2) + (4 + 4 + 4 + 4 * (layers / 2 + 1)))   # two norms and convolutions, the depth average
    return {
        "prefill": {"attention": {"flops": n_att * 4.0 * H * D * pairs},
                    "recurrence": {"flops": 0.0, "bytes": n_rec * T * rh * (4.0 * (2 * rd + rv) + 4.0 * rv + 6.0 * rv)},
                    "experts": {"flops": layers * 2.0 * T * z["top"] * 3 * z["expert_ff"] * width},
                    "norm": {"flops": 0.0, "bytes": norm_bytes(T)}},
        "decode": {"attention": {"flops": n_att * 4.0 * H * D * batch * seen, "bytes": n_att * 2.0 * batch * seen * G * 2 * D},
                   "recurrence": {"flops": 0.0, "bytes": n_rec * batch * rh * (8.0 * rd * rv + 4.0 * (2 * rd + rv) + 10.0 * rv)},
                   "experts": {"flops": layers * 2.0 * batch * z["top"] * 3 * z["expert_ff"] * width,
                               "bytes": layers * 2.0 * min(batch * z["top"], z["experts"]) * 3 * z["expert_ff"] * width},
                   "norm": {"flops": 0.0, "bytes": norm_bytes(batch)}},
    }


# Lulenex at layer sizes that resemble small hybrid models: chunked grouped-query attention with heads of 128 (blocks of 1,536 positions:
# a prompt of 2,048 crosses one edge and a decoded token at 2,048 sees the 513 keys of its block) beside a fixed-decay recurrence whose
# heads hold a 128 x 128 state, every fourth layer (from the third) a selective scan, dense xIELU feed-forwards; layers 1 and 2 run twice.
# Beside it Busadra, the closest design (windowed attention and a gated recurrence of the same head sizes, two experts a token).
LULENEX_SIZES = {
    "small": dict(width=1024, heads=8, kv_heads=2, dim=128, chunk=1536, rec_heads=8, rec_dim=128, rec_vdim=128, inner=2048, state=16, dt_rank=64, conv=4, ff=4096, vocab=32768,
                  experts=8, top=2, expert_ff=1408),
    "mid": dict(width=2048, heads=16, kv_heads=4, dim=128, chunk=1536, rec_heads=16, rec_dim=128, rec_vdim=128, inner=4096, state=16, dt_rank=128, conv=4, ff=8192, vocab=32768,
                experts=8, top=2, expert_ff=2688),
}
# A third size, run on its own (`--size large`): it is not among the default sizes.
LULENEX_EXTRA_SIZES = {
    "large": dict(width=4096, heads=32, kv_heads=8, dim=128, chunk=1536, rec_heads=32, rec_dim=128, rec_vdim=128, inner=8192, state=16, dt_rank=256, conv=4, ff=16384, vocab=32768,
                  experts=8, top=2, expert_ff=5504),
}


def lulenex_layer_types(layers: int) -> list:
    return ["mamba1" if i % 4 == 2 else "parallel" for i in range(layers)]


def lulenex_loop(layers: int):
    return {"start": 1, "stop": 3, "times": 2} if layers >= 3 else None


def lulenex_config(z: dict, layers: int) -> dict:
    par = {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["dim"], "mask": {"size": z["chunk"]}, "scale": z["dim"] ** -0.5,
                    "rot": {"base": 1000000.0, "dims": z["dim"] // 2}}, "left_scale": 0.8,
           "right": {"heads": z["rec_heads"], "dim": z["rec_dim"], "vdim": z["rec_vdim"], "decay": [1.0 - 0.5 ** (1 + 8 * h / z["rec_heads"]) for h in range(z["rec_heads"])]},
           "right_scale": 0.5}
    scan = {"inner": z["inner"], "state": z["state"], "dt_rank": z["dt_rank"], "conv": z["conv"]}
    ls = [{"type": t, "mixer": scan if t == "mamba1" else par, "mlp": {"kind": "dense", "ff": z["ff"]}} for t in lulenex_layer_types(layers)]
    return {"architecture": "Lulenex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6}, "loop": lulenex_loop(layers), "layers": ls}


def busadra_like_lulenex(z: dict, layers: int) -> dict:
    return busadra_config(dict(z, window=z["chunk"]), layers)


def lulenex_runs(layers: int) -> list:
    types, lp = lulenex_layer_types(layers), lulenex_loop(layers)
    if lp is None:
        return types
    return types[:lp["start"]] + types[lp["start"]:lp["stop"]] * lp["times"] + types[lp["stop"]:]


def lulenex_work(z: dict, layers: int, T: int, ctx: int, batch: int) -> tuple:
    """Algorithmic FLOPs and bytes of the design's kinds of kernel for a prefill of T tokens and for a decode step of `batch` requests at
    `ctx` tokens of context (per step, every run of a layer counted), and the matrix products' weights (elements, per step). The
    recurrence and the scan are float32 FMAs, not tensor-core work: their floors are the bytes they must move (float32 sums of the
    projections in, activations out and, per decoded token, the state's trip from memory and back)."""
    runs = lulenex_runs(layers)
    n_par, n_scan, n = runs.count("parallel"), runs.count("mamba1"), len(runs)
    passes = lulenex_loop(layers)["times"] if lulenex_loop(layers) else 0
    W, H, G, D, c = z["width"], z["heads"], z["kv_heads"], z["dim"], z["chunk"]
    rh, rd, rv, I, N, R, ff = z["rec_heads"], z["rec_dim"], z["rec_vdim"], z["inner"], z["state"], z["dt_rank"], z["ff"]
    pairs = sum(t % c + 1 for t in range(T))
    seen = ctx % c + 1
    rec_row = rh * (4.0 * (2 * rd + rv) + 4.0 * rv + 10.0 * rv)         # q, k, v in; o out; o and the gate in, the gated norm out
    scan_row = I * (4.0 + 4 + 2 + 4 + 4 + 2) + 4.0 * (R + 2 * N)          # u in, x out twice; x, z in, y out; the step, B and C in
    norm_row = n * (W * (16.0 + 6 + 14) + 6.0 * ff) + n_par * ((H + G) * D * 4.0 + 2.0 * H * D + 4.0 * G * D) + passes * W * 20.0
    lin = n_par * ((H + G) * D + H + 2 * rh * (rd + rv) + H * D + rh * rv) * W + n_scan * (3 * I * W + (R + 2 * N) * I) + n * 2 * ff * W + passes * 2 * W * W + z["vocab"] * W
    work = {
        "prefill": {"attention": {"flops": n_par * 4.0 * H * D * pairs}, "recurrence": {"flops": 0.0, "bytes": n_par * T * rec_row},
                    "scan": {"flops": 0.0, "bytes": n_scan * T * scan_row}, "norm": {"flops": 0.0, "bytes": T * norm_row}},
        "decode": {"attention": {"flops": n_par * 4.0 * H * D * batch * seen, "bytes": n_par * 2.0 * batch * seen * G * 2 * D},
                   "recurrence": {"flops": 0.0, "bytes": n_par * batch * (rec_row + rh * 8.0 * rd * rv)},
                   "scan": {"flops": 0.0, "bytes": n_scan * batch * (scan_row + 8.0 * I * N)}, "norm": {"flops": 0.0, "bytes": batch * norm_row}},
    }
    return work, lin


def kernel_times(engine, entries) -> dict:
    """Milliseconds per library entry point in one step run outside a graph: every call stands between two CUDA events, and a
    long idle kernel goes first so that the whole step is queued before its first kernel starts (the events then measure the
    kernels, not the host). A kernel timed this way stands alone: it overlaps nothing of its neighbours."""
    import torch
    from inference_bench_b200.kernels import lib as L
    real, log = L.call, []

    def timed(name, *a):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        real(name, *a)
        e1.record()
        log.append((name, e0, e1))

    torch.cuda.synchronize()
    torch.cuda._sleep(40_000_000)
    L.call = timed
    try:
        engine.runner.step(entries, check=False)
    finally:
        L.call = real
    torch.cuda.synchronize()
    out: dict = {}
    for name, e0, e1 in log:
        t = out.setdefault(name, [0.0, 0])
        t[0] += e0.elapsed_time(e1)
        t[1] += 1
    return out


def zabonex_config(z: dict, layers: int) -> dict:
    mixer = {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["rank"], "scale": (z["dim"] + z["rot"]) ** -0.5,
             "rot": {"base": 10000.0, "dims": z["rot"]}}
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["shared_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 1.0, "groups": {"count": z["groups"][0], "keep": z["groups"][1]}}}
    ls = []
    for i in range(layers):
        m = dict(mixer, kv_from=i - 1) if i % 2 else dict(mixer)
        ls.append({"type": "latent_attention", "mixer": m, "mlp": {"kind": "dense", "ff": z["dense_ff"]} if i == 0 else moe})
    return {"architecture": "Zabonex", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-5}, "residual_mult": 0.7, "layers": ls}


def qwen3_like(z: dict, layers: int) -> dict:
    return dict(QWEN3_8B, vocab_size=z["vocab"], hidden_size=z["width"], num_hidden_layers=layers, num_attention_heads=z["heads"],
                num_key_value_heads=max(1, z["heads"] // 4), head_dim=128 if z["dim"] + z["rot"] > 96 else 64, intermediate_size=z["top"] * z["expert_ff"] + z["shared_ff"])


def design_work(z: dict, layers: int, T: int, ctx: int, batch: int) -> dict:
    """Algorithmic FLOPs and bytes of the new design's own kinds of kernel, for a prefill of T tokens and for a decode step of `batch`
    requests at `ctx` tokens of context (per step, all layers)."""
    H, D, r = z["heads"], z["rank"] + z["rot"], z["rank"]
    moe_layers = layers - 1
    pairs = T * (T + 1) / 2
    return {
        "prefill": {"attention": {"flops": layers * 2.0 * H * pairs * (D + r)},
                    "experts": {"flops": moe_layers * 2.0 * T * z["top"] * 3 * z["expert_ff"] * z["width"]},
                    "heads": {"flops": layers * 2.0 * T * H * r * (z["dim"] + z["vdim"])}},
        "decode": {"attention": {"flops": layers * 2.0 * H * batch * ctx * (D + r), "bytes": layers * 2.0 * batch * ctx * D},
                   "experts": {"flops": moe_layers * 2.0 * batch * z["top"] * 3 * z["expert_ff"] * z["width"],
                               "bytes": moe_layers * 2.0 * min(batch * z["top"], z["experts"]) * 3 * z["expert_ff"] * z["width"]},
                   "heads": {"flops": layers * 2.0 * batch * H * r * (z["dim"] + z["vdim"]), "bytes": layers * 2.0 * H * r * (z["dim"] + z["vdim"])}},
    }


def qwen3_work(cfg: dict, layers: int, T: int, ctx: int, batch: int) -> dict:
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    W = cfg.get("sliding_window") if cfg.get("use_sliding_window") else None
    pairs = T * (T + 1) / 2 if not W else sum(min(t + 1, W) for t in range(T))
    seen = ctx if not W else min(ctx, W)
    width = cfg["hidden_size"]
    norm_bytes = lambda rows: layers * rows * (2 * width * (4 + 4 + 4 + 2) + (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * cfg["head_dim"] * (4 + 2))
    return {"prefill": {"attention": {"flops": layers * 4.0 * pairs * q}, "norm": {"flops": 0.0, "bytes": norm_bytes(T)}},
            "decode": {"attention": {"flops": layers * 4.0 * batch * seen * q, "bytes": batch * seen * kv_bytes_per_token(cfg, layers)},
                       "norm": {"flops": 0.0, "bytes": norm_bytes(batch)}}}


def run_design(args) -> dict:
    """Prefill (one portion of 2,048 tokens) and decode (batch 1, 8, 64 at 2,048 tokens of context) of Zabonex at sizes that resemble
    real models, beside the Qwen3 shape of equal width, heads and active feed-forward; and every kind of kernel of one prefill step
    and one decode step of 8 requests timed alone with CUDA events, with how far that is from the kind's roofline (the slower of
    its FLOPs at the measured matrix-product peak and its bytes at the measured copy bandwidth)."""
    import gc

    import torch
    from inference_bench_b200 import Engine
    from inference_bench_b200.engine.step import StepEntry
    pk, pk_src = peaks()
    layers = args.layers or 4
    steps, warmup = min(args.steps, 32), max(args.warmup, 3)
    out = {"design": args.design, "layers": layers, "peaks": pk_src, "sizes": {}}
    sizes = {"busadra": BUSADRA_SIZES, "lulenex": LULENEX_SIZES, "ditalorn": DITALORN_SIZES}.get(args.design, DESIGN_SIZES)
    for name in (args.size.split(",") if args.size else list(sizes)):
        z = sizes[name] if name in sizes or args.design != "lulenex" else LULENEX_EXTRA_SIZES[name]
        report = {}
        if args.design == "lulenex":
            zb = dict(z, window=z["chunk"])
            pair = (("lulenex", lulenex_config(z, layers)), ("busadra", busadra_like_lulenex(z, layers)))
        elif args.design == "busadra":
            zb = z
            pair = (("busadra", busadra_config(z, layers)), ("qwen3", qwen3_like_busadra(z, layers)))
        elif args.design == "ditalorn":
            pair = (("ditalorn", ditalorn_config(z, layers)), ("zabonex", zabonex_config(z, layers)))
        else:
            pair = (("zabonex", zabonex_config(z, layers)), ("qwen3", qwen3_like(z, layers)))
        for arch, cfg in pair:
            engine = Engine(cfg, dtype="bfloat16", max_ctx=CONTEXT, page_size=PAGE_ENGINE, num_pages=64 * (CONTEXT // PAGE_ENGINE) + 64, max_num_seqs=64,
                            max_batched_tokens=8192, prefill_chunk=PROMPT, random_weights_seed=0)
            vocab = engine.decoder.plan.vocab_size
            if arch == "zabonex":
                work = design_work(z, layers, PROMPT, PROMPT, 8)
                lin = layers * (z["heads"] * (z["dim"] + z["rot"]) + z["heads"] * z["vdim"]) * z["width"] + (layers + 1) // 2 * (z["rank"] + z["rot"]) * z["width"] + \
                    3 * z["dense_ff"] * z["width"] + (layers - 1) * (3 * z["shared_ff"] + z["experts"]) * z["width"] + vocab * z["width"]
            elif arch == "lulenex":
                work, lin = lulenex_work(z, layers, PROMPT, PROMPT, 8)
            elif arch == "ditalorn":
                work, lin = ditalorn_work(z, layers, PROMPT, PROMPT, 8)
            elif arch == "busadra":
                work = busadra_work(zb, layers, PROMPT, PROMPT, 8)
                n_att = sum(1 for i in range(layers) if i % 4 in (0, 3))
                lin = n_att * (2 * z["heads"] + 2 * z["kv_heads"]) * z["dim"] * z["width"] + \
                    (layers - n_att) * z["rec_heads"] * (2 * z["rec_dim"] + 2 * z["rec_vdim"]) * z["width"] + layers * z["experts"] * z["width"] + vocab * z["width"]
            else:
                work = qwen3_work(cfg, layers, PROMPT, PROMPT, 8)
                lin = weight_bytes(cfg, layers) // 2
            work["prefill"]["gemm"] = {"flops": 2.0 * PROMPT * (lin - vocab * z["width"]) + 2.0 * vocab * z["width"]}
            work["decode"]["gemm"] = {"flops": 2.0 * 8 * lin, "bytes": 2.0 * lin}
            r = {"prefill_ms": measure_prefill(engine, 3, 2)}
            r["prefill_tok_s"] = PROMPT * 1e3 / r["prefill_ms"]
            for b in (1, 8, 64):
                ms, launches = measure_decode_device(engine, b, steps, warmup)
                r[f"decode_b{b}_ms"], r[f"decode_b{b}_tok_s"] = ms, b * 1e3 / ms
                if b == 8:
                    r["launches_per_decode_step"] = launches
            # kernels alone: the prefill of one request, then one step of 8 decoded tokens at 2,048 tokens of context
            ids = [("k", i) for i in range(8)]
            for i, rid in enumerate(ids):
                engine.cache.admit(rid)
                e = [StepEntry(rid, _prompt(4000 + i, PROMPT, vocab), [PROMPT - 1])]
                if i < 7:
                    engine.runner.step(e, check=False)
                else:
                    times_p = kernel_times(engine, e)
            kernel_times(engine, [StepEntry(rid, [1 + i], [0]) for i, rid in enumerate(ids)])   # once for lazy set-up
            times_d = kernel_times(engine, [StepEntry(rid, [9 + i], [0]) for i, rid in enumerate(ids)])
            for rid in ids:
                engine.cache.release(rid)
            engine.rt.check_status()
            kinds = {}
            for kind, names in DESIGN_KINDS[arch].items():
                k = {}
                for phase, times in (("prefill", times_p), ("decode", times_d)):
                    ms, n = sum(times[x][0] for x in names if x in times), sum(times[x][1] for x in names if x in times)
                    if not n:
                        continue
                    k[f"{phase}_ms"], k[f"{phase}_calls"] = ms, n
                    w = work[phase].get(kind)
                    if w:
                        floor = max(w["flops"] / (pk["bf16_tflops"] * 1e12), w.get("bytes", 0.0) / (pk["hbm_gbs"] * 1e9)) * 1e3
                        k[f"{phase}_roofline_frac"] = floor / ms
                if k:
                    kinds[kind] = k
            r["kinds"] = kinds
            r["kernels_alone_ms"] = {"prefill": sum(t[0] for t in times_p.values()), "decode_b8": sum(t[0] for t in times_d.values())}
            report[arch] = r
            del engine
            gc.collect()
            torch.cuda.empty_cache()
        out["sizes"][name] = report
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes: the benchmark's Qwen3-8B, or the larger shapes the baseline names")
    ap.add_argument("--page-size", type=int, default=PAGE, help="keys per cache page (the benchmark configuration names 16)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prefill-after", type=int, default=0, help="with --only prefill: the 2,048-token portion follows this many cached tokens of the same request")
    ap.add_argument("--context-start", type=int, default=PROMPT, help="with --only decode: the context each request starts from (default: the benchmark's 2,048)")
    ap.add_argument("--leave-out", default="", help="with --only decode or prefill: also time the step without each of these kinds of kernel (comma separated; "
                    "a+b leaves both out): " + ", ".join(sorted(LEAVE_OUT)))
    ap.add_argument("--only", default="", choices=["", "prefill", "decode", "mixed"], help="run one part alone (for profiling); prints a short report")
    ap.add_argument("--design", default="", choices=["", "zabonex", "busadra", "lulenex", "ditalorn"],
                    help="measure another design beside the closest existing one at equal size (Qwen3; for lulenex, Busadra; for ditalorn, Zabonex) instead of the benchmark (prints its own report)")
    ap.add_argument("--size", default="", help="with --design: which of its sizes (comma separated; default all): " + ", ".join(DESIGN_SIZES) + " (zabonex); " + ", ".join(BUSADRA_SIZES) + " (busadra); " + ", ".join(LULENEX_SIZES) + " (lulenex); " + ", ".join(DITALORN_SIZES) + " (ditalorn)")
    args = ap.parse_args()
    if args.design:
        print(json.dumps(run_design(args)))
        return 0
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "the reference is a Rust workspace (no setup.py/pyproject.toml): pip cannot install it and no Rust toolchain is present"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine: --gpus {args.gpus} is not supported, run with --gpus 1")
        return 2
    if args.steps + max(args.warmup, 3) + 8 > CONTEXT - PROMPT:
        print(f"--steps + --warmup must stay below {CONTEXT - PROMPT - 8}: contexts start at {PROMPT} and end at {CONTEXT}")
        return 2
    print(json.dumps(run_ours(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
