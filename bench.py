#!/usr/bin/env python3
"""Benchmark of velox_b200: decode tokens per second of a Qwen3-8B-shaped model
with random weights on one B200, plus prefill, batch-1 and batch-64 points and
roofline fractions.  Prints ONE JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]

A "step" is one decode step of the whole batch.  The timed decode steps are the
last K before the requests reach the context length, so the cache they read is
as long as it gets.  Weights (15 GB) and cache are far larger than L2, so every
step reads them from memory; nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B shape: the benchmark configuration (36 layers, hidden 4096, 32 query
# heads, 8 kv heads of 128, intermediate 12288, vocabulary 151936, untied head).
MODEL = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
             num_attention_heads=32, head_dim=128, attention_bias=False, num_key_value_heads=8,
             max_position_embeddings=40960, tie_word_embeddings=False, rope_theta=1000000.0,
             rms_norm_eps=1e-6, hidden_act="silu")
# Other shapes of the same architecture, for measurements beside the benchmark's (`--shape`).
SHAPES = {
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
    "1.7b": dict(hidden_size=2048, intermediate_size=6144, num_hidden_layers=28, num_attention_heads=16, tie_word_embeddings=True),
    "4b": dict(hidden_size=2560, intermediate_size=9728, num_hidden_layers=36, num_attention_heads=32, tie_word_embeddings=True),
    "8b": {},
    "14b": dict(hidden_size=5120, intermediate_size=17408, num_hidden_layers=40, num_attention_heads=40),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64),
}
CONTEXT, PROMPT, PAGE, BATCH, SEED = 4096, 2048, 16, 8, 2
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                raw = json.load(f)
            out = dict(FALLBACK_PEAKS)
            for k in out:
                if isinstance(raw.get(k), (int, float)):
                    out[k] = float(raw[k])
            out["source"] = "measured"
            return out
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz)}


def weight_bytes(cfg, layers, elt=2):
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hk, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    return (layers * ((H + 2 * Hk) * D * E + E * H * D + 3 * I * E) + 2 * V * E) * elt


def decode_bytes(cfg, layers, batch, kv_len, elt=2):
    """Bytes a decode step has to read: every weight once, and the live requests' cache."""
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hk, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = ((H + 2 * Hk) * D * E + E * H * D + 3 * I * E) * elt
    weights = layers * per_layer + V * E * elt  # head; the embedding rows read are negligible
    kv = layers * 2 * Hk * D * elt * batch * kv_len
    return weights + kv


def prefill_flops(cfg, layers, tokens):
    E, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, Hk, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = 2 * tokens * layers * ((H + 2 * Hk) * D * E + E * H * D + 3 * I * E)
    attn = layers * H * 2 * D * tokens * tokens  # causal: half of 4 D T^2
    return linear + attn + 2 * V * E


def stream_workload(args, cfg, layers):
    """Continuous batching under arrivals: 64 requests with prompts of 128 to 4,096
    random tokens and 256 new tokens each arrive as a Poisson stream; every step goes
    through `Engine.step`.  Reports generated tokens a second over the whole run,
    time to the first token and time between tokens (host clock around the steps,
    which end with the read of the sampled ids), and the scheduler's counters."""
    import random

    import torch
    from velox_b200 import Engine, EngineConfig, SamplingParams

    n_req, new_tokens, longest = 64, 256, 4096
    rng = random.Random(SEED + 1)
    lens = [rng.randint(128, longest) for _ in range(n_req)]
    arrivals, t = [], 0.0
    for _ in range(n_req):
        t += rng.expovariate(args.arrival_rate)
        arrivals.append(t)
    pool = args.pool_tokens or n_req * (longest + new_tokens + PAGE)
    engine = Engine(model_config=cfg, random_seed=SEED, config=EngineConfig(
        dtype="bfloat16", page_size=PAGE, num_pages=-(-pool // PAGE), max_running_requests=n_req,
        max_batch_tokens=args.max_batch_tokens, max_model_len=longest + new_tokens + PAGE))
    gen = torch.Generator().manual_seed(SEED + 2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist() for n in lens]
    # warm-up: kernels, graphs of a few batch sizes, the library's handles
    engine.generate([prompts[0][:300], prompts[1][:40]], SamplingParams(max_tokens=4, ignore_eos=True))
    # as a server does before it listens: the decode steps' graphs are captured now, not under load
    t_cap = time.perf_counter()
    captured = 0 if args.lazy_graphs else engine.capture_decode_graphs()
    torch.cuda.synchronize()
    t_cap = time.perf_counter() - t_cap
    first, last, gaps, submitted_at = {}, {}, [], {}
    nxt, done = 0, 0
    t0 = time.perf_counter()
    while done < n_req:
        now = time.perf_counter() - t0
        while nxt < n_req and arrivals[nxt] <= now:
            rid = engine.add_request(prompts[nxt], SamplingParams(max_tokens=new_tokens, ignore_eos=True))
            submitted_at[rid] = arrivals[nxt]
            nxt += 1
        if not engine.scheduler.has_work():
            time.sleep(max(0.0, arrivals[nxt] - (time.perf_counter() - t0)))
            continue
        out = engine.step()
        now = time.perf_counter() - t0
        for rid, _tok, finished in out:
            if rid in last:
                gaps.append(now - last[rid])
            else:
                first[rid] = now - submitted_at[rid]
            last[rid] = now
            done += bool(finished)
    wall = time.perf_counter() - t0
    st = engine.stats()

    def pct(v, q):
        v = sorted(v)
        return round(1000.0 * v[min(len(v) - 1, int(q * len(v)))], 2)
    return {"metric": "generated tok/s, continuous batching, Qwen3-%s bf16" % args.shape.upper(), "unit": "tokens/s",
            "value": round(n_req * new_tokens / wall, 1), "wall_s": round(wall, 3), "n_gpus": 1,
            "requests": n_req, "prompt_tokens": sum(lens), "new_tokens": n_req * new_tokens,
            "arrival_rate": args.arrival_rate, "pool_tokens": pool, "max_batch_tokens": args.max_batch_tokens,
            "ttft_ms": {"p50": pct(first.values(), 0.5), "p90": pct(first.values(), 0.9), "p99": pct(first.values(), 0.99)},
            "itl_ms": {"p50": pct(gaps, 0.5), "p90": pct(gaps, 0.9), "p99": pct(gaps, 0.99)},
            "steps": st["steps"], "preemptions": st["preemptions"], "layers": layers,
            "mean_step_ms": round(st["total_step_us"] / max(st["steps"], 1) / 1000.0, 3),   # (the scheduler's own clock)
            "graphs_captured_before": captured, "capture_s": round(t_cap, 2),
            "data": "synthetic: random weights, uniform random token ids, seeded arrivals"}


# ---- Dobepel beside Qwen3 at equal size (`--workload dobepel`) ---------------------------------------
# Layer sizes that resemble a real model's (random weights): width, layers, query / kv heads of the softmax
# attention (heads of 128, values of 128, window 1,024, 4 first tokens kept), heads of the linear attention
# (128 x 128 state a head), 8 experts of which 2 run plus a shared expert.  The Qwen3 model beside each has the
# same width, layers and heads and an intermediate size of what a Dobepel token runs through (2 experts + shared).
DOBEPEL_SIZES = {
    "1k": dict(width=1024, layers=4, heads=8, kv_heads=2, lin_heads=8, expert_ff=512, shared_ff=512),
    "2k": dict(width=2048, layers=4, heads=16, kv_heads=4, lin_heads=16, expert_ff=1024, shared_ff=1024),
    "4k": dict(width=4096, layers=2, heads=32, kv_heads=8, lin_heads=32, expert_ff=2048, shared_ff=2048),
}
DOBEPEL_VOCAB, DOBEPEL_WINDOW, DOBEPEL_KEEP, DOBEPEL_EXPERTS, DOBEPEL_TOP = 32000, 1024, 4, 8, 2


def dobepel_raw(sz):
    left = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
            "mask": {"size": DOBEPEL_WINDOW, "keep_first": DOBEPEL_KEEP}}
    right = {"heads": sz["lin_heads"], "dim": 128, "vdim": 128,
             "decay": [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(1, sz["lin_heads"] - 1)) for h in range(sz["lin_heads"])]}
    mlp = {"kind": "moe", "expert": {"ff": sz["expert_ff"]}, "router": {"experts": DOBEPEL_EXPERTS, "top": DOBEPEL_TOP},
           "shared": {"ff": sz["shared_ff"]}}
    layer = {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}
    return {"architecture": "Dobepel", "vocab": DOBEPEL_VOCAB, "width": sz["width"], "residual_mult": 0.5, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 8191}},
            "layers": [json.loads(json.dumps(layer)) for _ in range(sz["layers"])]}


def qwen_raw_like(sz):
    return dict(MODEL, vocab_size=DOBEPEL_VOCAB, hidden_size=sz["width"], num_hidden_layers=sz["layers"],
                num_attention_heads=sz["heads"], num_key_value_heads=sz["kv_heads"], head_dim=128,
                intermediate_size=DOBEPEL_TOP * sz["expert_ff"] + sz["shared_ff"], tie_word_embeddings=False)


def timed(fn, steps):
    """Milliseconds a call of `fn`, by CUDA events around `steps` calls."""
    import torch
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def model_points(cfg, vocab, T, B, CTX, K, W, gen):
    """Prefill (one prompt of T tokens in one step) and decode (batch B at CTX cached tokens) of a model with
    random weights through the step function."""
    import torch
    from velox_b200 import Engine, EngineConfig
    from velox_b200.csrc import ops
    from velox_b200.engine import StepEntry
    eng = Engine(model_config=cfg, random_seed=SEED, config=EngineConfig(
        dtype="bfloat16", page_size=PAGE, num_pages=(B + 1) * ((CTX + 64) // PAGE + 1), max_running_requests=B + 1,
        max_batch_tokens=T, max_model_len=CTX + 64))
    toks = torch.randint(0, vocab, (B + 1, CTX), generator=gen).tolist()

    def prefill():
        eng.cache.add_request("p")
        eng.run_step([StepEntry("p", toks[B][:T], [T - 1])])
        eng.cache.release("p")
    for _ in range(3):
        prefill()
    pms = timed(prefill, 5)
    for i in range(B):
        eng.cache.add_request(i)
        eng.run_step([StepEntry(i, toks[i][:CTX - K - W - 2], [])])
    entries = [StepEntry(i, [toks[i][-1]], [0]) for i in range(B)]
    zeros, ones = [0.0] * B, [1.0] * B

    def step():
        eng.runner.step_and_sample(entries, zeros, ones, zeros)
    for _ in range(W):
        step()
    n0 = ops.launch_count()
    dms = timed(step, K)
    launches = (ops.launch_count() - n0) // K
    ops.check_device_errors()
    del eng
    torch.cuda.empty_cache()
    return {"prefill_ms": round(pms, 3), "prefill_tok_s": round(T * 1000.0 / pms, 1), "decode_ms_per_step": round(dms, 4),
            "decode_tok_s": round(B * 1000.0 / dms, 1), "launches_per_decode_step": int(launches)}


def kernel_rows(pk):
    """(rows, row, us): a table of kernel timings; `row(name, microseconds, flops, bytes)` adds a line with its fraction
    of the roofline; `us(fn, n)` measures a call."""
    import torch
    hbm, tf = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = {}

    def row(name, us_, flops=0.0, nbytes=0.0):
        t = us_ * 1e-6
        frac_c, frac_m = flops / t / tf, nbytes / t / hbm
        rows[name] = {"us": round(us_, 2), "bound": "tensor" if frac_c >= frac_m else "hbm",
                      "frac": round(max(frac_c, frac_m), 4)}

    def us(fn, n=20):
        """Microseconds a call of `fn`: n calls recorded in one CUDA graph (so that the host's share of a launch
        does not count), replayed three times for warm-up and five times under CUDA events."""
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(n):
                fn()
        for _ in range(3):
            g.replay()
        return timed(g.replay, 5) * 1000.0 / n
    return rows, row, us


def dobepel_workload(args, pk):
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 at 2,048 cached tokens) of Dobepel
    and of Qwen3 at equal size, through the step function, timed with CUDA events; then the design's own kernels
    beside the like kernels of Qwen3 at the 2k size, each as a fraction of its roofline."""
    import torch
    from velox_b200.config import DobepelConfig, Qwen3Config

    T, B, CTX = 2048, 8, 2048
    K, W = max(1, min(args.steps, 32)), max(3, args.warmup)
    gen = torch.Generator().manual_seed(SEED)

    sizes = {}
    for name, sz in DOBEPEL_SIZES.items():
        sizes[name] = {"dobepel": model_points(DobepelConfig.from_dict(dobepel_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "qwen3": model_points(Qwen3Config.from_dict(qwen_raw_like(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "shape": sz}
    out = {"metric": "Dobepel beside Qwen3 at equal size: prefill of %d tokens, decode at batch %d with %d cached tokens, bf16"
                     % (T, B, CTX), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "sizes": sizes,
           "value": sizes["2k"]["dobepel"]["decode_tok_s"], "higher_is_better": True,
           "kernels": dobepel_kernels(pk, DOBEPEL_SIZES["2k"]), "peaks": pk,
           "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids; inputs of the kernel rows rotate "
                   "through buffers larger than L2 where they are bound by memory"}
    return out


def dobepel_kernels(pk, sz):
    """Microseconds and fractions of the roofline of Dobepel's kernels and of Qwen3's like kernels at one size."""
    import torch
    from velox_b200.csrc import ops
    dev, bf = "cuda:0", torch.bfloat16
    E, H, G, HL, D = sz["width"], sz["heads"], sz["kv_heads"], sz["lin_heads"], 128
    T, B, CTX, S, win, keep = 2048, 8, 2048, PAGE, DOBEPEL_WINDOW, DOBEPEL_KEEP
    rows, row, us = kernel_rows(pk)
    ints = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    pages = B * (CTX // S)
    kp = torch.randn((pages, G, S, D), device=dev).to(bf)
    vp = torch.randn((pages, G, S, D), device=dev).to(bf)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(B, CTX // S)
    # -- attention over a prompt of T tokens (one request), window 1,024 --
    q = torch.randn((T, (H + 2 * G) * D), device=dev).to(bf)
    cu, off = ints([0, T]), ints([0])
    vis = sum(min(i + 1, win) + (min(keep, i + 1 - win) if i + 1 > win else 0) for i in range(T))
    fl = 2.0 * vis * 2 * D * H
    row("prompt attention, biased window (mma.sync, P in two halves)",
        us(lambda: ops.biased_prefill_attention(q, q.shape[1], kp, vp, bt, cu, off, D ** -0.5, win, keep, 8.0, H, G, D, D, 1, T, T)), fl)
    row("prompt attention, Qwen3 (mma.sync)",
        us(lambda: ops.paged_prefill_attention(q, q.shape[1], kp, vp, bt, cu, off, D ** -0.5, win, H, G, D, 1, T, T)), fl)
    row("prompt attention, Qwen3 (tcgen05)",
        us(lambda: ops.paged_prefill_attention_tc(q, q.shape[1], kp, vp, bt, cu, off, D ** -0.5, win, H, G, D, 1, T, T)), fl)
    # -- attention of B single tokens at CTX cached tokens --
    qd = torch.randn((B, (H + 2 * G) * D), device=dev).to(bf)
    seqs, pos = ints(list(range(B))), ints([CTX - 1] * B)
    nb = B * G * (win + keep) * 2 * D * 2.0
    row("decode attention, biased window", us(lambda: ops.biased_decode_attention(
        qd, qd.shape[1], kp, vp, bt, seqs, pos, D ** -0.5, win, keep, 8.0, H, G, D, D, B, max_kv=CTX), 50), 0.0, nb)
    row("decode attention, Qwen3", us(lambda: ops.paged_decode_attention(
        qd, qd.shape[1], kp, vp, bt, seqs, pos, D ** -0.5, win, H, G, D, B, CTX), 50), 0.0, B * G * win * 2 * D * 2.0)
    # -- linear attention --
    x = (torch.randn((T, 4 * HL * D), device=dev) * 0.5).to(bf)
    decay = torch.full((HL,), 0.97, device=dev)
    state = torch.zeros((B, HL, D, D), device=dev)
    lin_fl = T * HL * 2.0 * (32 * 2 * D + 2 * D * D)   # scores and values within chunks of 64 (half of them), state read and update
    slot0, cu_b, slots_b = ints([0]), ints(list(range(B + 1))), ints(list(range(B)))
    row("prompt linear attention, chunks side by side (mma.sync, halves)", us(lambda: ops.linear_attention(
        x, 0, HL * D, 2 * HL * D, decay, state, cu, slot0, 1, T, HL, D, D)), lin_fl)
    xd = (torch.randn((B, 4 * HL * D), device=dev) * 0.5).to(bf)
    row("decode linear attention, recurrent", us(lambda: ops.linear_attention(
        xd, 0, HL * D, 2 * HL * D, decay, state, cu_b, slots_b, B, 1, HL, D, D), 50),
        0.0, B * HL * D * D * 4 * 2.0)
    # -- feed-forward: routed experts against the dense gated product --
    NE, top, F = DOBEPEL_EXPERTS, DOBEPEL_TOP, sz["expert_ff"]
    h = torch.randn((T, E), device=dev).to(bf)
    wr, gu = torch.randn((NE, E), device=dev) * 0.1, (torch.randn((NE, 2 * F, E), device=dev) * 0.02).to(bf)
    dn = (torch.randn((NE, E, F), device=dev) * 0.02).to(bf)
    plan = ops.moe_route(h, wr, None, NE, top)
    a = ops.moe_gemm(h, gu, plan, True, bf, gated_activation="silu")
    row("experts gate_up, %d rows (grouped mma.sync)" % (T * top), us(lambda: ops.moe_gemm(h, gu, plan, True, bf, gated_activation="silu")),
        2.0 * T * top * 2 * F * E)
    row("experts down, %d rows (grouped mma.sync)" % (T * top), us(lambda: ops.moe_gemm(a, dn, plan, False, torch.float32)),
        2.0 * T * top * F * E)
    row("router and plan, %d tokens" % T, us(lambda: ops.moe_route(h, wr, None, NE, top)), 0.0, T * E * 2.0)
    plan128 = ops.moe_route(h, wr, None, NE, top, ops.MOE_TCGEN05_TILE_ROWS)
    hs = ops.moe_gather_rows(h, plan128)
    a128 = ops.moe_gemm_tcgen05(hs, gu, plan128, gated_activation="silu")
    row("experts: rows into expert order, %d rows" % (T * top), us(lambda: ops.moe_gather_rows(h, plan128)), 0.0, 2.0 * T * top * E * 2)
    row("experts gate_up, %d rows (grouped tcgen05, fused activation)" % (T * top),
        us(lambda: ops.moe_gemm_tcgen05(hs, gu, plan128, gated_activation="silu")), 2.0 * T * top * 2 * F * E)
    row("experts down, %d rows (grouped tcgen05)" % (T * top), us(lambda: ops.moe_gemm_tcgen05(a128, dn, plan128)),
        2.0 * T * top * F * E)
    I = top * F + sz["shared_ff"]
    wq = (torch.randn((2 * I, E), device=dev) * 0.02).to(bf)
    row("Qwen3 gate_up, %d rows (tcgen05, fused activation)" % T, us(lambda: ops.gemm_tcgen05(
        h, wq, None, gated_activation="silu", pair=ops.tcgen05_pair_better(T, 2 * I, h.device))), 2.0 * T * 2 * I * E)
    hd = torch.randn((B, E), device=dev).to(bf)
    pland = ops.moe_route(hd, wr, None, NE, top, ops.moe_tile_rows(hd, B * top))
    many = [(torch.randn((NE, 2 * F, E), device=dev) * 0.02).to(bf) for _ in range(max(2, int(3e8 // (NE * 2 * F * E * 2))))]
    k = [0]

    def experts_decode():
        k[0] = (k[0] + 1) % len(many)
        ops.moe_gemm(hd, many[k[0]], pland, True, bf, gated_activation="silu")
    touched = min(NE, B * top)
    row("experts gate_up, %d tokens (decode, grouped mma.sync, row tiles of 16)" % B, us(experts_decode, 50), 0.0,
        touched * 2 * F * E * 2.0)
    manyq = [(torch.randn((2 * I, E), device=dev) * 0.02).to(bf) for _ in range(max(2, int(3e8 // (2 * I * E * 2))))]

    def dense_decode():
        k[0] = (k[0] + 1) % len(manyq)
        ops.gemm_skinny(hd, manyq[k[0]], None, bf, gated_activation="silu")
    row("Qwen3 gate_up, %d tokens (decode, skinny)" % B, us(dense_decode, 50), 0.0, 2 * I * E * 2.0)
    # -- norms and residual --
    big = 16384   # rows: float32 residual + two branches, far larger than L2
    res = torch.randn((big, E), device=dev)
    y0, y1 = torch.randn((big, E), device=dev).to(bf), torch.randn((big, E), device=dev).to(bf)
    w = torch.ones(E, device=dev)
    row("two branch norms + sum + norm + residual + next norm, %d rows" % big,
        us(lambda: ops.merge_norm_add_norm(res, y0, w, 0.5, 1e-6, w, 0.5, y1, w, 0.5, w_next=w), 10), 0.0, big * E * (4 + 4 + 2 + 2 + 2.0))
    row("Qwen3 residual add + norm, %d rows" % big, us(lambda: ops.add_rmsnorm(res, y0, w, 1e-6, bf), 10), 0.0, big * E * (4 + 4 + 2 + 2.0))
    return rows


# ---- Buvuzen beside Dobepel and Qwen3 at equal size (`--workload buvuzen`) ------------------------------
# The same layer sizes as above: heads of 128 with values of 128, window 1,024, 8 experts and 2 identity experts in
# 5 groups of which 3 are kept, 2 chosen, a gated shared expert.  Dobepel is the closest existing model (attention
# without rotation under a window through the same kernels, routed experts with a shared one; it has a linear-attention
# member more), Qwen3 the dense one with the same q/k norm.
BUVUZEN_IDENTITY, BUVUZEN_GROUPS, BUVUZEN_KEEP = 2, 5, 3


def buvuzen_raw(sz):
    mixer = {"heads": sz["heads"], "kv_heads": sz["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
             "mask": {"size": DOBEPEL_WINDOW}}
    mlp = {"kind": "moe", "expert": {"ff": sz["expert_ff"]},
           "router": {"experts": DOBEPEL_EXPERTS, "identity": BUVUZEN_IDENTITY, "top": DOBEPEL_TOP, "scale": 2.0,
                      "groups": {"count": BUVUZEN_GROUPS, "keep": BUVUZEN_KEEP}}, "shared": {"ff": sz["shared_ff"]}}
    layer = {"type": "attention", "mixer": mixer, "mlp": mlp}
    return {"architecture": "Buvuzen", "vocab": DOBEPEL_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 2.0}, "logit_scale": 0.5, "layers": [json.loads(json.dumps(layer)) for _ in range(sz["layers"])]}


def buvuzen_workload(args, pk):
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 at 2,048 cached tokens) of Buvuzen, of
    Dobepel and of Qwen3 at equal size, through the step function, timed with CUDA events; then the kernels that the
    design added or changed beside the like kernels of the other two at the 2k size, each as a fraction of its roofline."""
    import torch
    from velox_b200.config import BuvuzenConfig, DobepelConfig, Qwen3Config

    T, B, CTX = 2048, 8, 2048
    K, W = max(1, min(args.steps, 32)), max(3, args.warmup)
    gen = torch.Generator().manual_seed(SEED)
    sizes = {}
    # (the first model of a process pays for the libraries' first calls well beyond its three warm-up steps: one run
    # of the smallest size is thrown away)
    model_points(BuvuzenConfig.from_dict(buvuzen_raw(DOBEPEL_SIZES["1k"])), DOBEPEL_VOCAB, T, B, CTX, K, W, gen)
    for name, sz in DOBEPEL_SIZES.items():
        sizes[name] = {"buvuzen": model_points(BuvuzenConfig.from_dict(buvuzen_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "dobepel": model_points(DobepelConfig.from_dict(dobepel_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "qwen3": model_points(Qwen3Config.from_dict(qwen_raw_like(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "shape": sz}
    return {"metric": "Buvuzen beside Dobepel and Qwen3 at equal size: prefill of %d tokens, decode at batch %d with %d cached "
                      "tokens, bf16" % (T, B, CTX), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "sizes": sizes,
            "value": sizes["2k"]["buvuzen"]["decode_tok_s"], "higher_is_better": True,
            "kernels": buvuzen_kernels(pk, DOBEPEL_SIZES["2k"]), "peaks": pk,
            "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids; inputs of the kernel rows rotate "
                    "through buffers larger than L2 where they are bound by memory"}


def buvuzen_kernels(pk, sz):
    """Microseconds and fractions of the roofline of the kernels Buvuzen added to or changed, beside the like kernels of
    Dobepel and Qwen3 at one size.  (The grouped products of the experts and the dense products are the same kernels as
    Dobepel's and Qwen3's: `--workload dobepel` has their rows.)"""
    import torch
    from velox_b200.csrc import ops
    dev, bf = "cuda:0", torch.bfloat16
    E, H, G, D = sz["width"], sz["heads"], sz["kv_heads"], 128
    T, B, CTX, S, win, keep = 2048, 8, 2048, PAGE, DOBEPEL_WINDOW, DOBEPEL_KEEP
    rows, row, us = kernel_rows(pk)
    ints = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    pages = B * (CTX // S)
    kp = torch.randn((pages, G, S, D), device=dev).to(bf)
    vp = torch.randn((pages, G, S, D), device=dev).to(bf)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(B, CTX // S)
    sinks = torch.randn(H, device=dev)
    width = (H + 2 * G) * D + (H + 7) // 8 * 8     # q | k | v | gates (padded to 8)
    gate_col = (H + 2 * G) * D
    # -- attention over a prompt of T tokens (one request), window 1,024 --
    q = torch.randn((T, width), device=dev).to(bf)
    cu, off = ints([0, T]), ints([0])
    fl = 2.0 * sum(min(i + 1, win) for i in range(T)) * 2 * D * H
    flk = 2.0 * sum(min(i + 1, win) + (min(keep, i + 1 - win) if i + 1 > win else 0) for i in range(T)) * 2 * D * H
    row("prompt attention, window + sink + gate (mma.sync, P in two halves)", us(lambda: ops.biased_prefill_attention(
        q, width, kp, vp, bt, cu, off, D ** -0.5, win, 0, 0.0, H, G, D, D, 1, T, T, sinks=sinks, gate_col=gate_col)), fl)
    row("prompt attention, window + sink + gate (tcgen05, P in two halves)", us(lambda: ops.paged_prefill_attention_tc(
        q, width, kp, vp, bt, cu, off, D ** -0.5, win, H, G, D, 1, T, T, max_kv=T, halves=True, sinks=sinks, gate_col=gate_col)), fl)
    row("prompt attention, Dobepel (biased window, kept first tokens)", us(lambda: ops.biased_prefill_attention(
        q, width, kp, vp, bt, cu, off, D ** -0.5, win, keep, 8.0, H, G, D, D, 1, T, T)), flk)
    row("prompt attention, Qwen3 (tcgen05)", us(lambda: ops.paged_prefill_attention_tc(
        q, width, kp, vp, bt, cu, off, D ** -0.5, win, H, G, D, 1, T, T)), fl)
    # -- attention of B single tokens at CTX cached tokens --
    qd = torch.randn((B, width), device=dev).to(bf)
    seqs, pos = ints(list(range(B))), ints([CTX - 1] * B)
    row("decode attention, window + sink + gate", us(lambda: ops.biased_decode_attention(
        qd, width, kp, vp, bt, seqs, pos, D ** -0.5, win, 0, 0.0, H, G, D, D, B, max_kv=CTX, sinks=sinks, gate_col=gate_col), 50),
        0.0, B * G * win * 2 * D * 2.0)
    row("decode attention, Dobepel (biased window)", us(lambda: ops.biased_decode_attention(
        qd, width, kp, vp, bt, seqs, pos, D ** -0.5, win, keep, 8.0, H, G, D, D, B, max_kv=CTX), 50),
        0.0, B * G * (win + keep) * 2 * D * 2.0)
    row("decode attention, Qwen3", us(lambda: ops.paged_decode_attention(
        qd, width, kp, vp, bt, seqs, pos, D ** -0.5, win, H, G, D, B, CTX), 50), 0.0, B * G * win * 2 * D * 2.0)
    # -- q/k norm and the write of keys and values into the pages (no rotation here; Qwen3 rotates) --
    slots = torch.randperm(pages * S, device=dev)[:T].to(torch.int32)
    wn = torch.ones(D, device=dev)
    positions = ints(list(range(T)))
    inv_freq = (1e6 ** (-torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D)).contiguous()
    nb = T * (H + 2 * G) * D * 2 * 2.0
    row("q/k norm + cache write, %d tokens" % T, us(lambda: ops.qk_norm_rope_kv(
        q, wn, wn, 1e-6, None, 0, positions, slots, kp, vp, H, G, D, D)), 0.0, nb)
    row("q/k norm + rotation + cache write, Qwen3, %d tokens" % T, us(lambda: ops.qk_norm_rope_kv(
        q, wn, wn, 1e-6, inv_freq, D, positions, slots, kp, vp, H, G, D)), 0.0, nb)
    # -- router and combination --
    NE, ident, top, F = DOBEPEL_EXPERTS, BUVUZEN_IDENTITY, DOBEPEL_TOP, sz["expert_ff"]
    R = NE + ident
    h = torch.randn((T, E), device=dev).to(bf)
    wr = torch.randn((R + 1, E), device=dev) * 0.1
    corr = torch.randn(R, device=dev) * 0.05
    route_b = lambda x, rows_: ops.moe_route(x, wr, None, R, top, rows_, scores="softmax_all", correction=corr,
                                             groups=BUVUZEN_GROUPS, keep_groups=BUVUZEN_KEEP, route_scale=2.0, identity=ident,
                                             shared_gate=True)
    wr_d = wr[:NE].contiguous()
    row("router and plan, %d tokens (softmax over all, groups, shared gate)" % T, us(lambda: route_b(h, ops.MOE_TCGEN05_TILE_ROWS)),
        0.0, T * E * 2.0)
    row("router and plan, Dobepel, %d tokens" % T, us(lambda: ops.moe_route(h, wr_d, None, NE, top, ops.MOE_TCGEN05_TILE_ROWS)),
        0.0, T * E * 2.0)
    plan, plan_d = route_b(h, ops.MOE_TCGEN05_TILE_ROWS), ops.moe_route(h, wr_d, None, NE, top, ops.MOE_TCGEN05_TILE_ROWS)
    y = torch.randn((T * top, E), device=dev).to(bf)
    shared = torch.randn((T, E), device=dev).to(bf)
    nbc = T * E * 2.0 * (top + 2)
    row("combination with identity experts and a gated shared expert, %d tokens" % T,
        us(lambda: ops.moe_combine(y, plan, shared, bf, h=h)), 0.0, nbc + T * E * 2.0)
    row("combination, Dobepel, %d tokens" % T, us(lambda: ops.moe_combine(y, plan_d, shared, bf)), 0.0, nbc)
    hd = torch.randn((B, E), device=dev).to(bf)
    row("router and plan, %d tokens (decode)" % B, us(lambda: route_b(hd, ops.MOE_SMALL_TILE_ROWS), 50), 0.0, (R + 1) * E * 4.0)
    row("router and plan, Dobepel, %d tokens (decode)" % B,
        us(lambda: ops.moe_route(hd, wr_d, None, NE, top, ops.MOE_SMALL_TILE_ROWS), 50), 0.0, NE * E * 4.0)
    # -- norms and residual --
    big = 16384   # rows: float32 residual + a branch, far larger than L2
    res = torch.randn((big, E), device=dev)
    y0, y1 = torch.randn((big, E), device=dev).to(bf), torch.randn((big, E), device=dev).to(bf)
    w = torch.ones(E, device=dev)
    row("norm of a sublayer's output + residual + rounded stream, %d rows" % big,
        us(lambda: ops.merge_norm_add_norm(res, y0, w, 1.0, 1e-6, rounded=True), 10), 0.0, big * E * (4 + 4 + 2 + 2.0))
    row("Dobepel: two branch norms + sum + norm + residual + next norm, %d rows" % big,
        us(lambda: ops.merge_norm_add_norm(res, y0, w, 0.5, 1e-6, w, 0.5, y1, w, 0.5, w_next=w), 10), 0.0, big * E * (4 + 4 + 2 + 2 + 2.0))
    row("Qwen3 residual add + norm, %d rows" % big, us(lambda: ops.add_rmsnorm(res, y0, w, 1e-6, bf), 10), 0.0, big * E * (4 + 4 + 2 + 2.0))
    tok = torch.randint(0, DOBEPEL_VOCAB, (big,), device=dev, dtype=torch.int32)
    table = torch.randn((DOBEPEL_VOCAB, E), device=dev).to(bf)
    rounded = torch.empty((big, E), device=dev, dtype=bf)
    row("embedding times a number + rounded stream, %d rows" % big, us(lambda: ops.embedding(tok, table, scale=2.0, rounded=rounded), 10),
        0.0, big * E * (2 + 4 + 2.0))
    row("embedding, Qwen3, %d rows" % big, us(lambda: ops.embedding(tok, table), 10), 0.0, big * E * (2 + 4.0))
    return rows


# ---- Kapuvik beside Dobepel at equal size (`--workload kapuvik`) ----------------------------------------
# The same widths and head counts as above, four layers: latent attention (heads of 128 + 64 rotated channels, values of
# 128, a latent row of 512), two layers of linear attention with a decay per channel (128 x 128 state a head, a decay
# projection through 16 channels), and one with softmax attention (heads of 128, scores bounded at 30) beside rotated
# linear attention with a fixed decay.  The dense feed-forward has the size that a Dobepel token runs through.  Dobepel is
# the closest existing model: the same side-by-side mixer of softmax attention and fixed-decay linear attention.
KAPUVIK_RANK, KAPUVIK_ROT, KAPUVIK_DECAY_RANK, KAPUVIK_CAP = 512, 64, 16, 30.0


def kapuvik_raw(sz):
    ff = {"kind": "dense", "ff": DOBEPEL_TOP * sz["expert_ff"] + sz["shared_ff"], "limit": 7.0}
    H, HL = sz["heads"], sz["lin_heads"]
    latent = {"type": "latent_attention", "mlp": ff, "mixer": {
        "heads": H, "dim": 128, "rot_dim": KAPUVIK_ROT, "vdim": 128, "kv_rank": KAPUVIK_RANK, "scale": 192 ** -0.5,
        "rot": {"base": 10000.0, "dims": KAPUVIK_ROT}}}
    gla = {"type": "gla", "mlp": ff, "mixer": {"heads": HL, "dim": 128, "vdim": 128, "tau": 16.0, "rank": KAPUVIK_DECAY_RANK}}
    left = {"heads": H, "kv_heads": sz["kv_heads"], "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": KAPUVIK_CAP,
            "rot": {"base": 10000.0, "dims": 128}}
    right = {"heads": HL, "dim": 128, "vdim": 128, "rot": {"base": 10000.0, "dims": 64},
             "decay": [1.0 - 2.0 ** (-5.0 - 5.0 * h / max(1, HL - 1)) for h in range(HL)]}
    both = {"type": "parallel", "mlp": ff, "mixer": {"left": left, "right": right, "left_scale": 0.8, "right_scale": 0.9}}
    return {"architecture": "Kapuvik", "vocab": DOBEPEL_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": 0.5}, "logit_softcap": 15.0,
            "layers": [json.loads(json.dumps(x)) for x in (latent, gla, gla, both)]}


def kapuvik_workload(args, pk):
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 at 2,048 cached tokens) of Kapuvik and of
    Dobepel at equal width and depth, through the step function, timed with CUDA events; then the design's own kernels
    beside Dobepel's like kernels at the 2k size, each as a fraction of its roofline."""
    import torch
    from velox_b200.config import DobepelConfig, KapuvikConfig

    T, B, CTX = 2048, 8, 2048
    K, W = max(1, min(args.steps, 32)), max(3, args.warmup)
    gen = torch.Generator().manual_seed(SEED)
    sizes = {}
    four = lambda sz: dict(sz, layers=4)
    model_points(KapuvikConfig.from_dict(kapuvik_raw(four(DOBEPEL_SIZES["1k"]))), DOBEPEL_VOCAB, T, B, CTX, K, W, gen)  # thrown away
    for name, sz in DOBEPEL_SIZES.items():
        sz = four(sz)
        sizes[name] = {"kapuvik": model_points(KapuvikConfig.from_dict(kapuvik_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "dobepel": model_points(DobepelConfig.from_dict(dobepel_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "shape": sz}
    return {"metric": "Kapuvik beside Dobepel at equal size: prefill of %d tokens, decode at batch %d with %d cached tokens, bf16"
                      % (T, B, CTX), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "sizes": sizes,
            "value": sizes["2k"]["kapuvik"]["decode_tok_s"], "higher_is_better": True,
            "kernels": kapuvik_kernels(pk, four(DOBEPEL_SIZES["2k"])), "peaks": pk,
            "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids"}


def kapuvik_kernels(pk, sz):
    """Microseconds and fractions of the roofline of Kapuvik's kernels beside Dobepel's like kernels at one size."""
    import torch
    from velox_b200.csrc import ops
    dev, bf = "cuda:0", torch.bfloat16
    E, H, G, HL, D = sz["width"], sz["heads"], sz["kv_heads"], sz["lin_heads"], 128
    C, R = KAPUVIK_RANK, KAPUVIK_ROT
    T, B, CTX, S = 2048, 8, 2048, PAGE
    rows, row, us = kernel_rows(pk)
    ints = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    pages = B * (CTX // S)
    kp = torch.randn((pages, G, S, D), device=dev).to(bf)
    vp = torch.randn((pages, G, S, D), device=dev).to(bf)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(B, CTX // S)
    cu, off = ints([0, T]), ints([0])
    seq_t, pos_t = ints([0] * T), ints(list(range(T)))
    seqs, pos = ints(list(range(B))), ints([CTX - 1] * B)
    # -- softmax attention with bounded scores: a prompt of T tokens, then B single tokens at CTX cached tokens --
    q = torch.randn((T, (H + 2 * G) * D), device=dev).to(bf)
    qd = torch.randn((B, (H + 2 * G) * D), device=dev).to(bf)
    fl = 2.0 * (T * (T + 1) // 2) * 2 * D * H
    nb = B * G * CTX * 2 * D * 2.0
    if ops.biased_attention_supported(bf, D, D, S):
        row("prompt attention, bounded scores (mma.sync, P in two halves)", us(lambda: ops.biased_prefill_attention(
            q, q.shape[1], kp, vp, bt, cu, off, D ** -0.5, 0, 0, 0.0, H, G, D, D, 1, T, T, softcap=KAPUVIK_CAP)), fl)
        row("prompt attention, Dobepel (biased, no window)", us(lambda: ops.biased_prefill_attention(
            q, q.shape[1], kp, vp, bt, cu, off, D ** -0.5, 0, 0, 8.0, H, G, D, D, 1, T, T)), fl)
        row("decode attention, bounded scores", us(lambda: ops.biased_decode_attention(
            qd, qd.shape[1], kp, vp, bt, seqs, pos, D ** -0.5, 0, 0, 0.0, H, G, D, D, B, max_kv=CTX, softcap=KAPUVIK_CAP), 50), 0.0, nb)
        row("decode attention, Dobepel (biased, no window)", us(lambda: ops.biased_decode_attention(
            qd, qd.shape[1], kp, vp, bt, seqs, pos, D ** -0.5, 0, 0, 8.0, H, G, D, D, B, max_kv=CTX), 50), 0.0, nb)
    # -- latent attention: rows of C + R elements, one key/value head for all query heads --
    lp = torch.randn((pages, 1, S, C + R), device=dev).to(bf)
    qa = torch.randn((T, H, C + R), device=dev).to(bf)
    qad = torch.randn((B, H, C + R), device=dev).to(bf)
    lfl = 2.0 * (T * (T + 1) // 2) * (2 * C + R) * H
    lnb = B * CTX * (C + R) * 2.0
    row("prompt latent attention (folded queries over cached rows)", us(lambda: ops.latent_attention(
        qa, lp, bt, seq_t, pos_t, 192 ** -0.5, H, C, R, max_kv=T), 3), lfl)
    if ops.raised_attention_supported(bf, D + R, D):
        # the same prompt the other way round: rows gathered out of the pages, keys and values raised by one product, the
        # tensor-core prompt kernel on them (heads of D + R keys and D values); FLOPs of the raised form
        plan = ops.RaisedPlan([T], dev)
        w_raise = (torch.randn((H * (2 * D + R), C + R), device=dev) * 0.05).to(bf)
        qr = torch.randn((T, H * (D + R)), device=dev).to(bf)
        rfl = 2.0 * (T * (T + 1) // 2) * (2 * D + R) * H
        kv_rows = ops.gemm_bf16(ops.latent_gather(lp, bt, cu, off, plan), w_raise)
        row("prompt latent attention, raised: tensor-core kernel on raised rows (keys of %d, values of %d)" % (D + R, D), us(
            lambda: ops.raised_attention(qr, qr.shape[1], kv_rows, cu, off, plan, 192 ** -0.5, H, D + R, D, T)), rfl)
        row("prompt latent attention, raised: gather of %d cached rows + product that raises them" % T, us(
            lambda: ops.gemm_bf16(ops.latent_gather(lp, bt, cu, off, plan), w_raise)), 2.0 * T * (C + R) * H * (2 * D + R))
    row("decode latent attention", us(lambda: ops.latent_attention(
        qad, lp, bt, seqs, pos, 192 ** -0.5, H, C, R, max_kv=CTX), 20), 0.0, lnb)
    down, qq = torch.randn((T, C + R), device=dev).to(bf), torch.randn((T, H * (D + R)), device=dev).to(bf)
    slots = torch.randperm(pages * S, device=dev)[:T].to(torch.int32)
    inv64 = (1e4 ** (-torch.arange(0, R, 2, device=dev, dtype=torch.float32) / R)).contiguous()
    wl = torch.ones(C, device=dev)
    qa3 = qa
    row("latent row: norm + rotation + cache write + query rotation, %d tokens" % T, us(lambda: ops.latent_prep(
        down, qq, qa3, wl, 1e-6, inv64, True, pos_t, slots, lp, H, D, R, C)), 0.0, T * ((C + R) * 4 + H * R * 4.0))
    inv128 = (1e4 ** (-torch.arange(0, D, 2, device=dev, dtype=torch.float32) / D)).contiguous()
    row("Dobepel/Qwen3: q/k rotation + cache write, %d tokens" % T, us(lambda: ops.qk_norm_rope_kv(
        q, None, None, 1e-6, inv128, D, pos_t, slots, kp, vp, H, G, D, D)), 0.0, T * (H + 2 * G) * D * 2 * 2.0)
    # -- linear attention --
    x = (torch.randn((T, 4 * HL * D), device=dev) * 0.5).to(bf)
    xd = (torch.randn((B, 4 * HL * D), device=dev) * 0.5).to(bf)
    decay = torch.full((HL,), 0.97, device=dev)
    state = torch.zeros((B, HL, D, D), device=dev)
    gate, gated = torch.randn((T, HL * D), device=dev) + 2.0, torch.randn((B, HL * D), device=dev) + 2.0
    slot0, cu_b, slots_b = ints([0]), ints(list(range(B + 1))), ints(list(range(B)))
    lin_fl = T * HL * 2.0 * (32 * 2 * D + 2 * D * D)
    sb = B * HL * D * D * 4 * 2.0
    inv_r = (1e4 ** (-torch.arange(0, 64, 2, device=dev, dtype=torch.float32) / 64)).contiguous()
    plan = ops.StretchPlan([T], dev)
    row("prompt linear attention, decay per channel (float32 operands, stretches side by side)", us(lambda: ops.linear_attention_walk(
        x, 0, HL * D, 2 * HL * D, state, cu, slot0, 1, HL, D, D, gate=gate, gate_mul=1 / 16.0, q_mul=D ** -0.5, stretches=plan), 5), lin_fl)
    row("prompt linear attention, rotated, fixed decay (float32 operands, stretches side by side)", us(lambda: ops.linear_attention_walk(
        x, 0, HL * D, 2 * HL * D, state, cu, slot0, 1, HL, D, D, decay=decay, inv_freq=inv_r, rot_dim=64, positions=pos_t,
        k_mul=D ** -0.5, stretches=plan), 5), lin_fl)
    row("prompt linear attention, decay per channel, in order (one walk)", us(lambda: ops.linear_attention_walk(
        x, 0, HL * D, 2 * HL * D, state, cu, slot0, 1, HL, D, D, gate=gate, gate_mul=1 / 16.0, q_mul=D ** -0.5), 3), lin_fl)
    row("prompt linear attention, Dobepel (chunks side by side, mma.sync, halves)", us(lambda: ops.linear_attention(
        x, 0, HL * D, 2 * HL * D, decay, state, cu, slot0, 1, T, HL, D, D)), lin_fl)
    posd = ints([CTX - 1] * B)
    row("decode linear attention, decay per channel", us(lambda: ops.linear_attention_walk(
        xd, 0, HL * D, 2 * HL * D, state, cu_b, slots_b, B, HL, D, D, gate=gated, gate_mul=1 / 16.0, q_mul=D ** -0.5), 50), 0.0, sb)
    row("decode linear attention, rotated, fixed decay", us(lambda: ops.linear_attention_walk(
        xd, 0, HL * D, 2 * HL * D, state, cu_b, slots_b, B, HL, D, D, decay=decay, inv_freq=inv_r, rot_dim=64, positions=posd,
        k_mul=D ** -0.5), 50), 0.0, sb)
    row("decode linear attention, Dobepel (recurrent)", us(lambda: ops.linear_attention(
        xd, 0, HL * D, 2 * HL * D, decay, state, cu_b, slots_b, B, 1, HL, D, D), 50), 0.0, sb)
    big = 16384
    o = torch.randn((big, HL * D), device=dev)
    g = torch.randn((big, HL * D), device=dev).to(bf)
    wv = torch.ones(D, device=dev)
    row("per-head norm + silu gate, %d rows" % big, us(lambda: ops.head_norm_gate(o, g, wv, HL, 1e-6, "silu"), 10), 0.0, big * HL * D * 8.0)
    wj = torch.ones(HL * D, device=dev)
    row("Dobepel: joined norm + sigmoid gate, %d rows" % big, us(lambda: ops.gated_rmsnorm(o, g, wj, 1e-6), 10), 0.0, big * HL * D * 8.0)
    # -- feed-forward activation, stream update --
    I = DOBEPEL_TOP * sz["expert_ff"] + sz["shared_ff"]
    sums = torch.randn((big, 2 * I), device=dev)
    bias = torch.randn(2 * I, device=dev)
    row("bounded gated activation on float32 sums + biases, %d rows" % big, us(lambda: ops.capped_gated_act(sums, bias, 7.0, 1.702, bf), 10),
        0.0, big * I * (8 + 2.0))
    res = torch.randn((big, E), device=dev)
    y0, y1 = torch.randn((big, E), device=dev).to(bf), torch.randn((big, E), device=dev).to(bf)
    w = torch.ones(E, device=dev)
    row("stream += mixer + feed-forward, then the next norm, %d rows" % big,
        us(lambda: ops.sum_add_rmsnorm(res, [(y0, 1.0), (y1, 1.0)], weight=w, eps=1e-6), 10), 0.0, big * E * (4 + 4 + 2 + 2 + 2.0))
    row("Dobepel: two branch norms + sum + norm + residual + next norm, %d rows" % big,
        us(lambda: ops.merge_norm_add_norm(res, y0, w, 0.5, 1e-6, w, 0.5, y1, w, 0.5, w_next=w), 10), 0.0, big * E * (4 + 4 + 2 + 2 + 2.0))
    return rows


# ---- Fovenex beside Kapuvik at equal size (`--workload fovenex`) ----------------------------------------
# The same widths and head counts as above, four layers: latent attention (heads of 128 + 64 rotated channels, values of
# 128, a latent row of 512 + 64, queries through a latent of 768, a window of 1,024), two layers of differential attention
# (every head two maps of 64 channels over values of 128, grouped key/value heads, stretched rotation), and a latent layer
# that reads the first one's rows.  Four copies of the stream; the dense feed-forward has the size that a Dobepel token runs
# through.  Kapuvik is the closest existing model: latent attention through the same kernels, softmax attention through the
# same tensor-core kernels, a dense feed-forward, one elementwise kernel a sublayer.
FOVENEX_QRANK, FOVENEX_WINDOW, FOVENEX_STREAMS = 768, 1024, 4


def fovenex_raw(sz):
    ff = {"kind": "dense", "ff": DOBEPEL_TOP * sz["expert_ff"] + sz["shared_ff"]}
    H = sz["heads"]
    lat = {"heads": H, "dim": 128, "rot_dim": KAPUVIK_ROT, "vdim": 128, "kv_rank": KAPUVIK_RANK, "q_rank": FOVENEX_QRANK,
           "scale": 192 ** -0.5, "rot": {"base": 10000.0, "dims": KAPUVIK_ROT}, "mask": {"size": FOVENEX_WINDOW}}
    att = {"heads": H, "kv_heads": sz["kv_heads"], "dim": 64, "vdim": 128, "scale": 64 ** -0.5, "diff": 0.3,
           "rot": {"base": 10000.0, "dims": 32, "scaling": {"factor": 2.0, "original": 1024, "fast": 32.0, "slow": 1.0}}}
    layers = [{"type": "latent_attention", "mixer": lat, "mlp": ff}, {"type": "attention", "mixer": att, "mlp": ff},
              {"type": "attention", "mixer": att, "mlp": ff}, {"type": "latent_attention", "mixer": dict(lat, kv_from=0), "mlp": ff}]
    return {"architecture": "Fovenex", "vocab": DOBEPEL_VOCAB, "width": sz["width"], "norm": {"eps": 1e-6}, "residual_mult": 0.7,
            "streams": FOVENEX_STREAMS, "layers": json.loads(json.dumps(layers))}


def fovenex_workload(args, pk):
    """Prefill (one prompt of 2,048 tokens in one step) and decode (batch 8 at 2,048 cached tokens) of Fovenex and of
    Kapuvik at equal width and depth, through the step function, timed with CUDA events; then the design's own kernels
    beside the like kernels of Kapuvik and Qwen3 at the 2k size, each as a fraction of its roofline."""
    import torch
    from velox_b200.config import FovenexConfig, KapuvikConfig

    T, B, CTX = 2048, 8, 2048
    K, W = max(1, min(args.steps, 32)), max(3, args.warmup)
    gen = torch.Generator().manual_seed(SEED)
    sizes = {}
    four = lambda sz: dict(sz, layers=4)
    model_points(FovenexConfig.from_dict(fovenex_raw(four(DOBEPEL_SIZES["1k"]))), DOBEPEL_VOCAB, T, B, CTX, K, W, gen)  # thrown away
    for name, sz in DOBEPEL_SIZES.items():
        sz = four(sz)
        sizes[name] = {"fovenex": model_points(FovenexConfig.from_dict(fovenex_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "kapuvik": model_points(KapuvikConfig.from_dict(kapuvik_raw(sz)), DOBEPEL_VOCAB, T, B, CTX, K, W, gen),
                       "shape": sz}
    return {"metric": "Fovenex beside Kapuvik at equal size: prefill of %d tokens, decode at batch %d with %d cached tokens, bf16"
                      % (T, B, CTX), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "sizes": sizes,
            "value": sizes["2k"]["fovenex"]["decode_tok_s"], "higher_is_better": True,
            "kernels": fovenex_kernels(pk, four(DOBEPEL_SIZES["2k"])), "peaks": pk,
            "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids"}


def fovenex_kernels(pk, sz):
    """Microseconds and fractions of the roofline of Fovenex's kernels beside the like kernels of Kapuvik and Qwen3."""
    import torch
    from velox_b200.csrc import ops
    dev, bf = "cuda:0", torch.bfloat16
    E, H, G = sz["width"], sz["heads"], sz["kv_heads"]
    D, Dv, DL = 64, 128, 128
    C, R, WIN = KAPUVIK_RANK, KAPUVIK_ROT, FOVENEX_WINDOW
    T, B, CTX, S = 2048, 8, 2048, PAGE
    rows, row, us = kernel_rows(pk)
    ints = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    pages = B * (CTX // S)
    bt = torch.arange(pages, dtype=torch.int32, device=dev).view(B, CTX // S)
    cu, off = ints([0, T]), ints([0])
    pos_t = ints(list(range(T)))
    seqs, pos = ints(list(range(B))), ints([CTX - 1] * B)
    # -- differential attention: 2 H query heads of 64 over 2 G key heads of 64 and G value heads of 128 --
    kp2 = torch.randn((pages, 2 * G, S, D), device=dev).to(bf)
    vp1 = torch.randn((pages, G, S, Dv), device=dev).to(bf)
    width = 2 * (H + G) * D + G * Dv + H
    width += (-width) % 8
    q = torch.randn((T, width), device=dev).to(bf)
    qd = torch.randn((B, width), device=dev).to(bf)
    fl = 2.0 * (T * (T + 1) // 2) * (D + Dv) * 2 * H
    nb = B * CTX * (2 * G * D + G * Dv) * 2.0
    row("prompt differential attention: both maps (mma.sync, P in two halves, shared values, float32 out)", us(
        lambda: ops.biased_prefill_attention(q, width, kp2, vp1, bt, cu, off, D ** -0.5, 0, 0, 0.0, 2 * H, 2 * G, D, Dv, 1, T, T,
                                             v_share=2, out_float32=True)), fl)
    row("decode differential attention: both maps", us(
        lambda: ops.biased_decode_attention(qd, width, kp2, vp1, bt, seqs, pos, D ** -0.5, 0, 0, 0.0, 2 * H, 2 * G, D, Dv, B, max_kv=CTX,
                                            v_share=2, out_float32=True), 50), 0.0, nb)
    # the like kernel of Kapuvik: the same kernels on H heads of 128 over G key and G value heads of 128, bounded scores
    kp = torch.randn((pages, G, S, DL), device=dev).to(bf)
    vp = torch.randn((pages, G, S, DL), device=dev).to(bf)
    qk = torch.randn((T, (H + 2 * G) * DL), device=dev).to(bf)
    qkd = torch.randn((B, (H + 2 * G) * DL), device=dev).to(bf)
    row("Kapuvik: prompt attention, bounded scores (the same kernel)", us(lambda: ops.biased_prefill_attention(
        qk, qk.shape[1], kp, vp, bt, cu, off, DL ** -0.5, 0, 0, 0.0, H, G, DL, DL, 1, T, T, softcap=KAPUVIK_CAP)),
        2.0 * (T * (T + 1) // 2) * 2 * DL * H)
    row("Kapuvik: decode attention, bounded scores (the same kernel)", us(lambda: ops.biased_decode_attention(
        qkd, qkd.shape[1], kp, vp, bt, seqs, pos, DL ** -0.5, 0, 0, 0.0, H, G, DL, DL, B, max_kv=CTX, softcap=KAPUVIK_CAP), 50),
        0.0, B * G * CTX * 2 * DL * 2.0)
    maps = torch.randn((T, 2 * H * Dv), device=dev)
    row("difference of the maps + per-head norm + gate, %d tokens" % T, us(lambda: ops.diff_combine(
        maps, q, 2 * (H + G) * D + G * Dv, 0.4, 0.7, 1e-6, H, H // G, Dv, bf)), 0.0, T * H * Dv * (8 + 2.0))
    og = torch.randn((T, H * Dv), device=dev)
    gg = torch.randn((T, H * Dv), device=dev).to(bf)
    wv = torch.ones(Dv, device=dev)
    row("Kapuvik: per-head norm + silu gate, %d tokens" % T, us(lambda: ops.head_norm_gate(og, gg, wv, H, 1e-6, "silu")), 0.0,
        T * H * Dv * (4 + 2 + 2.0))
    slots = torch.randperm(pages * S, device=dev)[:T].to(torch.int32)
    inv32 = (1e4 ** (-torch.arange(0, 32, 2, device=dev, dtype=torch.float32) / 32)).contiguous()
    qn = torch.ones(D, device=dev)
    row("q/k norm + stretched rotation + cache write, shared values, %d tokens" % T, us(lambda: ops.qk_norm_rope_kv(
        q, qn, qn, 1e-6, inv32, 32, pos_t, slots, kp2, vp1, 2 * H, 2 * G, D, Dv, num_v_heads=G, magnitude=1.07)), 0.0,
        T * (2 * (H + G) * D + G * Dv) * 2 * 2.0)
    inv128 = (1e4 ** (-torch.arange(0, DL, 2, device=dev, dtype=torch.float32) / DL)).contiguous()
    row("Qwen3/Kapuvik: q/k rotation + cache write, %d tokens" % T, us(lambda: ops.qk_norm_rope_kv(
        qk, None, None, 1e-6, inv128, DL, pos_t, slots, kp, vp, H, G, DL, DL)), 0.0, T * (H + 2 * G) * DL * 2 * 2.0)
    qn128 = torch.ones(DL, device=dev)
    row("Qwen3: q/k norm + rotation + cache write, %d tokens" % T, us(lambda: ops.qk_norm_rope_kv(
        qk, qn128, qn128, 1e-6, inv128, DL, pos_t, slots, kp, vp, H, G, DL, DL)), 0.0, T * (H + 2 * G) * DL * 2 * 2.0)
    # -- latent attention under a window --
    lp = torch.randn((pages, 1, S, C + R), device=dev).to(bf)
    qad = torch.randn((B, H, C + R), device=dev).to(bf)
    row("decode latent attention, window %d (folded)" % WIN, us(lambda: ops.latent_attention(
        qad, lp, bt, seqs, pos, 192 ** -0.5, H, C, R, max_kv=CTX, window=WIN), 20), 0.0, B * WIN * (C + R) * 2.0)
    row("Kapuvik: decode latent attention, all %d rows (the same kernel)" % CTX, us(lambda: ops.latent_attention(
        qad, lp, bt, seqs, pos, 192 ** -0.5, H, C, R, max_kv=CTX), 20), 0.0, B * CTX * (C + R) * 2.0)
    if ops.raised_attention_supported(bf, DL + R, DL):
        w_raise = (torch.randn((H * (2 * DL + R), C + R), device=dev) * 0.05).to(bf)
        qr = torch.randn((T, H * (DL + R)), device=dev).to(bf)
        for name, win in (("prompt latent attention, window %d, raised rows (mma.sync portion kernel, keys of 192)" % WIN, WIN),
                          ("Kapuvik: prompt latent attention, no window (the same kernel)", 0)):
            plan = ops.RaisedPlan([T], dev, [0], win)
            kv_rows = ops.gemm_bf16(ops.latent_gather(lp, bt, cu, off, plan), w_raise)
            pairs = sum(min(i + 1, win) if win else i + 1 for i in range(T))
            row(name, us(lambda: ops.raised_attention(qr, qr.shape[1], kv_rows, cu, off, plan, 192 ** -0.5, H, DL + R, DL, T)),
                2.0 * pairs * (2 * DL + R) * H)
        # a portion of 256 tokens on 1,792 cached rows: only the window's rows are gathered and raised
        cu2, off2 = ints([0, 256]), ints([CTX - 256])
        for name, win in (("gather + raise for 256 new tokens at 1,792 cached, window %d" % WIN, WIN),
                          ("Kapuvik: gather + raise for 256 new tokens at 1,792 cached, no window", 0)):
            plan2 = ops.RaisedPlan([CTX], dev, [CTX - 256], win)
            row(name, us(lambda: ops.gemm_bf16(ops.latent_gather(lp, bt, cu2, off2, plan2), w_raise)),
                2.0 * plan2.rows * (C + R) * H * (2 * DL + R))
    og2 = torch.randn((T, H * DL), device=dev).to(bf)
    row("gate element by element, %d tokens" % T, us(lambda: ops.sigmoid_gate(og2, gg)), 0.0, T * H * DL * 6.0)
    # -- the stream in four copies --
    big, n = 16384, FOVENEX_STREAMS
    xs = torch.randn((big, n * E), device=dev)
    y = torch.randn((big, E), device=dev).to(bf)
    w, ls = torch.ones(E, device=dev), torch.ones(E, device=dev)
    mix = [[1.0 if a == b else 0.05 for b in range(n)] for a in range(n)]
    coef = [0.25] * n
    row("stream in %d copies: update + mixing + next weighted sum + layer norm, %d rows" % (n, big),
        us(lambda: ops.stream_update(xs, n, mix, coef, 0.7, ls, y, coef, w, 1e-6), 10), 0.0, big * E * (2 * n * 4 + 2 + 2.0))
    x1 = torch.randn((big, E), device=dev)
    row("one copy: update + layer scale + next layer norm, %d rows" % big,
        us(lambda: ops.stream_update(x1, 1, None, None, 0.7, ls, y, None, w, 1e-6), 10), 0.0, big * E * (4 + 4 + 2 + 2.0))
    row("Kapuvik: stream += one term, then the next RMS norm, %d rows" % big,
        us(lambda: ops.sum_add_rmsnorm(x1, [(y, 1.0)], weight=w, eps=1e-6), 10), 0.0, big * E * (4 + 4 + 2 + 2.0))
    rows_i = ints(list(range(0, big, 64)))
    row("sum of %d copies + last layer norm of %d wanted rows" % (n, big // 64),
        us(lambda: ops.stream_norm(xs, n, None, w, 1e-6, bf, rows=rows_i), 10), 0.0, (big // 64) * E * (n * 4 + 2.0))
    return rows


def main() -> int:
    global CONTEXT, PROMPT
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the model has (recorded in config)")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--workload", default="decode", choices=["decode", "stream", "dobepel", "buvuzen", "kapuvik", "fovenex"],
                    help="decode: the benchmark (steady decoding at a fixed batch). stream: continuous batching "
                         "under arrivals (64 requests, prompts of 128-4,096 tokens, 256 new tokens each, Poisson "
                         "arrivals); prints its own JSON line. dobepel: the Dobepel design beside Qwen3 at equal size "
                         "(prefill, decode, and the design's kernels against their rooflines); its own JSON line. buvuzen: the same for "
                         "the Buvuzen design beside Dobepel and Qwen3. kapuvik: the same for the Kapuvik design beside Dobepel. "
                         "fovenex: the same for the Fovenex design beside Kapuvik")
    ap.add_argument("--arrival-rate", type=float, default=16.0, help="stream: mean arrivals a second")
    ap.add_argument("--lazy-graphs", action="store_true",
                    help="stream: capture each decode graph when a step first needs it, inside the run")
    ap.add_argument("--pool-tokens", type=int, default=0, help="stream: cache pool in tokens (0: room for all)")
    ap.add_argument("--max-batch-tokens", type=int, default=2048,
                    help="stream: new tokens of one step (a decoded token that rides with a prompt portion waits for it)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES),
                    help="layer sizes: 8b is the benchmark's; the others are Qwen3-0.6B / 1.7B / 4B / 14B / 32B")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64 and prefill")
    ap.add_argument("--context", type=int, default=CONTEXT,
                    help="context length the decoding requests reach (the benchmark's is %d; others for measurements "
                         "beside it; the prefill point is a prompt of half of it)" % CONTEXT)
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust project whose GPU path is Apple Metal: pip finds neither setup.py "
                          "nor pyproject.toml, there is no Rust toolchain, and no Metal device on this box"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus %d is not supported" % args.gpus)
        return 2
    K, W = max(1, args.steps), max(3, args.warmup)
    CONTEXT, PROMPT = int(args.context), int(args.context) // 2

    import torch
    from velox_b200 import Engine, EngineConfig, Qwen3Config, SamplingParams
    from velox_b200.csrc import ops
    from velox_b200.engine import StepEntry

    if args.workload in ("dobepel", "buvuzen", "kapuvik", "fovenex"):
        with ClockSampler() as clocks:
            res = {"dobepel": dobepel_workload, "buvuzen": buvuzen_workload, "kapuvik": kapuvik_workload, "fovenex": fovenex_workload}[args.workload](args, peaks())
        res["clocks"] = clocks.summary()
        print(json.dumps(res))
        return 0
    model = dict(MODEL, **SHAPES[args.shape])
    layers = args.layers or model["num_hidden_layers"]
    raw = dict(model, num_hidden_layers=layers)
    cfg = Qwen3Config.from_dict(raw)
    pk = peaks()
    if args.workload == "stream":
        with ClockSampler() as clocks:
            res = stream_workload(args, cfg, layers)
        res["clocks"] = clocks.summary()
        print(json.dumps(res))
        return 0
    # the points' largest batch: 64, or what the cache of so many requests at this context leaves room for
    per_token = 2 * layers * cfg.num_key_value_heads * cfg.head_dim * 2
    free_bytes = torch.cuda.mem_get_info()[0] - weight_bytes(raw, layers)
    big = 64
    while big > args.batch and big * (CONTEXT + PAGE) * per_token > 0.8 * free_bytes:
        big //= 2
    max_batch = max(big, args.batch) if not args.skip_points else args.batch
    engine = Engine(model_config=cfg, random_seed=SEED, config=EngineConfig(
        dtype="bfloat16", page_size=PAGE, num_pages=max_batch * (CONTEXT // PAGE + 1) + 8,
        max_running_requests=max_batch, max_batch_tokens=2048, max_model_len=CONTEXT + PAGE))
    gen = torch.Generator().manual_seed(SEED)

    def prompts(n, length):
        return torch.randint(0, cfg.vocab_size, (n, length), generator=gen).tolist()

    def timed(fn, steps):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps

    def decode_run(batch, steps, warmup, context=None):
        context = context or CONTEXT
        """`batch` requests prefilled so that the timed steps end at the context
        length.  Times `steps` steps through the public entry point (host ids in,
        sampled ids out, every step), then `steps` steps of the step function and
        sampler alone (ids stay on the device).  Returns (ms end to end, ms on the
        device, kernel launches per device step, mean cached tokens per request
        during the device steps)."""
        # Requests whose prompts are done start decoding while the others' prompts
        # are still going in (2,048 new tokens a step), so the first one decodes
        # `stagger` tokens more than the last; it is the one that ends at CONTEXT.
        budget = 2 * steps + warmup + 1
        stagger = -(-batch * context // 2048) + 2 if batch > 1 else 0
        start = context - budget - stagger
        sp = SamplingParams(max_tokens=budget + stagger, ignore_eos=True)
        for p in prompts(batch, start):
            engine.add_request(p, SamplingParams(**vars(sp)))
        while engine.scheduler.waiting or any(engine.cache.length(r) < start for r in engine.scheduler.running):
            engine.step()
        assert len(engine.scheduler.running) == batch, "a request ended during the prompts"
        for _ in range(warmup):
            engine.step()
        e2e_ms = timed(engine.step, steps)
        assert len(engine.scheduler.running) == batch
        entries = [StepEntry(r.request_id, [r.last_token], [0]) for r in engine.scheduler.running.values()]
        zeros, ones = [0.0] * batch, [1.0] * batch
        held = sum(engine.cache.length(r) for r in engine.scheduler.running) / batch

        def device_step():
            engine.runner.step_and_sample(entries, zeros, ones, zeros)
        n0 = ops.launch_count()
        dev_ms = timed(device_step, steps)
        launches = (ops.launch_count() - n0) // steps
        assert max(engine.cache.length(r) for r in engine.scheduler.running) <= context
        for r in list(engine.scheduler.running.values()):
            engine.scheduler._finish(r, "length")
        return e2e_ms, dev_ms, launches, held + steps / 2.0

    out = {"metric": "decode tok/s @ batch %d, Qwen3-%s bf16, context %d" % (args.batch, args.shape.upper(), CONTEXT),
           "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02) seed 2, uniform random token ids"}

    with ClockSampler() as clocks:
        e2e_ms, ms, launches, kv_mid = decode_run(args.batch, K, W)
    out["clocks"] = clocks.summary()
    out.update({"value": round(args.batch * 1000.0 / ms, 1), "ms_per_step": round(ms, 4),
                "gpu_launches": int(launches * K)})
    # per step through the entry point: the step's description (token ids, positions,
    # block tables, slot mapping) goes up in one pinned copy, the sampled ids come back
    h2d = max(4 * g.host.numel() for (b, _), g in engine.runner.graphs.graphs.items() if b == args.batch)
    out["e2e"] = {"value": round(args.batch * 1000.0 / e2e_ms, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch}
    nbytes = decode_bytes(raw, layers, args.batch, kv_mid)
    ach = nbytes / (ms * 1e-3) / 1e9
    out["roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                       "frac": round(ach / pk["hbm_gbs"], 4), "peak_source": pk["source"]}

    if not args.skip_points:
        # prefill: one prompt of 2,048 tokens in one step
        toks = prompts(1, PROMPT)[0]

        last_logits = []

        def one_prefill():
            engine.cache.add_request("prefill")
            last_logits[:] = [engine.run_step([StepEntry("prefill", toks, [PROMPT - 1])])]
            engine.cache.release("prefill")
        for _ in range(3):
            one_prefill()
        pms = timed(one_prefill, 5)
        # a kernel whose bounded wait gave up returns early and would be timed as fast:
        # `run_step` reads the kernels' error word after every step, and the result must be finite
        ops.check_device_errors()
        assert bool(torch.isfinite(last_logits[0]).all()), "the timed prefill gave non-finite logits"
        fl = prefill_flops(raw, layers, PROMPT)
        out["prefill"] = {"value": round(PROMPT * 1000.0 / pms, 1), "tokens": PROMPT, "ms": round(pms, 3),
                          "frac": round(fl / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        pts = {}
        steps = min(K, 32)
        for b in ((1, 32, big) if args.shape == "32b" and big > 32 else (1, big)):
            _, m, _, _ = decode_run(b, steps, 4)
            pts["decode_b%d" % b] = round(b * 1000.0 / m, 1)
        for b in (1, args.batch, big):  # the same with half the context behind each request
            _, m, _, _ = decode_run(b, steps, 4, context=CONTEXT // 2)
            pts["decode_b%d_ctx%d" % (b, CONTEXT // 2)] = round(b * 1000.0 / m, 1)
        out["points"] = pts

    out["config"] = {"model": "Qwen3-%s shape" % args.shape.upper(), "layers": layers,
                     "layers_full": model["num_hidden_layers"],
                     "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                     "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                     "global_batch": args.batch, "seq_len": CONTEXT, "prompt_len": PROMPT, "page_size": PAGE,
                     "parallelism": "single GPU", "l2": "inputs larger than L2 (weights %.0f GB)" % (weight_bytes(raw, layers) / 1e9),
                     "peaks": pk["source"]}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
