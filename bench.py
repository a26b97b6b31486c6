#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, at the Qwen3-8B layer sizes with
random weights and seeded synthetic token ids.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--shape 8b|4b|32b] [--serve] [--design zasesun|balivik|fikudra|nisotar]

A *step* is one decode step of a batch of 8 requests that each hold 1,024 tokens of context.
``value`` is decoded tokens per second over exactly K steps, timed on the device with CUDA events
after W warm-up steps, through the same captured step and host loop that generation uses.
``e2e`` is the same quantity through ``Engine.generate`` with host token lists in and out.
The line also carries a 2,048-token prefill, the decode step's HBM roofline, and decode at batch
1 and 64.  Weights (15 GB) are far larger than L2, so every step reads them from HBM.
``--shape`` runs the same at the 4B or 32B layer sizes (the 32B at 2,048 tokens of context and
batch 1, 8 and 32), and ``--serve`` times a mixed workload of 16 requests through the scheduler.
``--design zasesun`` measures the Zasesun decoder (latent attention, sandwich norms, dense and
routed feed-forwards) beside the Qwen3 decoder at equal widths, depths and head counts: prefill of
2,048 tokens and decode at batch 8, each with its own FLOP and byte counts against the peaks.
``--design balivik`` does the same for the Balivik decoder (differential attention, decay attention
and a channel-wise delta rule under four residual streams, dense and table-routed feed-forwards).
``--design fikudra`` measures the Fikudra decoder (gated linear attention, attention with a sink and
a gate per head that may read an earlier layer's pages, group-limited routed experts with a shared
expert, four residual streams, a hashed bigram embedding) beside the Balivik decoder at equal
widths, depths, head counts and expert sizes.
``--design nisotar`` measures the Nisotar decoder (a chunked attention whose values are its keys
beside a gated delta rule, attention and latent attention under sliding windows, all under layer
norms; a clamped dense and logit-routed feed-forwards) beside the Fikudra decoder at equal widths,
depths, head counts and expert sizes.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

QWEN3_8B = dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                head_dim=128, intermediate_size=12288, vocab_size=151936, max_position_embeddings=8192,
                rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False)
# the other layer shapes the baseline names, for --shape (the default run is the 8B shape)
SHAPES = {
    "8b": ("Qwen3-8B", QWEN3_8B, 1024),
    "4b": ("Qwen3-4B", dict(QWEN3_8B, hidden_size=2560, intermediate_size=9728, max_position_embeddings=32768,
                            tie_word_embeddings=True), 1024),
    "32b": ("Qwen3-32B", dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                              intermediate_size=25600), 2048),
}
CONTEXT = 1024
PREFILL_TOKENS = 2048


def load_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            data = json.load(f)
        peaks = {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                 "source": "measured"}
        if "bf16_tflops_sustained" in data:
            peaks["bf16_tflops_sustained"] = float(data["bf16_tflops_sustained"])
        return peaks
    except (OSError, KeyError, ValueError, TypeError):
        return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                max_clock = float(parts[1])
            except ValueError:
                continue
            for name, value in zip(names, parts[2:6]):
                if value.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "samples": len(clocks), "reasons": sorted(reasons)}


def seeded_tokens(vocab: int, n: int, seed: int):
    import numpy as np
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def fill_requests(executor, batch: int, context: int, vocab: int, tag: str):
    """Admits ``batch`` requests and brings each to ``context`` tokens; returns them with the
    last token fed still to come (so the next step is a decode step at that context)."""
    from mrun_b200.engine import StepEntry
    requests = [executor.admit((tag, i)) for i in range(batch)]
    per_step = max(1, PREFILL_TOKENS // context)
    for start in range(0, batch, per_step):
        group = requests[start:start + per_step]
        executor.step([StepEntry(r, seeded_tokens(vocab, context - 1, 1000 + start + i), [])
                       for i, r in enumerate(group)])
    return requests


def time_decode(executor, requests, vocab: int, steps: int, warmup: int, profiler_range: bool = False,
                repeats: int = 1):
    """Device times (ms, one per repeat) of ``steps`` decode steps the way generation runs them: a
    step is launched with the tokens of the step before it taken on the device, then that step's
    tokens are read back into pinned host memory.  Also the kernel launches of one repeat."""
    import torch
    from mrun_b200.engine import StepEntry
    n = len(requests)
    first = seeded_tokens(vocab, n, 7)
    pinned = [torch.empty(n, dtype=torch.int32, pin_memory=True) for _ in range(2)]
    state = {"event": None, "turn": 0}

    def one(first_step: bool):
        tokens = first if first_step else [0] * n
        sources = None if first_step else list(range(n))
        out = executor.decode_step([StepEntry(r, [t], [0]) for r, t in zip(requests, tokens)], None, sources)
        pinned[state["turn"]].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        if state["event"] is not None:
            state["event"].synchronize()
            pinned[state["turn"] ^ 1].tolist()          # the step before is read here
        state["event"], state["turn"] = event, state["turn"] ^ 1

    one(True)
    for _ in range(warmup - 1):
        one(False)
    times, launches = [], 0
    for repeat in range(repeats):
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = executor.launches.total
        if profiler_range and repeat == 0:   # lets a profiler started with --profile-from-start off see only this
            torch.cuda.profiler.start()
        begin.record()
        for _ in range(steps):
            one(False)
        end.record()
        torch.cuda.synchronize()
        if profiler_range and repeat == 0:
            torch.cuda.profiler.stop()
        times.append(begin.elapsed_time(end))
        launches = executor.launches.total - before
    return times, launches


def serve(args, config, model_name: str, full_layers: int, page_size: int, peaks: dict) -> int:
    """The baseline's mixed workload: 16 requests whose prompts hold 64 to 16,384 seeded tokens,
    prompts cut into portions under a budget of 2,048 tokens a step beside the decoding of the
    others, 256 tokens decoded for each.  Everything goes through ``Engine.generate``; the times
    are the host's clock around that one call (it ends when the last token is on the host)."""
    import numpy as np
    import torch
    from mrun_b200 import Engine
    from mrun_b200.kernels import lib as kernel_lib

    requests, decode_tokens = 16, 256
    lengths = np.random.default_rng(11).integers(64, 16384 + 1, size=requests).tolist()
    prompts = [seeded_tokens(config.vocab_size, n, 200 + i) for i, n in enumerate(lengths)]
    capacity = sum(-(-(n + decode_tokens) // page_size) for n in lengths) + 64
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_size=page_size, num_pages=capacity,
                                max_requests=requests, max_batch_tokens=PREFILL_TOKENS)
    engine.generate([p[:300] for p in prompts[:4]], max_tokens=8, ignore_eos=True)       # warm-up: shapes, graphs
    engine.generate(prompts[:2], max_tokens=4, ignore_eos=True)
    sampler = ClockSampler()
    sampler.start()
    steps_before, launches = engine.stats.steps, engine.executor.launches.total
    torch.cuda.synchronize()
    begin = time.perf_counter()
    generations = engine.generate(prompts, max_tokens=decode_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - begin
    clocks = sampler.stop()
    decoded = sum(len(g.tokens) for g in generations)
    last_first = max(g.first_token_time for g in generations)
    finished = max(g.finished_time for g in generations)
    tail = sum(sum(1 for t in g.token_times if t > last_first) for g in generations)
    steps = engine.stats.steps - steps_before
    line = {
        "metric": f"tokens/s, prompts and decoded, {requests} mixed requests ({model_name} bf16)",
        "value": round((sum(lengths) + decoded) / seconds, 1), "unit": "tok/s", "n_gpus": 1,
        "steps": steps, "warmup": 2, "ms_per_step": round(seconds * 1e3 / max(1, steps), 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (seeded uniform token ids, N(0,0.02) weights)", "impl": "ours",
        "config": {"model": f"{model_name} shape", "layers": config.num_hidden_layers, "layers_of_config": full_layers,
                   "hidden": config.hidden_size, "heads": config.num_attention_heads,
                   "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
                   "intermediate": config.intermediate_size, "vocab": config.vocab_size,
                   "tied": config.tie_word_embeddings, "global_batch": requests, "prompt_tokens": sum(lengths),
                   "longest_prompt": max(lengths), "decoded_per_request": decode_tokens,
                   "max_batch_tokens": PREFILL_TOKENS, "page_size": page_size, "parallelism": "single GPU"},
        "seconds": round(seconds, 3), "decoded": decoded,
        "time_to_first_token_s": {"median": round(statistics.median(g.time_to_first_token_s for g in generations), 3),
                                  "max": round(max(g.time_to_first_token_s for g in generations), 3)},
        "decode_tail": {"value": round(tail / max(finished - last_first, 1e-9), 1), "unit": "tok/s",
                        "note": "all 16 decoding side by side, after the last prompt ended"},
        "preemptions": sum(g.preemptions for g in generations),
        "gpu_launches": engine.executor.launches.total - launches, "clocks": clocks, "peaks": peaks,
        "kernel_entry_calls": kernel_lib.call_count(),
    }
    print(json.dumps(line))
    return 0


# Layer sizes for --design: (name, Zasesun sizes, the Qwen3 sizes of equal width, depth and heads).
# The cache row of the latent attention (kv_rank + rot_dim) is 128, 256 and 576 features: the
# first two are head sizes the tensor-core attention kernels are built for, the third is not.
def _zasesun_sizes(width, heads, dim, rot_dim, vdim, q_rank, kv_rank, ff, experts, top, expert_ff, shared_ff,
                   layers, vocab):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
             "scale": (dim + rot_dim) ** -0.5,
             "rot": {"base": 10000.0, "dims": rot_dim,
                     "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff},
           "shared": {"ff": shared_ff}}
    return {"architecture": "Zasesun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "residual_mult": 0.7,
            "logit_softcap": 30.0,
            "layers": [{"type": "latent_attention", "mixer": mixer, "mlp": dense if i % 2 == 0 else moe}
                       for i in range(layers)]}


DESIGN_SIZES = {
    "row128": (_zasesun_sizes(2048, 16, 64, 32, 64, 768, 96, 8192, 8, 2, 2048, 2048, 8, 32768),
               dict(QWEN3_8B, num_hidden_layers=8, hidden_size=2048, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=128, intermediate_size=8192, vocab_size=32768, tie_word_embeddings=True)),
    "row256": (_zasesun_sizes(4096, 16, 128, 64, 128, 1536, 192, 12288, 8, 2, 3072, 3072, 8, 32768),
               dict(QWEN3_8B, num_hidden_layers=8, hidden_size=4096, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=128, intermediate_size=12288, vocab_size=32768, tie_word_embeddings=True)),
    "row576": (_zasesun_sizes(2048, 16, 128, 64, 128, 1536, 512, 8192, 8, 2, 2048, 2048, 4, 32768),
               dict(QWEN3_8B, num_hidden_layers=4, hidden_size=2048, num_attention_heads=16, num_key_value_heads=2,
                    head_dim=128, intermediate_size=8192, vocab_size=32768, tie_word_embeddings=True)),
}


def zasesun_counts(cfg: dict, tokens: int):
    """(FLOPs of a prompt of ``tokens`` tokens as the design states them, bytes of one token's
    cache rows over all layers) of a Zasesun configuration: products count two FLOPs a weight and
    token, a routed layer its chosen and its shared experts only, attention the scores over the
    cache row and the weighted sum over the latent for every visible key."""
    h, flops, row_bytes = cfg["width"], 0.0, 0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        params = ((m["q_rank"] + m["kv_rank"] + m["rot_dim"]) * h + m["heads"] * (m["dim"] + m["rot_dim"]) * m["q_rank"]
                  + m["heads"] * (m["dim"] + m["vdim"]) * m["kv_rank"] + h * m["heads"] * m["vdim"])
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            params += 3 * h * mlp["ff"]
        elif mlp:
            params += 2 * h * (mlp["router"]["top"] * mlp["expert"]["ff"] + mlp["shared"]["ff"]) + h * mlp["router"]["experts"]
        flops += 2.0 * tokens * params + 2.0 * (tokens * tokens / 2.0) * m["heads"] * (2 * m["kv_rank"] + m["rot_dim"])
        row_bytes += 2 * (-(-(m["kv_rank"] + m["rot_dim"]) // 16) * 16)
    return flops + 2.0 * cfg["vocab"] * h, row_bytes


# Layer sizes for --design balivik: (Balivik sizes, the Qwen3 sizes of equal width, depth, head count
# and dense feed-forward size).  Eight layers in the order decay attention, delta rule, two
# differential attentions, twice (the second block's last layer is a decay attention); key
# sizes of 64 and 128 (the differential attention's values are two chunks of its key size, so its
# maps go through the tensor-core attention kernels), four residual streams, an input convolution
# of four taps, dense and table-routed feed-forwards alternating (8 experts, 2 chosen).
def _balivik_sizes(width, heads, kv_heads, att_dim, dim, ff, experts, top, expert_ff, rank, layers, vocab):
    att = {"heads": heads, "kv_heads": kv_heads, "dim": att_dim, "vdim": 2 * att_dim, "scale": att_dim ** -0.5, "diff": 0.3,
           "rot": {"base": 10000.0, "dims": att_dim}}
    lin = {"heads": heads, "dim": dim, "vdim": dim, "decay": [1.0 - 2.0 ** -(2 + 6 * i / max(1, heads - 1)) for i in range(heads)]}
    delta = {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": 4, "decay_rank": rank, "gate_rank": rank}
    kinds = [("lightning", lin), ("channel_delta", delta), ("attention", att), ("attention", att)]
    dense = {"kind": "dense", "ff": ff}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff, "limit": 7.0}}
    return {"architecture": "Balivik", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "streams": 4,
            "canon": {"taps": 4}, "logit_scale": 0.5,
            "layers": [{"type": kinds[i % 4][0], "mixer": kinds[i % 4][1], "mlp": dense if i % 2 == 0 else moe}
                       for i in range(layers)]}


BALIVIK_SIZES = {
    "w2048": (_balivik_sizes(2048, 16, 4, 64, 128, 8192, 8, 2, 2048, 128, 8, 32768),
              dict(QWEN3_8B, num_hidden_layers=8, hidden_size=2048, num_attention_heads=16, num_key_value_heads=4,
                   head_dim=128, intermediate_size=8192, vocab_size=32768, tie_word_embeddings=False)),
    "w4096": (_balivik_sizes(4096, 32, 8, 128, 128, 12288, 8, 2, 3072, 256, 8, 32768),
              dict(QWEN3_8B, num_hidden_layers=8, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                   head_dim=128, intermediate_size=12288, vocab_size=32768, tie_word_embeddings=False)),
}


def balivik_counts(cfg: dict, tokens: int):
    """(FLOPs of a prompt of ``tokens`` tokens as the design states them, bytes of one token's
    cache rows over all layers, bytes of one request's recurrent states over all layers) of a
    Balivik configuration: products count two FLOPs a weight and token (a table-routed layer its
    chosen experts only), a differential attention both maps' scores and weighted sums for every
    visible key, a recurrent mixer the update and the read-out of its state for every token."""
    h, flops, row_bytes, state_bytes = cfg["width"], 0.0, 0, 0
    for layer in cfg["layers"]:
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            params = h * (2 * m["heads"] * m["dim"] + 2 * m["kv_heads"] * m["dim"] + m["kv_heads"] * m["vdim"]
                          + m["heads"] * m["vdim"])
            flops += 2.0 * (tokens * tokens / 2.0) * m["heads"] * 2 * (m["dim"] + m["vdim"])
            row_bytes += 2 * m["kv_heads"] * (2 * m["dim"] + m["vdim"])
        elif kind == "lightning":
            params = h * (2 * m["heads"] * m["dim"] + 3 * m["heads"] * m["vdim"])
            flops += 2.0 * tokens * m["heads"] * 2 * m["dim"] * m["vdim"]
            state_bytes += 4 * m["heads"] * m["dim"] * m["vdim"]
        else:
            inner, keyed = m["heads"] * m["vdim"], m["heads"] * m["dim"]
            params = h * (2 * m["kv_heads"] * m["dim"] + 2 * inner + m["heads"] + m["decay_rank"] + m["gate_rank"]) \
                + keyed * m["decay_rank"] + inner * m["gate_rank"]
            flops += 2.0 * tokens * m["heads"] * 4 * m["dim"] * m["vdim"]
            state_bytes += 4 * m["heads"] * m["dim"] * m["vdim"]
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            params += 3 * h * mlp["ff"]
        elif mlp:
            params += 3 * h * mlp["router"]["top"] * mlp["expert"]["ff"]
        flops += 2.0 * tokens * params
    return flops + 2.0 * cfg["vocab"] * h, row_bytes, state_bytes


# Layer sizes for --design fikudra: (Fikudra sizes, the Balivik sizes of equal width, depth, head
# counts and expert sizes, from the table above).  Eight layers: an attention, three gated linear
# attentions, an attention that reads the first one's pages, three more linear attentions; keys and
# values of one size (the tensor-core attention kernels), half of the features rotated; every layer
# a mixture of 8 experts in 4 groups of which 2 stay, 2 chosen, with a shared expert; four streams.
def _fikudra_sizes(width, heads, kv_heads, att_dim, dim, experts, top, expert_ff, shared_ff, rank, layers, vocab):
    att = {"heads": heads, "kv_heads": kv_heads, "dim": att_dim, "vdim": att_dim, "scale": att_dim ** -0.5,
           "rot": {"base": 10000.0, "dims": att_dim // 2, "scaling": {"factor": 4.0}}}
    gla = {"heads": heads, "dim": dim, "vdim": dim, "tau": 8.0, "rank": rank}
    moe = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": 1.5, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": expert_ff}, "shared": {"ff": shared_ff}}

    def entry(i):
        if i % 4:
            return {"type": "gla", "mixer": gla, "mlp": moe}
        return {"type": "attention", "mixer": dict(att, kv_from=0) if i else att, "mlp": moe}
    return {"architecture": "Fikudra", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "streams": 4,
            "embedding": {"scale": 8.0, "bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 7}},
            "layers": [entry(i) for i in range(layers)]}


FIKUDRA_SIZES = {
    "w2048": (_fikudra_sizes(2048, 16, 4, 128, 128, 8, 2, 2048, 2048, 128, 8, 32768), BALIVIK_SIZES["w2048"][0]),
    "w4096": (_fikudra_sizes(4096, 32, 8, 128, 128, 8, 2, 3072, 3072, 256, 8, 32768), BALIVIK_SIZES["w4096"][0]),
}


def fikudra_counts(cfg: dict, tokens: int):
    """(FLOPs of a prompt of ``tokens`` tokens as the design states them, bytes of one token's
    cache rows over all layers, bytes of one request's recurrent states over all layers) of a
    Fikudra configuration: products count two FLOPs a weight and token (a routed layer its chosen
    experts and the shared one), an attention the scores and weighted sums of every visible key, a
    linear attention the update and the read-out of its state for every token."""
    h, flops, row_bytes, state_bytes = cfg["width"], 0.0, 0, 0
    for layer in cfg["layers"]:
        m = layer["mixer"]
        if layer["type"] == "attention":
            own = m.get("kv_from") is None
            params = h * (m["heads"] * (m["dim"] + m["vdim"] + 1) + (m["kv_heads"] * (m["dim"] + m["vdim"]) if own else 0))
            flops += 2.0 * (tokens * tokens / 2.0) * m["heads"] * (m["dim"] + m["vdim"])
            row_bytes += 2 * m["kv_heads"] * (m["dim"] + m["vdim"])       # read by every layer that uses these pages
        else:
            keyed, inner = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            params = h * (2 * keyed + 3 * inner + m["rank"]) + keyed * m["rank"]
            flops += 2.0 * tokens * m["heads"] * 2 * m["dim"] * m["vdim"]
            state_bytes += 4 * m["heads"] * m["dim"] * m["vdim"]
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            params += 3 * h * mlp["ff"]
        elif mlp:
            shared = (mlp.get("shared") or {}).get("ff", 0)
            params += h * (mlp["router"]["experts"] + 1) + 3 * h * (mlp["router"]["top"] * mlp["expert"]["ff"] + shared)
        flops += 2.0 * tokens * params
    return flops + 2.0 * cfg["vocab"] * h, row_bytes, state_bytes


# Layer sizes for --design nisotar: (Nisotar sizes, the Fikudra sizes of equal width, depth, head
# counts and expert sizes, from the table above).  Eight layers: parallel (a chunked attention whose
# values are its keys beside a gated delta rule), attention under a sliding window, latent attention
# under a sliding window, and again; keys and values of one size (the tensor-core attention
# kernels), half of the features rotated, the latent row 256 features wide; the first layer's
# feed-forward dense with clamped branches, the others mixtures of 8 experts of which 2 are chosen.
def _nisotar_sizes(width, heads, kv_heads, att_dim, dim, experts, top, expert_ff, dense_ff, rank, layers, vocab):
    att = {"heads": heads, "kv_heads": kv_heads, "dim": att_dim, "vdim": att_dim, "scale": att_dim ** -0.5,
           "mask": {"size": 512},
           "rot": {"base": 10000.0, "dims": att_dim // 2, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    left = {"heads": heads, "kv_heads": kv_heads, "dim": att_dim, "vdim": att_dim, "scale": att_dim ** -0.5,
            "mask": {"size": 256}, "rot": {"base": 100000.0, "dims": att_dim // 2}}
    right = {"heads": heads, "kv_heads": heads, "dim": dim, "vdim": dim, "conv": 4, "decay_rank": rank, "gate_rank": rank}
    # 16 heads over the one latent row at every width: more take the tiled kernel, whose tile list is
    # made on the host, and a model with it decodes uncaptured
    lat = {"heads": min(heads, 16), "dim": att_dim, "rot_dim": att_dim // 2, "vdim": att_dim, "kv_rank": 256 - att_dim // 2,
           "scale": (att_dim + att_dim // 2) ** -0.5, "mask": {"size": 384}, "rot": {"base": 10000.0, "dims": att_dim // 2}}
    kinds = [("parallel", {"left": left, "right": right}), ("attention", att), ("latent_attention", lat)]
    moe = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": expert_ff}}
    dense = {"kind": "dense", "ff": dense_ff, "limit": 7.0}
    return {"architecture": "Nisotar", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
            "layers": [{"type": kinds[i % 3][0], "mixer": kinds[i % 3][1], "mlp": moe if i else dense} for i in range(layers)]}


NISOTAR_SIZES = {
    "w2048": (_nisotar_sizes(2048, 16, 4, 128, 128, 8, 2, 2048, 8192, 128, 8, 32768), FIKUDRA_SIZES["w2048"][0]),
    "w4096": (_nisotar_sizes(4096, 32, 8, 128, 128, 8, 2, 3072, 12288, 256, 8, 32768), FIKUDRA_SIZES["w4096"][0]),
}


def nisotar_counts(cfg: dict, tokens: int, context: int):
    """(FLOPs of a prompt of ``tokens`` tokens as the design states them, bytes of cache rows a
    decoded token at ``context`` reads over all layers divided by ``context``, bytes of one
    request's recurrent states over all layers) of a Nisotar configuration: products count two
    FLOPs a weight and token (a routed layer its chosen experts), an attention the scores and
    weighted sums of every key its mask lets it see, the delta rule the decay, the correction, the
    update and the read-out of its state for every token."""
    h, flops, row_bytes, state_bytes = cfg["width"], 0.0, 0.0, 0

    def seen(size, chunked):        # (token, key) pairs of the prompt that the mask lets through
        if chunked:
            whole, rest = divmod(tokens, size)
            return whole * size * (size + 1) / 2.0 + rest * (rest + 1) / 2.0
        short = min(tokens, size)
        return short * (short + 1) / 2.0 + max(0, tokens - size) * size

    def softmax_attention(m, chunked, keys):
        nonlocal flops, row_bytes
        groups = m.get("kv_heads") or m["heads"]
        flops += 2.0 * seen(m["mask"]["size"], chunked) * m["heads"] * (m["dim"] + m["vdim"])
        held = min(context, m["mask"]["size"]) if not chunked else (m["mask"]["size"] + 1) / 2.0
        row_bytes += 2 * groups * (m["dim"] + m["vdim"]) * held / context
        return h * (m["heads"] * (m["dim"] + m["vdim"]) + groups * (m["dim"] + (0 if keys else m["vdim"])))
    for layer in cfg["layers"]:
        m, kind = layer["mixer"], layer["type"]
        if kind == "attention":
            params = softmax_attention(m, False, False)
        elif kind == "latent_attention":
            params = h * (m["heads"] * (m["dim"] + m["rot_dim"] + m["vdim"]) + m["kv_rank"] + m["rot_dim"]) \
                + m["kv_rank"] * m["heads"] * (m["dim"] + m["vdim"])
            flops += 2.0 * seen(m["mask"]["size"], False) * m["heads"] * (m["dim"] + m["rot_dim"] + m["vdim"])
            row_bytes += 2 * (m["kv_rank"] + m["rot_dim"]) * min(context, m["mask"]["size"]) / context
        else:
            params = softmax_attention(m["left"], True, True)
            r = m["right"]
            inner, keyed = r["heads"] * r["vdim"], r["heads"] * r["dim"]
            params += h * (2 * r["kv_heads"] * r["dim"] + 2 * inner + r["heads"] + r["decay_rank"] + r["gate_rank"]) \
                + keyed * r["decay_rank"] + inner * r["gate_rank"]
            flops += 2.0 * tokens * r["heads"] * 4 * r["dim"] * r["vdim"]
            state_bytes += 4 * r["heads"] * r["dim"] * r["vdim"]
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            params += 3 * h * mlp["ff"]
        elif mlp:
            params += h * mlp["router"]["experts"] + 3 * h * mlp["router"]["top"] * mlp["expert"]["ff"]
        flops += 2.0 * tokens * params
    return flops + 2.0 * cfg["vocab"] * h, row_bytes, state_bytes


def compare_designs(args, peaks: dict) -> int:
    """Prefill of 2,048 tokens and decode at batch 8 with 1,024-token contexts, the named design
    beside Qwen3 (Fikudra: beside Balivik; Nisotar: beside Fikudra) at equal sizes, each through
    the same ``Executor.step`` and captured decode step."""
    import torch
    from mrun_b200 import Engine
    from mrun_b200.config import Qwen3Config, ZasesunConfig
    from mrun_b200.config.balivik import BalivikConfig
    from mrun_b200.config.fikudra import FikudraConfig
    from mrun_b200.config.nisotar import NisotarConfig
    from mrun_b200.engine import StepEntry
    context, batch = 1024, 8
    out = {}
    sampler = ClockSampler()
    sampler.start()
    size_sets = {"zasesun": DESIGN_SIZES, "balivik": BALIVIK_SIZES, "fikudra": FIKUDRA_SIZES,
                 "nisotar": NISOTAR_SIZES}[args.design]
    beside = {"fikudra": "balivik", "nisotar": "fikudra"}.get(args.design, "qwen3")
    for name in (args.sizes.split(",") if args.sizes else sorted(size_sets)):
        z_sizes, q_sizes = size_sets[name]
        row = {}
        for design in (args.design, beside):
            state_bytes = 0
            if design == "nisotar":
                config = NisotarConfig.from_dict(z_sizes)
                vocab, h = z_sizes["vocab"], z_sizes["width"]
                flops, kv_bytes, state_bytes = nisotar_counts(z_sizes, PREFILL_TOKENS, context)
            elif design == "fikudra" and args.design == "nisotar":
                config = FikudraConfig.from_dict(q_sizes)
                vocab, h = q_sizes["vocab"], q_sizes["width"]
                flops, kv_bytes, state_bytes = fikudra_counts(q_sizes, PREFILL_TOKENS)
            elif design == "fikudra":
                config = FikudraConfig.from_dict(z_sizes)
                vocab, h = z_sizes["vocab"], z_sizes["width"]
                flops, kv_bytes, state_bytes = fikudra_counts(z_sizes, PREFILL_TOKENS)
            elif design == "balivik" and args.design == "fikudra":
                config = BalivikConfig.from_dict(q_sizes)
                vocab, h = q_sizes["vocab"], q_sizes["width"]
                flops, kv_bytes, state_bytes = balivik_counts(q_sizes, PREFILL_TOKENS)
            elif design == "zasesun":
                config = ZasesunConfig.from_dict(z_sizes)
                vocab, h = z_sizes["vocab"], z_sizes["width"]
                flops, kv_bytes = zasesun_counts(z_sizes, PREFILL_TOKENS)
            elif design == "balivik":
                config = BalivikConfig.from_dict(z_sizes)
                vocab, h = z_sizes["vocab"], z_sizes["width"]
                flops, kv_bytes, state_bytes = balivik_counts(z_sizes, PREFILL_TOKENS)
            else:
                config = Qwen3Config(**dict(q_sizes, max_position_embeddings=8192))
                vocab, h, d = config.vocab_size, config.hidden_size, config.head_dim
                params = config.num_hidden_layers * ((2 * config.num_attention_heads + 2 * config.num_key_value_heads) * d * h
                                                     + 3 * h * config.intermediate_size)
                flops = 2.0 * PREFILL_TOKENS * params + 2.0 * vocab * h \
                    + config.num_hidden_layers * 2.0 * PREFILL_TOKENS ** 2 * config.num_attention_heads * d
                kv_bytes = config.kv_bytes_per_token(2)
            slack = args.steps * 2 + args.warmup + 64
            capacity = batch * (context + slack) + PREFILL_TOKENS + 256
            engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_size=args.page_size,
                                        num_pages=-(-capacity // args.page_size), max_requests=16,
                                        max_batch_tokens=PREFILL_TOKENS)
            executor = engine.executor
            prompt, times = seeded_tokens(vocab, PREFILL_TOKENS, 3), []
            for i in range(5):
                request = executor.admit(("prefill", i))
                torch.cuda.synchronize()
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                executor.step([StepEntry(request, prompt, [PREFILL_TOKENS - 1])])
                end.record()
                torch.cuda.synchronize()
                executor.release(request)
                if i >= 2:
                    times.append(begin.elapsed_time(end))
            prefill_ms = statistics.median(times)
            requests = fill_requests(executor, batch, context, vocab, "decode")
            decode_times, launches = time_decode(executor, requests, vocab, args.steps, args.warmup, repeats=2)
            ms = statistics.median(decode_times) / args.steps
            weight_bytes = executor.model.weight_bytes()
            # recurrent states are read and written once a step and request
            step_bytes = weight_bytes + batch * (context + args.warmup + args.steps) * kv_bytes + 2 * batch * state_bytes
            row[design] = {
                "layers": len(executor.model.order), "weights_gb": round(weight_bytes / 1e9, 2),
                "prefill_tok_s": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "prefill_ms": round(prefill_ms, 3),
                "prefill_frac": round(flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4),
                "decode_b8_tok_s": round(batch / (ms * 1e-3), 1), "decode_ms_per_step": round(ms, 4),
                "decode_frac": round(step_bytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], 4),
                "decode_launches": launches // max(1, args.steps), "cache_bytes_per_token": kv_bytes}
            for r in requests:
                executor.release(r)
            del engine, executor, requests
            torch.cuda.empty_cache()
        out[name] = row
    print(json.dumps({"metric": f"prefill and decode tok/s, {args.design.capitalize()} beside {beside.capitalize()} at equal sizes (bf16)", "unit": "tok/s",
                      "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "dtype": "bf16",
                      "data": "synthetic (seeded uniform token ids, N(0,0.02) weights)",
                      "config": {"prefill_tokens": PREFILL_TOKENS, "decode_batch": batch, "context": context,
                                 "page_size": args.page_size, "of": peaks["source"]},
                      "sizes": out, "clocks": sampler.stop(), "peaks": peaks}))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--layers", type=int, default=None,
                        help="run fewer layers than the configuration has (both numbers are reported)")
    parser.add_argument("--skip-points", action="store_true", help="only the batch-8 decode and the prefill")
    parser.add_argument("--batches", default=None,
                        help="decode batch sizes to run, comma separated (for profiling one point)")
    parser.add_argument("--skip-prefill", action="store_true")
    parser.add_argument("--shape", choices=sorted(SHAPES), default="8b",
                        help="layer sizes: the baseline's 8B shape, or its 4B and 32B shapes")
    parser.add_argument("--serve", action="store_true",
                        help="instead of the decode step: 16 requests with prompts of 64 to 16,384 tokens and "
                             "256 decoded tokens each through Engine.generate, prompts cut at 2,048 tokens")
    parser.add_argument("--context", type=int, default=None,
                        help="tokens each request holds when decoding is timed (the default is the baseline's)")
    parser.add_argument("--prefill-depth", type=int, default=0,
                        help="tokens already in the cache before the timed portion of 2,048 (0: a fresh prompt)")
    parser.add_argument("--skip-e2e", action="store_true")
    parser.add_argument("--page-size", type=int, default=16, help="keys a cache page holds")
    parser.add_argument("--repeats", type=int, default=5,
                        help="how many times the K timed steps are run (the line carries the median, the "
                             "fastest and the slowest)")
    parser.add_argument("--profiler-range", nargs="?", const="decode", default=None, choices=["decode", "prefill"],
                        help="bracket the timed decode steps (or the last timed prefill) with "
                             "cudaProfilerStart/Stop, for a profiler started with --profile-from-start off")
    parser.add_argument("--design", choices=["zasesun", "balivik", "fikudra", "nisotar"], default=None,
                        help="instead of the default workload: the named design beside Qwen3 (fikudra: beside Balivik; nisotar: beside Fikudra) at equal sizes "
                             "(prefill of 2,048 tokens, decode at batch 8)")
    parser.add_argument("--sizes", default=None, help="with --design: which of its size sets to run, comma separated")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "hupe1980/mrun is a Rust workspace over an Apple Metal array library (nuvec): "
                          "no cargo/rustc here, no pip-installable package, no Metal device"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path, --gpus {args.gpus} is not run")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import torch
    from mrun_b200 import Engine
    from mrun_b200.config import Qwen3Config
    from mrun_b200.kernels import lib as kernel_lib

    peaks = load_peaks()
    if args.design:
        return compare_designs(args, peaks)
    model_name, shape_sizes, shape_context = SHAPES[args.shape]
    sizes = dict(shape_sizes)
    if args.context is None:
        args.context = shape_context
    full_layers = sizes["num_hidden_layers"]
    if args.layers is not None:
        sizes["num_hidden_layers"] = args.layers
    if args.serve:
        sizes["max_position_embeddings"] = max(sizes["max_position_embeddings"], 16384 + 256 + 64)
    config = Qwen3Config(**sizes)
    page_size = args.page_size
    if args.serve:
        return serve(args, config, model_name, full_layers, page_size, peaks)
    batches = [8] if args.skip_points else [8, 1, 32 if args.shape == "32b" else 64]
    if args.batches:
        batches = [int(b) for b in args.batches.split(",")]
    args.repeats = max(1, args.repeats)
    slack = args.repeats * args.steps + args.warmup + 64
    context = args.context
    # the requests of every batch size are alive together, so that the clocks can be sampled over all of them
    capacity = max(sum(batches) * (context + slack), 8 * (context + 2 * slack)) + args.prefill_depth + PREFILL_TOKENS + 4 * 64
    sizes["max_position_embeddings"] = max(sizes["max_position_embeddings"], context + slack + 64,
                                           args.prefill_depth + PREFILL_TOKENS + 64)
    config = Qwen3Config(**sizes)
    engine = Engine.from_config(config, seed=0, dtype="bfloat16", page_size=page_size,
                                num_pages=-(-capacity // page_size), max_requests=max(64, sum(batches)),
                                max_batch_tokens=max(PREFILL_TOKENS, args.prefill_depth))
    executor = engine.executor
    vocab = config.vocab_size
    kv_bytes = config.kv_bytes_per_token(2)
    # every weight the step uses, once; of an embedding table that is not also the head only B rows
    weight_bytes = executor.model.weight_bytes()
    if not config.tie_word_embeddings:
        weight_bytes -= vocab * config.hidden_size * 2

    # ---------------------------------------------------------------- prefill, 2,048 tokens
    from mrun_b200.engine import StepEntry
    prompt = seeded_tokens(vocab, PREFILL_TOKENS, 3)
    times = []
    for i in range(0 if args.skip_prefill else 2 + 3):
        request = executor.admit(("prefill", i))
        for start in range(0, args.prefill_depth, 4 * PREFILL_TOKENS):        # the depth, untimed
            executor.step([StepEntry(request, seeded_tokens(vocab, min(4 * PREFILL_TOKENS, args.prefill_depth - start), 5), [])])
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ranged = args.profiler_range == "prefill" and i == 4
        if ranged:
            torch.cuda.profiler.start()
        begin.record()
        executor.step([StepEntry(request, prompt, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        if ranged:
            torch.cuda.profiler.stop()
        executor.release(request)
        if i >= 2:
            times.append(begin.elapsed_time(end))
    prefill_ms = statistics.median(times) if times else float("nan")
    h, d = config.hidden_size, config.head_dim
    linear_params = config.num_hidden_layers * ((config.num_attention_heads + 2 * config.num_key_value_heads) * d * h
                                                + config.num_attention_heads * d * h
                                                + 3 * h * config.intermediate_size)
    prefill_flops = 2.0 * PREFILL_TOKENS * linear_params + 2.0 * vocab * h \
        + config.num_hidden_layers * (2.0 * PREFILL_TOKENS ** 2 + 4.0 * PREFILL_TOKENS * args.prefill_depth) \
        * config.num_attention_heads * d
    prefill = {"value": round(PREFILL_TOKENS / prefill_ms * 1e3, 1), "tokens": PREFILL_TOKENS,
               "ms": round(prefill_ms, 3), **({"depth": args.prefill_depth} if args.prefill_depth else {}),
               "frac": round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops"] * 1e12), 4)}
    if "bf16_tflops_sustained" in peaks:
        prefill["frac_sustained"] = round(prefill_flops / (prefill_ms * 1e-3) / (peaks["bf16_tflops_sustained"] * 1e12), 4)
    if not times:                        # --skip-prefill: nothing was measured, and NaN is no JSON
        prefill = {"skipped": True, "tokens": PREFILL_TOKENS}

    # ---------------------------------------------------------------- decode at batch 8 / 1 / 64
    results = {}
    launches = 0
    all_requests = {batch: fill_requests(executor, batch, context, vocab, f"decode{batch}") for batch in batches}
    sampler = ClockSampler()             # clocks and throttle reasons over every timed decode region
    sampler.start()
    for batch in batches:
        times, n_launch = time_decode(executor, all_requests[batch], vocab, args.steps, args.warmup,
                                      args.profiler_range == "decode", args.repeats)
        if batch == batches[0]:
            launches = n_launch
        results[batch] = times
    clocks = sampler.stop()
    for requests in all_requests.values():
        for r in requests:
            executor.release(r)
    main_batch = batches[0]
    context_mid = context + args.warmup + args.repeats * args.steps / 2.0

    def point(batch):
        """tok/s and the HBM roofline of a batch size: every weight once and the live requests' cache."""
        ms = statistics.median(results[batch]) / args.steps
        step_bytes = weight_bytes + batch * context_mid * kv_bytes + batch * h * 2
        achieved = step_bytes / (ms * 1e-3) / 1e9
        return ms, {"value": round(batch / (ms * 1e-3), 1), "ms_per_step": round(ms, 4),
                    "ms_per_step_min": round(min(results[batch]) / args.steps, 4),
                    "ms_per_step_max": round(max(results[batch]) / args.steps, 4),
                    "bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / peaks["hbm_gbs"], 4), "of": peaks["source"]}

    ms_per_step, main_point = point(main_batch)
    value = main_point["value"]
    roofline = {k: main_point[k] for k in ("bound", "achieved", "peak", "unit", "frac", "of")}
    repeats = {"n": args.repeats, "ms_per_step_min": main_point["ms_per_step_min"],
               "ms_per_step_max": main_point["ms_per_step_max"], "value_is": "median over the repeats"}
    others = {f"decode_b{b}": point(b)[1] for b in batches if b != main_batch}
    points = {name: p["value"] for name, p in others.items()}
    points_roofline = {name: {k: p[k] for k in ("ms_per_step", "ms_per_step_min", "ms_per_step_max", "achieved", "frac")}
                       for name, p in others.items()}

    # ---------------------------------------------------------------- end to end, Engine.generate
    if args.skip_e2e:
        line = {"metric": f"decode tok/s at batch {main_batch}", "value": round(value, 1), "ms_per_step": round(ms_per_step, 4),
                "roofline": roofline, "points": points, "points_roofline": points_roofline, "repeats": repeats,
                "gpu_launches": launches, "prefill": prefill}
        print(json.dumps(line))
        return 0
    # Token lists in, token lists out, through Engine.generate.  The token budget of this engine
    # takes the eight prompts in one step, so all eight decode side by side for every step of
    # the window that is timed: from the first token of each (read back on the host) to the last.
    from mrun_b200.engine.engine import Engine as EngineClass
    e2e_engine = EngineClass(executor, max_batch_tokens=main_batch * context)
    out_tokens = args.steps + 1
    prompts = [seeded_tokens(vocab, context, 50 + i) for i in range(main_batch)]
    e2e_engine.generate(prompts, max_tokens=4, ignore_eos=True)         # warm the prompt step's shapes
    uploaded = executor.staging.bytes_uploaded
    steps_before = e2e_engine.stats.steps
    d2h_before = e2e_engine.stats.d2h_bytes
    torch.cuda.synchronize()
    generations = e2e_engine.generate(prompts, max_tokens=out_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    short = [len(g.tokens) for g in generations if len(g.tokens) != out_tokens or g.finish_reason != "length"]
    if short:
        raise RuntimeError(f"end-to-end run: generations ended early ({short} of {out_tokens} tokens)")
    last_first = max(g.first_token_time for g in generations)
    finished = max(g.finished_time for g in generations)
    decoded = sum(sum(1 for t in g.token_times if t > last_first) for g in generations)
    e2e_value = decoded / max(finished - last_first, 1e-9)
    n_steps = max(1, e2e_engine.stats.steps - steps_before)
    engine = e2e_engine
    e2e = {"value": round(e2e_value, 1), "unit": "tok/s",
           "h2d_bytes_per_step": round((executor.staging.bytes_uploaded - uploaded) / n_steps, 1),
           "d2h_bytes_per_step": round((engine.stats.d2h_bytes - d2h_before) / n_steps, 1)}

    line = {
        "metric": f"decode tok/s at batch {main_batch} ({model_name} bf16, {context:,}-token prompts)",
        "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded uniform token ids, N(0,0.02) weights)",
        "impl": "ours",
        "config": {
            "model": f"{model_name} shape", "layers": config.num_hidden_layers, "layers_of_config": full_layers,
            "hidden": h, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": d, "intermediate": config.intermediate_size, "vocab": vocab,
            "rope_theta": config.rope_theta, "rms_norm_eps": config.rms_norm_eps,
            "tied": config.tie_word_embeddings, "global_batch": main_batch, "seq_len": context,
            "max_context": config.max_position_embeddings, "page_size": page_size,
            "parallelism": "single GPU", "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.0f} GB of weights per step)",
        },
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        "prefill": prefill, "roofline": roofline, "points": points, "points_roofline": points_roofline,
        "repeats": repeats, "peaks": peaks, "kernel_entry_calls": kernel_lib.call_count(),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
