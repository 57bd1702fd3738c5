#!/usr/bin/env python3
"""Measures decoding and prefill speed of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 4b|8b|32b] [--layers L]
                    [--batch B] [--context C] [--dtype bfloat16|float32] [--no-points]
    python bench.py --impl reference ...     (prints why it is unavailable)
    python bench.py --only decode|prefill|timeline ...   (one part, for profiling)
    python bench.py --only generate [--model 8b] ...      (unequal prompts, then 256 tokens each)

The default run has the layer sizes of Qwen3-4B (36 layers, hidden 2560, 32
heads, 8 KV heads, head size 128, feed-forward 9728, vocabulary 151936, tied
head) with random weights, a batch of 8 sequences and 2,048 tokens of context in
the cache.  A step is one decode step of the whole batch: the step function on
the last token of every sequence, and the choice of the next token on the device.

One JSON line is printed: ``value`` is decoded tokens per second, timed with CUDA
events around exactly K steps after W warm-up steps; ``e2e`` is the same
through the Python entry point (host tokens in, host tokens out, every step's
inputs copied from pinned host memory and its tokens read back); ``prefill`` is
one prompt of 2,048 tokens; ``roofline`` divides the bytes a decode step has to
read (every weight once and the cache of the live sequences) by its time;
``points`` holds decoding at batch 1 and 64.  Peaks come from
MEASURED_PEAKS.json beside this file when it exists.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_4B = dict(
    architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36,
    hidden_size=2560, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    intermediate_size=9728, vocab_size=151936, rope_theta=1e6, rms_norm_eps=1e-6,
    tie_word_embeddings=True, max_position_embeddings=8192)
FULL_LAYERS = QWEN3_4B["num_hidden_layers"]
# the other sizes of the same architecture, for --model (the default run is the 4B one)
MODELS = {
    "4b": QWEN3_4B,
    "8b": dict(QWEN3_4B, hidden_size=4096, intermediate_size=12288, tie_word_embeddings=False),
    "32b": dict(QWEN3_4B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64,
                intermediate_size=25600, tie_word_embeddings=False, max_position_embeddings=4096),
}

# used only when MEASURED_PEAKS.json is absent: an earlier measurement on this pool
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)

            def find(obj, key):
                if isinstance(obj, dict):
                    if key in obj and isinstance(obj[key], (int, float)):
                        return float(obj[key])
                    for v in obj.values():
                        r = find(v, key)
                        if r is not None:
                            return r
                return None
            hbm, tf = find(d, "hbm_gbs"), find(d, "bf16_tflops")
            if hbm and tf:
                return {"hbm_gbs": hbm, "bf16_tflops": tf, "source": "measured",
                        "bf16_tflops_sustained": find(d, "bf16_tflops_sustained")}
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS)


class Clocks:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) > 2 + i and r[2 + i].lower().startswith("active")
                          for r in self.rows)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": mx[0] if mx else None, "reasons": reasons,
                "samples": len(mhz)}


def build_engine(args, n_layers, max_tokens, max_seqs):
    import torch
    from janas_b200.config import config_from_dict
    from janas_b200.engine import DecoderModel, Engine
    from janas_b200.weights import random_tensors
    cfg = config_from_dict(dict(MODELS[args.model], num_hidden_layers=n_layers))
    dt = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    model = DecoderModel(cfg.to_model_spec(), dt, "cuda:0")
    with torch.cuda.device(0):
        model.load(random_tensors(model.tensors(), 0, dt, device="cuda:0"))
        eng = Engine(model, max_tokens=max_tokens, max_seqs=max_seqs)
        for g in eng.cache.groups:      # see fill()
            g.k.normal_()
            g.v.normal_()
    eng.config = cfg
    return eng


def fill(eng, batch, context, rng):
    """New sequences that hold ``context`` tokens each.  Their pages are taken from
    the pool as a prefill would take them; the keys and values in them are the
    random numbers the cache was filled with once (build_engine), which cost a
    decode step the same reads as computed ones.  Returns the slots and a random
    next token for each."""
    vocab = eng.model.spec.vocab_size
    slots = [eng.new_sequence() for _ in range(batch)]
    eng.cache.reserve(slots, [context] * batch)
    eng.cache.advance(slots, [context] * batch)
    return slots, rng.integers(0, vocab, size=batch).tolist()


def drive(eng, slots, tokens, n):
    """n decode steps of the same sequences, one step ahead where the engine allows
    it; every step's tokens are read on the host.  Returns the last ones."""
    if n <= 0:
        return tokens
    if not getattr(eng, "decodes_ahead", False):
        for _ in range(n):
            tokens = eng.decode(slots, tokens).tolist()
        return tokens
    cur = eng.decode_begin(slots, tokens)
    for i in range(n):
        nxt = eng.decode_begin(slots, None) if i + 1 < n else None
        tokens = eng.decode_end(cur).tolist()
        cur = nxt
    return tokens


def decode_device_timed(eng, slots, tokens, steps, warmup):
    """K decode steps of the whole batch (the engine's decode step: the step
    function's kernels and the choice of the next token, replayed from a CUDA
    graph), timed on the device.  The steps are driven as the generation loop
    drives them: each step's inputs are copied from pinned host memory, its chosen
    tokens are read back on the host every step, and where the engine can feed a
    step the tokens of the step before it, the next step is queued while this one
    runs."""
    import torch
    from janas_b200.csrc import ops

    run = lambda n, tokens: drive(eng, slots, tokens, n)
    tokens = run(warmup, tokens)
    torch.cuda.synchronize()
    l0 = ops.COUNTERS["launches"]
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    tokens = run(steps, tokens)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps, ops.COUNTERS["launches"] - l0, tokens


def decode_timeline(eng, slots, tokens, warmup):
    """Prints, for the last of three decode steps recorded with torch.profiler
    (CUPTI activity records; the step is the replayed CUDA graph), when each kernel
    started and ended and how long after the kernel before it ended.  Kernels start
    before their predecessors end (programmatic dependent launch), so a kernel's
    cost on the step's critical path is the last column, not its duration."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    tokens = drive(eng, slots, tokens, warmup + 2)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        tokens = drive(eng, slots, tokens, 3)
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    last = evs[-(len(evs) // 3):]
    t0 = last[0].time_range.start
    prev_end = t0
    print("start us   duration   end us   after the one before   kernel")
    for e in last:
        s, en = e.time_range.start - t0, e.time_range.end - t0
        print(f"{s:8.1f} {en - s:10.1f} {en:8.1f} {en - (prev_end - t0):10.1f}   {e.name[:64]}")
        prev_end = max(prev_end, e.time_range.end)
    print(f"step: {prev_end - t0:.1f} us")


def step_bytes(eng, batch, context):
    """Bytes a decode step has to read: every weight once, and the keys and
    values of the live sequences."""
    kv = 0
    for g in eng.cache.groups:
        per_token = 2 * len(g.entries) * g.spec.num_kv_heads * g.spec.head_dim * g.k.element_size()
        kv += per_token * batch * context
    return eng.model.weight_bytes() + kv


def prefill_flops(cfg, n_layers, tokens):
    """Multiply-adds times two of one prompt of ``tokens`` tokens: the matrix
    products of every layer, the causal attention, and the head for one row."""
    dm, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_token = 2 * (dm * (qd + 2 * kvd) + qd * dm + 3 * dm * ff)
    attn = 4 * qd * tokens * (tokens + 1) / 2
    return n_layers * (per_token * tokens + attn) + 2 * dm * cfg["vocab_size"]


def generate_workload(eng, args, rng, new_tokens=256):
    """A batch of unequal prompts through the entry point: host token lists in, host
    token lists out.  Prints one line per run; the first run pays for graph captures."""
    import janas_b200
    from janas_b200.engine.generate import GenOptions
    vocab = MODELS[args.model]["vocab_size"]
    llm = janas_b200.LLM(eng, janas_b200.LLMParams(n_ctx=eng.max_positions, dtype=args.dtype,
                                                  max_batch=args.batch))
    for run in range(3):
        lens = rng.integers(64, args.context + 1, size=args.batch).tolist()
        prompts = [rng.integers(0, vocab, size=n).tolist() for n in lens]
        t0 = time.perf_counter()
        outs, st = llm.generate_batch(prompts, new_tokens, GenOptions(eos=-1))
        wall = time.perf_counter() - t0
        print(f"generate run {run}: prompts {lens} ({sum(lens)} tokens) prefill "
              f"{1e3 * st.prefill_seconds:.1f} ms ({sum(lens) / st.prefill_seconds:,.0f} tokens/s), "
              f"{st.new_tokens} new tokens in {st.passes} steps, "
              f"{1e3 * st.decode_seconds / max(st.passes, 1):.3f} ms a step "
              f"({args.batch * st.passes / st.decode_seconds:,.0f} tokens/s), "
              f"whole call {wall:.3f} s", flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="4b", choices=sorted(MODELS),
                    help="layer sizes: Qwen3-4B (the default run), 8B or 32B")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-points", action="store_true", help="skip decoding at batch 1 and 64")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "timeline", "generate"],
                    help="run one part only and print its time (for profiling; no JSON line); "
                         "timeline: when each kernel of one replayed decode step ends; "
                         "generate: --batch prompts of lengths uniform in [64, --context], all in "
                         "one step, then 256 tokens each through the Python entry point")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "prabanta-dev/janas is a C program without setup.py or pyproject.toml "
                          "(pip: 'not installable'); it runs quantized .jns files only and has no "
                          "bfloat16 or sm_100 path"}))
        return 0
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    full_layers = MODELS[args.model]["num_hidden_layers"]
    if args.layers <= 0:
        args.layers = full_layers
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch
    import janas_b200
    from janas_b200.csrc import ops
    from janas_b200.engine.generate import GenOptions

    pk = peaks()
    rng = np.random.default_rng(0)
    total_steps = args.warmup + args.steps + 8
    room = (args.context + 2 * total_steps + 63) // 64 * 64
    big_batch = 64 if not args.no_points else args.batch
    if args.only == "generate":
        room, big_batch = (args.context + 256 + 127) // 64 * 64, args.batch
    eng = build_engine(args, args.layers, room * max(big_batch, args.batch), max(big_batch, args.batch))
    cfg = dict(MODELS[args.model])

    if args.only == "timeline":
        slots, toks = fill(eng, args.batch, args.context, rng)
        decode_timeline(eng, slots, toks, args.warmup)
        return 0

    if args.only == "generate":
        generate_workload(eng, args, rng)
        return 0

    if args.only == "decode":
        slots, toks = fill(eng, args.batch, args.context, rng)
        ms, launches, _ = decode_device_timed(eng, slots, toks, args.steps, args.warmup)
        print(f"decode batch {args.batch} context {args.context}: {ms:.4f} ms a step, "
              f"{launches // args.steps} kernels a step")
        return 0

    # ---- prefill of one prompt
    from janas_b200.engine import StepEntry
    T = args.prefill_tokens
    times = []
    for it in range(6):         # the first pays for allocations; the best of the rest counts
        s = eng.new_sequence()
        toks = rng.integers(0, cfg["vocab_size"], size=T).tolist()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.step([StepEntry(s, toks, [T - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        eng.free_sequence(s)
    pre_ms = min(times[1:])
    if args.only == "prefill":
        print(f"prefill {T} tokens: {pre_ms:.3f} ms")
        return 0
    flops = prefill_flops(cfg, args.layers, T)
    dense_peak = pk["bf16_tflops"] * 1e12 * (1.0 if args.dtype == "bfloat16" else 1.0)
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / dense_peak, 4)}
    if pk.get("bf16_tflops_sustained"):
        # against the library's throughput in a seconds-long loop under the power cap
        prefill["frac_sustained"] = round(
            flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    # ---- decoding, device-timed
    def decode_point(batch, steps, warmup):
        slots, toks = fill(eng, batch, args.context, rng)
        ms, launches, _ = decode_device_timed(eng, slots, toks, steps, warmup)
        for s in slots:
            eng.free_sequence(s)
        return ms, launches

    with Clocks() as clk:
        ms, launches = decode_point(args.batch, args.steps, args.warmup)
    clocks = clk.summary()
    value = args.batch / (ms / 1e3)
    mid_context = args.context + args.warmup + args.steps // 2
    nbytes = step_bytes(eng, args.batch, mid_context)
    achieved = nbytes / (ms / 1e3) / 1e9

    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _ = decode_point(b, max(8, args.steps // 4), 3)
            points[f"decode_b{b}"] = round(b / (pms / 1e3), 1)

    # ---- the same through the Python entry point: host tokens in and out
    llm = janas_b200.LLM(eng, janas_b200.LLMParams(n_ctx=eng.max_positions, dtype=args.dtype,
                                                  max_batch=args.batch))
    prompts = [rng.integers(0, cfg["vocab_size"], size=args.context).tolist()
               for _ in range(args.batch)]
    _, st = llm.generate_batch(prompts, args.steps + 1, GenOptions(eos=-1))
    e2e_value = args.batch * st.passes / st.decode_seconds
    e2e = {"value": round(e2e_value, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": st.h2d_bytes // max(st.passes, 1),
           "d2h_bytes_per_step": st.d2h_bytes // max(st.passes, 1)}

    out = {
        "metric": "decode tokens/s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.dtype == "bfloat16" else "fp32", "data": "synthetic",
        "config": {"model": f"Qwen3-{args.model.upper()} sizes, random weights",
                   "layers": args.layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "ffn": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "tied_head": bool(cfg["tie_word_embeddings"]),
                   "global_batch": args.batch,
                   "seq_len": args.context, "max_context": cfg["max_position_embeddings"],
                   "parallelism": "1 GPU", "l2": "inputs larger than L2 (weights read once a step)",
                   "peaks": pk["source"]},
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
