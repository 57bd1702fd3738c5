#!/usr/bin/env python3
"""Measures decoding and prefill speed of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--model 4b|8b|32b] [--layers L]
                    [--batch B] [--context C] [--dtype bfloat16|float32] [--no-points]
                    [--all-configs]
    python bench.py --impl reference ...     (the reference's own bench program, on the CPU)
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
``points`` holds decoding at batch 1 and 64 and the 32-bit path's decode and
prefill speeds.  The cache that the timed steps read was written by the engine's
own prefill of random prompts.  ``checked`` says that, after the timed regions,
the kernels' error words were clear and the last decode step replayed from its CUDA
graph chose the tokens that the same step chooses when its kernels are launched one
by one.  Peaks come from MEASURED_PEAKS.json beside this file when it exists.
``--all-configs`` adds the other workloads (8B sizes: eight unequal prompts and
256 decode steps; 32B sizes: prefill and decoding) as further points; each runs in
a process of its own.
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

# used only when MEASURED_PEAKS.json is absent: figures of an earlier measurement
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


def model_cfg(args):
    """The chosen model's config.json; the context it allows grows with --context."""
    cfg = dict(MODELS[args.model])
    need = (args.context + 1024 + 1023) // 1024 * 1024
    cfg["max_position_embeddings"] = max(cfg["max_position_embeddings"], need)
    return cfg


def build_engine(args, n_layers, max_tokens, max_seqs, dtype=None):
    """A model of the chosen sizes with weights made at random on the device, and a
    cache of ``max_tokens``."""
    from janas_b200.engine import Engine
    cfg = dict(model_cfg(args), num_hidden_layers=n_layers)
    return Engine.open_random(cfg, seed=0, dtype=dtype or args.dtype, max_tokens=max_tokens,
                              max_seqs=max_seqs, n_ctx=cfg["max_position_embeddings"])


def fill(eng, batch, context, rng):
    """New sequences that hold ``context`` tokens each, computed by the engine's own
    prefill of random prompts (one prompt a step, so that the step's temporaries
    stay small).  Returns the slots and a random next token for each."""
    from janas_b200.engine import StepEntry
    vocab = eng.vocab_size
    slots = []
    for _ in range(batch):
        s = eng.new_sequence()
        eng.step([StepEntry(s, rng.integers(0, vocab, size=context).tolist(), [])])
        slots.append(s)
    return slots, rng.integers(0, vocab, size=batch).tolist()


def drive(eng, slots, tokens, n):
    """n decode steps of the same sequences, one step ahead where the engine allows
    it; every step's tokens are read on the host.  Returns the last ones."""
    if n <= 0:
        return tokens
    if not eng.decodes_ahead:
        for _ in range(n):
            tokens = eng.decode(slots, tokens).tolist()
        return tokens
    cur = eng.decode_begin(slots, tokens)
    for i in range(n):
        nxt = eng.decode_begin(slots, None) if i + 1 < n else None
        tokens = eng.decode_end(cur).tolist()
        cur = nxt
    return tokens


def launches():
    from janas_b200 import lib
    return lib.call("llm.launches")["launches"]


class DeviceTimer:
    """CUDA events on the engine's own stream."""

    def __init__(self, eng):
        import torch
        self.torch = torch
        self.stream = torch.cuda.ExternalStream(eng.stream)
        self.a = torch.cuda.Event(enable_timing=True)
        self.b = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.stream.synchronize()
        self.a.record(self.stream)
        return self

    def __exit__(self, *exc):
        self.b.record(self.stream)
        self.stream.synchronize()
        self.ms = self.a.elapsed_time(self.b)


def decode_device_timed(eng, slots, tokens, steps, warmup):
    """K decode steps of the whole batch (the engine's decode step: the step
    function's kernels and the choice of the next token, replayed from a CUDA
    graph), timed on the device.  The steps are driven as the generation loop
    drives them: each step's inputs are copied from pinned host memory, its chosen
    tokens are read back on the host every step, and where the engine can feed a
    step the tokens of the step before it, the next step is queued while this one
    runs."""
    tokens = drive(eng, slots, tokens, warmup)
    l0 = launches()
    with DeviceTimer(eng) as t:
        tokens = drive(eng, slots, tokens, steps)
    return t.ms / steps, launches() - l0, tokens


def check_last_step(eng, slots, tokens):
    """One more decode step replayed from its graph, then the same step again with
    its kernels launched one by one (the sequences are taken back by the one token
    in between): both must choose the same tokens.  And the kernels' error words
    must be clear.  Raises when not."""
    a = eng.decode(slots, tokens).tolist()
    for s in slots:
        if not eng.truncate_sequence(s, eng.length(s) - 1):
            raise RuntimeError("the cache cannot go back one token")
    graphs = eng.use_graphs
    eng.use_graphs = False
    try:
        b = eng.decode(slots, tokens).tolist()
    finally:
        eng.use_graphs = graphs
    eng.check()
    if a != b:
        raise RuntimeError(f"the replayed decode step chose {a}, the launched one {b}")
    return True


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
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
           and "memcpy" not in e.name.lower()]
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
    info = eng.info()
    esz = 2 if info["dtype"] == "bfloat16" else 4
    kv = 0
    for g in info["cache"]["groups"]:
        per_token = 2 * len(g["entries"]) * g["num_kv_heads"] * g["head_dim"] * esz
        kv += per_token * batch * context
    return info["weight_bytes"] + kv


def prefill_flops(cfg, n_layers, tokens):
    """Multiply-adds times two of one prompt of ``tokens`` tokens: the matrix
    products of every layer, the causal attention, and the head for one row."""
    dm, ff = cfg["hidden_size"], cfg["intermediate_size"]
    qd = cfg["num_attention_heads"] * cfg["head_dim"]
    kvd = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_token = 2 * (dm * (qd + 2 * kvd) + qd * dm + 3 * dm * ff)
    attn = 4 * qd * tokens * (tokens + 1) / 2
    return n_layers * (per_token * tokens + attn) + 2 * dm * cfg["vocab_size"]


def prefill_timed(eng, rng, T, rounds=6):
    """One prompt of T tokens in one step, the logits of its last token wanted;
    the best of ``rounds`` after a first that pays for allocations."""
    from janas_b200.engine import StepEntry
    times = []
    for _ in range(rounds):
        s = eng.new_sequence()
        toks = rng.integers(0, eng.vocab_size, size=T).tolist()
        with DeviceTimer(eng) as t:
            eng.step([StepEntry(s, toks, [T - 1])])
        times.append(t.ms)
        eng.free_sequence(s)
    return min(times[1:])


def prefill_timeline(eng, rng, T):
    """Prints, for one prompt of T tokens recorded with torch.profiler, how much of
    the step each kernel accounts for: the sum, over its launches, of the time from
    the end of the kernel before it to its own end (kernels overlap their
    predecessors, so durations would count the overlap twice)."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    from janas_b200.engine import StepEntry
    prefill_timed(eng, rng, T, rounds=3)
    s = eng.new_sequence()
    toks = rng.integers(0, eng.vocab_size, size=T).tolist()
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.step([StepEntry(s, toks, [T - 1])])
        torch.cuda.synchronize()
    eng.free_sequence(s)
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA
           and "memcpy" not in e.name.lower()]
    evs.sort(key=lambda e: e.time_range.start)
    t0 = evs[0].time_range.start
    prev_end = t0
    per = {}
    for e in evs:
        gain = max(0.0, e.time_range.end - prev_end)
        name = e.name.split("(")[0][:60]
        c = per.setdefault(name, [0, 0.0, 0.0])
        c[0] += 1
        c[1] += gain
        c[2] += e.time_range.end - e.time_range.start
        prev_end = max(prev_end, e.time_range.end)
    total = prev_end - t0
    print(f"prefill of {T} tokens: {total / 1e3:.3f} ms from the first kernel's start to the last one's end")
    print("launches   on the critical path (us)   share   sum of durations (us)   kernel")
    for name, (cnt, gain, dur) in sorted(per.items(), key=lambda kv: -kv[1][1]):
        print(f"{cnt:8d} {gain:16.1f} {gain / total:18.1%} {dur:16.1f}   {name}")


def generate_workload(eng, args, rng, new_tokens=256, runs=3):
    """A batch of unequal prompts through the entry point: host token lists in, host
    token lists out.  Prints one line per run (the first pays for graph captures);
    returns the last run's prefill and decode speeds."""
    import janas_b200
    from janas_b200.engine.generate import GenOptions
    vocab = eng.vocab_size
    llm = janas_b200.LLM(eng, janas_b200.LLMParams(n_ctx=eng.max_positions, dtype=args.dtype,
                                                  max_batch=args.batch))
    out = {}
    for run in range(runs):
        lens = rng.integers(64, args.context + 1, size=args.batch).tolist()
        prompts = [rng.integers(0, vocab, size=n).tolist() for n in lens]
        t0 = time.perf_counter()
        outs, st = llm.generate_batch(prompts, new_tokens, GenOptions(eos=-1))
        wall = time.perf_counter() - t0
        out = {"prefill_tok_s": sum(lens) / st.prefill_seconds,
               "decode_tok_s": args.batch * st.passes / st.decode_seconds,
               "ms_per_step": 1e3 * st.decode_seconds / max(st.passes, 1),
               "prompt_tokens": sum(lens)}
        print(f"generate run {run}: prompts {lens} ({sum(lens)} tokens) prefill "
              f"{1e3 * st.prefill_seconds:.1f} ms ({out['prefill_tok_s']:,.0f} tokens/s), "
              f"{st.new_tokens} new tokens in {st.passes} steps, "
              f"{out['ms_per_step']:.3f} ms a step ({out['decode_tok_s']:,.0f} tokens/s), "
              f"whole call {wall:.3f} s", file=sys.stderr, flush=True)
    return out


def other_config(model, extra):
    """Runs this program for another model size in a process of its own (its
    weights and cache are given back when it ends); returns its JSON line."""
    cmd = [sys.executable, os.path.abspath(__file__), "--model", model, "--no-points"] + extra
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    for line in reversed(r.stdout.strip().splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise RuntimeError(f"{' '.join(cmd)} printed no result:\n{r.stdout[-500:]}\n{r.stderr[-1500:]}")


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
    ap.add_argument("--no-points", action="store_true",
                    help="skip decoding at batch 1 and 64 and the 32-bit points")
    ap.add_argument("--all-configs", action="store_true",
                    help="also the 8B workload (unequal prompts, 256 steps) and the 32B points")
    ap.add_argument("--only", default="", choices=["", "decode", "prefill", "timeline", "prefill-timeline", "generate"],
                    help="run one part only and print its time (for profiling; no JSON line "
                         "but for generate); prefill-timeline: each kernel's share of one prefill "
                         "step; timeline: when each kernel of one replayed decode "
                         "step ends; generate: --batch prompts of lengths uniform in [64, "
                         "--context], all in one step, then 256 tokens each through the Python "
                         "entry point")
    args = ap.parse_args()

    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    full_layers = MODELS[args.model]["num_hidden_layers"]
    if args.layers <= 0:
        args.layers = full_layers
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import janas_b200
    from janas_b200.engine.generate import GenOptions

    pk = peaks()
    rng = np.random.default_rng(0)
    total_steps = args.warmup + args.steps + 10
    room = (args.context + 2 * total_steps + 63) // 64 * 64
    big_batch = 64 if not args.no_points else args.batch
    if args.only == "generate":
        room, big_batch = (args.context + 256 + 127) // 64 * 64, args.batch
    eng = build_engine(args, args.layers, room * max(big_batch, args.batch), max(big_batch, args.batch))
    cfg = model_cfg(args)

    if args.only == "timeline":
        slots, toks = fill(eng, args.batch, args.context, rng)
        decode_timeline(eng, slots, toks, args.warmup)
        return 0

    if args.only == "generate":
        r = generate_workload(eng, args, rng)
        eng.check()
        print(json.dumps({"model": args.model, "layers": args.layers, "batch": args.batch,
                          **{k: round(v, 3) for k, v in r.items()}}))
        return 0

    if args.only == "decode":
        slots, toks = fill(eng, args.batch, args.context, rng)
        ms, n_launch, _ = decode_device_timed(eng, slots, toks, args.steps, args.warmup)
        print(f"decode batch {args.batch} context {args.context}: {ms:.4f} ms a step, "
              f"{n_launch // args.steps} kernels a step")
        return 0

    # ---- prefill of one prompt
    T = args.prefill_tokens
    if args.only == "prefill-timeline":
        prefill_timeline(eng, rng, T)
        return 0
    pre_ms = prefill_timed(eng, rng, T)
    if args.only == "prefill":
        print(f"prefill {T} tokens: {pre_ms:.3f} ms")
        return 0
    flops = prefill_flops(cfg, args.layers, T)
    prefill = {"value": round(T / (pre_ms / 1e3), 1), "tokens": T, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    if pk.get("bf16_tflops_sustained"):
        # against the library's throughput in a seconds-long loop under the power cap
        prefill["frac_sustained"] = round(
            flops / (pre_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    # ---- decoding, device-timed
    checked = True

    def decode_point(e, batch, steps, warmup):
        nonlocal checked
        slots, toks = fill(e, batch, args.context, rng)
        ms, n_launch, toks = decode_device_timed(e, slots, toks, steps, warmup)
        checked = check_last_step(e, slots, toks) and checked
        for s in slots:
            e.free_sequence(s)
        return ms, n_launch

    with Clocks() as clk:
        ms, n_launch = decode_point(eng, args.batch, args.steps, args.warmup)
    clocks = clk.summary()
    value = args.batch / (ms / 1e3)
    mid_context = args.context + args.warmup + args.steps // 2
    nbytes = step_bytes(eng, args.batch, mid_context)
    achieved = nbytes / (ms / 1e3) / 1e9

    points = {}
    if not args.no_points:
        for b in (1, 64):
            pms, _ = decode_point(eng, b, max(8, args.steps // 4), 3)
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
    eng.check()
    eng.close()

    # ---- the whole model in true 32-bit: decoding at the same batch, and the prefill
    if not args.no_points and args.dtype == "bfloat16":
        e32 = build_engine(args, args.layers, room * args.batch, args.batch, dtype="float32")
        p32 = prefill_timed(e32, rng, T, rounds=3)
        d32, _ = decode_point(e32, args.batch, max(8, args.steps // 4), 3)
        points["fp32_decode_b%d" % args.batch] = round(args.batch / (d32 / 1e3), 1)
        points["fp32_prefill_tok_s"] = round(T / (p32 / 1e3), 1)
        points["fp32_prefill_tflops"] = round(flops / (p32 / 1e3) / 1e12, 2)
        e32.close()

    if args.all_configs:
        g8 = other_config("8b", ["--only", "generate", "--batch", "8", "--context", "2048"])
        points["8b_generate_prefill_tok_s"] = round(g8["prefill_tok_s"], 1)
        points["8b_generate_decode_tok_s"] = round(g8["decode_tok_s"], 1)
        big = other_config("32b", ["--steps", "16"])
        points["32b_decode_b8"] = big["value"]
        points["32b_roofline_frac"] = big["roofline"]["frac"]
        points["32b_prefill_tok_s"] = big["prefill"]["value"]

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
        "e2e": e2e, "gpu_launches": n_launch, "clocks": clocks, "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points, "checked": bool(checked),
    }
    print(json.dumps(out))
    return 0


def write_q8_gguf(path, cfg, seed=0):
    """A random model of ``cfg``'s sizes in the reference's eight-bit weight type
    (Q8_0: blocks of 32 signed bytes and a half-precision scale), as a GGUF version 3
    file (src/llm/gguf.c:6-9; the keys its converter wants: tools/gguf2jns.c:377-399;
    tensor names: src/llm/model_load.c:403-503,999-1007).  Written tensor by tensor."""
    import struct
    import numpy as np
    L, dm, ff, V = (cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"],
                    cfg["vocab_size"])
    hd = cfg["head_dim"]
    qd, kvd = cfg["num_attention_heads"] * hd, cfg["num_key_value_heads"] * hd
    names = [("token_embd.weight", (V, dm)), ("output_norm.weight", (dm,))]
    for l in range(L):
        g = f"blk.{l}."
        names += [(g + "attn_norm.weight", (dm,)), (g + "attn_q.weight", (qd, dm)),
                  (g + "attn_k.weight", (kvd, dm)), (g + "attn_v.weight", (kvd, dm)),
                  (g + "attn_output.weight", (dm, qd)), (g + "attn_q_norm.weight", (hd,)),
                  (g + "attn_k_norm.weight", (hd,)), (g + "ffn_norm.weight", (dm,)),
                  (g + "ffn_gate.weight", (ff, dm)), (g + "ffn_up.weight", (ff, dm)),
                  (g + "ffn_down.weight", (dm, ff))]
    if not cfg["tie_word_embeddings"]:
        names.append(("output.weight", (V, dm)))
    string = lambda t: struct.pack("<Q", len(t.encode())) + t.encode()
    u32 = lambda k, v: string(k) + struct.pack("<II", 4, v)
    f32 = lambda k, v: string(k) + struct.pack("<If", 6, v)
    text = lambda k, v: string(k) + struct.pack("<I", 8) + string(v)
    kvs = [text("general.architecture", "qwen3"), text("general.name", "random qwen3"),
           u32("general.alignment", 32), u32("qwen3.block_count", L),
           u32("qwen3.context_length", cfg["max_position_embeddings"]),
           u32("qwen3.embedding_length", dm), u32("qwen3.feed_forward_length", ff),
           u32("qwen3.attention.head_count", cfg["num_attention_heads"]),
           u32("qwen3.attention.head_count_kv", cfg["num_key_value_heads"]),
           u32("qwen3.attention.key_length", hd), u32("qwen3.attention.value_length", hd),
           f32("qwen3.attention.layer_norm_rms_epsilon", cfg["rms_norm_eps"]),
           f32("qwen3.rope.freq_base", cfg["rope_theta"])]
    size = lambda shape: (int(np.prod(shape)) // 32 * 34) if len(shape) == 2 else shape[0] * 4
    infos, at = b"", 0
    for name, shape in names:
        at = (at + 31) // 32 * 32
        dims = list(reversed(shape))                 # the row's length first
        infos += string(name) + struct.pack("<I", len(dims))
        infos += b"".join(struct.pack("<Q", d) for d in dims)
        infos += struct.pack("<IQ", 8 if len(shape) == 2 else 0, at)
        at += size(shape)
    head = b"GGUF" + struct.pack("<IQQ", 3, len(names), len(kvs)) + b"".join(kvs) + infos
    head += b"\0" * ((len(head) + 31) // 32 * 32 - len(head))
    rng = np.random.default_rng(seed)
    with open(path, "wb") as f:
        f.write(head)
        at = 0
        for name, shape in names:
            pad = (at + 31) // 32 * 32 - at
            f.write(b"\0" * pad)
            at += pad
            if len(shape) == 1:
                raw = (1.0 + 0.1 * rng.standard_normal(shape[0])).astype("<f4").tobytes()
            else:
                # weights of about N(0, 0.02): uniform bytes (standard deviation 73) times a scale
                rows, blocks = shape[0], shape[1] // 32
                raw = np.empty((rows, blocks, 34), dtype=np.uint8)
                raw[..., :2] = np.frombuffer(np.float16(0.02 / 73.0).tobytes(), dtype=np.uint8)
                raw[..., 2:] = rng.integers(-127, 128, size=(rows, blocks, 32), dtype=np.int8).view(np.uint8)
                raw = raw.tobytes()
            f.write(raw)
            at += len(raw)


def reference_arm(args):
    """The reference's own generation program on this machine's CPU.

    prabanta-dev/janas is a C program for quantized models on CPUs (and, through a
    graphics API, on GPUs); pip has nothing of it to install, and it has no bfloat16 or
    sm_100 path.  What can be run of it here, unmodified, is what its own build
    (./build.sh release) makes: ``gguf2jns`` and ``llm_gen`` (tests/llm_gen.c, which
    calls janas_llm_generate on given token ids and reports prefill and decoding
    speed), kept under baseline/_ref/bin.  This arm writes a random model of the same
    layer sizes in the reference's eight-bit weight type, converts it with the
    reference's converter and lets llm_gen read a prompt of --prefill-tokens tokens and
    write --steps tokens, one sequence, on all CPU cores.  It is not the same
    configuration (said in the line it prints): eight-bit weights, activations and
    cache, a CPU, batch 1."""
    import re
    import shutil
    import tempfile
    import numpy as np

    def unavailable(why):
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    bin_dir = os.path.join(ROOT, "baseline", "_ref", "bin")
    tools = {t: os.path.join(bin_dir, t) for t in ("gguf2jns", "llm_gen")}
    if not all(os.path.isfile(p) and os.access(p, os.X_OK) for p in tools.values()):
        return unavailable(
            "prabanta-dev/janas is a C program without setup.py or pyproject.toml (pip: 'not "
            "installable'); its own build's gguf2jns and llm_gen are not under baseline/_ref/bin")
    cfg = dict(MODELS[args.model])
    if args.layers > 0:
        cfg["num_hidden_layers"] = args.layers
    uid = os.getuid() if hasattr(os, "getuid") else 0
    work = os.path.join(tempfile.gettempdir(), f"janas_b200_reference_{uid}")
    os.makedirs(work, exist_ok=True)
    tag = f"qwen3_{args.model}_{cfg['num_hidden_layers']}l_q8_0"
    jns = os.path.join(work, tag + ".jns")
    env = dict(os.environ, HOME=work)          # the reference writes tuning notes below HOME
    try:
        if not os.path.isfile(jns):
            # the GGUF file and the converted copy lie side by side for a moment
            need = 2.3 * 1.07 * (
                cfg["vocab_size"] * cfg["hidden_size"] * (1 if cfg["tie_word_embeddings"] else 2) +
                cfg["num_hidden_layers"] * cfg["hidden_size"] * (
                    (cfg["num_attention_heads"] * 2 + cfg["num_key_value_heads"] * 2) * cfg["head_dim"] +
                    3 * cfg["intermediate_size"]))
            if shutil.disk_usage(work).free < need:
                return unavailable(f"{work} has no room for a {need / 1e9:.0f} GB model file and its copy")
            gguf = os.path.join(work, tag + ".gguf")
            write_q8_gguf(gguf, cfg)
            r = subprocess.run([tools["gguf2jns"], gguf, jns + ".tmp"], env=env, capture_output=True,
                               text=True, timeout=1200)
            os.remove(gguf)
            if r.returncode != 0:
                return unavailable("the reference's gguf2jns refused the random model: "
                                   + (r.stderr or r.stdout).strip()[-300:])
            os.replace(jns + ".tmp", jns)
        T, gen = args.prefill_tokens, max(args.steps, 1)
        if T > 8191:
            return unavailable("the reference's llm_gen reads prompts of up to 8192 tokens")
        rng = np.random.default_rng(0)
        prompt = os.path.join(work, "prompt.int32")
        rng.integers(0, cfg["vocab_size"], size=T).astype("<i4").tofile(prompt)
        cmd = [tools["llm_gen"], jns, prompt, str(T), str(gen), "1", "threads=100000",
               f"ctx={min(cfg['max_position_embeddings'], T + gen + 64)}"]
        t0 = time.perf_counter()
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500)
        wall = time.perf_counter() - t0
    except (OSError, subprocess.SubprocessError, MemoryError) as e:
        return unavailable(f"the reference's tools could not be run here: {type(e).__name__}: {e}"[:400])
    m = re.search(r"prefill (\d+) tokens ([\d.]+) s \(([\d.]+) token/s\); decode (\d+) tokens "
                  r"([\d.]+) s \(([\d.]+) token/s\), (\d+) passes", r.stdout)
    if r.returncode != 0 or not m:
        return unavailable("the reference's llm_gen did not report speeds: "
                           + ((r.stderr or "") + (r.stdout or "")).strip()[-300:])
    n_new, dec_s = int(m.group(4)), float(m.group(5))
    out = {
        "impl": "reference", "metric": "decode tokens/s", "value": round(n_new / dec_s, 2),
        "unit": "tokens/s", "n_gpus": 1, "steps": n_new, "warmup": args.warmup,
        "ms_per_step": round(1e3 * dec_s / max(int(m.group(7)), 1), 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "q8_0 weights, int8 activations and cache",
        "data": "synthetic", "same_config": False,
        "differences": "the reference's own CPU code (it has no bfloat16 and no sm_100 path): "
                       "eight-bit weights, activations and cache; one sequence (batch 1); all CPU "
                       "cores of this machine; its test program llm_gen (janas_llm_generate), the "
                       "measured run after one warm-up run",
        "config": {"model": f"Qwen3-{args.model.upper()} sizes, random Q8_0 weights",
                   "layers": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "ffn": cfg["intermediate_size"],
                   "vocab": cfg["vocab_size"], "global_batch": 1, "seq_len": T,
                   "parallelism": f"{os.cpu_count()} CPU threads"},
        "prefill": {"value": float(m.group(3)), "tokens": int(m.group(1)),
                    "ms": round(1e3 * float(m.group(2)), 1)},
        "wall_seconds": round(wall, 1),
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
