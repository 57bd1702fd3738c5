"""The command line, with the reference's option names where it has them.

    janas-b200 <model-dir> [--prompt-tokens FILE | --tokens "1 2 3" | --prompt-len N]
               [--ctx N] [--temp T] [--top-k K] [--top-p P] [--min-p P] [--seed S]
               [--max N] [--eos ID] [--stop ID ...] [--batch B] [--dtype bfloat16|float32]
               [--stats]
    janas-b200 <model-dir> --chat [the sampling options, --ctx, --max]     (turns on standard input)
    janas-b200 <model-dir> --bench [--prompt N] [--gen N] [--rounds N] [--ctx N] [--batch B]
    janas-b200 --random-weights <config.json> --out <model-dir> [--seed S] [--store bfloat16|float32]

``--ctx --temp --top-k --top-p --min-p --seed --max`` mean what they mean for
janas-chat (src/chat/main.c:1346-1427); ``--prompt --gen --rounds`` what they
mean for janas-bench (src/bench/main.c:10-30: tokens of prompt, tokens
generated, rounds, prefill timed apart from decoding: :140-169).  There is no
tokenizer: prompts are token ids (as tests/llm_gen.c:10-15 takes them from an
int32 file) and the output is token ids, one request a line.  ``--chat`` is a
conversation as janas-chat holds one (src/chat/main.c: every turn goes on from
what the model has computed): each line of standard input is a turn's token
ids, the reply's ids come back as a line (it ends after a stop token, at
``--max`` tokens or when the context is full), until the input ends.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from typing import List


def _read_prompts(args, vocab: int) -> List[List[int]]:
    import numpy as np
    if args.prompt_tokens:
        if args.prompt_tokens.endswith(".int32"):
            return [np.fromfile(args.prompt_tokens, dtype="<i4").tolist()]
        with open(args.prompt_tokens, "r", encoding="utf-8") as f:
            rows = [[int(t) for t in line.replace(",", " ").split()] for line in f]
        return [r for r in rows if r]
    if args.tokens:
        return [[int(t) for t in args.tokens.replace(",", " ").split()]]
    rng = np.random.default_rng(args.seed)
    return [rng.integers(0, vocab, size=args.prompt_len).tolist() for _ in range(args.batch)]


def _chat(llm, options, args) -> int:
    """One session; a turn a line.  A line that cannot be taken (no ids, an id
    outside the vocabulary, more than the context holds) is answered on standard
    error and the conversation goes on."""
    from . import api
    stops = options.stop_set()
    s = llm.session(options)
    try:
        for line in sys.stdin:
            try:
                turn = [int(t) for t in line.replace(",", " ").split()]
                if not turn:
                    continue
                s.append(turn)
            except ValueError as e:
                print(f"janas-b200: {e}", file=sys.stderr)
                continue
            reply: List[int] = []
            while len(reply) < args.max:
                try:
                    status, tok = s.next()
                except (api.LLMError, ValueError, RuntimeError) as e:
                    print(f"janas-b200: {e}", file=sys.stderr)
                    return 2
                if status != 0:
                    print("janas-b200: the context is full", file=sys.stderr)
                    break
                reply.append(tok)
                if tok in stops:
                    break
            print(" ".join(str(t) for t in reply), flush=True)
        if args.stats:
            st = s.stats
            print(f"{s.length} tokens in the conversation; prompt {st.prompt_tokens} tokens in "
                  f"{st.prefill_seconds:.3f} s; {st.new_tokens} new tokens in "
                  f"{st.decode_seconds:.3f} s", file=sys.stderr)
    finally:
        s.close()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="janas-b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    ap.add_argument("--prompt-tokens", help="token ids: a text file, one request a line, "
                                            "or a raw .int32 file")
    ap.add_argument("--tokens", help="token ids of one prompt, separated by blanks")
    ap.add_argument("--prompt-len", type=int, default=16, help="random prompts of this length")
    ap.add_argument("--ctx", type=int, default=4096, help="context, in tokens")
    ap.add_argument("--temp", type=float, default=0.0, help="temperature; 0: greedy")
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--max", type=int, default=32, help="most new tokens of a reply")
    ap.add_argument("--eos", type=int, default=None, help="stop token (default: config.json's)")
    ap.add_argument("--stop", type=int, nargs="*", default=[], help="more stop tokens (up to 4)")
    ap.add_argument("--batch", type=int, default=1, help="sequences that run together")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--stats", action="store_true")
    ap.add_argument("--chat", action="store_true", help="turns of token ids on standard input, "
                                                        "one a line; replies as lines of ids")
    ap.add_argument("--bench", action="store_true", help="measure prefill and decoding speed")
    ap.add_argument("--prompt", type=int, default=256, help="bench: tokens of prompt")
    ap.add_argument("--gen", type=int, default=64, help="bench: tokens generated")
    ap.add_argument("--rounds", type=int, default=3, help="bench: rounds")
    ap.add_argument("--random-weights", metavar="CONFIG", help="write a model folder with "
                                                               "random weights for this config.json")
    ap.add_argument("--out", help="with --random-weights: the folder to write")
    ap.add_argument("--store", default="bfloat16", choices=["bfloat16", "float32"])
    args = ap.parse_args(argv)

    if args.random_weights:
        import torch
        from .config import ConfigError, config_from_dict
        from .weights import write_random_model
        if not args.out:
            ap.error("--random-weights needs --out")
        with open(args.random_weights, "r", encoding="utf-8") as f:
            cfg = config_from_dict(json.load(f))
        write_random_model(args.out, cfg, args.seed,
                           torch.bfloat16 if args.store == "bfloat16" else torch.float32)
        print(f"wrote {args.out}")
        return 0
    if not args.model:
        ap.error("a model folder is needed")

    from . import api
    from .engine.generate import GenOptions
    need = args.ctx if not args.bench else max(args.ctx, args.prompt + args.gen)
    params = api.LLMParams(n_ctx=need, dtype=args.dtype, max_batch=args.batch,
                           max_tokens=(need + 63) // 64 * 64 * args.batch)
    try:
        llm = api.open(args.model, params)
    except api.LLMError as e:
        print(f"janas-b200: {e}", file=sys.stderr)
        return 2
    eos_ids = tuple(getattr(getattr(llm.engine, "config", None), "eos_token_ids", ()) or ())
    eos = args.eos if args.eos is not None else (eos_ids[0] if eos_ids else -1)
    stops = list(args.stop) + [e for e in eos_ids[1:] if args.eos is None]

    if args.bench:
        import numpy as np
        rng = np.random.default_rng(args.seed)
        best_p, best_d = 0.0, 0.0
        for r in range(args.rounds + 1):      # the first round warms up
            prompts = [rng.integers(0, llm.n_vocab, size=args.prompt).tolist()
                       for _ in range(args.batch)]
            _, st = llm.generate_batch(prompts, args.gen + 1, GenOptions(eos=-1))
            if r == 0:
                continue
            p = args.batch * args.prompt / st.prefill_seconds
            d = args.batch * args.gen / st.decode_seconds if st.decode_seconds else 0.0
            print(f"round {r}: prefill {p:.1f} tok/s, decode {d:.1f} tok/s")
            best_p, best_d = max(best_p, p), max(best_d, d)
        print(f"prompt {args.prompt} x {args.batch}: {best_p:.1f} tok/s; "
              f"gen {args.gen} x {args.batch}: {best_d:.1f} tok/s")
        return 0

    if args.chat:
        return _chat(llm, GenOptions(eos=eos, temperature=args.temp, top_k=args.top_k,
                                     top_p=args.top_p, min_p=args.min_p, seed=args.seed,
                                     stop=stops[:4]), args)

    prompts = _read_prompts(args, llm.n_vocab)
    opts = [GenOptions(eos=eos, temperature=args.temp, top_k=args.top_k, top_p=args.top_p,
                       min_p=args.min_p, seed=args.seed + i, stop=stops[:4])
            for i in range(len(prompts))]
    t0 = time.perf_counter()
    try:
        outs, st = llm.generate_batch(prompts, args.max, opts)
    except api.LLMError as e:
        print(f"janas-b200: {e}", file=sys.stderr)
        return 2
    for o in outs:
        print(" ".join(str(t) for t in o))
    if args.stats:
        print(f"prompt {st.prompt_tokens} tokens in {st.prefill_seconds:.3f} s; "
              f"{st.new_tokens} new tokens, {st.passes} passes in {st.decode_seconds:.3f} s; "
              f"{st.batches} batches; {time.perf_counter() - t0:.3f} s in all", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
