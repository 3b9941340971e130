"""The command line, in the manner of `kapel run` (crates/kapel-cli/src/main.rs:25-72).

    python -m kapel_b200 run MODEL --tokens 2,651,6037 --max-tokens 64 --greedy
    python -m kapel_b200 run MODEL --prompt "text" --temperature 0.8 --seed 7 --stats
    python -m kapel_b200 run --random gemma2-27b --seed-weights 0 --prompt-len 2048 --max-tokens 64 --greedy --stats
    python -m kapel_b200 init CONFIG.json --output DIR --seed 0        (random weights)

Options keep Kapel's names and meanings where it has them. This engine's own: `--tokens` (token
ids instead of text), `--prompt-len N` (N seeded random token ids as the prompt), `--random
CONFIG --seed-weights S` (no folder: a model of CONFIG, a config.json or a preset's name, with
random weights made on the device), `--pages`, `--max-pass-tokens`, `--max-sequences` (Kapel's
engine options, crates/kapel-infer/src/engine.rs:36-64), `--strict`, and `init`.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

USAGE_NOTE = """Generates tokens with MODEL, a folder with config.json and model.safetensors.
--prompt needs the folder's tokenizer.json and the `tokenizers` package; --tokens needs neither."""


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="kapel_b200", description=USAGE_NOTE)
    sub = ap.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="generate with MODEL")
    run.add_argument("model", nargs="?", help="a folder with config.json and model.safetensors (or --random CONFIG)")
    run.add_argument("--random", metavar="CONFIG", help="instead of MODEL: random weights for this config.json (a path, or a preset's name)")
    run.add_argument("--seed-weights", type=int, default=0, help="the seed of --random's weights (default 0)")
    run.add_argument("--prompt-len", type=int, default=None, help="the prompt is N random token ids drawn with --seed")
    run.add_argument("--pages", type=int, default=None, help="pages of 16 positions in each layer group's pool (default: room for 65536 positions)")
    run.add_argument("--max-pass-tokens", type=int, default=2048, help="the most tokens one pass holds: prompts are cut into such portions (default 2048)")
    run.add_argument("--max-sequences", type=int, default=256, help="the most requests running at once (default 256)")
    run.add_argument("--strict", action="store_true", help="a tensor in the file that the model does not name is an error")
    run.add_argument("--prompt", help="answer TEXT, then exit")
    run.add_argument("--tokens", help="the prompt as comma-separated token ids")
    run.add_argument("--device", default="cuda", help="cuda or cuda:N (this engine has no cpu path)")
    run.add_argument("--dtype", default=None, choices=["f32", "bf16"], help="the type of the float weights (default bf16)")
    run.add_argument("--max-tokens", type=int, default=512, help="the most tokens per answer (default 512)")
    run.add_argument("--greedy", action="store_true", help="always the most likely token")
    run.add_argument("--temperature", type=float, default=None, help="sampling (defaults: the model's generation_config.json)")
    run.add_argument("--top-k", type=int, default=None)
    run.add_argument("--top-p", type=float, default=None)
    run.add_argument("--min-p", type=float, default=None)
    run.add_argument("--repetition-penalty", type=float, default=None)
    run.add_argument("--seed", type=int, default=0, help="the seed of the draws (default 0)")
    run.add_argument("--stop", action="append", default=[], help="end the answer at TEXT (repeatable); with --tokens, comma-separated ids")
    run.add_argument("--kv-cache", default=None, help="the type of the cache of keys and values (only the compute dtype here)")
    run.add_argument("--quantize", default=None, help="not built in this engine")
    run.add_argument("--stats", action="store_true", help="speeds on the standard error")
    run.add_argument("--ignore-eos", action="store_true", help="go on past an end-of-sequence token")
    init = sub.add_parser("init", help="write a model folder with random weights")
    init.add_argument("config", help="a config.json")
    init.add_argument("--output", required=True)
    init.add_argument("--seed", type=int, default=0)
    return ap


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "init":
        from .config import config_from_json
        from .weights import write_random_model

        with open(args.config) as f:
            config = config_from_json(json.load(f))
        print(write_random_model(args.output, config, args.seed))
        return 0

    if sum(x is not None for x in (args.prompt, args.tokens, args.prompt_len)) != 1:
        print("error: give exactly one of --prompt, --tokens and --prompt-len", file=sys.stderr)
        return 2
    if (args.model is None) == (args.random is None):
        print("error: give either MODEL or --random CONFIG", file=sys.stderr)
        return 2
    if args.prompt_len is not None and args.prompt_len <= 0:
        print("error: --prompt-len must be positive", file=sys.stderr)
        return 2
    from .config import ConfigError
    from .model import KapelError, Model

    try:
        t0 = time.perf_counter()
        if args.random is not None:
            if args.quantize is not None:
                raise KapelError("quantized weights are not built in this engine")
            try:
                model = Model.random(args.random, seed=args.seed_weights, dtype=args.dtype or "bf16", pages=args.pages,
                                     max_sequences=args.max_sequences, max_pass_tokens=args.max_pass_tokens)
            except (ConfigError, ValueError) as e:
                raise KapelError(str(e)) from e
        else:
            model = Model(args.model, device=args.device, dtype=args.dtype, quantize=args.quantize, kv_cache=args.kv_cache,
                          pages=args.pages, max_sequences=args.max_sequences, max_pass_tokens=args.max_pass_tokens, strict=args.strict)
        t_load = time.perf_counter() - t0
        if args.prompt_len is not None:
            import numpy as np

            vocab = model.engine.vocab_size
            prompt = [int(t) for t in np.random.default_rng(args.seed).integers(0, vocab, size=args.prompt_len)]
            stop = [[int(t) for t in s.split(",")] for s in args.stop]
        elif args.tokens is not None:
            prompt = [int(t) for t in args.tokens.split(",") if t.strip()]
            stop = [[int(t) for t in s.split(",")] for s in args.stop]
        else:
            prompt, stop = args.prompt, list(args.stop)
        temperature = 0.0 if args.greedy else args.temperature
        t0 = time.perf_counter()
        first = None
        out = []
        for piece in model.generate(prompt, max_tokens=args.max_tokens, temperature=temperature, top_k=args.top_k,
                                    top_p=args.top_p, min_p=args.min_p, repetition_penalty=args.repetition_penalty,
                                    seed=args.seed, stop=stop, stream=True, ignore_eos=args.ignore_eos):
            if first is None:
                first = time.perf_counter() - t0
            out.append(piece)
            if args.prompt is not None:
                print(piece, end="", flush=True)
        total = time.perf_counter() - t0
        if args.prompt is None:
            print(",".join(str(t) for t in out))
        else:
            print()
        if args.stats:
            n = len(out)
            rate = (n - 1) / (total - first) if n > 1 and total > first else float("nan")
            n_prompt = len(prompt) if not isinstance(prompt, str) else len(model.tokenize(prompt))
            print(f"load {t_load:.2f} s; prompt {n_prompt} tokens; first token {first or 0:.3f} s; {n} tokens; {rate:.1f} tokens/s decoding",
                  file=sys.stderr)
            st = model.last_scheduler.stats()
            print(f"passes {st.passes} ({st.recorded_passes} recorded); preemptions {st.preemptions}; pages {st.pages}, free {st.free_pages}; "
                  f"released by windows {st.released_pages}", file=sys.stderr)
        return 0
    except KapelError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
