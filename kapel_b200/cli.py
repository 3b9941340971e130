"""The command line, in the manner of `kapel run` (crates/kapel-cli/src/main.rs:25-72).

    python -m kapel_b200 run MODEL --tokens 2,651,6037 --max-tokens 64 --greedy
    python -m kapel_b200 run MODEL --prompt "text" --temperature 0.8 --seed 7 --stats
    python -m kapel_b200 init CONFIG.json --output DIR --seed 0        (random weights)

Options keep Kapel's names and meanings where it has them; `--tokens` (token ids instead of
text) and `init` are this engine's own.
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
    run.add_argument("model")
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

    if (args.prompt is None) == (args.tokens is None):
        print("error: give exactly one of --prompt and --tokens", file=sys.stderr)
        return 2
    from .model import KapelError, Model

    try:
        t0 = time.perf_counter()
        model = Model(args.model, device=args.device, dtype=args.dtype, quantize=args.quantize, kv_cache=args.kv_cache)
        t_load = time.perf_counter() - t0
        if args.tokens is not None:
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
            if args.tokens is None:
                print(piece, end="", flush=True)
        total = time.perf_counter() - t0
        if args.tokens is not None:
            print(",".join(str(t) for t in out))
        else:
            print()
        if args.stats:
            n = len(out)
            rate = (n - 1) / (total - first) if n > 1 and total > first else float("nan")
            print(f"load {t_load:.2f} s; first token {first or 0:.3f} s; {n} tokens; {rate:.1f} tokens/s decoding", file=sys.stderr)
        return 0
    except KapelError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
