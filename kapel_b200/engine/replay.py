"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and owns nothing: it drives `Engine.step`, the step function that
generation uses, with its cache and kernels. Kapel has no such program; the nearest are its
parity checks (crates/kapel-models/examples/parity.rs:11-58, crates/kapel-models/tests/parity.rs:43-65).

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
    trace_run --random CONFIG --seed-weights S --dtype ... --out DIR --max-tokens N

`--random` takes the place of `--model`: a model of CONFIG (a config.json, or the name of one
that comes with the package) with random weights made on the device from the seed, for sizes
whose folder nobody wants to write.

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, `OUT/<step>.f32` receives the logits at the wanted
places, in the order of the entries and of `want`, as little-endian float32 [wanted, vocab].
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", help="a folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG", help="instead of --model: random weights for this config.json (a path, or a preset's name)")
    ap.add_argument("--seed-weights", type=int, default=0, help="the seed of --random's weights (default 0)")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="the folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="the most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    if (args.model is None) == (args.random is None):
        ap.error("give either --model DIR or --random CONFIG")

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    print(f"trace_run: loading {args.model or args.random} ({args.dtype}); kernels are compiled at the first call", file=sys.stderr, flush=True)

    from .step import Engine, StepEntry

    if args.random is not None:
        from ..config import read_config_file

        engine = Engine.random(read_config_file(args.random), seed=args.seed_weights, dtype=args.dtype,
                               max_tokens=args.max_tokens, max_sequences=16)
    else:
        engine = Engine.from_dir(args.model, dtype=args.dtype, max_tokens=args.max_tokens, max_sequences=16)
    print("trace_run: ready", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in record.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                host = logits.float().cpu().contiguous().numpy().astype("<f4", copy=False)
                (out / f"{step}.f32").write_bytes(host.tobytes())
        for seq_id in record.get("end", []):
            engine.end(seq_id)
        print(f"done {step}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
