"""Where a decoding step's time goes between and inside its kernels.

    python -m kapel_b200.step_timeline [--config gemma2-2b] [--layers 2] [--batch 8] [--history 6144]

builds the library with time stamps compiled into the decoding kernels (KAPEL_B200_TIMELINE=1: see
csrc/timeline.cuh; a folder of its own, the ordinary library is not touched), makes a model of the
preset's layer sizes with random weights and `--layers` layers, fills `--batch` requests with
`--history` tokens each, runs a few recorded decode steps as serving does, and prints the stamps that
the last step's last layer left, in order: when block 0 and the last block of each kernel entered,
when block 0 got past its wait on the kernel before, landmarks inside it, and when the blocks left.
A launch list gives each kernel's duration; only this shows the waits between dependent kernels, what
overlaps what, and a tail inside a kernel. The stamps cost a few hundred nanoseconds a kernel: read
differences, and take a step's time from bench.py.
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", default="gemma2-2b", help="a preset's name or a config.json")
    ap.add_argument("--layers", type=int, default=2, help="layers of the model that is stepped (the last one's stamps are printed)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--history", type=int, default=6144)
    ap.add_argument("--steps", type=int, default=6)
    args = ap.parse_args(argv)
    if args.layers < 2:
        ap.error("--layers must be at least 2: the last layer's first product waits on the layer before")

    os.environ["KAPEL_B200_TIMELINE"] = "1"                # before the package builds or finds its library
    import numpy as np
    import torch

    from kapel_b200 import kernels as K
    from kapel_b200.config.registry import read_config_file
    from kapel_b200.engine import StepEntry
    from kapel_b200.model import Model

    cfg = dict(read_config_file(args.config), num_hidden_layers=args.layers)
    room = args.batch * (-(-(args.history + args.steps + 64) // 64) * 64) + 64
    model = Model.random(cfg, seed=0, dtype="bf16", max_tokens_cached=room, max_sequences=args.batch + 1)
    engine = model.engine
    rng = np.random.default_rng(0)
    vocab = cfg["vocab_size"]
    ids = [f"r{i}" for i in range(args.batch)]
    for r in ids:
        for at in range(0, args.history, 2048):
            n = min(2048, args.history - at)
            engine.step([StepEntry(r, [int(t) for t in rng.integers(0, vocab, size=n)], [])])
    for _ in range(args.steps):
        engine.step([StepEntry(r, [int(rng.integers(0, vocab))], [0]) for r in ids])
    torch.cuda.synchronize()
    K.check_async_errors()

    lib = K.library()
    kinds = {0: "product", 1: "gated product", 2: "add and norm", 3: "rotate and append", 4: "attention", 5: "attention's merge"}
    events = []
    for unit in ("gemm", "norm", "elementwise", "attention"):
        buf = (ctypes.c_ulonglong * (16 * 10))()
        slots = getattr(lib, "kb_timeline_" + unit)(buf)
        if slots <= 0:
            print("this library was built without the time stamps (KAPEL_B200_TIMELINE=1 was set too late?)", file=sys.stderr)
            return 1
        for s in range(slots):
            f = buf[s * 10 : s * 10 + 10]
            if f[1] == 0:
                continue
            kind, a, b = int(f[7]), int(f[8]), int(f[9])
            name = kinds.get(kind, f"kind {kind}")
            if kind in (0, 1):
                name += f" [{a} x {b}]"
            elif kind == 2:
                name += f" ({a} slices{', then the next norm' if b else ', last of the model'})"
            elif kind == 3:
                name += f" ({b} slices)"
            else:
                name += f" ({a} slots, {'window ' + str(b) if b else 'all keys'})"
            marks = {0: "last block enters", 1: "block 0 enters", 2: "block 0 past its wait", 5: "last block leaves", 6: "block 0 leaves"}
            if kind in (0, 1):
                marks.update({3: "block 0: first tile landed", 4: "block 0: sums done"})
            if kind == 4:
                marks.update({3: "block 0: loop over keys begins", 4: "block 0: loop done"})
            if kind == 2:
                marks.update({3: "block 0: slices and residual loaded", 4: "block 0: both sums known"})
            events.extend((int(f[i]), f"{name}: {what}") for i, what in marks.items() if f[i])
    if not events:
        print("no kernel left a stamp", file=sys.stderr)
        return 1
    events.sort()
    # The head's product runs once a step, after the last layer: everything from the last layer's
    # first product on belongs to one step. Start there.
    t0 = events[0][0]
    print(f"# {args.config}, {args.layers} layers, batch {args.batch}, {args.history} tokens of history: the last step, us from the first stamp")
    for t, what in events:
        print(f"{(t - t0) / 1000:10.2f}  {what}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
