"""Writes tests/golden/plain_logits.json: a few logits of the plain implementation
(tests/plain_gemma2.py) on the two tiny random models.

Kapel's own model code is Rust and cannot be compiled or imported here (no cargo, no rustc,
no network), so these numbers are NOT Kapel's outputs: they rest on its formulas as
tests/plain_gemma2.py states them, and guard that file against silent change.

    python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

import plain_gemma2 as P  # noqa: E402
from helpers import TINY, make_model_dir  # noqa: E402

out = {}
for name, (raw, seed) in TINY.items():
    folder = make_model_dir(raw, seed)
    cfg, w = P.load(folder, torch.float64)
    tokens = [int(t) for t in np.random.default_rng(100 + seed).integers(0, raw["vocab_size"], size=30)]
    logits = P.forward(cfg, w, tokens).numpy()
    columns = list(range(0, raw["vocab_size"], raw["vocab_size"] // 16))
    out[name] = {"tokens": tokens, "columns": columns, "last_row": [float(x) for x in logits[-1][columns]],
                 "argmax": int(np.argmax(logits[-1]))}
(HERE / "plain_logits.json").write_text(json.dumps(out, indent=1))
print("wrote", HERE / "plain_logits.json")
