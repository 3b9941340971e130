"""Tiny configurations, model folders in temporary places, traces and the comparison metric."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

import plain_gemma2 as P

ROOT = Path(__file__).resolve().parent.parent

# Two tiny configurations that differ in every size and option.
TINY_A = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    intermediate_size=128, vocab_size=512, rope_theta=10000.0, sliding_window=16,
    query_pre_attn_scalar=16, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    rms_norm_eps=1e-6, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
    max_position_embeddings=128,
)
TINY_B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=1, head_dim=32,
    intermediate_size=320, vocab_size=1000, rope_theta=500000.0, sliding_window=24,
    layer_types=["sliding_attention", "full_attention", "sliding_attention"],
    query_pre_attn_scalar=24, attn_logit_softcapping=20.0, final_logit_softcapping=15.0,
    rms_norm_eps=1e-5, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
    max_position_embeddings=256,
)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1)}

# Tolerances: the largest difference of logits over the largest logit of the plain result. In
# 32-bit the reference's own bar (2e-5; these tests see about 1e-6). In bfloat16 the tiny models,
# whose logits are a few tenths, see up to 1.2e-2 in the worst cut; the bound leaves a quarter above that.
TOL = {"float32": 2e-5, "bfloat16": 1.5e-2}


def make_model_dir(raw_config: dict, seed: int, folder=None, scale_up: float = 1.0, device="cpu") -> Path:
    """config.json and model.safetensors with seeded random weights, in a temporary folder."""
    from kapel_b200.config import config_from_json
    from kapel_b200.weights import write_random_model

    folder = Path(folder or tempfile.mkdtemp(prefix="kapel_b200_model_"))
    write_random_model(folder, config_from_json(raw_config), seed, device=device)
    return folder


_PLAIN_CACHE = {}


def plain_model(folder, dtype=torch.float64):
    key = (str(folder), dtype)
    if key not in _PLAIN_CACHE:
        _PLAIN_CACHE[key] = P.load(folder, dtype)
    return _PLAIN_CACHE[key]


def plain_logits(folder, tokens, embed_scale=None, dtype=torch.float64) -> np.ndarray:
    cfg, w = plain_model(folder, dtype)
    return P.forward(cfg, w, tokens, embed_scale=embed_scale).to(torch.float64).numpy()


def embed_scale_for(raw_config: dict, dtype: str) -> float:
    """sqrt(hidden) as the path holds it: rounded to bfloat16 on the bfloat16 path
    (crates/kapel-models/src/model.rs:2079-2083), to float32 on the 32-bit path."""
    s = torch.tensor(float(raw_config["hidden_size"]) ** 0.5, dtype=torch.float32)
    if dtype == "bfloat16":
        s = s.to(torch.bfloat16)
    return float(s.float())


def rel_err(got: np.ndarray, want: np.ndarray) -> float:
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (got.shape, want.shape)
    if not np.isfinite(got).all():
        return float("inf")
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def random_tokens(rng: np.random.Generator, n: int, vocab: int):
    return [int(t) for t in rng.integers(0, vocab, size=n)]


# ------------------------------------------------------------------------------------------
# traces: lists of steps as bin/trace_run reads them


def run_trace_engine(engine, steps):
    """Feeds `steps` to an Engine; returns {step: float32 array [wanted, vocab]}."""
    from kapel_b200.engine import StepEntry

    out = {}
    for rec in steps:
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec["entries"]]
        if entries:
            logits = engine.step(entries)
            if logits.shape[0]:
                out[rec["step"]] = logits.float().cpu().numpy()
        for s in rec.get("end", []):
            engine.end(s)
    return out


def run_trace_program(model_dir, dtype, steps, max_tokens, env=None, timeout=900):
    """Runs bin/trace_run as a program; returns {step: array}."""
    out_dir = Path(tempfile.mkdtemp(prefix="kapel_b200_trace_"))
    text = "".join(json.dumps(s) + "\n" for s in steps)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    r = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, f"trace_run failed ({r.returncode}):\n{r.stdout}\n{r.stderr}"
    done = [l for l in r.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in steps], r.stdout
    vocab = json.loads((Path(model_dir) / "config.json").read_text())["vocab_size"]
    res = {}
    for f in out_dir.glob("*.f32"):
        res[int(f.stem)] = np.fromfile(f, dtype="<f4").reshape(-1, vocab)
    return res


def max_tokens_for(lengths, live=None):
    """--max-tokens for requests of these lengths all live at once, each rounded up to 64."""
    return sum(-(-n // 64) * 64 for n in lengths)


def check_against_plain(results, expect, tol, what=""):
    """`expect` is {step: [(request tokens so far ... )]}: a list per step of (full token list,
    positions wanted); compares each wanted row with the plain logits at that position."""
    worst = 0.0
    for step, wanted in expect.items():
        rows = results[step]
        want = np.stack(wanted)
        err = rel_err(rows, want)
        worst = max(worst, err)
        assert err <= tol, f"{what}: step {step}: relative error {err:.3e} > {tol:.1e}"
    return worst


class TraceBuilder:
    """Builds steps and remembers, for every wanted row, which (request, position) it is."""

    def __init__(self):
        self.steps = []
        self.rows = {}           # step -> [(request id, absolute position)]
        self.fed = {}            # request id -> tokens fed so far

    def step(self, entries, end=()):
        n = len(self.steps)
        recs, rows = [], []
        for rid, tokens, want in entries:
            base = self.fed.get(rid, 0)
            recs.append({"id": rid, "tokens": list(tokens), "want": list(want)})
            rows.extend((rid, base + w) for w in want)
            self.fed[rid] = base + len(tokens)
        self.steps.append({"step": n, "entries": recs, "end": list(end)})
        if rows:
            self.rows[n] = rows
        for rid in end:
            self.fed.pop(rid, None)
        return n


def compare_trace(results, builder: TraceBuilder, plain_by_request, tol, what=""):
    """Every wanted row against the plain logits of its request at its position."""
    worst = 0.0
    for step, rows in builder.rows.items():
        assert step in results, f"{what}: step {step} wrote no logits"
        got = results[step]
        assert got.shape[0] == len(rows), f"{what}: step {step}: {got.shape[0]} rows for {len(rows)} wanted"
        for i, (rid, pos) in enumerate(rows):
            err = rel_err(got[i], plain_by_request[rid][pos])
            worst = max(worst, err)
            assert err <= tol, f"{what}: step {step}, request {rid}, position {pos}: relative error {err:.3e} > {tol:.1e}"
    return worst
