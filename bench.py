"""Throughput of the engine at Gemma 2 2B sizes with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A "step" is one decode step. The default run has the layer sizes of the 2B configuration
(26 layers, hidden 2304, 8 heads over 4 kv heads of 256, intermediate 9216, vocabulary 256000,
window 4096 on even layers, page 16), a batch of 8 sequences that each hold 6,144 tokens of
history, bfloat16. It prints ONE JSON line:

  value        decoded tokens a second, timed on the device with CUDA events over K steps
  e2e          the same through the Python entry point (`Model.scheduler().step()`): every step
               copies its token ids and block tables from pinned host memory and reads the
               sampled tokens back
  prefill      one step of 2,048 prompt tokens: tokens a second, and flops / time / peak
  roofline     the decode step against the bytes it has to read (every weight once, and the
               cached keys and values the live requests see) at the measured copy bandwidth
  points       decode at batch 1 and 64
  clocks       SM clocks sampled with nvidia-smi during the timed regions

Weights (5.2 GB) are larger than L2, so consecutive timed steps cannot reuse them from cache.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GEMMA2_2B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=26, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4, head_dim=256,
    intermediate_size=9216, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
    query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    rms_norm_eps=1e-6, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
    max_position_embeddings=8192,
)
# The other two sizes, for `--size`; the line the contract asks for is the 2B one.
GEMMA2_9B = dict(GEMMA2_2B, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=14336)
GEMMA2_27B = dict(GEMMA2_2B, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
                  intermediate_size=36864, query_pre_attn_scalar=144)
SIZES = {"2b": (GEMMA2_2B, 6144), "9b": (GEMMA2_9B, 6144), "27b": (GEMMA2_27B, 2048)}      # configuration, tokens of history
FULL_LAYERS = GEMMA2_2B["num_hidden_layers"]
HISTORY = 6144
CONTEXT = 8192
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                    "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons while `active`: one nvidia-smi process that prints a
    line every 50 ms, read by a thread."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index=0):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.active = False
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i", str(index), "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        for line in self.proc.stdout:
            out = line.strip().split(",")
            if not self.active or len(out) < 6:
                continue
            try:
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
            except ValueError:
                continue
            for name, v in zip(self.NAMES, out[2:6]):
                if v.strip().lower().startswith("active"):
                    self.reasons.add(name)

    def close(self):
        if self.proc is not None:
            self.proc.terminate()                     # this object's own child, by its handle
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self._thread.join(timeout=2)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def weight_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h + 4 * h
    return 2 * (layers * per_layer + v * h + h)


def kv_bytes_seen(cfg, layers, context):
    """Bytes of keys and values one sequence's decode step reads at `context` positions."""
    hkv, d, w = cfg["num_key_value_heads"], cfg["head_dim"], cfg["sliding_window"]
    total = 0
    for l in range(layers):
        seen = min(context, w) if l % 2 == 0 else context
        total += seen * hkv * d * 2 * 2
    return total


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d, w = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["sliding_window"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h
    gemm = 2 * tokens * layers * per_layer + 2 * v * h            # the head runs on one row
    att = 0
    for l in range(layers):
        win = w if l % 2 == 0 else None
        pairs = sum(min(c, win) if win else c for c in range(1, tokens + 1))
        att += 4 * pairs * hq * d
    return gemm + att


def breakdown(model, batch, tokens) -> int:
    """Where a step's time goes: each kernel entry point timed with CUDA events (every call
    synchronises, so the sums are device times, not a step time)."""
    import torch

    from kapel_b200 import kernels as K
    from kapel_b200.engine import StepEntry

    engine = model.engine
    engine.graphs = None                                  # eager steps only
    ids = [f"s{i}" for i in range(batch)]
    for s in ids:                                         # history in portions of 2,048
        for at in range(0, HISTORY, PREFILL_TOKENS):
            engine.step([StepEntry(s, tokens(PREFILL_TOKENS), [])])
    engine.step([StepEntry("p", tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
    engine.end("p")
    engine.step([StepEntry(s, tokens(1), [0]) for s in ids])
    torch.cuda.synchronize()
    K.enable_timing()
    engine.step([StepEntry("p", tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
    engine.end("p")
    rows = K.timing_report()
    print(f"prefill of {PREFILL_TOKENS} tokens: {sum(r[3] for r in rows):.3f} ms in kernels")
    for name, shape, calls, ms in rows:
        print(f"  {ms:9.3f} ms  {calls:4d} x {name} {shape}")
    engine.step([StepEntry(s, tokens(1), [0]) for s in ids])
    rows = K.timing_report()
    print(f"decode step, batch {batch}, {HISTORY} tokens of history: {sum(r[3] for r in rows):.3f} ms in kernels")
    for name, shape, calls, ms in rows:
        print(f"  {ms:9.3f} ms  {calls:4d} x {name} {shape}")
    K.disable_timing()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="2b", choices=sorted(SIZES), help="layer sizes: Gemma 2 2B (the default and the contract's line), 9B or 27B")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64")
    ap.add_argument("--breakdown", action="store_true",
                    help="instead of the JSON line: device time by kernel for one prefill step and one eager decode step")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "smallbard/kapel is a Rust workspace; this image has no cargo/rustc and no network, so it cannot be built or installed offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import numpy as np
    import torch

    from kapel_b200 import kernels as K
    from kapel_b200.engine import StepEntry
    from kapel_b200.engine.scheduler import EngineOptions, Request
    from kapel_b200.model import Model
    from kapel_b200.sampling import Sampling

    torch.cuda.set_device(0)
    pk = peaks()
    global HISTORY, FULL_LAYERS
    base, HISTORY = SIZES[args.size]
    FULL_LAYERS = base["num_hidden_layers"]
    args.layers = args.layers or FULL_LAYERS
    cfg = dict(base, num_hidden_layers=args.layers)
    batches = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    room = max(batches) * (-(-(HISTORY + 4 * (warmup + steps) + 64) // 64) * 64) + PREFILL_TOKENS + 64
    model = Model.random(cfg, seed=0, dtype="bf16", max_tokens_cached=room, max_sequences=max(batches) + 1)
    engine = model.engine
    vocab = cfg["vocab_size"]
    rng = np.random.default_rng(0)
    clocks = ClockSampler()

    def tokens(n):
        return [int(t) for t in rng.integers(1000, vocab - 1000, size=n)]

    def timed(fn, n):
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        clocks.active = True
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        clocks.active = False
        return a.elapsed_time(b) / n

    if args.breakdown:
        return breakdown(model, args.batch, tokens)

    # ---------------------------------------------------------------- prefill of 2,048 tokens
    def prefill_once():
        engine.step([StepEntry("p", tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
        engine.end("p")

    for _ in range(2):
        prefill_once()
    prefill_ms = min(timed(prefill_once, 1) for _ in range(3))
    pf_flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / prefill_ms * 1e3, "tokens": PREFILL_TOKENS, "ms": prefill_ms,
               "frac": pf_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    # ---------------------------------------------------------------- decode
    def decode_point(batch):
        """(device ms a step, e2e ms a step, launches a step, h2d bytes, d2h bytes)"""
        sched = model.scheduler(max_pass_tokens=PREFILL_TOKENS, max_sequences=batch)
        greedy = Sampling()
        rids = [sched.add(Request(prompt=tokens(HISTORY), sampling=greedy, max_tokens=10 ** 6, ignore_eos=True)) for _ in range(batch)]
        while any(sched._pending(r) > 1 for r in rids):       # prompts in portions until every request decodes
            sched.step()
        for _ in range(warmup):
            sched.step()
        torch.cuda.synchronize()
        clocks.active = True
        t0 = time.perf_counter()
        for _ in range(steps):
            events = sched.step()
            assert len(events) == batch
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) / steps * 1e3
        clocks.active = False
        h2d = engine.last_h2d_bytes
        # the same step on the device clock, fed from the step function directly
        last = {r: sched.entries[r].sequence[-1] for r in rids}

        def one():
            engine.step([StepEntry(r, [last[r]], [0]) for r in rids])

        one()
        launches_before = K.launch_count() + (engine.graphs.replayed_kernels if engine.graphs else 0)
        dev_ms = timed(one, steps)
        launches = K.launch_count() + (engine.graphs.replayed_kernels if engine.graphs else 0) - launches_before
        for r in rids:
            sched.cancel(r)
        return dev_ms, e2e_ms, launches / steps, h2d, batch * 4

    results = {b: decode_point(b) for b in batches}
    clocks.close()
    dev_ms, e2e_ms, launches, h2d, d2h = results[args.batch]
    step_bytes = weight_bytes(cfg, args.layers) + args.batch * kv_bytes_seen(cfg, args.layers, HISTORY + warmup + steps)
    achieved = step_bytes / (dev_ms * 1e-3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} (Gemma 2 {args.size.upper()} sizes, bf16, {HISTORY} tokens of history per sequence)",
        "value": args.batch / dev_ms * 1e3,
        "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": dev_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform-random token ids",
        "config": {
            "model": f"gemma2-{args.size}-shape", "global_batch": args.batch, "seq_len": CONTEXT, "history": HISTORY, "parallelism": "single-gpu",
            "layers": args.layers, "layers_of_config": FULL_LAYERS, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "window": cfg["sliding_window"], "page": engine.cache.page_size,
            "l2": f"inputs larger than L2 ({weight_bytes(cfg, args.layers) / 1e9:.1f} GB of weights a step)", "peaks": pk["source"],
        },
        "e2e": {"value": args.batch / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(round(launches * steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"], "bytes": step_bytes},
        "points": {f"decode_b{b}": b / results[b][0] * 1e3 for b in batches if b != args.batch},
        "clocks": clocks.summary(),
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
