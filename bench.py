"""Throughput of the engine at Gemma 2 sizes with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--size 2b|9b|27b] [--layers L] [--impl reference]

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
  points       decode at batch 1 and 64; and, in the default run, the same figures at the 9B
               and 27B sizes ("9b_decode_b8", "27b_prefill", ...) and the 9B mixed workload
  sizes        the details behind the other sizes' points (ms, fractions of the peaks)
  logits       after the timed steps, one more decode step's logits for one request against
               the engine's own 32-bit path over the same weights and the same tokens: they must
               be finite and within the bfloat16 bound, or the run fails
  clocks       SM clocks sampled with nvidia-smi during the timed regions

The 9B mixed workload (`--size 9b --workload mixed`, and "9b_mixed" in the default run) is the
one Kapel's bench example runs (crates/kapel-cli/examples/bench.rs:125-203 with
crates/kapel-infer/src/batch.rs:20-88): prompts of seeded lengths uniform in 64..4096, 256
tokens decoded for each, through the scheduler with 2,048 tokens a pass.

Weights (5.2 GB and more) are larger than L2, so consecutive timed steps cannot reuse them from cache.
"""
from __future__ import annotations

import argparse
import gc
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

# size -> (the configuration's file under kapel_b200/config/presets, tokens of history a sequence holds)
SIZES = {"2b": ("gemma2-2b", 6144), "9b": ("gemma2-9b", 6144), "27b": ("gemma2-27b", 2048)}
CONTEXT = 8192
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
LOGITS_TOL = 2e-2              # bfloat16 against 32-bit through a whole model (the tests see 1e-2 at 26 layers)


def preset(size):
    with open(os.path.join(ROOT, "kapel_b200", "config", "presets", SIZES[size][0] + ".json")) as f:
        return json.load(f)


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


def layer_windows(cfg, layers):
    """The window of each of the first `layers` layers (None: every key), as config.json says it:
    `layer_types` where given, else the even layers slide."""
    w, types = cfg.get("sliding_window"), cfg.get("layer_types")
    out = []
    for l in range(layers):
        slides = (types[l] == "sliding_attention") if types else (l % 2 == 0)
        out.append(w if (w and slides) else None)
    return out


def weight_bytes(cfg, layers):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h + 4 * h
    return 2 * (layers * per_layer + v * h + h)


def kv_bytes_seen(cfg, layers, context):
    """Bytes of keys and values one sequence's decode step reads at `context` positions."""
    hkv, d = cfg["num_key_value_heads"], cfg["head_dim"]
    return sum((min(context, w) if w else context) * hkv * d * 2 * 2 for w in layer_windows(cfg, layers))


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (hq + 2 * hkv) * d * h + hq * d * h + 3 * i * h
    gemm = 2 * tokens * layers * per_layer + 2 * v * h            # the head runs on one row
    att = 0
    for win in layer_windows(cfg, layers):
        pairs = sum(min(c, win) if win else c for c in range(1, tokens + 1))
        att += 4 * pairs * hq * d
    return gemm + att


def breakdown(model, batch, tokens, history) -> int:
    """Where a step's time goes: each kernel entry point timed with CUDA events (every call
    synchronises, so the sums are device times, not a step time)."""
    import torch

    from kapel_b200 import kernels as K
    from kapel_b200.engine import StepEntry

    engine = model.engine
    engine.graphs = None                                  # eager steps only
    ids = [f"s{i}" for i in range(batch)]
    for s in ids:                                         # history in portions of 2,048
        for at in range(0, history, PREFILL_TOKENS):
            engine.step([StepEntry(s, tokens(min(PREFILL_TOKENS, history - at)), [])])
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
    print(f"decode step, batch {batch}, {history} tokens of history: {sum(r[3] for r in rows):.3f} ms in kernels")
    for name, shape, calls, ms in rows:
        print(f"  {ms:9.3f} ms  {calls:4d} x {name} {shape}")
    K.disable_timing()
    return 0


class Bench:
    """One model of one size and what is measured on it."""

    def __init__(self, size, layers, batches, steps, warmup, clocks, pk, seed=0):
        import numpy as np
        import torch

        from kapel_b200.model import Model

        self.torch = torch
        self.size = size
        base = preset(size)
        self.history = SIZES[size][1]
        self.full_layers = base["num_hidden_layers"]
        self.layers = layers or self.full_layers
        self.cfg = dict(base, num_hidden_layers=self.layers)
        self.batches, self.steps, self.warmup, self.clocks, self.pk, self.seed = batches, steps, warmup, clocks, pk, seed
        room = max(batches) * (-(-(self.history + 4 * (warmup + steps) + 64) // 64) * 64) + PREFILL_TOKENS + 64
        self.model = Model.random(self.cfg, seed=seed, dtype="bf16", max_tokens_cached=room, max_sequences=max(batches) + 1)
        self.engine = self.model.engine
        self.rng = np.random.default_rng(0)
        self.vocab = self.cfg["vocab_size"]

    def tokens(self, n):
        return [int(t) for t in self.rng.integers(1000, self.vocab - 1000, size=n)]

    def timed(self, fn, n):
        torch = self.torch
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.clocks.active = True
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        self.clocks.active = False
        return a.elapsed_time(b) / n

    def prefill(self):
        from kapel_b200.engine import StepEntry

        def once():
            self.engine.step([StepEntry("p", self.tokens(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            self.engine.end("p")

        for _ in range(2):
            once()
        ms = min(self.timed(once, 1) for _ in range(3))
        flops = prefill_flops(self.cfg, self.layers, PREFILL_TOKENS)
        pg = getattr(self.engine, "prompt_graphs", None)
        return {"value": PREFILL_TOKENS / ms * 1e3, "tokens": PREFILL_TOKENS, "ms": ms,
                "frac": flops / (ms * 1e-3) / (self.pk["bf16_tflops"] * 1e12),
                "recorded": bool(pg is not None and pg.replays > 0)}      # the pass's shape was seen before: the engine replays its recording

    def decode_point(self, batch, check_logits=False):
        """dict: device ms a step, e2e ms a step, launches a step, h2d and d2h bytes a step, hbm fraction."""
        from kapel_b200 import kernels as K
        from kapel_b200.engine import StepEntry
        from kapel_b200.engine.scheduler import Request
        from kapel_b200.sampling import Sampling

        torch, engine, steps = self.torch, self.engine, self.steps
        sched = self.model.scheduler(max_pass_tokens=PREFILL_TOKENS, max_sequences=batch)
        rids = [sched.add(Request(prompt=self.tokens(self.history), sampling=Sampling(), max_tokens=10 ** 6, ignore_eos=True))
                for _ in range(batch)]
        while any(sched._pending(r) > 1 for r in rids):       # prompts in portions until every request decodes
            sched.step()
        for _ in range(self.warmup):
            sched.step()
        torch.cuda.synchronize()
        self.clocks.active = True
        t0 = time.perf_counter()
        for _ in range(steps):
            events = sched.step()
            assert len(events) == batch
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) / steps * 1e3
        self.clocks.active = False
        h2d = engine.last_h2d_bytes
        sched.settle()              # the pass enqueued ahead of the host is read: the cache is one token behind each sequence again
        # The same step on the device clock, fed from the step function directly. Nothing is waited
        # for between steps: the staging buffers of a recorded step are guarded by events, so each
        # step runs on its own inputs and the host is at most two steps ahead.
        fed = {r: list(sched.entries[r].sequence) for r in rids}          # fed[r][:-1] is in the cache; the last is fed next

        def one():
            engine.step([StepEntry(r, [fed[r][-1]], [0]) for r in rids])
            for r in rids:
                fed[r].append(fed[r][-1])

        one()
        launches_before = K.launch_count() + (engine.graphs.replayed_kernels if engine.graphs else 0)
        dev_ms = self.timed(one, steps)
        launches = K.launch_count() + (engine.graphs.replayed_kernels if engine.graphs else 0) - launches_before
        context = len(fed[rids[0]]) - 1
        step_bytes = weight_bytes(self.cfg, self.layers) + batch * kv_bytes_seen(self.cfg, self.layers, context)
        achieved = step_bytes / (dev_ms * 1e-3) / 1e9
        out = {"ms": dev_ms, "e2e_ms": e2e_ms, "launches": launches / steps, "h2d": h2d, "d2h": batch * 4, "tok_s": batch / dev_ms * 1e3,
               "bytes": step_bytes, "gbs": achieved, "frac": achieved / self.pk["hbm_gbs"], "context": context}
        if check_logits:
            logits = engine.step([StepEntry(r, [fed[r][-1]], [0]) for r in rids]).clone()
            torch.cuda.synchronize()
            out["logits_row"] = logits[0].cpu()
            out["logits_tokens"] = list(fed[rids[0]])          # the tokens fed to request 0, the last one at the checked place
            out["logits_finite"] = bool(torch.isfinite(logits).all())
        for r in rids:
            sched.cancel(r)
        K.check_async_errors()
        return out

    def check_against_32_bit(self, tokens_fed, row):
        """The bfloat16 logits `row` (of the last of `tokens_fed`) against the engine's 32-bit path over
        the same weights (the same seed gives the same values; the 32-bit path widens them)."""
        from kapel_b200.engine import Engine, StepEntry

        torch = self.torch
        engine = Engine.random(self.cfg, seed=self.seed, dtype="float32", max_tokens=len(tokens_fed) + 64, max_sequences=2)
        logits = None
        for at in range(0, len(tokens_fed), PREFILL_TOKENS):
            part = tokens_fed[at : at + PREFILL_TOKENS]
            last = at + len(part) == len(tokens_fed)
            logits = engine.step([StepEntry("check", part, [len(part) - 1] if last else [])])
        want = logits[0].cpu().double()
        engine.end("check")
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        got = row.double()
        err = float((got - want).abs().max() / want.abs().max())
        return {"rel_err": err, "tol": LOGITS_TOL, "finite": bool(torch.isfinite(got).all()), "positions": len(tokens_fed),
                "same_argmax": bool(int(got.argmax()) == int(want.argmax())), "against": "the engine's float32 path, same weights and tokens"}

    def mixed(self, running, requests, decode=256, lo=64, hi=4096):
        """Kapel's mixed workload: `requests` prompts of seeded lengths uniform in lo..hi, `decode` tokens
        each, at most `running` at once, 2,048 tokens a pass, through the scheduler, host tokens in and out."""
        import numpy as np

        from kapel_b200.engine.scheduler import Request
        from kapel_b200.sampling import Sampling

        torch = self.torch
        rng = np.random.default_rng(7)
        lengths = [int(n) for n in rng.integers(lo, hi + 1, size=requests)]
        sched = self.model.scheduler(max_pass_tokens=PREFILL_TOKENS, max_sequences=running)
        for n in lengths:
            sched.add(Request(prompt=self.tokens(n), sampling=Sampling(), max_tokens=decode, ignore_eos=True))
        weights = weight_bytes(self.cfg, self.layers)
        torch.cuda.synchronize()
        self.clocks.active = True
        t0 = time.perf_counter()
        generated = passes = 0
        must_read = 0
        while sched.has_work():
            events = sched.step()
            passes += 1
            generated += sum(1 for e in events if e.token is not None)
            assert not any(e.finish == "error" for e in events), [e.error for e in events if e.finish == "error"]
            # what the pass had to read: every weight once, and the keys and values each running request sees
            must_read += weights + sum(kv_bytes_seen(self.cfg, self.layers, sched._cached(r)) for r in sched.running)
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        self.clocks.active = False
        st = sched.stats()
        return {"tok_s": generated / seconds, "all_tok_s": (generated + sum(lengths)) / seconds, "seconds": seconds, "requests": requests,
                "running": running, "prompt_tokens": sum(lengths), "generated": generated, "passes": passes, "preemptions": st.preemptions,
                "recorded_passes": st.recorded_passes, "gbs": must_read / seconds / 1e9, "frac": must_read / seconds / 1e9 / self.pk["hbm_gbs"]}

    def close(self):
        self.model = self.engine = None
        gc.collect()
        self.torch.cuda.empty_cache()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size", default="2b", choices=sorted(SIZES), help="layer sizes: Gemma 2 2B (the default and the contract's line), 9B or 27B")
    ap.add_argument("--workload", default="fixed", choices=["fixed", "mixed"],
                    help="fixed: decode at a fixed history and a 2,048-token prefill; mixed: prompts of 64..4096 and 256 decoded tokens each through the scheduler")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64 and the other sizes")
    ap.add_argument("--skip-sizes", action="store_true", help="leave out the 9B and 27B points of the default run")
    ap.add_argument("--skip-check", action="store_true", help="leave out the check of the timed logits against the 32-bit path")
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

    import torch

    torch.cuda.set_device(0)
    pk = peaks()
    clocks = ClockSampler()
    batches = [args.batch] if args.skip_points else sorted({1, args.batch, 64})
    bench = Bench(args.size, args.layers, batches, steps, warmup, clocks, pk)
    cfg, history = bench.cfg, bench.history

    if args.breakdown:
        return breakdown(bench.model, args.batch, bench.tokens, history)

    if args.workload == "mixed":
        res = {f"running_{r}": bench.mixed(r, n) for r, n in ((8, 16), (64, 96))}
        clocks.close()
        main_res = res["running_64"]
        print(json.dumps({
            "metric": f"generated tok/s, mixed workload (Gemma 2 {args.size.upper()} sizes, bf16, prompts 64..4096, 256 decoded each, 64 running)",
            "value": main_res["tok_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic: seeded random weights, seeded prompt lengths and uniform-random token ids",
            "config": {"model": f"gemma2-{args.size}-shape", "layers": bench.layers, "layers_of_config": bench.full_layers, "max_pass_tokens": PREFILL_TOKENS,
                       "requests": main_res["requests"], "running": 64, "decode": 256, "peaks": pk["source"]},
            "mixed": res, "clocks": clocks.summary(), "impl": "ours"}))
        return 0

    prefill = bench.prefill()
    results = {b: bench.decode_point(b, check_logits=(b == args.batch and not args.skip_check)) for b in batches}
    main_res = results[args.batch]
    check = None
    if not args.skip_check:
        row, fed = main_res.pop("logits_row"), main_res.pop("logits_tokens")
        bench.close()                                        # the 32-bit weights need the room at the larger sizes
        check = bench.check_against_32_bit(fed, row)
    else:
        bench.close()

    points = {f"decode_b{b}": results[b]["tok_s"] for b in batches if b != args.batch}
    sizes = {}
    if args.size == "2b" and not args.skip_points and not args.skip_sizes:
        for other in ("9b", "27b"):
            try:
                ob = Bench(other, 0, [1, 8, 64], min(steps, 30), warmup, clocks, pk)
                rec = {"layers": ob.layers, "history": ob.history, "prefill": ob.prefill()}
                for b in (1, 8, 64):
                    r = ob.decode_point(b)
                    rec[f"decode_b{b}"] = {k: r[k] for k in ("tok_s", "ms", "e2e_ms", "frac", "gbs")}
                    points[f"{other}_decode_b{b}"] = r["tok_s"]
                points[f"{other}_prefill"] = rec["prefill"]["value"]
                if other == "9b":
                    rec["mixed"] = ob.mixed(64, 96)
                    points["9b_mixed"] = rec["mixed"]["tok_s"]
                sizes[other] = rec
                ob.close()
            except Exception as e:                          # the contract's line must not be lost to another size
                sizes[other] = {"error": f"{type(e).__name__}: {e}"}
    clocks.close()

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Gemma 2 {args.size.upper()} sizes, bf16, {history} tokens of history per sequence)",
        "value": main_res["tok_s"],
        "unit": "tokens/s",
        "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": main_res["ms"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights and uniform-random token ids",
        "config": {
            "model": f"gemma2-{args.size}-shape", "global_batch": args.batch, "seq_len": CONTEXT, "history": history, "parallelism": "single-gpu",
            "layers": bench.layers, "layers_of_config": bench.full_layers, "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "window": cfg["sliding_window"], "page": 16,
            "l2": f"inputs larger than L2 ({weight_bytes(cfg, bench.layers) / 1e9:.1f} GB of weights a step)", "peaks": pk["source"],
        },
        "e2e": {"value": args.batch / main_res["e2e_ms"] * 1e3, "unit": "tokens/s", "ms_per_step": main_res["e2e_ms"],
                "h2d_bytes_per_step": main_res["h2d"], "d2h_bytes_per_step": main_res["d2h"]},
        "gpu_launches": int(round(main_res["launches"] * steps)),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": main_res["gbs"], "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": main_res["frac"],
                     "bytes": main_res["bytes"]},
        "points": points,
        "logits": check,
        "sizes": sizes,
        "clocks": clocks.summary(),
        "impl": "ours",
    }
    print(json.dumps(line))
    if check is not None and not (check["finite"] and check["rel_err"] <= check["tol"]):
        print(f"bench.py: the timed logits differ from the 32-bit path by {check['rel_err']:.3e} (bound {check['tol']}): the figures above are not valid",
              file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
