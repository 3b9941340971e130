"""Times each kernel of a decode step (and of a prompt step) alone, at given layer sizes.

    python -m kapel_b200.kernel_bench [--batch 8] [--history 6144] [--prompt 2048] [--iters 20]

For every kernel: device time by CUDA events (mean of `iters` launches after 3 warm-ups), the
bytes it has to move, and the bandwidth that makes. Operands rotate through enough copies to
exceed L2, so a launch never finds its weights or its cache pages in L2 from the launch before.
Sizes default to Gemma 2 2B's; they are arguments, not constants of the package.

    python -m kapel_b200.kernel_bench --host [--batch 8] [--history 6144] [--vocab 256000]

times the host library instead (no GPU needed): planning and committing a decode step in the cache
manager, and the host sampler's choice for one request and for the whole batch.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys

import numpy as np
import torch


def _time(fn, iters, warm=3):
    """Microseconds a call: `iters` calls recorded into one CUDA graph (so the host's launch cost
    is not in the figure), the graph replayed three times, the best replay taken."""
    import gc

    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            for i in range(iters):
                fn(warm + i)
    finally:
        gc.enable()
    best = float("inf")
    for _ in range(3):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        graph.replay()
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b))
    return best / iters * 1e3


def host_bench(args) -> int:
    """Wall-clock times of the host library's calls at the given batch, history and vocabulary."""
    import time

    from .cache import CacheManager, CacheNeeds, PagedKV
    from .sampling import Sampler, Sampling, choose_many

    def clock(fn, n):
        fn()
        t0 = time.perf_counter()
        for _ in range(n):
            fn()
        return (time.perf_counter() - t0) / n * 1e6

    B = args.batch
    needs = {0: CacheNeeds(paged=PagedKV(args.kv_heads, args.head_dim, args.window)), 1: CacheNeeds(paged=PagedKV(args.kv_heads, args.head_dim, None))}
    pages = B * (-(-(args.history + 1024) // 16))
    cache = CacheManager(needs, 16, pages, B)
    for i in range(B):
        cache.add_sequence(i)
    cache.commit(cache.plan([(i, args.history) for i in range(B)]))
    steps = [(i, 1) for i in range(B)]
    print(f"cache manager, batch {B}, {args.history} positions each: plan + commit of a decode step "
          f"{clock(lambda: cache.commit(cache.plan(steps)), 300):.1f} us")
    rows = (np.random.default_rng(0).normal(size=(B, args.vocab)) * 3).astype(np.float32)
    seq = list(range(100, 400))
    for name, st in (("top_k 50", Sampling(temperature=1.0, top_k=50)), ("top_p 0.9", Sampling(temperature=0.8, top_p=0.9)),
                     ("top_k 50, top_p 0.9, min_p 0.05, repetition 1.1", Sampling(temperature=0.8, top_k=50, top_p=0.9, min_p=0.05, repetition_penalty=1.1))):
        one = Sampler(st)
        many = [Sampler(st) for _ in range(B)]
        t_one = clock(lambda: one.choose(rows[0], seq, 50), 10)
        t_many = clock(lambda: choose_many(many, rows, [seq] * B, [50] * B), 10)
        print(f"host sampler, {args.vocab} logits, {name}: one request {t_one / 1e3:.2f} ms, {B} at once {t_many / 1e3:.2f} ms")
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--history", type=int, default=6144)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--hidden", type=int, default=2304)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--kv-heads", type=int, default=4)
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--intermediate", type=int, default=9216)
    ap.add_argument("--vocab", type=int, default=256000)
    ap.add_argument("--window", type=int, default=4096)
    ap.add_argument("--only", default="", help="comma-separated substrings of kernel names to run")
    ap.add_argument("--host", action="store_true", help="time the host library (cache manager, host sampler) instead; no GPU needed")
    args = ap.parse_args(argv)
    if args.host:
        return host_bench(args)

    from . import kernels as K
    from .engine.batch import cut_tiles, decode_split, prompt_costs_of, prompt_split, sm_count

    dev = torch.device("cuda", torch.cuda.current_device())
    K.library()
    B, H, Hq, Hkv, D, I, V = args.batch, args.hidden, args.heads, args.kv_heads, args.head_dim, args.intermediate, args.vocab
    bf = torch.bfloat16
    rows = []

    def want(name):
        return not args.only or any(s in name for s in args.only.split(","))

    def report(name, us, nbytes, flops=0.0):
        rows.append((name, us, nbytes, flops))
        gbs = nbytes / us / 1e3
        tf = flops / us / 1e6
        print(f"{name:44s} {us:9.2f} us  {nbytes / 1e6:9.2f} MB  {gbs:8.1f} GB/s" + (f"  {tf:8.1f} TFLOP/s" if flops else ""), flush=True)

    def copies(nbytes):
        return max(2, int(math.ceil(300e6 / max(nbytes, 1))))       # enough to exceed L2 (126 MB) twice over

    # ------------------------------------------------------------------ products
    def gemm_case(name, m, n, k, out_dtype=bf, softcap=None):
        if not want(name):
            return
        nbytes = n * k * 2
        c = min(copies(nbytes), 8)
        ws = [torch.randn(n, k, device=dev, dtype=torch.float32).mul_(0.02).to(bf) for _ in range(c)]
        a = torch.randn(m, k, device=dev).to(bf)
        us = _time(lambda i: K.gemm(a, ws[i % c], out_dtype=out_dtype, softcap=softcap), args.iters)
        report(f"{name} [{m}x{k}]x[{n}x{k}]", us, nbytes + m * k * 2 + m * n * 2, 2.0 * m * n * k)

    for m, tag in ((B, "decode"), (args.prompt, "prompt")):
        gemm_case(f"gemm qkv {tag}", m, (Hq + 2 * Hkv) * D, H)
        gemm_case(f"gemm o {tag}", m, H, Hq * D)
        gemm_case(f"gemm gate_up {tag}", m, 2 * I, H)
        gemm_case(f"gemm down {tag}", m, H, I)
    gemm_case("gemm head decode", B, V, H, out_dtype=torch.float32, softcap=30.0)

    def glu_case(name, m):
        """The gate|up product with the gated unit in its epilogue, as the feed-forward part calls it."""
        if not want(name):
            return
        ws = [torch.randn(2 * I, H, device=dev, dtype=torch.float32).mul_(0.02).to(bf) for _ in range(4)]
        a = torch.randn(m, H, device=dev).to(bf)
        if K.gemm_glu_fused(a, ws[0], "gelu_tanh") is None:
            return
        us = _time(lambda i: K.gemm_glu_fused(a, ws[i % 4], "gelu_tanh"), args.iters)
        report(f"{name} [{m}x{H}]x[{2 * I}x{H}]", us, 2 * I * H * 2 + m * H * 2 + m * I * 2, 4.0 * m * I * H)

    glu_case("gemm gate_up+glu decode", B)
    glu_case("gemm gate_up+glu prompt", args.prompt)

    # ------------------------------------------------------------------ small kernels
    for m, tag in ((B, "decode"), (args.prompt, "prompt")):
        if want(f"add_rmsnorm {tag}"):
            res = torch.randn(m, H, device=dev)
            br = torch.randn(m, H, device=dev).to(bf)
            w1, w2 = torch.randn(H, device=dev).to(bf), torch.randn(H, device=dev).to(bf)
            us = _time(lambda i: K.add_rmsnorm(res, br, (w1, 1e-6, 1.0), (w2, 1e-6, 1.0), bf), args.iters)
            report(f"add_rmsnorm {tag} [{m}x{H}]", us, m * H * (4 + 4 + 2 + 2))
        if m <= 64 and want(f"add_rmsnorm {tag} of partial sums"):
            for splits in (8, 16):                           # what the o and down products of a decode step leave
                res = torch.randn(m, H, device=dev)
                parts = K.SplitSum(torch.randn(splits, m, H, device=dev))
                w1, w2 = torch.randn(H, device=dev).to(bf), torch.randn(H, device=dev).to(bf)
                us = _time(lambda i: K.add_rmsnorm(res, parts, (w1, 1e-6, 1.0), (w2, 1e-6, 1.0), bf), args.iters)
                report(f"add_rmsnorm {tag} of partial sums [{splits}x{m}x{H}]", us, m * H * (4 * splits + 4 + 4 + 2))
        if want(f"glu {tag}"):
            x = torch.randn(m, 2 * I, device=dev).to(bf)
            us = _time(lambda i: K.glu(x, "gelu_tanh"), args.iters)
            report(f"glu {tag} [{m}x{2 * I}]", us, m * I * 6)

    # ------------------------------------------------------------------ attention over a paged cache
    page = 16
    ctx = args.history
    pages_per_seq = -(-(ctx + 1) // page)
    n_layers_rot = 2
    n_pages = B * pages_per_seq
    tables = [(torch.randn(n_pages, Hkv, page, D, device=dev).to(bf), torch.randn(n_pages, Hkv, page, D, device=dev).to(bf))
              for _ in range(n_layers_rot)]
    perm = torch.randperm(n_pages).to(torch.int32).reshape(B, pages_per_seq)
    bt = perm.to(dev)
    scale, cap = 1.0 / math.sqrt(D), 50.0

    def decode_case(window):
        name = f"attention decode window={window}"
        if not want(name):
            return
        q = torch.randn(B, Hq, D, device=dev).to(bf)
        rc = torch.full((B,), ctx + 1, dtype=torch.int32, device=dev)
        q_start, q_len = np.arange(B, dtype=np.int32), np.ones(B, np.int32)
        per_tile = max(1, K.attention_mma_rows(True) // (Hq // Hkv))
        tiles = tuple(torch.from_numpy(a).to(dev) for a in cut_tiles(q_start, q_len, per_tile))
        split, slots = decode_split(B * Hkv, ctx + 1, sm_count(dev), window, True)
        seen = min(ctx + 1, window) if window else ctx + 1
        us = _time(lambda i: K.paged_attention_mma(q, tables[i % 2][0], tables[i % 2][1], bt, rc, tiles, page, window, scale, cap,
                                                   Hq // Hkv, split, slots, True), args.iters)
        report(f"{name} split={split}x{slots}", us, B * seen * Hkv * D * 2 * 2)

    def decode_fused_case(window):
        """The same step from the q|k|v product's partial sums: the attention kernel adds up the slices,
        rotates and writes the cache's newest line itself. Beside it, the rotation kernel followed by
        the attention kernel over the same input."""
        name = f"attention decode from q|k|v slices window={window}"
        if not want(name):
            return
        splits = 9
        parts = K.SplitSum(torch.randn(splits, B, (Hq + 2 * Hkv) * D, device=dev) * 0.3)
        if not K.attention_decode_fused_takes(parts, Hq, Hkv, D, D, page, bf):
            return
        rc = torch.full((B,), ctx + 1, dtype=torch.int32, device=dev)
        cs = K.rope_table(torch.full((B,), ctx, dtype=torch.int32, device=dev), D, 10000.0)
        lines = (bt[:, ctx // page].to(torch.int64) * page + ctx % page).to(torch.int32)
        split, slots = decode_split(B * Hkv, ctx + 1, sm_count(dev), window, True)
        seen = min(ctx + 1, window) if window else ctx + 1
        tiles = tuple(torch.from_numpy(a).to(dev) for a in cut_tiles(np.arange(B, dtype=np.int32), np.ones(B, np.int32), 1))
        us = _time(lambda i: K.paged_attention_decode_fused(parts, cs, lines, tables[i % 2][0], tables[i % 2][1], bt, rc, Hq, Hkv, D,
                                                            True, page, window, scale, cap, split, slots), args.iters)
        nbytes = B * seen * Hkv * D * 2 * 2 + splits * B * (Hq + 2 * Hkv) * D * 4
        report(f"{name} split={split}x{slots}", us, nbytes)

        def two(i):
            q = K.rope_append(parts, cs, lines, tables[i % 2][0], tables[i % 2][1], Hq, Hkv, D, D, out_dtype=bf)
            return K.paged_attention_mma(q, tables[i % 2][0], tables[i % 2][1], bt, rc, tiles, page, window, scale, cap,
                                         Hq // Hkv, split, slots, True)

        report(f"rotation, then attention decode window={window} split={split}x{slots}", _time(two, args.iters), nbytes)

    decode_case(None)
    decode_case(args.window)
    decode_fused_case(None)
    decode_fused_case(args.window)

    def prompt_case(window):
        name = f"attention prompt window={window}"
        if not want(name):
            return
        t = args.prompt
        q = torch.randn(t, Hq, D, device=dev).to(bf)
        rc = torch.arange(1, t + 1, dtype=torch.int32, device=dev)
        per_tile = max(1, K.attention_tile_rows(False, K.attention_prompt_kernel(Hq, Hkv, D, page, cap), D) // (Hq // Hkv))
        tiles = tuple(torch.from_numpy(a).to(dev) for a in cut_tiles(np.zeros(1, np.int32), np.asarray([t], np.int32), per_tile))
        firsts = tiles[1].cpu().numpy() + 1
        split, slots = prompt_split(firsts, firsts + tiles[2].cpu().numpy() - 1, Hkv, sm_count(dev), window, t, Hq, D,
                                    prompt_costs_of(K.attention_prompt_kernel(Hq, Hkv, D, page, cap), D))
        pairs = sum(min(c, window) if window else c for c in range(1, t + 1))
        us = _time(lambda i: K.paged_attention_mma(q, tables[i % 2][0], tables[i % 2][1], bt, rc, tiles, page, window, scale, cap,
                                                   0, split, slots), max(3, args.iters // 4))
        report(f"{name} [{t} tokens] split={split}x{slots}", us, t * Hkv * D * 2 * 2 + 2 * t * Hq * D * 2, 4.0 * pairs * Hq * D)

    def portion_case(window):
        """The last `--prompt` tokens of a request of `--history` tokens: a portion of a long prompt,
        every row of which sees the history before it."""
        name = f"attention portion window={window}"
        if not want(name):
            return
        t = min(args.prompt, ctx)
        before = ctx - t
        q = torch.randn(t, Hq, D, device=dev).to(bf)
        rc = torch.arange(before + 1, ctx + 1, dtype=torch.int32, device=dev)
        per_tile = max(1, K.attention_tile_rows(False, K.attention_prompt_kernel(Hq, Hkv, D, page, cap), D) // (Hq // Hkv))
        tiles = tuple(torch.from_numpy(a).to(dev) for a in cut_tiles(np.zeros(1, np.int32), np.asarray([t], np.int32), per_tile))
        firsts = tiles[1].cpu().numpy() + before + 1
        split, slots = prompt_split(firsts, firsts + tiles[2].cpu().numpy() - 1, Hkv, sm_count(dev), window, t, Hq, D,
                                    prompt_costs_of(K.attention_prompt_kernel(Hq, Hkv, D, page, cap), D))
        pairs = sum(min(c, window) if window else c for c in range(before + 1, ctx + 1))
        seen = min(ctx, window + t) if window else ctx
        us = _time(lambda i: K.paged_attention_mma(q, tables[i % 2][0], tables[i % 2][1], bt, rc, tiles, page, window, scale, cap,
                                                   0, split, slots), max(3, args.iters // 4))
        report(f"{name} [{t} tokens behind {before}] split={split}x{slots}", us, seen * Hkv * D * 2 * 2 + 2 * t * Hq * D * 2, 4.0 * pairs * Hq * D)

    if args.prompt <= ctx:
        prompt_case(None)
        prompt_case(args.window)
    if args.prompt < ctx:
        portion_case(None)
        portion_case(args.window)

    if want("rope_append"):
        for m, tag in ((B, "decode"), (args.prompt, "prompt")):
            qkv = torch.randn(m, (Hq + 2 * Hkv) * D, device=dev).to(bf)
            pos = torch.arange(m, dtype=torch.int32, device=dev)
            cs = K.rope_table(pos, D, 10000.0)
            lines = torch.arange(m, dtype=torch.int32, device=dev)
            us = _time(lambda i: K.rope_append(qkv, cs, lines, tables[0][0], tables[0][1], Hq, Hkv, D, D), args.iters)
            report(f"rope_append {tag} [{m}]", us, m * (Hq + 2 * Hkv) * D * 4)
            if m <= 64:                                      # as a decode step has it: the q|k|v product's partial sums
                parts = K.SplitSum(torch.randn(9, m, (Hq + 2 * Hkv) * D, device=dev))
                us = _time(lambda i: K.rope_append(parts, cs, lines, tables[0][0], tables[0][1], Hq, Hkv, D, D, out_dtype=bf), args.iters)
                report(f"rope_append {tag} of partial sums [9x{m}]", us, m * (Hq + 2 * Hkv) * D * (4 * 9 + 2))
    for name, sampled in (("sample greedy", False), ("sample draw", True)):
        if want(name):
            c = min(copies(B * V * 4), 16)
            logits = [torch.randn(B, V, device=dev) for _ in range(c)]
            temps = torch.full((B,), 0.8, device=dev) if sampled else None
            us_ = torch.rand(B, device=dev) if sampled else None
            us = _time(lambda i: K.sample(logits[i % c], temps, us_), args.iters)
            report(f"{name} [{B}x{V}]", us, B * V * 4)
    return 0


if __name__ == "__main__":
    sys.exit(main())
