"""A long prompt in portions over a window much shorter than the prompt, then decoding: the
tensor-core prompt kernels with a long history behind a short portion (key slots, a window's edge
inside a tile, pages of the windowed group given back and used again), at a head size that the
tcgen05 kernel takes, against the plain implementation.
"""
import numpy as np
import pytest

from helpers import TOL, TraceBuilder, compare_trace, embed_scale_for, make_model_dir, plain_logits, random_tokens, run_trace_engine

pytestmark = pytest.mark.gpu

RAW = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2",
    num_hidden_layers=2, hidden_size=128, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
    intermediate_size=256, vocab_size=512, rope_theta=10000.0, sliding_window=1000,
    query_pre_attn_scalar=64, attn_logit_softcapping=30.0, final_logit_softcapping=30.0,
    rms_norm_eps=1e-6, hidden_activation="gelu_pytorch_tanh", tie_word_embeddings=True,
    max_position_embeddings=8192,
)


@pytest.fixture(scope="module")
def case():
    folder = make_model_dir(RAW, seed=9)
    rng = np.random.default_rng(31)
    reqs = {"a": random_tokens(rng, 2600, RAW["vocab_size"]), "b": random_tokens(rng, 900, RAW["vocab_size"])}
    plain = {dtype: {rid: plain_logits(folder, toks, embed_scale=embed_scale_for(RAW, dtype)) for rid, toks in reqs.items()}
             for dtype in ("float32", "bfloat16")}
    return folder, reqs, plain


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompt_in_portions_over_a_short_window(case, dtype):
    from kapel_b200.engine import Engine

    folder, reqs, plain = case
    # The global group holds everything (2,600 + 900 positions in 224 pages); the windowed group gives
    # back what has left the window, and its pool hands the pages given back last out first.
    engine = Engine.from_dir(folder, dtype=dtype, max_tokens=3584, max_sequences=4)
    a, b = reqs["a"], reqs["b"]
    tb = TraceBuilder()
    at = 0
    for n in (700, 64, 513, 2, 300, 800, 130):           # a's prompt in portions of changing size, b's beside it
        entries = [("a", a[at : at + n], [0, n - 1])]
        if at == 700:
            entries.append(("b", b[:450], [449]))
        if at == 764:
            entries.append(("b", b[450:890], [0, 439]))
        tb.step(entries)
        at += n
    assert at == 2509
    for i in range(10):                                   # then both decode
        entries = [("b", [b[890 + i]], [0])]
        entries.append(("a", [a[at + i]], [0]))
        tb.step(entries, end=(["b"] if i == 9 else []))
    tb.step([("a", a[at + 10 : 2600], [2600 - at - 11])], end=["a"])
    got = run_trace_engine(engine, tb.steps)
    worst = compare_trace(got, tb, plain[dtype], TOL[dtype], f"long {dtype}")
    print(f"long {dtype}: worst {worst:.2e}, pages given back by the window: {engine.cache.released_pages}")
    assert engine.cache.released_pages >= 100           # (2,600 - 1,000) / 16
    engine.cache.check()
    assert engine.cache.free_pages() == engine.cache.total_pages()
