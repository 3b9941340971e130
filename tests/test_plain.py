"""The plain implementation checked against itself and against cases worked by hand
(the micro-cases of crates/kapel-ref/src/lib.rs:296-343 and the rules of crates/kapel-ops/src/paged.rs:16-25)."""
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gemma2 as P
from helpers import TINY, make_model_dir, rel_err


def test_rope_of_a_unit_vector():
    x = torch.zeros(1, 1, 4, dtype=torch.float64)
    x[0, 0, 0] = 1.0
    y = P.rope(x, torch.tensor([3]), 10000.0)
    # pair (0, 2) turns by 3 * 1; pair (1, 3) by 3 * 10000^(-1/2)
    assert torch.allclose(y[0, 0], torch.tensor([math.cos(3.0), 0.0, math.sin(3.0), 0.0], dtype=torch.float64))
    assert torch.allclose(P.rope(x, torch.tensor([0]), 10000.0), x)
    z = torch.randn(5, 2, 8, dtype=torch.float64)
    assert torch.allclose(P.rope(z, torch.arange(5), 5e5).norm(dim=-1), z.norm(dim=-1))


def test_norm_with_zero_weight_is_plain_rms():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.rms_norm(x, torch.zeros(2, dtype=torch.float64), 0.0)
    assert torch.allclose(y, x / math.sqrt(12.5))
    assert torch.allclose(P.rms_norm(x, torch.ones(2, dtype=torch.float64), 0.0), 2 * y)


def test_attention_first_query_window_edge_and_groups():
    t, hq, hkv, d = 6, 4, 2, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(t, h, d, generator=g, dtype=torch.float64) for h in (hq, hkv, hkv))
    y = P.attention(q, k, v, 0.3, None, None)
    assert torch.allclose(y[0, 0], v[0, 0]) and torch.allclose(y[0, 3], v[0, 1])      # the first query sees itself only
    # equal scores average the values
    y0 = P.attention(torch.zeros_like(q), k, v, 0.3, None, None)
    assert torch.allclose(y0[3, 1], v[:4, 0].mean(dim=0))
    # window 2: the query at position 4 sees positions 3 and 4 only
    yw = P.attention(torch.zeros_like(q), k, v, 0.3, None, 2)
    assert torch.allclose(yw[4, 2], v[3:5, 1].mean(dim=0))
    # a soft cap far below the scores makes them equal again
    yc = P.attention(q * 1e4, k, v, 1.0, 1e-9, None)
    assert torch.allclose(yc[5, 0], v[:6, 0].mean(dim=0), atol=1e-6)


def test_gelu_tanh_and_soft_cap_values():
    assert abs(float(P.gelu_tanh(torch.tensor(1.0, dtype=torch.float64))) - 0.8411919906082768) < 1e-12
    assert float(P.gelu_tanh(torch.tensor(0.0))) == 0.0


@pytest.mark.parametrize("name", ["A", "B"])
def test_32_bit_agrees_with_64_bit_and_a_prefix_is_a_prefix(name):
    raw, seed = TINY[name]
    folder = make_model_dir(raw, seed)
    cfg, w64 = P.load(folder, torch.float64)
    _, w32 = P.load(folder, torch.float32)
    ids = [int(t) for t in np.random.default_rng(3).integers(0, raw["vocab_size"], size=45)]
    l64 = P.forward(cfg, w64, ids).numpy()
    l32 = P.forward(cfg, w32, ids).double().numpy()
    assert rel_err(l32, l64) < 2e-5
    # causal: the logits of a prefix are the prefix of the logits
    assert rel_err(P.forward(cfg, w64, ids[:20]).numpy(), l64[:20]) < 1e-12
    # the window matters: without it the late logits change
    cfg2 = dict(cfg, sliding_window=None)
    assert rel_err(P.forward(cfg2, w64, ids).numpy()[-1], l64[-1]) > 1e-6


def test_golden_outputs_are_still_what_this_file_computes():
    """tests/golden/ holds small outputs of this implementation (made by tests/golden/make_golden.py):
    a change of the formulas shows here before it shows anywhere else."""
    path = Path(__file__).parent / "golden" / "plain_logits.json"
    golden = json.loads(path.read_text())
    for name, rec in golden.items():
        raw, seed = TINY[name]
        folder = make_model_dir(raw, seed)
        cfg, w = P.load(folder, torch.float64)
        logits = P.forward(cfg, w, rec["tokens"]).numpy()
        got = logits[-1][rec["columns"]]
        assert np.abs(got - np.array(rec["last_row"])).max() < 1e-9, name
        assert int(np.argmax(logits[-1])) == rec["argmax"]


def test_blocked_attention_equals_the_loop():
    """`attention_blocked` (matrix products over blocks of rows) against the loop of `attention`:
    groups of heads, a window's edge inside and across blocks, a soft cap, blocks that do not divide
    the length."""
    g = torch.Generator().manual_seed(1)
    for t, hq, hkv, d, window, cap, block in ((37, 4, 2, 8, None, 50.0, 16), (50, 6, 1, 16, 24, 20.0, 7),
                                              (33, 3, 3, 4, 5, None, 64), (20, 2, 1, 8, 1, 30.0, 3)):
        q, k, v = (torch.randn(t, h, d, generator=g, dtype=torch.float64) * 3 for h in (hq, hkv, hkv))
        want = P.attention(q, k, v, 0.25, cap, window)
        got = P.attention_blocked(q, k, v, 0.25, cap, window, block)
        assert (got - want).abs().max() < 1e-12, (t, hq, hkv, d, window, cap, block)


@pytest.mark.parametrize("name", ["A", "B"])
def test_streamed_forward_equals_the_whole_forward(name):
    """`forward_streamed` (a layer's weights at a time, blocked attention, logits at chosen places,
    several sequences in one pass over the file) against `forward` on the tiny configurations."""
    raw, seed = TINY[name]
    folder = make_model_dir(raw, seed)
    cfg, w = P.load(folder, torch.float64)
    rng = np.random.default_rng(4)
    a = [int(t) for t in rng.integers(0, raw["vocab_size"], size=70)]
    b = [int(t) for t in rng.integers(0, raw["vocab_size"], size=9)]
    want_a, want_b = [0, 15, 16, 17, 69], [8]
    got = P.forward_streamed(folder, [(a, want_a, None), (b, want_b, 9.8125)], block=13)
    assert rel_err(got[0].numpy(), P.forward(cfg, w, a).numpy()[want_a]) < 1e-12
    assert rel_err(got[1].numpy(), P.forward(cfg, w, b, embed_scale=9.8125).numpy()[want_b]) < 1e-12
