"""A toy feed-forward with routing and a toy position encoding, registered, built and stepped from
this file alone: neither is a part of any real model, and the package's files are not touched.

The routed feed-forward sends each row to the one of its experts whose router logit (32-bit) is
largest and scales the expert's output by the softmax weight of that logit. The position
encoding rotates like RoPE but with frequencies 1 / (1 + j) and positions divided by a factor: it
only has to give the mixer the table its kernels take. The toy model puts both in its first layer
and the package's own rope and gated feed-forward in its second.
"""
import math
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_gemma2 as P
from helpers import TraceBuilder, random_tokens, rel_err, run_trace_engine

pytestmark = pytest.mark.gpu


@dataclass(frozen=True)
class ToyRoutedSpec:
    hidden: int
    inner: int
    experts: int
    weights: dict                      # "router", and "in.{e}", "out.{e}" for each expert
    kind: str = "toy_routed"


@dataclass(frozen=True)
class ToyPositionSpec:
    rotary_dim: int
    factor: float
    kind: str = "toy_harmonic"
    theta: float = 0.0                 # unused; attention specs print it


def make_parts():
    from kapel_b200 import kernels as K
    from kapel_b200.parts import Part, linear, matrix_for

    class ToyRoutedFeedForward(Part):
        @staticmethod
        def expected_tensors(spec):
            out = {spec.weights["router"]: (spec.experts, spec.hidden)}
            for e in range(spec.experts):
                out[spec.weights[f"in.{e}"]] = (spec.inner, spec.hidden)
                out[spec.weights[f"out.{e}"]] = (spec.hidden, spec.inner)
            return out

        def load(self, tensors):
            w = self.spec.weights
            self.router = tensors[w["router"]].float()                     # router logits are 32-bit on both paths
            self.w_in = [matrix_for(self.ctx, tensors[w[f"in.{e}"]]) for e in range(self.spec.experts)]
            self.w_out = [matrix_for(self.ctx, tensors[w[f"out.{e}"]]) for e in range(self.spec.experts)]

        def forward(self, h):
            logits = K.gemm(K.cast(h, torch.float32), self.router)           # [rows, experts], true 32-bit
            weight, chosen = torch.softmax(logits, dim=-1).max(dim=-1)
            out = torch.zeros((h.shape[0], self.spec.hidden), dtype=torch.float32, device=h.device)
            for e in range(self.spec.experts):
                rows = torch.nonzero(chosen == e).flatten()
                if rows.numel() == 0:
                    continue
                inner = torch.relu(linear(self.ctx, h[rows].contiguous(), self.w_in[e]).float())
                y = linear(self.ctx, K.cast(inner, self.ctx.dtype), self.w_out[e], out_dtype=torch.float32)
                out[rows] = y * weight[rows, None]
            return K.cast(out, self.ctx.dtype)

    class ToyHarmonicPosition(Part):
        @property
        def rotary_dim(self):
            return self.spec.rotary_dim

        def tables(self, batch):
            key = ("toy_harmonic", self.spec.rotary_dim, self.spec.factor)
            if key not in batch.memo:
                half = self.spec.rotary_dim // 2
                freq = 1.0 / (1.0 + torch.arange(half, dtype=torch.float64, device=batch.positions.device))
                angle = batch.positions.double()[:, None] / self.spec.factor * freq[None, :]
                batch.memo[key] = torch.stack([angle.cos(), angle.sin()], dim=-1).float().contiguous()
            return batch.memo[key]

    return ToyRoutedFeedForward, ToyHarmonicPosition


class ToyConfig:
    architecture = "ToyRoutedForCausalLM"

    def __init__(self, raw):
        self.raw = dict(raw)

    @classmethod
    def from_json(cls, raw):
        return cls(raw)

    def to_json(self):
        return dict(self.raw, architectures=[self.architecture])

    def init_std(self, name, shape):
        if name.endswith("router"):
            return 1.0                  # clear margins between the experts
        return 0.1 if len(shape) == 1 else 0.08

    def to_spec(self):
        from kapel_b200.config import (AttentionSpec, BlockSpec, EmbedSpec, GatedMLPSpec, HeadSpec, ModelSpec, NormSpec,
                                       PositionSpec, ScheduleEntry)

        r = self.raw
        h = r["hidden"]
        norm = lambda n: NormSpec(width=h, eps=r["eps"], offset=1.0, weight=n)
        att = lambda p, position, window: AttentionSpec(
            hidden=h, num_heads=r["heads"], num_kv_heads=r["kv_heads"], head_dim=r["head_dim"], scale=1 / math.sqrt(r["head_dim"]),
            softcap=None, window=window, position=position, weights={k: f"{p}.att.{k}" for k in "qkvo"})
        routed = ToyRoutedSpec(hidden=h, inner=r["inner"], experts=r["experts"],
                               weights=dict({"router": "l0.moe.router"},
                                            **{f"{io}.{e}": f"l0.moe.{io}.{e}" for io in ("in", "out") for e in range(r["experts"])}))
        gated = GatedMLPSpec(hidden=h, intermediate=r["inter"], activation="gelu_tanh",
                             weights={k: f"l1.ffn.{k}" for k in ("gate", "up", "down")})
        layers = (
            BlockSpec(kind="prenorm", mixer=att("l0", ToyPositionSpec(rotary_dim=r["rotary"], factor=r["factor"]), None), ffn=routed,
                      norms={"pre_mixer": norm("l0.n1"), "pre_ffn": norm("l0.n2")}),
            BlockSpec(kind="prenorm", mixer=att("l1", PositionSpec(theta=r["theta"], rotary_dim=r["head_dim"]), r["window"]), ffn=gated,
                      norms={"pre_mixer": norm("l1.n1"), "pre_ffn": norm("l1.n2")}),
        )
        return ModelSpec(architecture=self.architecture, vocab_size=r["vocab"], hidden_size=h,
                         embed=EmbedSpec(weight="embed", scale=1.0, round_scale=False), layers=layers,
                         schedule=(ScheduleEntry(0, 0), ScheduleEntry(1, 1)), final_norm=norm("final"),
                         head=HeadSpec(weight="embed", softcap=None), max_positions=None)


RAW = dict(hidden=48, inner=40, experts=3, inter=72, heads=4, kv_heads=2, head_dim=16, rotary=8, factor=2.5, theta=1e4, window=20,
           eps=1e-5, vocab=200)


def plain_toy(w, ids):
    """The toy model on a whole sequence in 64-bit; also the smallest router margin."""
    r = RAW
    t = len(ids)
    pos = torch.arange(t)
    x = w["embed"][torch.tensor(ids)]
    n = lambda name, v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + r["eps"]) * (1.0 + w[name])

    def harmonic(v):                                     # [t, heads, d]: the first `rotary` components rotate
        half = r["rotary"] // 2
        freq = 1.0 / (1.0 + torch.arange(half, dtype=torch.float64))
        ang = pos.double()[:, None] / r["factor"] * freq[None, :]
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        a, b = v[..., :half], v[..., half : 2 * half]
        return torch.cat([a * c - b * s, b * c + a * s, v[..., 2 * half :]], dim=-1)

    def heads(p, hh, rot):
        q = rot((hh @ w[f"{p}.att.q"].T).reshape(t, r["heads"], r["head_dim"]))
        k = rot((hh @ w[f"{p}.att.k"].T).reshape(t, r["kv_heads"], r["head_dim"]))
        v = (hh @ w[f"{p}.att.v"].T).reshape(t, r["kv_heads"], r["head_dim"])
        return q, k, v

    scale = 1 / math.sqrt(r["head_dim"])
    q, k, v = heads("l0", n("l0.n1", x), harmonic)
    x = x + P.attention(q, k, v, scale, None, None).reshape(t, -1) @ w["l0.att.o"].T
    hh = n("l0.n2", x)
    logits = hh @ w["l0.moe.router"].T
    top = torch.sort(logits, dim=-1).values
    margin = float((top[:, -1] - top[:, -2]).min())
    weight, chosen = torch.softmax(logits, dim=-1).max(dim=-1)
    y = torch.zeros_like(x)
    for i in range(t):
        e = int(chosen[i])
        y[i] = weight[i] * (torch.relu(hh[i] @ w[f"l0.moe.in.{e}"].T) @ w[f"l0.moe.out.{e}"].T)
    x = x + y
    q, k, v = heads("l1", n("l1.n1", x), lambda z: P.rope(z, pos, r["theta"]))
    x = x + P.attention(q, k, v, scale, None, r["window"]).reshape(t, -1) @ w["l1.att.o"].T
    hh = n("l1.n2", x)
    x = x + (P.gelu_tanh(hh @ w["l1.ffn.gate"].T) * (hh @ w["l1.ffn.up"].T)) @ w["l1.ffn.down"].T
    return (n("final", x) @ w["embed"].T).numpy(), margin


@pytest.fixture()
def registered():
    from kapel_b200.config import register_architecture, unregister_architecture
    from kapel_b200.parts import register_feed_forward, register_position, unregister_part

    routed, position = make_parts()
    register_feed_forward("toy_routed", routed)
    register_position("toy_harmonic", position)
    register_architecture(ToyConfig, ToyConfig.architecture)
    yield
    unregister_part("feed_forward", "toy_routed")
    unregister_part("position", "toy_harmonic")
    unregister_architecture(ToyConfig.architecture)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 5e-2)])
def test_toy_routed_feed_forward_and_toy_position_are_registered_built_and_stepped(registered, dtype, tol, tmp_path):
    from kapel_b200.engine import Engine
    from kapel_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "toy", ToyConfig(RAW), seed=6)
    engine = Engine.from_dir(folder, dtype=dtype, max_tokens=256, max_sequences=4)
    w = P.read_safetensors(folder / "model.safetensors")
    rng = np.random.default_rng(7)          # with these weights and tokens the smallest router margin is 0.74
    reqs = {"a": random_tokens(rng, 45, RAW["vocab"]), "b": random_tokens(rng, 26, RAW["vocab"])}
    plain, margins = {}, []
    for key, ids in reqs.items():
        plain[key], m = plain_toy(w, ids)
        margins.append(m)
    if dtype == "bfloat16" and min(margins) < 0.05:
        pytest.skip(f"a router margin of {min(margins):.3f} is within bfloat16's error of a tie")

    a, b = reqs["a"], reqs["b"]
    tb = TraceBuilder()
    tb.step([("a", a[:17], range(17))])
    tb.step([("a", a[17:19], range(2)), ("b", b[:20], range(20))])
    tb.step([("a", a[19:35], range(16)), ("b", b[20:21], [0])])
    for i in range(35, 45):
        entries = [("a", a[i : i + 1], [0])]
        if i - 14 < len(b):
            entries.append(("b", b[i - 14 : i - 13], [0]))
        tb.step(entries, end=(["a"] if i == 44 else []))
    got = run_trace_engine(engine, tb.steps)
    worst = 0.0
    for step, rows in tb.rows.items():
        for i, (rid, pos) in enumerate(rows):
            err = rel_err(got[step][i], plain[rid][pos])
            worst = max(worst, err)
            assert err < tol, f"step {step} request {rid} position {pos}: {err:.2e}"
    print(f"toy routed {dtype}: worst {worst:.2e}, smallest router margin {min(margins):.3f}")
    engine.end("b")
    assert engine.cache.free_pages() == engine.cache.total_pages()
