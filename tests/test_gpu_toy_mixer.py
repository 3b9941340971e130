"""A toy mixer with state of its own, a toy architecture and a schedule that shares a cache:
registered, built and stepped from this file alone, with no change to the package's files.

The toy mixer keeps one vector per request in a slot: s_t = decay * s_(t-1) + W_in h_t, and
gives W_out s_t. The toy model runs it in a prenorm block, then a sandwich attention layer,
then another attention layer that reads the second layer's keys and values.
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
class ToyStateSpec:
    hidden: int
    width: int
    decay: float
    weights: dict
    kind: str = "toy_state"


def make_toy_parts():
    from kapel_b200 import kernels as K
    from kapel_b200.cache import CacheNeeds, StateSpec
    from kapel_b200.parts import Part, linear, matrix_for

    class ToyStateMixer(Part):
        @staticmethod
        def expected_tensors(spec):
            return {spec.weights["in"]: (spec.width, spec.hidden), spec.weights["out"]: (spec.hidden, spec.width)}

        def load(self, tensors):
            self.w_in = matrix_for(self.ctx, tensors[self.spec.weights["in"]])
            self.w_out = matrix_for(self.ctx, tensors[self.spec.weights["out"]])

        def cache_needs(self):
            return CacheNeeds(state=StateSpec((self.spec.width,)))

        def forward(self, h, batch, cache):
            u = linear(self.ctx, h, self.w_in, out_dtype=torch.float32)      # [rows, width]
            table = cache.state()                                            # [slots + 1, width] float32
            out = torch.empty_like(u)
            plan = batch.plan
            for e in range(len(plan.entries)):                               # rows of a request in order
                slot, r0, n = int(plan.slots[e]), int(plan.q_start[e]), int(plan.q_len[e])
                s = table[slot]
                for r in range(r0, r0 + n):
                    s = self.spec.decay * s + u[r]
                    out[r] = s
                table[slot] = s
            return linear(self.ctx, K.cast(out, self.ctx.dtype), self.w_out)

    return ToyStateMixer


class ToyConfig:
    architecture = "ToyStateForCausalLM"

    def __init__(self, raw):
        self.raw = dict(raw)

    @classmethod
    def from_json(cls, raw):
        return cls(raw)

    def to_json(self):
        return dict(self.raw, architectures=[self.architecture])

    def init_std(self, name, shape):
        return 0.1 if len(shape) == 1 else 0.08

    def to_spec(self):
        from kapel_b200.config import (AttentionSpec, BlockSpec, EmbedSpec, GatedMLPSpec, HeadSpec, ModelSpec, NormSpec,
                                       PositionSpec, ScheduleEntry)

        r = self.raw
        h = r["hidden"]
        norm = lambda n: NormSpec(width=h, eps=r["eps"], offset=1.0, weight=n)
        ffn = lambda p: GatedMLPSpec(hidden=h, intermediate=r["inter"], activation="silu",
                                     weights={k: f"{p}.ffn.{k}" for k in ("gate", "up", "down")})
        att = lambda p, window: AttentionSpec(hidden=h, num_heads=r["heads"], num_kv_heads=r["kv_heads"], head_dim=r["head_dim"],
                                              scale=1 / math.sqrt(r["head_dim"]), softcap=None, window=window,
                                              position=PositionSpec(theta=r["theta"], rotary_dim=r["head_dim"]),
                                              weights={k: f"{p}.att.{k}" for k in "qkvo"})
        toy = ToyStateSpec(hidden=h, width=r["state"], decay=r["decay"], weights={"in": "l0.toy.in", "out": "l0.toy.out"})
        layers = (
            BlockSpec(kind="prenorm", mixer=toy, ffn=ffn("l0"), norms={"pre_mixer": norm("l0.n1"), "pre_ffn": norm("l0.n2")}),
            BlockSpec(kind="sandwich", mixer=att("l1", None), ffn=ffn("l1"),
                      norms={k: norm(f"l1.{k}") for k in ("pre_mixer", "post_mixer", "pre_ffn", "post_ffn")}),
            BlockSpec(kind="prenorm", mixer=att("l2", None), ffn=ffn("l2"), norms={"pre_mixer": norm("l2.n1"), "pre_ffn": norm("l2.n2")}),
        )
        # layer 2 reads layer 1's keys and values and writes none
        schedule = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 1))
        return ModelSpec(architecture=self.architecture, vocab_size=r["vocab"], hidden_size=h,
                         embed=EmbedSpec(weight="embed", scale=1.0, round_scale=False), layers=layers, schedule=schedule,
                         final_norm=norm("final"), head=HeadSpec(weight="embed", softcap=None), max_positions=None)


RAW = dict(hidden=48, inter=72, heads=4, kv_heads=2, head_dim=16, state=24, decay=0.9, theta=1e4, eps=1e-5, vocab=200)


def plain_toy(w, ids):
    """The toy model on a whole sequence, in 64-bit."""
    r = RAW
    t = len(ids)
    pos = torch.arange(t)
    x = w["embed"][torch.tensor(ids)]

    def ffn(p, h):
        g = h @ w[f"{p}.ffn.gate"].T
        return ((g * torch.sigmoid(g)) * (h @ w[f"{p}.ffn.up"].T)) @ w[f"{p}.ffn.down"].T

    def qkv(p, h):
        q = P.rope((h @ w[f"{p}.att.q"].T).reshape(t, r["heads"], r["head_dim"]), pos, r["theta"])
        k = P.rope((h @ w[f"{p}.att.k"].T).reshape(t, r["kv_heads"], r["head_dim"]), pos, r["theta"])
        v = (h @ w[f"{p}.att.v"].T).reshape(t, r["kv_heads"], r["head_dim"])
        return q, k, v

    n = lambda name, v: P.rms_norm(v, w[name], r["eps"])
    # layer 0: the toy mixer
    u = n("l0.n1", x) @ w["l0.toy.in"].T
    s, outs = torch.zeros(r["state"], dtype=torch.float64), []
    for i in range(t):
        s = r["decay"] * s + u[i]
        outs.append(s)
    x = x + torch.stack(outs) @ w["l0.toy.out"].T
    x = x + ffn("l0", n("l0.n2", x))
    # layer 1: sandwich attention
    q, k1, v1 = qkv("l1", n("l1.pre_mixer", x))
    a = P.attention(q, k1, v1, 1 / math.sqrt(r["head_dim"]), None, None).reshape(t, -1) @ w["l1.att.o"].T
    x = x + n("l1.post_mixer", a)
    x = x + n("l1.post_ffn", ffn("l1", n("l1.pre_ffn", x)))
    # layer 2: attention over layer 1's keys and values
    q, _, _ = qkv("l2", n("l2.n1", x))
    a = P.attention(q, k1, v1, 1 / math.sqrt(r["head_dim"]), None, None).reshape(t, -1) @ w["l2.att.o"].T
    x = x + a
    x = x + ffn("l2", n("l2.n2", x))
    return (n("final", x) @ w["embed"].T).numpy()


@pytest.fixture()
def registered():
    from kapel_b200.config import register_architecture, unregister_architecture
    from kapel_b200.parts import register_mixer, unregister_part

    register_mixer("toy_state", make_toy_parts())
    register_architecture(ToyConfig, ToyConfig.architecture)
    yield
    unregister_part("mixer", "toy_state")
    unregister_architecture(ToyConfig.architecture)


@pytest.mark.parametrize("dtype,tol", [("float32", 2e-5), ("bfloat16", 5e-2)])
def test_toy_architecture_is_registered_built_and_stepped(registered, dtype, tol, tmp_path):
    from kapel_b200.config import config_from_dir
    from kapel_b200.engine import Engine
    from kapel_b200.weights import write_random_model

    folder = write_random_model(tmp_path / "toy", ToyConfig(RAW), seed=3)
    config, _ = config_from_dir(folder)
    assert isinstance(config, ToyConfig)
    engine = Engine.from_dir(folder, dtype=dtype, max_tokens=256, max_sequences=4)
    assert len(engine.cache.groups) == 1 and engine.cache.group_of_layer == {1: 0}, "layers 1 and 2 share one cache"
    assert list(engine.cache.states) == [0]
    w = P.read_safetensors(folder / "model.safetensors")
    rng = np.random.default_rng(0)
    reqs = {"a": random_tokens(rng, 40, RAW["vocab"]), "b": random_tokens(rng, 23, RAW["vocab"])}
    plain = {k: plain_toy(w, v) for k, v in reqs.items()}

    tb = TraceBuilder()
    a, b = reqs["a"], reqs["b"]
    tb.step([("a", a[:9], range(9))])
    tb.step([("a", a[9:11], range(2)), ("b", b[:20], range(20))])
    tb.step([("a", a[11:30], range(19)), ("b", b[20:21], [0])])
    for i in range(30, 40):
        entries = [("a", a[i : i + 1], [0])]
        if i - 9 < len(b):
            entries.append(("b", b[i - 9 : i - 8], [0]))
        tb.step(entries, end=(["a"] if i == 39 else []))
    got = run_trace_engine(engine, tb.steps)
    worst = 0.0
    for step, rows in tb.rows.items():
        for i, (rid, pos) in enumerate(rows):
            err = rel_err(got[step][i], plain[rid][pos])
            worst = max(worst, err)
            assert err < tol, f"step {step} request {rid} position {pos}: {err:.2e}"
    print(f"toy {dtype}: worst {worst:.2e}")
    # a slot that is used again starts from a cleared state
    engine.end("b")
    tb2 = TraceBuilder()
    tb2.step([("c", a[:12], range(12))], end=["c"])
    got = run_trace_engine(engine, tb2.steps)
    assert rel_err(got[0], plain["a"][:12]) < tol
