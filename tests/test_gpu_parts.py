"""Each part of a layer alone, built from its spec, against the plain function of the same part."""
import math

import numpy as np
import pytest
import torch

import plain_gemma2 as P
from helpers import rel_err

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def ctx_for(dtype):
    from kapel_b200.parts import BuildContext

    return BuildContext(dtype=DT[dtype], device=torch.device("cuda"), page_size=16)


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).bfloat16()


def plan_batch(manager, entries, chunk):
    """A StepBatch for [(sequence, count)] with sequences added as needed."""
    from kapel_b200.engine.batch import StepBatch

    for s, _ in entries:
        if s not in manager:
            manager.add_sequence(s)
    plan = manager.plan(entries)
    batch = StepBatch(plan, [0] * plan.rows, list(range(plan.rows)), torch.device("cuda"), chunk)
    return plan, batch


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    from kapel_b200.config import NormSpec
    from kapel_b200.parts import build_part

    spec = NormSpec(width=100, eps=1e-5, offset=1.0, weight="n.weight")
    part = build_part("norm", spec, ctx_for(dtype))
    assert type(part).expected_tensors(spec) == {"n.weight": (100,)}
    w = rnd(100, seed=1, scale=0.1)
    part.load({"n.weight": w.cuda()})
    x = rnd(6, 100, seed=2, scale=2.0).float()
    got = part.forward(x.cuda()).cpu().double()
    assert got.dtype == torch.float64 and rel_err(got.numpy(), P.rms_norm(x.double(), w.double(), 1e-5).numpy()) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_mlp_part(dtype):
    from kapel_b200.config import GatedMLPSpec
    from kapel_b200.parts import build_part

    spec = GatedMLPSpec(hidden=72, intermediate=200, activation="gelu_tanh", weights={"gate": "g", "up": "u", "down": "d"})
    part = build_part("feed_forward", spec, ctx_for(dtype))
    assert type(part).expected_tensors(spec) == {"g": (200, 72), "u": (200, 72), "d": (72, 200)}
    w = {"g": rnd(200, 72, seed=3, scale=0.2), "u": rnd(200, 72, seed=4, scale=0.2), "d": rnd(72, 200, seed=5, scale=0.2)}
    part.load({k: v.cuda() for k, v in w.items()})
    h = rnd(9, 72, seed=6)
    got = part.forward(h.cuda().to(DT[dtype])).cpu().double()
    want = P.geglu_ffn(h.double(), w["g"].double(), w["u"].double(), w["d"].double())
    assert rel_err(got.numpy(), want.numpy()) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [None, 20])
def test_attention_part_whole_then_in_portions(dtype, window):
    from kapel_b200 import kernels as K
    from kapel_b200.cache import CacheManager
    from kapel_b200.config import AttentionSpec, PositionSpec
    from kapel_b200.parts import LayerCache, build_part

    hidden, hq, hkv, d, t = 48, 6, 2, 32, 50
    spec = AttentionSpec(hidden=hidden, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=1 / math.sqrt(40.0), softcap=25.0,
                         window=window, position=PositionSpec(theta=5e4, rotary_dim=d), weights={"q": "q", "k": "k", "v": "v", "o": "o"})
    part = build_part("mixer", spec, ctx_for(dtype))
    w = {"q": rnd(hq * d, hidden, seed=7, scale=0.3), "k": rnd(hkv * d, hidden, seed=8, scale=0.3),
         "v": rnd(hkv * d, hidden, seed=9, scale=0.3), "o": rnd(hidden, hq * d, seed=10, scale=0.3)}
    part.load({k_: v_.cuda() for k_, v_ in w.items()})
    h = rnd(t, hidden, seed=11)

    # the plain mixer on the whole sequence
    cfg = dict(num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, hidden_size=hidden, rope_theta=5e4,
               query_pre_attn_scalar=40.0, attn_logit_softcapping=25.0)
    names = {f"L.self_attn.{n}_proj.weight": w[n].double() for n in "qkvo"}
    want = P.attention_mixer(h.double(), torch.arange(t), names, "L", cfg, window).numpy()

    def alloc(shape, dt):
        return torch.zeros(shape, dtype=dt, device="cuda")

    for cuts in ([t], [7, 2, 25, 1, 15]):
        manager = CacheManager({0: part.cache_needs()}, 16, 8, 2, allocate=alloc, dtype=DT[dtype])
        cache = LayerCache(manager, 0, owns=True)
        outs, at = [], 0
        for n in cuts:
            plan, batch = plan_batch(manager, [("s", n)], K.attention_chunk())
            outs.append(part.forward(h[at : at + n].cuda().to(DT[dtype]), batch, cache).cpu().double())
            manager.commit(plan)
            at += n
        assert rel_err(torch.cat(outs).numpy(), want) < TOL[dtype], f"cuts {cuts}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["sandwich", "prenorm"])
def test_block_part(dtype, kind):
    from kapel_b200 import kernels as K
    from kapel_b200.cache import CacheManager
    from kapel_b200.config import AttentionSpec, BlockSpec, GatedMLPSpec, NormSpec, PositionSpec
    from kapel_b200.parts import LayerCache, build_part, part_class

    hidden, hq, hkv, d, inter, t, eps = 40, 2, 1, 16, 88, 21, 1e-5
    p = "model.layers.0"
    mixer = AttentionSpec(hidden=hidden, num_heads=hq, num_kv_heads=hkv, head_dim=d, scale=0.25, softcap=None, window=None,
                          position=PositionSpec(theta=1e4, rotary_dim=d),
                          weights={n: f"{p}.self_attn.{n}_proj.weight" for n in "qkvo"})
    ffn = GatedMLPSpec(hidden=hidden, intermediate=inter, activation="gelu_tanh",
                       weights={n: f"{p}.mlp.{n}_proj.weight" for n in ("gate", "up", "down")})
    roles = {"pre_mixer": "input_layernorm", "post_mixer": "post_attention_layernorm", "pre_ffn": "pre_feedforward_layernorm",
             "post_ffn": "post_feedforward_layernorm"}
    if kind == "prenorm":
        roles = {k: v for k, v in roles.items() if k.startswith("pre")}
    norms = {r: NormSpec(width=hidden, eps=eps, offset=1.0, weight=f"{p}.{n}.weight") for r, n in roles.items()}
    spec = BlockSpec(kind=kind, mixer=mixer, ffn=ffn, norms=norms)
    expected = part_class("block", kind).expected_tensors(spec)
    tensors = {n: rnd(*s, seed=i, scale=0.1 if len(s) == 1 else 0.3) for i, (n, s) in enumerate(sorted(expected.items()))}
    block = build_part("block", spec, ctx_for(dtype))
    block.load({n: v.cuda() for n, v in tensors.items()})
    x = rnd(t, hidden, seed=50).float()
    w = {n: v.double() for n, v in tensors.items()}
    cfg = dict(num_attention_heads=hq, num_key_value_heads=hkv, head_dim=d, hidden_size=hidden, rope_theta=1e4,
               query_pre_attn_scalar=16.0, rms_norm_eps=eps)
    if kind == "sandwich":
        want = P.sandwich_block(x.double(), torch.arange(t), w, p, cfg, None)
    else:
        xd = x.double()
        a = P.attention_mixer(P.rms_norm(xd, w[f"{p}.input_layernorm.weight"], eps), torch.arange(t), w, p, cfg, None)
        xd = xd + a
        hh = P.rms_norm(xd, w[f"{p}.pre_feedforward_layernorm.weight"], eps)
        want = xd + P.geglu_ffn(hh, w[f"{p}.mlp.gate_proj.weight"], w[f"{p}.mlp.up_proj.weight"], w[f"{p}.mlp.down_proj.weight"])

    manager = CacheManager({0: block.mixer.cache_needs()}, 16, 4, 2,
                           allocate=lambda s, dt: torch.zeros(s, dtype=dt, device="cuda"), dtype=DT[dtype])
    plan, batch = plan_batch(manager, [("s", t)], K.attention_chunk())
    xr = x.cuda().clone()
    out, h_next = block.forward(xr, None, batch, LayerCache(manager, 0, True), block.norms["pre_mixer"])
    assert out.data_ptr() == xr.data_ptr(), "the residual is updated in place"
    assert rel_err(out.cpu().double().numpy(), want.numpy()) < TOL[dtype]
    nxt = P.rms_norm(want, w[f"{p}.input_layernorm.weight"], eps)
    assert rel_err(h_next.cpu().double().numpy(), nxt.numpy()) < TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_head_parts(dtype):
    from kapel_b200.config import EmbedSpec, HeadSpec
    from kapel_b200.parts import build_part

    table = rnd(300, 56, seed=60, scale=0.5)
    emb = build_part("embedding", EmbedSpec(weight="t", scale=math.sqrt(56.0)), ctx_for(dtype))
    emb.load({"t": table.cuda()})
    ids = torch.tensor([3, 299, 0], dtype=torch.int32)
    scale = float(torch.tensor(math.sqrt(56.0)).to(DT[dtype]).float())
    assert emb.scale == scale
    got = emb.forward(ids.cuda()).cpu().double()
    assert rel_err(got.numpy(), (table.double()[ids.long()] * scale).numpy()) < 1e-6
    head = build_part("head", HeadSpec(weight="t", softcap=5.0), ctx_for(dtype))
    head.load({"t": table.cuda()})
    h = rnd(4, 56, seed=61)
    logits = head.forward(h.cuda().to(DT[dtype])).cpu()
    assert logits.dtype == torch.float32
    want = 5.0 * torch.tanh((h.double() @ table.double().T) / 5.0)
    assert rel_err(logits.double().numpy(), want.numpy()) < (1e-5 if dtype == "float32" else 1e-4)


def test_a_weight_stored_in_32_bit_stays_so_on_the_bfloat16_path():
    from kapel_b200.config import GatedMLPSpec
    from kapel_b200.parts import build_part

    spec = GatedMLPSpec(hidden=24, intermediate=40, activation="silu", weights={"gate": "g", "up": "u", "down": "d"})
    part = build_part("feed_forward", spec, ctx_for("bfloat16"))
    w = {k: torch.randn(s, generator=torch.Generator().manual_seed(i)) * 0.3 for i, (k, s) in enumerate({"g": (40, 24), "u": (40, 24), "d": (24, 40)}.items())}
    part.load({k: v.cuda() for k, v in w.items()})
    assert part.w_gate_up.dtype == torch.float32 and part.w_down.dtype == torch.float32
    h = rnd(5, 24, seed=70)
    got = part.forward(h.cuda()).cpu().double()
    g, u = h.double() @ w["g"].double().T, h.double() @ w["u"].double().T
    want = ((g * torch.sigmoid(g)) * u) @ w["d"].double().T
    assert rel_err(got.numpy(), want.numpy()) < 2e-2
