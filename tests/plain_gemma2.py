"""A plain, slow Gemma 2 forward pass: whole sequences, no cache, one function a part.

It rests on the formulas of smallbard/kapel's sources, cited at each function by the file's
path within that project and its lines. Kapel's own model code is Rust and cannot be compiled
here (no Rust toolchain, no network for its dependencies), so this file rests on the formulas
alone; `tests/golden/` holds outputs of this file, not of Kapel.

It shares no code with `kapel_b200`: it reads config.json and model.safetensors with its own
few lines, and uses torch on the CPU only as an array library. Everything is computed in the
dtype given (`torch.float64` by default, as kapel-ref computes; `torch.float32` on request).
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


# ----------------------------------------------------------------------------------------
# files


def read_config(folder):
    """config.json as a dict (crates/kapel-hub/src/checkpoint.rs:47-127 reads the same file)."""
    return json.loads((Path(folder) / "config.json").read_text())


def read_safetensors(path, dtype=torch.float64):
    """Every tensor of a safetensors file, widened to `dtype`.

    Format as crates/kapel-hub/src/safetensors.rs:110-204 checks it: 8 bytes little-endian
    header length, a JSON object name -> {dtype, shape, data_offsets}, then the bytes.
    """
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    base = 8 + n
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        buf = raw[base + a : base + b]
        kind = meta["dtype"]
        if kind == "BF16":
            u = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = u.view(np.float32)
        elif kind == "F32":
            arr = np.frombuffer(buf, dtype=np.float32)
        elif kind == "F16":
            arr = np.frombuffer(buf, dtype=np.float16).astype(np.float32)
        elif kind == "F64":
            arr = np.frombuffer(buf, dtype=np.float64)
        else:
            raise ValueError(f"{name}: dtype {kind} not handled by the plain reader")
        out[name] = torch.tensor(np.array(arr), dtype=dtype).reshape(meta["shape"])
    return out


# ----------------------------------------------------------------------------------------
# configuration, as crates/kapel-models/src/config.rs reads it for model_type "gemma2"


def layer_windows(cfg):
    """The window of each layer, None for a layer that sees every key.

    crates/kapel-models/src/config.rs:349-369: `layer_types[i] == "sliding_attention"` slides;
    without `layer_types`, the even layers of a gemma2 model slide.
    """
    n = cfg["num_hidden_layers"]
    window = cfg.get("sliding_window")
    types = cfg.get("layer_types")
    out = []
    for i in range(n):
        if window is None:
            out.append(None)
        elif types is not None:
            out.append(window if types[i] == "sliding_attention" else None)
        else:
            out.append(window if i % 2 == 0 else None)
    return out


def head_dim_of(cfg):
    """crates/kapel-models/src/config.rs:296-300: head_dim, else hidden / heads."""
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def score_scale(cfg):
    """crates/kapel-models/src/config.rs:498 and crates/kapel-ops/src/paged.rs:59-61:
    1/sqrt(query_pre_attn_scalar), else 1/sqrt(head_dim)."""
    q = cfg.get("query_pre_attn_scalar")
    return 1.0 / math.sqrt(q if q is not None else head_dim_of(cfg))


# ----------------------------------------------------------------------------------------
# parts


def embed(table, ids, scale):
    """x = table[ids] * scale (crates/kapel-models/src/model.rs:633,653-656).

    `scale` is sqrt(hidden) rounded to the activation dtype (model.rs:2079-2083); the caller
    passes the value it wants compared.
    """
    return table[ids] * scale


def rms_norm(x, weight, eps, offset=1.0):
    """y = x / sqrt(mean(x^2) + eps) * (offset + w)
    (crates/kapel-ops/src/norm.rs:123-135; crates/kapel-ref/src/norm.rs:134-148,206-218)."""
    mean_square = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inv = 1.0 / torch.sqrt(mean_square + eps)
    return x * inv * (offset + weight)


def rope_frequencies(theta, rotary, dtype=torch.float64):
    """w_j = theta^(-2j/r), j < r/2 (crates/kapel-ops/src/rope.rs:95-101), in 64-bit."""
    j = torch.arange(rotary // 2, dtype=torch.float64)
    return (float(theta) ** (-(2.0 * j) / rotary)).to(dtype)


def rope(x, positions, theta):
    """Rotation of every head vector by its position's angles, Half pairing (j, j + r/2):
    a' = a cos - b sin, b' = b cos + a sin (crates/kapel-ref/src/rope.rs:12-34).
    Angles in 64-bit as the device table is made (kernels/src/lib.rs:1092-1110).

    x: [T, heads, D]; positions: [T] integers.
    """
    d = x.shape[-1]
    w = rope_frequencies(theta, d)
    angle = positions.to(torch.float64)[:, None] * w[None, :]          # [T, D/2]
    cos = torch.cos(angle).to(x.dtype)[:, None, :]
    sin = torch.sin(angle).to(x.dtype)[:, None, :]
    a, b = x[..., : d // 2], x[..., d // 2 :]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def attention(q, k, v, scale, softcap, window):
    """Causal attention of one sequence, all of it at once.

    Scores s_j = scale * (q . k_j); softcap s <- cap * tanh(s / cap) after the scale and
    before the mask (crates/kapel-ops/src/attention.rs:26-27; crates/kapel-ref/src/paged.rs:58-62);
    a query that has seen `c` positions (its own is c-1) sees j in [max(0, c - window), c)
    (crates/kapel-ops/src/paged.rs:16-20,65-70); head h reads kv head h / (Hq / Hkv) (paged.rs:19-20);
    softmax over the visible keys, then the weighted sum of values
    (crates/kapel-ref/src/paged.rs:63-78).

    q: [T, Hq, D]; k, v: [T, Hkv, D]. Returns [T, Hq, D].
    """
    t, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = torch.zeros_like(q)
    for r in range(t):
        count = r + 1
        first = max(0, count - window) if window is not None else 0
        for h in range(hq):
            kv = h // group
            keys = k[first:count, kv, :]                  # [n, D]
            s = scale * (keys @ q[r, h, :])
            if softcap is not None:
                s = softcap * torch.tanh(s / softcap)
            wgt = torch.exp(s - s.max())
            wgt = wgt / wgt.sum()
            out[r, h, :] = wgt @ v[first:count, kv, :]
    return out


def gelu_tanh(x):
    """x/2 * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3))) (crates/kapel-ops/src/elementwise.rs:33-35)."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)))


def geglu_ffn(h, w_gate, w_up, w_down):
    """m = (gelu_tanh(h Wg^T) * (h Wu^T)) Wd^T (crates/kapel-models/src/model.rs:1429-1456)."""
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def attention_mixer(h, positions, w, prefix, cfg, window):
    """q/k/v products, RoPE on q and k, attention, output product
    (crates/kapel-models/src/model.rs:1506-1517,1541-1590,1633-1637)."""
    hq, hkv, d = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    t = h.shape[0]
    q = (h @ w[f"{prefix}.self_attn.q_proj.weight"].T).reshape(t, hq, d)
    k = (h @ w[f"{prefix}.self_attn.k_proj.weight"].T).reshape(t, hkv, d)
    v = (h @ w[f"{prefix}.self_attn.v_proj.weight"].T).reshape(t, hkv, d)
    theta = cfg.get("rope_theta", 10000.0)
    q = rope(q, positions, theta)
    k = rope(k, positions, theta)
    y = attention(q, k, v, score_scale(cfg), cfg.get("attn_logit_softcapping"), window)
    return y.reshape(t, hq * d) @ w[f"{prefix}.self_attn.o_proj.weight"].T


def sandwich_block(x, positions, w, prefix, cfg, window):
    """h=norm_in(x); a=attn(h); a=norm_post_attn(a); x=x+a; h=norm_pre_ffn(x); m=mlp(h);
    m=norm_post_ffn(m); x=x+m (crates/kapel-models/src/model.rs:1401-1460)."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = rms_norm(x, w[f"{prefix}.input_layernorm.weight"], eps)
    a = attention_mixer(h, positions, w, prefix, cfg, window)
    a = rms_norm(a, w[f"{prefix}.post_attention_layernorm.weight"], eps)
    x = x + a
    h = rms_norm(x, w[f"{prefix}.pre_feedforward_layernorm.weight"], eps)
    m = geglu_ffn(
        h,
        w[f"{prefix}.mlp.gate_proj.weight"],
        w[f"{prefix}.mlp.up_proj.weight"],
        w[f"{prefix}.mlp.down_proj.weight"],
    )
    m = rms_norm(m, w[f"{prefix}.post_feedforward_layernorm.weight"], eps)
    return x + m


def logits_head(x, w, cfg):
    """Final norm, product by the tied table (or lm_head.weight), soft cap cap*tanh(l/cap)
    (crates/kapel-models/src/model.rs:1369-1381,281-285)."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = rms_norm(x, w["model.norm.weight"], eps)
    table = w["lm_head.weight"] if "lm_head.weight" in w and not cfg.get("tie_word_embeddings", True) else w["model.embed_tokens.weight"]
    logits = h @ table.T
    cap = cfg.get("final_logit_softcapping")
    if cap is not None:
        logits = cap * torch.tanh(logits / cap)
    return logits


def forward(cfg, w, ids, embed_scale=None, upto_layer=None):
    """Logits [T, V] of a whole sequence `ids` (a list of ints), no cache
    (crates/kapel-models/src/model.rs:1272-1383)."""
    any_w = w["model.embed_tokens.weight"]
    ids_t = torch.tensor(list(ids), dtype=torch.long)
    positions = torch.arange(len(ids))
    if embed_scale is None:
        embed_scale = math.sqrt(cfg["hidden_size"])
    x = embed(any_w, ids_t, embed_scale)
    windows = layer_windows(cfg)
    n_layers = cfg["num_hidden_layers"] if upto_layer is None else upto_layer
    for i in range(n_layers):
        x = sandwich_block(x, positions, w, f"model.layers.{i}", cfg, windows[i])
    if upto_layer is not None:
        return x
    return logits_head(x, w, cfg)


def load(folder, dtype=torch.float64):
    """(config dict, weights dict) of a model folder."""
    folder = Path(folder)
    return read_config(folder), read_safetensors(folder / "model.safetensors", dtype)


# ----------------------------------------------------------------------------------------
# sampling, as crates/kapel-infer/src/sampling.rs


class PlainRng:
    """xoshiro256** seeded by four SplitMix64 outputs (crates/kapel-infer/src/sampling.rs:91-121)."""

    M = (1 << 64) - 1

    def __init__(self, seed):
        z = seed & self.M
        s = []
        for _ in range(4):
            z = (z + 0x9E3779B97F4A7C15) & self.M
            x = z
            x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & self.M
            x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & self.M
            s.append(x ^ (x >> 31))
        self.s = s

    @staticmethod
    def _rotl(x, k):
        return ((x << k) | (x >> (64 - k))) & PlainRng.M

    def next_u64(self):
        s = self.s
        result = (self._rotl((s[1] * 5) & self.M, 7) * 9) & self.M
        t = (s[1] << 17) & self.M
        s[2] ^= s[0]
        s[3] ^= s[1]
        s[1] ^= s[2]
        s[0] ^= s[3]
        s[2] ^= t
        s[3] = self._rotl(s[3], 45)
        return result

    def uniform(self):
        return (self.next_u64() >> 11) / float(1 << 53)


def plain_argmax(values):
    """First largest, NaN never unless all are (crates/kapel-infer/src/sampling.rs:291-299)."""
    best = None
    for i, v in enumerate(values):
        if not math.isnan(v) and (best is None or v > values[best]):
            best = i
    return best or 0


def plain_choose(logits, temperature, u):
    """Temperature sampling without filters: softmax in 64-bit, first index whose running
    total exceeds u (crates/kapel-infer/src/sampling.rs:190-195,232-260,302-310)."""
    if temperature <= 0:
        return plain_argmax(logits)
    scaled = [l / temperature for l in logits]
    m = max(scaled)
    e = [math.exp(l - m) for l in scaled]
    total_e = sum(e)
    total = 0.0
    last = 0
    for i, x in enumerate(e):
        p = x / total_e
        if p > 0:
            total += p
            last = i
            if u < total:
                return i
    return last
