"""A plain, slow Gemma 2 forward pass: whole sequences, no cache, one function a part.

It rests on the formulas of smallbard/kapel's sources, cited at each function by the file's
path within that project and its lines. Kapel's own model code is Rust and cannot be compiled
here (no Rust toolchain, no network for its dependencies), so this file rests on the formulas
alone; `tests/golden/` holds outputs of this file, not of Kapel.

It shares no code with `kapel_b200`: it reads config.json and model.safetensors with its own
few lines, and uses torch only as an array library. Everything is computed in the dtype given
(`torch.float64` by default, as kapel-ref computes; `torch.float32` on request).

For the sizes of the real models there is a second way through the same functions:
`forward_streamed` reads one layer's weights at a time from the file (so memory is one layer)
and uses `attention_blocked`, the same attention written as matrix products over a block of
query rows at a time; both run wherever torch puts their arrays (a GPU's 64-bit arithmetic
makes 4,000 tokens through 26 layers a matter of seconds). `attention_blocked` is proved equal
to the loop of `attention` on the tiny configurations in tests/test_plain.py.
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
    w = rope_frequencies(theta, d).to(x.device)
    angle = positions.to(device=x.device, dtype=torch.float64)[:, None] * w[None, :]          # [T, D/2]
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


def attention_blocked(q, k, v, scale, softcap, window, block=256):
    """`attention` again, the same formulas in the same order (scale, soft cap, mask, softmax over
    the visible keys, weighted sum; the same citations), for a block of query rows at a time as
    matrix products, so that thousands of positions take seconds, not hours.

    q: [T, Hq, D]; k, v: [T, Hkv, D]. Returns [T, Hq, D].
    """
    t, hq, d = q.shape
    hkv = k.shape[1]
    group = hq // hkv
    out = torch.empty_like(q)
    for r0 in range(0, t, block):
        r1 = min(t, r0 + block)
        j0 = max(0, r0 + 1 - window) if window is not None else 0       # the first key the block's first row sees
        qb = q[r0:r1].permute(1, 0, 2)                                                   # [Hq, rows, D]
        kb = k[j0:r1].permute(1, 2, 0).repeat_interleave(group, dim=0)                   # [Hq, D, keys]: head h reads kv head h // group
        vb = v[j0:r1].permute(1, 0, 2).repeat_interleave(group, dim=0)                   # [Hq, keys, D]
        s = scale * (qb @ kb)
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        rows = torch.arange(r0, r1, device=q.device)[:, None]
        cols = torch.arange(j0, r1, device=q.device)[None, :]
        visible = cols <= rows                                            # j < c, the row's own position included
        if window is not None:
            visible = visible & (rows - cols < window)                    # c - 1 - j < window
        s = s.masked_fill(~visible[None], float("-inf"))
        wgt = torch.exp(s - s.max(dim=-1, keepdim=True).values)
        wgt = wgt / wgt.sum(dim=-1, keepdim=True)
        out[r0:r1] = (wgt @ vb).permute(1, 0, 2)
    return out


def gelu_tanh(x):
    """x/2 * (1 + tanh(sqrt(2/pi) * (x + 0.044715 x^3))) (crates/kapel-ops/src/elementwise.rs:33-35)."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)))


def geglu_ffn(h, w_gate, w_up, w_down):
    """m = (gelu_tanh(h Wg^T) * (h Wu^T)) Wd^T (crates/kapel-models/src/model.rs:1429-1456)."""
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def attention_mixer(h, positions, w, prefix, cfg, window, attention_fn=None):
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
    y = (attention_fn or attention)(q, k, v, score_scale(cfg), cfg.get("attn_logit_softcapping"), window)
    return y.reshape(t, hq * d) @ w[f"{prefix}.self_attn.o_proj.weight"].T


def sandwich_block(x, positions, w, prefix, cfg, window, attention_fn=None):
    """h=norm_in(x); a=attn(h); a=norm_post_attn(a); x=x+a; h=norm_pre_ffn(x); m=mlp(h);
    m=norm_post_ffn(m); x=x+m (crates/kapel-models/src/model.rs:1401-1460)."""
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = rms_norm(x, w[f"{prefix}.input_layernorm.weight"], eps)
    a = attention_mixer(h, positions, w, prefix, cfg, window, attention_fn)
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


class TensorFile:
    """One safetensors file read a tensor at a time (the format as `read_safetensors` takes it):
    what `forward_streamed` needs so that only one layer's weights are held at once."""

    def __init__(self, path):
        self.raw = np.memmap(path, dtype=np.uint8, mode="r")
        (n,) = struct.unpack("<Q", self.raw[:8].tobytes())
        self.header = json.loads(self.raw[8 : 8 + n].tobytes())
        self.base = 8 + n

    def names(self):
        return [n for n in self.header if n != "__metadata__"]

    def tensor(self, name, dtype=torch.float64, device="cpu"):
        meta = self.header[name]
        a, b = meta["data_offsets"]
        buf = self.raw[self.base + a : self.base + b]
        kind = meta["dtype"]
        if kind == "BF16":                       # the 16 bits are the upper half of a float32
            bits = torch.from_numpy(np.array(buf.view(np.uint16)).astype(np.int32)).to(device)
            t = (bits << 16).view(torch.float32)
        elif kind == "F32":
            t = torch.from_numpy(np.array(buf.view(np.float32))).to(device)
        elif kind == "F16":
            t = torch.from_numpy(np.array(buf.view(np.float16))).to(device)
        elif kind == "F64":
            t = torch.from_numpy(np.array(buf.view(np.float64))).to(device)
        else:
            raise ValueError(f"{name}: dtype {kind} not handled by the plain reader")
        return t.to(dtype).reshape(meta["shape"])


def forward_streamed(folder, sequences, dtype=torch.float64, device="cpu", block=256):
    """Logits at chosen positions of several whole sequences of one model folder, with one layer's
    weights in memory at a time and the blocked attention: `forward` for the real sizes.

    `sequences` is a list of (ids, wanted positions, embed_scale or None); the result a list of
    float64 CPU tensors [wanted, V], one a sequence. The same functions as `forward` run, layer by
    layer over every sequence, so what is computed is the same; only the order of reading differs.
    """
    folder = Path(folder)
    cfg = read_config(folder)
    file = TensorFile(folder / "model.safetensors")
    table = file.tensor("model.embed_tokens.weight", dtype, device)
    xs, positions = [], []
    for ids, _, scale in sequences:
        ids_t = torch.tensor(list(ids), dtype=torch.long, device=device)
        xs.append(embed(table, ids_t, math.sqrt(cfg["hidden_size"]) if scale is None else scale))
        positions.append(torch.arange(len(ids), device=device))
    windows = layer_windows(cfg)

    def blocked(q, k, v, scale, softcap, window):
        return attention_blocked(q, k, v, scale, softcap, window, block)

    for i in range(cfg["num_hidden_layers"]):
        prefix = f"model.layers.{i}"
        w = {n: file.tensor(n, dtype, device) for n in file.names() if n.startswith(prefix + ".")}
        for s in range(len(xs)):
            xs[s] = sandwich_block(xs[s], positions[s], w, prefix, cfg, windows[i], blocked)
        del w
    head = {"model.embed_tokens.weight": table, "model.norm.weight": file.tensor("model.norm.weight", dtype, device)}
    if "lm_head.weight" in file.header and not cfg.get("tie_word_embeddings", True):
        head["lm_head.weight"] = file.tensor("lm_head.weight", dtype, device)
    out = []
    for x, (_, want, _) in zip(xs, sequences):
        rows = x[torch.tensor(list(want), dtype=torch.long, device=device)]
        out.append(logits_head(rows, head, cfg).to(torch.float64).cpu())
    return out


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
