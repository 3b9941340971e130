"""Each kernel alone against its plain reference, at sizes other than the engine's."""
import math

import numpy as np
import pytest
import torch

import plain_gemma2 as P
from helpers import rel_err

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def K():
    from kapel_b200 import kernels

    return kernels


def dev(t):
    return t.cuda().contiguous()


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embed(dtype):
    table = rnd(300, 100, seed=1, dtype=DT[dtype])
    ids = torch.tensor([0, 299, 17, 17, 5], dtype=torch.int32)
    out = K().embed(dev(table), dev(ids), 9.8125).cpu()
    want = P.embed(table.double(), ids.long(), 9.8125)
    assert rel_err(out.numpy(), want.numpy()) < 1e-6
    bad = K().embed(dev(table), dev(torch.tensor([300, -1], dtype=torch.int32)), 1.0).cpu()
    assert torch.isnan(bad).all(), "an id outside the table must not give a silent row"


def test_rope_table():
    pos = torch.tensor([0, 1, 7, 100, 8191, 131071], dtype=torch.int32)
    for theta, rotary in [(10000.0, 16), (500000.0, 48), (1e6, 256)]:
        got = K().rope_table(dev(pos), rotary, theta).cpu().double()
        w = P.rope_frequencies(theta, rotary)
        angle = pos.double()[:, None] * w[None, :]
        assert (got[..., 0] - torch.cos(angle)).abs().max() < 1e-6
        assert (got[..., 1] - torch.sin(angle)).abs().max() < 1e-6


@pytest.mark.parametrize("hq,hkv,d,rotary", [(8, 4, 256, 256), (32, 16, 128, 128), (4, 2, 16, 16), (6, 1, 32, 16), (2, 1, 64, 32), (3, 3, 48, 48),
                                            (5, 1, 64, 64)])
@pytest.mark.parametrize("rows,splits", [(1, 2), (8, 9), (9, 24), (64, 5), (7, 30)])
def test_rope_append_over_split_sums(hq, hkv, d, rotary, rows, splits):
    """Rotation and append over a stack of float32 partial sums, as a decode step has them: the
    sizes whose slices come in by bulk copies (a block's 256 pairs are whole heads of one row) and
    the others, 2 to 30 slices, 1 to 64 rows, a rotary width below the head size; rows with no line
    write nothing, and what nobody wrote stays as it was."""
    g = torch.Generator().manual_seed(hq * 100 + d + rows + splits)
    heads = hq + 2 * hkv
    parts = (torch.randn(splits, rows, heads * d, generator=g) * 0.5).float()
    page, pages = 16, 8
    pos = torch.randint(0, 5000, (rows,), generator=g, dtype=torch.int32)
    perm = torch.randperm(page * pages, generator=g)[:rows].to(torch.int32)
    lines = perm.clone()
    lines[rows // 2] = -1
    kt = torch.full((pages, hkv, page, d), 7.0, dtype=torch.bfloat16)
    vt = torch.full((pages, hkv, page, d), 7.0, dtype=torch.bfloat16)
    kd, vd = dev(kt), dev(vt)
    cs = K().rope_table(dev(pos), rotary, 10000.0)
    q = K().rope_append(K().SplitSum(dev(parts)), cs, dev(lines), kd, vd, hq, hkv, d, rotary, out_dtype=torch.bfloat16).cpu().double()
    K().check_async_errors()
    x = parts.double().sum(0).reshape(rows, heads, d)

    def rot(t):
        return torch.cat([P.rope(t[..., :rotary], pos, 10000.0), t[..., rotary:]], dim=-1)

    assert rel_err(q.numpy(), rot(x[:, :hq]).numpy()) < 1e-2
    k_want, v_want = rot(x[:, hq : hq + hkv]), x[:, hq + hkv :]
    kc = kd.cpu().double().permute(0, 2, 1, 3).reshape(page * pages, hkv, d)
    vc = vd.cpu().double().permute(0, 2, 1, 3).reshape(page * pages, hkv, d)
    written = set()
    for r in range(rows):
        l = int(lines[r])
        if l < 0:
            continue
        written.add(l)
        assert rel_err(kc[l].numpy(), k_want[r].numpy()) < 1e-2 and rel_err(vc[l].numpy(), v_want[r].numpy()) < 1e-2
    for l in range(page * pages):
        if l not in written:
            assert (kc[l] == 7.0).all() and (vc[l] == 7.0).all(), f"line {l} was written by no row"
    # the same bits as the slices added up first and rotated by the kernel that takes one input
    whole = K().finish(K().SplitSum(dev(parts)), torch.float32)
    kd2, vd2 = dev(kt), dev(vt)
    q2 = K().rope_append(whole, cs, dev(lines), kd2, vd2, hq, hkv, d, rotary, out_dtype=torch.bfloat16).cpu().double()
    assert torch.equal(q, q2) and torch.equal(kd.cpu(), kd2.cpu()) and torch.equal(vd.cpu(), vd2.cpu())
    # a layer that reads another layer's cache: the same queries, no line written (and none given)
    kd3, vd3 = dev(kt), dev(vt)
    q3 = K().rope_append(K().SplitSum(dev(parts)), cs, None, kd3, vd3, hq, hkv, d, rotary, write_kv=False, out_dtype=torch.bfloat16).cpu().double()
    K().check_async_errors()
    assert torch.equal(q, q3) and (kd3.cpu() == 7.0).all() and (vd3.cpu() == 7.0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hq,hkv,d,rotary", [(4, 2, 16, 16), (6, 1, 32, 32), (3, 3, 48, 48), (2, 1, 64, 32)])
def test_rope_append(dtype, hq, hkv, d, rotary):
    rows, page, pages = 9, 8, 5
    lines_total = page * pages
    qkv = rnd(rows, (hq + 2 * hkv) * d, seed=2, dtype=DT[dtype])
    pos = torch.tensor([0, 1, 2, 3, 50, 51, 7, 1000, 0], dtype=torch.int32)
    lines = torch.tensor([5, 6, 7, 39, 0, 1, 17, -1, 20], dtype=torch.int32)
    kt = torch.full((pages, hkv, page, d), 7.0, dtype=DT[dtype])      # [pages, kv heads, page, d]
    vt = torch.full((pages, hkv, page, d), 7.0, dtype=DT[dtype])
    kd, vd = dev(kt), dev(vt)
    cs = K().rope_table(dev(pos), rotary, 10000.0)
    q = K().rope_append(dev(qkv), cs, dev(lines), kd, vd, hq, hkv, d, rotary).cpu()
    x = qkv.double().reshape(rows, hq + 2 * hkv, d)

    def rot(t):
        r = P.rope(t[..., :rotary], pos, 10000.0)
        return torch.cat([r, t[..., rotary:]], dim=-1)

    tol = 1e-6 if dtype == "float32" else 1e-2
    assert rel_err(q.double().numpy(), rot(x[:, :hq]).numpy()) < tol
    k_want, v_want = rot(x[:, hq : hq + hkv]), x[:, hq + hkv :]
    # line = page * page_size + offset; bring the tables to [lines, kv heads, d] to look lines up
    kc = kd.cpu().double().permute(0, 2, 1, 3).reshape(lines_total, hkv, d)
    vc = vd.cpu().double().permute(0, 2, 1, 3).reshape(lines_total, hkv, d)
    written = set()
    for r in range(rows):
        l = int(lines[r])
        if l < 0:
            continue
        written.add(l)
        assert rel_err(kc[l].numpy(), k_want[r].numpy()) < tol
        assert rel_err(vc[l].numpy(), v_want[r].numpy()) < tol
    for l in range(lines_total):
        if l not in written:
            assert (kc[l] == 7.0).all() and (vc[l] == 7.0).all(), f"line {l} was written by no row"


@pytest.mark.parametrize("xdt,wdt,ydt", [("float32", "float32", "float32"), ("float32", "bfloat16", "bfloat16"),
                                          ("bfloat16", "bfloat16", "bfloat16"), ("bfloat16", "float32", "float32")])
@pytest.mark.parametrize("width", [24, 100, 2304, 5000])
def test_rmsnorm(xdt, wdt, ydt, width):
    x = rnd(7, width, seed=3, dtype=DT[xdt], scale=3.0)
    w = rnd(width, seed=4, dtype=DT[wdt], scale=0.1)
    for eps, offset in [(1e-6, 1.0), (1e-5, 0.0)]:
        got = K().rmsnorm(dev(x), dev(w), eps, offset, DT[ydt]).cpu().double()
        want = P.rms_norm(x.double(), w.double(), eps, offset)
        assert rel_err(got.numpy(), want.numpy()) < (1e-6 if ydt == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 2304])
def test_add_rmsnorm(dtype, width):
    res = rnd(5, width, seed=5, scale=2.0)
    br = rnd(5, width, seed=6, dtype=DT[dtype])
    w1 = rnd(width, seed=7, dtype=DT[dtype], scale=0.1)
    w2 = rnd(width, seed=8, dtype=DT[dtype], scale=0.1)
    tol = 1e-6 if dtype == "float32" else 1e-2
    for post, nxt in [(True, True), (True, False), (False, True), (False, False)]:
        r = dev(res.clone())
        h = K().add_rmsnorm(r, dev(br), (dev(w1), 1e-6, 1.0) if post else None, (dev(w2), 1e-5, 1.0) if nxt else None, DT[dtype])
        b = P.rms_norm(br.double(), w1.double(), 1e-6) if post else br.double()
        want_r = res.double() + b
        assert rel_err(r.cpu().double().numpy(), want_r.numpy()) < 1e-6
        if nxt:
            assert rel_err(h.cpu().double().numpy(), P.rms_norm(want_r, w2.double(), 1e-5).numpy()) < tol
        else:
            assert h is None


@pytest.mark.parametrize("m", [1, 3, 64, 65, 130])
@pytest.mark.parametrize("n,k", [(8, 8), (100, 96), (1000, 520), (72, 17)])
def test_gemm_f32(m, n, k):
    a, w = rnd(m, k, seed=9), rnd(n, k, seed=10)
    got = K().gemm(dev(a), dev(w)).cpu().double()
    want = a.double() @ w.double().T
    assert rel_err(got.numpy(), want.numpy()) < 2e-6
    # A cap above the largest product keeps tanh's slope from magnifying the sums' own rounding.
    got = K().gemm(dev(a), dev(w), softcap=30.0).cpu().double()
    assert rel_err(got.numpy(), (30.0 * torch.tanh(want / 30.0)).numpy()) < 2e-6


def test_gemm_f32_does_not_depend_on_the_batch():
    a, w = rnd(70, 200, seed=11), rnd(90, 200, seed=12)
    whole = K().gemm(dev(a), dev(w)).cpu()
    alone = K().gemm(dev(a[33:34]), dev(w)).cpu()
    assert torch.equal(whole[33:34], alone)


@pytest.mark.parametrize("m", [1, 5, 16, 17, 33, 64, 65, 200, 300])
@pytest.mark.parametrize("n,k", [(8, 8), (72, 32), (1000, 96), (2304, 520), (520, 2304), (136, 4104)])
def test_gemm_bf16(m, n, k):
    a, w = rnd(m, k, seed=13, dtype=torch.bfloat16), rnd(n, k, seed=14, dtype=torch.bfloat16)
    want = a.double() @ w.double().T
    got = K().gemm(dev(a), dev(w), out_dtype=torch.float32).cpu().double()
    assert rel_err(got.numpy(), want.numpy()) < 2e-5, "float32 output of bfloat16 inputs"
    got = K().gemm(dev(a), dev(w)).cpu().double()
    assert rel_err(got.numpy(), want.numpy()) < 1e-2
    got = K().gemm(dev(a), dev(w), out_dtype=torch.float32, softcap=30.0).cpu().double()
    assert rel_err(got.numpy(), (30.0 * torch.tanh(want / 30.0)).numpy()) < 2e-5


@pytest.mark.parametrize("kernel", ["tcgen05", "single", "pair", "mma"])
@pytest.mark.parametrize("m,n,k", [(65, 256, 64), (128, 256, 128), (129, 300, 200), (257, 520, 136), (2048, 2304, 2048), (300, 4104, 72),
                                   (1000, 18432, 2304), (700, 2304, 9216)])
def test_gemm_tcgen05(kernel, m, n, k):
    """More than 64 rows: the tcgen05 kernels (one block a tile; persistent pairs of blocks; the
    library's choice between them) and, as a yardstick, the mma.sync tile kernel."""
    import kapel_b200.kernels as KK

    a, w = rnd(m, k, seed=40, dtype=torch.bfloat16), rnd(n, k, seed=41, dtype=torch.bfloat16, scale=0.1)
    want = a.double() @ w.double().T
    old = KK.GEMM_LARGE
    KK.GEMM_LARGE = kernel
    try:
        got = K().gemm(dev(a), dev(w), out_dtype=torch.float32).cpu().double()
        K().check_async_errors()
        assert rel_err(got.numpy(), want.numpy()) < 2e-5
        got = K().gemm(dev(a), dev(w)).cpu().double()
        assert rel_err(got.numpy(), want.numpy()) < 1e-2
        got = K().gemm(dev(a), dev(w), out_dtype=torch.float32, softcap=30.0).cpu().double()
        assert rel_err(got.numpy(), (30.0 * torch.tanh(want / 30.0)).numpy()) < 2e-5
    finally:
        KK.GEMM_LARGE = old
    K().check_async_errors()


@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
@pytest.mark.parametrize("m,n,k", [(65, 128, 64), (300, 328, 200), (129, 100, 72), (2048, 9216, 2304), (513, 1000, 520),
                                   (1, 64, 64), (8, 9216, 2304), (17, 328, 200), (40, 100, 72), (64, 1000, 520)])
def test_gemm_with_the_gated_unit_in_its_epilogue(act, m, n, k):
    """act(a . gate^T) * (a . up^T) from the stacked weight in one kernel, against the two products
    in 64-bit; and against the two-step path, which rounds both products to bfloat16 first."""
    a, w = rnd(m, k, seed=44, dtype=torch.bfloat16), rnd(2 * n, k, seed=45, dtype=torch.bfloat16, scale=0.1)
    prod = a.double() @ w.double().T
    gate, up = prod[:, :n], prod[:, n:]
    if act == "gelu_tanh":
        want = 0.5 * gate * (1.0 + torch.tanh(0.7978845608028654 * (gate + 0.044715 * gate ** 3))) * up
    else:
        want = gate / (1.0 + torch.exp(-gate)) * up
    got = K().gemm_glu_fused(dev(a), dev(w), act)
    K().check_async_errors()
    assert got is not None and got.dtype == torch.bfloat16 and tuple(got.shape) == (m, n)
    assert rel_err(got.cpu().double().numpy(), want.numpy()) < 6e-3          # one rounding to bfloat16
    two_step = K().glu(K().gemm(dev(a), dev(w)), act)
    assert rel_err(two_step.cpu().double().numpy(), want.numpy()) < 2e-2
    assert K().gemm_glu_fused(dev(a.float()), dev(w.float()), act) is None    # 32-bit operands: the caller takes two steps


@pytest.mark.parametrize("small", ["skinny", "stream"])
@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 50, 64])
@pytest.mark.parametrize("n,k", [(8, 8), (136, 72), (2304, 2048), (4096, 2304), (1000, 520)])
def test_gemm_bf16_up_to_64_rows_both_kernels(small, m, n, k):
    import kapel_b200.kernels as KK

    a, w = rnd(m, k, seed=42, dtype=torch.bfloat16), rnd(n, k, seed=43, dtype=torch.bfloat16, scale=0.1)
    want = a.double() @ w.double().T
    old = KK.GEMM_SMALL
    KK.GEMM_SMALL = small
    try:
        got = K().gemm(dev(a), dev(w), out_dtype=torch.float32).cpu().double()
        capped = K().gemm(dev(a), dev(w), out_dtype=torch.float32, softcap=30.0).cpu().double()
        kept = K().gemm(dev(a), dev(w), keep_split=True)
    finally:
        KK.GEMM_SMALL = old
    K().check_async_errors()
    assert rel_err(got.numpy(), want.numpy()) < 2e-5
    assert rel_err(capped.numpy(), (30.0 * torch.tanh(want / 30.0)).numpy()) < 2e-5
    assert rel_err(K().finish(kept, torch.float32).cpu().double().numpy(), want.numpy()) < (2e-5 if isinstance(kept, K().SplitSum) else 1e-2)


def test_gemm_bf16_refuses_what_it_cannot_take():
    a, w = rnd(4, 12, dtype=torch.bfloat16), rnd(8, 12, dtype=torch.bfloat16)
    with pytest.raises(K().KernelError, match="multiple of 8"):
        K().gemm(dev(a), dev(w))


def test_gemm_bf16_small_rows_do_not_depend_on_the_batch():
    """Within a kernel (17..64 rows here; up to 16 rows in a test of its own below) a row's sums
    are added in the same order whatever else is in the batch: bit for bit. Across kernels the
    order differs, and the results agree to rounding."""
    a, w = rnd(40, 2304, seed=15, dtype=torch.bfloat16), rnd(520, 2304, seed=16, dtype=torch.bfloat16)
    whole = K().gemm(dev(a), dev(w), out_dtype=torch.float32).cpu()
    part = K().gemm(dev(a[7:40]), dev(w), out_dtype=torch.float32).cpu()
    assert torch.equal(whole[7:40], part)
    part = K().gemm(dev(a[20:38]), dev(w), out_dtype=torch.float32).cpu()
    assert torch.equal(whole[20:38], part)
    for r in (0, 17, 39):
        alone = K().gemm(dev(a[r : r + 1]), dev(w), out_dtype=torch.float32).cpu()
        assert rel_err(alone.numpy(), whole[r : r + 1].numpy()) < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("act", ["gelu_tanh", "silu"])
def test_glu(dtype, act):
    x = rnd(6, 2 * 50, seed=17, dtype=DT[dtype], scale=2.0)
    got = K().glu(dev(x), act).cpu().double()
    g, u = x.double()[:, :50], x.double()[:, 50:]
    want = (P.gelu_tanh(g) if act == "gelu_tanh" else g * torch.sigmoid(g)) * u
    assert rel_err(got.numpy(), want.numpy()) < (1e-6 if dtype == "float32" else 1e-2)


# ------------------------------------------------------------------------------------------
def paged_reference(q, k_table, v_table, block_table, row_entry, row_count, page, window, scale, cap, only=None):
    """Row by row in 64-bit, as crates/kapel-ref/src/paged.rs:28-92. With `only`, just those rows
    (the others stay zero): for histories of thousands of keys, where a sample of rows is checked."""
    rows, hq, d = q.shape
    hkv = k_table.shape[1]                      # tables are [pages, kv heads, page, d]
    group = hq // hkv
    kt = k_table.double().permute(0, 2, 1, 3).reshape(-1, hkv, d)        # [lines, kv heads, d]
    vt = v_table.double().permute(0, 2, 1, 3).reshape(-1, hkv, d)
    out = torch.zeros(rows, hq, d, dtype=torch.float64)
    for r in (range(rows) if only is None else only):
        e, c = int(row_entry[r]), int(row_count[r])
        first = max(0, c - window) if window else 0
        if c <= first:
            continue
        lines = [int(block_table[e, j // page]) * page + j % page for j in range(first, c)]
        for h in range(hq):
            keys, vals = kt[lines, h // group], vt[lines, h // group]
            s = scale * (keys @ q[r, h].double())
            if cap:
                s = cap * torch.tanh(s / cap)
            p = torch.exp(s - s.max())
            out[r, h] = (p / p.sum()) @ vals
    return out


def make_paged_case(dtype, hq, hkv, d, lengths, q_lens, page=16, seed=0, n_pages=None):
    """Sequences of `lengths` already in a scrambled paged cache; the last q_lens[i] positions of
    sequence i are this step's query rows."""
    g = torch.Generator().manual_seed(seed)
    need = sum(-(-n // page) for n in lengths)
    n_pages = n_pages or need + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lengths)
    bt = torch.full((len(lengths), width), -1, dtype=torch.int32)
    k_table = torch.randn(n_pages, hkv, page, d, generator=g).to(DT[dtype])
    v_table = torch.randn(n_pages, hkv, page, d, generator=g).to(DT[dtype])
    for i, n in enumerate(lengths):
        for p in range(-(-n // page)):
            bt[i, p] = perm.pop()
    row_entry, row_count = [], []
    for i, (n, ql) in enumerate(zip(lengths, q_lens)):
        for c in range(n - ql + 1, n + 1):
            row_entry.append(i)
            row_count.append(c)
    q = torch.randn(len(row_entry), hq, d, generator=g).to(DT[dtype])
    return q, k_table, v_table, bt, torch.tensor(row_entry, dtype=torch.int32), torch.tensor(row_count, dtype=torch.int32)


def run_rows(q, kt, vt, bt, re, rc, page, window, scale, cap):
    from kapel_b200.engine.batch import _chunks_touched

    slots = _chunks_touched(rc.numpy(), window, K().attention_chunk())
    return K().paged_attention_rows(dev(q), dev(kt), dev(vt), dev(bt), dev(re), dev(rc), page, window, scale, cap, slots).cpu()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 16), (6, 1, 32), (3, 3, 48), (12, 1, 64), (8, 4, 128), (2, 1, 256), (9, 1, 80)])
@pytest.mark.parametrize("window,cap", [(None, None), (24, 20.0), (300, 50.0)])
def test_paged_attention_rows(dtype, hq, hkv, d, window, cap):
    lengths, q_lens = [1, 37, 300, 700], [1, 5, 1, 33]
    q, kt, vt, bt, re, rc = make_paged_case(dtype, hq, hkv, d, lengths, q_lens, seed=hq * 100 + d)
    scale = 1.0 / math.sqrt(d * 1.5)
    got = run_rows(q, kt, vt, bt, re, rc, 16, window, scale, cap).double()
    want = paged_reference(q, kt, vt, bt, re, rc, 16, window, scale, cap)
    assert rel_err(got.numpy(), want.numpy()) < (1e-5 if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_paged_attention_far_key_and_window_edge(dtype):
    """One key among hundreds is made to stand out, first far away, then exactly at the window's
    edge, then one position beyond it: the output must follow that key's value, then not."""
    hq, hkv, d, n, page, window = 2, 1, 32, 600, 16, 128
    q, kt, vt, bt, re, rc = make_paged_case(dtype, hq, hkv, d, [n], [1], seed=3)
    q = q * 0.05
    scale = 1.0

    def plant(pos):
        kt2, vt2 = kt.clone(), vt.clone()
        kt2[int(bt[0, pos // page]), 0, pos % page] = (q[0, 0].float() * 400).to(kt.dtype)      # a score far above the rest
        vt2[int(bt[0, pos // page]), 0, pos % page] = 5.0
        return kt2, vt2

    tol = 1e-5 if dtype == "float32" else 1.5e-2
    for pos, win, seen in [(3, None, True), (n - window, window, True), (n - window - 1, window, False)]:
        kt2, vt2 = plant(pos)
        got = run_rows(q, kt2, vt2, bt, re, rc, page, win, scale, None).double()
        want = paged_reference(q, kt2, vt2, bt, re, rc, page, win, scale, None)
        assert rel_err(got.numpy(), want.numpy()) < tol
        assert (abs(float(got[0, 0].mean()) - 5.0) < 0.1) == seen


def test_paged_attention_row_that_sees_nothing_gives_zeros():
    q, kt, vt, bt, re, rc = make_paged_case("float32", 4, 2, 16, [20], [2], seed=4)
    rc[0] = 0
    got = run_rows(q, kt, vt, bt, re, rc, 16, None, 0.25, None)
    assert (got[0] == 0).all() and torch.isfinite(got).all()


# ------------------------------------------------------------------------------------------
def test_sample_greedy_rules():
    nan = float("nan")
    logits = torch.tensor([[1.0, 5.0, 5.0, 2.0], [nan, -3.0, nan, -3.0], [nan, nan, nan, nan], [-1e30, -2e30, -1e30, -3e30]])
    got = K().sample(dev(logits)).cpu().tolist()
    assert got == [P.plain_argmax(row) for row in logits.tolist()] == [1, 1, 0, 0]
    big = rnd(3, 256000, seed=20)
    big[1, 123456] = 100.0
    big[2, 255999] = 100.0
    got = K().sample(dev(big)).cpu().tolist()
    assert got == big.argmax(dim=1).tolist()
    # the two-step choice of a large vocabulary: a tie across two blocks' shares (the first wins), a
    # row of NaN but one value, a row of nothing but NaN, the largest in the last column
    big = rnd(5, 256000, seed=22)
    big[0, 9000] = big[0, 200000] = 50.0
    big[1, :] = nan
    big[1, 131072] = -7.0
    big[2, :] = nan
    big[3, 255999] = 60.0
    got = K().sample(dev(big)).cpu().tolist()
    assert got == [9000, 131072, 0, 255999, int(big[4].argmax())]


def test_sample_temperature_follows_plain_rule_and_probabilities():
    vocab = 1000
    logits = rnd(1, vocab, seed=21, scale=2.0)
    temps = torch.tensor([0.8])
    rng = P.PlainRng(7)
    agree = 0
    n = 300
    rows = logits.repeat(n, 1)
    us = torch.tensor([rng.uniform() for _ in range(n)], dtype=torch.float32)
    got = K().sample(dev(rows), dev(temps.repeat(n)), dev(us)).cpu().tolist()
    want = [P.plain_choose(logits[0].double().tolist(), 0.8, float(u)) for u in us]
    agree = sum(int(a == b) for a, b in zip(got, want))
    assert agree >= n - 3, f"{n - agree} of {n} draws differ from the plain rule (32-bit against 64-bit sums)"
    # draws follow the probabilities
    small = torch.tensor([[0.0, math.log(2.0), math.log(4.0), -1e9]])
    m = 20000
    g = torch.Generator().manual_seed(5)
    us = torch.rand(m, generator=g)
    got = K().sample(dev(small.repeat(m, 1)), dev(torch.ones(m)), dev(us)).cpu()
    freq = torch.bincount(got.long(), minlength=4).double() / m
    assert (freq - torch.tensor([1 / 7, 2 / 7, 4 / 7, 0.0], dtype=torch.float64)).abs().max() < 0.015
    # temperature 0 in a row of a sampled batch is greedy
    got = K().sample(dev(small.repeat(2, 1)), dev(torch.tensor([0.0, 1.0])), dev(torch.tensor([0.99, 0.0]))).cpu().tolist()
    assert got == [2, 0]


def test_sample_draws_over_a_large_vocabulary_in_two_steps():
    """A vocabulary of 65,536 and more is drawn from in two steps (shares of the columns, then one
    share walked). The plain rule in 64-bit: the first index whose running total exceeds u x total.
    32-bit sums of 256,000 terms differ from 64-bit ones in the seventh digit, so a draw may fall
    on a neighbour where the target is that close to a token's edge: the chosen token's own
    interval, widened by 4e-6 of the total, must hold the target. A peaked row (a few tokens carry
    everything) must agree exactly but for such edges."""
    vocab, n = 256000, 96
    for scale, temp in ((1.0, 0.8), (12.0, 1.3)):
        row = rnd(1, vocab, seed=31, scale=scale)[0]
        row[5] = row[77777] = float("nan")
        row[250000:] = -1e30                              # impossible tokens at the end
        us = torch.rand(n, generator=torch.Generator().manual_seed(9))
        us[0], us[1], us[2] = 0.0, 0.99999994, 0.5
        got = K().sample(dev(row.repeat(n, 1)), dev(torch.full((n,), temp)), dev(us)).cpu().numpy()
        x = row.double().numpy() / temp
        ok = ~np.isnan(x)
        p = np.where(ok, np.exp(x - x[ok].max()), 0.0)
        c = np.cumsum(p)
        total = c[-1]
        want = np.searchsorted(c, us.double().numpy() * total, side="right")
        exact = 0
        for g, w, u in zip(got, want, us.double().numpy()):
            assert 0 <= g < 250000 and p[g] > 0, f"token {g} cannot be drawn"
            lo, hi = (c[g - 1] if g else 0.0), c[g]
            assert lo - 4e-6 * total <= u * total <= hi + 4e-6 * total, f"u {u}: token {g} holds [{lo / total}, {hi / total}), the plain rule gives {w}"
            exact += int(g == w)
        if scale > 4:
            assert exact >= n - 3, f"{n - exact} of {n} draws on a peaked row differ from the plain rule"
    # a row whose target lies beyond every total gets the last possible token; greedy rows beside drawn ones
    rows = rnd(3, vocab, seed=33)
    rows[0, 200000:] = float("nan")
    rows[1, 1000] = rows[1, 130000] = 40.0              # a tie across two shares: the first wins
    rows[2, :] = -1e30
    rows[2, 123] = 0.0                                    # all the probability in one token
    got = K().sample(dev(rows), dev(torch.tensor([1.0, 0.0, 0.7])), dev(torch.tensor([1.0, 0.3, 0.9]))).cpu().tolist()
    assert got == [199999, 1000, 123]


# ------------------------------------------------------------------------------------------
def run_mma(q, kt, vt, bt, rc, q_lens, page, window, scale, cap, decode, split, relative=False):
    from kapel_b200.engine.batch import cut_tiles

    hq, hkv = q.shape[1], kt.shape[1]
    kernel = "mma" if decode else K().attention_prompt_kernel(hq, hkv, q.shape[2], page, cap)
    per_tile = max(1, K().attention_tile_rows(decode, kernel, q.shape[2]) // (hq // hkv))
    q_len = np.asarray(q_lens, np.int32)
    q_start = np.concatenate(([0], np.cumsum(q_len)[:-1])).astype(np.int32)
    tiles = tuple(dev(torch.from_numpy(a)) for a in cut_tiles(q_start, q_len, per_tile))
    longest = int(rc.max())
    if relative and window:
        longest = min(longest, window)                  # slots counted from each row's first visible key
    slots = max(1, -(-longest // split)) if split else 1
    rows = int(q_len.max()) * (hq // hkv) if decode else 0
    return K().paged_attention_mma(dev(q), dev(kt), dev(vt), dev(bt), dev(rc), tiles, page, window, scale, cap, rows, split, slots,
                                   relative).cpu()


@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 16), (6, 1, 32), (3, 3, 48), (16, 1, 64), (8, 4, 128), (8, 4, 256), (5, 1, 80)])
@pytest.mark.parametrize("window,cap", [(None, None), (24, 20.0), (300, 50.0)])
@pytest.mark.parametrize("split", [0, 64, 256])
@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05_single", "mma"])
def test_paged_attention_mma_prompt_mode(kernel, hq, hkv, d, window, cap, split):
    """Prompt portions: the tcgen05 kernels where they apply (head sizes 64, 128, 256 with a soft
    cap; pairs of blocks at 128 and 256, and single blocks at all three) and the mma.sync kernel
    everywhere."""
    import kapel_b200.kernels as KK

    takes = d in (64, 128, 256) and cap is not None
    if kernel.startswith("tcgen05") and not takes:
        pytest.skip("the mma.sync kernel runs these sizes under either setting")
    if kernel == "tcgen05_single" and d == 64:
        pytest.skip("head size 64 runs on single blocks under either setting")
    lengths, q_lens = [1, 37, 300, 700], [1, 37, 130, 33]
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, q_lens, seed=hq * 100 + d)
    scale = 1.0 / math.sqrt(d * 1.5)
    old = KK.ATTENTION_PROMPT, KK.ATTENTION_PAIRS
    KK.ATTENTION_PROMPT, KK.ATTENTION_PAIRS = kernel.split("_")[0], (0 if kernel == "tcgen05_single" else 1)
    try:
        got = run_mma(q, kt, vt, bt, rc, q_lens, 16, window, scale, cap, False, split).double()
    finally:
        KK.ATTENTION_PROMPT, KK.ATTENTION_PAIRS = old
    K().check_async_errors()
    want = paged_reference(q, kt, vt, bt, re, rc, 16, window, scale, cap)
    assert rel_err(got.numpy(), want.numpy()) < 1.5e-2


@pytest.mark.parametrize("d", [64, 128, 256])
def test_paged_attention_tcgen05_far_key_and_window_edge(d):
    """One key among hundreds carries the weight: seen at the far end and at the window's first
    position, not one position before it. Scores are capped, so the planted key stands out by
    about e^(2 cap) only."""
    hq, hkv, n, page, window, cap = 2, 1, 600, 16, 128, 12.0
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, [n], [70], seed=5)
    q = q * 0.05
    first = n - 70 + 1                                  # keys the first of the 70 tokens sees
    for pos, win, seen in [(3, None, True), (first - window, window, True), (first - window - 1, window, False)]:
        kt2, vt2 = kt.clone(), vt.clone()
        kt2[int(bt[0, pos // page]), 0, pos % page] = (q[0, 0].float() * 4000).to(kt.dtype)
        vt2[int(bt[0, pos // page]), 0, pos % page] = 5.0
        got = run_mma(q, kt2, vt2, bt, rc, [70], page, win, 1.0, cap, False, 0).double()
        K().check_async_errors()
        want = paged_reference(q, kt2, vt2, bt, re, rc, page, win, 1.0, cap)
        assert rel_err(got.numpy(), want.numpy()) < 1.5e-2
        assert (abs(float(got[0, 0].mean()) - 5.0) < 0.5) == seen


@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 16), (6, 1, 32), (16, 1, 64), (8, 4, 128), (8, 4, 256), (2, 2, 96)])
@pytest.mark.parametrize("window,cap", [(None, None), (24, 20.0), (300, 50.0)])
@pytest.mark.parametrize("split", [64, 256])
def test_paged_attention_mma_decode_mode(hq, hkv, d, window, cap, split):
    group = hq // hkv
    lengths = [1, 37, 300, 700, 64, 65]
    q_lens = [1, min(2, 16 // group), 1, max(1, 16 // group), 1, 1]
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, q_lens, seed=hq * 100 + d + 1)
    rc[0] = 0                      # a padding row: sees nothing, gives zeros
    scale = 1.0 / math.sqrt(d * 1.5)
    got = run_mma(q, kt, vt, bt, rc, q_lens, 16, window, scale, cap, True, split).double()
    want = paged_reference(q, kt, vt, bt, re, rc, 16, window, scale, cap)
    assert (got[0] == 0).all()
    assert rel_err(got.numpy(), want.numpy()) < 1.5e-2


@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 16), (6, 1, 32), (16, 1, 64), (8, 4, 128), (8, 4, 256)])
@pytest.mark.parametrize("window,cap", [(None, None), (24, 20.0), (300, 50.0), (128, 50.0)])
@pytest.mark.parametrize("split", [64, 128, 256])
def test_paged_attention_decode_slots_counted_from_the_windows_start(hq, hkv, d, window, cap, split):
    """One token a request: the key slots may be counted from each row's first visible key, so a
    windowed row fills ceil(window / split) slots however long its history."""
    lengths = [1, 37, 300, 700, 64, 65, 129, 428]
    q_lens = [1] * len(lengths)
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, q_lens, seed=hq * 100 + d + 2)
    rc[0] = 0                      # a padding row
    scale = 1.0 / math.sqrt(d * 1.5)
    got = run_mma(q, kt, vt, bt, rc, q_lens, 16, window, scale, cap, True, split, relative=True).double()
    want = paged_reference(q, kt, vt, bt, re, rc, 16, window, scale, cap)
    assert (got[0] == 0).all()
    assert rel_err(got.numpy(), want.numpy()) < 1.5e-2


@pytest.mark.parametrize("hq,hkv,d", [(8, 4, 256), (8, 4, 128), (4, 2, 64), (16, 1, 64), (6, 1, 128), (2, 2, 256)])
@pytest.mark.parametrize("window,cap", [(None, None), (300, 50.0), (128, 50.0)])
@pytest.mark.parametrize("split,splits", [(64, 9), (256, 5), (128, 1)])
def test_decode_attention_from_the_qkv_products_slices(hq, hkv, d, window, cap, split, splits):
    """The decode kernel that takes the stacked q|k|v product's partial sums (one token a request)
    gives, bit for bit, what the rotation kernel followed by the decode attention gives: the same
    output and the same key and value tables (the newest line written, nothing else touched). A
    padding row (count 0, line -1) writes nothing and gives zeros. A layer that reads another
    layer's cache writes no line."""
    from kapel_b200.engine.batch import cut_tiles
    import kapel_b200.kernels as KK

    lengths = [1, 37, 300, 700, 64, 65, 129, 428]
    rows, page, group = len(lengths), 16, hq // hkv
    _, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, [1] * rows, seed=hq * 100 + d + 7)
    rc[0] = 0                                               # a padding row
    lines = torch.tensor([-1] + [int(bt[r, (n - 1) // page]) * page + (n - 1) % page for r, n in enumerate(lengths)][1:], dtype=torch.int32)
    parts = rnd(splits, rows * (hq + 2 * hkv) * d, seed=d + splits).reshape(splits, rows, (hq + 2 * hkv) * d)
    positions = torch.tensor([max(n - 1, 0) for n in lengths], dtype=torch.int32)
    cs = K().rope_table(dev(positions), d, 10000.0)
    scale = 1.0 / math.sqrt(d * 1.5)
    assert K().attention_decode_fused_takes(KK.SplitSum(dev(parts)), hq, hkv, d, d, page, torch.bfloat16)
    q_len = np.ones(rows, np.int32)
    tiles = tuple(dev(torch.from_numpy(a)) for a in cut_tiles(np.arange(rows, dtype=np.int32), q_len, 1))
    longest = min(max(lengths), window) if window else max(lengths)
    slots = max(1, -(-longest // split))
    for write_kv in (False, True):
        kt_a, vt_a, kt_b, vt_b = dev(kt.clone()), dev(vt.clone()), dev(kt.clone()), dev(vt.clone())
        q = K().rope_append(KK.SplitSum(dev(parts)), cs, dev(lines), kt_a, vt_a, hq, hkv, d, d, write_kv=write_kv, out_dtype=torch.bfloat16)
        want = K().paged_attention_mma(q, kt_a, vt_a, dev(bt), dev(rc), tiles, page, window, scale, cap, group, split, slots, True)
        got = K().paged_attention_decode_fused(KK.SplitSum(dev(parts)), cs, dev(lines), kt_b, vt_b, dev(bt), dev(rc), hq, hkv, d,
                                               write_kv, page, window, scale, cap, split, slots)
        torch.cuda.synchronize()
        K().check_async_errors()
        assert torch.equal(kt_a, kt_b) and torch.equal(vt_a, vt_b), "the cache differs"
        assert (kt_a.cpu() != kt).any() == write_kv
        assert (got[0] == 0).all()
        assert torch.equal(got, want), f"write_kv {write_kv}: {(got != want).sum().item()} values differ"
    # and against the plain rule, with the newest key in the cache
    want = paged_reference(q.cpu(), kt_a.cpu(), vt_a.cpu(), bt, re, rc, page, window, scale, cap)
    assert rel_err(got.cpu().double().numpy(), want.numpy()) < 1.5e-2


@pytest.mark.parametrize("decode", [False, True])
def test_paged_attention_mma_far_key_and_window_edge(decode):
    hq, hkv, d, n, page, window = 2, 1, 32, 600, 16, 128
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, [n], [1], seed=3)
    q = q * 0.05

    def plant(pos):
        kt2, vt2 = kt.clone(), vt.clone()
        kt2[int(bt[0, pos // page]), 0, pos % page] = (q[0, 0].float() * 400).to(kt.dtype)
        vt2[int(bt[0, pos // page]), 0, pos % page] = 5.0
        return kt2, vt2

    for pos, win, seen in [(3, None, True), (n - window, window, True), (n - window - 1, window, False)]:
        kt2, vt2 = plant(pos)
        got = run_mma(q, kt2, vt2, bt, rc, [1], page, win, 1.0, None, decode, 256 if decode else 0).double()
        want = paged_reference(q, kt2, vt2, bt, re, rc, page, win, 1.0, None)
        assert rel_err(got.numpy(), want.numpy()) < 1.5e-2
        assert (abs(float(got[0, 0].mean()) - 5.0) < 0.1) == seen


@pytest.mark.parametrize("slots_wanted", [19, 150, 333])
def test_decode_attention_over_many_key_slots_merges_them_all(slots_wanted):
    """One request alone with a long history is cut into more key slots than the merge kernel keeps
    in registers at once (16 values a thread, 128 maxima a warp): 19, 150 and 333 slots of 64 keys,
    beside a short request that fills one slot. One key far back carries a value that stands out, so
    a slot that the merge dropped or weighted wrongly shows."""
    hq, hkv, d, page = 2, 1, 64, 16
    lengths = [64 * slots_wanted - 7, 40]
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, [1, 1], seed=slots_wanted)
    # the long request's key at position 70 (in its second slot) answers its query with a large score
    line = int(bt[0, 70 // page]) * page + 70 % page
    kt.view(-1, hkv, page, d)[line // page, 0, line % page] = (q[0, 0] * 3.0).to(kt.dtype)
    vt.view(-1, hkv, page, d)[line // page, 0, line % page] = 5.0
    from kapel_b200.engine.batch import cut_tiles

    tiles = tuple(dev(torch.from_numpy(a)) for a in cut_tiles(np.arange(2, dtype=np.int32), np.ones(2, np.int32), 1))
    got = K().paged_attention_mma(dev(q), dev(kt), dev(vt), dev(bt), dev(rc), tiles, page, None, 1.0 / 8, None, hq // hkv, 64,
                                  slots_wanted, True).cpu().double()
    K().check_async_errors()
    want = paged_reference(q, kt, vt, bt, re, rc, page, None, 1.0 / 8, None)
    assert rel_err(got.numpy(), want.numpy()) < 1.5e-2
    assert float(want[0, 0].mean()) > 2.0, "the planted key decides the long request's first head"


@pytest.mark.parametrize("hq,hkv,d,scalar", [(8, 4, 256, 256), (32, 16, 128, 144)])
@pytest.mark.parametrize("window", [4096, None])
def test_paged_attention_at_the_sizes_and_histories_that_are_timed(hq, hkv, d, scalar, window):
    """The decode kernel and the tcgen05 prompt kernel at the head counts and head sizes of Gemma 2
    2B (8 over 4 of 256) and 27B (32 over 16 of 128), with the window of 4,096 and without, over
    histories of 4,097, 4,100 and 6,144 positions, cut into key slots as the engine's planners cut
    them. A sample of rows (each request's first and last, and those around the window's first move)
    against the row-by-row reference."""
    from kapel_b200.engine.batch import decode_split, prompt_split, sm_count

    scale, cap = 1.0 / math.sqrt(scalar), 50.0
    sms = sm_count(torch.device("cuda"))
    # decoding: one token of each of three requests
    lengths = [4100, 6144, 4097]
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, [1, 1, 1], seed=d + hq)
    q = q * 4.0                                            # scores of a few units: the soft cap bends them
    split, slots = decode_split(len(lengths) * hkv, max(lengths), sms, window, True)
    from kapel_b200.engine.batch import cut_tiles

    tiles = tuple(dev(torch.from_numpy(a)) for a in cut_tiles(np.arange(3, dtype=np.int32), np.ones(3, np.int32), 1))
    got = K().paged_attention_mma(dev(q), dev(kt), dev(vt), dev(bt), dev(rc), tiles, 16, window, scale, cap, hq // hkv, split, slots, True).cpu().double()
    K().check_async_errors()
    want = paged_reference(q, kt, vt, bt, re, rc, 16, window, scale, cap)
    assert rel_err(got.numpy(), want.numpy()) < 1.5e-2, f"decode, split {split} x {slots}"
    # a prompt portion of 200 tokens behind 3,950 (it crosses position 4,096) beside a whole prompt of 2,048
    lengths, q_lens = [4150, 2048], [200, 2048]
    q, kt, vt, bt, re, rc = make_paged_case("bfloat16", hq, hkv, d, lengths, q_lens, seed=d + hq + 1)
    q = q * 4.0
    per_tile = max(1, K().attention_tile_rows(False, "tcgen05", d) // (hq // hkv))
    q_len = np.asarray(q_lens, np.int32)
    q_start = np.asarray([0, 200], np.int32)
    arrays = cut_tiles(q_start, q_len, per_tile)
    firsts = rc.numpy()[arrays[1]]
    kernel = K().attention_prompt_kernel(hq, hkv, d, 16, cap)
    assert kernel == "tcgen05"
    from kapel_b200.engine.batch import prompt_costs_of

    split, slots = prompt_split(firsts, firsts + arrays[2] - 1, hkv, sms, window, int(q_len.sum()), hq, d, prompt_costs_of(kernel, d))
    tiles = tuple(dev(torch.from_numpy(a)) for a in arrays)
    sample = [0, 1, 144, 145, 146, 147, 199, 200, 201, 263, 264, 200 + 1023, 200 + 2047]     # rows 145/146 see 4,096/4,097 positions
    want = paged_reference(q, kt, vt, bt, re, rc, 16, window, scale, cap, only=sample)
    # as the planner cuts it, and cut into slots of 1,024 keys whatever the planner thinks of that
    for split, slots in {(split, slots), (1024, -(-4150 // 1024))}:
        got = K().paged_attention_mma(dev(q), dev(kt), dev(vt), dev(bt), dev(rc), tiles, 16, window, scale, cap, 0, split, slots).cpu().double()
        K().check_async_errors()
        assert rel_err(got[sample].numpy(), want[sample].numpy()) < 1.5e-2, f"prompt, split {split} x {slots}"


# ------------------------------------------------------------------------------------------
def test_split_sums_are_added_up_by_their_readers():
    """A decode-size product split over K stays a stack of partial sums; the norm, the gated unit
    and the rotation add the slices up themselves and give what they give for the finished sum."""
    m, k = 5, 2304
    a = rnd(m, k, seed=30, dtype=torch.bfloat16)
    for n in (2304, 4096):
        w = rnd(n, k, seed=31, dtype=torch.bfloat16, scale=0.05)
        split = K().gemm(dev(a), dev(w), keep_split=True)
        assert isinstance(split, K().SplitSum) and split.splits > 1 and split.shape == (m, n)
        whole = K().gemm(dev(a), dev(w), out_dtype=torch.float32)
        done = K().finish(split, torch.float32)
        assert torch.equal(done, whole), "the same kernel and the same order of additions"
        assert rel_err(done.cpu().numpy(), (a.double() @ w.double().T).numpy()) < 2e-5
    # the residual sum with both norms
    n = 2304
    w = rnd(n, k, seed=32, dtype=torch.bfloat16, scale=0.05)
    split = K().gemm(dev(a), dev(w), keep_split=True)
    branch = (a.double() @ w.double().T)
    res = rnd(m, n, seed=33)
    w1, w2 = rnd(n, seed=34, dtype=torch.bfloat16, scale=0.1), rnd(n, seed=35, dtype=torch.bfloat16, scale=0.1)
    r = dev(res.clone())
    h = K().add_rmsnorm(r, split, (dev(w1), 1e-6, 1.0), (dev(w2), 1e-6, 1.0), torch.bfloat16)
    want_r = res.double() + P.rms_norm(branch, w1.double(), 1e-6)
    assert rel_err(r.cpu().double().numpy(), want_r.numpy()) < 1e-5
    assert rel_err(h.cpu().double().numpy(), P.rms_norm(want_r, w2.double(), 1e-6).numpy()) < 1e-2
    # the gated unit
    n = 2 * 1152
    w = rnd(n, k, seed=36, dtype=torch.bfloat16, scale=0.05)
    split = K().gemm(dev(a), dev(w), keep_split=True)
    assert isinstance(split, K().SplitSum)
    x = a.double() @ w.double().T
    got = K().glu(split, "gelu_tanh", out_dtype=torch.bfloat16).cpu().double()
    assert rel_err(got.numpy(), (P.gelu_tanh(x[:, :1152]) * x[:, 1152:]).numpy()) < 1e-2
    # the rotation and the cache append
    hq, hkv, d = 8, 4, 64
    w = rnd((hq + 2 * hkv) * d, k, seed=37, dtype=torch.bfloat16, scale=0.05)
    split = K().gemm(dev(a), dev(w), keep_split=True)
    assert isinstance(split, K().SplitSum)
    pos = torch.tensor([0, 3, 9, 100, 7], dtype=torch.int32)
    lines = torch.tensor([4, 0, 9, -1, 2], dtype=torch.int32)
    kt = torch.zeros(1, hkv, 10, d, dtype=torch.bfloat16).cuda()         # one page of 10 lines
    vt = torch.zeros(1, hkv, 10, d, dtype=torch.bfloat16).cuda()
    cs = K().rope_table(dev(pos), d, 10000.0)
    q = K().rope_append(split, cs, dev(lines), kt, vt, hq, hkv, d, d, out_dtype=torch.bfloat16).cpu().double()
    x = (a.double() @ w.double().T).reshape(m, hq + 2 * hkv, d)
    assert rel_err(q.numpy(), P.rope(x[:, :hq], pos, 10000.0).numpy()) < 1e-2
    assert rel_err(kt.cpu().double()[0, :, 4].numpy(), P.rope(x[:, hq : hq + hkv], pos, 10000.0)[0].numpy()) < 1e-2
    assert rel_err(vt.cpu().double()[0, :, 9].numpy(), x[2, hq + hkv :].numpy()) < 1e-2


@pytest.mark.parametrize("rows", [1, 8, 9, 64, 200])
@pytest.mark.parametrize("width", [40, 520, 2304, 4608, 8200])
@pytest.mark.parametrize("splits", [2, 8, 9, 16, 17, 35])
def test_add_rmsnorm_over_split_sums_at_other_sizes(rows, width, splits):
    """The residual sum with both norms over a stack of float32 partial sums: 2 to 35 slices (full
    batches of eight in flight and what is left over), widths that leave a thread without a group of
    four, with and without either norm; and a row's result does not depend on how many rows came
    with it."""
    g = torch.Generator().manual_seed(rows * 1000 + width + splits)
    parts = (torch.randn(splits, rows, width, generator=g) * 0.7).float()
    res = torch.randn(rows, width, generator=g).float() * 2
    w1 = (torch.randn(width, generator=g) * 0.1).bfloat16()
    w2 = (torch.randn(width, generator=g) * 0.1).bfloat16()
    branch = parts.double().sum(0)
    for post, nxt in [(True, True), (True, False), (False, True)]:
        r = dev(res.clone())
        h = K().add_rmsnorm(r, K().SplitSum(dev(parts)), (dev(w1), 1e-6, 1.0) if post else None, (dev(w2), 1e-5, 1.0) if nxt else None,
                            torch.bfloat16)
        b = P.rms_norm(branch, w1.double(), 1e-6) if post else branch
        want_r = res.double() + b
        assert rel_err(r.cpu().double().numpy(), want_r.numpy()) < 2e-6
        if nxt:
            assert rel_err(h.cpu().double().numpy(), P.rms_norm(want_r, w2.double(), 1e-5).numpy()) < 1e-2
    if rows > 1:
        r_all, r_one = dev(res.clone()), dev(res[:1].clone())
        h_all = K().add_rmsnorm(r_all, K().SplitSum(dev(parts)), (dev(w1), 1e-6, 1.0), (dev(w2), 1e-5, 1.0), torch.bfloat16)
        h_one = K().add_rmsnorm(r_one, K().SplitSum(dev(parts[:, :1].contiguous())), (dev(w1), 1e-6, 1.0), (dev(w2), 1e-5, 1.0), torch.bfloat16)
        if rows <= 64:
            assert torch.equal(r_all[:1], r_one) and torch.equal(h_all[:1], h_one), "the same kernel and the same order of additions"
        else:                                             # more rows than a decode step has go through another kernel
            assert rel_err(r_all[:1].cpu().double().numpy(), r_one.cpu().double().numpy()) < 1e-6
            assert rel_err(h_all[:1].cpu().double().numpy(), h_one.cpu().double().numpy()) < 1e-2


@pytest.mark.parametrize("m", [65, 130, 300, 512, 1000])
@pytest.mark.parametrize("n,k", [(2304, 9216), (2304, 2048), (4096, 2304), (72, 1000 * 8), (520, 4104)])
def test_products_of_a_few_hundred_rows_split_over_k(m, n, k):
    """A prompt portion's product by a narrow weight is cut over K (by the few-rows kernels up to 256
    rows, by the many-rows kernel beyond) and comes back as partial sums when the caller can take
    them; finished, they are the product, and the readers that add slices up themselves get the same."""
    a, w = rnd(m, k, seed=m + n, dtype=torch.bfloat16), rnd(n, k, seed=m + k, dtype=torch.bfloat16, scale=0.05)
    want = a.double() @ w.double().T
    kept = K().gemm(dev(a), dev(w), keep_split=True)
    K().check_async_errors()
    got = K().finish(kept, torch.float32).cpu().double() if isinstance(kept, K().SplitSum) else kept.cpu().double()
    assert rel_err(got.numpy(), want.numpy()) < (2e-5 if isinstance(kept, K().SplitSum) else 1e-2)
    whole = K().gemm(dev(a), dev(w), out_dtype=torch.float32).cpu().double()
    assert rel_err(whole.numpy(), want.numpy()) < 2e-5
    if isinstance(kept, K().SplitSum) and n == 2304:
        res = rnd(m, n, seed=3)
        w1, w2 = rnd(n, seed=4, dtype=torch.bfloat16, scale=0.1), rnd(n, seed=5, dtype=torch.bfloat16, scale=0.1)
        r = dev(res.clone())
        h = K().add_rmsnorm(r, kept, (dev(w1), 1e-6, 1.0), (dev(w2), 1e-6, 1.0), torch.bfloat16)
        want_r = res.double() + P.rms_norm(want, w1.double(), 1e-6)
        assert rel_err(r.cpu().double().numpy(), want_r.numpy()) < 1e-5
        assert rel_err(h.cpu().double().numpy(), P.rms_norm(want_r, w2.double(), 1e-6).numpy()) < 1e-2


@pytest.mark.parametrize("m", [1, 7, 8, 9, 16])
def test_gemm_bf16_rows_up_to_16_do_not_depend_on_the_batch(m):
    a, w = rnd(16, 2304, seed=38, dtype=torch.bfloat16), rnd(520, 2304, seed=39, dtype=torch.bfloat16)
    whole = K().gemm(dev(a[:m]), dev(w), out_dtype=torch.float32).cpu()
    alone = K().gemm(dev(a[m - 1 : m]), dev(w), out_dtype=torch.float32).cpu()
    assert torch.equal(whole[m - 1 : m], alone)
