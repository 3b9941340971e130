"""Tensor-level entry points of the CUDA library (`kapel_b200/csrc`).

Every function here checks devices, dtypes, shapes and contiguity, then calls one C launcher
on torch's current stream. There is no other implementation behind them: without the built
library, or without a CUDA device, they raise. Tensors are torch tensors only as owners of
device memory; no torch operator computes anything on this path.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

_lib = None
_lock = threading.Lock()

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}

ACT_CODES = {"gelu_tanh": 0, "silu": 1}

# Which kernel multiplies more than 64 rows of bfloat16: "tcgen05" (TMA, TMEM, tcgen05.mma; the
# library picks between one block a tile and persistent pairs of blocks, "single" and "pair" force
# one) or "mma" (the warp-level mma.sync tile kernel, kept as the yardstick the tcgen05 kernels are
# measured against).
import os as _os

GEMM_LARGE = _os.environ.get("KAPEL_B200_GEMM_LARGE", "tcgen05")
# Which kernel multiplies up to 64 rows of bfloat16: "skinny" (tcgen05 with the operands swapped: the
# weights stream through shared memory by TMA) or "stream" (the mma.sync kernels that read the weights
# straight into registers).
GEMM_SMALL = _os.environ.get("KAPEL_B200_GEMM_SMALL", "skinny")
# Which kernel runs attention over prompt portions where both apply: "tcgen05" (products by
# tcgen05.mma, scores and probabilities in tensor memory) or "mma" (the mma.sync flash kernel, which
# also takes what the first does not: no soft cap, other head sizes).
ATTENTION_PROMPT = _os.environ.get("KAPEL_B200_ATTENTION_PROMPT", "tcgen05")
# Whether the tcgen05 prompt attention runs on pairs of blocks (tcgen05.mma.cta_group::2, 256 rows to one
# tile of 128 keys and values): 0 never, 1 at both head sizes that have such a kernel (128 and 256), 2 (the
# default) where it measured faster than single blocks (256).
ATTENTION_PAIRS = int(_os.environ.get("KAPEL_B200_ATTENTION_PAIRS", "2"))
# Whether the kernels of a decode step are launched as programmatic dependents of one another, so
# that a kernel sets up (and asks for its first weights) while the one before it finishes.
PDL = _os.environ.get("KAPEL_B200_PDL", "1") == "1"


class KernelError(RuntimeError):
    """A launcher refused its arguments or a launch failed; the message is the library's."""


def library():
    """The loaded library; builds it at the first call if it is missing or stale."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                from ..csrc.build import ensure_built

                path = ensure_built()
                lib = ctypes.CDLL(str(path))
                lib.kb_last_error.restype = ctypes.c_char_p
                for name in ("kb_gemm_bf16_scratch_floats", "kb_paged_attention_scratch_floats", "kb_attention_mma_scratch_floats", "kb_sample_scratch_floats"):
                    getattr(lib, name).restype = ctypes.c_longlong
                lib.kb_launch_count.restype = ctypes.c_ulonglong
                lib.kb_set_pdl(1 if PDL else 0)
                _lib = lib
    return _lib


def check_async_errors() -> None:
    """Raises if a bounded wait inside a kernel (on an mbarrier: a TMA copy or a tensor-core
    commit that never arrived) ran out since the last check. Synchronises the device."""
    lib = library()
    bad = []
    if lib.kb_attention_error() != 0:
        bad.append("paged attention (a bulk copy into shared memory never completed)")
    if lib.kb_tcgen05_error() != 0:
        bad.append("tcgen05 product (a TMA load or an MMA commit never arrived)")
    if lib.kb_attention_tc_error() != 0:
        bad.append("tcgen05 attention (a TMA load, an MMA commit or a softmax warp never arrived)")
    if lib.kb_rope_error() != 0:
        bad.append("rotate and append (a bulk copy of partial sums into shared memory never completed)")
    if lib.kb_norm_error() != 0:
        bad.append("add-and-norm (a bulk copy of partial sums into shared memory never completed)")
    if bad:
        raise KernelError("a wait inside a kernel gave up after its time limit: " + "; ".join(bad))


def wait_probe(limit_clocks: int = 2_000_000) -> None:
    """Launches one small block whose bounded wait (the products' own) runs out after
    `limit_clocks` because nothing ever arrives at its barrier. For testing that the flag reaches
    `check_async_errors` and that the device goes on working afterwards."""
    _check(library().kb_wait_probe(ctypes.c_longlong(int(limit_clocks)), _stream()))


def launch_count() -> int:
    """Kernels launched (or recorded under a graph capture) by this library so far."""
    return int(library().kb_launch_count())


def library_path() -> str:
    library()
    from ..csrc.build import ensure_built

    return str(ensure_built(verbose=False))


def _check(code: int) -> None:
    if code != 0:
        raise KernelError(library().kb_last_error().decode("utf-8", "replace"))


# torch's current stream as a raw handle. The public route (torch.cuda.current_stream) builds a
# Stream object and resolves the device each time, about 15 us a call, once a kernel: more host
# time than everything else a launch does. torch's own C entry points give the same handle in
# well under a microsecond; without them the public route stands.
_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_RAW_DEVICE = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    if _RAW_STREAM is not None and _RAW_DEVICE is not None:
        return ctypes.c_void_p(_RAW_STREAM(_RAW_DEVICE()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _dt(t: torch.Tensor, what: str) -> int:
    if t.dtype not in _CODES:
        raise KernelError(f"{what}: dtype {t.dtype} is not float32 or bfloat16")
    return _CODES[t.dtype]


def _need(t: torch.Tensor, what: str, dtype=None, shape=None) -> torch.Tensor:
    if not t.is_cuda:
        raise KernelError(f"{what}: tensor is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{what}: tensor is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dtype}")
    if shape is not None:
        if len(shape) != t.dim() or any(s is not None and s != a for s, a in zip(shape, t.shape)):
            raise KernelError(f"{what}: shape {tuple(t.shape)}, expected {tuple(shape)}")
    return t


def _f(x: float) -> ctypes.c_float:
    return ctypes.c_float(float(x))


# With KAPEL_B200_POISON=1 every buffer a kernel is about to write (outputs, scratch, split-K partial
# sums) is first filled with NaN, so that a kernel which reads what nobody wrote, or leaves part
# of its output unwritten, shows in the logits instead of passing on whatever the allocator left
# there. Kapel's debugging switch of the same kind is `poison_buffers` (crates/kapel-cuda/src/device.rs:1019).
POISON = _os.environ.get("KAPEL_B200_POISON", "0") == "1"


def set_poison(on: bool) -> None:
    global POISON
    POISON = bool(on)


_fail_allocation_in = 0


def fail_allocation_in(calls: int) -> None:
    """Failure injection on the host, for tests: the `calls`-th buffer asked for from now on is
    refused with torch's out-of-memory error, as if the device had no room (0 turns it off)."""
    global _fail_allocation_in
    _fail_allocation_in = int(calls)


def _fresh(shape, dtype, device) -> torch.Tensor:
    """A new buffer for a kernel to write; NaN all over in the poisoning mode."""
    global _fail_allocation_in
    if _fail_allocation_in > 0:
        _fail_allocation_in -= 1
        if _fail_allocation_in == 0:
            raise torch.OutOfMemoryError(f"injected: no room for a buffer of shape {tuple(shape)}")
    t = torch.empty(tuple(shape), dtype=dtype, device=device)
    if POISON and dtype in _CODES and t.numel():
        _check(library().kb_poison(_ptr(t), _CODES[dtype], ctypes.c_longlong(t.numel()), _stream()))
    return t


def fill_rows(table: torch.Tensor, rows: torch.Tensor, value: float = 0.0) -> None:
    """table[rows[i]] = value for a float32 table [n, ...] and int32 row numbers on the device."""
    _need(table, "fill_rows table", torch.float32)
    _need(rows, "fill_rows rows", torch.int32)
    if table.dim() < 1 or table.shape[0] == 0 or rows.numel() == 0:
        return
    width = table.numel() // table.shape[0]
    _check(library().kb_fill_rows_f32(_ptr(table), _ptr(rows), int(rows.numel()), ctypes.c_longlong(width), int(table.shape[0]),
                                      _f(value), _stream()))


class SplitSum:
    """A product that is still a stack of split-K partial sums: `partials` is float32
    [splits, rows, cols] and the value is their sum over the first dimension. The kernels that
    read a product next (the norm with the residual sum, the gated unit, the rotation) add the
    slices up on the way in, so the sum is never written out and read back; `finish` does it
    for anything else."""

    __slots__ = ("partials",)

    def __init__(self, partials: torch.Tensor):
        self.partials = partials

    @property
    def shape(self):
        return tuple(self.partials.shape[1:])

    @property
    def splits(self) -> int:
        return int(self.partials.shape[0])

    @property
    def device(self):
        return self.partials.device


def _src(x, what: str):
    """(tensor to read, dtype code, slices, elements between slices) of a tensor or a SplitSum."""
    if isinstance(x, SplitSum):
        t = _need(x.partials, what, torch.float32)
        return t, F32, x.splits, t.shape[1] * t.shape[2]
    _need(x, what)
    return x, _dt(x, what), 1, 0


def finish(x, dtype: torch.dtype) -> torch.Tensor:
    """A SplitSum added up into a tensor of `dtype`; a tensor as it is (cast if need be)."""
    if isinstance(x, SplitSum):
        _need(x.partials, "finish partials", torch.float32)
        out = _fresh(x.shape, dtype, x.device)
        _check(library().kb_splitk_reduce(_ptr(out), _dt(out, "finish output"), _ptr(x.partials),
                                          ctypes.c_longlong(out.numel()), x.splits, _stream()))
        return out
    return x if x.dtype == dtype else cast(x, dtype)


# ------------------------------------------------------------------------------------------
def embed(table: torch.Tensor, ids: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = table[ids[r]] * scale in float32."""
    _need(table, "embed table")
    _need(ids, "embed ids", torch.int32)
    vocab, width = table.shape
    rows = ids.numel()
    if out is None:
        out = _fresh((rows, width), torch.float32, table.device)
    _need(out, "embed out", torch.float32, (rows, width))
    _check(library().kb_embed(_ptr(out), _ptr(table), _dt(table, "embed table"), _ptr(ids), rows, width, vocab, _f(scale), _stream()))
    return out


def rope_table(positions: torch.Tensor, rotary: int, theta: float) -> torch.Tensor:
    """[rows, rotary/2, 2] float32 of (cos, sin); angles in float64 on the device."""
    _need(positions, "rope positions", torch.int32)
    rows = positions.numel()
    out = _fresh((rows, rotary // 2, 2), torch.float32, positions.device)
    _check(library().kb_rope_table(_ptr(out), _ptr(positions), rows, int(rotary), ctypes.c_double(float(theta)), _stream()))
    return out


def rope_append(qkv, cos_sin, lines, k_table, v_table, hq: int, hkv: int, d: int, rotary: int, write_kv: bool = True,
                out_dtype: Optional[torch.dtype] = None):
    """Rotates the q and k heads of the stacked product `qkv` [rows, (hq + 2 hkv) d] (a tensor or a
    SplitSum), returns q [rows, hq, d], and writes k and v at each row's line (page * page_size +
    offset) of the tables [pages, hkv, page_size, d]."""
    src, in_dt, splits, stride = _src(qkv, "rope_append qkv")
    rows = qkv.shape[0]
    if tuple(qkv.shape) != (rows, (hq + 2 * hkv) * d):
        raise KernelError(f"rope_append: qkv {tuple(qkv.shape)}, expected {(rows, (hq + 2 * hkv) * d)}")
    out_dtype = out_dtype or (src.dtype if not isinstance(qkv, SplitSum) else k_table.dtype)
    if rotary:
        _need(cos_sin, "rope_append cos_sin", torch.float32, (rows, rotary // 2, 2))
    q = _fresh((rows, hq, d), out_dtype, src.device)
    table_lines, page_size = 0, 0
    if write_kv:
        _need(lines, "rope_append lines", torch.int32, (rows,))
        _need(k_table, "rope_append k table", out_dtype)
        _need(v_table, "rope_append v table", out_dtype)
        if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[3] != d or v_table.shape != k_table.shape:
            raise KernelError(f"rope_append: tables {tuple(k_table.shape)} / {tuple(v_table.shape)} are not [pages, {hkv}, page_size, {d}]")
        table_lines = k_table.shape[0] * k_table.shape[2]
        page_size = k_table.shape[2]
    _check(
        library().kb_rope_append(
            _ptr(src), in_dt, splits, ctypes.c_longlong(stride), _ptr(cos_sin if rotary else None),
            _ptr(lines if write_kv else None), _ptr(q), _ptr(k_table if write_kv else None), _ptr(v_table if write_kv else None),
            _dt(q, "rope_append output"), rows, hq, hkv, d, int(rotary), int(bool(write_kv)), ctypes.c_longlong(table_lines), int(page_size), _stream(),
        )
    )
    return q


def glu(x, activation: str, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """act(x[:, :n]) * x[:, n:] for a stacked gate|up product (a tensor or a SplitSum)."""
    src, in_dt, splits, stride = _src(x, "glu input")
    if activation not in ACT_CODES:
        raise KernelError(f"glu: activation {activation!r} is not known")
    rows, two_n = x.shape
    n = two_n // 2
    out_dtype = out_dtype or (src.dtype if not isinstance(x, SplitSum) else torch.bfloat16)
    out = _fresh((rows, n), out_dtype, src.device)
    _check(library().kb_glu(_ptr(out), _dt(out, "glu output"), _ptr(src), in_dt, splits, ctypes.c_longlong(stride),
                            ctypes.c_longlong(rows), n, ACT_CODES[activation], _stream()))
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _need(x, "cast input")
    out = _fresh(x.shape, dtype, x.device)
    _check(library().kb_cast(_ptr(out), _dt(out, "cast output"), _ptr(x), _dt(x, "cast input"), ctypes.c_longlong(x.numel()), _stream()))
    return out


def gather_rows(x: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    _need(x, "gather_rows input", torch.float32)
    _need(rows, "gather_rows rows", torch.int32)
    n, width = rows.numel(), x.shape[1]
    out = _fresh((n, width), torch.float32, x.device)
    _check(library().kb_gather_rows_f32(_ptr(out), _ptr(x), _ptr(rows), n, width, x.shape[0], _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, offset: float, out_dtype: torch.dtype) -> torch.Tensor:
    _need(x, "rmsnorm input")
    rows, width = x.shape
    _need(weight, "rmsnorm weight", shape=(width,))
    y = _fresh((rows, width), out_dtype, x.device)
    _check(
        library().kb_rmsnorm(_ptr(y), _dt(y, "rmsnorm output"), _ptr(x), _dt(x, "rmsnorm input"), _ptr(weight),
                             _dt(weight, "rmsnorm weight"), rows, width, _f(eps), _f(offset), _stream())
    )
    return y


def add_rmsnorm(residual, branch, post, nxt, out_dtype):
    """residual += norm_post(branch) (post = (weight, eps, offset) or None: plain add); returns
    norm_next(residual) when nxt = (weight, eps, offset) is given, else None. In place on
    residual. `branch` is a tensor or a SplitSum."""
    rows, width = residual.shape
    _need(residual, "add_rmsnorm residual", torch.float32)
    src, b_dt, splits, stride = _src(branch, "add_rmsnorm branch")
    if tuple(branch.shape) != (rows, width):
        raise KernelError(f"add_rmsnorm: branch {tuple(branch.shape)} against residual {(rows, width)}")
    w_post, eps_post, off_post = post if post is not None else (None, 0.0, 0.0)
    w_next, eps_next, off_next = nxt if nxt is not None else (None, 0.0, 0.0)
    ws = [w for w in (w_post, w_next) if w is not None]
    for w in ws:
        _need(w, "add_rmsnorm weight", shape=(width,))
    if len({w.dtype for w in ws}) > 1:
        raise KernelError("add_rmsnorm: the two norms' weights differ in dtype; call the norms one by one")
    w_dt = _dt(ws[0], "add_rmsnorm weight") if ws else F32
    h = _fresh((rows, width), out_dtype, residual.device) if w_next is not None else None
    _check(
        library().kb_add_rmsnorm(_ptr(residual), _ptr(src), b_dt, splits, ctypes.c_longlong(stride), _ptr(w_post), _f(eps_post),
                                 _f(off_post), _ptr(w_next), _f(eps_next), _f(off_next), _ptr(h), _CODES[out_dtype], w_dt,
                                 rows, width, _stream())
    )
    return h


# Up to 64 rows, and up to SKINNY_ROWS where the kernels for many rows would have few tiles, a
# product streams the weights once through many blocks that split K (the "few-rows" kernels, whose
# MMA takes the rows as its N, up to 256). With one or two row tiles and a narrow weight the kernels
# for many rows leave most multiprocessors idle: the way down of Gemma 2 2B at 128 rows took 50 us by
# 9 blocks against 15 us, o 17 against 7; a wide weight has tiles enough (gate|up: 22 us either way).
SKINNY_ROWS = int(_os.environ.get("KAPEL_B200_SKINNY_ROWS", "256"))
SKINNY_TILES = 24          # tiles of 128 x 256 below which the few-rows kernel is taken beyond 64 rows


def few_rows_product(m: int, n: int) -> bool:
    """Whether a product of m rows by a weight of n rows goes to the few-rows kernels."""
    if m <= 0:
        return False
    if m <= 64:
        return True
    return m <= SKINNY_ROWS and -(-m // 128) * -(-n // 256) <= SKINNY_TILES


def gemm(a: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, softcap: Optional[float] = None,
         keep_split: bool = False):
    """a [m, k] . w [n, k]^T -> [m, n]; float32 x float32 in true 32-bit, bfloat16 x bfloat16 on
    tensor cores with 32-bit sums. `softcap` c applies c * tanh(x / c) to the result. With
    `keep_split`, a product that the kernel splits over K comes back as a SplitSum (its partial
    sums, not yet added up) for a kernel that adds them on the way in."""
    _need(a, "gemm input")
    _need(w, "gemm weight")
    m, k = a.shape
    n, k2 = w.shape
    if k != k2:
        raise KernelError(f"gemm: input [{m}, {k}] against weight [{n}, {k2}]")
    if a.dtype != w.dtype:
        raise KernelError(f"gemm: input {a.dtype} against weight {w.dtype}")
    epi, cap = (1, softcap) if softcap is not None else (0, 0.0)
    lib = library()
    if a.dtype == torch.float32:
        out = _fresh((m, n), torch.float32, a.device)
        _check(lib.kb_gemm_f32(_ptr(out), _ptr(a), _ptr(w), m, n, k, epi, _f(cap), _stream()))
        if out_dtype is not None and out_dtype != torch.float32:
            out = cast(out, out_dtype)
        return out
    out_dtype = out_dtype or torch.bfloat16
    if few_rows_product(m, n) and GEMM_SMALL == "skinny":
        splits = int(lib.kb_gemm_skinny_splits_for(m, n, k))
        if splits == 1:
            out = _fresh((m, n), out_dtype, a.device)
            _check(lib.kb_gemm_skinny(_ptr(out), _dt(out, "gemm output"), None, _ptr(a), _ptr(w), m, n, k, epi, _f(cap), _stream()))
            return out
        if softcap is None:
            partials = _fresh((splits, m, n), torch.float32, a.device)
            _check(lib.kb_gemm_skinny(None, 0, _ptr(partials), _ptr(a), _ptr(w), m, n, k, 0, _f(0.0), _stream()))
            split_sum = SplitSum(partials)
            return split_sum if keep_split else finish(split_sum, out_dtype)
        # a soft cap over partial sums: the streaming kernels' reduction applies it
    if keep_split and softcap is None and 0 < m <= 16:
        splits = int(lib.kb_gemm_bf16_row16_splits(n, k))
        if splits > 1:
            partials = _fresh((splits, m, n), torch.float32, a.device)
            _check(lib.kb_gemm_bf16_partial(_ptr(partials), _ptr(a), _ptr(w), m, n, k, _stream()))
            return SplitSum(partials)
    if keep_split and softcap is None and m > 64 and GEMM_LARGE == "tcgen05":
        # a few hundred rows by a narrow weight: few tiles, each walking all of K; cut over K instead
        splits = int(lib.kb_gemm_tcgen05_splits(m, n, k))
        if splits > 1:
            partials = _fresh((splits, m, n), torch.float32, a.device)
            _check(lib.kb_gemm_tcgen05_split(_ptr(partials), _ptr(a), _ptr(w), m, n, k, _stream()))
            return SplitSum(partials)
    out = _fresh((m, n), out_dtype, a.device)
    if m > 64 and GEMM_LARGE in _TCGEN05_KERNELS:
        _check(lib.kb_gemm_tcgen05(_ptr(out), _dt(out, "gemm output"), _ptr(a), _ptr(w), m, n, k, epi, _f(cap),
                                   _TCGEN05_KERNELS[GEMM_LARGE], _stream()))
        return out
    need = lib.kb_gemm_bf16_scratch_floats(m, n, k)
    scratch = _fresh((need,), torch.float32, a.device) if need else None
    _check(lib.kb_gemm_bf16(_ptr(out), _dt(out, "gemm output"), _ptr(a), _ptr(w), m, n, k, epi, _f(cap), _ptr(scratch), _stream()))
    return out


_TCGEN05_KERNELS = {"tcgen05": 0, "single": 1, "pair": 2}       # the kernel chooses; one block a tile; persistent pairs


def gemm_glu_fused(a: torch.Tensor, w: torch.Tensor, act: str) -> Optional[torch.Tensor]:
    """act(a . gate^T) * (a . up^T) for a stacked gate|up weight w [2 n, k], in one kernel whose
    epilogue applies the gated unit to the 32-bit sums; None where no such kernel applies
    (32-bit operands, the mma.sync yardsticks selected) and the caller multiplies and gates in two steps."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or a.shape[0] == 0:
        return None
    few = a.shape[0] <= 64
    if (few and GEMM_SMALL != "skinny") or (not few and GEMM_LARGE not in ("tcgen05", "pair")):
        return None
    if act not in ACT_CODES:
        raise KernelError(f"gemm_glu: activation {act!r} is not known")
    _need(a, "gemm input")
    _need(w, "gemm weight")
    m, k = a.shape
    n2, k2 = w.shape
    if k != k2 or n2 % 2:
        raise KernelError(f"gemm_glu: input [{m}, {k}] against stacked weight [{n2}, {k2}]")
    out = _fresh((m, n2 // 2), torch.bfloat16, a.device)
    if few:
        _check(library().kb_gemm_skinny_glu(_ptr(out), _ptr(a), _ptr(w), m, n2 // 2, k, ACT_CODES[act], _stream()))
        return out
    _check(library().kb_gemm_tcgen05_glu(_ptr(out), _ptr(a), _ptr(w), m, n2 // 2, k, ACT_CODES[act], _stream()))
    return out


_ATT_CHUNK = None


def attention_chunk() -> int:
    global _ATT_CHUNK
    if _ATT_CHUNK is None:
        _ATT_CHUNK = int(library().kb_attention_chunk())
    return _ATT_CHUNK


def paged_attention_rows(q, k_table, v_table, block_table, row_entry, row_count, page_size: int, window: Optional[int],
                         scale: float, softcap: Optional[float], slots: int) -> torch.Tensor:
    """Attention of each query row over its sequence's pages; `slots` is the largest number of
    key chunks (of `attention_chunk()` positions, cut at absolute multiples) any row touches."""
    rows, hq, d = q.shape
    _need(q, "attention q")
    _need(k_table, "attention k table", q.dtype)
    _need(v_table, "attention v table", q.dtype)
    if k_table.dim() != 4 or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.shape != k_table.shape:
        raise KernelError(f"attention: tables {tuple(k_table.shape)} are not [pages, kv_heads, {page_size}, {d}]")
    n_pages, hkv = k_table.shape[0], k_table.shape[1]
    _need(block_table, "attention block table", torch.int32)
    _need(row_entry, "attention row_entry", torch.int32, (rows,))
    _need(row_count, "attention row_count", torch.int32, (rows,))
    out = _fresh(q.shape, q.dtype, q.device)
    lib = library()
    need = lib.kb_paged_attention_scratch_floats(rows, hq, d, int(slots))
    scratch = _fresh((need,), torch.float32, q.device) if need else None
    _check(
        lib.kb_paged_attention_rows(_ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _dt(q, "attention q"), _ptr(block_table),
                                    _ptr(row_entry), _ptr(row_count), rows, hq, hkv, d, int(page_size), int(block_table.shape[1]),
                                    int(n_pages), int(window or 0), int(slots), _f(scale), _f(softcap or 0.0), _ptr(scratch), _stream())
    )
    return out


def attention_mma_rows(decode: bool) -> int:
    """Rows (token, query head of one kv head's group) a tile of the tensor-core kernel holds."""
    return int(library().kb_attention_mma_rows(int(bool(decode))))


def prompt_pairs(rows: int, longest: int) -> int:
    """The pairs setting for a pass of `rows` query rows whose longest request sees `longest` keys:
    ATTENTION_PAIRS, except that a small pass runs on single blocks (setting 0) where pairs would be
    the default only for head size 256: a pair's launch costs a few microseconds more than it saves
    until there are some hundreds of keys to walk (128 tokens at Gemma 2 2B sizes: 13.4 us on single
    blocks, 17.2 us on pairs; 2,048 tokens: 55 against 42)."""
    if ATTENTION_PAIRS == 2 and rows < 768 and longest < 2048:
        return 0
    return ATTENTION_PAIRS


def attention_tile_rows(decode: bool, prompt_kernel: str = "mma", d: int = 0, pairs: Optional[int] = None) -> int:
    """Rows a tile holds for the kernel that will run: the decode kernel's, the mma.sync prompt
    kernel's, or the tcgen05 prompt kernel's (twice as many where pairs of blocks run it)."""
    if not decode and prompt_kernel == "tcgen05":
        return int(library().kb_attention_tc_rows(int(d), int(ATTENTION_PAIRS if pairs is None else pairs)))
    return attention_mma_rows(decode)


def attention_mma_takes(dtype, d: int, heads_per_kv: int) -> bool:
    """Whether the tensor-core kernel takes these sizes (else the row-wise kernel does)."""
    return dtype == torch.bfloat16 and d % 16 == 0 and d <= 256 and heads_per_kv <= 16


def attention_prompt_kernel(hq: int, hkv: int, d: int, page_size: int, softcap: Optional[float]) -> str:
    """Which kernel `paged_attention_mma` runs for prompt portions of these sizes: "tcgen05" or "mma"."""
    if ATTENTION_PROMPT == "tcgen05" and library().kb_attention_tc_takes(int(hq), int(hkv), int(d), int(page_size), _f(softcap or 0.0)):
        return "tcgen05"
    return "mma"


# KAPEL_B200_DECODE_FUSED=0: the rotation and the cache's newest line stay a kernel of their own
# ahead of the decode attention (the yardstick of the kernel that takes both over). Measured at
# Gemma 2 2B sizes with 6,144 tokens of history, both ways in one call: +2 % at one request, +6 % at 8,
# +4 % at 64. DECODE_FUSED_ROWS is the number of requests from which it is used.
DECODE_FUSED = _os.environ.get("KAPEL_B200_DECODE_FUSED", "1") != "0"
DECODE_FUSED_ROWS = int(_os.environ.get("KAPEL_B200_DECODE_FUSED_ROWS", "1"))


def attention_decode_fused_takes(qkv, hq: int, hkv: int, d: int, rotary: int, page_size: int, dtype: torch.dtype) -> bool:
    """Whether `paged_attention_decode_fused` takes this stacked product: float32 split sums on the
    bfloat16 path, the whole head rotated, sizes the kernel is built for."""
    if not DECODE_FUSED or not isinstance(qkv, SplitSum) or dtype != torch.bfloat16 or rotary != d:
        return False
    if qkv.shape[0] < DECODE_FUSED_ROWS:
        return False
    return bool(library().kb_attention_decode_fused_takes(int(hq), int(hkv), int(d), int(page_size), qkv.splits))


def paged_attention_decode_fused(qkv: "SplitSum", cos_sin, lines, k_table, v_table, block_table, row_count, hq: int, hkv: int,
                                 d: int, write_kv: bool, page_size: int, window: Optional[int], scale: float,
                                 softcap: Optional[float], split: int, slots: int) -> torch.Tensor:
    """A decode step in which every request brings one token (row r is request r), straight from
    the stacked q|k|v product's partial sums: the attention kernel adds up the slices of its row's
    query heads, rotates them, and where a block's keys end with the row's own position it does the
    same for the key and the value, writes them to the cache at `lines[row]` (with `write_kv`) and
    uses them. The result is `rope_append` followed by `paged_attention_mma(decode, relative)`, bit
    for bit, one kernel and one wait between kernels fewer."""
    parts = qkv.partials
    _need(parts, "attention qkv slices", torch.float32)
    splits, rows, width = parts.shape
    if width != (hq + 2 * hkv) * d:
        raise KernelError(f"attention: qkv slices {tuple(parts.shape)}, expected a width of {(hq + 2 * hkv) * d}")
    _need(cos_sin, "attention cos_sin", torch.float32, (rows, d // 2, 2))
    _need(lines, "attention lines", torch.int32, (rows,))
    _need(k_table, "attention k table", torch.bfloat16)
    _need(v_table, "attention v table", torch.bfloat16)
    if k_table.dim() != 4 or k_table.shape[1] != hkv or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.shape != k_table.shape:
        raise KernelError(f"attention: tables {tuple(k_table.shape)} are not [pages, {hkv}, {page_size}, {d}]")
    _need(block_table, "attention block table", torch.int32)
    if block_table.dim() != 2 or block_table.shape[0] < rows:
        raise KernelError(f"attention: a block table of {tuple(block_table.shape)} for {rows} requests")
    _need(row_count, "attention row_count", torch.int32, (rows,))
    out = _fresh((rows, hq, d), torch.bfloat16, parts.device)
    lib = library()
    need = lib.kb_attention_mma_scratch_floats(rows, hq, d, int(slots))
    scratch = _fresh((need,), torch.float32, parts.device) if need else None
    n_pages = k_table.shape[0]
    _check(
        lib.kb_attention_decode_fused(
            _ptr(out), _ptr(parts), int(splits), ctypes.c_longlong(rows * width), _ptr(cos_sin), _ptr(lines), _ptr(k_table),
            _ptr(v_table), int(bool(write_kv)), ctypes.c_longlong(n_pages * page_size), _ptr(block_table), _ptr(row_count), rows,
            hq, hkv, d, int(page_size), int(block_table.shape[1]), int(n_pages), int(window or 0), int(split), int(slots),
            _f(scale), _f(softcap or 0.0), _ptr(scratch), _stream(),
        )
    )
    return out


def paged_attention_mma(q, k_table, v_table, block_table, row_count, tiles, page_size: int, window: Optional[int],
                        scale: float, softcap: Optional[float], decode: int, split: int, slots: int,
                        relative: bool = False, pairs: Optional[int] = None) -> torch.Tensor:
    """Attention over the paged cache on tensor cores (bfloat16). `tiles` = (tile_entry, tile_row0,
    tile_nq) int32 device tensors: each tile is up to `attention_mma_rows(decode) // group` tokens of
    one request at consecutive positions. `decode` is 0 for prompt portions, else the most rows
    (tokens x query heads of a kv head) any tile holds, at most 16. `split` > 0 cuts the keys at
    absolute multiples of it over `slots` blocks (slots >= ceil(longest count / split)). With
    `relative` (decode mode, every tile one token) the multiples are counted from each row's first
    visible key, so a windowed row needs ceil(window / split) slots however long its history."""
    rows, hq, d = q.shape
    _need(q, "attention q", torch.bfloat16)
    _need(k_table, "attention k table", torch.bfloat16)
    _need(v_table, "attention v table", torch.bfloat16)
    if k_table.dim() != 4 or k_table.shape[2] != page_size or k_table.shape[3] != d or v_table.shape != k_table.shape:
        raise KernelError(f"attention: tables {tuple(k_table.shape)} are not [pages, kv_heads, {page_size}, {d}]")
    n_pages, hkv = k_table.shape[0], k_table.shape[1]
    tile_entry, tile_row0, tile_nq = tiles
    n_tiles = tile_entry.numel()
    for t in tiles:
        _need(t, "attention tiles", torch.int32, (n_tiles,))
    _need(block_table, "attention block table", torch.int32)
    _need(row_count, "attention row_count", torch.int32, (rows,))
    out = _fresh(q.shape, q.dtype, q.device)
    lib = library()
    need = lib.kb_attention_mma_scratch_floats(rows, hq, d, int(slots))
    scratch = _fresh((need,), torch.float32, q.device) if need else None
    if not decode and attention_prompt_kernel(hq, hkv, d, page_size, softcap) == "tcgen05":
        _check(
            lib.kb_attention_tc(_ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _ptr(block_table), _ptr(row_count),
                                _ptr(tile_entry), _ptr(tile_row0), _ptr(tile_nq), n_tiles, rows, hq, hkv, d, int(page_size),
                                int(block_table.shape[1]), int(n_pages), int(window or 0), int(split), int(slots), _f(scale),
                                _f(softcap or 0.0), _ptr(scratch), int(ATTENTION_PAIRS if pairs is None else pairs), _stream())
        )
        if slots > 1:
            _check(lib.kb_attention_mma_combine(_ptr(out), _ptr(row_count), _ptr(scratch), rows, hq, d, int(window or 0), int(split),
                                                int(slots), _stream()))
        return out
    _check(
        lib.kb_attention_mma(_ptr(out), _ptr(q), _ptr(k_table), _ptr(v_table), _ptr(block_table), _ptr(row_count),
                             _ptr(tile_entry), _ptr(tile_row0), _ptr(tile_nq), n_tiles, rows, hq, hkv, d, int(page_size),
                             int(block_table.shape[1]), int(n_pages), int(window or 0), int(split), int(slots), _f(scale),
                             _f(softcap or 0.0), int(decode), int(bool(relative) and bool(decode)), _ptr(scratch), _stream())
    )
    return out


def sample(logits: torch.Tensor, temperature: Optional[torch.Tensor] = None, uniform: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token a row: the first largest logit where temperature <= 0 (or none is given), else
    a draw with the row's uniform number."""
    _need(logits, "sample logits", torch.float32)
    rows, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "sample temperature", torch.float32, (rows,))
        _need(uniform, "sample uniform", torch.float32, (rows,))
    out = _fresh((rows,), torch.int32, logits.device)
    lib = library()
    need = int(lib.kb_sample_scratch_floats(rows, vocab))
    scratch = _fresh((need,), torch.float32, logits.device) if need else None
    _check(lib.kb_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(uniform), rows, vocab, _ptr(scratch), _stream()))
    return out


# ------------------------------------------------------------------------------------------
# Timing by kernel name, in the manner of Kapel's `Timed<B>` wrapper backend
# (crates/kapel-cli/examples/profile.rs:17-56): every entry point above is bracketed by CUDA
# events and its device time added up under its name and its largest argument's shape.
_TIMED = ("embed", "rope_table", "rope_append", "glu", "cast", "gather_rows", "rmsnorm", "add_rmsnorm", "gemm",
          "paged_attention_rows", "paged_attention_mma", "sample")
_timing = None
_originals = {}


def enable_timing() -> None:
    """Wraps the entry points with CUDA-event timers (each call then synchronises: for
    measuring where a step's time goes, never while timing the step itself, and not with
    recorded steps)."""
    global _timing
    if _timing is not None:
        return
    _timing = {}
    g = globals()
    for name in _TIMED:
        fn = g[name]
        _originals[name] = fn

        def timed(*args, __fn=fn, __name=name, **kw):
            shape = max((tuple(a.shape) for a in args if isinstance(a, torch.Tensor)), key=lambda s: int(torch.Size(s).numel()), default=())
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            out = __fn(*args, **kw)
            b.record()
            b.synchronize()
            rec = _timing.setdefault((__name, shape), [0, 0.0])
            rec[0] += 1
            rec[1] += a.elapsed_time(b)
            return out

        g[name] = timed


def disable_timing() -> None:
    global _timing
    for name, fn in _originals.items():
        globals()[name] = fn
    _originals.clear()
    _timing = None


def timing_report(reset: bool = True):
    """[(name, shape, calls, total ms)] sorted by total time."""
    rows = sorted(((n, s, c, ms) for (n, s), (c, ms) in (_timing or {}).items()), key=lambda r: -r[3])
    if reset and _timing is not None:
        _timing.clear()
    return rows
