"""The entry point for callers that cannot allocate device memory (kapel_b200/csrc/no_alloc.h).

Some users of the library run where cudaMalloc is not theirs to call: inside a host application
that owns the device heap, or inside a region where a call that may synchronise the device is
not allowed. `kb_gemm_bf16_no_alloc` gives them the decode-size product with its scratch memory
built into the library. This test calls it through its exported C symbol, as such a caller
would, twice in a row, and checks it against the ordinary entry point. It is collected last, so
a run that stops at the first failure has run every other test before it.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_FLOATS = 4 * 1024 * 1024


def _call(lib, out, a, w, cap=None):
    m, k = a.shape
    n = w.shape[0]
    code = lib.kb_gemm_bf16_no_alloc(
        ctypes.c_void_p(out.data_ptr()), 1 if out.dtype == torch.bfloat16 else 0, ctypes.c_void_p(a.data_ptr()),
        ctypes.c_void_p(w.data_ptr()), m, n, k, 1 if cap else 0, ctypes.c_float(cap or 0.0),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    return code, lib.kb_last_error().decode()


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    from kapel_b200 import kernels as K

    lib = ctypes.CDLL(K.library_path())          # the exported C symbol, not the package's wrapper
    lib.kb_last_error.restype = ctypes.c_char_p
    lib.kb_gemm_bf16_scratch_floats.restype = ctypes.c_longlong
    g = torch.Generator().manual_seed(0)
    # Both products split K (few columns, long rows), so both go through the scratch array; the
    # second is smaller than the first and must not see anything the first left there.
    cases = [((40, 2304), (520, 2304), torch.float32, None), ((3, 9216), (2304, 9216), torch.bfloat16, 30.0)]
    for (ashape, wshape, odt, cap) in cases:
        a = torch.randn(*ashape, generator=g).bfloat16().cuda()
        w = (torch.randn(*wshape, generator=g) * 0.05).bfloat16().cuda()
        assert lib.kb_gemm_bf16_scratch_floats(ashape[0], wshape[0], ashape[1]) > 0, "the case must use scratch"
        out = torch.full((ashape[0], wshape[0]), float("nan"), dtype=odt, device="cuda")
        code, msg = _call(lib, out, a, w, cap)
        assert code == 0, msg
        # the existing entry point, kb_gemm_bf16, with scratch memory that the caller allocates
        need = lib.kb_gemm_bf16_scratch_floats(ashape[0], wshape[0], ashape[1])
        scratch = torch.empty((need,), dtype=torch.float32, device="cuda")
        want = torch.empty_like(out)
        code = lib.kb_gemm_bf16(
            ctypes.c_void_p(want.data_ptr()), 1 if odt == torch.bfloat16 else 0, ctypes.c_void_p(a.data_ptr()),
            ctypes.c_void_p(w.data_ptr()), ashape[0], wshape[0], ashape[1], 1 if cap else 0, ctypes.c_float(cap or 0.0),
            ctypes.c_void_p(scratch.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
        )
        assert code == 0, lib.kb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        ref = a.double().cpu() @ w.double().cpu().T
        if cap:
            ref = cap * torch.tanh(ref / cap)
        tol = 2e-5 if odt == torch.float32 else 1e-2
        err = float((out.double().cpu() - ref).abs().max() / ref.abs().max())
        assert err < tol, err
        assert torch.equal(out, want), "same kernels, same split of K: the same bits as kb_gemm_bf16"


def test_a_product_that_fills_the_built_in_scratch_to_its_end():
    """An accepted product whose partial sums end within a few percent of the array's last value
    (found by asking the library how much each size needs): a bound off by one in the entry point,
    or a split that writes past its share at the far end, would show as a refusal or as other bits
    than kb_gemm_bf16 gives with scratch of the exact size the library asks for."""
    from kapel_b200 import kernels as K

    lib = ctypes.CDLL(K.library_path())
    lib.kb_last_error.restype = ctypes.c_char_p
    lib.kb_gemm_bf16_scratch_floats.restype = ctypes.c_longlong
    best = None
    for m, k in ((64, 1024), (64, 2048), (64, 512), (48, 1024), (16, 2048), (16, 4096)):
        for n in range(65536, 1024, -8):
            need = lib.kb_gemm_bf16_scratch_floats(m, n, k)
            if 0 < need <= MAX_FLOATS and (best is None or need > best[0]):
                best = (need, m, n, k)
    assert best is not None and best[0] >= 0.97 * MAX_FLOATS, f"no size found that fills the array: {best}"
    need, m, n, k = best
    g = torch.Generator().manual_seed(1)
    a = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16().cuda()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    for _ in range(2):                                     # two calls in a row over the same, nearly full array
        code, msg = _call(lib, out, a, w)
        assert code == 0, msg
    scratch = torch.empty((need,), dtype=torch.float32, device="cuda")
    want = torch.empty_like(out)
    code = lib.kb_gemm_bf16(
        ctypes.c_void_p(want.data_ptr()), 0, ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(w.data_ptr()), m, n, k, 0,
        ctypes.c_float(0.0), ctypes.c_void_p(scratch.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
    )
    assert code == 0, lib.kb_last_error().decode()
    torch.cuda.synchronize()
    assert torch.isfinite(out).all() and torch.equal(out, want)
    ref = a.double().cpu() @ w.double().cpu().T
    assert float((out.double().cpu() - ref).abs().max() / ref.abs().max()) < 2e-5
    print(f"[{m}, {k}] x [{n}, {k}]: {need} of {MAX_FLOATS} scratch values")


def test_sizes_beyond_the_built_in_scratch_are_refused():
    from kapel_b200 import kernels as K

    lib = ctypes.CDLL(K.library_path())
    lib.kb_last_error.restype = ctypes.c_char_p
    lib.kb_gemm_bf16_scratch_floats.restype = ctypes.c_longlong
    a = torch.zeros(65, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(65, 8, dtype=torch.bfloat16, device="cuda")
    code, msg = _call(lib, out, a, w)
    assert code != 0 and "at most 64 rows" in msg
    # 64 rows x 37,760 columns x 2 splits of K = 4.8 M values: more than the 4 Mi the array holds
    n, k = 37760, 1024
    assert lib.kb_gemm_bf16_scratch_floats(64, n, k) > MAX_FLOATS
    a = torch.zeros(64, k, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(n, k, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(64, n, dtype=torch.bfloat16, device="cuda")
    code, msg = _call(lib, out, a, w)
    assert code != 0 and "scratch values" in msg
