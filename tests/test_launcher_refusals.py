"""What the kernels' launchers refuse, and how they say it. A launcher checks its sizes before it
touches the device, so a refusal needs no GPU: only the built library (nvcc), which is why these
tests skip where it cannot be built. Every call here must be refused; nothing is launched.
"""
import ctypes

import pytest

vp, i32, i64, f32, f64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double


@pytest.fixture(scope="module")
def lib():
    try:
        from kapel_b200 import kernels as K

        lib = K.library()
    except Exception as err:                                 # no nvcc, no CUDA runtime library
        pytest.skip(f"the CUDA library cannot be built or loaded here: {err}")
    lib.kb_gemm_bf16.argtypes = [vp, i32, vp, vp, i32, i32, i32, i32, f32, vp, vp]
    lib.kb_gemm_tcgen05.argtypes = [vp, i32, vp, vp, i32, i32, i32, i32, f32, i32, vp]
    lib.kb_gemm_skinny.argtypes = [vp, i32, vp, vp, vp, i32, i32, i32, i32, f32, vp]
    lib.kb_gemm_f32.argtypes = [vp, vp, vp, i32, i32, i32, i32, f32, vp]
    lib.kb_rope_table.argtypes = [vp, vp, i32, i32, f64, vp]
    lib.kb_rope_append.argtypes = [vp, i32, i32, i64, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i64, i32, vp]
    lib.kb_glu.argtypes = [vp, i32, vp, i32, i32, i64, i64, i32, i32, vp]
    lib.kb_attention_tc.argtypes = [vp] * 9 + [i32] * 11 + [f32, f32, vp, i32, vp]
    lib.kb_attention_tc_takes.argtypes = [i32, i32, i32, i32, f32]
    return lib


def refused(lib, code, *words):
    assert code != 0
    msg = lib.kb_last_error().decode()
    for w in words:
        assert w in msg, msg
    return msg


A = 4096                                                     # a 16-byte aligned stand-in address; never dereferenced
BF16, F32 = 1, 0


def test_products_refuse_rows_that_are_no_multiple_of_16_bytes_and_unknown_choices(lib):
    refused(lib, lib.kb_gemm_bf16(A, BF16, A, A, 4, 64, 36, 0, 0.0, None, None), "gemm_bf16", "multiple of 8")
    refused(lib, lib.kb_gemm_bf16(A, BF16, A, A, 4, 0, 64, 0, 0.0, None, None), "n 0")
    refused(lib, lib.kb_gemm_bf16(A, 7, A, A, 4, 64, 64, 0, 0.0, None, None), "dtype code 7")
    refused(lib, lib.kb_gemm_bf16(A, BF16, A, A, 4, 64, 64, 1, 0.0, None, None), "epilogue 1 with cap 0")
    refused(lib, lib.kb_gemm_bf16(A, BF16, A + 2, A, 4, 64, 64, 0, 0.0, None, None), "16-byte aligned")
    refused(lib, lib.kb_gemm_tcgen05(A, BF16, A, A, 128, 64, 36, 0, 0.0, 0, None), "gemm_tcgen05", "multiple of 8")
    refused(lib, lib.kb_gemm_tcgen05(A, BF16, A, A, 128, 64, 64, 0, 0.0, 5, None), "kernel choice 5")
    refused(lib, lib.kb_gemm_tcgen05(A, BF16, A, A, 0, 64, 64, 0, 0.0, 0, None), "m 0")
    refused(lib, lib.kb_gemm_skinny(A, BF16, None, A, A, 257, 64, 64, 0, 0.0, None), "gemm_skinny", "m 257 (1..256)")
    refused(lib, lib.kb_gemm_skinny(A, BF16, None, A + 8, A, 8, 64, 64, 0, 0.0, None), "16-byte aligned")
    refused(lib, lib.kb_gemm_f32(A, A, A, 4, 64, 0, 0, 0.0, None), "gemm_f32", "k 0")


def test_rotation_refuses_odd_sizes(lib):
    refused(lib, lib.kb_rope_table(A, A, 4, 7, 10000.0, None), "rope_table", "rotary 7 (must be even)")
    refused(lib, lib.kb_rope_table(A, A, 4, 8, 0.0, None), "theta 0 must be positive")
    refused(lib, lib.kb_rope_append(A, BF16, 1, 0, A, A, A, A, A, BF16, 4, 2, 1, 15, 14, 1, 64, 16, None), "rope_append", "head_dim 15")
    refused(lib, lib.kb_rope_append(A, BF16, 1, 0, A, A, A, A, A, BF16, 4, 2, 1, 16, 18, 1, 64, 16, None), "rotary 18", "at most head_dim 16")
    refused(lib, lib.kb_rope_append(A, BF16, 0, 0, A, A, A, A, A, BF16, 4, 2, 1, 16, 16, 1, 64, 16, None), "0 slices")
    refused(lib, lib.kb_rope_append(A, BF16, 1, 0, A, A, A, A, A, BF16, 4, 2, 1, 16, 16, 1, 64, 0, None), "page_size 0")
    refused(lib, lib.kb_glu(A, BF16, A, BF16, 1, 0, 4, 64, 2, None), "glu", "activation code 2")


def test_tcgen05_attention_says_what_it_takes(lib):
    takes = lib.kb_attention_tc_takes
    assert takes(8, 4, 256, 16, 50.0) == 1 and takes(32, 16, 128, 16, 50.0) == 1 and takes(4, 2, 64, 16, 30.0) == 1
    assert takes(8, 4, 96, 16, 50.0) == 0                    # head sizes 64, 128 and 256 only
    assert takes(8, 4, 128, 16, 0.0) == 0                    # the fixed softmax reference needs a soft cap
    assert takes(8, 4, 128, 16, 100.0) == 0                  # ... of at most 64
    assert takes(8, 3, 128, 16, 50.0) == 0                   # heads must divide into kv heads
    args = [A] * 9 + [1, 64, 8, 4, 96, 16, 8, 8, 0, 0, 1]
    refused(lib, lib.kb_attention_tc(*args, 0.1, 50.0, None, 1, None), "attention_tc", "head_dim 96", "are not taken")
    args = [A] * 9 + [1, 64, 8, 4, 128, 16, 8, 8, 0, 96, 2]
    refused(lib, lib.kb_attention_tc(*args, 0.1, 50.0, None, 1, None), "attention_tc", "split 96")
    assert lib.kb_attention_tc_rows(256, 1) == 256 and lib.kb_attention_tc_rows(128, 1) == 256
    assert lib.kb_attention_tc_rows(64, 1) == 128 and lib.kb_attention_tc_rows(256, 0) == 128
    assert lib.kb_attention_tc_rows(256, 2) == 256 and lib.kb_attention_tc_rows(128, 2) == 128


def test_decode_attention_from_slices_says_what_it_takes(lib):
    takes = lib.kb_attention_decode_fused_takes
    takes.argtypes = [i32, i32, i32, i32, i32]
    assert takes(8, 4, 256, 16, 9) == 1 and takes(32, 16, 128, 16, 5) == 1 and takes(16, 1, 64, 16, 30) == 1
    assert takes(8, 4, 96, 16, 9) == 0                       # head sizes 64, 128 and 256 only
    assert takes(34, 2, 128, 16, 4) == 0                     # at most 16 query heads a kv head
    assert takes(8, 3, 128, 16, 4) == 0                      # heads must divide into kv heads
    assert takes(8, 4, 256, 24, 9) == 0                      # pages of a multiple of 16 positions
    assert takes(8, 4, 256, 16, 12) == 1 and takes(8, 4, 256, 16, 13) == 0     # thirteen slices of two heads of 256 do not fit beside the pipelines
    assert takes(8, 4, 256, 16, 0) == 0
    fused = lib.kb_attention_decode_fused
    fused.argtypes = [vp, vp, i32, i64, vp, vp, vp, vp, i32, i64, vp, vp] + [i32] * 10 + [f32, f32, vp, vp]

    def call(parts=A, splits=9, stride=8 * 4096, d=256, split=1024, slots=4, scratch=A, hq=8, hkv=4):
        return fused(A, parts, splits, stride, A, A, A, A, 1, 1 << 20, A, A, 8, hq, hkv, d, 16, 64, 4096, 0, split, slots,
                     0.1, 50.0, scratch, None)

    refused(lib, call(d=96), "attention_decode_fused", "not taken")
    refused(lib, call(parts=A + 4), "multiples of 16 bytes")
    refused(lib, call(stride=8 * 4096 + 1), "multiples of 16 bytes")
    refused(lib, call(split=100), "split 100")
    refused(lib, call(scratch=None), "4 slots need scratch memory")
    refused(lib, call(hq=9), "heads 9 over 4")
