"""The CPU oracle against libraries compiled from the reference's own sources
(oracle/_ref, built by `make -C oracle ref` where the reference tree exists).
Skipped where those libraries are absent; the golden-vector tests then carry
the same pins."""
import ctypes
from ctypes import c_int, c_size_t, c_void_p

import numpy as np
import pytest


def p(a):
    return a.ctypes.data_as(c_void_p)


@pytest.fixture(scope="module")
def ref(oracle):
    lib = oracle.ref_lib()
    if lib is None:
        pytest.skip("oracle/_ref/libchoreo_ref.so not built on this machine")
    return lib


@pytest.fixture(scope="module")
def cuda_codecs(oracle):
    lib = oracle.codec_lib()
    if lib is None:
        pytest.skip("oracle/_ref/libcuda_codecs.so not built on this machine")
    return lib


def test_gemm_loop_bitwise_equals_reference(oracle, ref):
    rng = np.random.default_rng(11)
    ref.ref_mma_exec_row_row_f32.argtypes = [c_void_p] * 4 + [c_int] * 3
    for M, N, K in [(1, 1, 1), (17, 9, 40), (64, 128, 64), (130, 70, 200)]:
        a = oracle.f16_to_f32(oracle.f32_to_f16((rng.random((M, K)) * 2 - 1).astype(np.float32)))
        b = oracle.f16_to_f32(oracle.f32_to_f16((rng.random((N, K)) * 2 - 1).astype(np.float32)))
        want = np.zeros((M, N), np.float32)
        ref.ref_mma_exec_row_row_f32(p(want), p(a), p(b), p(np.zeros((M, N), np.float32)), M, N, K)
        got = oracle.gemm_row_row(a, b, tile=(64, 128, max(K, 1)))
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_hilbert_equals_reference_builder(oracle, ref):
    ref.ref_build_hilbert_schedule.restype = c_int
    ref.ref_build_hilbert_schedule.argtypes = [c_int, c_int, c_void_p, c_void_p]
    for tm in (1, 2, 3, 5, 8, 13, 32):
        for tn in (1, 2, 4, 7, 16, 32):
            sm = np.zeros(4096, np.int32)
            sn = np.zeros(4096, np.int32)
            n = ref.ref_build_hilbert_schedule(tm, tn, p(sm), p(sn))
            om, on = oracle.hilbert_schedule(tm, tn)
            assert n == len(om) == tm * tn
            np.testing.assert_array_equal(om, sm[:n])
            np.testing.assert_array_equal(on, sn[:n])


def test_sparse_encoder_equals_reference_policy(oracle, ref):
    rng = np.random.default_rng(12)
    ref.ref_sparse24_encode_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int]
    for M, K in [(4, 8), (64, 64), (33, 128)]:
        dense = oracle.f16_to_f32(oracle.f32_to_f16((rng.random((M, K)) * 2 - 1).astype(np.float32)))
        keep = np.zeros((M, K // 4, 4), bool)
        for r in range(M):
            for g in range(K // 4):
                keep[r, g, rng.choice(4, rng.integers(0, 5), replace=False)] = True
        dense = np.where(keep.reshape(M, K), dense, 0).astype(np.float32)
        pk = np.zeros((M, K // 2), np.float32)
        meta = np.zeros((M, K // 8), np.uint8)
        ref.ref_sparse24_encode_f32(p(np.ascontiguousarray(dense)), p(pk), p(meta), M, K)
        got_p, got_m = oracle.sparse24_encode(oracle.f32_to_f16(dense))
        np.testing.assert_array_equal(got_m, meta)
        np.testing.assert_array_equal(got_p, oracle.f32_to_f16(pk))


def test_codecs_equal_cuda_host_conversions(oracle, cuda_codecs):
    rng = np.random.default_rng(13)
    x = np.concatenate([rng.standard_normal(200000), rng.standard_normal(100000) * 200,
                        rng.standard_normal(100000) * 1e-3, rng.standard_normal(50000) * 1e-7,
                        rng.standard_normal(50000) * 1e5]).astype(np.float32)
    for name, fn, dt in [("cuda_f32_to_f16_n", oracle.f32_to_f16, np.uint16),
                         ("cuda_f32_to_bf16_n", oracle.f32_to_bf16, np.uint16),
                         ("cuda_f32_to_e4m3_n", oracle.f32_to_e4m3, np.uint8)]:
        want = np.zeros(x.size, dt)
        f = getattr(cuda_codecs, name)
        f.argtypes = [c_void_p, c_void_p, c_size_t]
        f(p(x), p(want), x.size)
        np.testing.assert_array_equal(fn(x), want, err_msg=name)
