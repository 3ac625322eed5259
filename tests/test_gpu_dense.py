"""GPU parity of the persistent f16/bf16 GEMM (croq_matmul_f16/bf16) against
the CPU oracle, through the C ABI. Shapes and tolerances follow the
reference's own tests (tests/gpu/end2end/wgmma_persis.co:200-258,
wgmma_ss.co:312-404); the stricter bound is max relative error 5e-3."""
import hashlib

import numpy as np
import pytest
import torch

from croqtile_b200 import api, hilbert_schedule, row_major_schedule
from croqtile_b200._lib import CroqError
from tests.gpu_util import bits_of, max_rel_err, poisoned, to_dev, to_dev_16
from tests.test_oracle_golden import kat1_inputs

pytestmark = pytest.mark.gpu
REL_TOL = 5e-3  # f16/bf16 inputs, fp32 accumulation


def run_matmul(oracle, lhs_f32, rhs_f32, dtype, sched=None, tile=(256, 256)):
    """Rounds inputs to `dtype`, runs the library and the oracle on the same bits."""
    lb, rb = oracle.round_to(lhs_f32, dtype), oracle.round_to(rhs_f32, dtype)
    M, N = lb.shape[0], rb.shape[0]
    out = poisoned((M, N), dtype)
    sm = sn = None
    if sched is not None:
        sm, sn = to_dev(sched[0]), to_dev(sched[1])
    api.matmul(to_dev_16(lb, dtype), to_dev_16(rb, dtype), out, sm, sn, tile[0], tile[1])
    api.synchronize()
    ref = oracle.gemm_row_row(oracle.decode(lb, dtype), oracle.decode(rb, dtype))
    return bits_of(out), ref


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_kat1_mod3_pattern_is_bit_exact(oracle, golden, dtype):
    lhs, rhs = kat1_inputs()
    got, ref = run_matmul(oracle, lhs, rhs, dtype)
    assert hashlib.sha256(ref.tobytes()).digest() == golden["mma_row_row"]["kat1_sha256"].tobytes()
    np.testing.assert_array_equal(got, oracle.round_to(ref, dtype))
    # the reference's own acceptance: full compare, abs tol 0.1
    assert np.abs(oracle.decode(got, dtype) - ref).max() <= 0.1


def test_golden_small_case(oracle, golden):
    g = golden["mma_row_row"]
    out = poisoned((40, 24), "f16")
    api.matmul(to_dev_16(g["lhs_f16"], "f16"), to_dev_16(g["rhs_f16"], "f16"), out)
    api.synchronize()
    assert max_rel_err(oracle.f16_to_f32(bits_of(out)), g["out_f32"], floor=1e-2) <= REL_TOL


def test_config1_f16_512_cubed_row_major_schedule(oracle):
    rng = np.random.default_rng(1001)
    lhs = (rng.random((512, 512)) * 2 - 1).astype(np.float32)
    rhs = (np.random.default_rng(1002).random((512, 512)) * 2 - 1).astype(np.float32)
    got, ref = run_matmul(oracle, lhs, rhs, "f16", sched=row_major_schedule(2, 2))
    assert max_rel_err(oracle.f16_to_f32(got), ref, floor=0.05) <= REL_TOL


def test_reference_persistent_test_shape_hilbert_64x128(oracle):
    """1536x2048x128, uniform(0,2), Hilbert schedule over 64x128 tiles, checked
    with the reference's sampled verifier (256 samples, 0.5 + 0.02|ref|)."""
    rng = np.random.default_rng(5)
    m, n, k = 1536, 2048, 128
    lhs = (rng.random((m, k)) * 2).astype(np.float32)
    rhs = (rng.random((n, k)) * 2).astype(np.float32)
    got, ref = run_matmul(oracle, lhs, rhs, "f16", sched=hilbert_schedule(m // 64, n // 128),
                          tile=(64, 128))
    gotf = oracle.f16_to_f32(got)
    pos = oracle.sample_positions(m, n, 256)
    diff = np.abs(gotf.ravel()[pos] - ref.ravel()[pos])
    assert (diff <= 0.5 + 0.02 * np.abs(ref.ravel()[pos])).all()
    assert max_rel_err(gotf, ref, floor=1.0) <= REL_TOL


@pytest.mark.parametrize("shape,dtype", [((1000, 776, 264), "bf16"), ((70, 130, 72), "f16"),
                                         ((1, 8, 8), "f16"), ((129, 257, 8), "bf16"),
                                         ((300, 520, 1032), "f16")])
def test_ragged_shapes(oracle, shape, dtype):
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + n)
    lhs = (rng.random((m, k)) * 2 - 1).astype(np.float32)
    rhs = (rng.random((n, k)) * 2 - 1).astype(np.float32)
    got, ref = run_matmul(oracle, lhs, rhs, dtype)
    assert max_rel_err(oracle.decode(got, dtype), ref, floor=0.05 * np.sqrt(k)) <= REL_TOL


def test_schedule_order_does_not_change_bits(oracle):
    rng = np.random.default_rng(9)
    m, n, k = 768, 1024, 256
    a = to_dev_16(oracle.f32_to_bf16(rng.standard_normal((m, k)).astype(np.float32)), "bf16")
    b = to_dev_16(oracle.f32_to_bf16(rng.standard_normal((n, k)).astype(np.float32)), "bf16")
    base = bits_of(api.matmul(a, b, poisoned((m, n), "bf16")))
    for tile in [(256, 256), (128, 256), (64, 128), (192, 128), (100, 300)]:
        tm, tn = -(-m // tile[0]), -(-n // tile[1])
        for sched in (hilbert_schedule(tm, tn), row_major_schedule(tm, tn)):
            perm = rng.permutation(tm * tn)
            sm = np.concatenate([sched[0][perm], np.zeros(3, np.int32)])   # T > tiles is allowed
            sn = np.concatenate([sched[1][perm], np.zeros(3, np.int32)])
            out = api.matmul(a, b, poisoned((m, n), "bf16"), to_dev(sm), to_dev(sn), *tile)
            api.synchronize()
            np.testing.assert_array_equal(bits_of(out), base)


def test_bad_schedule_entry_is_reported_not_faulted(oracle):
    a = torch.ones((256, 64), dtype=torch.float16, device="cuda")
    b = torch.ones((256, 64), dtype=torch.float16, device="cuda")
    sm = torch.tensor([0, 7], dtype=torch.int32, device="cuda")   # tile row 7 does not exist
    sn = torch.tensor([0, 0], dtype=torch.int32, device="cuda")
    api.matmul(a, b, poisoned((256, 256), "f16"), sm, sn, 128, 256)
    with pytest.raises(CroqError) as err:
        api.synchronize()
    assert err.value.name == "CROQ_ERR_SCHEDULE"
    api.synchronize()  # status was cleared; the context is still usable
    out = api.matmul(a, b, poisoned((256, 256), "f16"))
    api.synchronize()
    assert (out == 64).all()


def test_k_zero_gives_zeros():
    a = torch.empty((128, 0), dtype=torch.bfloat16, device="cuda")
    b = torch.empty((64, 0), dtype=torch.bfloat16, device="cuda")
    out = api.matmul(a, b, poisoned((128, 64), "bf16"))
    api.synchronize()
    assert (out == 0).all()


def test_config2_bf16_8192_cubed_hilbert_properties(oracle):
    """Full BASELINE size: sampled rows against the oracle, an identity right
    operand (bit-exact copy of lhs), and a checksum of row sums."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(2001)
    lhs = (torch.randn((n, n), generator=g, device="cuda") / np.sqrt(n)).to(torch.bfloat16)
    g.manual_seed(2002)
    rhs = (torch.randn((n, n), generator=g, device="cuda") / np.sqrt(n)).to(torch.bfloat16)
    sm, sn = hilbert_schedule(32, 32)
    sm, sn = to_dev(sm), to_dev(sn)
    out = api.matmul(lhs, rhs, poisoned((n, n), "bf16"), sm, sn, 256, 256)
    api.synchronize()
    rows = np.array([0, 1, 127, 128, 4095, 4096, 8063, 8191])
    ref = oracle.gemm_row_row(oracle.bf16_to_f32(bits_of(lhs[rows])), oracle.bf16_to_f32(bits_of(rhs)),
                              tile=(8, 256, 64))
    got = oracle.bf16_to_f32(bits_of(out[rows]))
    assert max_rel_err(got, ref, floor=0.05) <= REL_TOL
    # checksum of checksums: sum_n out[m,n] == lhs[m,:] . (sum_n rhs[n,:])
    want = lhs.double() @ rhs.double().sum(0)
    gotsum = out.double().sum(1)
    assert ((gotsum - want).abs() <= 0.05 + 1e-2 * want.abs()).all()
    # identity right operand: the product must reproduce lhs bit for bit
    eye = torch.eye(n, dtype=torch.bfloat16, device="cuda")
    out2 = api.matmul(lhs, eye, poisoned((n, n), "bf16"), sm, sn, 256, 256)
    api.synchronize()
    assert torch.equal(out2.view(torch.int16), lhs.view(torch.int16))
