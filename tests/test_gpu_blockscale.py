"""GPU parity of the FP8 e4m3 block-scaled GEMM (croq_blockscale_gemm_e4m3)
against the CPU oracle, through the C ABI. Test instances follow
tests/gpu/end2end/wgmma_persis.co:271-336 and wgmma_ss.co:312-404; the bound is
max relative error 2e-2."""
import numpy as np
import pytest
import torch

from croqtile_b200 import api
from tests.gpu_util import bits_of, max_rel_err, poisoned, to_dev, to_dev_e4m3
from tests.test_oracle_golden import kat1_inputs

pytestmark = pytest.mark.gpu
REL_TOL = 2e-2


def run(oracle, a_q, sa, b_q, sb, dtype="bf16", rows=None):
    out = poisoned((a_q.shape[0], b_q.shape[0]), dtype)
    api.blockscale_gemm_e4m3(to_dev_e4m3(a_q), to_dev(sa), to_dev_e4m3(b_q), to_dev(sb), out)
    api.synchronize()
    ref = oracle.blockscale_gemm_e4m3(a_q, sa, b_q, sb, rows=rows)
    return oracle.decode(bits_of(out), dtype), ref


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_kat1_unit_scales_bit_exact(oracle, dtype):
    lhs, rhs = kat1_inputs()
    got, ref = run(oracle, oracle.f32_to_e4m3(lhs), np.ones((384, 1), np.float32),
                   oracle.f32_to_e4m3(rhs), np.ones((3, 1), np.float32), dtype)
    np.testing.assert_array_equal(got, oracle.decode(oracle.round_to(ref, dtype), dtype))
    assert np.abs(got - ref).max() <= 0.1     # the reference's acceptance for this case


def test_reference_blockscale_instance(oracle):
    """512x2048x128, values uniform(0,2), scales uniform(1,3): the reference's
    256 samples at (37 s mod M, 53 s mod N) within 0.5 + 0.08|ref|."""
    rng = np.random.default_rng(21)
    m, n, k = 512, 2048, 128
    a = oracle.f32_to_e4m3((rng.random((m, k)) * 2).astype(np.float32))
    b = oracle.f32_to_e4m3((rng.random((n, k)) * 2).astype(np.float32))
    sa = (1 + 2 * rng.random((m, 1))).astype(np.float32)
    sb = (1 + 2 * rng.random((n // 128, 1))).astype(np.float32)
    got, ref = run(oracle, a, sa, b, sb, "f16")
    s = np.arange(256)
    r, c = (s * 37) % m, (s * 53) % n
    assert (np.abs(got[r, c] - ref[r, c]) <= 0.5 + 0.08 * np.abs(ref[r, c])).all()
    assert max_rel_err(got, ref, floor=1.0) <= REL_TOL


@pytest.mark.parametrize("shape", [(256, 384, 1024), (200, 136, 272), (1, 128, 128), (130, 260, 4096),
                                   (513, 1000, 400)])
def test_quantised_normal_inputs(oracle, shape):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a, sa = oracle.quant_rows_e4m3(rng.standard_normal((m, k)).astype(np.float32))
    b, sb = oracle.quant_blocks_e4m3(rng.standard_normal((n, k)).astype(np.float32))
    got, ref = run(oracle, a, sa, b, sb)
    assert max_rel_err(got, ref, floor=0.05 * np.sqrt(k)) <= REL_TOL


def test_scale_linearity_is_exact(oracle):
    """Scaling scale_lhs by a power of two scales every output by exactly it."""
    rng = np.random.default_rng(33)
    m, n, k = 384, 512, 768
    a, sa = oracle.quant_rows_e4m3(rng.standard_normal((m, k)).astype(np.float32))
    b, sb = oracle.quant_blocks_e4m3(rng.standard_normal((n, k)).astype(np.float32))
    d = [to_dev_e4m3(a), to_dev(sa), to_dev_e4m3(b), to_dev(sb)]
    base = api.blockscale_gemm_e4m3(*d, poisoned((m, n), "bf16"))
    d[1] = d[1] * 4.0
    quad = api.blockscale_gemm_e4m3(*d, poisoned((m, n), "bf16"))
    api.synchronize()
    assert torch.equal((base.float() * 4.0), quad.float())


def make_config3(m, n, k, seed_a, seed_b):
    """Benchmark recipe: N(0,1) sources, A quantised per 1x128, B per 128x128."""
    g = torch.Generator(device="cuda").manual_seed(seed_a)
    a = torch.randn((m, k), generator=g, device="cuda")
    g.manual_seed(seed_b)
    b = torch.randn((n, k), generator=g, device="cuda")
    amax = a.view(m, k // 128, 128).abs().amax(-1)
    sa = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    aq = (a.view(m, k // 128, 128) / sa[..., None]).view(m, k).to(torch.float8_e4m3fn)
    bmax = b.view(n // 128, 128, k // 128, 128).abs().amax((1, 3))
    sb = torch.where(bmax > 0, bmax / 448.0, torch.ones_like(bmax))
    bq = (b.view(n // 128, 128, k // 128, 128) / sb[:, None, :, None]).view(n, k).to(torch.float8_e4m3fn)
    return aq, sa.contiguous(), bq, sb.contiguous()


@pytest.mark.parametrize("shape", [(4096, 7168, 7168), (8192, 8192, 8192)])
def test_config3_full_size_sampled_rows(oracle, shape):
    m, n, k = shape
    aq, sa, bq, sb = make_config3(m, n, k, 3001, 3002)
    out = api.blockscale_gemm_e4m3(aq, sa, bq, sb, poisoned((m, n), "bf16"))
    api.synchronize()
    assert torch.isfinite(out.float()).all()
    rows = np.array([0, 127, 128, m // 2 + 5, m - 1])
    ref = oracle.blockscale_gemm_e4m3(bits_of(aq[rows]), sa[rows].cpu().numpy(), bits_of(bq),
                                      sb.cpu().numpy())
    got = oracle.bf16_to_f32(bits_of(out[rows]))
    assert max_rel_err(got, ref, floor=0.05 * np.sqrt(k)) <= REL_TOL
    # checksum of checksums over the whole output, per row, in float64 on the device
    deq_b = (bq.float().view(n // 128, 128, k // 128, 128) * sb[:, None, :, None]).view(n, k).double()
    colsum = deq_b.sum(0)
    del deq_b
    deq_a = (aq.float().view(m, k // 128, 128) * sa[..., None]).view(m, k).double()
    want = deq_a @ colsum
    got_sum = out.double().sum(1)
    scale = (deq_a.abs() @ colsum.abs()).clamp_min(1.0)
    assert ((got_sum - want).abs() / scale).max().item() < 2e-3


@pytest.mark.parametrize("shape", [(256, 384, 1024), (200, 136, 272), (513, 1000, 400)])
def test_k_major_lhs_scales_give_identical_bits(oracle, shape):
    """scale_lhs stored [K/128, M] (the `[1, M_tile]` view mma.scale accepts,
    lib/semacheck.cpp:1481-1486): same arithmetic, so the output bits equal the
    row-major call's, on the single-CTA (M <= 128 rows per tile) and pair kernels."""
    m, n, k = shape
    rng = np.random.default_rng(m * 7 + k)
    a, sa = oracle.quant_rows_e4m3(rng.standard_normal((m, k)).astype(np.float32))
    b, sb = oracle.quant_blocks_e4m3(rng.standard_normal((n, k)).astype(np.float32))
    a_d, b_d, sb_d = to_dev_e4m3(a), to_dev_e4m3(b), to_dev(sb)
    row_major = api.blockscale_gemm_e4m3(a_d, to_dev(sa), b_d, sb_d, poisoned((m, n), "bf16"))
    k_major = api.blockscale_gemm_e4m3(a_d, to_dev(np.ascontiguousarray(sa.T)), b_d, sb_d,
                                       poisoned((m, n), "bf16"), scale_lhs_k_major=True)
    api.synchronize()
    np.testing.assert_array_equal(bits_of(k_major), bits_of(row_major))
    ref = oracle.blockscale_gemm_e4m3(a, sa, b, sb)
    assert max_rel_err(oracle.decode(bits_of(k_major), "bf16"), ref, floor=0.05 * np.sqrt(k)) <= REL_TOL
