"""GPU parity of the MoE path (routing, permutation, quantiser, grouped GEMM,
combine) against the CPU oracle, through the C ABI. The reference has no MoE
code; the oracle's definitions are normative. Integer results (indices,
counts, offsets, permutation maps, quantised bytes) must match bit for bit."""
import numpy as np
import pytest
import torch

from croqtile_b200 import api
from croqtile_b200._lib import CroqError
from tests.gpu_util import bits_of, max_rel_err, to_dev, to_dev_16, to_dev_e4m3

pytestmark = pytest.mark.gpu


def check_routing(oracle, logits, k, norm=True):
    got = api.moe_route_topk(to_dev(logits), k, norm)
    api.synchronize()
    ref = oracle.moe_route_topk(logits, k, norm)
    for key in ("topk_idx", "expert_counts", "expert_offsets", "perm_to_src", "src_to_perm"):
        np.testing.assert_array_equal(got[key].cpu().numpy(), ref[key], err_msg=key)
    np.testing.assert_allclose(got["topk_w"].cpu().numpy(), ref["topk_w"], rtol=1e-5, atol=1e-9)
    return got, ref


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (64, 256, 8), (1000, 256, 8), (333, 64, 6), (130, 384, 4),
                                   (77, 1000, 32), (4096, 256, 8)])
def test_routing_bit_exact(oracle, T, E, k):
    rng = np.random.default_rng(T * 31 + E)
    check_routing(oracle, rng.standard_normal((T, E)).astype(np.float32), k)


def test_routing_ties_signed_zero_and_inf(oracle):
    rng = np.random.default_rng(9)
    logits = rng.standard_normal((256, 256)).astype(np.float32)
    logits[0] = 0.0                       # all equal
    logits[1, ::2] = -0.0                 # +0 and -0 compare equal: index decides
    logits[1, 1::2] = 0.0
    logits[2, 5] = logits[2, 200] = 9.0   # duplicate maximum
    logits[3, :] = -np.inf
    logits[3, 17] = 1.0
    logits[4, 3] = np.inf
    logits[5] = np.round(logits[5] * 2) / 2   # many ties
    check_routing(oracle, logits, 8)
    check_routing(oracle, logits[:, :32].copy(), 4, norm=False)


def test_routing_skewed_and_empty_experts(oracle):
    rng = np.random.default_rng(10)
    logits = rng.standard_normal((2048, 256)).astype(np.float32)
    logits[:, :8] += 20.0                 # every token picks experts 0..7: the rest stay empty
    got, ref = check_routing(oracle, logits, 8)
    assert (ref["expert_counts"][8:] == 0).all() and ref["expert_counts"][:8].min() == 2048


def test_config5_routing_full_size(oracle):
    """T=16384, E=256, top-8: bit-exact integers plus permutation properties."""
    logits = np.random.default_rng(5002).standard_normal((16384, 256)).astype(np.float32)
    got, ref = check_routing(oracle, logits, 8)
    p2s = got["perm_to_src"].long()
    assert torch.equal(got["src_to_perm"][p2s].long(), torch.arange(16384 * 8, device="cuda"))
    assert int(got["expert_offsets"][-1]) == 16384 * 8


def test_permute_and_combine_bit_exact(oracle):
    rng = np.random.default_rng(11)
    T, E, k, H = 512, 64, 4, 1024
    r = oracle.moe_route_topk(rng.standard_normal((T, E)).astype(np.float32), k)
    x = oracle.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    xp = api.moe_permute(to_dev_16(x, "bf16"), to_dev(r["perm_to_src"]), k)
    api.synchronize()
    np.testing.assert_array_equal(bits_of(xp), oracle.moe_permute(x, r["perm_to_src"], k))
    y = oracle.f32_to_bf16(rng.standard_normal((T * k, H)).astype(np.float32))
    out = api.moe_unpermute(to_dev_16(y, "bf16"), to_dev(r["src_to_perm"]), to_dev(r["topk_w"]))
    api.synchronize()
    np.testing.assert_array_equal(bits_of(out), oracle.moe_unpermute(y, r["src_to_perm"], r["topk_w"]))


def test_ragged_row_width_uses_scalar_path(oracle):
    rng = np.random.default_rng(12)
    T, k, H = 40, 2, 100                  # H not a multiple of 8
    r = oracle.moe_route_topk(rng.standard_normal((T, 16)).astype(np.float32), k)
    x = oracle.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    xp = api.moe_permute(to_dev_16(x, "bf16"), to_dev(r["perm_to_src"]), k)
    out = api.moe_unpermute(xp, to_dev(r["src_to_perm"]), to_dev(r["topk_w"]))
    api.synchronize()
    np.testing.assert_array_equal(bits_of(xp), oracle.moe_permute(x, r["perm_to_src"], k))
    np.testing.assert_array_equal(bits_of(out), oracle.moe_unpermute(bits_of(xp), r["src_to_perm"], r["topk_w"]))


def test_quantisers_bit_exact(oracle):
    rng = np.random.default_rng(13)
    T, E, k, H = 300, 32, 4, 7168
    x = rng.standard_normal((T, H)).astype(np.float32)
    x[3, 128:256] = 0.0                   # an all-zero block: scale 1
    x[4] *= 1e-30                         # tiny values
    x[5, 7] = 3e38                        # huge value
    xb = oracle.f32_to_bf16(x)
    q, s = api.quant_rows_e4m3(to_dev_16(xb, "bf16"))
    api.synchronize()
    rq, rs = oracle.quant_rows_e4m3(oracle.bf16_to_f32(xb))
    np.testing.assert_array_equal(s.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    np.testing.assert_array_equal(bits_of(q), rq)
    r = oracle.moe_route_topk(rng.standard_normal((T, E)).astype(np.float32), k)
    q2, s2 = api.moe_permute_quant_e4m3(to_dev_16(xb, "bf16"), to_dev(r["perm_to_src"]), k)
    api.synchronize()
    src_row = r["perm_to_src"] // k
    np.testing.assert_array_equal(bits_of(q2), rq[src_row])
    np.testing.assert_array_equal(s2.cpu().numpy().view(np.uint32), rs[src_row].view(np.uint32))
    # quantise once, gather the quantised rows: the same bytes
    q3, s3 = api.moe_permute_q_e4m3(q, s, to_dev(r["perm_to_src"]), k)
    api.synchronize()
    np.testing.assert_array_equal(bits_of(q3), rq[src_row])
    np.testing.assert_array_equal(s3.cpu().numpy().view(np.uint32), rs[src_row].view(np.uint32))


def test_bad_permutation_index_is_reported(oracle):
    x = torch.zeros((8, 128), dtype=torch.bfloat16, device="cuda")
    perm = torch.tensor([0, 1, 99, 3], dtype=torch.int32, device="cuda")   # row 99/1 does not exist
    api.moe_permute(x, perm, 1)
    with pytest.raises(CroqError) as err:
        api.synchronize()
    assert err.value.name == "CROQ_ERR_INDEX"
    api.synchronize()


def grouped_case(oracle, rng, counts, N, K):
    E = len(counts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    R = int(offsets[-1])
    x, xs = oracle.quant_rows_e4m3(rng.standard_normal((R, K)).astype(np.float32))
    w, ws = oracle.quant_blocks_e4m3((rng.standard_normal((E, N, K)) / np.sqrt(K)).astype(np.float32))
    return x, xs, w, ws, offsets


@pytest.mark.parametrize("swiglu", [False, True])
@pytest.mark.parametrize("counts,N,K", [([5, 0, 130, 128, 1, 300], 512, 384), ([257, 3], 256, 1024),
                                         ([0, 0, 64], 768, 128)])
def test_grouped_gemm(oracle, counts, N, K, swiglu):
    rng = np.random.default_rng(sum(counts) + N)
    x, xs, w, ws, offsets = grouped_case(oracle, rng, counts, N, K)
    out = api.moe_grouped_gemm_e4m3(to_dev_e4m3(x), to_dev(xs), to_dev_e4m3(w), to_dev(ws), to_dev(offsets),
                                    swiglu=swiglu,
                                    out=torch.full((x.shape[0], N // 2 if swiglu else N), float("nan"),
                                                   dtype=torch.bfloat16, device="cuda"))
    api.synchronize()
    ref = oracle.bf16_to_f32(oracle.moe_grouped_gemm_e4m3(x, xs, w, ws, offsets, swiglu))
    got = oracle.bf16_to_f32(bits_of(out))
    assert max_rel_err(got, ref, floor=0.05) <= 2e-2


def test_grouped_gemm_equals_dense_kernel_per_expert(oracle):
    """The grouped kernel and the dense block-scaled kernel share the pipeline:
    per expert their outputs must agree bit for bit."""
    rng = np.random.default_rng(21)
    x, xs, w, ws, offsets = grouped_case(oracle, rng, [200, 56, 384], 512, 512)
    dx, dxs, dw, dws = to_dev_e4m3(x), to_dev(xs), to_dev_e4m3(w), to_dev(ws)
    out = api.moe_grouped_gemm_e4m3(dx, dxs, dw, dws, to_dev(offsets))
    for e in range(3):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        ref = api.blockscale_gemm_e4m3(dx[lo:hi].contiguous(), dxs[lo:hi].contiguous(), dw[e], dws[e])
        api.synchronize()
        assert torch.equal(out[lo:hi].view(torch.int16), ref.view(torch.int16))


def test_moe_forward_small_model_against_oracle(oracle):
    """End-to-end layer at a reduced size: T=256, H=512, I=256, E=8, top-2."""
    rng = np.random.default_rng(22)
    T, H, I, E, k = 256, 512, 256, 8, 2
    x = oracle.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    logits = rng.standard_normal((T, E)).astype(np.float32)
    w13, w13s = oracle.quant_blocks_e4m3((rng.standard_normal((E, 2 * I, H)) / np.sqrt(H)).astype(np.float32))
    w2, w2s = oracle.quant_blocks_e4m3((rng.standard_normal((E, H, I)) / np.sqrt(I)).astype(np.float32))
    out = api.moe_forward(to_dev_16(x, "bf16"), to_dev(logits), to_dev_e4m3(w13), to_dev(w13s),
                          to_dev_e4m3(w2), to_dev(w2s), k)
    api.synchronize()
    r = oracle.moe_route_topk(logits, k)
    xq, xs = oracle.quant_rows_e4m3(oracle.bf16_to_f32(x)[r["perm_to_src"] // k])
    g = oracle.moe_grouped_gemm_e4m3(xq, xs, w13, w13s, r["expert_offsets"], True)
    gq, gs = oracle.quant_rows_e4m3(oracle.bf16_to_f32(g))
    y = oracle.moe_grouped_gemm_e4m3(gq, gs, w2, w2s, r["expert_offsets"], False)
    ref = oracle.bf16_to_f32(oracle.moe_unpermute(y, r["src_to_perm"], r["topk_w"]))
    got = oracle.bf16_to_f32(bits_of(out))
    # requantisation of g can flip an e4m3 code where GPU and CPU differ by one
    # bf16 ulp, so the bound is the FP8 one with an absolute floor of 1e-2
    assert max_rel_err(got, ref, floor=1e-2 * max(1.0, np.abs(ref).max())) <= 2e-2
