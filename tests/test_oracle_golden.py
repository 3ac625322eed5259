"""The CPU oracle against the golden vectors produced by the reference's own
code (tests/golden/make_golden.py) — the pin that lets the oracle stand in for
the reference on machines without the reference tree."""
import hashlib

import numpy as np
import pytest


def test_hilbert_schedule_matches_reference(oracle, golden):
    g = golden["hilbert"]
    for key in g.files:
        if not key.startswith("m_"):
            continue
        dims = key[2:]
        tm, tn = map(int, dims.split("x"))
        sm, sn = oracle.hilbert_schedule(tm, tn)
        np.testing.assert_array_equal(sm, g[f"m_{dims}"].astype(np.int32))
        np.testing.assert_array_equal(sn, g[f"n_{dims}"].astype(np.int32))


def test_package_hilbert_schedule_matches_reference(golden):
    from croqtile_b200 import hilbert_schedule
    g = golden["hilbert"]
    for dims in ("32x32", "24x16", "5x7", "1x1", "3x1", "1x6"):
        tm, tn = map(int, dims.split("x"))
        sm, sn = hilbert_schedule(tm, tn)
        np.testing.assert_array_equal(sm, g[f"m_{dims}"].astype(np.int32))
        np.testing.assert_array_equal(sn, g[f"n_{dims}"].astype(np.int32))


def test_hilbert_schedule_is_a_permutation(oracle):
    for tm, tn in [(32, 32), (7, 3), (64, 28)]:
        sm, sn = oracle.hilbert_schedule(tm, tn)
        assert len(sm) == tm * tn
        assert len(set(zip(sm.tolist(), sn.tolist()))) == tm * tn
        assert sm.min() == 0 and sm.max() == tm - 1 and sn.max() == tn - 1


def test_codecs_match_cuda_host_conversions(oracle, golden):
    g = golden["codecs"]
    x = g["x"]
    np.testing.assert_array_equal(oracle.f32_to_f16(x), g["f16"])
    np.testing.assert_array_equal(oracle.f32_to_bf16(x), g["bf16"])
    np.testing.assert_array_equal(oracle.f32_to_e4m3(x), g["e4m3"])
    dec = oracle.e4m3_to_f32(np.arange(256, dtype=np.uint8)).view(np.uint32)
    want = g["e4m3_decode"]
    nan = (np.arange(256) & 0x7F) == 0x7F
    np.testing.assert_array_equal(dec[~nan], want[~nan])
    assert np.isnan(dec[nan].view(np.float32)).all()
    got = oracle.f16_to_f32(g["f16_bits"]).view(np.uint32)
    wantf = g["f16_decode"]
    isnan = np.isnan(wantf.view(np.float32))
    np.testing.assert_array_equal(got[~isnan], wantf[~isnan])


def test_f16_codec_agrees_with_numpy_everywhere(oracle):
    bits = np.arange(65536, dtype=np.uint16)
    ours = oracle.f16_to_f32(bits)
    ref = bits.view(np.float16).astype(np.float32)
    ok = ~np.isnan(ref)
    np.testing.assert_array_equal(ours[ok].view(np.uint32), ref[ok].view(np.uint32))
    rng = np.random.default_rng(1)
    x = np.concatenate([rng.standard_normal(50000), rng.standard_normal(50000) * 1e-5,
                        rng.standard_normal(20000) * 4e4]).astype(np.float32)
    np.testing.assert_array_equal(oracle.f32_to_f16(x), x.astype(np.float16).view(np.uint16))


def test_mma_row_row_matches_reference_loop(oracle, golden):
    g = golden["mma_row_row"]
    lhs = oracle.f16_to_f32(g["lhs_f16"])
    rhs = oracle.f16_to_f32(g["rhs_f16"])
    for tile in [(128, 256, 1024), (16, 8, 1024)]:
        # tk >= K keeps the reference's single k-ascending chain per output
        out = oracle.gemm_row_row(lhs, rhs, tile=tile)
        np.testing.assert_array_equal(out.view(np.uint32), g["out_f32"].view(np.uint32))


def kat1_inputs():
    """Deterministic inputs of the reference's dense / FP8 test
    (tests/gpu/end2end/wgmma_ss.co:324-336)."""
    M = N = 384
    K = 128
    m, k = np.meshgrid(np.arange(M), np.arange(K), indexing="ij")
    n, k2 = np.meshgrid(np.arange(N), np.arange(K), indexing="ij")
    lhs = (((m + 2 * k) % 3) * 0.5).astype(np.float32)
    rhs = (((2 * n + k2) % 3) * 0.5).astype(np.float32)
    return lhs, rhs


def test_kat1_mod3_pattern(oracle, golden):
    g = golden["mma_row_row"]
    lhs, rhs = kat1_inputs()
    out = oracle.gemm_row_row(lhs, rhs, tile=(64, 128, 64))
    # every partial sum is a multiple of 0.25 below 2^24: exact in any order
    assert hashlib.sha256(out.tobytes()).digest() == g["kat1_sha256"].tobytes()
    np.testing.assert_array_equal(out[0], g["kat1_row0"])
    np.testing.assert_array_equal(out, (lhs.astype(np.float64) @ rhs.astype(np.float64).T).astype(np.float32))
    # block-scaled path with unit scales gives the same numbers (wgmma_ss.co:337-338)
    q_l, q_r = oracle.f32_to_e4m3(lhs), oracle.f32_to_e4m3(rhs)
    np.testing.assert_array_equal(oracle.e4m3_to_f32(q_l), lhs)
    bs = oracle.blockscale_gemm_e4m3(q_l, np.ones((384, 1), np.float32), q_r, np.ones((3, 1), np.float32))
    np.testing.assert_array_equal(bs, out)


def test_sparse_metadata_prepack_matches_reference(oracle, golden):
    """prepack / prepack_v2 (runtime/choreo.h:1573-1661) on the seed-42 metadata and on
    random bytes; the golden words come from the reference's own functions."""
    g = golden["sparse"]
    for tag, meta in (("kat", g["meta"]), ("rnd", g["rnd_meta"])):
        for layout in (1, 2):
            np.testing.assert_array_equal(oracle.sparse24_prepack_meta(meta, layout),
                                          g[f"{tag}_prepack_v{layout}"])
    with pytest.raises(ValueError):
        oracle.sparse24_prepack_meta(np.zeros((8, 4), np.uint8), 1)     # M % 16


def test_sparse_encoder_matches_reference(oracle, golden):
    g = golden["sparse"]
    for dense, packed, meta in [(g["dense_a"], g["packed"], g["meta"]),
                                (g["irr_dense"], g["irr_packed"], g["irr_meta"])]:
        bits = oracle.f32_to_f16(dense)
        p, m = oracle.sparse24_encode(bits)
        np.testing.assert_array_equal(m, meta)
        np.testing.assert_array_equal(p, oracle.f32_to_f16(packed))
    # structured input: exactly two non-zeros per group, so decode inverts encode
    bits = oracle.f32_to_f16(g["dense_a"])
    p, m = oracle.sparse24_encode(bits)
    np.testing.assert_array_equal(oracle.sparse24_decode(p, m), bits)
    nz = (bits.reshape(64, 16, 4) & 0x7FFF) != 0
    assert (nz.sum(-1) == 2).all()


def test_sample_positions_use_reference_stride(oracle, golden):
    for m, n, s, stride in golden["sample_stride"]["cases"]:
        pos = oracle.sample_positions(int(m), int(n), int(s))
        assert len(pos) >= 1
        if len(pos) > 1:
            assert (np.diff(pos) == stride).all()
        assert pos[0] == 0 and pos[-1] < m * n


def test_blockscale_oracle_against_float64(oracle):
    rng = np.random.default_rng(7)
    M, N, K = 37, 200, 300
    a, sa = oracle.quant_rows_e4m3(rng.standard_normal((M, K)).astype(np.float32))
    b, sb = oracle.quant_blocks_e4m3(rng.standard_normal((N, K)).astype(np.float32))
    out = oracle.blockscale_gemm_e4m3(a, sa, b, sb)
    af = oracle.e4m3_to_f32(a).astype(np.float64)
    bf = oracle.e4m3_to_f32(b).astype(np.float64)
    ref = np.zeros((M, N))
    for kb in range(3):
        sl = slice(kb * 128, min(K, kb * 128 + 128))
        ref += (af[:, sl] @ bf[:, sl].T) * (sa[:, kb:kb + 1].astype(np.float64) *
                                           np.repeat(sb[:, kb], 128)[:N][None, :])
    np.testing.assert_allclose(out, ref, rtol=2e-5, atol=1e-5)
    # quantisation recipe: every block's largest magnitude maps to +-448
    assert np.abs(af).reshape(M, -1).max() == 448.0


def test_quantisers_edge_cases(oracle):
    x = np.zeros((2, 256), np.float32)
    x[1, 130] = -3.0
    q, s = oracle.quant_rows_e4m3(x)
    assert s[0, 0] == 1.0 and s[0, 1] == 1.0 and s[1, 0] == 1.0
    assert s[1, 1] == np.float32(3.0) / np.float32(448.0)
    assert (q[0] == 0).all() and q[1, 130] == 0xFE


def test_moe_routing_definition(oracle):
    rng = np.random.default_rng(3)
    T, E, k = 64, 32, 4
    logits = rng.standard_normal((T, E)).astype(np.float32)
    logits[5, 3] = logits[5, 9] = logits[5].max() + 1.0   # tie: lower index first
    logits[6, :] = 0.25                                   # all equal: experts 0..k-1
    r = oracle.moe_route_topk(logits, k)
    idx = r["topk_idx"]
    assert idx[5, 0] == 3 and idx[5, 1] == 9
    np.testing.assert_array_equal(idx[6], np.arange(k))
    order = np.argsort(-logits.astype(np.float64), axis=1, kind="stable")[:, :k]
    np.testing.assert_array_equal(idx, order.astype(np.int32))
    np.testing.assert_allclose(r["topk_w"].sum(1), 1.0, rtol=1e-6)
    sm = np.exp(logits - logits.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    w = np.take_along_axis(sm, idx, 1)
    np.testing.assert_allclose(r["topk_w"], w / w.sum(1, keepdims=True), rtol=1e-5)
    counts = np.bincount(idx.ravel(), minlength=E)
    np.testing.assert_array_equal(r["expert_counts"], counts)
    np.testing.assert_array_equal(r["expert_offsets"], np.concatenate([[0], np.cumsum(counts)]))
    p2s, s2p = r["perm_to_src"], r["src_to_perm"]
    np.testing.assert_array_equal(p2s[s2p], np.arange(T * k))
    flat = idx.ravel()
    assert (np.diff(flat[p2s]) >= 0).all()                 # grouped by expert
    for e in range(E):                                      # stable inside a group
        seg = p2s[r["expert_offsets"][e]:r["expert_offsets"][e + 1]]
        assert (np.diff(seg) > 0).all()
    w_raw = oracle.moe_route_topk(logits, k, norm_topk=False)["topk_w"]
    np.testing.assert_allclose(w_raw, w, rtol=1e-5)


def test_moe_permute_unpermute_roundtrip(oracle):
    rng = np.random.default_rng(4)
    T, E, k, H = 48, 16, 2, 64
    r = oracle.moe_route_topk(rng.standard_normal((T, E)).astype(np.float32), k)
    x = oracle.f32_to_bf16(rng.standard_normal((T, H)).astype(np.float32))
    xp = oracle.moe_permute(x, r["perm_to_src"], k)
    np.testing.assert_array_equal(xp[r["src_to_perm"]].reshape(T, k, H)[:, 0], x)
    # with weights summing to one and identical rows the combine returns the row
    out = oracle.moe_unpermute(xp, r["src_to_perm"], np.full((T, k), 0.5, np.float32))
    np.testing.assert_array_equal(out, x)


def test_grouped_gemm_equals_per_expert_blockscale(oracle):
    rng = np.random.default_rng(5)
    E, N, K = 3, 256, 256
    offsets = np.array([0, 5, 5, 12], np.int32)            # one empty expert
    x, xs = oracle.quant_rows_e4m3(rng.standard_normal((12, K)).astype(np.float32))
    w, ws = oracle.quant_blocks_e4m3(rng.standard_normal((E, N, K)).astype(np.float32))
    out = oracle.moe_grouped_gemm_e4m3(x, xs, w, ws, offsets, swiglu=False)
    for e in range(E):
        lo, hi = offsets[e], offsets[e + 1]
        if lo == hi:
            continue
        ref = oracle.blockscale_gemm_e4m3(x[lo:hi], xs[lo:hi], w[e], ws[e])
        np.testing.assert_array_equal(out[lo:hi], oracle.f32_to_bf16(ref))
    g = oracle.moe_grouped_gemm_e4m3(x, xs, w, ws, offsets, swiglu=True)
    h = oracle.bf16_to_f32(out).astype(np.float64)          # bf16-rounded h: loose check only
    want = h[:, :128] / (1 + np.exp(-h[:, :128])) * h[:, 128:]
    np.testing.assert_allclose(oracle.bf16_to_f32(g), want, rtol=3e-2, atol=3e-2)
