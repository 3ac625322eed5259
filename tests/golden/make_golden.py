"""Generates the golden fixtures in this folder from the REFERENCE's own code.

Run in a container that has the reference tree (``make -C oracle ref`` first):

    python tests/golden/make_golden.py

Every array written here comes out of ``oracle/_ref/libchoreo_ref.so`` (built
from the reference's runtime headers and its Hilbert test helpers) or
``oracle/_ref/libcuda_codecs.so`` (CUDA's host-side f16/bf16/e4m3 conversions,
the ones the reference's GPU path uses). The oracle itself is NOT used to make
them, so that tests can check the oracle against them on machines that have no
reference tree. Input recipes follow the reference's tests:
tests/gpu/end2end/wgmma_ss.co:324-344 (mod-3 pattern), gemm_sp.co:296-334
(seed 42 sparse case), wgmma_persis.co:156-197 (Hilbert schedule).
"""
from __future__ import annotations

import ctypes
import hashlib
import sys
from ctypes import c_int, c_size_t, c_uint, c_void_p
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
OUT = Path(__file__).resolve().parent


def p(a):
    return a.ctypes.data_as(c_void_p)


def main() -> None:
    ref = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libchoreo_ref.so"))
    cod = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libcuda_codecs.so"))

    # ---- Hilbert schedules ------------------------------------------------
    ref.ref_build_hilbert_schedule.restype = c_int
    ref.ref_build_hilbert_schedule.argtypes = [c_int, c_int, c_void_p, c_void_p]
    hil = {}
    for tm, tn in [(32, 32), (24, 16), (5, 7), (1, 1), (3, 1), (1, 6), (2, 2)]:
        sm = np.zeros(4096, np.int32)
        sn = np.zeros(4096, np.int32)
        n = ref.ref_build_hilbert_schedule(tm, tn, p(sm), p(sn))
        assert n == tm * tn
        hil[f"m_{tm}x{tn}"] = sm[:n].astype(np.int16)
        hil[f"n_{tm}x{tn}"] = sn[:n].astype(np.int16)
    np.savez_compressed(OUT / "hilbert.npz", **hil)

    # ---- scalar codecs ----------------------------------------------------
    rng = np.random.default_rng(20260101)
    parts = [
        rng.standard_normal(1024).astype(np.float32),
        (rng.standard_normal(512) * 300).astype(np.float32),
        (rng.standard_normal(512) * 1e-3).astype(np.float32),
        (rng.standard_normal(512) * 6e-5).astype(np.float32),
        (rng.standard_normal(256) * 6e-8).astype(np.float32),
        (rng.standard_normal(256) * 7e4).astype(np.float32),
        np.array([0.0, -0.0, 448.0, 449.0, 464.0, 465.0, 480.0, 1e9, -1e9, np.inf, -np.inf,
                  np.nan, 65504.0, 65519.9, 65520.0, 2.0 ** -24, 2.0 ** -25, 1.5 * 2.0 ** -25,
                  2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 2.0 ** -10 * 1.0000001,
                  0.1, 500.0, 6e-5, 0.0009765625, 0.0029296875, 0.00390625], np.float32),
    ]
    # every midpoint between neighbouring e4m3 values (ties) and a nudge either side
    e4 = np.arange(256, dtype=np.uint8)
    e4f = np.zeros(256, np.float32)
    cod.cuda_e4m3_to_f32_n.argtypes = [c_void_p, c_void_p, c_size_t]
    cod.cuda_e4m3_to_f32_n(p(e4), p(e4f), 256)
    pos = np.sort(e4f[:127])
    mids = ((pos[:-1].astype(np.float64) + pos[1:].astype(np.float64)) / 2).astype(np.float32)
    parts += [mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(1e9)), -mids]
    x = np.concatenate(parts).astype(np.float32)
    f16 = np.zeros(x.size, np.uint16)
    bf16 = np.zeros(x.size, np.uint16)
    e4m3 = np.zeros(x.size, np.uint8)
    for fn, dst in [(cod.cuda_f32_to_f16_n, f16), (cod.cuda_f32_to_bf16_n, bf16),
                    (cod.cuda_f32_to_e4m3_n, e4m3)]:
        fn.argtypes = [c_void_p, c_void_p, c_size_t]
        fn(p(x), p(dst), x.size)
    h_bits = np.concatenate([np.arange(0, 2048, dtype=np.uint16),
                             rng.integers(0, 65536, 2048).astype(np.uint16),
                             np.array([0x7C00, 0xFC00, 0x7BFF, 0x8000, 0x0001, 0x03FF, 0x0400], np.uint16)])
    h_f32 = np.zeros(h_bits.size, np.float32)
    cod.cuda_f16_to_f32_n.argtypes = [c_void_p, c_void_p, c_size_t]
    cod.cuda_f16_to_f32_n(p(h_bits), p(h_f32), h_bits.size)
    np.savez_compressed(OUT / "codecs.npz", x=x, f16=f16, bf16=bf16, e4m3=e4m3,
                        e4m3_decode=e4f.view(np.uint32), f16_bits=h_bits,
                        f16_decode=h_f32.view(np.uint32))

    # ---- reference CPU MMA loop on a small seeded case --------------------
    ref.ref_mma_exec_row_row_f32.argtypes = [c_void_p] * 4 + [c_int] * 3
    M, N, K = 40, 24, 136
    a = np.zeros(M * K, np.uint16)
    b = np.zeros(N * K, np.uint16)
    af = (rng.random(M * K) * 2 - 1).astype(np.float32)
    bf = (rng.random(N * K) * 2 - 1).astype(np.float32)
    cod.cuda_f32_to_f16_n(p(af), p(a), a.size)
    cod.cuda_f32_to_f16_n(p(bf), p(b), b.size)
    a32 = np.zeros(a.size, np.float32)
    b32 = np.zeros(b.size, np.float32)
    cod.cuda_f16_to_f32_n(p(a), p(a32), a.size)
    cod.cuda_f16_to_f32_n(p(b), p(b32), b.size)
    c = np.zeros(M * N, np.float32)
    d = np.zeros(M * N, np.float32)
    ref.ref_mma_exec_row_row_f32(p(d), p(a32), p(b32), p(c), M, N, K)
    mma = dict(lhs_f16=a.reshape(M, K), rhs_f16=b.reshape(N, K), out_f32=d.reshape(M, N))

    # KAT-1: mod-3 pattern, 384x384x128 — exact in every format; keep digests.
    M1, N1, K1 = 384, 384, 128
    m_i, k_i = np.meshgrid(np.arange(M1), np.arange(K1), indexing="ij")
    n_i, k_j = np.meshgrid(np.arange(N1), np.arange(K1), indexing="ij")
    l1 = (((m_i + 2 * k_i) % 3) * 0.5).astype(np.float32)
    r1 = (((2 * n_i + k_j) % 3) * 0.5).astype(np.float32)
    d1 = np.zeros(M1 * N1, np.float32)
    ref.ref_mma_exec_row_row_f32(p(d1), p(np.ascontiguousarray(l1)), p(np.ascontiguousarray(r1)),
                                 p(np.zeros(M1 * N1, np.float32)), M1, N1, K1)
    mma["kat1_sha256"] = np.frombuffer(hashlib.sha256(d1.tobytes()).digest(), np.uint8)
    mma["kat1_row0"] = d1.reshape(M1, N1)[0].copy()
    mma["kat1_sum"] = np.array([d1.astype(np.float64).sum()])
    np.savez_compressed(OUT / "mma_row_row.npz", **mma)

    # ---- sparse: seed-42 inputs + reference encoder output ----------------
    ref.ref_sparse_kat_inputs.argtypes = [c_uint, c_void_p, c_int, c_int, c_void_p, c_int]
    ref.ref_sparse24_encode_f32.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int]
    Ms, Ks, Ns = 64, 64, 32
    da = np.zeros(Ms * Ks, np.float32)
    rb = np.zeros(Ns * Ks, np.float32)
    ref.ref_sparse_kat_inputs(42, p(da), Ms, Ks, p(rb), Ns)
    pk = np.zeros(Ms * Ks // 2, np.float32)
    meta = np.zeros(Ms * Ks // 8, np.uint8)
    ref.ref_sparse24_encode_f32(p(da), p(pk), p(meta), Ms, Ks)
    # a second, irregular case: groups with 0, 1, 3 and 4 non-zeros exercise the fallback
    irr = (rng.random(16 * 32) * 2 - 1).astype(np.float32)
    irr[rng.random(irr.size) < 0.5] = 0.0
    irr[:8] = 0.0
    irr[8:12] = [0.5, 0.25, -1.0, 2.0]
    pk2 = np.zeros(irr.size // 2, np.float32)
    meta2 = np.zeros(irr.size // 8, np.uint8)
    ref.ref_sparse24_encode_f32(p(irr), p(pk2), p(meta2), 16, 32)
    # metadata re-layouts of the reference (prepack, prepack_v2) on the seed-42 metadata and
    # on random bytes (48 rows x 12 bytes: three 16-row blocks, three K fragments)
    ref.ref_sparse24_prepack_meta.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int]
    rnd_meta = rng.integers(0, 256, 48 * 12, dtype=np.uint8)
    pre = {}
    for tag, mm, rows, km in (("kat", meta, Ms, Ks // 8), ("rnd", rnd_meta, 48, 12)):
        for layout in (1, 2):
            o = np.zeros(rows * km // 4, np.uint32)
            ref.ref_sparse24_prepack_meta(p(mm), p(o), rows, km, layout)
            pre[f"{tag}_prepack_v{layout}"] = o.reshape(rows, km // 4)
    np.savez_compressed(OUT / "sparse.npz", dense_a=da.reshape(Ms, Ks), rhs=rb.reshape(Ns, Ks),
                        packed=pk.reshape(Ms, Ks // 2), meta=meta.reshape(Ms, Ks // 8),
                        irr_dense=irr.reshape(16, 32), irr_packed=pk2.reshape(16, 16),
                        irr_meta=meta2.reshape(16, 4), rnd_meta=rnd_meta.reshape(48, 12), **pre)

    # ---- sampled-verifier stride -----------------------------------------
    ref.ref_pick_coprime_stride.restype = c_size_t
    ref.ref_pick_coprime_stride.argtypes = [c_size_t] * 3
    cases = [(1536, 2048, 256), (512, 2048, 256), (8192, 8192, 256), (384, 384, 512), (70, 130, 64),
             (4096, 7168, 256)]
    strides = np.array([[m, n, s, ref.ref_pick_coprime_stride(m * n, n, s)] for m, n, s in cases],
                       np.int64)
    np.savez_compressed(OUT / "sample_stride.npz", cases=strides)
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
