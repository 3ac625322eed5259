// Thin extern "C" shim over the reference's OWN host code, compiled from the
// sources where they lie in the reference tree (no source is copied into this
// repository). It exists to pin oracle/croq_oracle.c: tests compare the
// oracle's output with these functions, and tests/golden/make_golden.py stores
// their outputs as fixtures. Test infrastructure only; the shipped library
// never loads it.
//
// Build (oracle/Makefile, target `ref`):
//   g++ -O2 -std=c++17 -D__CHOREO_TARGET_CC__ -I<reference>/runtime \
//       -DCROQ_REF_HILBERT_INC='"<extract>"' -shared -fPIC ref_shim.cpp
// where <extract> is lines 156-197 of tests/gpu/end2end/wgmma_persis.co
// (hilbert_rotate, hilbert_index_to_xy, build_hilbert_schedule), cut out at
// build time into a temporary file that the recipe deletes again.
#include <cstdint>
#include <algorithm>
#include <cmath>
#include <cstring>
#include <random>

#include "choreo.h"
#include "choreo_cc.h"

#ifdef CROQ_REF_HILBERT_INC
#include CROQ_REF_HILBERT_INC
#endif

extern "C" {

// choreo::cc::mma_exec_row_row (runtime/choreo_cc.h:37-47) on fp32 operands.
__attribute__((visibility("default"))) void ref_mma_exec_row_row_f32(
    float* D, const float* A, const float* B, const float* C, int M, int N, int K) {
  choreo::cc::mma_exec_row_row<float, float, float, float>(D, A, B, C, M, N, K);
}

// Sparse2to4HostPolicyWGMMA<float,64>::encode (runtime/choreo.h:1539-1571).
__attribute__((visibility("default"))) void ref_sparse24_encode_f32(
    const float* dense, float* packed, uint8_t* meta, int M, int K) {
  auto d = choreo::make_spandata<float>((size_t)M, (size_t)K);
  auto p = choreo::make_spandata<float>((size_t)M, (size_t)K / 2);
  auto m = choreo::make_spandata<choreo::u8>((size_t)M, (size_t)K / 8);
  std::memcpy(d.data(), dense, sizeof(float) * (size_t)M * K);
  std::memset(m.data(), 0, (size_t)M * (K / 8));
  choreo::utils::Sparse2to4HostPolicyWGMMA<float, 64>::encode(d, p, m);
  std::memcpy(packed, p.data(), sizeof(float) * (size_t)M * (K / 2));
  std::memcpy(meta, m.data(), (size_t)M * (K / 8));
}

// Sparse2to4HostPolicyWGMMA<float,64>::prepack (layout 1, runtime/choreo.h:1573-1623)
// and ::prepack_v2 (layout 2, 1631-1661) on u8 metadata [M, KM].
__attribute__((visibility("default"))) void ref_sparse24_prepack_meta(
    const uint8_t* meta_u8, uint32_t* meta_u32, int M, int KM, int layout) {
  auto in = choreo::make_spandata<choreo::u8>((size_t)M, (size_t)KM);
  auto out = choreo::make_spandata<choreo::u32>((size_t)M, (size_t)KM / 4);
  std::memcpy(in.data(), meta_u8, (size_t)M * KM);
  if (layout == 1) choreo::utils::Sparse2to4HostPolicyWGMMA<float, 64>::prepack(in, out);
  else choreo::utils::Sparse2to4HostPolicyWGMMA<float, 64>::prepack_v2(in, out);
  std::memcpy(meta_u32, out.data(), sizeof(uint32_t) * (size_t)M * (KM / 4));
}

// Sparse2to4HostPolicyWGMMA<float,64>::init_structured_sparse_A with
// std::mt19937(seed) (runtime/choreo.h:1508-1537; the sparse tests seed 42,
// tests/gpu/end2end/gemm_sp.co:296-334), followed by the test's B recipe
// (gemm_sp.co:12-21: uniform(-1,1), |v| < 0.1 snapped to +-0.25) drawn from
// the same generator, rhs[col][k] filled k-outer as f16_init_b does.
__attribute__((visibility("default"))) void ref_sparse_kat_inputs(
    unsigned seed, float* dense_a, int M, int K, float* rhs, int N) {
  std::mt19937 gen(seed);
  auto d = choreo::make_spandata<float>((size_t)M, (size_t)K);
  choreo::utils::Sparse2to4HostPolicyWGMMA<float, 64>::init_structured_sparse_A(d, gen);
  std::memcpy(dense_a, d.data(), sizeof(float) * (size_t)M * K);
  std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
  for (int kk = 0; kk < K; ++kk)
    for (int col = 0; col < N; ++col) {
      float value = dist(gen);
      if (std::fabs(value) < 0.1f) value = (value < 0.0f ? -0.25f : 0.25f);
      rhs[(size_t)col * K + kk] = value;
    }
}

// Block-scaled FP8 GEMM in the structure the reference's CPU target gives
// `blockscale_gemm_e4m3_ws_persis` (tests/gpu/end2end/wgmma_persis.co:94-154):
// sequential loops over 64x128 output tiles (cc_codegen.cpp:1046-1066), per
// 128-wide K block the operands are staged (strided copy), the partial product
// comes from the reference's own choreo::cc::mma_exec_row_row on a zeroed
// scratch tile, and `mma.scale` adds partial * (sa[row] * sb) into the fp32
// accumulators (operation order of runtime/choreo_cute.h:3812-3813,3851-3860;
// the CPU target's own A-only scaling, cc_codegen.cpp:1267-1283, would drop
// scale_rhs). Operands arrive as e4m3 bytes with a 256-entry decode table
// (the CC target has no fp8 type: cc_codegen.cpp:36,55-61). Computes the tiles
// [tile_m_begin, tile_m_end) x [tile_n_begin, tile_n_end) so that callers can
// spread tiles over host threads or time a bounded sample.
__attribute__((visibility("default"))) void ref_blockscale_gemm_e4m3(
    const uint8_t* lhs, const float* scale_lhs, const uint8_t* rhs, const float* scale_rhs,
    float* out, const float* decode_lut, int M, int N, int K, int tile_m_begin, int tile_m_end,
    int tile_n_begin, int tile_n_end) {
  constexpr int TM = 64, TN = 128, TK = 128;
  const int KB = (K + TK - 1) / TK;
  const int tiles_n = (N + TN - 1) / TN;
  alignas(64) static thread_local float a_s[TM * TK];
  alignas(64) static thread_local float b_s[TN * TK];
  alignas(64) static thread_local float part[TM * TN];
  alignas(64) static thread_local float zero[TM * TN];
  alignas(64) static thread_local float acc[TM * TN];
  std::memset(zero, 0, sizeof(zero));
  for (int bm = tile_m_begin; bm < tile_m_end; ++bm)
    for (int bn = tile_n_begin; bn < tile_n_end && bn < tiles_n; ++bn) {
      const int m0 = bm * TM, n0 = bn * TN;
      const int mm = std::min(TM, M - m0), nn = std::min(TN, N - n0);
      if (mm <= 0 || nn <= 0) continue;
      std::memset(acc, 0, sizeof(acc));
      for (int kb = 0; kb < KB; ++kb) {
        const int k0 = kb * TK, kk = std::min(TK, K - k0);
        for (int i = 0; i < mm; ++i)
          for (int k = 0; k < kk; ++k) a_s[i * kk + k] = decode_lut[lhs[(size_t)(m0 + i) * K + k0 + k]];
        for (int j = 0; j < nn; ++j)
          for (int k = 0; k < kk; ++k) b_s[j * kk + k] = decode_lut[rhs[(size_t)(n0 + j) * K + k0 + k]];
        choreo::cc::mma_exec_row_row<float, float, float, float>(part, a_s, b_s, zero, mm, nn, kk);
        const float sb = scale_rhs[(size_t)(n0 / 128) * KB + kb];
        for (int i = 0; i < mm; ++i) {
          const float s = scale_lhs[(size_t)(m0 + i) * KB + kb] * sb;
          for (int j = 0; j < nn; ++j) acc[i * nn + j] = std::fmaf(part[i * nn + j], s, acc[i * nn + j]);
        }
      }
      for (int i = 0; i < mm; ++i)
        std::memcpy(out + (size_t)(m0 + i) * N + n0, acc + i * nn, sizeof(float) * nn);
    }
}

// choreo::pick_coprime_stride (runtime/choreo.h:498-512).
__attribute__((visibility("default"))) size_t ref_pick_coprime_stride(size_t total, size_t n,
                                                                      size_t num_samples) {
  return choreo::pick_coprime_stride(total, n, num_samples);
}

#ifdef CROQ_REF_HILBERT_INC
// build_hilbert_schedule (tests/gpu/end2end/wgmma_persis.co:178-197).
__attribute__((visibility("default"))) int ref_build_hilbert_schedule(int tiles_m, int tiles_n,
                                                                      int* schedule_m,
                                                                      int* schedule_n) {
  return build_hilbert_schedule(tiles_m, tiles_n, schedule_m, schedule_n);
}
#endif

}  // extern "C"
