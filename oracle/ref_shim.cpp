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
