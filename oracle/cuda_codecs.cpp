// CUDA's own host-side scalar conversions behind a C ABI, to pin the oracle's
// codecs. The reference's GPU path converts through exactly these types
// (runtime/choreo_types.h:207-213 __half, 356-362 __nv_bfloat16, 385
// __nv_fp8_e4m3). Host code only (compiled with g++ against the CUDA headers): builds and runs without a GPU. Test
// infrastructure; built by oracle/Makefile (target `ref`) into oracle/_ref/.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <string.h>

extern "C" {

__attribute__((visibility("default"))) void cuda_f32_to_f16_n(const float* s, uint16_t* d, size_t n) {
  for (size_t i = 0; i < n; ++i) { __half h = __float2half_rn(s[i]); memcpy(&d[i], &h, 2); }
}
__attribute__((visibility("default"))) void cuda_f32_to_bf16_n(const float* s, uint16_t* d, size_t n) {
  for (size_t i = 0; i < n; ++i) { __nv_bfloat16 h = __float2bfloat16_rn(s[i]); memcpy(&d[i], &h, 2); }
}
__attribute__((visibility("default"))) void cuda_f32_to_e4m3_n(const float* s, uint8_t* d, size_t n) {
  for (size_t i = 0; i < n; ++i) { __nv_fp8_e4m3 h(s[i]); memcpy(&d[i], &h, 1); }
}
__attribute__((visibility("default"))) void cuda_f16_to_f32_n(const uint16_t* s, float* d, size_t n) {
  for (size_t i = 0; i < n; ++i) { __half h; memcpy(&h, &s[i], 2); d[i] = __half2float(h); }
}
__attribute__((visibility("default"))) void cuda_e4m3_to_f32_n(const uint8_t* s, float* d, size_t n) {
  for (size_t i = 0; i < n; ++i) { __nv_fp8_e4m3 h; memcpy(&h, &s[i], 1); d[i] = float(h); }
}

}  // extern "C"
