// 2:4 sparsity tooling on the GPU: the compressor that turns a dense matrix
// with at most two non-zeros per group of four into (packed values, metadata),
// and the two metadata re-layouts the reference ships for its Hopper kernels.
// All three are byte-for-byte restatements of host loops in the reference's
// runtime (runtime/choreo.h:1536-1571 encode, 1573-1623 prepack, 1631-1661
// prepack_v2) as HBM-bound kernels: every element is read once and written
// once, accesses are 16 / 8 / 4 bytes per lane and contiguous across a warp.
//
// Algorithmic bytes per row of K positions (16-bit values): encode reads 2K and
// writes K + K/8; prepack reads K/8 and writes K/8.

#include "croq_host.h"

namespace croq {
namespace {

constexpr int kToolThreads = 256;

// Non-zero test of the reference: to_f32(v) != 0.0f, i.e. everything except
// +0 and -0 (NaN counts as non-zero). Same bit test for f16 and bf16.
__device__ __forceinline__ bool nonzero16(uint32_t bits16) { return (bits16 & 0x7FFFu) != 0u; }

// One group of four 16-bit values g[0..3] -> two kept values and a nibble
// idx0 | idx1 << 2 with idx0 < idx1. A group that does not hold exactly two
// non-zeros keeps positions 0 and 1, as the reference's encoder does.
__device__ __forceinline__ void encode_group(const uint16_t (&g)[4], uint16_t& v0, uint16_t& v1,
                                             uint32_t& nibble) {
  int idx0 = -1, idx1 = -1, nz = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (nonzero16(g[i])) {
      if (nz == 0) idx0 = i;
      else if (nz == 1) idx1 = i;
      ++nz;
    }
  }
  if (nz != 2) { idx0 = 0; idx1 = 1; }
  // idx0 < idx1 by construction
  v0 = (idx0 == 0) ? g[0] : (idx0 == 1) ? g[1] : g[2];
  v1 = (idx1 == 1) ? g[1] : (idx1 == 2) ? g[2] : g[3];
  nibble = static_cast<uint32_t>(idx0) | (static_cast<uint32_t>(idx1) << 2);
}

// One unit = 8 consecutive K positions of one row = two groups = one metadata
// byte. K % 8 == 0, so units never straddle rows and unit u lives at element
// offset 8u of the dense matrix, 4u of the packed one and byte u of the metadata.
__global__ void __launch_bounds__(kToolThreads)
sparse24_encode_kernel(const uint4* __restrict__ dense, uint2* __restrict__ packed,
                       uint8_t* __restrict__ meta, size_t units) {
  const size_t stride = static_cast<size_t>(gridDim.x) * kToolThreads;
  for (size_t u = static_cast<size_t>(blockIdx.x) * kToolThreads + threadIdx.x; u < units;
       u += stride) {
    const uint4 d = __ldg(dense + u);
    const uint16_t g0[4] = {static_cast<uint16_t>(d.x & 0xFFFFu), static_cast<uint16_t>(d.x >> 16),
                            static_cast<uint16_t>(d.y & 0xFFFFu), static_cast<uint16_t>(d.y >> 16)};
    const uint16_t g1[4] = {static_cast<uint16_t>(d.z & 0xFFFFu), static_cast<uint16_t>(d.z >> 16),
                            static_cast<uint16_t>(d.w & 0xFFFFu), static_cast<uint16_t>(d.w >> 16)};
    uint16_t a0, a1, b0, b1;
    uint32_t n0, n1;
    encode_group(g0, a0, a1, n0);
    encode_group(g1, b0, b1, n1);
    uint2 pk;
    pk.x = static_cast<uint32_t>(a0) | (static_cast<uint32_t>(a1) << 16);
    pk.y = static_cast<uint32_t>(b0) | (static_cast<uint32_t>(b1) << 16);
    packed[u] = pk;
    meta[u] = static_cast<uint8_t>(n0 | (n1 << 4));   // even group -> low nibble
  }
}

// Metadata re-layout. Input u8 [M, KM] (KM = K/8), output u32 [M, KF] (KF =
// KM/4, one word per 32-wide K fragment). For a 16-row block and r in 0..7 the
// reference's `prepack` forms
//   word(block + 2r + 0, kf) = bytes 0,1 of row block+r   | bytes 0,1 of row block+r+8 << 16
//   word(block + 2r + 1, kf) = bytes 2,3 of row block+r   | bytes 2,3 of row block+r+8 << 16
// and `prepack_v2` stores the same words as [M/16, KF, 16] (the 16 words of
// one block and fragment contiguous). One thread produces one word; threads
// run along kf, so the 4-byte source reads and the v1 writes coalesce.
template <int kLayout>
__global__ void __launch_bounds__(kToolThreads)
sparse24_prepack_kernel(const uint8_t* __restrict__ meta_u8, uint32_t* __restrict__ meta_u32,
                        size_t M, size_t KF) {
  const size_t total = M * KF;
  const size_t stride = static_cast<size_t>(gridDim.x) * kToolThreads;
  for (size_t t = static_cast<size_t>(blockIdx.x) * kToolThreads + threadIdx.x; t < total;
       t += stride) {
    const size_t out_row = t / KF;
    const size_t kf = t - out_row * KF;
    const size_t block = out_row & ~static_cast<size_t>(15);
    const size_t rib = out_row & 15;           // row inside the block, = 2r + h
    const size_t r = rib >> 1, h = rib & 1;
    const uint8_t* lo = meta_u8 + (block + r) * (KF * 4) + kf * 4 + 2 * h;
    const uint8_t* hi = meta_u8 + (block + r + 8) * (KF * 4) + kf * 4 + 2 * h;
    const uint32_t lo16 = *reinterpret_cast<const uint16_t*>(lo);
    const uint32_t hi16 = *reinterpret_cast<const uint16_t*>(hi);
    const uint32_t word = lo16 | (hi16 << 16);
    if constexpr (kLayout == 1) {
      meta_u32[t] = word;
    } else {
      meta_u32[((block >> 4) * KF + kf) * 16 + rib] = word;
    }
  }
}

int grid_for(size_t work_items, int sm_count) {
  const size_t blocks = (work_items + kToolThreads - 1) / kToolThreads;
  const size_t cap = static_cast<size_t>(sm_count) * 16;   // grid-stride above that
  return static_cast<int>(blocks < cap ? (blocks ? blocks : 1) : cap);
}

}  // namespace
}  // namespace croq

extern "C" {

int croq_sparse24_encode_f16(const croq_view2* dense, const croq_view2* packed,
                             const croq_view2* meta_u8, croq_stream stream_) {
  using namespace croq;
  clear_error();
  if (!view_ok(dense) || !view_ok(packed) || !view_ok(meta_u8)) return CROQ_ERR_NULL;
  const size_t M = dense->dims[0], K = dense->dims[1];
  if ((K & 7) != 0) return CROQ_ERR_SHAPE;
  if (packed->dims[0] != M || packed->dims[1] != K / 2) return CROQ_ERR_SHAPE;
  if (meta_u8->dims[0] != M || meta_u8->dims[1] != K / 8) return CROQ_ERR_SHAPE;
  if (!aligned16(dense->ptr) || (reinterpret_cast<uintptr_t>(packed->ptr) & 7u) != 0)
    return CROQ_ERR_ALIGN;
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  const size_t units = M * (K / 8);
  if (units == 0) return CROQ_OK;
  sparse24_encode_kernel<<<grid_for(units, st->sm_count), kToolThreads, 0,
                           static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint4*>(dense->ptr), static_cast<uint2*>(packed->ptr),
      static_cast<uint8_t*>(meta_u8->ptr), units);
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

int croq_sparse24_prepack_meta(const croq_view2* meta_u8, const croq_view2* meta_u32, int layout,
                               croq_stream stream_) {
  using namespace croq;
  clear_error();
  if (!view_ok(meta_u8) || !view_ok(meta_u32)) return CROQ_ERR_NULL;
  if (layout != CROQ_SPARSE_META_PREPACK && layout != CROQ_SPARSE_META_PREPACK_V2)
    return CROQ_ERR_UNSUPPORTED;
  const size_t M = meta_u8->dims[0], KM = meta_u8->dims[1];
  // the reference asserts the same three conditions (runtime/choreo.h:1581-1590)
  if ((M & 15) != 0 || (KM & 3) != 0) return CROQ_ERR_SHAPE;
  if (meta_u32->dims[0] != M || meta_u32->dims[1] != KM / 4) return CROQ_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(meta_u8->ptr) & 1u) != 0 ||
      (reinterpret_cast<uintptr_t>(meta_u32->ptr) & 3u) != 0)
    return CROQ_ERR_ALIGN;
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  const size_t KF = KM / 4;
  if (M * KF == 0) return CROQ_OK;
  const int grid = grid_for(M * KF, st->sm_count);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (layout == CROQ_SPARSE_META_PREPACK) {
    sparse24_prepack_kernel<1><<<grid, kToolThreads, 0, stream>>>(
        static_cast<const uint8_t*>(meta_u8->ptr), static_cast<uint32_t*>(meta_u32->ptr), M, KF);
  } else {
    sparse24_prepack_kernel<2><<<grid, kToolThreads, 0, stream>>>(
        static_cast<const uint8_t*>(meta_u8->ptr), static_cast<uint32_t*>(meta_u32->ptr), M, KF);
  }
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

}  // extern "C"
