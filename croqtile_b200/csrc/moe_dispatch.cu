// Expert-parallel token exchange fused into the row kernels, over peer memory.
//
// With experts partitioned over GPUs, the dispatch (token rows -> owning GPU)
// and the combine (expert outputs -> token's GPU) are the two exchange steps of
// an MoE layer. Instead of staging rows for a library all-to-all and regrouping
// them afterwards, the row kernels address the peers' buffers directly through
// NVLink-mapped pointers:
//
//   dispatch  the gather + 1x128 e4m3 quantiser writes every row (and its
//             scales) straight into its final, expert-sorted position in the
//             owner's buffer with 8-byte peer stores;
//   combine   the weighted unpermute reads each of a token's k expert outputs
//             from the owner's buffer with 16-byte peer loads.
//
// Only plain loads and stores cross the link (no TMA, no multicast). Placement:
// the owner of expert e keeps its rows expert-major and, inside one expert,
// ordered by source rank; dest_base[e] is the row at which THIS rank's rows of
// expert e start in the owner's buffer (derived from the all-gathered counts),
// so expanded row r with expert e and local permuted position pos lands at
// dest_base[e] + (pos - expert_offsets[e]). The reference has no counterpart.
#include <cuda_fp8.h>

#include "croq_device.cuh"
#include "croq_host.h"
#include "croq_quant.cuh"

namespace croq {

namespace {

constexpr int kRowThreads = 256;

__global__ void __launch_bounds__(kRowThreads)
moe_dispatch_quant_kernel(const uint16_t* __restrict__ src, const int* __restrict__ perm_to_src,
                          const int* __restrict__ topk_idx, const int* __restrict__ expert_offsets,
                          const int* __restrict__ dest_base,
                          const unsigned long long* __restrict__ peer_q,
                          const unsigned long long* __restrict__ peer_scale, int k, int T, int E,
                          int experts_per_rank, int capacity_rows, int H, int* __restrict__ status) {
  const int pos = blockIdx.x;
  const int r = perm_to_src[pos];
  const int t = r / k;
  if (r < 0 || t >= T) {
    if (threadIdx.x == 0) *status = kDevBadIndex;
    return;
  }
  const int e = topk_idx[r];
  if (e < 0 || e >= E) {
    if (threadIdx.x == 0) *status = kDevBadIndex;
    return;
  }
  const int owner = e / experts_per_rank;
  const int dest_row = dest_base[e] + (pos - expert_offsets[e]);
  if (dest_row < 0 || dest_row >= capacity_rows) {   // owner's buffer too small for this imbalance
    if (threadIdx.x == 0) *status = kDevBadIndex;
    return;
  }
  const uint4* s4 = reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * H);
  uint2* q2 = reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(peer_q[owner]) +
                                       static_cast<size_t>(dest_row) * H);
  float* sc = reinterpret_cast<float*>(peer_scale[owner]) + static_cast<size_t>(dest_row) * (H / 128);
  const int chunks = H / 8;   // multiple of 16: whole 16-lane groups stay together
  for (int c = threadIdx.x; c < chunks; c += kRowThreads) {
    float scale;
    q2[c] = quant_chunk_e4m3(__ldg(s4 + c), scale);
    if ((threadIdx.x & 15) == 0) sc[c >> 4] = scale;
  }
}

// Dispatch of rows that were quantised once per token beforehand: a pure copy
// of H e4m3 bytes and H/128 scales per expanded row into the owner's buffers,
// 16-byte peer stores. Same placement rule as above; a CTA moves kRows rows and
// issues all its loads before the first store.
template <int kRows>
__global__ void __launch_bounds__(kRowThreads)
moe_dispatch_rows_q_kernel(const uint8_t* __restrict__ q_src, const float* __restrict__ s_src,
                           const int* __restrict__ perm_to_src, const int* __restrict__ topk_idx,
                           const int* __restrict__ expert_offsets, const int* __restrict__ dest_base,
                           const unsigned long long* __restrict__ peer_q,
                           const unsigned long long* __restrict__ peer_scale,
                           const unsigned long long* __restrict__ peer_ret, int my_rank, int k,
                           int T, int E, int rows, int experts_per_rank, int capacity_rows, int H,
                           int SB, int* __restrict__ status) {
  const int pos0 = blockIdx.x * kRows;
  const uint8_t* src_q[kRows];
  const float* src_s[kRows];
  uint8_t* dst_q[kRows];
  float* dst_s[kRows];
  bool live[kRows];
#pragma unroll
  for (int j = 0; j < kRows; ++j) {
    const int pos = pos0 + j;
    live[j] = false;
    src_q[j] = q_src; src_s[j] = s_src; dst_q[j] = nullptr; dst_s[j] = nullptr;
    if (pos >= rows) continue;
    const int r = perm_to_src[pos];
    const int t = r / k;
    bool ok = r >= 0 && t < T;
    int e = 0, dest_row = 0;
    if (ok) {
      e = topk_idx[r];
      ok = e >= 0 && e < E;
    }
    if (ok) {
      dest_row = dest_base[e] + (pos - expert_offsets[e]);
      ok = dest_row >= 0 && dest_row < capacity_rows;   // else: owner's buffer too small
    }
    if (!ok) {
      if (threadIdx.x == 0) *status = kDevBadIndex;
      continue;
    }
    const int owner = e / experts_per_rank;
    live[j] = true;
    src_q[j] = q_src + static_cast<size_t>(t) * H;
    src_s[j] = s_src + static_cast<size_t>(t) * SB;
    dst_q[j] = reinterpret_cast<uint8_t*>(peer_q[owner]) + static_cast<size_t>(dest_row) * H;
    dst_s[j] = reinterpret_cast<float*>(peer_scale[owner]) + static_cast<size_t>(dest_row) * SB;
    // return address of the row: (home rank, expanded row index), read by the
    // owner's down-projection when it sends the result row straight back
    if (peer_ret != nullptr && threadIdx.x == 0)
      reinterpret_cast<long long*>(peer_ret[owner])[dest_row] =
          (static_cast<long long>(my_rank) << 32) | static_cast<long long>(r);
  }
  const int chunks = H / 16;
  for (int c = threadIdx.x; c < chunks; c += kRowThreads) {
    uint4 v[kRows];
#pragma unroll
    for (int j = 0; j < kRows; ++j)
      v[j] = live[j] ? __ldg(reinterpret_cast<const uint4*>(src_q[j]) + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < kRows; ++j)
      if (live[j]) reinterpret_cast<uint4*>(dst_q[j])[c] = v[j];
  }
  for (int i = threadIdx.x; i < SB * kRows; i += kRowThreads) {
    const int r = i / SB, c = i - r * SB;
#pragma unroll
    for (int j = 0; j < kRows; ++j)
      if (j == r && live[j]) dst_s[j][c] = __ldg(src_s[j] + c);
  }
}

// Placement of this rank's rows in the owners' buffers from the all-gathered
// per-expert counts (counts[s][e] = rows rank s sends to expert e). One CTA:
//   total[e]      = sum_s counts[s][e]
//   start[e]      = rows of the owner's earlier experts (exclusive prefix of total inside
//                   the owner's group of experts_per_rank experts)
//   dest_base[e]  = start[e] + sum_{s < rank} counts[s][e]
//   offsets[i]    = exclusive prefix of total over THIS rank's experts (length e_loc + 1):
//                   the expert_offsets of the owner-side grouped GEMMs.
constexpr int kPlacementMaxExperts = 1024;

__global__ void __launch_bounds__(256)
moe_ep_placement_kernel(const int* __restrict__ counts, int world, int E, int rank,
                        int experts_per_rank, int* __restrict__ dest_base,
                        int* __restrict__ offsets) {
  __shared__ int total_s[kPlacementMaxExperts];
  __shared__ int before_s[kPlacementMaxExperts];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int total = 0, before = 0;
    for (int s = 0; s < world; ++s) {
      const int c = counts[static_cast<size_t>(s) * E + e];
      total += c;
      if (s < rank) before += c;
    }
    total_s[e] = total;
    before_s[e] = before;
  }
  __syncthreads();
  // one thread per owner walks its experts in order (experts_per_rank is small)
  for (int owner = threadIdx.x; owner < world; owner += blockDim.x) {
    int run = 0;
    for (int i = 0; i < experts_per_rank; ++i) {
      const int e = owner * experts_per_rank + i;
      dest_base[e] = run + before_s[e];
      if (owner == rank) offsets[i] = run;
      run += total_s[e];
    }
    if (owner == rank) offsets[experts_per_rank] = run;
  }
}

// out[t,:] = RN_bf16( sum_j w[t,j] * y_owner(t,j)[row(t,j), :] ), ascending j.
template <int kMaxK>
__global__ void __launch_bounds__(kRowThreads)
moe_combine_remote_kernel(const unsigned long long* __restrict__ peer_y,
                          const int* __restrict__ topk_idx, const int* __restrict__ src_to_perm,
                          const int* __restrict__ expert_offsets, const int* __restrict__ dest_base,
                          const float* __restrict__ topk_w, int k, int E, int experts_per_rank,
                          int capacity_rows, int H, uint16_t* __restrict__ out,
                          int* __restrict__ status) {
  __shared__ const uint16_t* row_s[kMaxK];
  __shared__ float w_s[kMaxK];
  __shared__ int bad;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  if (threadIdx.x < k) {
    const size_t r = static_cast<size_t>(t) * k + threadIdx.x;
    const int e = topk_idx[r];
    const uint16_t* ptr = nullptr;
    if (e < 0 || e >= E) {
      bad = 1;
    } else {
      const int row = dest_base[e] + (src_to_perm[r] - expert_offsets[e]);
      if (row < 0 || row >= capacity_rows) bad = 1;
      else ptr = reinterpret_cast<const uint16_t*>(peer_y[e / experts_per_rank]) + static_cast<size_t>(row) * H;
    }
    row_s[threadIdx.x] = ptr;
    w_s[threadIdx.x] = topk_w[r];
  }
  __syncthreads();
  if (bad) {
    if (threadIdx.x == 0) *status = kDevBadIndex;
    return;
  }
  uint16_t* o = out + static_cast<size_t>(t) * H;
  for (int c = threadIdx.x; c < H / 8; c += kRowThreads) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
    for (int j = 0; j < k; ++j) {
      // peer memory: plain (non-texture) 16-byte load
      const uint4 raw = *(reinterpret_cast<const uint4*>(row_s[j]) + c);
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
      const float wj = w_s[j];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[2 * i] = fmaf(wj, bf16_bits_to_f32(w[i] & 0xFFFFu), acc[2 * i]);
        acc[2 * i + 1] = fmaf(wj, bf16_bits_to_f32(w[i] >> 16), acc[2 * i + 1]);
      }
    }
    uint4 pk;
    pk.x = pack2<true>(acc[0], acc[1]);
    pk.y = pack2<true>(acc[2], acc[3]);
    pk.z = pack2<true>(acc[4], acc[5]);
    pk.w = pack2<true>(acc[6], acc[7]);
    reinterpret_cast<uint4*>(o)[c] = pk;
  }
}

}  // namespace

}  // namespace croq

extern "C" {

int croq_moe_dispatch_quant_e4m3(const croq_view2* src, const croq_view1* perm_to_src,
                                 const croq_view2* topk_idx, const croq_view1* expert_offsets,
                                 const croq_view1* dest_base, const croq_view1* peer_q_ptrs,
                                 const croq_view1* peer_scale_ptrs, int experts_per_rank,
                                 int capacity_rows, croq_stream stream_) {
  using namespace croq;
  clear_error();
  if (!view_ok(src) || !view_ok(perm_to_src) || !view_ok(topk_idx) || !view_ok(expert_offsets) ||
      !view_ok(dest_base) || !view_ok(peer_q_ptrs) || !view_ok(peer_scale_ptrs))
    return CROQ_ERR_NULL;
  const size_t T = src->dims[0], H = src->dims[1], rows = perm_to_src->dims[0];
  const size_t k = topk_idx->dims[1], E = dest_base->dims[0], W = peer_q_ptrs->dims[0];
  if (topk_idx->dims[0] != T || k == 0 || rows != T * k) return CROQ_ERR_SHAPE;
  if (expert_offsets->dims[0] != E + 1 || peer_scale_ptrs->dims[0] != W) return CROQ_ERR_SHAPE;
  if (experts_per_rank <= 0 || capacity_rows <= 0 || W * static_cast<size_t>(experts_per_rank) != E)
    return CROQ_ERR_SHAPE;
  if (H % 128 != 0) return CROQ_ERR_UNSUPPORTED;
  if (rows > 0x7FFFFFFFull || H > 0x7FFFFFFFull) return CROQ_ERR_SHAPE;
  if (!aligned16(src->ptr)) return CROQ_ERR_ALIGN;
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  if (rows == 0) return CROQ_OK;
  moe_dispatch_quant_kernel<<<static_cast<unsigned>(rows), kRowThreads, 0,
                              static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint16_t*>(src->ptr), static_cast<const int*>(perm_to_src->ptr),
      static_cast<const int*>(topk_idx->ptr), static_cast<const int*>(expert_offsets->ptr),
      static_cast<const int*>(dest_base->ptr),
      static_cast<const unsigned long long*>(peer_q_ptrs->ptr),
      static_cast<const unsigned long long*>(peer_scale_ptrs->ptr), static_cast<int>(k),
      static_cast<int>(T), static_cast<int>(E), experts_per_rank, capacity_rows, static_cast<int>(H),
      st->status_dev);
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

int croq_moe_dispatch_rows_q_e4m3(const croq_view2* q_src, const croq_view2* scale_src,
                                  const croq_view1* perm_to_src, const croq_view2* topk_idx,
                                  const croq_view1* expert_offsets, const croq_view1* dest_base,
                                  const croq_view1* peer_q_ptrs, const croq_view1* peer_scale_ptrs,
                                  const croq_view1* peer_ret_ptrs, int my_rank,
                                  int experts_per_rank, int capacity_rows, croq_stream stream_) {
  using namespace croq;
  clear_error();
  if (!view_ok(q_src) || !view_ok(scale_src) || !view_ok(perm_to_src) || !view_ok(topk_idx) ||
      !view_ok(expert_offsets) || !view_ok(dest_base) || !view_ok(peer_q_ptrs) ||
      !view_ok(peer_scale_ptrs))
    return CROQ_ERR_NULL;
  if (peer_ret_ptrs != nullptr &&
      (!view_ok(peer_ret_ptrs) || peer_ret_ptrs->dims[0] != peer_q_ptrs->dims[0] || my_rank < 0 ||
       static_cast<size_t>(my_rank) >= peer_q_ptrs->dims[0]))
    return peer_ret_ptrs->ptr == nullptr ? CROQ_ERR_NULL : CROQ_ERR_SHAPE;
  const size_t T = q_src->dims[0], H = q_src->dims[1], rows = perm_to_src->dims[0];
  const size_t SB = scale_src->dims[1];
  const size_t k = topk_idx->dims[1], E = dest_base->dims[0], W = peer_q_ptrs->dims[0];
  if (topk_idx->dims[0] != T || k == 0 || rows != T * k) return CROQ_ERR_SHAPE;
  if (scale_src->dims[0] != T || SB * 128 != H) return CROQ_ERR_SHAPE;
  if (expert_offsets->dims[0] != E + 1 || peer_scale_ptrs->dims[0] != W) return CROQ_ERR_SHAPE;
  if (experts_per_rank <= 0 || capacity_rows <= 0 || W * static_cast<size_t>(experts_per_rank) != E)
    return CROQ_ERR_SHAPE;
  if (rows > 0x7FFFFFFFull || H > 0x7FFFFFFFull) return CROQ_ERR_SHAPE;
  if (!aligned16(q_src->ptr) || (reinterpret_cast<uintptr_t>(scale_src->ptr) & 3u) != 0)
    return CROQ_ERR_ALIGN;
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  if (rows == 0) return CROQ_OK;
  constexpr int kRows = 4;
  moe_dispatch_rows_q_kernel<kRows><<<static_cast<unsigned>((rows + kRows - 1) / kRows), kRowThreads,
                                      0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const uint8_t*>(q_src->ptr), static_cast<const float*>(scale_src->ptr),
      static_cast<const int*>(perm_to_src->ptr), static_cast<const int*>(topk_idx->ptr),
      static_cast<const int*>(expert_offsets->ptr), static_cast<const int*>(dest_base->ptr),
      static_cast<const unsigned long long*>(peer_q_ptrs->ptr),
      static_cast<const unsigned long long*>(peer_scale_ptrs->ptr),
      peer_ret_ptrs != nullptr ? static_cast<const unsigned long long*>(peer_ret_ptrs->ptr) : nullptr,
      my_rank, static_cast<int>(k), static_cast<int>(T), static_cast<int>(E), static_cast<int>(rows),
      experts_per_rank, capacity_rows, static_cast<int>(H), static_cast<int>(SB), st->status_dev);
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

int croq_moe_ep_placement(const croq_view2* counts, int rank, const croq_view1* dest_base,
                          const croq_view1* owner_offsets, croq_stream stream_) {
  using namespace croq;
  clear_error();
  if (!view_ok(counts) || !view_ok(dest_base) || !view_ok(owner_offsets)) return CROQ_ERR_NULL;
  const size_t W = counts->dims[0], E = counts->dims[1];
  if (W == 0 || E == 0 || E % W != 0) return CROQ_ERR_SHAPE;
  if (E > static_cast<size_t>(kPlacementMaxExperts)) return CROQ_ERR_UNSUPPORTED;
  if (rank < 0 || static_cast<size_t>(rank) >= W) return CROQ_ERR_SHAPE;
  if (dest_base->dims[0] != E || owner_offsets->dims[0] != E / W + 1) return CROQ_ERR_SHAPE;
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  moe_ep_placement_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const int*>(counts->ptr), static_cast<int>(W), static_cast<int>(E), rank,
      static_cast<int>(E / W), static_cast<int*>(dest_base->ptr),
      static_cast<int*>(owner_offsets->ptr));
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

int croq_moe_combine_remote(const croq_view1* peer_y_ptrs, const croq_view2* topk_idx,
                            const croq_view1* src_to_perm, const croq_view1* expert_offsets,
                            const croq_view1* dest_base, const croq_view2* topk_w,
                            const croq_view2* out, int experts_per_rank, int capacity_rows,
                            croq_stream stream_) {
  using namespace croq;
  clear_error();
  if (!view_ok(peer_y_ptrs) || !view_ok(topk_idx) || !view_ok(src_to_perm) ||
      !view_ok(expert_offsets) || !view_ok(dest_base) || !view_ok(topk_w) || !view_ok(out))
    return CROQ_ERR_NULL;
  const size_t T = topk_idx->dims[0], k = topk_idx->dims[1], H = out->dims[1];
  const size_t E = dest_base->dims[0], W = peer_y_ptrs->dims[0];
  if (k == 0 || k > 32 || topk_w->dims[0] != T || topk_w->dims[1] != k) return CROQ_ERR_SHAPE;
  if (src_to_perm->dims[0] != T * k || out->dims[0] != T || expert_offsets->dims[0] != E + 1)
    return CROQ_ERR_SHAPE;
  if (experts_per_rank <= 0 || capacity_rows <= 0 || W * static_cast<size_t>(experts_per_rank) != E)
    return CROQ_ERR_SHAPE;
  if (H % 8 != 0) return CROQ_ERR_UNSUPPORTED;
  if (!aligned16(out->ptr)) return CROQ_ERR_ALIGN;
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  if (T == 0) return CROQ_OK;
  moe_combine_remote_kernel<32><<<static_cast<unsigned>(T), kRowThreads, 0,
                                  static_cast<cudaStream_t>(stream_)>>>(
      static_cast<const unsigned long long*>(peer_y_ptrs->ptr),
      static_cast<const int*>(topk_idx->ptr), static_cast<const int*>(src_to_perm->ptr),
      static_cast<const int*>(expert_offsets->ptr), static_cast<const int*>(dest_base->ptr),
      static_cast<const float*>(topk_w->ptr), static_cast<int>(k), static_cast<int>(E),
      experts_per_rank, capacity_rows, static_cast<int>(H), static_cast<uint16_t*>(out->ptr),
      st->status_dev);
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

}  // extern "C"
