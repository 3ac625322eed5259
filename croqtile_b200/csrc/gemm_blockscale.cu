// FP8 e4m3 GEMM with fp32 block scales for sm_100a.
//
//   acc = 0; for each 128-wide K block kb:
//     P   = sum_{k in kb} lhs[m,k] * rhs[n,k]                  (tensor core, fp32)
//     acc = fmaf(P, scale_lhs[m,kb] * scale_rhs[n/128,kb], acc)
//   output[m,n] = RN(acc)
//
// Replaces the kernel the reference emits for `blockscale_gemm_e4m3_ws_persis`
// (tests/gpu/end2end/wgmma_persis.co:94-154); the per-block promotion follows
// the fp32 branch of `scale_accumulator` (runtime/choreo_cute.h:3812-3813,
// 3851-3860: sa *= scale_b, then d = fmaf(partial, sa, d)).
//
// In the reference the consumer warpgroup alternates WGMMA and the CUDA-core
// promotion, so the tensor pipe idles during every promotion. Here the two
// run concurrently: the MMA warp writes the partial product of K block kb
// into one of two 256-column TMEM buffers while eight epilogue warps drain
// the other buffer into register accumulators.
//   warp 0      TMA producer (128x128 A tile + 256x128 B tile per stage)
//   warp 1      MMA issuer: 4 x tcgen05.mma kind::f8f6f4 128x256x32 per K block
//   warp 2      TMEM allocation
//   warps 4-11  promotion + store; warp w reads TMEM lanes 32*(w%4).., columns
//               128*((w-4)/4).. and keeps 128 fp32 accumulators per thread
#include "croq_device.cuh"
#include "croq_host.h"

namespace croq {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 128;  // one scale block; 128 x 1 B = one swizzle row
constexpr int kUmmaK = 32;
constexpr int kStages = 4;
constexpr int kThreads = 384;
constexpr int kTmemCols = 512;
constexpr uint32_t kABytes = kBlockM * kBlockK;
constexpr uint32_t kBBytes = kBlockN * kBlockK;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + 1024;
constexpr int kGroupM = 16;  // M tiles per rasterisation group

struct BlockScaleParams {
  uint16_t* out;
  const float* scale_a;  // [M, KB]
  const float* scale_b;  // [NB, KB]
  int M, N, K;
  int KB, NB;            // number of 128-wide K blocks / N blocks
  int tiles_m, tiles_n;
  int total_work;
  int* status;
};

// Tile order: groups of kGroupM tile rows, M fastest inside a group, so the
// CTAs that run together share a small set of A row panels and B column
// panels in L2.
__device__ __forceinline__ void decode_tile(const BlockScaleParams& p, int w, int& m0, int& n0) {
  const int per_group = kGroupM * p.tiles_n;
  const int g = w / per_group;
  const int first_m = g * kGroupM;
  const int rows = min(kGroupM, p.tiles_m - first_m);
  const int r = w - g * per_group;
  const int tn = r / rows;
  const int tm = first_m + (r - tn * rows);
  m0 = tm * kBlockM;
  n0 = tn * kBlockN;
}

template <bool kBf16>
__global__ void __launch_bounds__(kThreads, 1)
gemm_blockscale_kernel(const __grid_constant__ CUtensorMap map_a,
                       const __grid_constant__ CUtensorMap map_b, const BlockScaleParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kStages];
  __shared__ __align__(8) uint64_t bar_empty[kStages];
  __shared__ __align__(8) uint64_t bar_part_full[2];
  __shared__ __align__(8) uint64_t bar_part_empty[2];
  __shared__ __align__(8) uint64_t bar_drain;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_kb = p.KB;

  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_part_full[b]), 1);
      mbar_init(smem_u32(&bar_part_empty[b]), 8);  // one arrival per promotion warp
    }
    mbar_init(smem_u32(&bar_drain), 1);
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(&tmem_base_slot), kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abort_ptr = &abort_word;
  ClockProbe probe;
  if (blockIdx.x == 0 && threadIdx.x == 0) probe.begin();

  if (warp < 4) {
    reg_dealloc<56>();
    if (warp == 0) {
      // ---------------------------------------------------------- producer --
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
        int m0, n0;
        decode_tile(p, w, m0, n0);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, abort_ptr);
          if (!ok) break;
          if (lane == 0) {
            const uint32_t full = smem_u32(&bar_full[stage]);
            const uint32_t a_dst = smem_base + stage * kStageBytes;
            mbar_arrive_expect_tx(full, kStageBytes);
            tma_load_2d(a_dst, &map_a, full, kb * kBlockK, m0);
            tma_load_2d(a_dst + kABytes, &map_b, full, kb * kBlockK, n0);
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) {
        }
      }
    } else if (warp == 1) {
      // -------------------------------------------------------- MMA issuer --
      constexpr uint32_t idesc = umma_idesc(kFmtE4M3, kFmtE4M3, kBlockM, kBlockN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&bar_part_empty[buf]), buf_phase ^ 1u, abort_ptr);
          if (!ok) break;
          ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_ptr);
          if (!ok) break;
          tc_fence_after_sync();
          if (lane == 0) {
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kBlockN);
            const uint32_t a_src = smem_base + stage * kStageBytes;
            const uint64_t adesc = umma_desc_k_sw128(a_src);
            const uint64_t bdesc = umma_desc_k_sw128(a_src + kABytes);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              umma_f8(tmem_d, adesc + 2u * k, bdesc + 2u * k, idesc, k != 0 ? 1u : 0u);
            }
            umma_commit(smem_u32(&bar_empty[stage]));
            umma_commit(smem_u32(&bar_part_full[buf]));
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
          buf ^= 1;
          if (buf == 0) buf_phase ^= 1u;
        }
      }
      if (lane == 0) umma_commit(smem_u32(&bar_drain));
      __syncwarp();
      mbar_wait(smem_u32(&bar_drain), 0, abort_ptr);
    }
  } else {
    // ------------------------------------------------- promotion + store --
    reg_alloc<224>();
    const int quarter = warp & 3;
    const int half = (warp - 4) >> 2;
    const bool vec_ok = ((p.N & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0);
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    int buf = 0;
    uint32_t buf_phase = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
      int m0, n0;
      decode_tile(p, w, m0, n0);
      const int row = m0 + quarter * 32 + lane;
      const int col_base = n0 + half * 128;
      const float* sa_ptr = p.scale_a + static_cast<size_t>(min(row, p.M - 1)) * p.KB;
      const float* sb_ptr = p.scale_b + static_cast<size_t>(min(col_base >> 7, p.NB - 1)) * p.KB;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
      float scale_next = __ldg(sa_ptr) * __ldg(sb_ptr);
      for (int kb = 0; kb < num_kb; ++kb) {
        const float scale = scale_next;
        if (kb + 1 < num_kb) scale_next = __ldg(sa_ptr + kb + 1) * __ldg(sb_ptr + kb + 1);
        ok = mbar_wait(smem_u32(&bar_part_full[buf]), buf_phase, abort_ptr);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t taddr =
            tmem_base + static_cast<uint32_t>(buf * kBlockN + half * 128) + lane_field;
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(taddr, v0);
        tmem_ld_32x32(taddr + 32, v1);
        tmem_ld_wait_on(v0);
        tmem_ld_wait_on(v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(__uint_as_float(v0[i]), scale, acc[i]);
        tmem_ld_32x32(taddr + 64, v0);  // in flight while the next chunk is promoted
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(__uint_as_float(v1[i]), scale, acc[32 + i]);
        tmem_ld_32x32(taddr + 96, v1);
        tmem_ld_wait_on(v0);
        tmem_ld_wait_on(v1);
        // All four loads have landed in registers: hand the buffer back.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_part_empty[buf]));
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(__uint_as_float(v0[i]), scale, acc[64 + i]);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(__uint_as_float(v1[i]), scale, acc[96 + i]);
        buf ^= 1;
        if (buf == 0) buf_phase ^= 1u;
      }
      if (!ok) break;
      if (row < p.M && col_base < p.N) {
        uint16_t* out_row = p.out + static_cast<size_t>(row) * p.N + col_base;
        if (vec_ok && col_base + 128 <= p.N) {
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            uint4 pk;
            pk.x = pack2<kBf16>(acc[q * 8 + 0], acc[q * 8 + 1]);
            pk.y = pack2<kBf16>(acc[q * 8 + 2], acc[q * 8 + 3]);
            pk.z = pack2<kBf16>(acc[q * 8 + 4], acc[q * 8 + 5]);
            pk.w = pack2<kBf16>(acc[q * 8 + 6], acc[q * 8 + 7]);
            *reinterpret_cast<uint4*>(out_row + q * 8) = pk;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 128; ++i) {
            if (col_base + i < p.N) out_row[i] = pack1<kBf16>(acc[i]);
          }
        }
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && abort_word != 0) *p.status = abort_word;
  if (blockIdx.x == 0 && threadIdx.x == 0) probe.end(p.status);
}

template <bool kBf16>
int launch_blockscale(const croq_view2* lhs, const croq_view2* scale_lhs, const croq_view2* rhs,
                      const croq_view2* scale_rhs, const croq_view2* output,
                      cudaStream_t stream) {
  int rc = CROQ_OK;
  DeviceState* st = device_state(&rc);
  if (st == nullptr) return rc;
  const int M = static_cast<int>(lhs->dims[0]);
  const int K = static_cast<int>(lhs->dims[1]);
  const int N = static_cast<int>(rhs->dims[0]);
  if (K == 0) {
    CROQ_CUDA_TRY(cudaMemsetAsync(output->ptr, 0, static_cast<size_t>(M) * N * 2, stream));
    return CROQ_OK;
  }
  BlockScaleParams p;
  p.out = static_cast<uint16_t*>(output->ptr);
  p.scale_a = static_cast<const float*>(scale_lhs->ptr);
  p.scale_b = static_cast<const float*>(scale_rhs->ptr);
  p.M = M; p.N = N; p.K = K;
  p.KB = (K + kBlockK - 1) / kBlockK;
  p.NB = (N + 127) / 128;
  p.tiles_m = (M + kBlockM - 1) / kBlockM;
  p.tiles_n = (N + kBlockN - 1) / kBlockN;
  const long long total = 1ll * p.tiles_m * p.tiles_n;
  if (total > 0x7FFFFFFFll) return CROQ_ERR_SHAPE;
  p.total_work = static_cast<int>(total);
  p.status = st->status_dev;

  CUtensorMap map_a, map_b;
  rc = encode_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, lhs->ptr, M, K, kBlockM,
                            kBlockK);
  if (rc != CROQ_OK) return rc;
  rc = encode_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rhs->ptr, N, K, kBlockN,
                            kBlockK);
  if (rc != CROQ_OK) return rc;

  auto kernel = gemm_blockscale_kernel<kBf16>;
  static bool attr_set = false;
  if (!attr_set) {
    CROQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kSmemBytes)));
    attr_set = true;
  }
  const int grid = p.total_work < st->sm_count ? p.total_work : st->sm_count;
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  CROQ_CUDA_TRY(cudaGetLastError());
  return CROQ_OK;
}

}  // namespace

}  // namespace croq

extern "C" int croq_blockscale_gemm_e4m3(const croq_view2* lhs, const croq_view2* scale_lhs,
                                         const croq_view2* rhs, const croq_view2* scale_rhs,
                                         const croq_view2* output, int out_dtype,
                                         croq_stream stream) {
  using namespace croq;
  clear_error();
  if (!view_ok(lhs) || !view_ok(scale_lhs) || !view_ok(rhs) || !view_ok(scale_rhs) ||
      !view_ok(output))
    return CROQ_ERR_NULL;
  const size_t M = lhs->dims[0], K = lhs->dims[1], N = rhs->dims[0];
  if (rhs->dims[1] != K || output->dims[0] != M || output->dims[1] != N) return CROQ_ERR_SHAPE;
  if (M == 0 || N == 0) return CROQ_ERR_SHAPE;
  if (M > 0x7FFFFFFFull || N > 0x7FFFFFFFull || K > 0x7FFFFFFFull) return CROQ_ERR_SHAPE;
  const size_t KB = (K + 127) / 128, NB = (N + 127) / 128;
  if (K != 0) {
    if (scale_lhs->dims[0] != M || scale_lhs->dims[1] != KB) return CROQ_ERR_SHAPE;
    if (scale_rhs->dims[0] != NB || scale_rhs->dims[1] != KB) return CROQ_ERR_SHAPE;
  }
  if (out_dtype != CROQ_DTYPE_F16 && out_dtype != CROQ_DTYPE_BF16) return CROQ_ERR_UNSUPPORTED;
  if (!aligned16(lhs->ptr) || !aligned16(rhs->ptr)) return CROQ_ERR_ALIGN;
  if (K % 16 != 0) return CROQ_ERR_ALIGN;  // TMA row pitch
  if ((reinterpret_cast<uintptr_t>(output->ptr) & 1u) != 0) return CROQ_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(scale_lhs->ptr) & 3u) != 0 ||
      (reinterpret_cast<uintptr_t>(scale_rhs->ptr) & 3u) != 0)
    return CROQ_ERR_ALIGN;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  return out_dtype == CROQ_DTYPE_BF16
             ? launch_blockscale<true>(lhs, scale_lhs, rhs, scale_rhs, output, s)
             : launch_blockscale<false>(lhs, scale_lhs, rhs, scale_rhs, output, s);
}
