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
// run concurrently: the partial product of K block kb is written into one of
// two 256-column TMEM buffers while sixteen epilogue warps drain the other into
// register accumulators with packed two-wide fp32 FMAs.
//   warp 0      TMA producer (128x128 A tile + 256x128 B tile per stage)
//   warps 1,3   MMA issuers (even / odd K blocks): 4 x tcgen05.mma kind::f8f6f4
//               128x256x32 per K block, one commit
//   warp 2      TMEM allocation
//   warps 4-19  promotion + store; warp w reads TMEM lanes 32*(w%4).., columns
//               64*((w-4)/4).. and keeps 64 fp32 accumulators per thread
#include "croq_device.cuh"
#include "croq_host.h"

namespace croq {

namespace {

constexpr int kBlockM = 128;
constexpr int kBlockN = 256;
constexpr int kBlockK = 128;  // one scale block; 128 x 1 B = one swizzle row
constexpr int kUmmaK = 32;
constexpr int kStages = 4;
constexpr int kThreads = 640;        // 4 control warps + 16 promotion warps
constexpr int kEpiWarps = 16;
// Register hand-off between warpgroups (setmaxnreg). A CTA can only re-assign
// registers it owns: what the control warpgroup gives up must cover what the
// promotion warpgroups take, or setmaxnreg.inc would wait forever.
constexpr int kLaunchRegs = 96;   // per thread at launch: 65536 / 640, rounded down to 8
constexpr int kCtrlRegs = 32;
constexpr int kEpiRegs = 112;
static_assert((kLaunchRegs - kCtrlRegs) * 128 >= (kEpiRegs - kLaunchRegs) * kEpiWarps * 32,
              "control warps do not release enough registers for the promotion warps");
static_assert(kLaunchRegs * kThreads <= 65536, "launch allocation exceeds the register file");
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
  __shared__ __align__(8) uint64_t bar_full[kStages];      // TMA data of a stage has landed
  __shared__ __align__(8) uint64_t bar_mma_done[kStages];  // the stage's MMAs retired: the
                                                           // smem stage is free AND its TMEM
                                                           // partial is complete
  __shared__ __align__(8) uint64_t bar_part_empty[2];      // a TMEM partial buffer was drained
  __shared__ __align__(8) uint64_t bar_drain[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int num_kb = p.KB;
  const int my_tiles = (p.total_work - static_cast<int>(blockIdx.x) + static_cast<int>(gridDim.x) - 1) /
                       static_cast<int>(gridDim.x);
  const int total_kb = my_tiles * num_kb;   // K blocks this CTA walks, over all its tiles

  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_mma_done[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bar_part_empty[b]), kEpiWarps);  // one arrival per promotion warp
      mbar_init(smem_u32(&bar_drain[b]), 1);
    }
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
    reg_dealloc<kCtrlRegs>();
    // The control loops run warp-uniformly (all 32 lanes wait and compute the
    // descriptors, so those values stay in uniform registers) and only the
    // asynchronous instructions themselves are issued by one elected lane.
    if (warp == 0) {
      // ---------------------------------------------------------- producer --
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
        int m0, n0;
        decode_tile(p, w, m0, n0);
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&bar_mma_done[stage]), phase ^ 1u, abort_ptr);
          if (!ok) break;
          const uint32_t full = smem_u32(&bar_full[stage]);
          const uint32_t a_dst = smem_base + stage * kStageBytes;
          if (elect_one()) {
            mbar_arrive_expect_tx(full, kStageBytes);
            tma_load_2d(a_dst, &map_a, full, kb * kBlockK, m0);
            tma_load_2d(a_dst + kABytes, &map_b, full, kb * kBlockK, n0);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 1000000ull) {
        }
      }
    } else if (warp == 1 || warp == 3) {
      // ------------------------------------------------------- MMA issuers --
      // Two warps alternate: warp 1 takes the even K blocks (TMEM buffer 0),
      // warp 3 the odd ones (buffer 1). The blocks are independent (each starts
      // a fresh partial), so no order between the two is needed. One commit per
      // K block signals both "stage free" and "partial complete".
      constexpr uint32_t idesc = umma_idesc(kFmtE4M3, kFmtE4M3, kBlockM, kBlockN);
      const int buf = (warp == 1) ? 0 : 1;
      const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(buf * kBlockN);
      const uint32_t empty_bar = smem_u32(&bar_part_empty[buf]);
      bool ok = true;
      for (int g = buf; g < total_kb; g += 2) {
        const int stage = g % kStages;
        const uint32_t phase = static_cast<uint32_t>(g / kStages) & 1u;
        const uint32_t buf_phase = static_cast<uint32_t>(g >> 1) & 1u;
        const uint32_t a_src = smem_base + stage * kStageBytes;
        const uint64_t adesc = umma_desc_k_sw128(a_src);
        const uint64_t bdesc = umma_desc_k_sw128(a_src + kABytes);
        // operands usually land long before the partial buffer is free
        ok = mbar_wait(smem_u32(&bar_full[stage]), phase, abort_ptr);
        if (!ok) break;
        ok = mbar_wait(empty_bar, buf_phase ^ 1u, abort_ptr);
        if (!ok) break;
        tc_fence_after_sync();
        if (elect_one()) {
          umma_f8(tmem_d, adesc, bdesc, idesc, 0u);
          umma_f8(tmem_d, adesc + 2u, bdesc + 2u, idesc, 1u);
          umma_f8(tmem_d, adesc + 4u, bdesc + 4u, idesc, 1u);
          umma_f8(tmem_d, adesc + 6u, bdesc + 6u, idesc, 1u);
          umma_commit(smem_u32(&bar_mma_done[stage]));
        }
      }
      if (elect_one()) umma_commit(smem_u32(&bar_drain[buf]));
      __syncwarp();
      mbar_wait(smem_u32(&bar_drain[buf]), 0, abort_ptr);
    }
  } else {
    // ------------------------------------------------- promotion + store --
    // Draining a partial is latency-bound (barrier wake-up, TMEM load round
    // trips), so sixteen warps share it: warp w reads TMEM lanes 32*(w%4)..
    // and the 64 columns of column group (w-4)/4, four warps per scheduler.
    reg_alloc<kEpiRegs>();
    const int quarter = warp & 3;
    const int cgroup = (warp - 4) >> 2;
    const bool vec_ok = ((p.N & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15u) == 0);
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    int stage = 0;
    uint32_t phase = 0;
    int buf = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < p.total_work && ok; w += gridDim.x) {
      int m0, n0;
      decode_tile(p, w, m0, n0);
      const int row = m0 + quarter * 32 + lane;
      const int col_base = n0 + cgroup * 64;
      const float* sa_ptr = p.scale_a + static_cast<size_t>(min(row, p.M - 1)) * p.KB;
      const float* sb_ptr = p.scale_b + static_cast<size_t>(min(col_base >> 7, p.NB - 1)) * p.KB;
      float2 acc[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.0f, 0.0f);
      // Scales are fetched one K block ahead and multiplied only when used.
      float sa_next = __ldg(sa_ptr), sb_next = __ldg(sb_ptr);
      for (int kb = 0; kb < num_kb; ++kb) {
        const float scale = sa_next * sb_next;
        const unsigned long long scale2 = pack_f32x2(scale, scale);
        const int kn = min(kb + 1, num_kb - 1);
        sa_next = __ldg(sa_ptr + kn);
        sb_next = __ldg(sb_ptr + kn);
        ok = mbar_wait(smem_u32(&bar_mma_done[stage]), phase, abort_ptr);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t taddr =
            tmem_base + static_cast<uint32_t>(buf * kBlockN + cgroup * 64) + lane_field;
        uint32_t v[32];
        tmem_ld_32x32(taddr, v);
        tmem_ld_wait_on(v);
#pragma unroll
        for (int i = 0; i < 16; ++i) ffma2(acc[i], v[2 * i], v[2 * i + 1], scale2);
        tmem_ld_32x32(taddr + 32, v);
        tmem_ld_wait_on(v);
        // Both loads have landed in registers: hand the buffer back.
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_part_empty[buf]));
#pragma unroll
        for (int i = 0; i < 16; ++i) ffma2(acc[16 + i], v[2 * i], v[2 * i + 1], scale2);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
        buf ^= 1;
      }
      if (!ok) break;
      if (row < p.M && col_base < p.N) {
        uint16_t* out_row = p.out + static_cast<size_t>(row) * p.N + col_base;
        if (vec_ok && col_base + 64 <= p.N) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 pk;
            pk.x = pack2<kBf16>(acc[q * 4 + 0].x, acc[q * 4 + 0].y);
            pk.y = pack2<kBf16>(acc[q * 4 + 1].x, acc[q * 4 + 1].y);
            pk.z = pack2<kBf16>(acc[q * 4 + 2].x, acc[q * 4 + 2].y);
            pk.w = pack2<kBf16>(acc[q * 4 + 3].x, acc[q * 4 + 3].y);
            *reinterpret_cast<uint4*>(out_row + q * 8) = pk;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (col_base + 2 * i < p.N) out_row[2 * i] = pack1<kBf16>(acc[i].x);
            if (col_base + 2 * i + 1 < p.N) out_row[2 * i + 1] = pack1<kBf16>(acc[i].y);
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
    // The in-kernel register hand-off assumes the launch allocation; refuse to
    // launch if the compiler chose another one.
    cudaFuncAttributes fa;
    CROQ_CUDA_TRY(cudaFuncGetAttributes(&fa, kernel));
    if (fa.numRegs != kLaunchRegs)
      return record_text_error(CROQ_ERR_UNSUPPORTED,
                               "block-scaled kernel was built with an unexpected register count");
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
