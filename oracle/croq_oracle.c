/* CPU oracle for the libcroq_b200 hot path — TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic the reference defines for the GEMM
 * family, used by tests/, __graft_entry__.smoke() and bench.py's CPU-baseline
 * legs to check and to time against. Nothing in the shipped library links,
 * loads or calls this file; the product path has no CPU fallback.
 *
 * Parity status: the dense, block-scaled and sparse GEMM parts, the 2:4
 * encoder and the Hilbert schedule are pinned against code compiled from the
 * reference's own sources (oracle/ref_shim.cpp -> oracle/_ref) and against
 * CUDA's host-side f16/bf16/e4m3 conversions; the committed fixtures under
 * tests/golden/ carry those outputs. The MoE functions (routing, permutation,
 * quantiser, grouped GEMM, combine) have NO reference counterpart — the
 * reference contains no MoE code — so for them: parity unpinned; they define
 * the behaviour instead of restating it.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ codecs --
 * IEEE round-to-nearest-even conversions, the semantics of the CUDA native
 * types the reference's GPU path uses (runtime/choreo_types.h:207-213 f16,
 * 356-362 bf16, 385 e4m3 = __nv_fp8_e4m3 with saturation to +-448). */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

ORACLE_API uint16_t oracle_f32_to_bf16(float f) {
  uint32_t u = f32_bits(f);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu; /* NaN, as __float2bfloat16_rn */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

ORACLE_API float oracle_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

ORACLE_API uint16_t oracle_f32_to_f16(float f) {
  uint32_t u = f32_bits(f);
  uint32_t sign = (u >> 16) & 0x8000u;
  uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return 0x7FFFu;                 /* NaN, as __float2half_rn */
  if (a >= 0x47800000u) {                              /* >= 65536 or inf */
    return (uint16_t)(sign | 0x7C00u);
  }
  if (a >= 0x38800000u) {                              /* normal half range */
    uint32_t r = a - 0x38000000u;                      /* rebias exponent */
    r += 0xFFFu + ((r >> 13) & 1u);
    return (uint16_t)(sign | (r >> 13));               /* may carry to inf: correct */
  }
  if (a < 0x33000000u) return (uint16_t)sign;          /* < 2^-25: rounds to zero */
  {
    /* subnormal half: value = m * 2^-24, round to nearest even */
    int e = (int)(a >> 23);                            /* biased f32 exponent, 102..112 */
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;          /* 24-bit significand */
    int shift = 126 - e;                               /* 14..24 */
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q += 1u;
    return (uint16_t)(sign | q);
  }
}

ORACLE_API float oracle_f16_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1Fu;
  uint32_t m = h & 0x3FFu;
  if (e == 0x1Fu) return bits_f32(sign | 0x7F800000u | (m << 13));
  if (e != 0) return bits_f32(sign | ((e + 112u) << 23) | (m << 13));
  if (m == 0) return bits_f32(sign);
  {
    float v = (float)m * 5.9604644775390625e-8f;       /* m * 2^-24, exact */
    return sign ? -v : v;
  }
}

ORACLE_API float oracle_e4m3_to_f32(uint8_t b) {
  uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
  float v;
  if (e == 0xFu && m == 7u) return NAN;
  if (e == 0) v = (float)m * 0.001953125f;             /* m * 2^-9 */
  else v = ldexpf((float)(8u + m), (int)e - 10);       /* (1 + m/8) * 2^(e-7) */
  return (b & 0x80u) ? -v : v;
}

/* Saturating-finite RN conversion, as __nv_fp8_e4m3(float) (__NV_SATFINITE). */
ORACLE_API uint8_t oracle_f32_to_e4m3(float f) {
  uint32_t u = f32_bits(f);
  uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
  uint32_t a = u & 0x7FFFFFFFu;
  float x;
  if (a > 0x7F800000u) return (uint8_t)(sign | 0x7Fu);  /* NaN */
  x = bits_f32(a);
  if (x >= 448.0f) return (uint8_t)(sign | 0x7Eu);      /* saturate (inf too) */
  if (x < 0.0009765625f) return sign;                   /* < 2^-10: below half the least subnormal */
  {
    int e;
    float frac = frexpf(x, &e);                         /* x = frac * 2^e, frac in [0.5,1) */
    int exp_unb = e - 1;                                /* x = 1.xxx * 2^exp_unb */
    float scaled;
    uint32_t q;
    (void)frac;
    if (exp_unb < -6) exp_unb = -6;                     /* subnormal grid: step 2^-9 */
    scaled = ldexpf(x, 3 - exp_unb);                    /* in [8,16) for normals, [0,8) subnormal */
    q = (uint32_t)scaled;
    {
      float rem = scaled - (float)q;
      if (rem > 0.5f || (rem == 0.5f && (q & 1u))) q += 1u;
    }
    if (exp_unb == -6 && q < 8u) return (uint8_t)(sign | q);           /* subnormal */
    if (q == 16u) { q = 8u; exp_unb += 1; }
    {
      uint32_t code = ((uint32_t)(exp_unb + 7) << 3) | (q - 8u);
      if (code > 0x7Eu) code = 0x7Eu;
      return (uint8_t)(sign | code);
    }
  }
}

ORACLE_API void oracle_f32_to_bf16_n(const float* s, uint16_t* d, size_t n) { for (size_t i = 0; i < n; ++i) d[i] = oracle_f32_to_bf16(s[i]); }
ORACLE_API void oracle_f32_to_f16_n(const float* s, uint16_t* d, size_t n) { for (size_t i = 0; i < n; ++i) d[i] = oracle_f32_to_f16(s[i]); }
ORACLE_API void oracle_f32_to_e4m3_n(const float* s, uint8_t* d, size_t n) { for (size_t i = 0; i < n; ++i) d[i] = oracle_f32_to_e4m3(s[i]); }
ORACLE_API void oracle_bf16_to_f32_n(const uint16_t* s, float* d, size_t n) { for (size_t i = 0; i < n; ++i) d[i] = oracle_bf16_to_f32(s[i]); }
ORACLE_API void oracle_f16_to_f32_n(const uint16_t* s, float* d, size_t n) { for (size_t i = 0; i < n; ++i) d[i] = oracle_f16_to_f32(s[i]); }
ORACLE_API void oracle_e4m3_to_f32_n(const uint8_t* s, float* d, size_t n) { for (size_t i = 0; i < n; ++i) d[i] = oracle_e4m3_to_f32(s[i]); }

/* -------------------------------------------------------------- dense GEMM --
 * D[m][n] = C[m][n] + sum_k A[m][k] * B[n][k], fp32, k ascending — the loop of
 * choreo::cc::mma_exec_row_row<float,...> (runtime/choreo_cc.h:37-47). */
static void mma_row_row(float* D, const float* A, const float* B, const float* C,
                        int M, int N, int K, int lda, int ldb, int ldc) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float acc = C[(size_t)m * ldc + n];
      for (int k = 0; k < K; ++k) acc += A[(size_t)m * lda + k] * B[(size_t)n * ldb + k];
      D[(size_t)m * ldc + n] = acc;
    }
}

/* Whole-matrix GEMM in the structure the reference's CPU target gives the
 * persistent kernel (lib/Target/CPU/cc_codegen.cpp:1046-1066 sequential loops
 * over the parallel variables; tests/gpu/end2end/wgmma_persis.co:12-29): tiles
 * in schedule order, per K-tile one mma_exec_row_row on staged operands, fp32
 * accumulators. schedule_m/n may be NULL (row-major tile order). Rows
 * [row_begin,row_end) of the tile grid are computed (for threading/sampling). */
ORACLE_API void oracle_gemm_row_row(const float* lhs, const float* rhs, float* out,
                                    int M, int N, int K, int tm, int tn, int tk,
                                    const int32_t* schedule_m, const int32_t* schedule_n,
                                    int tile_begin, int tile_end) {
  const int tiles_n = (N + tn - 1) / tn;
  float* a_s = (float*)aligned_alloc(64, ((size_t)tm * tk * 4 + 63) / 64 * 64);
  float* b_s = (float*)aligned_alloc(64, ((size_t)tn * tk * 4 + 63) / 64 * 64);
  float* acc = (float*)aligned_alloc(64, ((size_t)tm * tn * 4 + 63) / 64 * 64);
  for (int t = tile_begin; t < tile_end; ++t) {
    const int bm = schedule_m ? schedule_m[t] : t / tiles_n;
    const int bn = schedule_n ? schedule_n[t] : t % tiles_n;
    const int m0 = bm * tm, n0 = bn * tn;
    const int mm = (M - m0 < tm) ? M - m0 : tm;
    const int nn = (N - n0 < tn) ? N - n0 : tn;
    if (mm <= 0 || nn <= 0) continue;
    memset(acc, 0, (size_t)tm * tn * 4);
    for (int k0 = 0; k0 < K; k0 += tk) {
      const int kk = (K - k0 < tk) ? K - k0 : tk;
      for (int i = 0; i < mm; ++i) memcpy(a_s + (size_t)i * tk, lhs + (size_t)(m0 + i) * K + k0, (size_t)kk * 4);
      for (int j = 0; j < nn; ++j) memcpy(b_s + (size_t)j * tk, rhs + (size_t)(n0 + j) * K + k0, (size_t)kk * 4);
      mma_row_row(acc, a_s, b_s, acc, mm, nn, kk, tk, tk, tn);
    }
    for (int i = 0; i < mm; ++i) memcpy(out + (size_t)(m0 + i) * N + n0, acc + (size_t)i * tn, (size_t)nn * 4);
  }
  free(a_s); free(b_s); free(acc);
}

/* ------------------------------------------------------- block-scaled GEMM --
 * Per 128-wide K block: P = A_kb * B_kb^T in fp32 (k ascending), then
 * acc = fmaf(P, sa[m,kb] * sb[n/128,kb], acc) — operation order of
 * scale_accumulator's fp32 branch (runtime/choreo_cute.h:3812-3813, 3851-3860)
 * applied once per K block as `mma.scale` does (wgmma_persis.co:136-143).
 * lhs/rhs are e4m3 bytes; out is fp32 (the caller rounds to the output type).
 * Computes output rows [row_begin,row_end). */
ORACLE_API void oracle_blockscale_gemm_e4m3(const uint8_t* lhs, const float* scale_lhs,
                                            const uint8_t* rhs, const float* scale_rhs,
                                            float* out, int M, int N, int K,
                                            int row_begin, int row_end) {
  const int KB = (K + 127) / 128;
  float lut[256];
  float* a_row = (float*)malloc((size_t)(K > 0 ? K : 1) * 4);
  float* b_f = (float*)malloc((size_t)N * (K > 0 ? K : 1) * 4);
  (void)M;
  for (int i = 0; i < 256; ++i) lut[i] = oracle_e4m3_to_f32((uint8_t)i);
  for (size_t i = 0; i < (size_t)N * K; ++i) b_f[i] = lut[rhs[i]];
  for (int m = row_begin; m < row_end; ++m) {
    for (int k = 0; k < K; ++k) a_row[k] = lut[lhs[(size_t)m * K + k]];
    for (int n = 0; n < N; ++n) {
      float acc = 0.0f;
      const float* b_row = b_f + (size_t)n * K;
      for (int kb = 0; kb < KB; ++kb) {
        const int k1 = (kb * 128 + 128 < K) ? kb * 128 + 128 : K;
        float p = 0.0f;
        for (int k = kb * 128; k < k1; ++k) p += a_row[k] * b_row[k];
        {
          const float s = scale_lhs[(size_t)m * KB + kb] * scale_rhs[(size_t)(n / 128) * KB + kb];
          acc = fmaf(p, s, acc);
        }
      }
      out[(size_t)m * N + n] = acc;
    }
  }
  free(a_row); free(b_f);
}

/* --------------------------------------------------------------- 2:4 sparse --
 * Metadata format of Sparse2to4HostPolicyWGMMA::encode (runtime/choreo.h:
 * 1539-1571): per group of four K positions a nibble idx0 | idx1<<2 with
 * idx0 < idx1; group 2j in the low nibble of byte j, group 2j+1 in the high
 * nibble; a group without exactly two non-zeros encodes (0,1). Elements are
 * 16-bit patterns (f16 or bf16); "non-zero" means to_f32(x) != 0, so +-0 are
 * zeros. */
ORACLE_API void oracle_sparse24_encode_u16(const uint16_t* dense, uint16_t* packed, uint8_t* meta,
                                           int M, int K) {
  const int groups = K / 4;
  memset(meta, 0, (size_t)M * (K / 8));
  for (int r = 0; r < M; ++r)
    for (int g = 0; g < groups; ++g) {
      const uint16_t* d = dense + (size_t)r * K + (size_t)g * 4;
      int idx[2] = {-1, -1}, nz = 0;
      for (int i = 0; i < 4; ++i)
        if ((d[i] & 0x7FFFu) != 0) { if (nz < 2) idx[nz] = i; ++nz; }
      if (nz != 2) { idx[0] = 0; idx[1] = 1; }
      packed[(size_t)r * (K / 2) + (size_t)g * 2 + 0] = d[idx[0]];
      packed[(size_t)r * (K / 2) + (size_t)g * 2 + 1] = d[idx[1]];
      {
        const uint8_t nib = (uint8_t)(idx[0] | (idx[1] << 2));
        uint8_t* b = meta + (size_t)r * (K / 8) + g / 2;
        if ((g & 1) == 0) *b = nib; else *b |= (uint8_t)(nib << 4);
      }
    }
}

/* Inverse: expands (packed, meta) into the dense [M,K] matrix. */
ORACLE_API void oracle_sparse24_decode_u16(const uint16_t* packed, const uint8_t* meta,
                                           uint16_t* dense, int M, int K) {
  memset(dense, 0, (size_t)M * K * 2);
  for (int r = 0; r < M; ++r)
    for (int g = 0; g < K / 4; ++g) {
      const uint8_t byte = meta[(size_t)r * (K / 8) + g / 2];
      const uint8_t nib = (g & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xF);
      const int i0 = nib & 3, i1 = (nib >> 2) & 3;
      dense[(size_t)r * K + (size_t)g * 4 + i0] = packed[(size_t)r * (K / 2) + (size_t)g * 2 + 0];
      dense[(size_t)r * K + (size_t)g * 4 + i1] = packed[(size_t)r * (K / 2) + (size_t)g * 2 + 1];
    }
}

/* Metadata re-layouts for the reference's Hopper kernels. `layout` 1 restates
 * Sparse2to4HostPolicyWGMMA::prepack (runtime/choreo.h:1573-1623): for every
 * 16-row block, row r in 0..7 and 32-wide K fragment kf (4 metadata bytes per
 * row), word (block+2r, kf) = bytes 0,1 of row block+r in the low half and
 * bytes 0,1 of row block+r+8 in the high half, word (block+2r+1, kf) the same
 * for bytes 2,3. `layout` 2 restates prepack_v2 (1631-1661): the same words
 * stored as [M/16, KF, 16]. M % 16 == 0, KM % 4 == 0. Returns 0, or -1 on a
 * shape the reference asserts against. */
ORACLE_API int oracle_sparse24_prepack_meta(const uint8_t* meta_u8, uint32_t* meta_u32, int M,
                                            int KM, int layout) {
  if (M % 16 != 0 || KM % 4 != 0 || (layout != 1 && layout != 2)) return -1;
  const int KF = KM / 4;
  for (int block = 0; block < M; block += 16)
    for (int r = 0; r < 8; ++r)
      for (int kf = 0; kf < KF; ++kf)
        for (int h = 0; h < 2; ++h) {
          const uint8_t* lo = meta_u8 + (size_t)(block + r) * KM + kf * 4 + 2 * h;
          const uint8_t* hi = meta_u8 + (size_t)(block + r + 8) * KM + kf * 4 + 2 * h;
          const uint32_t word = (uint32_t)lo[0] | ((uint32_t)lo[1] << 8) |
                                ((uint32_t)hi[0] << 16) | ((uint32_t)hi[1] << 24);
          const int rib = 2 * r + h;
          const size_t at = (layout == 1)
              ? (size_t)(block + rib) * KF + kf
              : ((size_t)(block / 16) * KF + kf) * 16 + rib;
          meta_u32[at] = word;
        }
  return 0;
}

/* --------------------------------------------------------- Hilbert schedule --
 * Restates build_hilbert_schedule (tests/gpu/end2end/wgmma_persis.co:156-197):
 * walk the Hilbert curve over the covering power-of-two square, keep cells
 * inside the tiles_m x tiles_n grid; schedule_m = x, schedule_n = y. */
ORACLE_API int oracle_hilbert_schedule(int tiles_m, int tiles_n, int32_t* schedule_m,
                                       int32_t* schedule_n) {
  int size = 1, count = 0;
  const int max_dim = tiles_m > tiles_n ? tiles_m : tiles_n;
  while (size < max_dim) size *= 2;
  for (int index = 0; index < size * size; ++index) {
    int x = 0, y = 0, d = index;
    for (int scale = 1; scale < size; scale *= 2) {
      const int rx = 1 & (d / 2);
      const int ry = 1 & (d ^ rx);
      if (ry == 0) {
        if (rx == 1) { x = scale - 1 - x; y = scale - 1 - y; }
        { const int tmp = x; x = y; y = tmp; }
      }
      x += scale * rx;
      y += scale * ry;
      d /= 4;
    }
    if (x < tiles_m && y < tiles_n) { schedule_m[count] = x; schedule_n[count] = y; ++count; }
  }
  return count;
}

/* Sample positions of the reference's sampled verifier (runtime/choreo.h:
 * 498-512 stride choice, 549-580 walk): flat indices idx = i*stride while
 * idx < M*N and fewer than num_samples were taken. Returns the count. */
ORACLE_API size_t oracle_sample_positions(size_t M, size_t N, size_t num_samples, size_t* idx_out) {
  const size_t total = M * N;
  size_t raw = total / num_samples, stride, n = 0;
  if (raw < 1) raw = 1;
  stride = raw;
  {
    size_t a = raw, b = N;
    while (b) { size_t t = b; b = a % b; a = t; }
    if (a != 1) {
      for (size_t s = raw + 1; s < total; ++s) {
        size_t x = s, y = N;
        while (y) { size_t t = y; y = x % y; x = t; }
        if (x == 1) { stride = s; break; }
      }
    }
  }
  for (size_t idx = 0; idx < total && n < num_samples; idx += stride) idx_out[n++] = idx;
  return n;
}

/* ---------------------------------------------------------------------- MoE --
 * No reference counterpart (parity unpinned). Definitions:
 *  topk_idx[t,0..k): the k largest raw logits of token t ordered by (logit
 *    descending, expert ascending); NaN logits order below every number.
 *  topk_w[t,j] = exp(l_j - max) / sum_all exp(l_i - max) in fp32 (sum in
 *    ascending expert order), then divided by the sum of the k selected
 *    (ascending j) when norm_topk.
 *  counts / offsets: histogram of topk_idx and its exclusive prefix sum.
 *  stable permutation: expanded row r = t*k+j goes to offsets[e] + (number of
 *    rows r' < r with the same expert). */
ORACLE_API void oracle_moe_route_topk(const float* logits, int T, int E, int k, int norm_topk,
                                      int32_t* topk_idx, float* topk_w, int32_t* counts,
                                      int32_t* offsets, int32_t* perm_to_src,
                                      int32_t* src_to_perm) {
  uint8_t* taken = (uint8_t*)malloc((size_t)E);
  int32_t* cursor = (int32_t*)malloc((size_t)(E + 1) * 4);
  memset(counts, 0, (size_t)E * 4);
  for (int t = 0; t < T; ++t) {
    const float* l = logits + (size_t)t * E;
    float mx = -INFINITY, denom = 0.0f, wsum = 0.0f;
    memset(taken, 0, (size_t)E);
    for (int e = 0; e < E; ++e) if (l[e] > mx) mx = l[e];
    for (int e = 0; e < E; ++e) denom += expf(l[e] - mx);
    for (int j = 0; j < k; ++j) {
      int best = -1;
      for (int e = 0; e < E; ++e) {
        if (taken[e]) continue;
        if (best < 0) { best = e; continue; }
        /* strictly greater wins; NaN never wins over a number */
        if (l[e] > l[best] || (isnan(l[best]) && !isnan(l[e]))) best = e;
      }
      taken[best] = 1;
      topk_idx[(size_t)t * k + j] = best;
      topk_w[(size_t)t * k + j] = expf(l[best] - mx) / denom;
      counts[best] += 1;
    }
    if (norm_topk) {
      for (int j = 0; j < k; ++j) wsum += topk_w[(size_t)t * k + j];
      for (int j = 0; j < k; ++j) topk_w[(size_t)t * k + j] /= wsum;
    }
  }
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  memcpy(cursor, offsets, (size_t)(E + 1) * 4);
  for (int r = 0; r < T * k; ++r) {
    const int e = topk_idx[r];
    const int pos = cursor[e]++;
    perm_to_src[pos] = r;
    src_to_perm[r] = pos;
  }
  free(taken); free(cursor);
}

/* Activation quantiser: per row and per 128-wide block scale = amax/448 (1 if
 * the block is all zero), q = RN_e4m3(x / scale). x is bf16 bits or fp32. */
ORACLE_API void oracle_quant_rows_e4m3_f32(const float* x, uint8_t* q, float* scale, int R, int H) {
  const int HB = (H + 127) / 128;
  for (int r = 0; r < R; ++r)
    for (int b = 0; b < HB; ++b) {
      const int c1 = (b * 128 + 128 < H) ? b * 128 + 128 : H;
      float amax = 0.0f, s;
      for (int c = b * 128; c < c1; ++c) { const float a = fabsf(x[(size_t)r * H + c]); if (a > amax) amax = a; }
      s = amax > 0.0f ? amax / 448.0f : 1.0f;
      scale[(size_t)r * HB + b] = s;
      for (int c = b * 128; c < c1; ++c) q[(size_t)r * H + c] = oracle_f32_to_e4m3(x[(size_t)r * H + c] / s);
    }
}

/* dst[pos,:] = src[perm_to_src[pos] / k, :], 16-bit elements. */
ORACLE_API void oracle_moe_permute_u16(const uint16_t* src, const int32_t* perm_to_src, int k,
                                       uint16_t* dst, int rows, int H) {
  for (int pos = 0; pos < rows; ++pos)
    memcpy(dst + (size_t)pos * H, src + (size_t)(perm_to_src[pos] / k) * H, (size_t)H * 2);
}

/* out[t,:] = RN_bf16( sum_j w[t,j] * y[src_to_perm[t*k+j], :] ), ascending j,
 * fp32 fmaf chain starting from 0. y and out are bf16 bits. */
ORACLE_API void oracle_moe_unpermute_bf16(const uint16_t* y, const int32_t* src_to_perm,
                                          const float* w, uint16_t* out, int T, int k, int H) {
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < H; ++c) {
      float acc = 0.0f;
      for (int j = 0; j < k; ++j) {
        const int pos = src_to_perm[(size_t)t * k + j];
        acc = fmaf(w[(size_t)t * k + j], oracle_bf16_to_f32(y[(size_t)pos * H + c]), acc);
      }
      out[(size_t)t * H + c] = oracle_f32_to_bf16(acc);
    }
}

/* Grouped block-scaled GEMM over expert-sorted rows; h fp32 [R,N] per the
 * block-scaled definition above with expert e's weights for rows in
 * [offsets[e], offsets[e+1]). When swiglu, out_bf16 [R,N/2] =
 * RN_bf16(silu(h[:, :N/2]) * h[:, N/2:]) with silu(v) = v / (1 + expf(-v));
 * otherwise out_bf16 [R,N] = RN_bf16(h). */
ORACLE_API void oracle_moe_grouped_gemm_e4m3(const uint8_t* x, const float* x_scale,
                                             const uint8_t* w, const float* w_scale,
                                             const int32_t* offsets, int E, int N, int K,
                                             int swiglu, uint16_t* out_bf16) {
  const int KB = (K + 127) / 128, NB = (N + 127) / 128;
  float* h = (float*)malloc((size_t)N * 4);
  float lut[256];
  for (int i = 0; i < 256; ++i) lut[i] = oracle_e4m3_to_f32((uint8_t)i);
  for (int e = 0; e < E; ++e) {
    const uint8_t* we = w + (size_t)e * N * K;
    const float* wse = w_scale + (size_t)e * NB * KB;
    for (int r = offsets[e]; r < offsets[e + 1]; ++r) {
      for (int n = 0; n < N; ++n) {
        float acc = 0.0f;
        for (int kb = 0; kb < KB; ++kb) {
          const int k1 = (kb * 128 + 128 < K) ? kb * 128 + 128 : K;
          float p = 0.0f;
          for (int kk = kb * 128; kk < k1; ++kk) p += lut[x[(size_t)r * K + kk]] * lut[we[(size_t)n * K + kk]];
          acc = fmaf(p, x_scale[(size_t)r * KB + kb] * wse[(size_t)(n / 128) * KB + kb], acc);
        }
        h[n] = acc;
      }
      if (swiglu) {
        const int Nh = N / 2;
        for (int c = 0; c < Nh; ++c) {
          const float g = h[c], u = h[Nh + c];
          out_bf16[(size_t)r * Nh + c] = oracle_f32_to_bf16((g / (1.0f + expf(-g))) * u);
        }
      } else {
        for (int n = 0; n < N; ++n) out_bf16[(size_t)r * N + n] = oracle_f32_to_bf16(h[n]);
      }
    }
  }
  free(h);
}
