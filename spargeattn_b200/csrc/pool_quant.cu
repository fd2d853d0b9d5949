// One pass over Q (128-row blocks) or K (64-row blocks): optional mean subtraction in the
// 16-bit type, block pooling, cosine self-similarity flag and per-block INT8 quantisation.
// Replaces triton_bmm_pool_sim_simmean_fuse_quant (spas_sage_attn/utils.py:161-214) and
// qk_quantize (utils.py:89-159). With 32-row blocks and no pooling it is the Q half of the per-warp
// quantiser (per_warp_int8, spas_sage_attn/quant_per_block.py:102-148: one scale per 32 query rows,
// ceil(N/128)*4 scales per head, 1e-7 for groups past the end).
//
// Arithmetic contract (shared with the CPU oracle):
//   * row sums (pool, sum of unit vectors): fp32 running sum over each run of 8 consecutive rows,
//     fp64 across the runs, one rounding to fp32;
//   * row norms: fp32 running sum of squares over each run of 8 consecutive channels, then an fp32
//     butterfly (partner = index xor D/16 ... xor 1) across the D/8 runs; sqrt and 1/x are IEEE;
//   * the self-similarity uses  sum_ij <a_i, a_j> = || sum_i a_i ||^2  with a_i = fp16(x_i * (1/||x_i||));
//   * a block with fewer than `BS` rows, or with an all-zero row, is never self-similar
//     (the reference gets there through a 0/0 NaN, utils.py:194-199);
//   * scale = fma(max|x|, RN(1/127), 1e-7): the compiled reference kernel contracts `max / 127. + 1e-7`
//     (utils.py:206-207) into one FMA with the reciprocal constant -- checked bit for bit against its output
//     on a B200; q = trunc(x / scale + 0.5 * sign) with the IEEE quotient (the reference's approximate
//     quotient gave the same INT8 value for every element compared);
// The quotient is formed without a per-element division: with r = RN(1/scale), y0 = x*r,
// e = fma(-scale, y0, x) (exact remainder), y = fma(e, r, y0) is the correctly rounded x/scale.
#include "common.cuh"

namespace sparge {

template <typename T>
__device__ __forceinline__ float unpack16(uint32_t w, int hi);
template <>
__device__ __forceinline__ float unpack16<__nv_bfloat16>(uint32_t w, int hi) {
  return __uint_as_float(hi ? (w & 0xffff0000u) : (w << 16));
}
template <>
__device__ __forceinline__ float unpack16<__half>(uint32_t w, int hi) {
  return __half2float(__ushort_as_half((unsigned short)(hi ? (w >> 16) : (w & 0xffffu))));
}
template <typename T>
__device__ __forceinline__ uint32_t bits16(float v);
template <>
__device__ __forceinline__ uint32_t bits16<__nv_bfloat16>(float v) { return __bfloat16_as_ushort(__float2bfloat16_rn(v)); }
template <>
__device__ __forceinline__ uint32_t bits16<__half>(float v) { return __half_as_ushort(__float2half_rn(v)); }

// Thread layout: TPR = D/8 threads per row (8 channels each), G = BS/8 row groups; thread (g, cg)
// owns rows 8g..8g+7 of channel group cg. blockDim = G * TPR (64 .. 256).
template <typename T, int D, int BS, bool HAS_KM, bool WANT_POOL>
__global__ void __launch_bounds__((BS / 8) * (D / 8))
pool_quant_kernel(const T* __restrict__ x, const T* __restrict__ km, const float* __restrict__ simthr,
                  T* __restrict__ pool, uint8_t* __restrict__ sim, int8_t* __restrict__ xq,
                  float* __restrict__ scale_out, int N, int H, int nb, long long sb, long long sh, long long sn) {
  constexpr int TPR = D / 8;
  constexpr int G = BS / 8;
  constexpr int NT = G * TPR;
  constexpr int NW = NT / 32;
  __shared__ float s_part[WANT_POOL ? 2 : 1][WANT_POOL ? G : 1][WANT_POOL ? D : 1];   // pooled / unit-vector partials
  __shared__ float s_amax[NW];
  __shared__ double s_tot[D / 32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid % TPR, g = tid / TPR;
  const int blk = blockIdx.x, bh = blockIdx.y;
  const int row_base = blk * BS;
  const int rows_here = max(0, min(BS, N - row_base));   // 0: a 32-row group past the end (scale 1e-7, nothing else)
  const T* xb = x + (size_t)(bh / H) * sb + (size_t)(bh % H) * sh + (size_t)row_base * sn;

  float kmv[8];
  if (HAS_KM) {
    const uint4 p = *reinterpret_cast<const uint4*>(km + (size_t)bh * D + cg * 8);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 8; i++) kmv[i] = unpack16<T>(w[i >> 1], i & 1);
  }

  // ---- load the thread's 8 rows (all loads in flight before the first use)
  uint4 raw[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = g * 8 + i;
    raw[i] = (row < rows_here) ? *reinterpret_cast<const uint4*>(xb + (size_t)row * sn + cg * 8) : make_uint4(0, 0, 0, 0);
  }

  float amax = 0.f;
  float pacc[8], hacc[8];
#pragma unroll
  for (int c = 0; c < 8; c++) { pacc[c] = 0.f; hacc[c] = 0.f; }
  int zero_row = 0;

#pragma unroll
  for (int i = 0; i < 8; i++) {
    const bool valid = (g * 8 + i) < rows_here;
    uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
    float v[8];
#pragma unroll
    for (int c = 0; c < 8; c++) v[c] = unpack16<T>(w[c >> 1], c & 1);
    if (HAS_KM) {
      if (valid) {
#pragma unroll
        for (int c = 0; c < 8; c += 2) {   // subtraction rounded to the 16-bit type; keep the rounded bits
          const uint32_t lo = bits16<T>(__fsub_rn(v[c], kmv[c])), hi = bits16<T>(__fsub_rn(v[c + 1], kmv[c + 1]));
          w[c >> 1] = lo | (hi << 16);
        }
        raw[i] = make_uint4(w[0], w[1], w[2], w[3]);
#pragma unroll
        for (int c = 0; c < 8; c++) v[c] = unpack16<T>(w[c >> 1], c & 1);
      }
    }
    amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))),
                             fmaxf(fmaxf(fabsf(v[4]), fabsf(v[5])), fmaxf(fabsf(v[6]), fabsf(v[7])))));
    if (WANT_POOL) {
      float ss = 0.f;
#pragma unroll
      for (int c = 0; c < 8; c++) {
        pacc[c] = __fadd_rn(pacc[c], v[c]);
        ss = __fmaf_rn(v[c], v[c], ss);
      }
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
      const float nrm = __fsqrt_rn(ss);
      if (valid) {
        if (nrm == 0.f) {
          zero_row = 1;
        } else {
          const float rinv = __fdiv_rn(1.0f, nrm);
#pragma unroll
          for (int c = 0; c < 8; c++)
            hacc[c] = __fadd_rn(hacc[c], __half2float(__float2half_rn(__fmul_rn(v[c], rinv))));
        }
      }
    }
  }

  // ---- block amax -> scale
  amax = warp_max(amax);
  if (lane == 0) s_amax[warp] = amax;
  if (WANT_POOL) {
#pragma unroll
    for (int c = 0; c < 8; c++) {
      s_part[0][g][cg * 8 + c] = pacc[c];
      s_part[WANT_POOL ? 1 : 0][g][cg * 8 + c] = hacc[c];
    }
  }
  const int any_zero = __syncthreads_or(zero_row);
  amax = s_amax[0];
#pragma unroll
  for (int w = 1; w < NW; w++) amax = fmaxf(amax, s_amax[w]);
  const float scale = __fmaf_rn(amax, 1.0f / 127.0f, 1e-7f);
  const float rs = __fdiv_rn(1.0f, scale);
  if (tid == 0) scale_out[(size_t)bh * nb + blk] = scale;

  // ---- quantise from registers
  int8_t* qb = xq + ((size_t)bh * N + row_base) * D;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = g * 8 + i;
    if (row < rows_here) {
      const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
      uint32_t out[2] = {0u, 0u};
#pragma unroll
      for (int c = 0; c < 8; c++) {
        const float xv = unpack16<T>(w[c >> 1], c & 1);
        const float y0 = __fmul_rn(xv, rs);
        const float e = __fmaf_rn(-scale, y0, xv);
        float y = __fmaf_rn(e, rs, y0);                      // == RN(xv / scale)
        y = __fadd_rn(y, y >= 0.f ? 0.5f : -0.5f);
        const int q = (int)y;                                // truncation toward zero
        out[c >> 2] |= (uint32_t)(q & 0xff) << ((c & 3) * 8);
      }
      *reinterpret_cast<uint2*>(qb + (size_t)row * D + cg * 8) = make_uint2(out[0], out[1]);
    }
  }

  if (WANT_POOL) {
    double sq = 0.0;
    if (tid < D) {
      double ps = 0.0, hs = 0.0;
#pragma unroll
      for (int r = 0; r < G; r++) {
        ps += (double)s_part[0][r][tid];
        hs += (double)s_part[WANT_POOL ? 1 : 0][r][tid];
      }
      pool[((size_t)bh * nb + blk) * D + tid] = Elem<T>::from_float(__fdiv_rn((float)ps, (float)rows_here));
      sq = hs * hs;
    }
    if (warp < D / 32) {
      sq = warp_sum(sq);
      if (lane == 0) s_tot[warp] = sq;
    }
    __syncthreads();
    if (tid == 0) {
      double tot = 0.0;
#pragma unroll
      for (int w = 0; w < D / 32; w++) tot += s_tot[w];
      const float bsf = (float)rows_here;
      const float val = __fdiv_rn((float)tot, __fmul_rn(bsf, bsf));
      const bool ok = (rows_here == BS) && !any_zero && (val > simthr[bh % H]);
      sim[(size_t)bh * nb + blk] = ok ? 1 : 0;
    }
  }
}

template <typename T, int D, int BS>
static int launch_pq(const void* x, const void* km, const float* thr, void* pool, uint8_t* sim, int8_t* xq, float* sc,
                     int BH, int H, int N, long long sb, long long sh, long long sn, cudaStream_t st) {
  const int nb = BS == 32 ? (N + 127) / 128 * 4 : (N + BS - 1) / BS;
  dim3 grid(nb, BH);
  const bool has_km = km != nullptr, want = thr != nullptr;
#define SPARGE_PQ(KM, WP)                                                                                         \
  pool_quant_kernel<T, D, BS, KM, WP><<<grid, (BS / 8) * (D / 8), 0, st>>>((const T*)x, (const T*)km, thr, (T*)pool, sim, xq, sc, \
                                                            N, H, nb, sb, sh, sn)
  if (has_km && want) SPARGE_PQ(true, true);
  else if (has_km) SPARGE_PQ(true, false);
  else if (want) SPARGE_PQ(false, true);
  else SPARGE_PQ(false, false);
#undef SPARGE_PQ
  return launch_status();
}

template <typename T>
static int dispatch_pq(const void* x, const void* km, const float* thr, void* pool, uint8_t* sim, int8_t* xq, float* sc,
                       int BH, int H, int N, int D, int block, long long sb, long long sh, long long sn, cudaStream_t st) {
  if (D == 64 && block == 32) return launch_pq<T, 64, 32>(x, km, thr, pool, sim, xq, sc, BH, H, N, sb, sh, sn, st);
  if (D == 128 && block == 32) return launch_pq<T, 128, 32>(x, km, thr, pool, sim, xq, sc, BH, H, N, sb, sh, sn, st);
  if (D == 64 && block == 128) return launch_pq<T, 64, 128>(x, km, thr, pool, sim, xq, sc, BH, H, N, sb, sh, sn, st);
  if (D == 64 && block == 64) return launch_pq<T, 64, 64>(x, km, thr, pool, sim, xq, sc, BH, H, N, sb, sh, sn, st);
  if (D == 128 && block == 128) return launch_pq<T, 128, 128>(x, km, thr, pool, sim, xq, sc, BH, H, N, sb, sh, sn, st);
  return launch_pq<T, 128, 64>(x, km, thr, pool, sim, xq, sc, BH, H, N, sb, sh, sn, st);
}

}  // namespace sparge

extern "C" int sparge_pool_quant_strided(const void* x, const void* km, const float* simthreshd1, void* pool,
                                         uint8_t* sim, int8_t* x_int8, float* scale, int B, int H, int N, int D,
                                         int block, int dtype, long long stride_b, long long stride_h,
                                         long long stride_n, sparge_stream_t stream) {
  using namespace sparge;
  if (!x || !x_int8 || !scale) return SPARGE_ERR_NULL;
  if (simthreshd1 && (!pool || !sim)) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (block != 32 && block != 64 && block != 128) ||
      (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if (block == 32 && simthreshd1) return SPARGE_ERR_UNSUPPORTED;   // 32-row groups are a quantiser granularity only
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  if (!strides_ok(x, stride_b, stride_h, stride_n)) return SPARGE_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == SPARGE_F16)
    return dispatch_pq<__half>(x, km, simthreshd1, pool, sim, x_int8, scale, B * H, H, N, D, block, stride_b, stride_h,
                               stride_n, st);
  return dispatch_pq<__nv_bfloat16>(x, km, simthreshd1, pool, sim, x_int8, scale, B * H, H, N, D, block, stride_b,
                                    stride_h, stride_n, st);
}

extern "C" int sparge_pool_quant(const void* x, const void* km, const float* simthreshd1, void* pool, uint8_t* sim,
                                 int8_t* x_int8, float* scale, int B, int H, int N, int D, int block, int dtype,
                                 sparge_stream_t stream) {
  return sparge_pool_quant_strided(x, km, simthreshd1, pool, sim, x_int8, scale, B, H, N, D, block, dtype,
                                   (long long)H * N * D, (long long)N * D, D, stream);
}
