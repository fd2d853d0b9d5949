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

// Packed helpers: two channels per 32-bit word in, two fp32 lanes out. Every arithmetic step below is the
// per-lane IEEE operation of the scalar formulation (packed f32x2 instructions round each lane on its own),
// so results are bit-identical to it while taking half the issue slots.
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t w);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2_rn(float2 v);
template <>
__device__ __forceinline__ uint32_t pack2_rn<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 h = __float22bfloat162_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2_rn<__half>(float2 v) {
  const __half2 h = __float22half2_rn(v);
  return *reinterpret_cast<const uint32_t*>(&h);
}
// {sat8(hi), sat8(lo)} into the low half of the result, the low half of `upper` into its high half
__device__ __forceinline__ uint32_t pack_s8x2(int hi, int lo, uint32_t upper) {
  uint32_t d;
  asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(hi), "r"(lo), "r"(upper));
  return d;
}

// Thread layout: TPR = D/8 threads per row (8 channels each), G = BS/8 row groups; thread (g, cg)
// owns rows 8g..8g+7 of channel group cg. blockDim = G * TPR (32 .. 256).
//
// Row norms: every thread has a partial sum of squares for each of its 8 rows. The butterfly over the TPR
// threads of a row is run as a reduce-scatter -- at the step with partner distance b a thread keeps the half of
// its rows selected by that bit of its index and receives the partner's partials for them -- so the additions
// are those of the plain butterfly (same partners, same order xor TPR/2 ... xor 1) but each row's total, its
// square root and its reciprocal are computed once instead of by all TPR threads; the reciprocals then go back
// to the row's threads with one shuffle per row.
// Registers are capped so that 768 threads stay resident per SM (three 128-row blocks of D = 128): measured
// 46 / 48 us for Q / K on a [1, 12, 32760, 128] tensor against 52 / 53 us with 512 resident threads and 63 / 50
// with 1024 (which spills).
#ifndef PQ_RESIDENT_THREADS
#define PQ_RESIDENT_THREADS 768
#endif
template <typename T, int D, int BS, bool HAS_KM, bool WANT_POOL>
__global__ void __launch_bounds__((BS / 8) * (D / 8), PQ_RESIDENT_THREADS / ((BS / 8) * (D / 8)))
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

  float2 kmv[4];
  if (HAS_KM) {
    const uint4 p = *reinterpret_cast<const uint4*>(km + (size_t)bh * D + cg * 8);
    const uint32_t w[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int c = 0; c < 4; c++) {
      kmv[c] = unpack2<T>(w[c]);
      kmv[c] = make_float2(-kmv[c].x, -kmv[c].y);          // x - m is evaluated as x + (-m): the same rounding
    }
  }

  // ---- load the thread's 8 rows (all loads in flight before the first use)
  uint4 raw[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = g * 8 + i;
    raw[i] = (row < rows_here) ? *reinterpret_cast<const uint4*>(xb + (size_t)row * sn + cg * 8) : make_uint4(0, 0, 0, 0);
  }

  // ---- pass 1: mean subtraction in the 16-bit type, amax, pooled sums, partial sums of squares
  float amax = 0.f;
  float2 pacc[4];
  float ss[8];
#pragma unroll
  for (int c = 0; c < 4; c++) pacc[c] = make_float2(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < 8; i++) {
    uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
    float2 v[4];
#pragma unroll
    for (int c = 0; c < 4; c++) v[c] = unpack2<T>(w[c]);
    if (HAS_KM) {
      if ((g * 8 + i) < rows_here) {   // padded rows stay zero
#pragma unroll
        for (int c = 0; c < 4; c++) {   // subtraction rounded to the 16-bit type; keep the rounded bits
          w[c] = pack2_rn<T>(__fadd2_rn(v[c], kmv[c]));
          v[c] = unpack2<T>(w[c]);
        }
        raw[i] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    amax = fmaxf(amax, fmaxf(fmaxf(fmaxf(fabsf(v[0].x), fabsf(v[0].y)), fmaxf(fabsf(v[1].x), fabsf(v[1].y))),
                             fmaxf(fmaxf(fabsf(v[2].x), fabsf(v[2].y)), fmaxf(fabsf(v[3].x), fabsf(v[3].y)))));
    if (WANT_POOL) {
      float q = 0.f;
#pragma unroll
      for (int c = 0; c < 4; c++) {
        pacc[c] = __fadd2_rn(pacc[c], v[c]);
        q = __fmaf_rn(v[c].x, v[c].x, q);                  // one chain over the 8 channels in ascending order
        q = __fmaf_rn(v[c].y, v[c].y, q);
      }
      ss[i] = q;
    }
  }

  // ---- row norms -> reciprocals, one row per thread (see the header)
  float rinv[8];
  int zero_row = 0;
  if (WANT_POOL) {
    float vals[8];
#pragma unroll
    for (int i = 0; i < 8; i++) vals[i] = ss[i];
    int n = 8;
#pragma unroll
    for (int b = TPR / 2; b > 0; b >>= 1) {
      if (n > 1) {
        const bool upper = (cg & b) != 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          if (j < n / 2) {
            const float keep = upper ? vals[n / 2 + j] : vals[j];
            const float send = upper ? vals[j] : vals[n / 2 + j];
            vals[j] = __fadd_rn(keep, __shfl_xor_sync(0xffffffffu, send, b));
          }
        }
        n >>= 1;
      } else {
        vals[0] = __fadd_rn(vals[0], __shfl_xor_sync(0xffffffffu, vals[0], b));
      }
    }
    // this thread now holds the total of row `mine` of its group's 8 rows
    const int mine = TPR == 16 ? (cg >> 1) : cg;
    const float nrm = __fsqrt_rn(vals[0]);
    const bool live = (g * 8 + mine) < rows_here;
    float r = 0.f;                                          // padded and all-zero rows add zeros to the unit-vector sum
    if (live && nrm == 0.f) zero_row = 1;
    if (live && nrm != 0.f) r = __fdiv_rn(1.0f, nrm);
    const int group_lane0 = lane & ~(TPR - 1);
#pragma unroll
    for (int i = 0; i < 8; i++) rinv[i] = __shfl_sync(0xffffffffu, r, group_lane0 + (TPR == 16 ? 2 * i : i));
  }

  // ---- block amax -> scale
  amax = warp_max(amax);
  if (lane == 0) s_amax[warp] = amax;
  if (WANT_POOL) {
#pragma unroll
    for (int c = 0; c < 4; c++) {
      s_part[0][g][cg * 8 + 2 * c] = pacc[c].x;
      s_part[0][g][cg * 8 + 2 * c + 1] = pacc[c].y;
    }
  }
  const int any_zero = __syncthreads_or(zero_row);
  amax = s_amax[0];
#pragma unroll
  for (int w = 1; w < NW; w++) amax = fmaxf(amax, s_amax[w]);
  const float scale = __fmaf_rn(amax, 1.0f / 127.0f, 1e-7f);
  const float rs = __fdiv_rn(1.0f, scale);
  if (tid == 0) scale_out[(size_t)bh * nb + blk] = scale;

  // ---- pass 2 from registers: unit vectors (fp16-rounded) summed per channel, INT8 quantisation
  const float2 rs2 = make_float2(rs, rs), nscale2 = make_float2(-scale, -scale);
  float2 hacc[4];
#pragma unroll
  for (int c = 0; c < 4; c++) hacc[c] = make_float2(0.f, 0.f);
  int8_t* qb = xq + ((size_t)bh * N + row_base) * D;
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int row = g * 8 + i;
    const uint32_t w[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
    int q[8];
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const float2 xv = unpack2<T>(w[c]);
      if (WANT_POOL) {
        const float2 u = __fmul2_rn(xv, make_float2(rinv[i], rinv[i]));
        hacc[c] = __fadd2_rn(hacc[c], __half22float2(__float22half2_rn(u)));
      }
      const float2 y0 = __fmul2_rn(xv, rs2);
      const float2 e = __ffma2_rn(nscale2, y0, xv);        // exact remainder
      float2 y = __ffma2_rn(e, rs2, y0);                   // == RN(xv / scale) per lane
      // + 0.5 with the sign of y, then truncation toward zero (y = -0 gives 0 either way)
      const float2 hlf = make_float2(__uint_as_float((__float_as_uint(y.x) & 0x80000000u) | 0x3f000000u),
                                     __uint_as_float((__float_as_uint(y.y) & 0x80000000u) | 0x3f000000u));
      y = __fadd2_rn(y, hlf);
      q[2 * c] = (int)y.x;
      q[2 * c + 1] = (int)y.y;
    }
    if (row < rows_here) {
      const uint32_t lo = pack_s8x2(q[1], q[0], pack_s8x2(q[3], q[2], 0u));
      const uint32_t hi = pack_s8x2(q[5], q[4], pack_s8x2(q[7], q[6], 0u));
      *reinterpret_cast<uint2*>(qb + (size_t)row * D + cg * 8) = make_uint2(lo, hi);
    }
  }

  if (WANT_POOL) {
#pragma unroll
    for (int c = 0; c < 4; c++) {
      s_part[1][g][cg * 8 + 2 * c] = hacc[c].x;
      s_part[1][g][cg * 8 + 2 * c + 1] = hacc[c].y;
    }
    __syncthreads();
    double sq = 0.0;
    if (tid < D) {
      double ps = 0.0, hs = 0.0;
#pragma unroll
      for (int r = 0; r < G; r++) {
        ps += (double)s_part[0][r][tid];
        hs += (double)s_part[1][r][tid];
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
