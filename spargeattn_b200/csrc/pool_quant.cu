// One pass over Q (128-row blocks) or K (64-row blocks): optional mean subtraction in the
// 16-bit type, block pooling, cosine self-similarity flag and per-block INT8 quantisation.
// Replaces triton_bmm_pool_sim_simmean_fuse_quant (spas_sage_attn/utils.py:161-214) and
// qk_quantize (utils.py:89-159).
//
// Arithmetic contract (shared with the CPU oracle):
//   * sums over rows / channels accumulate in fp64 and are rounded to fp32 once;
//   * the self-similarity uses  sum_ij <a_i, a_j> = || sum_i a_i ||^2  with a_i = fp16(x_i / ||x_i||);
//   * a block with fewer than `BS` rows, or with an all-zero row, is never self-similar
//     (the reference gets there through a 0/0 NaN, utils.py:194-199);
//   * scale = max|x| / 127 + 1e-7, q = trunc(x / scale + 0.5 * sign), IEEE fp32 division.
#include "common.cuh"

namespace sparge {

template <typename T, int D, int BS, bool HAS_KM, bool WANT_POOL>
__global__ void __launch_bounds__(256) pool_quant_kernel(const T* __restrict__ x, const T* __restrict__ km,
                                                         const float* __restrict__ simthr, T* __restrict__ pool,
                                                         uint8_t* __restrict__ sim, int8_t* __restrict__ xq,
                                                         float* __restrict__ scale_out, int N, int H, int nb) {
  constexpr int TPR = D / 8;          // threads per row (8 or 16)
  constexpr int RPP = 256 / TPR;      // rows per pass (32 or 16)
  constexpr int PASSES = BS / RPP;
  __shared__ double red[RPP][D];      // 16 KB
  __shared__ float s_amax[8];
  __shared__ double s_tot[8];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int cg = tid % TPR, r0 = tid / TPR;
  const int blk = blockIdx.x, bh = blockIdx.y;
  const int row_base = blk * BS;
  const int rows_here = min(BS, N - row_base);
  const T* xb = x + ((size_t)bh * N + row_base) * D;

  float kmv[8];
  if (HAS_KM) {
    Pack8<T> p = *reinterpret_cast<const Pack8<T>*>(km + (size_t)bh * D + cg * 8);
#pragma unroll
    for (int i = 0; i < 8; i++) kmv[i] = Elem<T>::to_float(p.v[i]);
  }

  float xv[PASSES][8];
  float amax = 0.f;
  double pacc[8], hacc[8];
#pragma unroll
  for (int i = 0; i < 8; i++) { pacc[i] = 0.0; hacc[i] = 0.0; }
  int zero_row = 0;

#pragma unroll
  for (int p = 0; p < PASSES; p++) {
    const int row = r0 + p * RPP;
    const bool valid = row < rows_here;
    if (valid) {
      Pack8<T> pk = *reinterpret_cast<const Pack8<T>*>(xb + (size_t)row * D + cg * 8);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        float v = Elem<T>::to_float(pk.v[i]);
        if (HAS_KM) v = Elem<T>::to_float(Elem<T>::from_float(__fsub_rn(v, kmv[i])));
        xv[p][i] = v;
        amax = fmaxf(amax, fabsf(v));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; i++) xv[p][i] = 0.f;
    }
    if (WANT_POOL) {
      double ss = 0.0;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        pacc[i] += (double)xv[p][i];
        ss += (double)xv[p][i] * (double)xv[p][i];
      }
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float nrm = __fsqrt_rn((float)ss);
      if (valid) {
        if (nrm == 0.f) {
          zero_row = 1;
        } else {
#pragma unroll
          for (int i = 0; i < 8; i++) hacc[i] += (double)__half2float(__float2half_rn(__fdiv_rn(xv[p][i], nrm)));
        }
      }
    }
  }

  // ---- block amax -> scale
  amax = warp_max(amax);
  if (lane == 0) s_amax[warp] = amax;
  __syncthreads();
  amax = s_amax[0];
#pragma unroll
  for (int w = 1; w < 8; w++) amax = fmaxf(amax, s_amax[w]);
  const float scale = __fadd_rn(__fdiv_rn(amax, 127.0f), 1e-7f);
  if (tid == 0) scale_out[(size_t)bh * nb + blk] = scale;

  // ---- quantise from registers
  int8_t* qb = xq + ((size_t)bh * N + row_base) * D;
#pragma unroll
  for (int p = 0; p < PASSES; p++) {
    const int row = r0 + p * RPP;
    if (row < rows_here) {
      uint32_t w[2] = {0u, 0u};
#pragma unroll
      for (int i = 0; i < 8; i++) {
        float y = __fdiv_rn(xv[p][i], scale);
        y = __fadd_rn(y, y >= 0.f ? 0.5f : -0.5f);
        const int q = (int)y;   // truncation toward zero
        w[i >> 2] |= (uint32_t)(q & 0xff) << ((i & 3) * 8);
      }
      *reinterpret_cast<uint2*>(qb + (size_t)row * D + cg * 8) = make_uint2(w[0], w[1]);
    }
  }

  if (WANT_POOL) {
    // ---- pooled mean
#pragma unroll
    for (int i = 0; i < 8; i++) red[r0][cg * 8 + i] = pacc[i];
    const int any_zero = __syncthreads_or(zero_row);
    if (tid < D) {
      double s = 0.0;
#pragma unroll 4
      for (int r = 0; r < RPP; r++) s += red[r][tid];
      pool[((size_t)bh * nb + blk) * D + tid] = Elem<T>::from_float(__fdiv_rn((float)s, (float)rows_here));
    }
    __syncthreads();
    // ---- || sum_i a_i ||^2
#pragma unroll
    for (int i = 0; i < 8; i++) red[r0][cg * 8 + i] = hacc[i];
    __syncthreads();
    double sq = 0.0;
    if (tid < D) {
      double s = 0.0;
#pragma unroll 4
      for (int r = 0; r < RPP; r++) s += red[r][tid];
      sq = s * s;
    }
    sq = warp_sum(sq);
    if (lane == 0) s_tot[warp] = sq;
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
                     int BH, int H, int N, cudaStream_t st) {
  const int nb = (N + BS - 1) / BS;
  dim3 grid(nb, BH);
  const bool has_km = km != nullptr, want = thr != nullptr;
#define SPARGE_PQ(KM, WP)                                                                                         \
  pool_quant_kernel<T, D, BS, KM, WP><<<grid, 256, 0, st>>>((const T*)x, (const T*)km, thr, (T*)pool, sim, xq, sc, \
                                                            N, H, nb)
  if (has_km && want) SPARGE_PQ(true, true);
  else if (has_km) SPARGE_PQ(true, false);
  else if (want) SPARGE_PQ(false, true);
  else SPARGE_PQ(false, false);
#undef SPARGE_PQ
  return launch_status();
}

template <typename T>
static int dispatch_pq(const void* x, const void* km, const float* thr, void* pool, uint8_t* sim, int8_t* xq, float* sc,
                       int BH, int H, int N, int D, int block, cudaStream_t st) {
  if (D == 64 && block == 128) return launch_pq<T, 64, 128>(x, km, thr, pool, sim, xq, sc, BH, H, N, st);
  if (D == 64 && block == 64) return launch_pq<T, 64, 64>(x, km, thr, pool, sim, xq, sc, BH, H, N, st);
  if (D == 128 && block == 128) return launch_pq<T, 128, 128>(x, km, thr, pool, sim, xq, sc, BH, H, N, st);
  return launch_pq<T, 128, 64>(x, km, thr, pool, sim, xq, sc, BH, H, N, st);
}

}  // namespace sparge

extern "C" int sparge_pool_quant(const void* x, const void* km, const float* simthreshd1, void* pool, uint8_t* sim,
                                 int8_t* x_int8, float* scale, int B, int H, int N, int D, int block, int dtype,
                                 sparge_stream_t stream) {
  using namespace sparge;
  if (!x || !x_int8 || !scale) return SPARGE_ERR_NULL;
  if (simthreshd1 && (!pool || !sim)) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (block != 64 && block != 128) ||
      (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == SPARGE_F16)
    return dispatch_pq<__half>(x, km, simthreshd1, pool, sim, x_int8, scale, B * H, H, N, D, block, st);
  return dispatch_pq<__nv_bfloat16>(x, km, simthreshd1, pool, sim, x_int8, scale, B * H, H, N, D, block, st);
}
