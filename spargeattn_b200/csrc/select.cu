// Mask predictor back end: pooled QK^T row -> softmax -> stable top-k (or cdf) selection ->
// forced blocks / causal / sink -> block mask + delta-encoded LUT, one CTA per (b, h, q-block) row.
// Replaces spas_sage_attn/utils.py:386-420 (bmm, masked fills, softmax, sort, cumsum,
// triton_fill_block_map_kernel :282-292, triton_fill_causal_mask :304-311) and
// triton_block_map_to_lut_kernel (utils.py:54-74).
//
// Arithmetic contract (shared with the CPU oracle):
//   score  = T( fma-chain over ascending d, fp32 ) ; score = T( float(score) * float(D^-0.5) )
//   p      = T( float( exp(double(score) - max) / sum ) )           (fp64 softmax)
//   top-k  = first n_sel of a stable descending order of p (ties -> lower block index),
//            n_sel = clamp(int(topk[h] * nk), 1, nk)
//   cdf    = n_sel = #{ r : T(prefix_r) <= cdfthreshd[h] } over that order, prefix in fp32,
//            clamped to [1, nk]
#include <cfloat>

#include "common.cuh"

namespace sparge {

constexpr int kSelThreads = 256;

// Exclusive prefix count of `flag` over the CTA's threads in thread order, plus CTA total.
// s_warp must hold kSelThreads/32 ints. Contains two __syncthreads.
__device__ __forceinline__ int block_exclusive_count(bool flag, int* s_warp, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned b = __ballot_sync(0xffffffffu, flag);
  const int within = __popc(b & ((1u << lane) - 1u));
  if (lane == 0) s_warp[warp] = __popc(b);
  __syncthreads();
  int before = 0, tot = 0;
#pragma unroll
  for (int w = 0; w < kSelThreads / 32; w++) {
    const int c = s_warp[w];
    before += (w < warp) ? c : 0;
    tot += c;
  }
  __syncthreads();
  total = tot;
  return before + within;
}

// Writes one LUT row from the list of live block indices idx[0..count).
__device__ __forceinline__ void write_lut_row(const int* idx, int count, int nk, int32_t* lut_row, int32_t* valid_out) {
  for (int r = threadIdx.x; r < nk; r += kSelThreads) {
    int v = 0;
    if (r < count) v = idx[r] - (r > 0 ? idx[r - 1] : 0);
    lut_row[r] = v;
  }
  if (threadIdx.x == 0) *valid_out = count;
}

template <typename T>
__device__ __forceinline__ uint32_t key_bits(T v);
template <>
__device__ __forceinline__ uint32_t key_bits<__half>(__half v) { return (uint32_t)__half_as_ushort(v); }
template <>
__device__ __forceinline__ uint32_t key_bits<__nv_bfloat16>(__nv_bfloat16 v) { return (uint32_t)__bfloat16_as_ushort(v); }
template <typename T>
__device__ __forceinline__ float key_value(uint32_t k);
template <>
__device__ __forceinline__ float key_value<__half>(uint32_t k) { return __half2float(__ushort_as_half((unsigned short)k)); }
template <>
__device__ __forceinline__ float key_value<__nv_bfloat16>(uint32_t k) {
  return __bfloat162float(__ushort_as_bfloat16((unsigned short)k));
}

// dynamic smem: double e[nk] | uint32 key[nk] | int idx[nk] | float qrow[D]
template <typename T, int D>
__global__ void __launch_bounds__(kSelThreads) select_kernel(const T* __restrict__ pq, const T* __restrict__ pk,
                                                             const uint8_t* __restrict__ sim_q,
                                                             const uint8_t* __restrict__ sim_k,
                                                             const float* __restrict__ topk,
                                                             const float* __restrict__ cdfthr, uint8_t* __restrict__ mask,
                                                             int32_t* __restrict__ lut, int32_t* __restrict__ valid, int H,
                                                             int nq, int nk, int is_causal, int sink) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  double* s_e = reinterpret_cast<double*>(smem_raw);
  uint32_t* s_key = reinterpret_cast<uint32_t*>(s_e + nk);
  int* s_idx = reinterpret_cast<int*>(s_key + nk);
  float* s_q = reinterpret_cast<float*>(s_idx + nk);
  __shared__ int s_warp[kSelThreads / 32];
  __shared__ float s_fred[kSelThreads / 32];
  __shared__ double s_dred[kSelThreads / 32];
  __shared__ int s_hist[256];
  __shared__ int s_sel[3];   // threshold byte, count above, remaining

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qi = blockIdx.x, bh = blockIdx.y, h = bh % H;
  const int k_limit = is_causal ? min(nk, (qi + 1) * (kBlockQ / kBlockK)) : nk;   // causal: k < (q+1)*2

  if (tid < D) s_q[tid] = Elem<T>::to_float(pq[((size_t)bh * nq + qi) * D + tid]);
  __syncthreads();

  // ---- scores (kept as fp32 copies of the 16-bit values in the low half of s_e's storage)
  float* s_s = reinterpret_cast<float*>(s_idx);   // reuse idx storage for the scores
  const float scale = (D == 64) ? 0.125f : 0.08838834764831845f;   // float(D ** -0.5)
  const T* pkb = pk + (size_t)bh * nk * D;
  const uint8_t* simk = sim_k + (size_t)bh * nk;
  float lmax = -INFINITY;
  for (int j = tid; j < nk; j += kSelThreads) {
    float s = -INFINITY;
    if (j < k_limit && simk[j]) {
      float acc = 0.f;
      const Pack8<T>* row = reinterpret_cast<const Pack8<T>*>(pkb + (size_t)j * D);
#pragma unroll 4
      for (int c = 0; c < D / 8; c++) {
        Pack8<T> p = row[c];
#pragma unroll
        for (int i = 0; i < 8; i++) acc = __fmaf_rn(s_q[c * 8 + i], Elem<T>::to_float(p.v[i]), acc);
      }
      s = Elem<T>::to_float(Elem<T>::from_float(acc));
      s = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(s, scale)));
    }
    s_s[j] = s;
    lmax = fmaxf(lmax, s);
  }
  lmax = warp_max(lmax);
  if (lane == 0) s_fred[warp] = lmax;
  __syncthreads();
  float m = s_fred[0];
#pragma unroll
  for (int w = 1; w < kSelThreads / 32; w++) m = fmaxf(m, s_fred[w]);

  // ---- fp64 softmax
  double lsum = 0.0;
  for (int j = tid; j < nk; j += kSelThreads) {
    const float s = s_s[j];
    const double e = (s == -INFINITY) ? 0.0 : exp((double)s - (double)m);
    s_e[j] = e;
    lsum += e;
  }
  lsum = warp_sum(lsum);
  if (lane == 0) s_dred[warp] = lsum;
  __syncthreads();
  double Z = 0.0;
#pragma unroll
  for (int w = 0; w < kSelThreads / 32; w++) Z += s_dred[w];
  const bool empty_row = (m == -INFINITY);
  for (int j = tid; j < nk; j += kSelThreads) {
    uint32_t key = 0;
    if (!empty_row) key = key_bits<T>(Elem<T>::from_float((float)(s_e[j] / Z)));
    s_key[j] = key;
  }
  __syncthreads();

  // ---- how many to select (top-k mode: same count for every row of a head)
  int n_sel = (int)__fmul_rn(topk[h], (float)nk);
  n_sel = max(1, min(n_sel, nk));

  // ---- 16-bit radix select of the n_sel-th largest key (two 8-bit digits)
  int thr_key = 0, remaining = 0;
  {
    for (int i = tid; i < 256; i += kSelThreads) s_hist[i] = 0;
    __syncthreads();
    for (int j = tid; j < nk; j += kSelThreads) atomicAdd(&s_hist[s_key[j] >> 8], 1);
    __syncthreads();
    if (tid == 0) {
      int acc = 0, b = 255;
      for (; b > 0; b--) {
        if (acc + s_hist[b] >= n_sel) break;
        acc += s_hist[b];
      }
      s_sel[0] = b;
      s_sel[1] = acc;
    }
    __syncthreads();
    const int hb = s_sel[0];
    const int above_hi = s_sel[1];
    __syncthreads();
    for (int i = tid; i < 256; i += kSelThreads) s_hist[i] = 0;
    __syncthreads();
    for (int j = tid; j < nk; j += kSelThreads) {
      const uint32_t key = s_key[j];
      if ((int)(key >> 8) == hb) atomicAdd(&s_hist[key & 0xff], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int acc = above_hi, b = 255;
      for (; b > 0; b--) {
        if (acc + s_hist[b] >= n_sel) break;
        acc += s_hist[b];
      }
      s_sel[0] = (hb << 8) | b;
      s_sel[1] = acc;
      s_sel[2] = n_sel - acc;
    }
    __syncthreads();
    thr_key = s_sel[0];
    remaining = s_sel[2];
  }

  // ---- final map, in index order (ties -> lower index), and compaction into idx[]
  const bool row_forced = sim_q[(size_t)bh * nq + qi] == 0;
  uint8_t* mrow = mask ? mask + ((size_t)bh * nq + qi) * nk : nullptr;
  int eq_seen = 0, live_seen = 0;
  for (int j0 = 0; j0 < nk; j0 += kSelThreads) {
    const int j = j0 + tid;
    const bool in = j < nk;
    const uint32_t key = in ? s_key[j] : 0u;
    const bool is_eq = in && (int)key == thr_key;
    int eq_total;
    const int eq_rank = eq_seen + block_exclusive_count(is_eq, s_warp, eq_total);
    eq_seen += eq_total;
    bool live = false;
    if (in) {
      live = ((int)key > thr_key) || (is_eq && eq_rank < remaining) || row_forced || (simk[j] == 0);
      if (is_causal) live = live && (j < k_limit);
      if (sink && j == 0) live = true;
      if (mrow) mrow[j] = live ? 1 : 0;
    }
    int live_total;
    const int pos = live_seen + block_exclusive_count(live, s_warp, live_total);
    live_seen += live_total;
    if (live) s_idx[pos] = j;
  }
  __syncthreads();
  write_lut_row(s_idx, live_seen, nk, lut + ((size_t)bh * nq + qi) * nk, valid + (size_t)bh * nq + qi);
}

// One CTA per mask row: compaction of a user block mask into the LUT.
// dynamic smem: int idx[nk]
__global__ void __launch_bounds__(kSelThreads) mask_to_lut_kernel(const uint8_t* __restrict__ mask, int elem_size,
                                                                  int32_t* __restrict__ lut, int32_t* __restrict__ valid,
                                                                  int nk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int* s_idx = reinterpret_cast<int*>(smem_raw);
  __shared__ int s_warp[kSelThreads / 32];
  const size_t row = blockIdx.x;
  const uint8_t* mrow = mask + row * (size_t)nk * elem_size;
  int live_seen = 0;
  for (int j0 = 0; j0 < nk; j0 += kSelThreads) {
    const int j = j0 + threadIdx.x;
    bool live = false;
    if (j < nk) {
      const uint8_t* p = mrow + (size_t)j * elem_size;
      switch (elem_size) {
        case 1: live = *p != 0; break;
        case 2: live = *reinterpret_cast<const uint16_t*>(p) != 0; break;
        case 4: live = *reinterpret_cast<const uint32_t*>(p) != 0; break;
        default: live = *reinterpret_cast<const uint64_t*>(p) != 0; break;
      }
    }
    int tot;
    const int pos = live_seen + block_exclusive_count(live, s_warp, tot);
    live_seen += tot;
    if (live) s_idx[pos] = j;
  }
  __syncthreads();
  write_lut_row(s_idx, live_seen, nk, lut + row * (size_t)nk, valid + row);
}

template <typename T, int D>
static int launch_select(const void* pq, const void* pk, const uint8_t* sim_q, const uint8_t* sim_k, const float* topk,
                         const float* cdf, uint8_t* mask, int32_t* lut, int32_t* valid, int BH, int H, int nq, int nk,
                         int causal, int sink, cudaStream_t st) {
  const size_t smem = (size_t)nk * (sizeof(double) + sizeof(uint32_t) + sizeof(int)) + D * sizeof(float);
  if (smem > 200 * 1024) return SPARGE_ERR_TOO_LARGE;
  auto kern = select_kernel<T, D>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return SPARGE_ERR_CUDA;
  }
  kern<<<dim3(nq, BH), kSelThreads, smem, st>>>((const T*)pq, (const T*)pk, sim_q, sim_k, topk, cdf, mask, lut, valid, H,
                                                nq, nk, causal, sink);
  return launch_status();
}

}  // namespace sparge

extern "C" int sparge_select(const void* pq, const void* pk, const uint8_t* sim_q, const uint8_t* sim_k,
                             const float* topk, const float* cdfthreshd, uint8_t* mask, int32_t* lut, int32_t* valid,
                             int B, int H, int nq, int nk, int D, int dtype, int is_causal, int attention_sink,
                             sparge_stream_t stream) {
  using namespace sparge;
  if (!pq || !pk || !sim_q || !sim_k || !lut || !valid) return SPARGE_ERR_NULL;
  if ((topk == nullptr) == (cdfthreshd == nullptr)) return SPARGE_ERR_INVALID_ARG;
  if (cdfthreshd != nullptr) return SPARGE_ERR_UNSUPPORTED;   // cdf selection: not built yet
  if (B <= 0 || H <= 0 || nq <= 0 || nk <= 0 || (D != 64 && D != 128) || (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const int BH = B * H;
#define SPARGE_SEL(T, DD) \
  launch_select<T, DD>(pq, pk, sim_q, sim_k, topk, cdfthreshd, mask, lut, valid, BH, H, nq, nk, is_causal, attention_sink, st)
  if (dtype == SPARGE_F16) return D == 64 ? SPARGE_SEL(__half, 64) : SPARGE_SEL(__half, 128);
  return D == 64 ? SPARGE_SEL(__nv_bfloat16, 64) : SPARGE_SEL(__nv_bfloat16, 128);
#undef SPARGE_SEL
}

extern "C" int sparge_mask_to_lut(const void* mask, int elem_size, int32_t* lut, int32_t* valid, int B, int H, int nq,
                                  int nk, sparge_stream_t stream) {
  using namespace sparge;
  if (!mask || !lut || !valid) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || nq <= 0 || nk <= 0 || (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8))
    return SPARGE_ERR_INVALID_ARG;
  const size_t smem = (size_t)nk * sizeof(int);
  if (smem > 200 * 1024) return SPARGE_ERR_TOO_LARGE;
  const long long rows = (long long)B * H * nq;
  if (rows > 2147483647LL) return SPARGE_ERR_TOO_LARGE;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(mask_to_lut_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return SPARGE_ERR_CUDA;
  }
  mask_to_lut_kernel<<<(unsigned)rows, kSelThreads, smem, (cudaStream_t)stream>>>((const uint8_t*)mask, elem_size, lut,
                                                                                    valid, nk);
  return launch_status();
}
