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
//   cdf    = the reference runs torch.cumsum on the sorted probabilities in the 16-bit type and takes
//            torch.searchsorted(cdf, cdfthreshd[h], right=True) (utils.py:398-403). On the device that
//            cumsum is ATen's chunked Sklansky scan (ATen/native/cuda/ScanUtils.cuh,
//            tensor_kernel_scan_innermost_dim: chunks of 2 * num_threads_x values, every combine rounded to
//            the 16-bit type, num_threads_x derived from the row count and row length), and its rounding
//            decides the count on long rows (a bf16 running sum stops growing once the terms fall below
//            half an ulp). The kernel runs the same scan in the same order and the same binary search with
//            the fp32 comparison torch uses, so n_sel equals the reference's wherever the 16-bit
//            probabilities themselves agree; clamped to [1, nk].
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

// ---- warp-per-row predictor --------------------------------------------------------------------
// One warp owns one (b, h, q-block) row; a CTA holds up to 4 consecutive rows of one head, so the
// pooled K rows it streams are shared through L1. Everything is warp-synchronous (shuffles and
// ballots), there is no block-wide barrier.
// dynamic smem: [32][D*2+16] byte staging tile of pooled K rows (shared by the CTA's rows), then per
// row: int idx[nk] (first the fp32 scores) | float q[D] | uint16 key[nk].  The fp64 exponentials are
// evaluated twice (once for the sum, once for the probabilities) instead of being stored: at long
// sequences shared memory per row, not arithmetic, limits how many rows an SM can hold.
constexpr int kSelRowsPerCta = 4;
__host__ __device__ inline int next_pow2(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}
// log2 of the x-extent of ATen's inner-dimension scan launch (get_log_num_threads_x_inner_scan, uint32 arithmetic)
__host__ __device__ inline int aten_scan_log_threads_x(uint32_t num_rows, uint32_t row_size) {
  uint32_t lx = 0, ly = 0;
  while ((1u << lx) < row_size) ++lx;
  while ((1u << ly) < num_rows) ++ly;
  const uint32_t diff = lx - ly;
  uint32_t v = (9u + diff) / 2u;
  v = v < 4u ? 4u : v;
  return (int)(v > 9u ? 9u : v);
}
// per-row shared memory: sort / index / score words [next_pow2(nk)] | q [D] floats | keys [nk] | cdf [cdf_len] 16-bit
__host__ __device__ inline size_t select_row_bytes(int nk, int D, int cdf_len) {
  return (((size_t)next_pow2(nk) * 4 + (size_t)D * 4 + (size_t)nk * 2 + (size_t)cdf_len * 2) + 15) / 16 * 16;
}

__device__ __forceinline__ int warp_sum_int(int x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <typename T, int D>
__global__ void __launch_bounds__(kSelRowsPerCta * 32)
select_kernel(const T* __restrict__ pq, const T* __restrict__ pk, const uint8_t* __restrict__ sim_q,
              const uint8_t* __restrict__ sim_k, const float* __restrict__ topk, const float* __restrict__ cdfthr,
              uint8_t* __restrict__ mask, int32_t* __restrict__ lut, int32_t* __restrict__ valid, int H, int nq, int nk,
              int is_causal, int sink, int rows_per_cta, int best_first, int scan_log_nx, int cdf_len) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qi = blockIdx.x * rows_per_cta + warp, bh = blockIdx.y, h = bh % H;
  const bool active = warp < rows_per_cta && qi < nq;       // inactive warps still help to stage K tiles
  constexpr int kTileRowBytes = D * (int)sizeof(T) + 16;   // 16-byte pad: conflict-free 128-bit reads, one row per lane
  unsigned char* s_tile = smem_raw;
  const size_t row_bytes = select_row_bytes(nk, D, cdf_len);
  const int P2 = next_pow2(nk);
  unsigned char* base = smem_raw + 32 * kTileRowBytes + (size_t)(active ? warp : 0) * row_bytes;
  int* s_idx = reinterpret_cast<int*>(base);
  float* s_s = reinterpret_cast<float*>(s_idx);            // scores share storage with the index list
  uint32_t* s_sort = reinterpret_cast<uint32_t*>(s_idx);   // ... and with the sort keys of the cdf mode
  float* s_q = reinterpret_cast<float*>(s_idx + P2);
  uint16_t* s_key = reinterpret_cast<uint16_t*>(s_q + D);
  uint16_t* s_cdf = s_key + nk;
  const int k_limit = is_causal ? min(nk, (qi + 1) * (kBlockQ / kBlockK)) : nk;   // causal: k < (q+1)*2

  if (active)
    for (int dd = lane; dd < D; dd += 32) s_q[dd] = Elem<T>::to_float(pq[((size_t)bh * nq + qi) * D + dd]);
  __syncwarp();

  // ---- scores: the CTA streams pooled K through shared memory in tiles of 32 rows (coalesced
  // 128-bit loads); lane l of every active warp then runs the fp32 FMA chain for key block j0 + l.
  const float scale = (D == 64) ? 0.125f : 0.08838834764831845f;   // float(D ** -0.5)
  const T* pkb = pk + (size_t)bh * nk * D;
  const uint8_t* simk = sim_k + (size_t)bh * nk;
  constexpr int kChunksPerRow = D * (int)sizeof(T) / 16;
  float m = -INFINITY;
  for (int j0 = 0; j0 < nk; j0 += 32) {
    __syncthreads();                                       // previous tile fully consumed
    for (int i = threadIdx.x; i < 32 * kChunksPerRow; i += blockDim.x) {
      const int r = i / kChunksPerRow, c = i % kChunksPerRow;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (j0 + r < nk) val = *reinterpret_cast<const uint4*>(pkb + (size_t)(j0 + r) * D + c * 8);
      *reinterpret_cast<uint4*>(s_tile + r * kTileRowBytes + c * 16) = val;
    }
    __syncthreads();
    const int j = j0 + lane;
    if (active && j < nk) {
      float sc = -INFINITY;
      if (j < k_limit && simk[j]) {
        float acc = 0.f;
        const unsigned char* row = s_tile + lane * kTileRowBytes;
#pragma unroll 4
        for (int c = 0; c < kChunksPerRow; c++) {
          const Pack8<T> p = *reinterpret_cast<const Pack8<T>*>(row + c * 16);
#pragma unroll
          for (int i = 0; i < 8; i++) acc = __fmaf_rn(s_q[c * 8 + i], Elem<T>::to_float(p.v[i]), acc);
        }
        sc = Elem<T>::to_float(Elem<T>::from_float(acc));
        sc = Elem<T>::to_float(Elem<T>::from_float(__fmul_rn(sc, scale)));
      }
      s_s[j] = sc;
      m = fmaxf(m, sc);
    }
  }
  if (!active) return;                                     // no block-wide barrier below this line
  m = warp_max(m);

  // ---- fp64 softmax -> 16-bit keys (p >= 0, so the bit pattern orders like the value)
  double Z = 0.0;
  for (int j = lane; j < nk; j += 32) {
    const float sc = s_s[j];
    Z += (sc == -INFINITY) ? 0.0 : exp((double)sc - (double)m);
  }
  Z = warp_sum(Z);
  const bool empty_row = (m == -INFINITY);
  for (int j = lane; j < nk; j += 32) {
    const float sc = s_s[j];
    const double e = (sc == -INFINITY) ? 0.0 : exp((double)sc - (double)m);
    s_key[j] = empty_row ? (uint16_t)0 : (uint16_t)key_bits<T>(Elem<T>::from_float((float)(e / Z)));
  }
  __syncwarp();

  // ---- how many blocks to select
  int n_sel;
  if (cdfthr == nullptr) {
    n_sel = (int)__fmul_rn(topk[h], (float)nk);            // top-k mode: same count for every row of a head
  } else {
    // cdf mode. Step 1: the stable descending order (ties -> lower block index) as an explicit sequence: a
    // bitonic sort of (probability bits << 16 | 0xFFFF - index) in shared memory by this warp.
    const float thr = cdfthr[h];
    for (int i = lane; i < P2; i += 32) s_sort[i] = (i < nk) ? (((uint32_t)s_key[i] << 16) | (uint32_t)(0xFFFF - i)) : 0u;
    __syncwarp();
    for (int kk = 2; kk <= P2; kk <<= 1) {
      for (int jj = kk >> 1; jj > 0; jj >>= 1) {
        for (int i = lane; i < P2; i += 32) {
          const int ixj = i ^ jj;
          if (ixj > i) {
            const uint32_t a = s_sort[i], b = s_sort[ixj];
            const bool first_larger = (i & kk) == 0;
            if (first_larger ? (a < b) : (a > b)) {
              s_sort[i] = b;
              s_sort[ixj] = a;
            }
          }
        }
        __syncwarp();
      }
    }
    // Step 2: ATen's cumsum of the sorted 16-bit values: chunks of W = 2 * nx values; the running total enters
    // the first value of a chunk; Sklansky combine steps, each sum rounded to the 16-bit type.
    const int nx = 1 << scan_log_nx, W = 2 * nx;
    auto add16 = [](uint16_t a, uint16_t b) -> uint16_t {
      return (uint16_t)key_bits<T>(Elem<T>::from_float(__fadd_rn(key_value<T>(a), key_value<T>(b))));
    };
    uint16_t total = 0;
    for (int c0 = 0; c0 < nk; c0 += W) {
      uint16_t* buf = s_cdf + c0;
      for (int i = lane; i < W; i += 32) buf[i] = (c0 + i < nk) ? (uint16_t)(s_sort[c0 + i] >> 16) : (uint16_t)0;
      __syncwarp();
      if (lane == 0) buf[0] = add16(buf[0], total);
      __syncwarp();
      for (int mm = 0; mm <= scan_log_nx; mm++) {
        const int sgm = 1 << mm;
        for (int t = lane; t < nx; t += 32) {
          const int a = ((t >> mm) << (mm + 1)) | sgm;
          const int ti = a + (t & (sgm - 1)), si = a - 1;
          buf[ti] = add16(buf[ti], buf[si]);
        }
        __syncwarp();
      }
      total = buf[W - 1];
      __syncwarp();
    }
    // Step 3: torch.searchsorted(..., right=True): upper-bound binary search, 16-bit cdf compared in fp32
    int lo_i = 0, hi_i = nk;
    while (lo_i < hi_i) {
      const int mid = lo_i + ((hi_i - lo_i) >> 1);
      if (!(key_value<T>(s_cdf[mid]) > thr)) lo_i = mid + 1; else hi_i = mid;
    }
    n_sel = lo_i;
    __syncwarp();
  }
  n_sel = max(1, min(n_sel, nk));

  // ---- n_sel-th largest key by bisection over the 16 key bits
  uint32_t thr_key = 0;
#pragma unroll 1
  for (int bit = 15; bit >= 0; bit--) {
    const uint32_t cand = thr_key | (1u << bit);
    int c = 0;
    for (int j = lane; j < nk; j += 32) c += (s_key[j] >= cand);
    c = warp_sum_int(c);
    if (c >= n_sel) thr_key = cand;
  }
  int above = 0;
  for (int j = lane; j < nk; j += 32) above += (s_key[j] > thr_key);
  above = warp_sum_int(above);
  const int remaining = n_sel - above;

  // ---- final map in index order (ties -> lower index) and compaction into idx[]
  const bool row_forced = sim_q[(size_t)bh * nq + qi] == 0;
  uint8_t* mrow = mask ? mask + ((size_t)bh * nq + qi) * nk : nullptr;
  int eq_seen = 0, live_seen = 0;
  __syncwarp();                                            // scores are dead from here on: idx[] may overwrite them
  for (int j0 = 0; j0 < nk; j0 += 32) {
    const int j = j0 + lane;
    const bool in = j < nk;
    const uint32_t key = in ? s_key[j] : 0u;
    const bool is_eq = in && key == thr_key;
    const unsigned eq_b = __ballot_sync(0xffffffffu, is_eq);
    const int eq_rank = eq_seen + __popc(eq_b & ((1u << lane) - 1u));
    eq_seen += __popc(eq_b);
    bool live = false;
    if (in) {
      live = (key > thr_key) || (is_eq && eq_rank < remaining) || row_forced || (simk[j] == 0);
      if (is_causal) live = live && (j < k_limit);
      if (sink && j == 0) live = true;
      if (mrow) mrow[j] = live ? 1 : 0;
    }
    const unsigned lv_b = __ballot_sync(0xffffffffu, live);
    if (live) s_idx[live_seen + __popc(lv_b & ((1u << lane) - 1u))] = j;
    live_seen += __popc(lv_b);
  }
  __syncwarp();
  int32_t* lrow = lut + ((size_t)bh * nq + qi) * nk;
  // Visiting order. Reference order: ascending block index. Best-first: the live block with the largest
  // pooled probability (lowest index on ties) is moved to the front and the rest stay ascending; the
  // deltas may then be negative. Attention is order-independent, but starting at the block that most
  // likely holds the row maxima makes later rescales of the running output rare.
  int rbest = 0;
  if (best_first && live_seen > 1) {
    uint32_t bk = 0;
    int bpos = 0x7fffffff;
    for (int r = lane; r < live_seen; r += 32) {
      const uint32_t key = s_key[s_idx[r]];
      if (key > bk || (key == bk && r < bpos)) { bk = key; bpos = r; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const uint32_t ok_ = __shfl_xor_sync(0xffffffffu, bk, o);
      const int op = __shfl_xor_sync(0xffffffffu, bpos, o);
      if (ok_ > bk || (ok_ == bk && op < bpos)) { bk = ok_; bpos = op; }
    }
    rbest = (bpos == 0x7fffffff) ? 0 : bpos;
  }
  const int jbest = (live_seen > 0) ? s_idx[rbest] : 0;
  for (int r = lane; r < nk; r += 32) {
    int vv = 0;
    if (r < live_seen) {
      // element at visiting position r: jbest first, then the ascending list without it
      const int cur = (r == 0) ? jbest : s_idx[r <= rbest ? r - 1 : r];
      const int prev = (r == 0) ? 0 : ((r == 1) ? jbest : s_idx[(r - 1) <= rbest ? r - 2 : r - 1]);
      vv = cur - prev;
    }
    lrow[r] = vv;
  }
  if (lane == 0) valid[(size_t)bh * nq + qi] = live_seen;
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
                         int causal, int sink, int best_first, cudaStream_t st) {
  // cdf mode reproduces torch.cumsum over the [B*H*nq, nk] matrix of sorted probabilities: the scan's chunking
  // depends on both extents
  const int scan_log_nx = aten_scan_log_threads_x((uint32_t)BH * (uint32_t)nq, (uint32_t)nk);
  const int scan_w = 2 << scan_log_nx;
  const int cdf_len = cdf ? (nk + scan_w - 1) / scan_w * scan_w : 0;
  const size_t row_bytes = select_row_bytes(nk, D, cdf_len);
  const size_t tile_bytes = 32 * (D * sizeof(T) + 16);
  const size_t budget = 200 * 1024 - tile_bytes;
  if (row_bytes > budget) return SPARGE_ERR_TOO_LARGE;
  const int rows = (int)min((size_t)kSelRowsPerCta, budget / row_bytes);
  const size_t smem = tile_bytes + rows * row_bytes;
  auto kern = select_kernel<T, D>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return SPARGE_ERR_CUDA;
  }
  kern<<<dim3((nq + rows - 1) / rows, BH), kSelRowsPerCta * 32, smem, st>>>(
      (const T*)pq, (const T*)pk, sim_q, sim_k, topk, cdf, mask, lut, valid, H, nq, nk, causal, sink, rows, best_first,
      scan_log_nx, cdf_len);
  return launch_status();
}

}  // namespace sparge

extern "C" int sparge_select(const void* pq, const void* pk, const uint8_t* sim_q, const uint8_t* sim_k,
                             const float* topk, const float* cdfthreshd, uint8_t* mask, int32_t* lut, int32_t* valid,
                             int B, int H, int nq, int nk, int D, int dtype, int is_causal, int attention_sink,
                             int lut_order, sparge_stream_t stream) {
  using namespace sparge;
  if (!pq || !pk || !sim_q || !sim_k || !lut || !valid) return SPARGE_ERR_NULL;
  if ((topk == nullptr) == (cdfthreshd == nullptr)) return SPARGE_ERR_INVALID_ARG;
  if (B <= 0 || H <= 0 || nq <= 0 || nk <= 0 || (D != 64 && D != 128) || (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  cudaStream_t st = (cudaStream_t)stream;
  const int BH = B * H;
#define SPARGE_SEL(T, DD) \
  launch_select<T, DD>(pq, pk, sim_q, sim_k, topk, cdfthreshd, mask, lut, valid, BH, H, nq, nk, is_causal, attention_sink, lut_order != 0, st)
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
