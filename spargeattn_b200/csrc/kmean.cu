// Mean of K over the token axis, computed with fp64 accumulation so that the result does not
// depend on the reduction order, then rounded fp64 -> fp32 -> 16-bit.
// Replaces `k.mean(dim=-2, keepdim=True)` at spas_sage_attn/core.py:119-120.
#include <mutex>

#include "common.cuh"

namespace sparge {

constexpr int kMeanRowsPerCta = 512;

// Scratch of the allocation-free entry point: lives in the library image, one copy per GPU that
// loads the library, for the life of the process. In host code this name is only a handle; the
// device address is obtained with cudaGetSymbolAddress (once per device) and passed to the kernels.
constexpr size_t kStaticScratchDoubles = SPARGE_K_MEAN_STATIC_MAX_BYTES / sizeof(double);
static __device__ __align__(256) double g_kmean_static_scratch[kStaticScratchDoubles];

// grid (chunks, B*H), 256 threads. Each thread owns 8 channels of every (256 / (D/8))-th row.
template <typename T, int D>
__global__ void __launch_bounds__(256) kmean_partial_kernel(const T* __restrict__ k, double* __restrict__ part, int N, int H,
                                                            long long sb, long long sh, long long sn) {
  constexpr int TPR = D / 8;        // threads per row
  constexpr int RPP = 256 / TPR;    // rows per pass
  __shared__ double red[RPP][D];
  const int tid = threadIdx.x, cg = tid % TPR, r0 = tid / TPR;
  const int chunk = blockIdx.x, bh = blockIdx.y, chunks = gridDim.x;
  const int row_begin = chunk * kMeanRowsPerCta;
  const int row_end = min(N, row_begin + kMeanRowsPerCta);
  const T* base = k + (size_t)(bh / H) * sb + (size_t)(bh % H) * sh;
  double acc[8];
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i] = 0.0;
  // Eight 128-bit loads in flight per thread: with one load per trip the kernel waited on memory with half of its
  // issue slots idle (33.6 -> 27.5 us for a 100 MB tensor, 165 -> 137 us = 5.4 TB/s for an 890 MB one).
  constexpr int KMEAN_UNROLL = 8;
  int row = row_begin + r0;
  for (; row + (KMEAN_UNROLL - 1) * RPP < row_end; row += KMEAN_UNROLL * RPP) {
    Pack8<T> p[KMEAN_UNROLL];
#pragma unroll
    for (int u = 0; u < KMEAN_UNROLL; u++) p[u] = *reinterpret_cast<const Pack8<T>*>(base + (size_t)(row + u * RPP) * sn + cg * 8);
#pragma unroll
    for (int u = 0; u < KMEAN_UNROLL; u++)
#pragma unroll
      for (int i = 0; i < 8; i++) acc[i] += (double)Elem<T>::to_float(p[u].v[i]);
  }
  for (; row < row_end; row += RPP) {
    Pack8<T> p = *reinterpret_cast<const Pack8<T>*>(base + (size_t)row * sn + cg * 8);
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i] += (double)Elem<T>::to_float(p.v[i]);
  }
#pragma unroll
  for (int i = 0; i < 8; i++) red[r0][cg * 8 + i] = acc[i];
  __syncthreads();
  if (tid < D) {
    double s = 0.0;
#pragma unroll 4
    for (int r = 0; r < RPP; r++) s += red[r][tid];
    part[((size_t)bh * chunks + chunk) * D + tid] = s;
  }
}

// grid (B*H), D threads.
template <typename T, int D>
__global__ void kmean_final_kernel(const double* __restrict__ part, T* __restrict__ km, int N, int chunks) {
  const int bh = blockIdx.x, d = threadIdx.x;
  double s = 0.0;
  for (int c = 0; c < chunks; c++) s += part[((size_t)bh * chunks + c) * D + d];
  km[(size_t)bh * D + d] = Elem<T>::from_float((float)(s / (double)N));
}

template <typename T, int D>
static int launch_kmean(const void* k, void* km, void* scratch, int BH, int H, int N, long long sb, long long sh,
                        long long sn, cudaStream_t st) {
  const int chunks = (N + kMeanRowsPerCta - 1) / kMeanRowsPerCta;
  kmean_partial_kernel<T, D><<<dim3(chunks, BH), 256, 0, st>>>((const T*)k, (double*)scratch, N, H, sb, sh, sn);
  kmean_final_kernel<T, D><<<BH, D, 0, st>>>((const double*)scratch, (T*)km, N, chunks);
  return launch_status();
}

}  // namespace sparge

extern "C" size_t sparge_k_mean_scratch_bytes(int B, int H, int N, int D) {
  if (B <= 0 || H <= 0 || N <= 0 || D <= 0) return 0;
  const size_t chunks = ((size_t)N + sparge::kMeanRowsPerCta - 1) / sparge::kMeanRowsPerCta;
  return (size_t)B * H * chunks * D * sizeof(double);
}

extern "C" int sparge_k_mean_strided(const void* k, void* km, void* scratch, int B, int H, int N, int D, int dtype,
                                     long long stride_b, long long stride_h, long long stride_n,
                                     sparge_stream_t stream) {
  using namespace sparge;
  if (!k || !km || !scratch) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  if (!strides_ok(k, stride_b, stride_h, stride_n)) return SPARGE_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int BH = B * H;
#define SPARGE_KM(T, DD) launch_kmean<T, DD>(k, km, scratch, BH, H, N, stride_b, stride_h, stride_n, st)
  if (dtype == SPARGE_F16) return D == 64 ? SPARGE_KM(__half, 64) : SPARGE_KM(__half, 128);
  return D == 64 ? SPARGE_KM(__nv_bfloat16, 64) : SPARGE_KM(__nv_bfloat16, 128);
#undef SPARGE_KM
}

extern "C" int sparge_k_mean(const void* k, void* km, void* scratch, int B, int H, int N, int D, int dtype,
                             sparge_stream_t stream) {
  return sparge_k_mean_strided(k, km, scratch, B, H, N, D, dtype, (long long)H * N * D, (long long)N * D, D, stream);
}

extern "C" int sparge_k_mean_static(const void* k, void* km, int B, int H, int N, int D, int dtype,
                                    sparge_stream_t stream) {
  using namespace sparge;
  if (!k || !km) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if (sparge_k_mean_scratch_bytes(B, H, N, D) > (size_t)SPARGE_K_MEAN_STATIC_MAX_BYTES) return SPARGE_ERR_TOO_LARGE;

  // Per-device set-up on the first call: resolve the device address of the static array with the
  // calling thread's current device. Nothing is allocated here or later.
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static double* dev_ptr[kMaxDevices] = {};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return SPARGE_ERR_CUDA;
  double* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_kmean_static_scratch) != cudaSuccess || p == nullptr) return SPARGE_ERR_CUDA;
      dev_ptr[dev] = static_cast<double*>(p);
    }
    scratch = dev_ptr[dev];
  }
  // The partial sums fill every scratch element that the second kernel reads, so nothing needs
  // clearing between calls.
  return sparge_k_mean(k, km, scratch, B, H, N, D, dtype, stream);
}
