// Shared definitions for the sparse-attention kernels: status codes, 16-bit element helpers,
// block geometry.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/sparge_b200.h"

namespace sparge {

constexpr int kBlockQ = 128;   // query rows per sparsity block
constexpr int kBlockK = 64;    // key rows per sparsity block

template <typename T>
struct Elem;
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// 8 consecutive 16-bit elements moved as one 128-bit access.
template <typename T>
struct alignas(16) Pack8 {
  T v[8];
};

__device__ __forceinline__ double warp_sum(double x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// Strided [B,H,N,D] views (D contiguous) are read with 128-bit loads: base and strides must keep 16-byte alignment.
inline bool strides_ok(const void* base, long long sb, long long sh, long long sn) {
  return (reinterpret_cast<uintptr_t>(base) % 16 == 0) && sb >= 0 && sh >= 0 && sn > 0 && sb % 8 == 0 && sh % 8 == 0 &&
         sn % 8 == 0;
}

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? SPARGE_OK : SPARGE_ERR_CUDA;
}

}  // namespace sparge
