// Per-channel FP8 (e4m3) quantisation of V: v16 = fp16(v); amax over tokens per (b,h,d);
// v_scale = amax / 2.25; v8 = e4m3_rn_satfinite(v16 * (2.25 / amax)).
// The reference builds this file with --use_fast_math (setup.py:60), so both quotients are the approximate
// `div.approx.ftz.f32` (dividend times the hardware reciprocal of the divisor). The same instruction is used
// here: div.approx(amax, 2.25) for the scale (equal to amax * RN(1/2.25) on every value checked) and
// div.approx(2.25, amax) for the multiplier, which makes scales and FP8 bytes equal to the reference's on the same GPU.
// Replaces the fp16 cast at spas_sage_attn/core.py:115-117, TransposePadPermuteKernel
// (csrc/fused/fused.cu:26-77) and MeanScaleKernel (fused.cu:80-191).
// Output is token-major [B,H,N_pad,D] with zero rows beyond N: the tcgen05 PV MMA takes V as an
// MN-major B operand straight from that layout, so no transposed copy is made.
// An all-zero channel is emitted as zeros (the reference produces NaN there).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sparge {

constexpr int kVRowsPerCta = 256;
constexpr float kVScaleMax = 2.25f;   // spas_sage_attn/core.py:151

// a / b as fused.cu computes it under --use_fast_math
__device__ __forceinline__ float div_approx(float a, float b) {
  float q;
  asm("div.approx.ftz.f32 %0, %1, %2;" : "=f"(q) : "f"(a), "f"(b));
  return q;
}

__global__ void div_approx_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = div_approx(a[i], b[i]);
}

template <typename T>
__device__ __forceinline__ float to_f16_value(T v);
template <>
__device__ __forceinline__ float to_f16_value<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_f16_value<__nv_bfloat16>(__nv_bfloat16 v) {
  return __half2float(__float2half_rn(__bfloat162float(v)));
}

// grid (chunks, B*H), 256 threads. amax accumulates as the bit pattern of a non-negative float.
template <typename T, int D>
__global__ void __launch_bounds__(256) v_amax_kernel(const T* __restrict__ v, unsigned int* __restrict__ amax_bits, int N, int H,
                                                     long long sb, long long sh, long long sn) {
  constexpr int TPR = D / 8, RPP = 256 / TPR;
  __shared__ float red[RPP][D];
  const int tid = threadIdx.x, cg = tid % TPR, r0 = tid / TPR;
  const int bh = blockIdx.y;
  const int row_begin = blockIdx.x * kVRowsPerCta, row_end = min(N, row_begin + kVRowsPerCta);
  const T* base = v + (size_t)(bh / H) * sb + (size_t)(bh % H) * sh;
  float mx[8];
#pragma unroll
  for (int i = 0; i < 8; i++) mx[i] = 0.f;
#ifndef VQ_UNROLL
#define VQ_UNROLL 4
#endif
  int row = row_begin + r0;
  for (; row + (VQ_UNROLL - 1) * RPP < row_end; row += VQ_UNROLL * RPP) {   // several 128-bit loads in flight per thread
    Pack8<T> p[VQ_UNROLL];
#pragma unroll
    for (int u = 0; u < VQ_UNROLL; u++) p[u] = *reinterpret_cast<const Pack8<T>*>(base + (size_t)(row + u * RPP) * sn + cg * 8);
#pragma unroll
    for (int u = 0; u < VQ_UNROLL; u++)
#pragma unroll
      for (int i = 0; i < 8; i++) mx[i] = fmaxf(mx[i], fabsf(to_f16_value<T>(p[u].v[i])));
  }
  for (; row < row_end; row += RPP) {
    Pack8<T> p = *reinterpret_cast<const Pack8<T>*>(base + (size_t)row * sn + cg * 8);
#pragma unroll
    for (int i = 0; i < 8; i++) mx[i] = fmaxf(mx[i], fabsf(to_f16_value<T>(p.v[i])));
  }
#pragma unroll
  for (int i = 0; i < 8; i++) red[r0][cg * 8 + i] = mx[i];
  __syncthreads();
  if (tid < D) {
    float m = 0.f;
#pragma unroll 4
    for (int r = 0; r < RPP; r++) m = fmaxf(m, red[r][tid]);
    atomicMax(amax_bits + (size_t)bh * D + tid, __float_as_uint(m));
  }
}

// grid (ceil(N_pad / rows), B*H), 256 threads.
template <typename T, int D>
__global__ void __launch_bounds__(256) v_quant_kernel(const T* __restrict__ v, const float* __restrict__ amax,
                                                      uint8_t* __restrict__ v8, int N, int N_pad, int H,
                                                      long long sb, long long sh, long long sn) {
  constexpr int TPR = D / 8, RPP = 256 / TPR;
  const int tid = threadIdx.x, cg = tid % TPR, r0 = tid / TPR;
#ifndef VQ_REVERSE
#define VQ_REVERSE 1
#endif
  // The amax pass has just read V front to back; this pass walks it back to front, so that it starts with the
  // rows that are still in L2 (a tensor larger than the cache would be re-read from DRAM in full either way).
  const int bh = VQ_REVERSE ? gridDim.y - 1 - blockIdx.y : blockIdx.y;
  const int chunk = VQ_REVERSE ? gridDim.x - 1 - blockIdx.x : blockIdx.x;
  const int row_begin = chunk * kVRowsPerCta, row_end = min(N_pad, row_begin + kVRowsPerCta);
  float r[8];
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const float a = amax[(size_t)bh * D + cg * 8 + i];
    r[i] = a > 0.f ? div_approx(kVScaleMax, a) : 0.f;
  }
  const T* base = v + (size_t)(bh / H) * sb + (size_t)(bh % H) * sh;
  uint8_t* out = v8 + (size_t)bh * N_pad * D;
  auto quantise = [&](const Pack8<T>& p) {
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; i++) f[i] = __fmul_rn(to_f16_value<T>(p.v[i]), r[i]);
    return make_uint2(cvt_e4m3x4(f[0], f[1], f[2], f[3]), cvt_e4m3x4(f[4], f[5], f[6], f[7]));
  };
  int row = row_begin + r0;
  const int full_end = min(row_end, N);                  // rows below N hold data, the rest of the pad is zeros
  for (; row + (VQ_UNROLL - 1) * RPP < full_end; row += VQ_UNROLL * RPP) {
    Pack8<T> p[VQ_UNROLL];
#pragma unroll
    for (int u = 0; u < VQ_UNROLL; u++) p[u] = *reinterpret_cast<const Pack8<T>*>(base + (size_t)(row + u * RPP) * sn + cg * 8);
#pragma unroll
    for (int u = 0; u < VQ_UNROLL; u++) *reinterpret_cast<uint2*>(out + (size_t)(row + u * RPP) * D + cg * 8) = quantise(p[u]);
  }
  for (; row < row_end; row += RPP) {
    uint2 w = make_uint2(0u, 0u);
    if (row < N) w = quantise(*reinterpret_cast<const Pack8<T>*>(base + (size_t)row * sn + cg * 8));
    *reinterpret_cast<uint2*>(out + (size_t)row * D + cg * 8) = w;
  }
}

__global__ void v_scale_final_kernel(float* __restrict__ v_scale, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) v_scale[i] = div_approx(v_scale[i], kVScaleMax);
}

template <typename T, int D>
static int launch_quant_v(const void* v, uint8_t* v8, float* v_scale, int BH, int H, int N, long long sb, long long sh,
                          long long sn, cudaStream_t st) {
  const int N_pad = (N + 127) / 128 * 128;
  if (cudaMemsetAsync(v_scale, 0, (size_t)BH * D * sizeof(float), st) != cudaSuccess) return SPARGE_ERR_CUDA;
  v_amax_kernel<T, D><<<dim3((N + kVRowsPerCta - 1) / kVRowsPerCta, BH), 256, 0, st>>>((const T*)v, (unsigned int*)v_scale, N, H, sb, sh, sn);
  v_quant_kernel<T, D><<<dim3((N_pad + kVRowsPerCta - 1) / kVRowsPerCta, BH), 256, 0, st>>>((const T*)v, v_scale, v8, N, N_pad, H, sb, sh, sn);
  v_scale_final_kernel<<<(BH * D + 255) / 256, 256, 0, st>>>(v_scale, BH * D);
  return launch_status();
}

}  // namespace sparge

extern "C" int sparge_quant_v_strided(const void* v, uint8_t* v8, float* v_scale, int B, int H, int N, int D, int dtype,
                                      long long stride_b, long long stride_h, long long stride_n,
                                      sparge_stream_t stream) {
  using namespace sparge;
  if (!v || !v8 || !v_scale) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (dtype != SPARGE_F16 && dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  if (!strides_ok(v, stride_b, stride_h, stride_n)) return SPARGE_ERR_INVALID_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  const int BH = B * H;
#define SPARGE_QV(T, DD) launch_quant_v<T, DD>(v, v8, v_scale, BH, H, N, stride_b, stride_h, stride_n, st)
  if (dtype == SPARGE_F16) return D == 64 ? SPARGE_QV(__half, 64) : SPARGE_QV(__half, 128);
  return D == 64 ? SPARGE_QV(__nv_bfloat16, 64) : SPARGE_QV(__nv_bfloat16, 128);
#undef SPARGE_QV
}

extern "C" int sparge_div_approx(const float* a, const float* b, float* out, int n, sparge_stream_t stream) {
  if (!a || !b || !out) return SPARGE_ERR_NULL;
  if (n <= 0) return SPARGE_ERR_INVALID_ARG;
  sparge::div_approx_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(a, b, out, n);
  return sparge::launch_status();
}

extern "C" int sparge_quant_v(const void* v, uint8_t* v8, float* v_scale, int B, int H, int N, int D, int dtype,
                              sparge_stream_t stream) {
  return sparge_quant_v_strided(v, v8, v_scale, B, H, N, D, dtype, (long long)H * N * D, (long long)N * D, D, stream);
}
