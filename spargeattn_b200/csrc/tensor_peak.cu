// Measures what the 8-bit tensor pipe of this GPU sustains: the denominator of the attention kernel's
// roofline.  Every CTA keeps one 128 x 128-byte A tile and one N x 128-byte B tile resident in shared
// memory (128B-swizzled K-major layout, the layout the attention kernel's Q and K tiles use) and one
// thread issues back-to-back tcgen05.mma (M = 128, K = 32 per instruction) into two alternating TMEM
// accumulators; nothing else runs, so the time is the tensor pipe's.  kind 0 = kind::i8 (s8 x s8 -> s32),
// kind 1 = kind::f8f6f4 (e4m3 x e4m3 -> f32).  No counterpart in the reference (it ships no benchmark).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sparge {

template <int KIND>
__global__ void __launch_bounds__(32) tensor_peak_kernel(int n, int iters, int tmem_cols, int32_t* dev_status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + 128 * 128;
  __shared__ uint64_t bar;
  __shared__ uint32_t s_tmem_base;
  const int lane = threadIdx.x;
  // pseudo-random operand bytes (finite e4m3 patterns: exponent field never all ones)
  for (int i = lane; i < (128 + n) * 128 / 4; i += 32) {
    uint32_t x = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    x ^= x >> 15;
    x *= 2246822519u;
    x ^= x >> 13;
    reinterpret_cast<uint32_t*>(sA)[i] = x & 0x37373737u;
  }
  fence_proxy_async_smem();
  tmem_alloc(&s_tmem_base, (uint32_t)tmem_cols);
  tmem_relinquish();
  if (lane == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  tc_fence_before();
  __syncwarp();
  tc_fence_after();
  const uint32_t tbase = s_tmem_base;
  if (lane == 0) {
    const uint32_t idesc = KIND == 0 ? make_idesc(2, 1, 1, 0, 0, 128, (uint32_t)n) : make_idesc(1, 0, 0, 0, 0, 128, (uint32_t)n);
    const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
    for (int it = 0; it < iters; it++) {
      const uint32_t acc = tbase + (uint32_t)((it & 1) * n);
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        const uint64_t ad = make_smem_desc(a0 + ks * 32, 16, 1024, kSwizzle128B);
        const uint64_t bd = make_smem_desc(b0 + ks * 32, 16, 1024, kSwizzle128B);
        if (KIND == 0) mma_i8_ss(acc, ad, bd, idesc, (it > 1 || ks > 0) ? 1u : 0u);
        else mma_f8_ss(acc, ad, bd, idesc, (it > 1 || ks > 0) ? 1u : 0u);
      }
    }
    tc_commit(&bar);
    if (!mbar_wait(&bar, 0) && dev_status) atomicCAS(dev_status, 0, SPARGE_DEV_TIMEOUT_MMA);
  }
  tc_fence_before();
  __syncwarp();
  tmem_dealloc(tbase, (uint32_t)tmem_cols);
}

}  // namespace sparge

extern "C" int sparge_tensor_peak(int kind, int n, int ctas_per_sm, int iters, int32_t* dev_status, float* ms_out,
                                  double* ops_out, sparge_stream_t stream) {
  using namespace sparge;
  if (!ms_out || !ops_out) return SPARGE_ERR_NULL;
  if ((kind != 0 && kind != 1) || (n != 64 && n != 128 && n != 256) || (ctas_per_sm != 1 && ctas_per_sm != 2) || iters < 2 ||
      iters > (1 << 22))
    return SPARGE_ERR_INVALID_ARG;
  if (ctas_per_sm == 2 && n == 256) return SPARGE_ERR_INVALID_ARG;   // two accumulators of 256 columns fill TMEM
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return SPARGE_ERR_CUDA;
  const int tmem_cols = ctas_per_sm == 2 ? 256 : 512;
  // one CTA per SM: ask for more than half of the shared memory so that a second CTA cannot join
  const int smem = ctas_per_sm == 2 ? 1024 + (128 + n) * 128 : 120 * 1024;
  auto kern = kind == 0 ? tensor_peak_kernel<0> : tensor_peak_kernel<1>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return SPARGE_ERR_CUDA;
  cudaStream_t st = (cudaStream_t)stream;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return SPARGE_ERR_CUDA;
  const int grid = sms * ctas_per_sm;
  kern<<<grid, 32, smem, st>>>(n, iters / 8 + 2, tmem_cols, dev_status);   // warm-up
  cudaEventRecord(e0, st);
  kern<<<grid, 32, smem, st>>>(n, iters, tmem_cols, dev_status);
  cudaEventRecord(e1, st);
  int rc = launch_status();
  if (cudaEventSynchronize(e1) != cudaSuccess) rc = SPARGE_ERR_CUDA;
  float ms = 0.f;
  if (rc == SPARGE_OK && cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) rc = SPARGE_ERR_CUDA;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  *ms_out = ms;
  *ops_out = (double)grid * iters * 4.0 * 2.0 * 128.0 * n * 32.0;
  return rc;
}
