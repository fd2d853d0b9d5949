// Peer-memory plumbing for the sequence-parallel exchange: buffers that other ranks (one process per GPU)
// can read and write with copy-engine transfers over NVLink. The transfers are plain cudaMemcpyAsync
// calls, one per chunk: no SM is used and nothing is multicast.
// The reference has no counterpart: its multi-GPU runs go through xfuser / torch.distributed
// (inference_examples/wan_infer.py), outside its attention package.
#include <cstring>

#include "common.cuh"

extern "C" int sparge_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64) return SPARGE_ERR_NULL;
  if (bytes == 0) return SPARGE_ERR_INVALID_ARG;
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return SPARGE_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return SPARGE_ERR_CUDA;
  }
  static_assert(sizeof(h) == 64, "IPC handle size");
  std::memcpy(handle64, &h, 64);
  *ptr = p;
  return SPARGE_OK;
}

extern "C" int sparge_peer_free(void* ptr) {
  if (!ptr) return SPARGE_ERR_NULL;
  if (cudaFree(ptr) != cudaSuccess) {
    cudaGetLastError();
    return SPARGE_ERR_CUDA;
  }
  return SPARGE_OK;
}

extern "C" int sparge_peer_open(const unsigned char* handle64, void** ptr) {
  if (!handle64 || !ptr) return SPARGE_ERR_NULL;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return SPARGE_ERR_CUDA;
  }
  *ptr = p;
  return SPARGE_OK;
}

extern "C" int sparge_peer_close(void* ptr) {
  if (!ptr) return SPARGE_ERR_NULL;
  if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) {
    cudaGetLastError();
    return SPARGE_ERR_CUDA;
  }
  return SPARGE_OK;
}

extern "C" int sparge_copy_async(void* dst, const void* src, size_t bytes, sparge_stream_t stream) {
  if (!dst || !src) return SPARGE_ERR_NULL;
  if (bytes == 0) return SPARGE_OK;
  if (cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return SPARGE_ERR_CUDA;
  }
  return SPARGE_OK;
}

// `height` rows of `width` bytes, rows `spitch` / `dpitch` bytes apart: one transfer for the same token range of
// several adjacent heads.
extern "C" int sparge_copy2d_async(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, size_t height,
                                   sparge_stream_t stream) {
  if (!dst || !src) return SPARGE_ERR_NULL;
  if (width == 0 || height == 0) return SPARGE_OK;
  if (dpitch < width || spitch < width) return SPARGE_ERR_INVALID_ARG;
  if (cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, height, cudaMemcpyDefault, (cudaStream_t)stream) != cudaSuccess) {
    cudaGetLastError();
    return SPARGE_ERR_CUDA;
  }
  return SPARGE_OK;
}
