// Peer buffers for the all-gather of y across the GPUs of one node: allocation with an inter-process handle, mapping
// of the other ranks' buffers, and the copy-engine push of a token block to every peer.  Host code only.
#include <cstring>

#include "common.cuh"

static_assert(sizeof(cudaIpcMemHandle_t) == TMOE_PEER_HANDLE_BYTES, "handle size is part of the ABI");

extern "C" {

int tmoe_peer_alloc(int64_t bytes, void **device_ptr, unsigned char *handle) {
  if (!device_ptr || !handle) return TMOE_ERR_NULL;
  if (bytes <= 0) return TMOE_ERR_SHAPE;
  const int64_t gran = 2 << 20;
  const size_t n = (size_t)((bytes + gran - 1) / gran * gran);
  void *p = nullptr;
  if (cudaMalloc(&p, n) != cudaSuccess) {
    cudaGetLastError();
    return TMOE_ERR_CUDA;
  }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return TMOE_ERR_CUDA;
  }
  std::memcpy(handle, &h, sizeof(h));
  *device_ptr = p;
  return TMOE_OK;
}

int tmoe_peer_open(const unsigned char *handle, void **device_ptr) {
  if (!device_ptr || !handle) return TMOE_ERR_NULL;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    cudaGetLastError();
    return TMOE_ERR_CUDA;
  }
  *device_ptr = p;
  return TMOE_OK;
}

int tmoe_peer_close(void *device_ptr) {
  if (!device_ptr) return TMOE_ERR_NULL;
  return tmoe::cuda_ok(cudaIpcCloseMemHandle(device_ptr));
}

int tmoe_peer_free(void *device_ptr) {
  if (!device_ptr) return TMOE_ERR_NULL;
  return tmoe::cuda_ok(cudaFree(device_ptr));
}

int tmoe_peer_push(void *const *dst, int32_t n_dst, const void *src, int64_t bytes, void *const *streams) {
  if (n_dst < 0 || bytes < 0) return TMOE_ERR_SHAPE;
  if (n_dst == 0 || bytes == 0) return TMOE_OK;
  if (!dst || !src || !streams) return TMOE_ERR_NULL;
  for (int i = 0; i < n_dst; ++i) {
    if (!dst[i]) return TMOE_ERR_NULL;
    if (cudaMemcpyAsync(dst[i], src, (size_t)bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)streams[i]) != cudaSuccess) {
      cudaGetLastError();
      return TMOE_ERR_CUDA;
    }
  }
  return TMOE_OK;
}

}  // extern "C"
