// tmoe_forward_static_scratch: the CUDA-core forward with its scratch in a fixed device array.
//
// Some hosts cannot give this library a workspace at call time: a serving process that hands all
// device memory to its own arena at start-up has nothing left to cudaMalloc from, and a
// latency-critical decode loop may not tolerate the implicit device-wide synchronisation that
// cudaMalloc / cudaFree perform.  For them the scratch of the CUDA-core path lives in the array
// below, which every GPU that loads the library carries until the process exits.
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace {

// 4 MiB.  What fits is whatever tmoe_workspace_bytes(layer, T, TMOE_PATH_SIMT) says fits: the CUDA-core layout keeps
// idx, gates, c, h [T, r3] and z [T, r2] in fp32, about 4 * (r3 + r2 + r1 + 2 * top_k) bytes per token -- roughly 800 tokens
// for (r3, r2) = (256, 1024) and 400 for (512, 2048).
static __device__ __align__(256) unsigned char g_static_scratch[TMOE_STATIC_SCRATCH_BYTES];

std::mutex g_setup_mutex;
void *g_scratch_addr[64] = {};  // device address of the array, per device ordinal; resolved once

// In host code `g_static_scratch` is only a handle; the address a kernel can use has to be asked for,
// with the right device current.
int scratch_address(void **out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TMOE_ERR_CUDA;
  if (dev < 0 || dev >= 64) return TMOE_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void *p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || !p) return TMOE_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return TMOE_OK;
}

}  // namespace

extern "C" int tmoe_forward_static_scratch(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *x,
                                           int64_t T, void *y, const tmoe_extras_t *extras, void *stream) {
  // size check first: tmoe_workspace_bytes validates the layer and the token count and touches no CUDA state
  const int64_t need = tmoe_workspace_bytes(layer, T, TMOE_PATH_SIMT);
  if (need < 0) return (int)need;
  if (need > (int64_t)TMOE_STATIC_SCRATCH_BYTES) return TMOE_ERR_WORKSPACE;
  // the same argument checks as tmoe_forward, before anything is enqueued (also for T == 0)
  if (!factors) return TMOE_ERR_NULL;
  const void *fp[7] = {factors->router_w, factors->U_in, factors->inner_norm_w, factors->U_expert, factors->core,
                       factors->U_out, factors->bias};
  for (const void *q : fp) {
    if (!q) return TMOE_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(q) & 15) return TMOE_ERR_ALIGN;
  }
  if (T == 0) return TMOE_OK;
  if (!x || !y) return TMOE_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) return TMOE_ERR_ALIGN;
  void *scratch = nullptr;
  int rc = scratch_address(&scratch);
  if (rc) return rc;
  // the array keeps whatever the previous call left; the status and hand-off words have to start at zero
  if (cudaMemsetAsync(scratch, 0, tmoe::kHeaderBytes, (cudaStream_t)stream) != cudaSuccess)
    return TMOE_ERR_CUDA;
  return tmoe_forward(layer, factors, nullptr, x, T, y, extras, scratch, (int64_t)TMOE_STATIC_SCRATCH_BYTES,
                      TMOE_PATH_SIMT, stream);
}
