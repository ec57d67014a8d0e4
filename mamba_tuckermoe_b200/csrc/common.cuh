// Shared host/device helpers for the Tucker-MoE kernels (sm_100a).
#pragma once
#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tmoe_b200.h"

namespace tmoe {

using bf16 = __nv_bfloat16;

// ---- workspace status words (first 256 bytes of every workspace) -------------------------
// word 0: 0 or TMOE_ERR_DEVICE_WAIT; word 1: kernel id; word 2: barrier tag; word 3: block id.
constexpr int kStatusBytes = 256;
// hand-off words between the in/core kernel's helper CTAs and the out-projection: 8 per 128-token tile, after the status words
constexpr int kHandoffBytes = 128 * 8 * 4;
// counters of the fused decode kernel (one per CTA rank of a cluster), after the hand-off words; zero between calls
constexpr int kCounterBytes = 256;
// everything in front of the per-call buffers: must be zero when a workspace is first used
constexpr int kHeaderBytes = kStatusBytes + kHandoffBytes + kCounterBytes;

// Counts kernel launches made by this library (read through tmoe_launch_count()).
extern unsigned long long g_launch_count;
inline void count_launch(int n = 1) { __atomic_fetch_add(&g_launch_count, (unsigned long long)n, __ATOMIC_RELAXED); }

inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

inline int cuda_ok(cudaError_t e) { return e == cudaSuccess ? TMOE_OK : TMOE_ERR_CUDA; }

// Launch check that does not synchronise: picks up launch-configuration errors only.
inline int launch_status() { return cuda_ok(cudaGetLastError()); }

// ---- element access -----------------------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Round an fp32 value to the storage type and back (what the reference's typed tensors do).
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&p);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Order used for expert selection: higher score first, equal scores -> lower index first.
__device__ __forceinline__ bool ranks_before(float va, int ia, float vb, int ib) {
  return (va > vb) || (va == vb && ia < ib);
}

// Launch that may begin while the previous kernel of the stream drains (programmatic dependent launch); the kernel calls
// ptx::griddep_wait() before it reads what that kernel wrote.  TMOE_PDL=0 turns the attribute off.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
  static const bool off = []() { const char *e = getenv("TMOE_PDL"); return e && atoi(e) == 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = off ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
// The same for a kernel whose grid is cut into clusters of `cluster_x` CTAs (grid.x a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, unsigned cluster_x,
                                      Args &&...args) {
  static const bool off = []() { const char *e = getenv("TMOE_PDL"); return e && atoi(e) == 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute at[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    at[n].id = cudaLaunchAttributeClusterDimension;
    at[n].val.clusterDim.x = cluster_x; at[n].val.clusterDim.y = 1; at[n].val.clusterDim.z = 1;
    ++n;
  }
  if (!off) {
    at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = at; cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace tmoe
