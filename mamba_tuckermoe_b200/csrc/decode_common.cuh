// Device helpers shared by the decode-shaped kernels (decode.cu, decode_fused.cu): bf16 unpacking, an 8-wide dot
// product, an L2 prefetch of a byte range by one warp and the transposed warp reduction of several partial sums.
#pragma once
#include "common.cuh"

namespace tmoe {

__device__ __forceinline__ void unpack8(const uint4 &v, float (&o)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    o[2 * q] = __uint_as_float(w[q] << 16);
    o[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
  }
}
__device__ __forceinline__ float dot8(const float (&a)[8], const float (&b)[8]) {
  float s = 0.f;
#pragma unroll
  for (int q = 0; q < 8; ++q) s = fmaf(a[q], b[q], s);
  return s;
}

// One warp asks L2 for [p, p + bytes) (128-byte lines).  Used for weight rows before griddep_wait(): they do not depend on
// the previous kernel, so their trip from HBM overlaps that kernel's tail.
__device__ __forceinline__ void warp_prefetch_l2(const void *p, int bytes, int lane) {
  const char *c = reinterpret_cast<const char *>(p);
  for (int o = lane * 128; o < bytes; o += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(c + o));
}

// Sums N per-lane partial values over the warp.  On return v[0] of lane l holds the total of
// value index (l % N) (N = 8 or 32): N + ... shuffles instead of 5 per value.
template <int N>
__device__ __forceinline__ void warp_reduce_many(float (&v)[N], int lane) {
  int n = N;
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
    if (m >= N) {  // more lanes than values: plain butterfly on every value
#pragma unroll
      for (int i = 0; i < N; ++i) v[i] += __shfl_xor_sync(0xffffffffu, v[i], m);
    } else {       // halve the value set: lanes with bit m keep the upper half
      n >>= 1;
      const bool up = (lane & m) != 0;
#pragma unroll
      for (int i = 0; i < N / 2; ++i) {
        if (i < n) {
          const float keep = up ? v[i + n] : v[i];
          const float send = up ? v[i] : v[i + n];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, m);
        }
      }
    }
  }
}

}  // namespace tmoe
