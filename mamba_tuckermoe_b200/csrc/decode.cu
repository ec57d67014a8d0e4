// Decode-shaped path (T <= 64 tokens, bf16): three bandwidth-shaped kernels that stream the
// K-major prepared factors once with 128-bit loads and keep the few token rows in shared memory.
// The layer is memory/latency bound here (7.6 MB of factors against <= 64 token rows), so the
// tensor cores are not used; every warp owns one output column and all T tokens.
//
//   decode_inproj_kernel   h_raw[T, r3] = x @ U_in, scores[T, E] = x @ router_w^T   (model.py:75, 80)
//                          grid = column groups x K slices of 256; fp32 atomics combine the slices
//   decode_core_kernel     per CTA prologue: inner RMSNorm statistics, top-k / softmax / c
//                          (model.py:76-77, 81, 93); then z[t, s] = sum_a c'[t,a] * (hw[t] . core[a][:, s])
//                          with one warp per z column reading the r1 interleaved core rows (model.py:95-98)
//   decode_out_kernel      y[t, n] = z[t] . U_out[:, n] + bias (+ residual epilogue)      (model.py:101)
#include "common.cuh"
#include "kernels.h"
#include "routing.cuh"
#include "ptx.cuh"
#include "decode_common.cuh"
#include <cstdlib>

namespace tmoe {

namespace {

constexpr int kDecWarps = 8;
constexpr int kKSlice = 256;      // K elements per CTA in the in-projection (one 16-byte load per lane)
constexpr int kInprojColsPerWarp = 4;
constexpr int kOutWarps = 16;
constexpr int kOutKChunk = 1024;  // z columns staged per pass in the out-projection

// ------------------------------------------------------------------------------------------
template <int TMAX>
__global__ void __launch_bounds__(kDecWarps * 32)
decode_inproj_kernel(const bf16 *__restrict__ x, const bf16 *__restrict__ uin_t, const bf16 *__restrict__ wr, int T,
                     int d_in, int r3, int E, float *__restrict__ h_raw, float *__restrict__ scores) {
  __shared__ __align__(16) bf16 xs[TMAX][kKSlice];
  ptx::griddep_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int k0 = blockIdx.y * kKSlice;
  // stage the K slice of all token rows (zeros beyond T or d_in)
  for (int i = threadIdx.x; i < TMAX * (kKSlice / 8); i += blockDim.x) {
    const int t = i / (kKSlice / 8), kk = (i % (kKSlice / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < T && k0 + kk < d_in) v = __ldg(reinterpret_cast<const uint4 *>(x + (int64_t)t * d_in + k0 + kk));
    *reinterpret_cast<uint4 *>(&xs[t][kk]) = v;
  }
  __syncthreads();
  const int k = k0 + lane * 8;
#pragma unroll 1
  for (int ci = 0; ci < kInprojColsPerWarp; ++ci) {
    const int n = (blockIdx.x * kDecWarps + warp) * kInprojColsPerWarp + ci;
    if (n >= r3 + E) break;
    const bf16 *row = (n < r3) ? uin_t + (int64_t)n * d_in : wr + (int64_t)(n - r3) * d_in;
    float w8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (k < d_in) unpack8(__ldg(reinterpret_cast<const uint4 *>(row + k)), w8);
    float *dst = (n < r3) ? h_raw + n : scores + (n - r3);
    const int ld = (n < r3) ? r3 : E;
#pragma unroll
    for (int tb = 0; tb < TMAX; tb += 32) {
      constexpr int NB = TMAX < 32 ? TMAX : 32;
      float acc[NB];
#pragma unroll
      for (int t = 0; t < NB; ++t) {
        float x8[8];
        unpack8(*reinterpret_cast<const uint4 *>(&xs[tb + t][lane * 8]), x8);
        acc[t] = dot8(x8, w8);
      }
      warp_reduce_many<NB>(acc, lane);
      const int t = tb + (lane % NB);
      if (lane < NB && t < T) atomicAdd(dst + (int64_t)t * ld, acc[0]);
    }
  }
}

// In-projection for T <= 8: every warp owns one column of h / the scores and the whole contraction, so there is no
// split-K, no atomics and nothing to clear beforehand (one launch fewer per call than the split-K form).  The few token
// rows sit in shared memory; a lane's weight loads of one batch are all issued before the first is used.
template <int TMAX>
__global__ void __launch_bounds__(kDecWarps * 32)
decode_inproj_fullk_kernel(const bf16 *__restrict__ x, const bf16 *__restrict__ uin_t, const bf16 *__restrict__ wr, int T,
                           int d_in, int r3, int E, float *__restrict__ h_raw, float *__restrict__ scores) {
  extern __shared__ __align__(16) uint8_t dsm[];
  bf16 *xs = reinterpret_cast<bf16 *>(dsm);  // [TMAX][d_in]
  ptx::griddep_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * kDecWarps + warp;
  const bf16 *row = nullptr;
  if (n < r3 + E) {
    row = (n < r3) ? uin_t + (int64_t)n * d_in : wr + (int64_t)(n - r3) * d_in;
    warp_prefetch_l2(row, d_in * 2, lane);
  }
  ptx::griddep_wait();  // x may come from the kernel before this one
  for (int i = threadIdx.x; i < TMAX * (d_in / 8); i += blockDim.x) {
    const int t = i / (d_in / 8), kk = (i % (d_in / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < T) v = __ldg(reinterpret_cast<const uint4 *>(x + (int64_t)t * d_in + kk));
    *reinterpret_cast<uint4 *>(&xs[t * d_in + kk]) = v;
  }
  __syncthreads();
  if (!row) return;
  float acc[TMAX];
#pragma unroll
  for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
  constexpr int B = 6;  // weight loads in flight per lane
  for (int k0 = lane * 8; k0 < d_in; k0 += 256 * B) {
    uint4 wv[B];
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int k = k0 + b * 256;
      wv[b] = (k < d_in) ? __ldg(reinterpret_cast<const uint4 *>(row + k)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
      const int k = k0 + b * 256;
      if (k < d_in) {
        float w8[8];
        unpack8(wv[b], w8);
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
          float x8[8];
          unpack8(*reinterpret_cast<const uint4 *>(&xs[t * d_in + k]), x8);
          acc[t] += dot8(x8, w8);
        }
      }
    }
  }
  warp_reduce_many<TMAX>(acc, lane);
  const int t = lane % TMAX;
  if (lane < TMAX && t < T) {
    if (n < r3) h_raw[(int64_t)t * r3 + n] = acc[0];
    else scores[(int64_t)t * E + (n - r3)] = acc[0];
  }
}

// ------------------------------------------------------------------------------------------
template <int TMAX, int R1, int KMAX>
__global__ void __launch_bounds__(kDecWarps * 32)
decode_core_kernel(const float *__restrict__ h_raw, const float *__restrict__ scores, const float *__restrict__ normw,
                   const float *__restrict__ uexp, const bf16 *__restrict__ g_t, int T, int r3, int r2, int E, int top_k,
                   float eps, bf16 *__restrict__ z, int32_t *__restrict__ idx_out, float *__restrict__ gates_out,
                   float *__restrict__ c_out, RouterCfg rc, const bf16 *__restrict__ x, int d_in, int pre_norm,
                   float pre_norm_eps) {
  constexpr int N2 = 256 / R1;
  extern __shared__ __align__(16) uint8_t dsm[];
  bf16 *hw = reinterpret_cast<bf16 *>(dsm);                                  // [TMAX][r3]
  float *cs = reinterpret_cast<float *>(dsm + (size_t)TMAX * r3 * 2);       // [TMAX][R1]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  ptx::griddep_launch_dependents();
  {
    constexpr int AC_PF = R1 < 8 ? R1 : 8, SPLIT_PF = R1 / AC_PF;
    const int s_pf = blockIdx.x * (kDecWarps / SPLIT_PF) + warp / SPLIT_PF;  // this warp's core rows: AC pieces of r3 values
    if (s_pf < r2) {
      const int j_pf = s_pf / N2;
      const bf16 *rows_pf = g_t + ((int64_t)j_pf * 256 + (s_pf - j_pf * N2)) * r3;
      for (int a = 0; a < AC_PF; ++a) warp_prefetch_l2(rows_pf + (int64_t)((warp % SPLIT_PF) * AC_PF + a) * N2 * r3, r3 * 2, lane);
    }
  }
  ptx::griddep_wait();  // h_raw and scores come from the in-projection kernel

  // prologue (redundant per CTA, T is tiny): norm statistics, h*w -> bf16, routing, c' = c / rms
  for (int t = warp; t < TMAX; t += kDecWarps) {
    if (t < T) {
      // callers' pre-norm applied here: its weight is folded into the prepared U_in / router rows, so h_raw and the scores
      // only lack the row's 1/rms(x) (same arithmetic as the tensor-core kernel's in-kernel pre-norm)
      float inv_x = 1.f;
      if (pre_norm) {
        float sx = 0.f;
        for (int i = lane * 8; i < d_in; i += 256) {
          float x8[8];
          unpack8(__ldg(reinterpret_cast<const uint4 *>(x + (int64_t)t * d_in + i)), x8);
          sx += dot8(x8, x8);
        }
        sx = warp_sum(sx);
        inv_x = 1.f / sqrtf(sx / (float)d_in + pre_norm_eps);
      }
      float ss = 0.f;
      for (int i = lane; i < r3; i += 32) {
        const float v = h_raw[(int64_t)t * r3 + i];
        ss = fmaf(v, v, ss);
        hw[t * r3 + i] = __float2bfloat16_rn(v * normw[i]);
      }
      ss = warp_sum(ss);
      const float inv_rms = inv_x / sqrtf(inv_x * inv_x * ss / (float)r3 + eps);
      TopList<KMAX> sel;
      sel.init();
      warp_select_topk<bf16, KMAX>(scores + (int64_t)t * E, E, top_k, lane, sel, inv_x, &rc);
      const bool tap = (blockIdx.x == 0);
      const float z_all = rc.mode == 1 ? warp_softmax_denominator<bf16, float>(scores + (int64_t)t * E, E, lane, rc, sel.v[0], inv_x) : 1.f;
      emit_token<bf16, KMAX, float>(sel, top_k, E, R1, uexp, 0, lane, tap && idx_out ? idx_out + (int64_t)t * top_k : nullptr,
                                    tap && gates_out ? gates_out + (int64_t)t * top_k : nullptr, cs + t * R1, rc, z_all);
      __syncwarp();
      if (lane < R1) {
        const float cv = cs[t * R1 + lane];
        if (tap && c_out) c_out[(int64_t)t * R1 + lane] = cv;
        cs[t * R1 + lane] = cv * inv_rms;
      }
    } else {
      for (int i = lane; i < r3; i += 32) hw[t * r3 + i] = __float2bfloat16_rn(0.f);
      if (lane < R1) cs[t * R1 + lane] = 0.f;
    }
  }
  __syncthreads();

  // A z column needs r1 core rows of r3 values.  Up to 8 slices fit a warp's registers at a time; with more slices
  // (r1 = 16, 32) SPLIT warps share a column, each with its own 8 slices, and their partial sums meet in shared memory:
  // 2-4 x as many CTAs stream the core tensor (8.4 MB at r1 = 32) than with one warp per column.
  constexpr int AC = R1 < 8 ? R1 : 8;
  constexpr int SPLIT = R1 / AC;
  constexpr int CPB = kDecWarps / SPLIT;  // z columns per CTA
  __shared__ float part[kDecWarps][32];
  const int s = blockIdx.x * CPB + warp / SPLIT;  // z column of this warp
  const int a0 = (warp % SPLIT) * AC;             // first core slice of this warp
  const bool valid = s < r2;
  const int sc = valid ? s : 0;
  const int j = sc / N2, sl = sc - j * N2;
  const bf16 *rows = g_t + ((int64_t)j * 256 + sl) * r3;  // slice a is N2 rows further
#pragma unroll
  for (int tb = 0; tb < TMAX; tb += 32) {
    constexpr int NB = TMAX < 32 ? TMAX : 32;
    float acc[NB];
#pragma unroll
    for (int t = 0; t < NB; ++t) acc[t] = 0.f;
    if (valid) {
      for (int k = lane * 8; k < r3; k += 256) {
        float g8[AC][8];
#pragma unroll
        for (int a = 0; a < AC; ++a)
          unpack8(__ldg(reinterpret_cast<const uint4 *>(rows + (int64_t)(a0 + a) * N2 * r3 + k)), g8[a]);
#pragma unroll
        for (int t = 0; t < NB; ++t) {
          float h8[8];
          unpack8(*reinterpret_cast<const uint4 *>(&hw[(tb + t) * r3 + k]), h8);
#pragma unroll
          for (int a = 0; a < AC; ++a) acc[t] = fmaf(cs[(tb + t) * R1 + a0 + a], dot8(h8, g8[a]), acc[t]);
        }
      }
    }
    warp_reduce_many<NB>(acc, lane);
    const int t = tb + (lane % NB);
    if (SPLIT == 1) {
      if (valid && lane < NB && t < T) z[(int64_t)t * r2 + s] = __float2bfloat16_rn(acc[0]);
    } else {
      if (lane < NB) part[warp][lane] = acc[0];
      __syncthreads();
      if ((warp % SPLIT) == 0 && valid && lane < NB && t < T) {
        float v = 0.f;
#pragma unroll
        for (int q = 0; q < SPLIT; ++q) v += part[warp + q][lane];
        z[(int64_t)t * r2 + s] = __float2bfloat16_rn(v);
      }
      __syncthreads();
    }
  }
}

// ------------------------------------------------------------------------------------------
template <int TMAX>
__global__ void __launch_bounds__(kOutWarps * 32)
decode_out_kernel(const bf16 *__restrict__ z, const bf16 *__restrict__ uout_t, const float *__restrict__ bias,
                  const bf16 *__restrict__ residual, const bf16 *__restrict__ gamma, const bf16 *__restrict__ silu_gate,
                  int T, int r2, int d_out, bf16 *__restrict__ y) {
  extern __shared__ __align__(16) uint8_t dsm[];
  bf16 *zs = reinterpret_cast<bf16 *>(dsm);  // [TMAX][kc]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n = blockIdx.x * kOutWarps + warp;
  ptx::griddep_launch_dependents();
  if (n < d_out) warp_prefetch_l2(uout_t + (int64_t)n * r2, r2 * 2, lane);
  ptx::griddep_wait();  // z comes from the core kernel
  constexpr int NB = TMAX < 32 ? TMAX : 32;
  constexpr int NG = TMAX / NB;
  float acc[NG][NB];
#pragma unroll
  for (int g = 0; g < NG; ++g)
#pragma unroll
    for (int t = 0; t < NB; ++t) acc[g][t] = 0.f;
  for (int kc0 = 0; kc0 < r2; kc0 += kOutKChunk) {
    const int kc = min(kOutKChunk, r2 - kc0);
    __syncthreads();
    for (int i = threadIdx.x; i < TMAX * (kc / 8); i += blockDim.x) {
      const int t = i / (kc / 8), kk = (i % (kc / 8)) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t < T) v = __ldg(reinterpret_cast<const uint4 *>(z + (int64_t)t * r2 + kc0 + kk));
      *reinterpret_cast<uint4 *>(&zs[t * kc + kk]) = v;
    }
    __syncthreads();
    if (n < d_out) {
      for (int k = lane * 8; k < kc; k += 256) {
        float w8[8];
        unpack8(__ldg(reinterpret_cast<const uint4 *>(uout_t + (int64_t)n * r2 + kc0 + k)), w8);
#pragma unroll
        for (int g = 0; g < NG; ++g)
#pragma unroll
          for (int t = 0; t < NB; ++t) {
            float z8[8];
            unpack8(*reinterpret_cast<const uint4 *>(&zs[(g * NB + t) * kc + k]), z8);
            acc[g][t] += dot8(z8, w8);
          }
      }
    }
  }
  if (n >= d_out) return;
#pragma unroll
  for (int g = 0; g < NG; ++g) {
    warp_reduce_many<NB>(acc[g], lane);
    const int t = g * NB + (lane % NB);
    if (lane < NB && t < T) {
      float v = acc[g][0] + bias[n];
      if (silu_gate) {
        const float gg = __bfloat162float(silu_gate[(int64_t)t * d_out + n]);
        v *= gg / (1.f + expf(-gg));
      }
      if (residual) v = __bfloat162float(residual[(int64_t)t * d_out + n]) + __bfloat162float(gamma[n]) * v;
      y[(int64_t)t * d_out + n] = __float2bfloat16_rn(v);
    }
  }
}

template <int TMAX>
int launch_decode_t(const tmoe_layer_t &L, const void *x, const char *pb, const PreparedLayout &P, int T, float *h_raw,
                    float *scores, void *z, int32_t *idx_out, float *gates_out, float *c_out, const OutEpilogue &epi,
                    void *y, int pre_norm, float pre_norm_eps, cudaStream_t st) {
  const int ncols = L.r3 + L.n_experts;
  cudaError_t e = cudaSuccess;
  if (TMAX <= 8) {
    const size_t smem1 = (size_t)TMAX * L.d_in * 2;
    e = cudaFuncSetAttribute(decode_inproj_fullk_kernel<TMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (e == cudaSuccess)
      e = launch_pdl(decode_inproj_fullk_kernel<TMAX>, dim3((ncols + kDecWarps - 1) / kDecWarps), dim3(kDecWarps * 32), smem1, st,
                     (const bf16 *)x, (const bf16 *)(pb + P.uin_t), (const bf16 *)(pb + P.wr_b), T, L.d_in, L.r3,
                     L.n_experts, h_raw, scores);
    if (e != cudaSuccess) return TMOE_ERR_CUDA;
  } else {
    // h_raw and scores are adjacent in the workspace: one clear for the split-K atomics
    const size_t clear_bytes = (size_t)((char *)(scores + (size_t)T * L.n_experts) - (char *)h_raw);
    if (cudaMemsetAsync(h_raw, 0, clear_bytes, st) != cudaSuccess) return TMOE_ERR_CUDA;
    dim3 g1((ncols + kDecWarps * kInprojColsPerWarp - 1) / (kDecWarps * kInprojColsPerWarp), (L.d_in + kKSlice - 1) / kKSlice);
    decode_inproj_kernel<TMAX><<<g1, kDecWarps * 32, 0, st>>>((const bf16 *)x, (const bf16 *)(pb + P.uin_t),
                                                             (const bf16 *)(pb + P.wr_b), T, L.d_in, L.r3, L.n_experts,
                                                             h_raw, scores);
  }
  const size_t smem2 = (size_t)TMAX * L.r3 * 2 + (size_t)TMAX * L.r1 * 4;
  const int split = L.r1 > 8 ? L.r1 / 8 : 1;      // warps per z column in decode_core_kernel
  const int cpb = kDecWarps / split;
  const dim3 g2((L.r2 + cpb - 1) / cpb);
#define TMOE_DC(R, K)                                                                                              \
  do {                                                                                                             \
    e = cudaFuncSetAttribute(decode_core_kernel<TMAX, R, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2); \
    if (e == cudaSuccess)                                                                                          \
      e = launch_pdl(decode_core_kernel<TMAX, R, K>, g2, dim3(kDecWarps * 32), smem2, st,                           \
          h_raw, scores, (const float *)(pb + P.normw), (const float *)(pb + P.uexp), (const bf16 *)(pb + P.g_t), T, \
          L.r3, L.r2, L.n_experts, L.top_k, L.eps, (bf16 *)z, idx_out, gates_out, c_out, router_cfg(L),          \
          (const bf16 *)x, L.d_in, pre_norm, pre_norm_eps);                           \
  } while (0)
  const bool k2 = L.top_k <= 2, k8 = L.top_k <= 8;
  if (L.r1 == 2) { if (k2) TMOE_DC(2, 2); else if (k8) TMOE_DC(2, 8); else TMOE_DC(2, 16); }
  else if (L.r1 == 4) { if (k2) TMOE_DC(4, 2); else if (k8) TMOE_DC(4, 8); else TMOE_DC(4, 16); }
  else if (L.r1 == 8) { if (k2) TMOE_DC(8, 2); else if (k8) TMOE_DC(8, 8); else TMOE_DC(8, 16); }
  else if (L.r1 == 16) { if (k2) TMOE_DC(16, 2); else if (k8) TMOE_DC(16, 8); else TMOE_DC(16, 16); }
  else if (L.r1 == 32) { if (k2) TMOE_DC(32, 2); else if (k8) TMOE_DC(32, 8); else TMOE_DC(32, 16); }
  else return TMOE_ERR_UNSUPPORTED;
#undef TMOE_DC
  if (e != cudaSuccess) return TMOE_ERR_CUDA;
  const int kc = L.r2 < kOutKChunk ? L.r2 : kOutKChunk;
  const size_t smem3 = (size_t)TMAX * kc * 2;
  e = cudaFuncSetAttribute(decode_out_kernel<TMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);
  if (e != cudaSuccess) return TMOE_ERR_CUDA;
  e = launch_pdl(decode_out_kernel<TMAX>, dim3((L.d_out + kOutWarps - 1) / kOutWarps), dim3(kOutWarps * 32), smem3, st,
      (const bf16 *)z, (const bf16 *)(pb + P.uout_t), (const float *)(pb + P.bias), (const bf16 *)epi.residual,
      (const bf16 *)epi.layer_scale, (const bf16 *)epi.silu_gate, T, L.r2, L.d_out, (bf16 *)y);
  if (e != cudaSuccess) return TMOE_ERR_CUDA;
  count_launch(3);
  return launch_status();
}

}  // namespace

int launch_decode(const tmoe_layer_t &L, const void *x, const void *prepared, const PreparedLayout &P, int64_t T,
                  float *h_raw, float *scores, void *z, int32_t *idx_out, float *gates_out, float *c_out,
                  const OutEpilogue &epi, void *y, cudaStream_t st, int pre_norm, float pre_norm_eps) {
  const char *pb = reinterpret_cast<const char *>(prepared);
  if (T > 64) return TMOE_ERR_UNSUPPORTED;
  if (T <= 8)
    return launch_decode_t<8>(L, x, pb, P, (int)T, h_raw, scores, z, idx_out, gates_out, c_out, epi, y, pre_norm, pre_norm_eps, st);
  return launch_decode_t<64>(L, x, pb, P, (int)T, h_raw, scores, z, idx_out, gates_out, c_out, epi, y, pre_norm, pre_norm_eps, st);
}

}  // namespace tmoe
