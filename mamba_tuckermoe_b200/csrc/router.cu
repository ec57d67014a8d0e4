// Router kernels (subsystem 1): scores, top-k, softmax over the winners, coefficient vector.
//
// Reference semantics (pure_torch_mlx/model.py:75-77, 93): scores = x @ router_w^T stored in
// the parameter dtype, torch.topk on the raw scores (values descending), softmax over the k
// selected values; then every selected expert contributes gate_k * U_expert[idx_k] to the
// per-token coefficient vector c.  Equal scores are ordered lowest expert index first.
//
// Two kernels share that selection rule:
//   router_fused_kernel  -- one warp per token: 128-bit loads of the x row and of the router
//                           rows, warp-shuffle reductions, running top-k list in registers.
//                           HBM traffic is one read of x; the router rows come from L1/L2.
//   select_kernel        -- the same selection from precomputed fp32 scores [T, E]
//                           (used when T*E is large enough that the scores are better made
//                           by a tiled GEMM).
#include "common.cuh"
#include "kernels.h"

namespace tmoe {

template <int KMAX>
struct TopList {
  float v[KMAX];
  int i[KMAX];
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int j = 0; j < KMAX; ++j) { v[j] = -INFINITY; i[j] = 0x7fffffff; }
  }
  // Insert (val, e) keeping the list sorted by ranks_before(); entries beyond k are ignored.
  __device__ __forceinline__ void insert(float val, int e, int k) {
    float cv = val; int ci = e;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < k && ranks_before(cv, ci, v[j], i[j])) {
        float tv = v[j]; int ti = i[j];
        v[j] = cv; i[j] = ci; cv = tv; ci = ti;
      }
    }
  }
};

// Writes idx / gates / c for one token from a finished selection list (all lanes hold it).
template <typename T, int KMAX>
__device__ __forceinline__ void emit_token(const TopList<KMAX> &sel, int k, int E, int r1, const T *__restrict__ uexp,
                                           int64_t t, int lane, int32_t *__restrict__ idx,
                                           float *__restrict__ gates, float *__restrict__ c) {
  float gate[KMAX];
  {
    float m = sel.v[0], den = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) { gate[j] = (j < k) ? expf(sel.v[j] - m) : 0.f; den += gate[j]; }
    float inv = 1.f / den;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) gate[j] = round_to<T>(gate[j] * inv);
  }
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < k && lane == (j & 31)) {
      if (idx) idx[t * k + j] = sel.i[j];
      if (gates) gates[t * k + j] = gate[j];
    }
  }
  for (int a = lane; a < r1; a += 32) {
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      if (j < k) {
        int e = min(max(sel.i[j], 0), E - 1);
        acc = fmaf(gate[j], to_f32(uexp[(int64_t)e * r1 + a]), acc);
      }
    }
    c[t * r1 + a] = acc;
  }
}

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static __forceinline__ void load(const float *p, float (&o)[4]) {
    float4 v = __ldg(reinterpret_cast<const float4 *>(p));
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
};
template <> struct Vec16<bf16> {
  static constexpr int N = 8;
  __device__ static __forceinline__ void load(const bf16 *p, float (&o)[8]) {
    uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      o[2 * q] = __uint_as_float(w[q] << 16);
      o[2 * q + 1] = __uint_as_float(w[q] & 0xffff0000u);
    }
  }
};

constexpr int kRouterWarps = 8;

template <typename T, int KMAX, int EG>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_fused_kernel(const T *__restrict__ x, const T *__restrict__ wr, const T *__restrict__ uexp, int64_t Tn,
                    int d_in, int E, int k, int r1, int32_t *__restrict__ idx, float *__restrict__ gates,
                    float *__restrict__ c) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  constexpr int V = Vec16<T>::N;
  const T *xr = x + t * d_in;
  TopList<KMAX> sel;
  sel.init();
  for (int e0 = 0; e0 < E; e0 += EG) {
    float acc[EG];
#pragma unroll
    for (int g = 0; g < EG; ++g) acc[g] = 0.f;
    for (int i = lane * V; i < d_in; i += 32 * V) {
      float xv[V];
      Vec16<T>::load(xr + i, xv);
#pragma unroll
      for (int g = 0; g < EG; ++g) {
        if (e0 + g < E) {
          float wv[V];
          Vec16<T>::load(wr + (int64_t)(e0 + g) * d_in + i, wv);
#pragma unroll
          for (int q = 0; q < V; ++q) acc[g] = fmaf(xv[q], wv[q], acc[g]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < EG; ++g) {
      float s = warp_sum(acc[g]);
      if (e0 + g < E) sel.insert(round_to<T>(s), e0 + g, k);
    }
  }
  emit_token<T, KMAX>(sel, k, E, r1, uexp, t, lane, idx, gates, c);
}

template <typename T, int KMAX>
__global__ void __launch_bounds__(kRouterWarps * 32)
select_kernel(const float *__restrict__ scores, const T *__restrict__ uexp, int64_t Tn, int E, int k, int r1,
              int32_t *__restrict__ idx, float *__restrict__ gates, float *__restrict__ c) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const float *sr = scores + t * E;
  TopList<KMAX> sel;
  sel.init();
  float pv = INFINITY; int pi = -1;
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < k) {
      float bv = -INFINITY; int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        float v = round_to<T>(sr[e]);
        if (ranks_before(pv, pi, v, e) && ranks_before(v, e, bv, bi)) { bv = v; bi = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ranks_before(ov, oi, bv, bi)) { bv = ov; bi = oi; }
      }
      sel.v[j] = bv; sel.i[j] = bi; pv = bv; pi = bi;
    }
  }
  emit_token<T, KMAX>(sel, k, E, r1, uexp, t, lane, idx, gates, c);
}

template <typename T>
static int launch_router_fused_t(const tmoe_layer_t &L, const void *x, const void *wr, const void *uexp, int64_t T_,
                                 int32_t *idx, float *gates, float *c, cudaStream_t st) {
  dim3 grid((unsigned)((T_ + kRouterWarps - 1) / kRouterWarps)), block(kRouterWarps * 32);
#define TMOE_RF(KM) router_fused_kernel<T, KM, 8><<<grid, block, 0, st>>>((const T *)x, (const T *)wr, (const T *)uexp, \
                       T_, L.d_in, L.n_experts, L.top_k, L.r1, idx, gates, c)
  if (L.top_k <= 2) TMOE_RF(2);
  else if (L.top_k <= 8) TMOE_RF(8);
  else TMOE_RF(16);
#undef TMOE_RF
  count_launch();
  return launch_status();
}

int launch_router_fused(const tmoe_layer_t &L, const void *x, const void *wr, const void *uexp, int64_t T_,
                        int32_t *idx, float *gates, float *c, cudaStream_t st) {
  if (L.dtype == TMOE_F32) return launch_router_fused_t<float>(L, x, wr, uexp, T_, idx, gates, c, st);
  return launch_router_fused_t<bf16>(L, x, wr, uexp, T_, idx, gates, c, st);
}

template <typename T>
static int launch_select_t(const tmoe_layer_t &L, const float *scores, const void *uexp, int64_t T_, int32_t *idx,
                           float *gates, float *c, cudaStream_t st) {
  dim3 grid((unsigned)((T_ + kRouterWarps - 1) / kRouterWarps)), block(kRouterWarps * 32);
#define TMOE_SEL(KM) select_kernel<T, KM><<<grid, block, 0, st>>>(scores, (const T *)uexp, T_, L.n_experts, L.top_k, \
                       L.r1, idx, gates, c)
  if (L.top_k <= 2) TMOE_SEL(2);
  else if (L.top_k <= 8) TMOE_SEL(8);
  else TMOE_SEL(16);
#undef TMOE_SEL
  count_launch();
  return launch_status();
}

int launch_select(const tmoe_layer_t &L, const float *scores, const void *uexp, int64_t T_, int32_t *idx,
                  float *gates, float *c, cudaStream_t st) {
  if (L.dtype == TMOE_F32) return launch_select_t<float>(L, scores, uexp, T_, idx, gates, c, st);
  return launch_select_t<bf16>(L, scores, uexp, T_, idx, gates, c, st);
}

}  // namespace tmoe
