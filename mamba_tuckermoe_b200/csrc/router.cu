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
#include "routing.cuh"

namespace tmoe {

constexpr int kRouterWarps = 8;

template <typename T, int KMAX, int EG>
__global__ void __launch_bounds__(kRouterWarps * 32)
router_fused_kernel(const T *__restrict__ x, const T *__restrict__ wr, const T *__restrict__ uexp, int64_t Tn,
                    int d_in, int E, int k, int r1, int32_t *__restrict__ idx, float *__restrict__ gates,
                    float *__restrict__ c, RouterCfg rc) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  constexpr int V = Vec16<T>::N;
  const T *xr = x + t * d_in;
  TopList<KMAX> sel;
  sel.init();
  float run_max = -INFINITY, run_sum = 0.f;  // online softmax over all experts' logits (mode 1)
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
      if (e0 + g < E) {
        const float sr = round_to<T>(s);
        sel.insert(rc.order_value(sr), e0 + g, k);
        if (rc.mode == 1) {
          const float l = rc.logit(sr);
          if (l > run_max) { run_sum = run_sum * expf(run_max - l) + 1.f; run_max = l; }
          else run_sum += expf(l - run_max);
        }
      }
    }
  }
  emit_token<T, KMAX>(sel, k, E, r1, uexp, t, lane, idx, gates, c, rc, run_sum);
}

// Selection from bf16 scores (the tensor-core path's separate router GEMM writes them), E <= 256 * NV.
// A lane loads its share of the row once with 16-byte loads and turns every score into a 32-bit key
// (order-preserving map of the bf16 bits << 16 | 0xFFFF - expert): unsigned order = "higher score first, equal scores ->
// lower expert index first", the rule of ranks_before().  Each of the k rounds is then a maximum over the lane's registers,
// one warp-wide integer maximum and the removal of the winner; the generic kernel below re-reads the row k times instead.
template <int KMAX, int NV>
__global__ void __launch_bounds__(kRouterWarps * 32)
select_bf16_keys_kernel(const bf16 *__restrict__ scores, int ld, const bf16 *__restrict__ uexp, int64_t Tn, int E, int k,
                        int r1, int32_t *__restrict__ idx, float *__restrict__ gates, float *__restrict__ c, RouterCfg rc) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const bf16 *sr = scores + t * ld;
  uint32_t key[NV * 8];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int e0 = i * 256 + lane * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (e0 < ld) v = __ldg(reinterpret_cast<const uint4 *>(sr + e0));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const int e = e0 + q;
      uint32_t b = (q & 1) ? (w[q >> 1] >> 16) : (w[q >> 1] & 0xffffu);
      if (rc.mode == 1) b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(rc.logit(__uint_as_float(b << 16))));
      b = (b == 0x8000u) ? 0u : b;                                   // -0 and +0 compare equal
      const uint32_t u = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
      key[i * 8 + q] = (e < E) ? ((u << 16) | (0xffffu - (uint32_t)e)) : 0u;
    }
  }
  TopList<KMAX> sel;
  sel.init();
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < k) {
      uint32_t m = 0u;
#pragma unroll
      for (int x = 0; x < NV * 8; ++x) m = max(m, key[x]);
      const uint32_t win = __reduce_max_sync(0xffffffffu, m);
#pragma unroll
      for (int x = 0; x < NV * 8; ++x) key[x] = (key[x] == win) ? 0u : key[x];
      const uint32_t u = win >> 16;
      const uint32_t b = (u & 0x8000u) ? (u & 0x7fffu) : (~u & 0xffffu);
      sel.v[j] = __uint_as_float(b << 16);
      sel.i[j] = (int)(0xffffu - (win & 0xffffu));
    }
  }
  float z_all = 1.f;
  if (rc.mode == 1) z_all = warp_softmax_denominator<bf16, bf16>(sr, E, lane, rc, sel.v[0]);
  emit_token<bf16, KMAX>(sel, k, E, r1, uexp, t, lane, idx, gates, c, rc, z_all);
}

template <typename T, int KMAX, typename TS>
__global__ void __launch_bounds__(kRouterWarps * 32)
select_kernel(const TS *__restrict__ scores, int ld, const T *__restrict__ uexp, int64_t Tn, int E, int k, int r1,
              int32_t *__restrict__ idx, float *__restrict__ gates, float *__restrict__ c, RouterCfg rc) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * kRouterWarps + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const TS *sr = scores + t * ld;
  TopList<KMAX> sel;
  sel.init();
  warp_select_topk<T, KMAX, TS>(sr, E, k, lane, sel, 1.f, &rc);
  const float z_all = rc.mode == 1 ? warp_softmax_denominator<T, TS>(sr, E, lane, rc, sel.v[0]) : 1.f;
  emit_token<T, KMAX>(sel, k, E, r1, uexp, t, lane, idx, gates, c, rc, z_all);
}

template <typename T>
static int launch_router_fused_t(const tmoe_layer_t &L, const void *x, const void *wr, const void *uexp, int64_t T_,
                                 int32_t *idx, float *gates, float *c, cudaStream_t st) {
  dim3 grid((unsigned)((T_ + kRouterWarps - 1) / kRouterWarps)), block(kRouterWarps * 32);
#define TMOE_RF(KM) router_fused_kernel<T, KM, 8><<<grid, block, 0, st>>>((const T *)x, (const T *)wr, (const T *)uexp, \
                       T_, L.d_in, L.n_experts, L.top_k, L.r1, idx, gates, c, router_cfg(L))
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
#define TMOE_SEL(KM) select_kernel<T, KM, float><<<grid, block, 0, st>>>(scores, L.n_experts, (const T *)uexp, T_, \
                       L.n_experts, L.top_k, L.r1, idx, gates, c, router_cfg(L))
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

int launch_select_bf16_scores(const tmoe_layer_t &L, const void *scores, int ld, const void *uexp, int64_t T_,
                              int32_t *idx, float *gates, float *c, cudaStream_t st) {
  dim3 grid((unsigned)((T_ + kRouterWarps - 1) / kRouterWarps)), block(kRouterWarps * 32);
  if (L.n_experts <= 1024 && (ld % 8) == 0 && !(reinterpret_cast<uintptr_t>(scores) & 15)) {
#define TMOE_SELK(KM, NV) select_bf16_keys_kernel<KM, NV><<<grid, block, 0, st>>>((const bf16 *)scores, ld, (const bf16 *)uexp, \
                       T_, L.n_experts, L.top_k, L.r1, idx, gates, c, router_cfg(L))
#define TMOE_SELK_E(KM) do { if (L.n_experts <= 256) TMOE_SELK(KM, 1); else if (L.n_experts <= 512) TMOE_SELK(KM, 2); else TMOE_SELK(KM, 4); } while (0)
    if (L.top_k <= 2) TMOE_SELK_E(2);
    else if (L.top_k <= 8) TMOE_SELK_E(8);
    else TMOE_SELK_E(16);
#undef TMOE_SELK_E
#undef TMOE_SELK
    count_launch();
    return launch_status();
  }
#define TMOE_SELB(KM) select_kernel<bf16, KM, bf16><<<grid, block, 0, st>>>((const bf16 *)scores, ld, (const bf16 *)uexp, \
                       T_, L.n_experts, L.top_k, L.r1, idx, gates, c, router_cfg(L))
  if (L.top_k <= 2) TMOE_SELB(2);
  else if (L.top_k <= 8) TMOE_SELB(8);
  else TMOE_SELB(16);
#undef TMOE_SELB
  count_launch();
  return launch_status();
}

}  // namespace tmoe
