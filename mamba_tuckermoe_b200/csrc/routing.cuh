// Device-side pieces of the routing rule shared by the router, select and decode kernels:
// a sorted top-k list (higher score first, equal scores -> lower expert index first), the
// softmax over the k winners and the coefficient vector c = sum_k gate_k * U_expert[idx_k]
// (pure_torch_mlx/model.py:76-77, 93).
#pragma once

#include "common.cuh"

namespace tmoe {

// Gate rule parameters (tmoe_layer_t::router_mode / router_cap / router_temperature).
struct RouterCfg {
  int mode;        // 0: softmax over the k winners' raw scores; 1: capped / tempered softmax over all experts
  float cap;
  float inv_temp;
  int bf16;        // bf16 layer: the capped score and the logit are rounded to bf16, as the reference's bf16 tensors are
  // logit of one score: cap * tanh(score / cap) in fp32, stored in the layer dtype (sft_cot_bundle/scripts/model.py:32-40,
  // 320), then divided by the temperature in the layer dtype (model.py:324).  At logits of 10-20 a bf16 step is 0.06-0.12,
  // i.e. several per cent of a probability: the rounding points have to be the reference's.
  __device__ __forceinline__ float logit(float score) const {
    float c = cap * tanhf(score / cap);
    if (bf16) c = __bfloat162float(__float2bfloat16_rn(c));
    float l = c * inv_temp;
    if (bf16) l = __bfloat162float(__float2bfloat16_rn(l));
    return l;
  }
  // What the top-k orders by: the raw score, or (rule 1) the tempered capped logit, as the reference's torch.topk does
  // (model.py:327).  In bf16 the two orders differ: where the cap saturates, different scores become the same logit and
  // the lower expert index wins.
  __device__ __forceinline__ float order_value(float score) const { return mode == 1 ? logit(score) : score; }
};
inline RouterCfg router_cfg(const tmoe_layer_t &L) {
  RouterCfg rc;
  rc.mode = L.router_mode;
  rc.cap = L.router_cap > 0.f ? L.router_cap : 10.f;
  rc.inv_temp = 1.f / (L.router_temperature > 0.f ? L.router_temperature : 0.5f);
  rc.bf16 = L.dtype == TMOE_BF16 ? 1 : 0;
  return rc;
}

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
// T: storage type the gates are rounded to; TU: element type of the U_expert table.
// Gate weights of the k selected experts (sel_v sorted descending), rounded to the storage type T.
// mode 0: softmax over the k raw scores (sel_v).  mode 1: sel_v holds the selected LOGITS (RouterCfg::order_value);
// p_j = exp(l_j - l_0) / z_all and
// z_all = sum over ALL experts of exp(l_e - l_0); gate_j = p_j / (sum_j p_j + 1e-6).
template <typename T, int KMAX>
__device__ __forceinline__ void gates_of(const float (&sel_v)[KMAX], int k, const RouterCfg &rc, float z_all,
                                         float (&gate)[KMAX]) {
  if (rc.mode == 0) {
    const float m = sel_v[0];
    float den = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) { gate[j] = (j < k) ? expf(sel_v[j] - m) : 0.f; den += gate[j]; }
    const float inv = 1.f / den;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) gate[j] = round_to<T>(gate[j] * inv);
  } else {
    const float l0 = sel_v[0];
    float den = 0.f;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) { gate[j] = (j < k) ? expf(sel_v[j] - l0) / z_all : 0.f; den += gate[j]; }
    const float inv = 1.f / (den + 1e-6f);
#pragma unroll
    for (int j = 0; j < KMAX; ++j) gate[j] = round_to<T>(gate[j] * inv);
  }
}

template <typename T, int KMAX, typename TU = T>
__device__ __forceinline__ void emit_token(const TopList<KMAX> &sel, int k, int E, int r1, const TU *__restrict__ uexp,
                                           int64_t t, int lane, int32_t *__restrict__ idx,
                                           float *__restrict__ gates, float *__restrict__ c,
                                           const RouterCfg &rc = RouterCfg{0, 10.f, 2.f, 0}, float z_all = 1.f) {
  float gate[KMAX];
  gates_of<T, KMAX>(sel.v, k, rc, z_all, gate);
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


// Top-k of one token's scores [E] by k passes over the row (all lanes end with the same list).
// Scores are multiplied by `scale` (1/rms(x) when the callers' pre-norm is applied in-kernel) and rounded to the storage
// type T before they are compared; with `rc` they are compared as rc->order_value() of that (the list then holds those).
template <typename T, int KMAX, typename TS = float>
__device__ __forceinline__ void warp_select_topk(const TS *__restrict__ sr, int E, int k, int lane, TopList<KMAX> &sel,
                                                 float scale = 1.f, const RouterCfg *rc = nullptr) {
  float pv = INFINITY; int pi = -1;
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < k) {
      float bv = -INFINITY; int bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        float v = round_to<T>(to_f32(sr[e]) * scale);
        if (rc) v = rc->order_value(v);
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
}

// sum over all experts of exp(logit(score_e) - top logit) for one token's score row (mode 1 only)
template <typename T, typename TS>
__device__ __forceinline__ float warp_softmax_denominator(const TS *__restrict__ sr, int E, int lane, const RouterCfg &rc,
                                                          float top_logit, float scale = 1.f) {
  const float l0 = top_logit;
  float z = 0.f;
  for (int e = lane; e < E; e += 32) z += expf(rc.logit(round_to<T>(to_f32(sr[e]) * scale)) - l0);
  return warp_sum(z);
}

}  // namespace tmoe
