// The whole layer forward for T <= 8 bf16 tokens in ONE launch (decode: T = 1, 66 calls per generated token,
// pure_torch_mlx/model.py:378-397).  The layer is memory / latency bound here: 7.6 - 15 MB of factors against a handful of
// token rows, and three dependent contractions (model.py:75/80 -> 95-98 -> 101).  Three launches cost three device-wide
// dependencies; this kernel has none that anybody waits on.
//
// Thread-block clusters of `csize` CTAs (16 where the device allows, else 8), `nc` clusters, 16 warps per CTA.
//   stage 1  every cluster computes ALL of h_raw = x @ U_in and scores = x @ router_w^T (its CTAs split the r3 + E columns,
//            one warp per column, 128-bit loads of the K-major rows) and each result is stored into the shared memory of
//            every CTA of the cluster (distributed shared memory).  The in-projection is the smallest factor (0.8 of
//            7.6 MB at the decode configuration), so repeating it per cluster costs L2 reads, not HBM reads.
//   stage 2  every CTA redoes the tiny per-token work (inner RMSNorm statistics, top-k, gates, c: model.py:76-77, 81, 93);
//            cluster q owns the z columns [k0, k0 + kc) (r2 split into nc slices of whole 8-column units), its warps take
//            (column, group of <= 8 core slices) items and store z partials into every CTA of the cluster.
//   stage 3  CTA `rank` of every cluster owns the same d_out / csize output columns: a thread per column, the cluster's K
//            slice of U_out^T, partial y to global memory.  The CTA that finds itself the last of the nc CTAs of its rank
//            (one atomic counter per rank, no spinning) sums the nc partials in a fixed order, adds the bias, applies the
//            optional silu-gate / residual epilogue and writes y: run-to-run reproducible, nobody waits for anybody.
// Everything a CTA will read in stages 2 and 3 is requested from L2 at the very start (before the programmatic-launch
// wait), so the factors stream from HBM while the previous kernel drains and while stage 1 runs.
#include "common.cuh"
#include "decode_common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "routing.cuh"

#include <cstdio>
#include <mutex>

namespace tmoe {

namespace {

// Diagnostic builds (-DTMOE_TRACE): thread 0 of CTA 0 writes %globaltimer stamps (ns, low 32 bits) of the kernel's stages
// to the counter words' neighbours in the workspace (words 32.. of the counter block).
#ifdef TMOE_TRACE
#define TMOE_DSTAMP(i)                                                                          \
  do {                                                                                          \
    if (blockIdx.x == 0 && threadIdx.x == 0) {                                                  \
      unsigned long long t_;                                                                    \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                    \
      p.counters[32 + (i)] = (unsigned int)t_;                                                  \
      p.counters[48 + (i)] = (unsigned int)clock64();                                           \
    }                                                                                           \
  } while (0)
#else
#define TMOE_DSTAMP(i) do { } while (0)
#endif

constexpr int kFWarps = 16;
constexpr int kFThreads = kFWarps * 32;

struct FusedP {
  const bf16 *x, *uin_t, *wr, *g_t, *uout_t;
  const float *normw, *bias, *uexp;
  const bf16 *residual, *gamma, *silu_gate;
  bf16 *y;
  float *partial;        // [nc][T][d_out]
  unsigned int *counters;  // [csize], zero between calls
  int32_t *idx_out;
  float *gates_out, *c_out;
  int T, d_in, r3, r2, E, top_k, d_out;
  float eps;
  RouterCfg rc;
  int pre_norm;
  float pre_norm_eps;
  int nc, csize, kc_max;
  int uexp_smem;   // U_expert is small enough to be copied to shared memory ahead of the routing
};

// Shared-memory carve-up, the same in every CTA of the launch (remote stores address it through mapa).
struct FusedSmem { uint32_t xs, hs, hw, cs, zs, nw, ue, total; };
__host__ __device__ inline FusedSmem fused_smem(int tmax, int d_in, int hcols, int r3, int r1, int kc_max, int ue_rows) {
  const int ac = r1 < 8 ? r1 : 8, g = r1 / ac;
  auto up = [](uint32_t v) { return (v + 15u) & ~15u; };
  FusedSmem m;
  m.xs = 0;                                                 // bf16 [tmax][d_in]
  m.hs = up(m.xs + (uint32_t)tmax * d_in * 2);              // f32  [tmax][r3 + E]
  m.hw = up(m.hs + (uint32_t)tmax * hcols * 4);             // bf16 [tmax][r3]
  m.cs = up(m.hw + (uint32_t)tmax * r3 * 2);                // f32  [tmax][r1] then [tmax] 1/rms(x)
  m.zs = up(m.cs + (uint32_t)(tmax * r1 + tmax) * 4);       // f32  [g][tmax][kc_max]
  m.nw = up(m.zs + (uint32_t)g * tmax * kc_max * 4);        // f32  [r3] inner-norm weight
  m.ue = up(m.nw + (uint32_t)r3 * 4);                       // f32  [ue_rows][r1] U_expert (0 rows: read from global memory)
  m.total = up(m.ue + (uint32_t)ue_rows * r1 * 4);
  return m;
}

__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  ptx::cluster_arrive();
  ptx::cluster_wait();
}
__device__ __forceinline__ float ld_cg_f32(const float *p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// 16-byte read-only load that stays where it is written: a plain __ldg may be sunk by the compiler to its first use (the
// data is invariant, so no barrier holds it back), which is exactly what a load issued AHEAD of a barrier must not do.
__device__ __forceinline__ uint4 ldg_early(const void *ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
__device__ __forceinline__ void cp_async_4(uint32_t smem_addr, const void *g) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_addr), "l"(g) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Top-k of up to 32 * NK scores held one per lane and slot, as 32-bit keys (order-preserving map of the bf16 bits << 16 |
// 0xFFFF - expert: unsigned order = "higher score first, equal scores -> lower expert index first", the rule of
// ranks_before()): k rounds of register maximum + one warp-wide integer maximum + removal of the winner.
template <int KMAX, int NK>
__device__ __forceinline__ void warp_select_topk_keys(const float *sc, int E, int k, int lane, float scale, TopList<KMAX> &sel,
                                                      const RouterCfg &rc) {
  uint32_t key[NK];
#pragma unroll
  for (int i = 0; i < NK; ++i) {
    const int e = i * 32 + lane;
    uint32_t b = e < E ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(sc[e] * scale)) : 0u;
    if (rc.mode == 1) b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(rc.logit(__uint_as_float(b << 16))));
    b = (b == 0x8000u) ? 0u : b;                                   // -0 and +0 compare equal
    const uint32_t u = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
    key[i] = e < E ? ((u << 16) | (0xffffu - (uint32_t)e)) : 0u;
  }
#pragma unroll
  for (int j = 0; j < KMAX; ++j) {
    if (j < k) {
      uint32_t m = 0u;
#pragma unroll
      for (int i = 0; i < NK; ++i) m = max(m, key[i]);
      const uint32_t win = __reduce_max_sync(0xffffffffu, m);
#pragma unroll
      for (int i = 0; i < NK; ++i) key[i] = (key[i] == win) ? 0u : key[i];
      const uint32_t u = win >> 16;
      const uint32_t b = (u & 0x8000u) ? (u & 0x7fffu) : (~u & 0xffffu);
      sel.v[j] = __uint_as_float(b << 16);
      sel.i[j] = (int)(0xffffu - (win & 0xffffu));
    }
  }
}

// Latency is what this kernel is made of: a dozen dependent trips to L2 / HBM and three cluster barriers if written naively
// (measured: 12.7 us of in-kernel chain for one token).  So
//  (a) everything that does not depend on x is started BEFORE the programmatic-launch wait: the norm weight and U_expert go
//      to shared memory with cp.async, the bias and the first weight rows of stage 1 to registers, and every other row the
//      CTA will read is requested from L2;
//  (b) the first weight rows of stage 2 and of stage 3 are loaded into registers before the cluster barrier that precedes
//      their use (ldg_early: the compiler would otherwise sink them behind it);
//  (c) the first cluster barrier (every CTA of the cluster has started) is split: arrive on entry, wait just before the
//      first remote store, by when it has long completed;
//  (d) the per-token work between stages 1 and 2 is spread over the CTA's warps: all of them convert h, one warp per token
//      takes the norm statistics while another one routes, with integer warp reductions instead of shuffle ladders.
template <int TMAX, int R1, int KMAX>
__global__ void __launch_bounds__(kFThreads, 1) decode_fused_kernel(const FusedP p) {
  constexpr int N2 = 256 / R1;
  constexpr int AC = R1 < 8 ? R1 : 8;   // core slices a warp keeps in registers at a time
  constexpr int G = R1 / AC;            // groups of slices per z column
  constexpr int B1 = 6;                 // 16-byte weight loads in flight per lane and row in stage 1
  constexpr int NR1 = TMAX == 1 ? 2 : 1;  // rows of stage 1 a warp fetches ahead of x
  constexpr int B3 = 10;                // ... per thread in stage 3
  static_assert(2 * TMAX <= kFWarps, "one warp per token for the statistics and one for the routing");
  extern __shared__ __align__(16) uint8_t dsm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rank = (int)ptx::cluster_ctarank();
  const int q = (int)blockIdx.x / p.csize;       // cluster index
  const int gw = rank * kFWarps + warp;          // warp index inside the cluster
  const int cw = p.csize * kFWarps;              // warps per cluster
  const int hcols = p.r3 + p.E;

  TMOE_DSTAMP(0);
  ptx::cluster_arrive();                 // "this CTA is running" -- waited for just before the first remote store
  ptx::griddep_launch_dependents();

  const FusedSmem sm = fused_smem(TMAX, p.d_in, hcols, p.r3, R1, p.kc_max, p.uexp_smem ? p.E : 0);
  bf16 *xs = reinterpret_cast<bf16 *>(dsm + sm.xs);
  float *hs = reinterpret_cast<float *>(dsm + sm.hs);
  bf16 *hw = reinterpret_cast<bf16 *>(dsm + sm.hw);
  float *cs = reinterpret_cast<float *>(dsm + sm.cs);
  float *invx = cs + TMAX * R1;
  float *zs = reinterpret_cast<float *>(dsm + sm.zs);
  float *nw_s = reinterpret_cast<float *>(dsm + sm.nw);
  float *ue_s = reinterpret_cast<float *>(dsm + sm.ue);
  __shared__ int last_s;
  __shared__ float invr_s[TMAX];

  // this cluster's slice of r2, in whole 8-column units
  const int units = p.r2 >> 3;
  const int u0 = (int)((int64_t)q * units / p.nc), u1 = (int)((int64_t)(q + 1) * units / p.nc);
  const int k0 = u0 * 8, kc = (u1 - u0) * 8;
  // this CTA's output columns in stage 3 (the same range in every cluster)
  const int rows_per = ((p.d_out + p.csize - 1) / p.csize + 7) & ~7;
  const int n_begin = rank * rows_per, n_end = min(p.d_out, n_begin + rows_per);
  const int n_first = n_begin + (int)threadIdx.x;   // this thread's first output column

  // ================= before the wait: everything that does not depend on the previous kernel =================
  // first rows of stage 1 straight into registers
  uint4 w1[NR1][B1];
#pragma unroll
  for (int r = 0; r < NR1; ++r) {
    const int n = gw + r * cw;
    const bf16 *row = (n < p.r3) ? p.uin_t + (int64_t)n * p.d_in : p.wr + (int64_t)(n - p.r3) * p.d_in;
#pragma unroll
    for (int b = 0; b < B1; ++b) {
      const int k = lane * 8 + b * 256;
      w1[r][b] = (n < hcols && k < p.d_in) ? ldg_early(row + k) : make_uint4(0, 0, 0, 0);
    }
  }
  // norm weight and U_expert into shared memory, asynchronously (needed after stage 1)
  for (int i = threadIdx.x; i < p.r3; i += kFThreads) cp_async_4(ptx::smem_u32(nw_s + i), p.normw + i);
  if (p.uexp_smem)
    for (int i = threadIdx.x; i < p.E * R1; i += kFThreads) cp_async_4(ptx::smem_u32(ue_s + i), p.uexp + i);
  const float *uexp = p.uexp_smem ? ue_s : p.uexp;
  const float bias0 = n_first < n_end ? __ldg(p.bias + n_first) : 0.f;
  {
    // the rest of stage 1 (further rows of this warp, the tail of long rows), stage 2 and stage 3: ask L2 for them, one bulk
    // prefetch per contiguous piece (a per-line prefetch loop here was measured at 0.7 us of issue time per call)
    if (lane == 0) {
      for (int n = gw; n < hcols; n += cw) {
        const bf16 *row = (n < p.r3) ? p.uin_t + (int64_t)n * p.d_in : p.wr + (int64_t)(n - p.r3) * p.d_in;
        const int from = (n < gw + NR1 * cw) ? B1 * 256 : 0;   // elements of the row already on their way to registers
        if (from < p.d_in) ptx::l2_prefetch_bulk(row + from, (p.d_in - from) * 2);
      }
    }
    for (int it = gw; it < kc * G; it += cw) {
      const int s_loc = it / G, g = it - s_loc * G;
      const int s = k0 + s_loc;
      const int j = s / N2, sl = s - j * N2;
      const bf16 *rows = p.g_t + ((int64_t)j * 256 + sl) * p.r3 + (int64_t)(g * AC) * N2 * p.r3;
      if (lane < AC) ptx::l2_prefetch_bulk(rows + (int64_t)lane * N2 * p.r3, p.r3 * 2);
    }
    for (int n = n_first; n < n_end; n += kFThreads) ptx::l2_prefetch_bulk(p.uout_t + (int64_t)n * p.r2 + k0, kc * 2);
  }
  TMOE_DSTAMP(1);
  ptx::griddep_wait();  // x (and the partial / counter words of the workspace) may belong to the kernel before this one
  TMOE_DSTAMP(2);

  // ================= stage 0: token rows into shared memory =================
  for (int i = threadIdx.x; i < TMAX * (p.d_in / 8); i += kFThreads) {
    const int t = i / (p.d_in / 8), kk = (i - t * (p.d_in / 8)) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t < p.T) v = __ldg(reinterpret_cast<const uint4 *>(p.x + (int64_t)t * p.d_in + kk));
    *reinterpret_cast<uint4 *>(&xs[t * p.d_in + kk]) = v;
  }
  __syncthreads();
  ptx::cluster_wait();   // every CTA of the cluster is running: its shared memory may be written from now on
  TMOE_DSTAMP(3);
  if (warp < TMAX) {
    // callers' pre-norm applied in-kernel: its weight is folded into the prepared U_in / router rows, the row's 1/rms(x) is found here
    float inv = 1.f;
    if (p.pre_norm && warp < p.T) {
      float sx = 0.f;
      for (int i = lane * 8; i < p.d_in; i += 256) {
        float x8[8];
        unpack8(*reinterpret_cast<const uint4 *>(&xs[warp * p.d_in + i]), x8);
        sx += dot8(x8, x8);
      }
      sx = warp_sum(sx);
      inv = 1.f / sqrtf(sx / (float)p.d_in + p.pre_norm_eps);
    }
    if (lane == 0) invx[warp] = inv;
  }
  TMOE_DSTAMP(4);

  // ================= stage 1: h_raw and scores, one warp per column, results into every CTA of the cluster =================
  {
    const uint32_t hs_addr = ptx::smem_u32(hs);
    int ri = 0;
    for (int n = gw; n < hcols; n += cw, ++ri) {
      const bf16 *row = (n < p.r3) ? p.uin_t + (int64_t)n * p.d_in : p.wr + (int64_t)(n - p.r3) * p.d_in;
      float acc[TMAX];
#pragma unroll
      for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
      for (int kb = lane * 8; kb < p.d_in; kb += 256 * B1) {
        uint4 wv[B1];
        const bool pre = (kb == lane * 8) && (ri < NR1);   // this batch of this row was fetched ahead
#pragma unroll
        for (int b = 0; b < B1; ++b) {
          const int k = kb + b * 256;
          if (pre) wv[b] = (NR1 > 1 && ri == 1) ? w1[NR1 - 1][b] : w1[0][b];   // (NR1 <= 2)
          else wv[b] = (k < p.d_in) ? __ldg(reinterpret_cast<const uint4 *>(row + k)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int b = 0; b < B1; ++b) {
          const int k = kb + b * 256;
          if (k < p.d_in) {
            float w8[8];
            unpack8(wv[b], w8);
#pragma unroll
            for (int t = 0; t < TMAX; ++t) {
              float x8[8];
              unpack8(*reinterpret_cast<const uint4 *>(&xs[t * p.d_in + k]), x8);
              acc[t] += dot8(x8, w8);
            }
          }
        }
      }
      warp_reduce_many<TMAX>(acc, lane);
      {  // lane l holds the total of token l % TMAX: lanes share the csize destinations between them
        const uint32_t a = hs_addr + (uint32_t)(((lane % TMAX) * hcols + n) * 4);
        for (int r = lane / TMAX; r < p.csize; r += 32 / TMAX) st_cluster_f32(ptx::mapa_u32(a, (uint32_t)r), acc[0]);
      }
    }
  }
  TMOE_DSTAMP(5);
  // first item of stage 2 on its way before the barrier
  uint4 g2[AC];
  {
    const int it = gw;
    const bool has = it < kc * G && lane * 8 < p.r3;
    const int s_loc = has ? it / G : 0, g = has ? it - s_loc * G : 0;
    const int s = k0 + s_loc;
    const int j = s / N2, sl = s - j * N2;
    const bf16 *rows = p.g_t + ((int64_t)j * 256 + sl) * p.r3 + (int64_t)(g * AC) * N2 * p.r3;
#pragma unroll
    for (int a = 0; a < AC; ++a) g2[a] = has ? ldg_early(rows + (int64_t)a * N2 * p.r3 + lane * 8) : make_uint4(0, 0, 0, 0);
  }
  cp_async_wait_all();  // this thread's pieces of the norm weight / U_expert have landed; the barrier publishes them CTA-wide
  cluster_sync_all();   // h_raw / scores complete in every CTA (release / acquire at cluster scope)
  TMOE_DSTAMP(6);

  // ================= between the stages (every CTA, T is tiny): h*w -> bf16 by all warps; per token one warp takes the norm
  // statistics and another one routes (top-k, gates, c); then c' = c / rms =================
  for (int i = threadIdx.x; i < TMAX * p.r3; i += kFThreads) {
    const int t = i / p.r3, col = i - t * p.r3;
    hw[i] = __float2bfloat16_rn(hs[t * hcols + col] * nw_s[col]);   // rows beyond T are zero: x was zero-filled
  }
  if (warp < TMAX) {
    const int t = warp;
    float ss = 0.f;
    for (int i = lane; i < p.r3; i += 32) {
      const float v = hs[t * hcols + i];
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    const float inv_x = invx[t];
    if (lane == 0) invr_s[t] = inv_x / sqrtf(inv_x * inv_x * ss / (float)p.r3 + p.eps);
  } else if (warp >= kFWarps / 2 && warp < kFWarps / 2 + TMAX) {
    const int t = warp - kFWarps / 2;
    if (t < p.T) {
      const float inv_x = invx[t];
      const float *sc = hs + t * hcols + p.r3;
      TopList<KMAX> sel;
      sel.init();
      if (p.E <= 32) warp_select_topk_keys<KMAX, 1>(sc, p.E, p.top_k, lane, inv_x, sel, p.rc);
      else if (p.E <= 128) warp_select_topk_keys<KMAX, 4>(sc, p.E, p.top_k, lane, inv_x, sel, p.rc);
      else warp_select_topk<bf16, KMAX>(sc, p.E, p.top_k, lane, sel, inv_x, &p.rc);
      const bool tap = (blockIdx.x == 0);
      const float z_all = p.rc.mode == 1 ? warp_softmax_denominator<bf16, float>(sc, p.E, lane, p.rc, sel.v[0], inv_x) : 1.f;
      emit_token<bf16, KMAX, float>(sel, p.top_k, p.E, R1, uexp, 0, lane, tap && p.idx_out ? p.idx_out + (int64_t)t * p.top_k : nullptr,
                                    tap && p.gates_out ? p.gates_out + (int64_t)t * p.top_k : nullptr, cs + t * R1, p.rc, z_all);
      __syncwarp();
      if (tap && p.c_out && lane < R1) p.c_out[(int64_t)t * R1 + lane] = cs[t * R1 + lane];
    } else if (lane < R1) {
      cs[t * R1 + lane] = 0.f;
    }
  }
  __syncthreads();
  if (threadIdx.x < TMAX * R1) cs[threadIdx.x] *= invr_s[threadIdx.x / R1];
  __syncthreads();
  TMOE_DSTAMP(7);

  // ================= stage 2: z columns of this cluster's slice; item = (column, group of AC core slices) =================
  {
    const uint32_t zs_addr = ptx::smem_u32(zs);
    for (int it = gw; it < kc * G; it += cw) {
      const int s_loc = it / G, g = it - s_loc * G;
      const int s = k0 + s_loc;
      const int j = s / N2, sl = s - j * N2;
      const bf16 *rows = p.g_t + ((int64_t)j * 256 + sl) * p.r3 + (int64_t)(g * AC) * N2 * p.r3;   // slice a is N2 rows further
      float acc[TMAX];
#pragma unroll
      for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
      for (int k = lane * 8; k < p.r3; k += 256) {
        uint4 gv[AC];
        const bool pre = (it == gw) && (k == lane * 8);
#pragma unroll
        for (int a = 0; a < AC; ++a) gv[a] = pre ? g2[a] : __ldg(reinterpret_cast<const uint4 *>(rows + (int64_t)a * N2 * p.r3 + k));
#pragma unroll
        for (int t = 0; t < TMAX; ++t) {
          float h8[8];
          unpack8(*reinterpret_cast<const uint4 *>(&hw[t * p.r3 + k]), h8);
#pragma unroll
          for (int a = 0; a < AC; ++a) {
            float g8[8];
            unpack8(gv[a], g8);
            acc[t] = fmaf(cs[t * R1 + g * AC + a], dot8(h8, g8), acc[t]);
          }
        }
      }
      warp_reduce_many<TMAX>(acc, lane);
      {
        const uint32_t a = zs_addr + (uint32_t)(((g * TMAX + (lane % TMAX)) * p.kc_max + s_loc) * 4);
        for (int r = lane / TMAX; r < p.csize; r += 32 / TMAX) st_cluster_f32(ptx::mapa_u32(a, (uint32_t)r), acc[0]);
      }
    }
  }
  TMOE_DSTAMP(8);
  // stage 3 works on (output column, part) items: with few columns per CTA two threads share a column's K slice (its
  // 16-byte chunks alternate between them), so that a thread's whole share fits one batch of loads.  The first item's
  // chunks are on their way before the barrier.
  const int rows_cta = max(n_end - n_begin, 0);
  const int tpr = (rows_cta * 2 <= kFThreads) ? 2 : 1;         // threads per output column
  const int part = (int)threadIdx.x & (tpr - 1);
  const int n3_first = n_begin + ((int)threadIdx.x >> (tpr - 1));
  const int nch = kc >> 3;                                     // 16-byte chunks in this cluster's K slice
  uint4 w3[B3];
  {
    const bf16 *row = p.uout_t + (int64_t)(n3_first < n_end ? n3_first : 0) * p.r2 + k0;
#pragma unroll
    for (int b = 0; b < B3; ++b) {
      const int c = part + b * tpr;
      w3[b] = (n3_first < n_end && c < nch) ? ldg_early(row + c * 8) : make_uint4(0, 0, 0, 0);
    }
  }
  cluster_sync_all();   // last access to another CTA's shared memory is behind this barrier
  if (G > 1) {          // groups summed in a fixed order
    for (int i = threadIdx.x; i < TMAX * kc; i += kFThreads) {
      const int t = i / kc, s_loc = i - t * kc;
      float v = 0.f;
#pragma unroll
      for (int g = 0; g < G; ++g) v += zs[(g * TMAX + t) * p.kc_max + s_loc];
      zs[t * p.kc_max + s_loc] = v;   // group 0's block becomes z (g = 0 reads index t * kc_max + s_loc itself)
    }
    __syncthreads();
  }
  TMOE_DSTAMP(9);

  // ================= stage 3: partial y over this cluster's K slice =================
  for (int n = n3_first; n - ((int)threadIdx.x >> (tpr - 1)) < n_begin + rows_cta; n += kFThreads >> (tpr - 1)) {
    // (the loop bound is the same for all threads of a warp: the shuffle below needs every lane)
    const bool valid = n < n_end;
    const bf16 *row = p.uout_t + (int64_t)(valid ? n : 0) * p.r2 + k0;
    float acc[TMAX];
#pragma unroll
    for (int t = 0; t < TMAX; ++t) acc[t] = 0.f;
    for (int c0 = part; c0 < nch; c0 += B3 * tpr) {
      uint4 wv[B3];
      const bool pre = (n == n3_first) && (c0 == part);
#pragma unroll
      for (int b = 0; b < B3; ++b) {
        const int c = c0 + b * tpr;
        wv[b] = pre ? w3[b] : ((valid && c < nch) ? __ldg(reinterpret_cast<const uint4 *>(row + c * 8)) : make_uint4(0, 0, 0, 0));
      }
#pragma unroll
      for (int b = 0; b < B3; ++b) {
        const int c = c0 + b * tpr;
        if (valid && c < nch) {
          float w8[8];
          unpack8(wv[b], w8);
#pragma unroll
          for (int t = 0; t < TMAX; ++t) {
            const float4 za = *reinterpret_cast<const float4 *>(&zs[t * p.kc_max + c * 8]);
            const float4 zb = *reinterpret_cast<const float4 *>(&zs[t * p.kc_max + c * 8 + 4]);
            const float z8[8] = {za.x, za.y, za.z, za.w, zb.x, zb.y, zb.z, zb.w};
            acc[t] += dot8(z8, w8);
          }
        }
      }
    }
    if (tpr == 2) {
#pragma unroll
      for (int t = 0; t < TMAX; ++t) acc[t] += __shfl_xor_sync(0xffffffffu, acc[t], 1);
    }
    if (valid && part == 0) {
#pragma unroll
      for (int t = 0; t < TMAX; ++t)
        if (t < p.T) p.partial[((int64_t)q * p.T + t) * p.d_out + n] = acc[t];
    }
  }
  TMOE_DSTAMP(10);

  // ================= the last of the nc CTAs of this rank adds the partials up =================
  __syncthreads();   // the CTA's partial sums are written ...
  if (threadIdx.x == 0) {
    // ... and this one release / acquire increment publishes them (cumulativity: what the barrier made visible to this
    // thread is released with it) and, for the CTA that finds itself last, acquires everybody else's
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + rank) : "memory");
    const int last = (old == (unsigned int)(p.nc - 1));
    if (last) p.counters[rank] = 0u;   // ready for the next call; nobody else touches it any more
    last_s = last;
  }
  __syncthreads();
  TMOE_DSTAMP(11);
  if (!last_s) return;
  for (int n = n_first; n < n_end; n += kFThreads) {
    const float b = (n == n_first) ? bias0 : p.bias[n];
    const float gam = p.residual ? __bfloat162float(p.gamma[n]) : 0.f;
#pragma unroll
    for (int t = 0; t < TMAX; ++t) {
      if (t < p.T) {
        float v = 0.f;
        for (int c = 0; c < p.nc; ++c) v += ld_cg_f32(p.partial + ((int64_t)c * p.T + t) * p.d_out + n);
        v += b;
        if (p.silu_gate) {
          const float gg = __bfloat162float(p.silu_gate[(int64_t)t * p.d_out + n]);
          v *= gg / (1.f + expf(-gg));
        }
        if (p.residual) v = __bfloat162float(p.residual[(int64_t)t * p.d_out + n]) + gam * v;
        p.y[(int64_t)t * p.d_out + n] = __float2bfloat16_rn(v);
      }
    }
  }
  TMOE_DSTAMP(12);
}

constexpr int kUexpSmemFloats = 4096;   // U_expert tables up to 16 KB are copied to shared memory
size_t fused_smem_bytes(int tmax, const tmoe_layer_t &L, int kc_max) {
  const int ue_rows = L.n_experts * L.r1 <= kUexpSmemFloats ? L.n_experts : 0;
  return fused_smem(tmax, L.d_in, L.r3 + L.n_experts, L.r3, L.r1, kc_max, ue_rows).total;
}

// Cluster size and count a kernel instantiation gets on a device: 16-CTA clusters where they can be scheduled (non-portable
// size, fewer repetitions of stage 1), else 8; as many clusters as are co-resident (they do not need to be -- nothing
// waits -- but a second wave would double the latency), looked up once per (kernel, device, shared-memory size).
struct ClusterPlan { int csize, max_clusters; };

using FusedKern = void (*)(const FusedP);

// All instantiations of the kernel have the same pointer type, so the function attributes (which are per kernel) and the
// plans are keyed by the kernel's address.
int plan_clusters(FusedKern kern, size_t smem, ClusterPlan *out) {
  struct Entry { FusedKern kern; int dev; size_t smem; ClusterPlan plan; };
  struct Limit { FusedKern kern; int dev; size_t bytes; };
  static std::mutex mu;
  static Entry cache[256];
  static Limit limits[256];
  static int n_cached = 0, n_limits = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TMOE_ERR_CUDA;
  const size_t bucket = (smem + 8191) / 8192 * 8192;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_cached; ++i)
    if (cache[i].kern == kern && cache[i].dev == dev && cache[i].smem == bucket) { *out = cache[i].plan; return TMOE_OK; }
  // the dynamic shared-memory limit of a kernel is only ever raised (its earlier plans keep launching)
  Limit *lim = nullptr;
  for (int i = 0; i < n_limits; ++i)
    if (limits[i].kern == kern && limits[i].dev == dev) lim = &limits[i];
  if (!lim) {
    if (n_limits >= 256) return TMOE_ERR_UNSUPPORTED;
    limits[n_limits] = Limit{kern, dev, 0};
    lim = &limits[n_limits++];
  }
  if (bucket > lim->bytes) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bucket) != cudaSuccess) {
      (void)cudaGetLastError();
      return TMOE_ERR_UNSUPPORTED;
    }
    lim->bytes = bucket;
  }
  static const int force = [] { const char *e = getenv("TMOE_DECODE_CLUSTER"); return e ? atoi(e) : 0; }();
  ClusterPlan plan{0, 0};
  for (int cs : {16, 8}) {
    if (force && cs != force) continue;
    if (cs > 8 && cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
      (void)cudaGetLastError();
      continue;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cs); cfg.blockDim = dim3(kFThreads); cfg.dynamicSmemBytes = bucket;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = (unsigned)cs; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); continue; }
    // prefer the larger cluster unless it leaves more than a fifth of the SMs the smaller one would use idle
    if (plan.csize == 0 || n * cs * 4 > plan.max_clusters * plan.csize * 5) plan = ClusterPlan{cs, n};
  }
  if (plan.csize == 0) return TMOE_ERR_UNSUPPORTED;
  if (n_cached < 256) cache[n_cached++] = Entry{kern, dev, bucket, plan};
  *out = plan;
  return TMOE_OK;
}

template <int TMAX, int R1, int KMAX>
int launch_fused_t(const tmoe_layer_t &L, FusedP p, cudaStream_t st) {
  FusedKern kern = decode_fused_kernel<TMAX, R1, KMAX>;
  // size the shared memory for the widest slice any plan could give (nc >= 1 is refined below)
  const int units = L.r2 / 8;
  ClusterPlan plan;
  // sized for a plan of at least 4 clusters (the widest slice any accepted plan gives); the launch uses the real width
  size_t smem = fused_smem_bytes(TMAX, L, ((units + 3) / 4) * 8);
  if (smem > 200 * 1024) return TMOE_ERR_UNSUPPORTED;
  int rc = plan_clusters(kern, smem, &plan);
  if (rc) return rc;
  int nc = plan.max_clusters < kMaxDecodeClusters ? plan.max_clusters : kMaxDecodeClusters;
  if (nc > units) nc = units;
  if (nc < 4 && nc < units) return TMOE_ERR_UNSUPPORTED;
  p.nc = nc; p.csize = plan.csize;
  p.uexp_smem = L.n_experts * L.r1 <= kUexpSmemFloats ? 1 : 0;
  static const bool debug = []() { const char *e = getenv("TMOE_DEBUG"); return e && atoi(e) != 0; }();
  if (debug) fprintf(stderr, "tmoe decode_fused<%d,%d,%d>: clusters %d x %d CTAs (device holds %d)\n", TMAX, R1, KMAX, nc, plan.csize, plan.max_clusters);
  p.kc_max = ((units + nc - 1) / nc) * 8;
  const size_t smem_now = fused_smem_bytes(TMAX, L, p.kc_max);
  if (smem_now > (smem + 8191) / 8192 * 8192) return TMOE_ERR_UNSUPPORTED;   // fewer clusters than guessed and a wider slice: not planned for
  static const bool pdl_off = []() { const char *e = getenv("TMOE_PDL"); return e && atoi(e) == 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(nc * plan.csize)); cfg.blockDim = dim3(kFThreads); cfg.dynamicSmemBytes = smem_now; cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)plan.csize; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = pdl_off ? 1 : 2;
  if (cudaLaunchKernelEx(&cfg, kern, p) != cudaSuccess) return TMOE_ERR_CUDA;
  count_launch();
  return launch_status();
}

}  // namespace

int launch_decode_fused(const tmoe_layer_t &L, const void *x, const void *prepared, const PreparedLayout &P, int64_t T,
                        float *partial, unsigned int *counters, int32_t *idx_out, float *gates_out, float *c_out,
                        const OutEpilogue &epi, void *y, cudaStream_t st, int pre_norm, float pre_norm_eps) {
  static const bool off = []() { const char *e = getenv("TMOE_DECODE_FUSED"); return e && atoi(e) == 0; }();
  if (off || T < 1 || T > kFusedDecodeMaxTokens || L.top_k > 16) return TMOE_ERR_UNSUPPORTED;
  const char *pb = reinterpret_cast<const char *>(prepared);
  FusedP p{};
  p.x = (const bf16 *)x; p.uin_t = (const bf16 *)(pb + P.uin_t); p.wr = (const bf16 *)(pb + P.wr_b);
  p.g_t = (const bf16 *)(pb + P.g_t); p.uout_t = (const bf16 *)(pb + P.uout_t);
  p.normw = (const float *)(pb + P.normw); p.bias = (const float *)(pb + P.bias); p.uexp = (const float *)(pb + P.uexp);
  p.residual = (const bf16 *)epi.residual; p.gamma = (const bf16 *)epi.layer_scale; p.silu_gate = (const bf16 *)epi.silu_gate;
  p.y = (bf16 *)y; p.partial = partial; p.counters = counters;
  p.idx_out = idx_out; p.gates_out = gates_out; p.c_out = c_out;
  p.T = (int)T; p.d_in = L.d_in; p.r3 = L.r3; p.r2 = L.r2; p.E = L.n_experts; p.top_k = L.top_k; p.d_out = L.d_out;
  p.eps = L.eps; p.rc = router_cfg(L); p.pre_norm = pre_norm; p.pre_norm_eps = pre_norm_eps;
#define TMOE_DF(TM, R, K) return launch_fused_t<TM, R, K>(L, p, st)
#define TMOE_DF_K(TM, R) do { if (L.top_k <= 2) TMOE_DF(TM, R, 2); else if (L.top_k <= 8) TMOE_DF(TM, R, 8); else TMOE_DF(TM, R, 16); } while (0)
#define TMOE_DF_R(TM)                                                     \
  do {                                                                     \
    if (L.r1 == 2) TMOE_DF_K(TM, 2); else if (L.r1 == 4) TMOE_DF_K(TM, 4);  \
    else if (L.r1 == 8) TMOE_DF_K(TM, 8); else if (L.r1 == 16) TMOE_DF_K(TM, 16); \
    else if (L.r1 == 32) TMOE_DF_K(TM, 32); else return TMOE_ERR_UNSUPPORTED; \
  } while (0)
  if (T == 1) TMOE_DF_R(1);
  if (T == 2) TMOE_DF_R(2);
  TMOE_DF_R(4);
#undef TMOE_DF_R
#undef TMOE_DF_K
#undef TMOE_DF
}

}  // namespace tmoe
