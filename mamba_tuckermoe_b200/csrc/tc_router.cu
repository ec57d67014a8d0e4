// Stand-alone router for bf16 layers (pure_torch_mlx/model.py:75-77, 93): scores = x @ router_w^T on the tensor cores,
// top-k, gate weights and c = sum_k gate_k * U_expert[idx_k], one launch whose only HBM traffic is one read of x.
//
// Persistent: one CTA per SM walks over the 128-token tiles it owns (tile = blockIdx.x, + gridDim.x, ...).
//   warp 0      TMA producer: ring of {x tile 128 x 64, router tile e_pad x 64} stages, running ahead into the NEXT tile while
//               the current one is being selected (a kernel with one tile per CTA pays a launch, a pipeline fill and an
//               exposed selection per tile: 37 us for the 100 MB of x of the prefill configuration against 31 us here, L2 flushed)
//   warp 1      one thread issues tcgen05.mma 128 x e_pad x 16 into one of two TMEM accumulators (256 columns each)
//   warps 2..5  one thread per token row (a warp reads TMEM lanes 32 * (warp % 4) .. + 31): keyed running top-k over the
//               score columns, gates, c, stores; the accumulator goes back to the MMA thread as soon as it has been read
// router_w [E, d_in] as the layer stores it is already the K-major B operand; rows beyond E are zero-filled by TMA.
// Every wait is bounded (status words of the workspace), the MMA thread retires on expiry, TMEM is freed by a warp that
// never leaves early.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "routing.cuh"

namespace tmoe {

using namespace ptx;

namespace {

constexpr int RT_TM = 128;
constexpr int RT_X_BYTES = RT_TM * 64 * 2;        // 16 KB
constexpr int RT_RING_BYTES = 216 * 1024;
constexpr int RT_SMEM_BYTES = RT_RING_BYTES + 1024;
constexpr int RT_STAGES_MAX = 12;
constexpr int RT_EPI_WARPS = 4;
constexpr int RT_THREADS = (2 + RT_EPI_WARPS) * 32;
constexpr int kKernelRouter = 5;

struct RouterParams {
  int64_t T;
  int d_in, E, e_pad, top_k, r1;
  int n_tiles, n_stages;
  int n_pass;         // expert chunks of e_pad (<= 256) columns per token tile: more than 256 experts take several passes over x
  RouterCfg rc;
  const bf16 *uexp;   // [E, r1], the layer's own table
  int32_t *idx_out;   // [T, top_k]
  float *gates_out;   // [T, top_k]
  float *c_out;       // [T, r1]
  int32_t *status;
};

// PAIR: launched as clusters of two CTAs on neighbouring token tiles; the even CTA issues every MMA for both (tcgen05
// cta_group::2, M = 256) and each CTA loads only half of the rows of a router tile.  The kernel's bandwidth is the bytes of x
// it keeps in flight per SM, and a stage that holds half a router tile leaves room for more of them (E = 256: 6 stages of
// 32 KB instead of 4 of 48 KB).
template <int RK, bool PAIR>
__global__ void __launch_bounds__(RT_THREADS, 1)
tc_router_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const RouterParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[RT_STAGES_MAX], bar_empty[RT_STAGES_MAX], bar_afull[2], bar_aempty[2];
  __shared__ uint32_t tmem_base_s;
  griddep_launch_dependents();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int NB = PAIR ? 2 : 1;   // CTAs that share one MMA
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const int w_rows = p.e_pad / NB;   // rows of a router tile in this CTA's stage
  const int stage_bytes = RT_X_BYTES + w_rows * 128;
  const int KA = p.d_in / 64;
  // token tiles of this CTA: first, first + step, ... (PAIR: the pair walks over tile pairs; the odd CTA of the last pair may
  // stand on a tile beyond the last one -- its loads return zeros and its rows are never stored)
  const int first = PAIR ? (int)(blockIdx.x >> 1) * 2 + (int)rank : (int)blockIdx.x;
  const int step = (int)gridDim.x;
  const int tile_end = PAIR ? ((p.n_tiles + 1) & ~1) : p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RT_STAGES_MAX; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_afull[s]), 1); mbar_init(smem_u32(&bar_aempty[s]), NB * RT_EPI_WARPS); }
    fence_mbar_init();
    prefetch_tmap(&tmX);
    prefetch_tmap(&tmW);
  }
  if (warp == 2) {
    if constexpr (PAIR) { tmem_alloc_pair(smem_u32(&tmem_base_s), 512); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {   // both CTAs' barriers are initialised before anyone signals across the pair
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  griddep_wait();   // x may come from the kernel before this one in the stream

  if (warp == 0) {
    // (Asking L2 for whole rows of the next tile ahead of its boxes -- one bulk prefetch per row -- was measured: 38 us
    // against 31 us per launch with L2 flushed; the boxes alone keep HBM busier.)
    uint32_t s = 0, ph = 0;
    bool ok = true;
    // a single pass reads x once: evict-first, the router rows stay (30.8 -> 28.3 us per launch right after an L2 flush)
    const uint64_t pol_x = p.n_pass == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
    for (int tile = first; tile < tile_end && ok; tile += step) {
      if (lane == 0) {
        for (int pass = 0; pass < p.n_pass && ok; ++pass) {   // passes after the first find the x tile in L2
          for (int kb = 0; kb < KA; ++kb) {
            if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, p.status, kKernelRouter, 2))) break;
            const uint32_t full = smem_u32(&bar_full[s]);
            const uint32_t sa = ring + s * (uint32_t)stage_bytes;
            if constexpr (PAIR) {   // both CTAs' bytes are counted on the barrier of the CTA that issues the MMAs
              if (rank == 0) mbar_arrive_expect_tx(full, 2u * (uint32_t)stage_bytes);
              const uint32_t full0 = mapa_u32(full, 0);
              tma_load_2d_pair_hint(sa, &tmX, kb * 64, tile * RT_TM, full0, pol_x);
              tma_load_2d_pair(sa + RT_X_BYTES, &tmW, kb * 64, pass * p.e_pad + (int)rank * w_rows, full0);
            } else {
              mbar_arrive_expect_tx(full, (uint32_t)stage_bytes);
              tma_load_2d_hint(sa, &tmX, kb * 64, tile * RT_TM, full, pol_x);
              tma_load_2d(sa + RT_X_BYTES, &tmW, kb * 64, pass * p.e_pad, full);
            }
            if (++s == (uint32_t)p.n_stages) { s = 0; ph ^= 1; }
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_bf16(NB * RT_TM, p.e_pad);
      const uint64_t desc0 = umma_desc_k_sw128(ring);
      const uint32_t stage16 = (uint32_t)stage_bytes >> 4;
      uint32_t s = 0, ph = 0, tcount = 0;
      const int n_acc = ((tile_end - first + step - 1) / step) * p.n_pass;   // (tile, pass) pairs of this CTA
      for (int ia = 0; ia < n_acc; ++ia, ++tcount) {
        const uint32_t slot = tcount & 1, aph = (tcount >> 1) & 1;
        mbar_wait_or_exit(smem_u32(&bar_aempty[slot]), aph ^ 1, p.status, kKernelRouter, 4);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + slot * 256;
        for (int kb = 0; kb < KA; ++kb) {
          mbar_wait_or_exit(smem_u32(&bar_full[s]), ph, p.status, kKernelRouter, 1);
          const uint64_t dx = desc0 + s * stage16, dw = dx + (RT_X_BYTES >> 4);
          const uint32_t acc0 = kb != 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            if constexpr (PAIR) umma_bf16_pair(d_tmem, dx + 2 * k, dw + 2 * k, idesc, acc0 | (uint32_t)(k != 0));
            else umma_bf16(d_tmem, dx + 2 * k, dw + 2 * k, idesc, acc0 | (uint32_t)(k != 0));
          }
          if constexpr (PAIR) umma_commit_pair(smem_u32(&bar_empty[s]), 3); else umma_commit(smem_u32(&bar_empty[s]));
          if (++s == (uint32_t)p.n_stages) { s = 0; ph ^= 1; }
        }
        if constexpr (PAIR) umma_commit_pair(smem_u32(&bar_afull[slot]), 3); else umma_commit(smem_u32(&bar_afull[slot]));
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const bool rule1 = p.rc.mode == 1;   // the top-k then orders by the tempered capped logit (RouterCfg::order_value)
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = first; tile < tile_end && ok; tile += step) {
      uint32_t key[RK];   // the running top-k list of this thread's token, carried across the expert chunks
#pragma unroll
      for (int j = 0; j < RK; ++j) key[j] = 0u;
      float z_all = 1.f;
      float sv[RK];
      int si[RK];
      for (int pass = 0; pass < p.n_pass; ++pass, ++tcount) {
        const uint32_t slot = tcount & 1, aph = (tcount >> 1) & 1;
        ok = mbar_wait(smem_u32(&bar_afull[slot]), aph, p.status, kKernelRouter, 3);
        ok = __all_sync(0xffffffffu, ok);   // the TMEM loads below are warp-collective
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + slot * 256;
        const int e0 = pass * p.e_pad;
        // Running top-k over the score columns, branch-free: a score rounded to bf16 (the reference's rounding of its logits)
        // has 16 significant bits, so (order-preserving map of those bits) << 16 | (0xFFFF - expert) is a 32-bit key whose
        // unsigned order is "higher score first, equal scores -> lower expert index first"; the sorted list is kept with
        // integer max / min only.
        for (int cc = 0; cc < p.e_pad / 16; ++cc) {
          uint32_t r[16];
          tmem_ld16(t_row + cc * 16, r);
          tmem_ld_wait(r);
#pragma unroll
          for (int q = 0; q < 16; ++q) {
            const int e = e0 + cc * 16 + q;
            uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[q])));
            if (rule1) b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(p.rc.logit(__uint_as_float(b << 16))));
            b = (b == 0x8000u) ? 0u : b;   // -0 and +0 compare equal
            const uint32_t u = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
            uint32_t carry = (e < p.E) ? ((u << 16) | (0xffffu - (uint32_t)e)) : 0u;
#pragma unroll
            for (int j = 0; j < RK; ++j) {
              const uint32_t hi = max(key[j], carry);
              carry = min(key[j], carry);
              key[j] = hi;
            }
          }
        }
#pragma unroll
        for (int j = 0; j < RK; ++j) {
          const uint32_t u = key[j] >> 16;
          const uint32_t b = (u & 0x8000u) ? (u & 0x7fffu) : (~u & 0xffffu);
          sv[j] = __uint_as_float(b << 16);
          si[j] = (int)(0xffffu - (key[j] & 0xffffu));
        }
        // capped-softmax rule only: its denominator runs over ALL experts, relative to the top logit (a second pass over the
        // columns, so that the default rule's scan above stays branch-free)
        if (p.rc.mode == 1) {   // (one expert chunk only: the launcher sends larger layers with this rule elsewhere)
          const float l0 = sv[0];   // the list holds logits under this rule
          z_all = 0.f;
          for (int cc = 0; cc < p.e_pad / 16; ++cc) {
            uint32_t r[16];
            tmem_ld16(t_row + cc * 16, r);
            tmem_ld_wait(r);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              const float sc = round_to<bf16>(__uint_as_float(r[q]));
              if (cc * 16 + q < p.E) z_all += expf(p.rc.logit(sc) - l0);
            }
          }
        }
        // the accumulator has been read: the MMA thread may start the tile after next in it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (PAIR) mbar_arrive_cluster(mapa_u32(smem_u32(&bar_aempty[slot]), 0)); else mbar_arrive(smem_u32(&bar_aempty[slot]));
        }
      }
      if (!ok) break;

      const int64_t grow = (int64_t)tile * RT_TM + row;
      if (grow < p.T) {
        float gate[RK];
        gates_of<bf16, RK>(sv, p.top_k, p.rc, z_all, gate);
#pragma unroll
        for (int j = 0; j < RK; ++j) {
          if (j < p.top_k) {
            p.idx_out[grow * p.top_k + j] = si[j];
            p.gates_out[grow * p.top_k + j] = gate[j];
          }
        }
        for (int a = 0; a < p.r1; ++a) {
          float ca = 0.f;
#pragma unroll
          for (int j = 0; j < RK; ++j) {
            if (j < p.top_k) {
              const int e = min(max(si[j], 0), p.E - 1);
              ca = fmaf(gate[j], __bfloat162float(__ldg(p.uexp + e * p.r1 + a)), ca);
            }
          }
          p.c_out[grow * p.r1 + a] = ca;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) {   // the other CTA may still be signalling this CTA's barriers, or its MMAs reading this CTA's tiles
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

// idx / gates / c for T tokens from x and the layer's own router_w [E, d_in] / U_expert [E, r1] (bf16).
// TMOE_ERR_UNSUPPORTED for more than 1024 experts, more than 256 with the capped-softmax rule, top_k > 8 or d_in % 64 != 0.
int launch_tc_router(const tmoe_layer_t &L, const void *x, const void *router_w, const void *uexp_bf16, int64_t T_, int32_t *idx,
                     float *gates, float *c, int32_t *status, cudaStream_t st) {
  // up to 256 experts: one accumulator of e_pad columns per token tile; up to 1024: chunks of 256 experts, one pass over the
  // tile's x per chunk (the later passes read it from L2), the top-k list carried from chunk to chunk
  const int e_all = (int)align_up(L.n_experts, 16);
  const int n_pass = (e_all + 255) / 256;
  const int e_pad = n_pass == 1 ? e_all : 256;
  if (n_pass > 4 || (n_pass > 1 && L.router_mode != 0) || L.top_k > 8 || (L.d_in % 64) != 0) return TMOE_ERR_UNSUPPORTED;
  CUtensorMap tmX, tmW;
  int rc = encode_tmap_bf16_2d(&tmX, x, (uint64_t)T_, (uint64_t)L.d_in, RT_TM);
  if (rc) return rc;
  // CTA pairs where the router tile is at least as large as the x tile (128 experts or more per chunk): there the ring is
  // only 4 stages deep and half a router tile per CTA makes it 6 (805 MB of x at E = 256: 162 us against 180 us; at E = 64,
  // 10 stages against 9, pairs are 4 % slower).  TMOE_ROUTER_PAIRS=0 / 1 forces the choice.
  static const int pairs_env = [] { const char *s = getenv("TMOE_ROUTER_PAIRS"); return s ? (atoi(s) != 0 ? 1 : 0) : -1; }();
  const bool pairs = T_ > RT_TM && (pairs_env >= 0 ? pairs_env == 1 : e_pad >= 128);
  const int nb = pairs ? 2 : 1;
  if ((rc = encode_tmap_bf16_2d(&tmW, router_w, (uint64_t)L.n_experts, (uint64_t)L.d_in, (uint32_t)(e_pad / nb)))) return rc;
  const int sms = current_device_sms();
  if (sms <= 0) return TMOE_ERR_CUDA;
  RouterParams p{};
  p.T = T_; p.d_in = L.d_in; p.E = L.n_experts; p.e_pad = e_pad; p.top_k = L.top_k; p.r1 = L.r1;
  p.n_tiles = (int)((T_ + RT_TM - 1) / RT_TM);
  p.n_pass = n_pass;
  const int stage_bytes = RT_X_BYTES + e_pad / nb * 128;
  p.n_stages = RT_RING_BYTES / stage_bytes < RT_STAGES_MAX ? RT_RING_BYTES / stage_bytes : RT_STAGES_MAX;
  p.rc = router_cfg(L);
  p.uexp = reinterpret_cast<const bf16 *>(uexp_bf16);
  p.idx_out = idx; p.gates_out = gates; p.c_out = c; p.status = status;
  unsigned grid = (unsigned)(p.n_tiles < sms ? p.n_tiles : sms);
  if (pairs) {   // whole pairs: as many as there are tile pairs, at most one per two SMs
    const unsigned want = (unsigned)((p.n_tiles + 1) / 2), have = (unsigned)(sms / 2);
    grid = 2u * (want < have ? want : have);
  }
  cudaError_t e;
#define TMOE_RT(K, PR)                                                                                                     \
  do {                                                                                                                     \
    e = cudaFuncSetAttribute(tc_router_kernel<K, PR>, cudaFuncAttributeMaxDynamicSharedMemorySize, RT_SMEM_BYTES);         \
    if (e == cudaSuccess)                                                                                                  \
      e = launch_pdl_cluster(tc_router_kernel<K, PR>, dim3(grid), dim3(RT_THREADS), (size_t)RT_SMEM_BYTES, st, PR ? 2u : 1u, tmX, tmW, p); \
  } while (0)
  if (L.top_k <= 2) { if (pairs) TMOE_RT(2, true); else TMOE_RT(2, false); }
  else { if (pairs) TMOE_RT(8, true); else TMOE_RT(8, false); }
#undef TMOE_RT
  if (e != cudaSuccess) return TMOE_ERR_CUDA;
  count_launch();
  return launch_status();
}

}  // namespace tmoe
