// Body of the single-CTA out-projection GEMM kernel (see tc_out_gemm.cu for the description) and the pieces it shares
// with the CTA-pair kernel: the parameter block, the epilogue of one 64-column chunk and the bounded wait for the
// "rows ready" words through which the kernel that produces A releases 128-row tiles one by one.
#pragma once
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace tmoe {

using namespace ptx;

// ------------------------------------------------------------------------------------------
constexpr int OM = 128, ON = 256, OKB = 64, OSTAGES = 4;
constexpr int O_A_BYTES = OM * OKB * 2;   // 16 KB
constexpr int O_B_BYTES = ON * OKB * 2;   // 32 KB
constexpr int O_STAGE_BYTES = O_A_BYTES + O_B_BYTES;
constexpr int O_EPI_WARPS = 8;
constexpr int O_THREADS = (2 + O_EPI_WARPS) * 32;
constexpr int O_Y_BYTES = 32 * 64 * 2;  // 4 KB per epilogue warp: 32 rows x 64 bf16 output columns
constexpr int O_SMEM_BYTES = OSTAGES * O_STAGE_BYTES + O_EPI_WARPS * O_Y_BYTES + 1024;
constexpr int kKernelOut = 3;

// Diagnostic builds (-DTMOE_TRACE): block 0 accumulates the cycles its roles spend in each wait into
// status words [40..47].
#ifdef TMOE_TRACE
#define TMOE_TIC() trace_tic = clock64()
#define TMOE_TOC(i)                                                                             \
  do {                                                                                          \
    if (blockIdx.x == 0) {                                                                      \
      const int dt_ = (int)(clock64() - trace_tic);                                             \
      atomicAdd(&p.status[40 + (i)], dt_);                                                      \
      if ((i) == 2) atomicAdd(&p.status[48 + (dt_ < 64 ? 0 : dt_ < 256 ? 1 : dt_ < 1024 ? 2 : 3)], 1); \
      if ((i) == 2 && dt_ >= 1024) atomicAdd(&p.status[52], dt_);                               \
    }                                                                                           \
  } while (0)
#else
#define TMOE_TIC() do { } while (0)
#define TMOE_TOC(i) do { } while (0)
#endif

// Tensor maps of the further destinations of every output tile (OutParams::n_peers of them are valid): this GPU's rows
// inside the result buffers of other GPUs, reached through peer mappings.  Same shape and box as the map of y.
struct PeerMaps {
  CUtensorMap m[TMOE_MAX_PEERS];
};

// One finished 32 x 64 staging tile to y and to every peer destination, as one bulk group.
// stream_y: y is larger than L2 can hold next to the operands, so its lines are marked evict-first (measured on the
// 16384 x 512 x 4608 out-projection: 68.9 us against 72.5 us; no difference at K = 1024).
__device__ __forceinline__ void store_tile_everywhere(const CUtensorMap *tmY, const PeerMaps *pm, int n_peers, uint32_t stage_buf,
                                                      int c0, int c1, bool stream_y) {
  if (stream_y) tma_store_2d_hint(tmY, stage_buf, c0, c1, l2_policy_evict_first());
  else tma_store_2d(tmY, stage_buf, c0, c1);
  for (int q = 0; q < n_peers; ++q) tma_store_2d(&pm->m[q], stage_buf, c0, c1);
  tma_store_commit();
}

struct OutParams {
  bf16 *y;
  const float *bias;
  const bf16 *residual;
  const bf16 *gamma;
  const bf16 *silu_gate;
  int64_t T;
  int N, K;
  int num_m, num_n;
  // Output columns per tile of the single-CTA kernel: 256 (0 means 256), or 128 when 256-wide tiles would leave more than
  // half of the SMs without one (few token rows); num_n counts tiles of this width and tmB's box has this many rows.
  int on;
  int n_peers;   // valid entries of the kernel's PeerMaps argument
  int stream_y;  // y does not fit in L2: store it with the evict-first hint
  int32_t *status;
  // Tile-by-tile hand-over from the kernel that produces A (CTA-pair kernel only; all three null / 0 otherwise).
  //   ready   8 words per 128-row tile of A, each set to `epoch` by one epilogue warp of the producing CTA once its rows
  //           are stored: rows [128 m, 128 m + 128) may be read when ready[8 m .. 8 m + 7] all equal `epoch`
  //   queue   64-bit word {epoch : 32 | tiles handed out : 32}: the pairs draw their output tiles from it in order, so a
  //           pair that becomes resident late (while the producing kernel's last wave still runs) simply takes what is left;
  //           queue[1] = {epoch : 32 | producing CTAs finished : 32}, n_producers of them in all
  const uint32_t *ready;
  uint32_t epoch;
  unsigned long long *queue;
  int n_producers;
};

// The bias of a warp's share of an output tile, one float4 per lane: lane l holds columns [cbase + 4 l, cbase + 4 l + 4).
// Loaded once per tile BEFORE the wait for the accumulator, so its trip to L2 (the SM's L1 is almost entirely shared
// memory here) is off the epilogue's chain; the chunks then fetch their values from the owning lanes by shuffle.
__device__ __forceinline__ float4 load_bias_lane(const OutParams &p, int cbase, int lane) {
  const int col = cbase + lane * 4;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  // volatile: a plain __ldg is sunk by the compiler to its first use, i.e. behind the wait it is meant to overlap
  if (p.bias && col < p.N)
    asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p.bias + col));
  return v;
}

// Epilogue of one 64-column chunk of an output row: accumulator registers r (two 32-column TMEM loads) + bias, optional
// silu(gate) * v and residual + layer_scale * v, rounded to bf16 into this lane's 128-byte row of the warp's staging
// tile (16-byte chunks XOR-swizzled as the TMA box expects).  `bias_lane` is load_bias_lane() of the warp's column base
// and col0 - cbase = `cofs` (a multiple of 64).  The shared stores carry no "memory" clobber: the staging
// tile is touched by nothing else the compiler sees, volatile asm statements keep their order, and the proxy fence
// that follows is the barrier.  Must be entered by all 32 lanes (shuffles).
__device__ __forceinline__ void out_epilogue_chunk(const OutParams &p, const uint32_t (&r)[2][32], int col0, int64_t row,
                                                   int lane, uint32_t stage_buf, const float4 &bias_lane, int cofs) {
  const bool extras = (p.silu_gate != nullptr) | (p.residual != nullptr);
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    float4 b[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const int src = (cofs >> 2) + h2 * 8 + g;   // the lane that holds this group of four columns
      b[g].x = __shfl_sync(0xffffffffu, bias_lane.x, src);
      b[g].y = __shfl_sync(0xffffffffu, bias_lane.y, src);
      b[g].z = __shfl_sync(0xffffffffu, bias_lane.z, src);
      b[g].w = __shfl_sync(0xffffffffu, bias_lane.w, src);
    }
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const int col = col0 + h2 * 32 + g * 8;
      float v[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = __uint_as_float(r[h2][g * 8 + q]);
      v[0] += b[2 * g].x; v[1] += b[2 * g].y; v[2] += b[2 * g].z; v[3] += b[2 * g].w;
      v[4] += b[2 * g + 1].x; v[5] += b[2 * g + 1].y; v[6] += b[2 * g + 1].z; v[7] += b[2 * g + 1].w;
      if (extras && col < p.N && row < p.T) {
        if (p.silu_gate) {
          const uint4 gv = __ldg(reinterpret_cast<const uint4 *>(p.silu_gate + row * p.N + col));
          const uint32_t gw2[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float g0 = __uint_as_float(gw2[q] << 16), g1 = __uint_as_float(gw2[q] & 0xffff0000u);
            v[2 * q] *= g0 / (1.f + __expf(-g0));
            v[2 * q + 1] *= g1 / (1.f + __expf(-g1));
          }
        }
        if (p.residual) {
          const uint4 rr = __ldg(reinterpret_cast<const uint4 *>(p.residual + row * p.N + col));
          const uint4 gg = __ldg(reinterpret_cast<const uint4 *>(p.gamma + col));
          const uint32_t rw[4] = {rr.x, rr.y, rr.z, rr.w}, gw[4] = {gg.x, gg.y, gg.z, gg.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            v[2 * q] = __uint_as_float(rw[q] << 16) + __uint_as_float(gw[q] << 16) * v[2 * q];
            v[2 * q + 1] = __uint_as_float(rw[q] & 0xffff0000u) + __uint_as_float(gw[q] & 0xffff0000u) * v[2 * q + 1];
          }
        }
      }
      const uint32_t chunk = (uint32_t)(h2 * 4 + g) ^ (uint32_t)(lane & 7);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(stage_buf + lane * 128 + chunk * 16),
                   "r"(pack_bf16x2(v[0], v[1])), "r"(pack_bf16x2(v[2], v[3])), "r"(pack_bf16x2(v[4], v[5])),
                   "r"(pack_bf16x2(v[6], v[7])));
    }
  }
}

// Bounded wait for the eight hand-off words of one 128-row tile of A (32-byte aligned; written with st.global after a
// __threadfence by the producing CTA's epilogue warps).  The words are polled with two 16-byte relaxed loads -- one trip
// to L2 per poll, this sits in front of every tile's first operand load -- and the acquire is a single fence once all
// eight match.  The TMA loads that follow read through the async proxy, hence the proxy fence.
__device__ __forceinline__ bool rows_ready_wait(const uint32_t *flags, uint32_t epoch, int32_t *status) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  for (;;) {
    uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "l"(flags) : "memory");
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "l"(flags + 4) : "memory");
    const bool all = (a0 == epoch) & (a1 == epoch) & (a2 == epoch) & (a3 == epoch) & (b0 == epoch) & (b1 == epoch) &
                     (b2 == epoch) & (b3 == epoch);
    if (all) break;
    if ((++spins & 0x3fu) == 0) {
      if (*reinterpret_cast<volatile int32_t *>(status) != 0) return false;
      if (clock64() - t0 > kWaitLimitCycles) {
        if (atomicCAS(status, 0, (int32_t)TMOE_ERR_DEVICE_WAIT) == 0) {
          status[1] = 3; status[2] = 11; status[3] = (int32_t)blockIdx.x;
          __threadfence();
        }
        return false;
      }
    }
    __nanosleep(100);
  }
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
  asm volatile("fence.proxy.async;" ::: "memory");
  return true;
}

// Processes tiles tile_first, tile_first + tile_step, ... < tile_end (tile = m * num_n + n, 128 x 256 outputs each).
// Must be entered by all O_THREADS threads of a CTA that holds O_SMEM_BYTES of dynamic shared memory and no TMEM.
// A must be complete when `dependent` is false; otherwise the body waits for the kernel before it in the stream.
__device__ __forceinline__ void tc_out_body(const CUtensorMap *tmA, const CUtensorMap *tmB, const CUtensorMap *tmY,
                                            const PeerMaps *pm, const OutParams &p, int tile_first, int tile_step, int tile_end,
                                            uint8_t *smem_raw, bool dependent = false) {
  __shared__ __align__(8) uint64_t bar_full[OSTAGES], bar_empty[OSTAGES], bar_tfull[2], bar_tempty[2];
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < OSTAGES; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_tfull[s]), 1); mbar_init(smem_u32(&bar_tempty[s]), O_EPI_WARPS); }
    fence_mbar_init();
    prefetch_tmap(tmA);
    prefetch_tmap(tmB);
    prefetch_tmap(tmY);
  }
  if (warp == 2) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }  // an epilogue warp: its lanes never retire early
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  // the barriers, the TMEM columns and the tensor-map prefetches above do not depend on the kernel that produces A
  if (dependent) griddep_wait();

  const int KB = (p.K + OKB - 1) / OKB;
  const int on = p.on ? p.on : ON;
#ifdef TMOE_TRACE
  const long long trace_t0 = clock64();
  long long trace_tic = 0;
#endif

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = tile_first; tile < tile_end && ok; tile += tile_step) {
        const int m0 = (tile / p.num_n) * OM, n0 = (tile % p.num_n) * on;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % OSTAGES, ph = (it / OSTAGES) & 1;
          TMOE_TIC();
          if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, p.status, kKernelOut, 2))) break;
          TMOE_TOC(0);  // producer waiting for a free stage
          const uint32_t full = smem_u32(&bar_full[s]);
          mbar_arrive_expect_tx(full, O_A_BYTES + on * 128);
          const uint32_t sa = ring + s * O_STAGE_BYTES;
          tma_load_2d(sa, tmA, kb * OKB, m0, full);
          tma_load_2d(sa + O_A_BYTES, tmB, kb * OKB, n0, full);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // The issuing thread's loop is the serial path (see mbar_wait_or_exit): fixed trip counts, no side exits,
      // ring position and descriptors kept incrementally.
      const uint32_t idesc = umma_idesc_bf16(OM, on);
      const uint64_t desc0 = umma_desc_k_sw128(ring);
      uint32_t s = 0, ph = 0, tcount = 0;
      for (int tile = tile_first; tile < tile_end; tile += tile_step, ++tcount) {
        const uint32_t slot = tcount & 1, aph = (tcount >> 1) & 1;
        TMOE_TIC();
        mbar_wait_or_exit(smem_u32(&bar_tempty[slot]), aph ^ 1, p.status, kKernelOut, 4);
        TMOE_TOC(1);  // MMA thread waiting for the epilogue to release an accumulator
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + slot * ON;
        for (int kb = 0; kb < KB; ++kb) {
          TMOE_TIC();
          mbar_wait_or_exit(smem_u32(&bar_full[s]), ph, p.status, kKernelOut, 1);
          TMOE_TOC(2);  // MMA thread waiting for operand tiles
          const uint64_t da = desc0 + s * (uint32_t)(O_STAGE_BYTES >> 4), db = da + (O_A_BYTES >> 4);
          const uint32_t acc0 = kb != 0;
#pragma unroll
          for (int k = 0; k < OKB / 16; ++k)  // +32 bytes (= 2 in >>4 units) per 16-element K step
            umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, acc0 | (uint32_t)(k != 0));
          umma_commit(smem_u32(&bar_empty[s]));
          if (++s == OSTAGES) { s = 0; ph ^= 1; }
        }
        umma_commit(smem_u32(&bar_tfull[slot]));
      }
    }
  } else {
    // Eight epilogue warps: warp w may read TMEM lanes 32*(w%4)..+31, so two warps share each row
    // quadrant and split the tile's 256 columns.  Each warp stages 32 rows x 64 columns (4 KB, swizzled)
    // and issues its own TMA store, so the warps never wait for one another.
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const int row_in_tile = quad * 32 + lane;
    const uint32_t stage_buf = ring + OSTAGES * O_STAGE_BYTES + ew * O_Y_BYTES;
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = tile_first; tile < tile_end && ok; tile += tile_step, ++tcount) {
      const int m0 = (tile / p.num_n) * OM, n0 = (tile % p.num_n) * on;
      const uint32_t slot = tcount & 1, aph = (tcount >> 1) & 1;
      const float4 bias_lane = load_bias_lane(p, n0 + half * (on >> 1), lane);
      TMOE_TIC();
      ok = mbar_wait(smem_u32(&bar_tfull[slot]), aph, p.status, kKernelOut, 3);
      if (threadIdx.x == 64) TMOE_TOC(3);  // epilogue warp 2 waiting for a finished accumulator
      ok = __all_sync(0xffffffffu, ok);  // the TMEM loads below are warp-collective
      if (!ok) break;
      tc_fence_after();
      const int64_t row = (int64_t)m0 + row_in_tile;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + slot * ON + half * (on >> 1);
      const int ncc = on >> 7;   // 64-column chunks per warp: 2 for 256-wide tiles, 1 for 128-wide
#pragma unroll 1
      for (int cc = 0; cc < ncc; ++cc) {
        const int col0 = n0 + half * (on >> 1) + cc * 64;
        uint32_t r[2][32];
        tmem_ld32(t_row + cc * 64, r[0]);
        tmem_ld32(t_row + cc * 64 + 32, r[1]);
        tmem_ld_wait(r[0], r[1]);
        if (cc == ncc - 1) {  // this warp has read its whole share of the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_tempty[slot]));
        }
        TMOE_TIC();
        if (lane == 0) tma_store_wait_read<0>();  // the previous store has finished reading the staging tile
        if (threadIdx.x == 64) TMOE_TOC(4);  // epilogue warp 2 waiting for its previous TMA store
        __syncwarp();
        out_epilogue_chunk(p, r, col0, row, lane, stage_buf, bias_lane, cc * 64);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && col0 < p.N) store_tile_everywhere(tmY, pm, p.n_peers, stage_buf, col0, m0 + quad * 32, p.stream_y != 0);
      }
    }
    if (lane == 0) tma_store_wait_all();
  }
#ifdef TMOE_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 64) p.status[40 + 7] = (int32_t)(clock64() - trace_t0);  // kernel cycles
#endif
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace tmoe
