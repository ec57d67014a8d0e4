// Out-projection on the 5th-generation tensor cores (subsystem 3):
//   y[T, d_out] = z[T, r2] @ U_out + bias                  (pure_torch_mlx/model.py:101)
//   optionally   y = residual + layer_scale * (...)         (model.py:260, 341)
//
// Persistent warp-specialised kernel, one CTA per SM:
//   warp 0   TMA producer: {64 x 128} tiles of z and {64 x 256} tiles of U_out^T (K-major bf16,
//            128-byte swizzle) into a 4-stage shared-memory ring, mbarrier complete_tx.
//   warp 1   one elected thread issues tcgen05.mma (128 x 256 x 16, bf16 -> fp32) into one of two
//            256-column TMEM accumulators and commits stage-free / accumulator-full barriers.
//   warps 2-9 epilogue: tcgen05.ld of the accumulator (thread = output row, two warps per row quadrant
//            splitting the columns), bias / residual / layer-scale in fp32, bf16 pack into a swizzled
//            4 KB staging tile per warp, TMA store; runs under the next tile's MMAs.
// Every mbarrier wait is bounded and reports through the workspace status words.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "tc_out_body.cuh"
#include <cstdlib>

namespace tmoe {

using namespace ptx;

// ------------------------------------------------------------------------------------------
// Tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
// ------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

int encode_tmap_bf16_2d(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return TMOE_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (cols % 8) || box_rows == 0 || box_rows > 256) return TMOE_ERR_ALIGN;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {cols * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? TMOE_OK : TMOE_ERR_DRIVER;
}

__global__ void __launch_bounds__(O_THREADS, 1)
tc_out_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
              const __grid_constant__ CUtensorMap tmY, const __grid_constant__ PeerMaps pm, OutParams p) {
  extern __shared__ uint8_t smem_raw[];
  griddep_launch_dependents();   // all CTAs of this persistent grid are resident: the next kernel may set up on SMs as they free
  tc_out_body(&tmA, &tmB, &tmY, &pm, p, (int)blockIdx.x, (int)gridDim.x, p.num_m * p.num_n, smem_raw, true);
}

// ------------------------------------------------------------------------------------------
// The same GEMM on CTA pairs (cluster of 2, tcgen05 cta_group::2): a pair owns a 256 x 256 output tile,
// each CTA its own 128 rows.  Per k block a CTA loads its 128 x 64 piece of A and HALF of the B tile
// (128 of the 256 rows); the MMA issued by CTA 0 reads both halves.  Shared-memory traffic per SM drops
// from 48 KB written + 48 KB read per k block to 32 KB + 32 KB, which is what bounds the single-CTA kernel
// (128 B/clk of shared-memory bandwidth against 96 B/clk of operand reads plus the TMA fills).
// Barriers: full[s] lives in CTA 0 and counts the bytes of both CTAs' loads; empty[s] and tfull[slot] are
// signalled in both CTAs by multicast commits; tempty[slot] lives in CTA 0 and collects 16 warp arrivals.
//
// Tile-by-tile hand-over (OutParams::queue != nullptr).  When the kernel that produces A runs its CTAs in more than one wave
// (256 token tiles on 148 SMs), the SMs its last, partial wave leaves free would idle until that kernel has completed.
// Launched as its programmatic dependent, this kernel's pairs become resident on exactly those SMs as soon as every CTA of
// the producer has started; instead of waiting for the producer to complete (griddepcontrol.wait) they draw output tiles
// from a queue in row order and wait, per 128-row tile of A, for the words the producing CTA sets once its rows are stored.
// Every producing CTA is running or done by then, so such a wait always ends; it is bounded all the same.  Pairs that become
// resident later (as the producer's last wave retires) take what is left.  The queue word carries the forward's epoch: a
// forward re-tags it instead of anybody resetting it, and a straggler of an older forward that finds a newer tag stops.
constexpr int P_STAGES = 6;
constexpr int P_STAGE_BYTES = O_A_BYTES + O_A_BYTES;  // 16 KB of A + 16 KB (half) of B
constexpr int P_SMEM_BYTES = P_STAGES * P_STAGE_BYTES + O_EPI_WARPS * O_Y_BYTES + 1024;
constexpr int P_SCHED = 16;   // ring of scheduled tile indices; the producer is never this many tiles ahead of the epilogue
constexpr int kKernelOutPair = 4;

// Next ticket of forward `epoch` from the queue word {epoch : 32 | tickets handed out : 32}, or -1 when all `total` are
// handed out.  The producing kernel tags the word with the forward's epoch (count 0) before any of its CTAs can have
// finished a tile, i.e. long before a CTA of this kernel runs; the tag is checked all the same (bounded).  The draw itself is
// one atomic add: a compare-and-swap loop starves here -- 74 pairs draw ten tickets per microsecond, more than one per
// load-to-CAS window, and the pairs furthest from the word's L2 slice were measured to lose every attempt for 300 us.
__device__ __forceinline__ int draw_ticket(unsigned long long *queue, uint32_t epoch, int total, int32_t *status) {
  const long long t0 = clock64();
  for (uint32_t spins = 0;; ++spins) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(queue) : "memory");
    const uint32_t e = (uint32_t)(v >> 32);
    if (e == epoch) break;
    if ((int32_t)(e - epoch) > 0) return -1;             // a newer forward owns the word: this one is complete
    if ((spins & 0x3fu) == 0x3fu) {
      if (*reinterpret_cast<volatile int32_t *>(status) != 0) return -1;
      if (clock64() - t0 > kWaitLimitCycles) {
        if (atomicCAS(status, 0, (int32_t)TMOE_ERR_DEVICE_WAIT) == 0) {
          status[1] = 4; status[2] = 12; status[3] = (int32_t)blockIdx.x;
          __threadfence();
        }
        return -1;
      }
    }
    __nanosleep(200);
  }
  const unsigned long long old = atomicAdd(queue, 1ull);
  if ((uint32_t)(old >> 32) != epoch) return -1;         // (re-tagged by a newer forward in between: complete)
  const uint32_t n = (uint32_t)old;
  return n < (uint32_t)total ? (int)n : -1;
}
// Every further draw is the atomic add alone.  Its result is only looked at one tile later (ticket_of), so the trip to
// L2 runs under the tile's operand loads instead of in front of them.
__device__ __forceinline__ unsigned long long draw_next(unsigned long long *queue) { return atomicAdd(queue, 1ull); }
__device__ __forceinline__ int ticket_of(unsigned long long old, uint32_t epoch, int total) {
  if ((uint32_t)(old >> 32) != epoch) return -1;
  const uint32_t n = (uint32_t)old;
  return n < (uint32_t)total ? (int)n : -1;
}

// DYN: tile-by-tile hand-over (the plain instantiation carries none of its code)
template <bool DYN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(O_THREADS, 1)
tc_out_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmY, const __grid_constant__ PeerMaps pm, OutParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[P_STAGES], bar_empty[P_STAGES], bar_tfull[2], bar_tempty[2], bar_sched[P_SCHED];
  __shared__ int tile_ring[P_SCHED];
  __shared__ uint32_t tmem_base_s;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t rank = cluster_ctarank();
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  constexpr bool dyn = DYN;
  griddep_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) { mbar_init(smem_u32(&bar_full[s]), 1); mbar_init(smem_u32(&bar_empty[s]), 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_tfull[s]), 1); mbar_init(smem_u32(&bar_tempty[s]), 2 * O_EPI_WARPS); }
    if (dyn)
      for (int s = 0; s < P_SCHED; ++s) mbar_init(smem_u32(&bar_sched[s]), 1);
    fence_mbar_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    prefetch_tmap(&tmY);
  }
  if (warp == 2) { tmem_alloc_pair(smem_u32(&tmem_base_s), 512); tmem_relinquish_pair(); }
  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // both CTAs' barriers are initialised before anyone signals across the pair
  cluster_wait();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  // everything above is independent of the kernel that produces A.  With the tile-by-tile hand-over this kernel does not
  // wait for that kernel to complete: rows of A are released through p.ready, and nothing else of the producer is read.
  if (!dyn) griddep_wait();
#ifdef TMOE_TRACE
  unsigned long long tr_t0; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(tr_t0));
  long long tr_flag = 0, tr_draw = 0; int tr_tiles = 0;
#endif

  const int num_tiles = p.num_m * p.num_n;  // num_m counts 256-row tiles here
  const int KB = (p.K + OKB - 1) / OKB;
#ifdef TMOE_TRACE
  const long long trace_t0 = clock64();
  long long trace_tic = 0;
#endif

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      bool all_rows = false;                 // the producing kernel was seen complete: no further per-tile checks
      unsigned long long pending = 0;        // result of the draw issued one tile ago
      for (uint32_t i = 0; ok; ++i) {
        int tile;
        const uint32_t slot = i % P_SCHED;
        if (!dyn) {
          tile = pair_id + (int)i * num_pairs;
          if (tile >= num_tiles) break;
        } else if (rank == 0) {
#ifdef TMOE_TRACE
          const long long c0_ = clock64();
#endif
          tile = i == 0 ? draw_ticket(p.queue, p.epoch, num_tiles, p.status) : ticket_of(pending, p.epoch, num_tiles);
          if (tile >= 0) pending = draw_next(p.queue);   // the next tile's ticket, on its way while this tile is loaded
#ifdef TMOE_TRACE
          tr_draw += clock64() - c0_; tr_tiles += tile >= 0;
#endif
          tile_ring[slot] = tile;
          st_cluster_u32(mapa_u32(smem_u32(&tile_ring[slot]), 1), (uint32_t)tile);
          mbar_arrive(smem_u32(&bar_sched[slot]));
          mbar_arrive_cluster(mapa_u32(smem_u32(&bar_sched[slot]), 1));
          if (tile < 0) break;
        } else {
          if (!(ok = mbar_wait_cluster(smem_u32(&bar_sched[slot]), (i / P_SCHED) & 1, p.status, kKernelOutPair, 5))) break;
          tile = *reinterpret_cast<volatile int *>(&tile_ring[slot]);
          if (tile < 0) break;
        }
        const int m0 = (tile / p.num_n) * (2 * OM) + (int)rank * OM;
        const int n0 = (tile % p.num_n) * ON + (int)rank * (ON / 2);
        // this CTA's 128 rows of A: wait until the CTA that produces them has stored them (rows beyond T do not exist)
#ifdef TMOE_TRACE
        const long long c1_ = clock64();
#endif
        if (dyn && !all_rows && m0 < p.T) {
          // one word says whether the whole producing grid is done (true for every pair that becomes resident after it)
          unsigned long long d;
          asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(d) : "l"(p.queue + 1) : "memory");
          if ((uint32_t)(d >> 32) == p.epoch && (uint32_t)d >= (uint32_t)p.n_producers) {
            all_rows = true;
            asm volatile("fence.proxy.async;" ::: "memory");
          } else if (!(ok = rows_ready_wait(p.ready + (m0 / OM) * 8, p.epoch, p.status))) {
            break;
          }
        }
#ifdef TMOE_TRACE
        tr_flag += clock64() - c1_;
#endif
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const uint32_t s = it % P_STAGES, ph = (it / P_STAGES) & 1;
          TMOE_TIC();
          if (!(ok = mbar_wait(smem_u32(&bar_empty[s]), ph ^ 1, p.status, kKernelOutPair, 2))) break;
          TMOE_TOC(0);
          const uint32_t full0 = mapa_u32(smem_u32(&bar_full[s]), 0);
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&bar_full[s]), 2 * P_STAGE_BYTES);  // both CTAs' bytes
          const uint32_t sa = ring + s * P_STAGE_BYTES;
          tma_load_2d_pair(sa, &tmA, kb * OKB, m0, full0);
          tma_load_2d_pair(sa + O_A_BYTES, &tmB, kb * OKB, n0, full0);
        }
      }
#ifdef TMOE_TRACE
      if (dyn && rank == 0 && pair_id < 120) {   // per pair: start (ns, low bits), end, tiles, cycles in flag waits, cycles in draws
        unsigned long long t1_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1_));
        int32_t *o = p.status + 64 + pair_id * 5;
        o[0] = (int32_t)(uint32_t)tr_t0; o[1] = (int32_t)(uint32_t)t1_; o[2] = tr_tiles; o[3] = (int32_t)tr_flag; o[4] = (int32_t)tr_draw;
      }
#endif
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc_bf16(2 * OM, ON);
      const uint64_t desc0 = umma_desc_k_sw128(ring);
      uint32_t s = 0, ph = 0;
      for (uint32_t tcount = 0;; ++tcount) {
        if (dyn) {
          mbar_wait_or_exit(smem_u32(&bar_sched[tcount % P_SCHED]), (tcount / P_SCHED) & 1, p.status, kKernelOutPair, 5);
          if (*reinterpret_cast<volatile int *>(&tile_ring[tcount % P_SCHED]) < 0) break;
        } else if (pair_id + (int)tcount * num_pairs >= num_tiles) {
          break;
        }
        const uint32_t slot = tcount & 1, aph = (tcount >> 1) & 1;
        TMOE_TIC();
        mbar_wait_or_exit(smem_u32(&bar_tempty[slot]), aph ^ 1, p.status, kKernelOutPair, 4);
        TMOE_TOC(1);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + slot * ON;
        for (int kb = 0; kb < KB; ++kb) {
          TMOE_TIC();
          mbar_wait_or_exit(smem_u32(&bar_full[s]), ph, p.status, kKernelOutPair, 1);
          TMOE_TOC(2);
          const uint64_t da = desc0 + s * (uint32_t)(P_STAGE_BYTES >> 4), db = da + (O_A_BYTES >> 4);
          const uint32_t acc0 = kb != 0;
#pragma unroll
          for (int k = 0; k < OKB / 16; ++k) umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, acc0 | (uint32_t)(k != 0));
          umma_commit_pair(smem_u32(&bar_empty[s]), 3);
          if (++s == P_STAGES) { s = 0; ph ^= 1; }
        }
        umma_commit_pair(smem_u32(&bar_tfull[slot]), 3);
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
    const uint32_t stage_buf = ring + P_STAGES * P_STAGE_BYTES + ew * O_Y_BYTES;
    bool ok = true;
    for (uint32_t tcount = 0; ok; ++tcount) {
      int tile;
      if (dyn) {
        ok = mbar_wait_cluster(smem_u32(&bar_sched[tcount % P_SCHED]), (tcount / P_SCHED) & 1, p.status, kKernelOutPair, 5);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tile = *reinterpret_cast<volatile int *>(&tile_ring[tcount % P_SCHED]);
      } else {
        tile = pair_id + (int)tcount * num_pairs;
        if (tile >= num_tiles) tile = -1;
      }
      if (tile < 0) break;
      const int m0 = (tile / p.num_n) * (2 * OM) + (int)rank * OM, n0 = (tile % p.num_n) * ON;
      const uint32_t slot = tcount & 1, aph = (tcount >> 1) & 1;
      const float4 bias_lane = load_bias_lane(p, n0 + half * 128, lane);
      TMOE_TIC();
      ok = mbar_wait(smem_u32(&bar_tfull[slot]), aph, p.status, kKernelOutPair, 3);
      if (threadIdx.x == 64) TMOE_TOC(5);  // epilogue warp 2 waiting for a finished accumulator
      ok = __all_sync(0xffffffffu, ok);  // the TMEM loads below are warp-collective
      if (!ok) break;
      tc_fence_after();
      const int64_t row = (int64_t)m0 + row_in_tile;
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + slot * ON + half * 128;
#pragma unroll 1
      for (int cc = 0; cc < 2; ++cc) {
        const int col0 = n0 + half * 128 + cc * 64;
        uint32_t r[2][32];
        TMOE_TIC();
        tmem_ld32(t_row + cc * 64, r[0]);
        tmem_ld32(t_row + cc * 64 + 32, r[1]);
        tmem_ld_wait(r[0], r[1]);
        if (threadIdx.x == 64) TMOE_TOC(3);  // epilogue warp 2: TMEM load round trip
        if (cc == 1) {  // this warp has read its whole share of the accumulator
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(mapa_u32(smem_u32(&bar_tempty[slot]), 0));  // the MMA thread lives in CTA 0
        }
        TMOE_TIC();
        if (lane == 0) tma_store_wait_read<0>();  // the previous store has finished reading the staging tile
        if (threadIdx.x == 64) TMOE_TOC(4);  // epilogue warp 2 waiting for its previous TMA store
        __syncwarp();
        TMOE_TIC();
        out_epilogue_chunk(p, r, col0, row, lane, stage_buf, bias_lane, cc * 64);
        fence_proxy_async_smem();
        __syncwarp();
        if (threadIdx.x == 64) TMOE_TOC(6);  // epilogue warp 2: bias / tail / staging of one 64-column chunk
        if (lane == 0 && col0 < p.N) store_tile_everywhere(&tmY, &pm, p.n_peers, stage_buf, col0, m0 + quad * 32, p.stream_y != 0);
      }
    }
    if (lane == 0) tma_store_wait_all();
  }
#ifdef TMOE_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 64) p.status[40 + 7] = (int32_t)(clock64() - trace_t0);
#endif
  tc_fence_before();
  __syncthreads();
  cluster_arrive();   // the other CTA may still be reading this CTA's shared memory or signalling its barriers
  cluster_wait();
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

// Launch that may begin while the previous kernel of the stream is draining (programmatic dependent launch): the GEMM
// kernels do their set-up, then griddep_wait() before they touch anything another kernel produced.
template <typename Kern>
static cudaError_t launch_dependent(Kern kern, int grid, int smem, cudaStream_t st, const CUtensorMap &a, const CUtensorMap &b,
                                    const CUtensorMap &y, const PeerMaps &pm, const OutParams &p) {
  static const bool off = []() { const char *e = getenv("TMOE_PDL"); return e && atoi(e) == 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(O_THREADS); cfg.dynamicSmemBytes = (size_t)smem; cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = off ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, a, b, y, pm, p);
}

// CTA pairs for GEMMs with at least two 256x256 tiles per pair of SMs (each CTA then streams 32 KB instead of 48 KB per
// k block and the ring is six stages deep: 112 us against 119 us on the prefill configuration); smaller GEMMs keep the
// single-CTA kernel, whose 128-row tiles cover more SMs.  TMOE_OUT_PAIRS=0 / 1 forces the choice.
// An output beyond this size cannot stay in the 126 MB L2 next to the operands: it is stored with the evict-first hint.
constexpr int64_t kStreamYBytes = 96ll << 20;

bool tc_gemm_uses_pairs(int64_t M, int N, int sms) {
  static const int pairs_env = []() { const char *e = getenv("TMOE_OUT_PAIRS"); return e ? (atoi(e) != 0 ? 1 : 0) : -1; }();
  const int64_t tiles256 = ((M + 2 * OM - 1) / (2 * OM)) * ((N + ON - 1) / ON);
  return pairs_env >= 0 ? pairs_env == 1 : tiles256 >= 2 * (int64_t)(sms / 2);
}

// Whether a forward of T tokens hands its z rows to the out-projection tile by tile (see tc_out_pair_kernel): the token
// tiles need more than one wave of CTAs, the out-projection runs on CTA pairs, programmatic dependent launch is on, and the
// caller asked for it with TMOE_HANDOFF=1 (read on every call, so a process can switch it).  Off by default: measured on the
// prefill configuration (256 token tiles on 148 SMs) the hand-over works as designed -- 14 pairs start 45 us early on the
// SMs of fully free TPCs and finish 5-6 tiles each before the last wave of token tiles ends, the tiles are drawn evenly --
// but a forward takes 223 us with it against 215 us without: every tile pays for its ticket and its ready words (the
// producer thread of this GEMM has no slack: 7.1 us per tile against 6.6 us), and the SMs it fills were idle on a
// power-capped part, where the busy ones clock higher for it.
bool plan_out_handoff(const tmoe_layer_t &L, int64_t T, int sms) {
  static const bool pdl_off = []() { const char *e = getenv("TMOE_PDL"); return e && atoi(e) == 0; }();
  const char *on = getenv("TMOE_HANDOFF");
  if (!on || atoi(on) != 1 || pdl_off || sms <= 0) return false;
  const int64_t token_tiles = (T + OM - 1) / OM;
  return token_tiles > sms && tc_gemm_uses_pairs(T, L.d_out, sms);
}

// y[M, N] (bf16) = A[M, K] (bf16, row-major) @ B_t[N, K]^T (bf16, K-major) + bias[N] (fp32, optional),
// then the optional OutEpilogue tail.  N and K multiples of 8.  `flags` (optional): tile-by-tile hand-over from the kernel
// that produces A; only honoured on the CTA-pair kernel (the caller asks plan_out_handoff first).
int launch_tc_gemm_bf16(const void *A, const void *B_t, const float *bias, const OutEpilogue &epi, int64_t M, int N,
                        int K, void *y, int32_t *status, cudaStream_t st, const OutFlags *flags) {
  CUtensorMap tmA, tmB, tmY;
  int rc = encode_tmap_bf16_2d(&tmY, y, (uint64_t)M, (uint64_t)N, 32);
  if (rc) return rc;
  rc = encode_tmap_bf16_2d(&tmA, A, (uint64_t)M, (uint64_t)K, OM);
  if (rc) return rc;
  rc = encode_tmap_bf16_2d(&tmB, B_t, (uint64_t)N, (uint64_t)K, ON);
  if (rc) return rc;
  PeerMaps pm;
  for (int i = 0; i < TMOE_MAX_PEERS; ++i) {   // unused entries repeat y's map: every entry is a valid descriptor
    if (i < epi.n_peers) {
      if ((rc = encode_tmap_bf16_2d(&pm.m[i], epi.peer_y[i], (uint64_t)M, (uint64_t)N, 32))) return rc;
    } else {
      pm.m[i] = tmY;
    }
  }
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return TMOE_ERR_CUDA;
  const int sms = current_device_sms();
  if (sms <= 0) return TMOE_ERR_CUDA;
  if (dev < 64 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(tc_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, O_SMEM_BYTES) != cudaSuccess)
      return TMOE_ERR_CUDA;
    attr_done[dev] = true;
  }
  const bool use_pairs = tc_gemm_uses_pairs(M, N, sms);
  if (flags && !use_pairs) return TMOE_ERR_UNSUPPORTED;
  if (use_pairs) {
    static bool attr2_done[64] = {};
    if (dev < 64 && !attr2_done[dev]) {
      if (cudaFuncSetAttribute(tc_out_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess ||
          cudaFuncSetAttribute(tc_out_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_SMEM_BYTES) != cudaSuccess)
        return TMOE_ERR_CUDA;
      attr2_done[dev] = true;
    }
    CUtensorMap tmBh;
    rc = encode_tmap_bf16_2d(&tmBh, B_t, (uint64_t)N, (uint64_t)K, ON / 2);
    if (rc) return rc;
    OutParams q{};
    q.y = (bf16 *)y; q.bias = bias; q.residual = (const bf16 *)epi.residual; q.gamma = (const bf16 *)epi.layer_scale;
    q.silu_gate = (const bf16 *)epi.silu_gate;
    q.T = M; q.N = N; q.K = K;
    q.num_m = (int)((M + 2 * OM - 1) / (2 * OM)); q.num_n = (N + ON - 1) / ON;
    q.status = status;
    q.n_peers = epi.n_peers;
    q.stream_y = (int64_t)M * N * 2 > kStreamYBytes;
    if (flags) {
      q.ready = flags->ready; q.epoch = flags->epoch; q.queue = flags->queue;
      q.n_producers = (int)((M + OM - 1) / OM);
    }
    const int tiles2 = q.num_m * q.num_n;
    // a persistent grid must be fully co-resident: ask how many 2-CTA clusters the device can hold at once
    static int max_pairs[64] = {};
    if (dev < 64 && max_pairs[dev] == 0) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * (sms / 2)); cfg.blockDim = dim3(O_THREADS); cfg.dynamicSmemBytes = P_SMEM_BYTES;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
      cfg.attrs = at; cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, tc_out_pair_kernel<false>, &cfg) != cudaSuccess || n <= 0) return TMOE_ERR_CUDA;
      max_pairs[dev] = n;
    }
    int pairs = dev < 64 ? max_pairs[dev] : sms / 2;
    if (tiles2 < pairs) pairs = tiles2;
    const cudaError_t le = flags ? launch_dependent(tc_out_pair_kernel<true>, 2 * pairs, P_SMEM_BYTES, st, tmA, tmBh, tmY, pm, q)
                                 : launch_dependent(tc_out_pair_kernel<false>, 2 * pairs, P_SMEM_BYTES, st, tmA, tmBh, tmY, pm, q);
    if (le != cudaSuccess) return TMOE_ERR_CUDA;
    count_launch();
    return launch_status();
  }
  OutParams p{};
  p.y = (bf16 *)y; p.bias = bias; p.residual = (const bf16 *)epi.residual; p.gamma = (const bf16 *)epi.layer_scale;
  p.silu_gate = (const bf16 *)epi.silu_gate;
  p.T = M; p.N = N; p.K = K;
  p.num_m = (int)((M + OM - 1) / OM); p.num_n = (N + ON - 1) / ON;
  p.on = ON;
  // few token rows: 128-column tiles put twice as many SMs to work (each CTA then streams half of B per k block);
  // and an output of at most 128 columns (the router-scores GEMM at E <= 128) never needs the wide tile
  static const int narrow_env = [] { const char *e = getenv("TMOE_OUT_NARROW"); return e ? atoi(e) : 1; }();
  if (narrow_env && (N <= ON / 2 || (int64_t)p.num_m * p.num_n * 2 <= sms)) {
    p.on = ON / 2;
    p.num_n = (N + p.on - 1) / p.on;
    if ((rc = encode_tmap_bf16_2d(&tmB, B_t, (uint64_t)N, (uint64_t)K, (uint32_t)p.on))) return rc;
  }
  p.status = status;
  p.n_peers = epi.n_peers;
  p.stream_y = (int64_t)M * N * 2 > kStreamYBytes;
  const int tiles = p.num_m * p.num_n;
  const int grid = tiles < sms ? tiles : sms;
  if (launch_dependent(tc_out_kernel, grid, O_SMEM_BYTES, st, tmA, tmB, tmY, pm, p) != cudaSuccess) return TMOE_ERR_CUDA;
  count_launch();
  return launch_status();
}

int launch_tc_out(const tmoe_layer_t &L, const void *z, const void *uout_t, const float *bias, const OutEpilogue &epi,
                  int64_t T_, void *y, int32_t *status, cudaStream_t st, const OutFlags *flags) {
  return launch_tc_gemm_bf16(z, uout_t, bias, epi, T_, L.d_out, L.r2, y, status, st, flags);
}

}  // namespace tmoe
