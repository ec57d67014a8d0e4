// In-projection, router scores, inner RMSNorm statistics and core contraction in one kernel
// (subsystem 2, with subsystem 1 folded in when the expert count allows):
//
//   phase A   acc_h[128, r3]  = x_tile[128, d_in] @ U_in            (model.py:80)
//             acc_s[128, E]   = x_tile @ router_w^T                 (model.py:75; same A operand)
//   epilogue A (thread = token row, TMEM -> registers)
//             top-k on the bf16-rounded scores, softmax over the winners, c = sum g_k U_expert[e_k]
//             (model.py:76-77, 93); sum of squares of the row of h; h*w -> bf16 -> shared memory in
//             the K-major 128-byte-swizzled layout the MMA reads; c *= 1/sqrt(mean(h^2)+eps)
//             (the RMSNorm scale of model.py:25-27 commutes with the linear core contraction, so it
//             is applied to the r1 coefficients instead of the r3 values of h)
//   phase B   for every r2 tile j (n2 = 256/r1 columns):
//             P[128, r1*n2] = h[128, r3] @ G_j   with the r1 core slices of the tile side by side
//   epilogue B z[t, j*n2 + s] = sum_a c[t,a] * P[t, a*n2 + s]  in registers -> bf16 -> 16-byte stores
//             (model.py:95-98 for all selected experts at once); P is double-buffered in TMEM so
//             this runs under the next tile's MMAs and the [T, r1*r2] intermediate never leaves the SM.
//
// One CTA per 128-token tile, 10 warps: TMA producer, MMA issuer, 8 epilogue warps.
// Shared memory: phase A uses a ring of {x tile, U_in^T tile, router tile} stages over the whole
// 224 KB; after the last phase-A MMA has completed, the first r3/64 * 16 KB become h and the rest becomes a
// ring of 32 KB core tiles (5 stages for r3 <= 256, 3 for r3 = 512; z leaves the SM as 16-byte stores
// straight from registers).  r3 = 512 fills all 512 TMEM columns with h, so the router scores then come
// from a separate GEMM launch.
// All mbarrier waits are bounded.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include "routing.cuh"

namespace tmoe {

using namespace ptx;

// Optional per-CTA phase timestamps (build with -DTMOE_TRACE): clock64 deltas from kernel start are written to
// status words [16 + 8*slot ...] by blocks 0 and gridDim.x-1.  Off in normal builds.
#ifdef TMOE_TRACE
#define TMOE_STAMP(i)                                                                       \
  do {                                                                                      \
    if (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)                                     \
      p.status[16 + (blockIdx.x == 0 ? 0 : 8) + (i)] = (int32_t)(clock64() - trace_t0);     \
  } while (0)
#else
#define TMOE_STAMP(i) do { } while (0)
#endif

constexpr int TM = 128;                    // tokens per CTA
constexpr int X_TILE_BYTES = TM * 64 * 2;  // 16 KB
constexpr int H_KBLOCK_BYTES = TM * 64 * 2;
constexpr int G_STAGE_BYTES = 256 * 64 * 2;         // 32 KB
constexpr int G_STAGES_MAX = 5;  // core-tile stages: (224 KB - h) / 32 KB -> 5 for r3 <= 256, 3 for r3 = 512
constexpr int IC_EPI_WARPS = 8;
constexpr int IC_THREADS = (2 + IC_EPI_WARPS) * 32;
constexpr int IC_RING_BYTES = 224 * 1024;
constexpr int IC_SMEM_BYTES = IC_RING_BYTES + 1024;
constexpr int A_STAGES_MAX = 8;   // 4 stages fit at r3 = 256 (48-56 KB each); layers with a narrower U_in tile get up to 8
constexpr int SCORE_COL = 256;  // TMEM column of the router scores during phase A
constexpr int kKernelInCore = 2;

struct InCoreParams {
  int64_t T;
  int d_in, r3, r2, E, e_pad, top_k, n_tiles2;
  float eps;
  int fuse_router;
  int pre_norm;        // 1: apply the callers' RMSNorm to x in-kernel (its weight is folded into the prepared U_in / router rows)
  float pre_norm_eps;
  RouterCfg rc;  // gate rule (tmoe_layer_t::router_mode)
  const float *normw;  // [r3]
  const float *uexp;   // [E, r1] fp32
  const float *c_in;   // [T, r1] when !fuse_router
  float *c_work;       // [T, r1] scratch: c scaled by 1/rms, handed from the routing warps to their twins
  int32_t *idx_out;
  float *gates_out;
  float *c_out;
  bf16 *z;  // [T, r2]
  int z_wide;  // z is 32-byte aligned (r2 is a multiple of 64, so every 16-column group then is): 256-bit stores
  int32_t *status;
  // ready != nullptr: every epilogue warp raises ready[8 * token tile + warp] = epoch once its z rows are stored (the
  // out-projection's CTA pairs pick the tile up from there; j_split == 1 in that case)
  // Few token tiles (small T): every tile is shared by j_split CTAs, each repeating phase A and taking n_tiles2 / j_split of
  // the core tiles, so that one tile's 40 us of work is spread over up to 16 SMs.  Split s > 0 keeps its c hand-off in
  // block s + 1 of c_work ([T, r1] each); block 0 may alias c_in / c_out.
  int j_split;
  uint32_t *ready;
  uint32_t epoch;
  unsigned long long *queue;   // the out-projection's tile queue word, tagged here with this forward's epoch
  int pair;                    // 1: the grid interleaves two layers on the same x (second parameter block / tensor maps)
};

// Phase-A issue loop of the MMA thread.  TWO_BOX: r3 = 512; a stage holding x and all 512 rows of U_in^T is 80 KB, two
// stages deep, and starves (measured 2300 cycles per k block against 1024 of tensor-pipe time), so h is made in two passes
// over K, each streaming x again (from L2) with one 256-row piece of U_in^T: 48 KB stages, four deep.  SCORES: the router
// tile follows U_in^T in the stage and a second, N = e_pad MMA accumulates the scores at TMEM column SCORE_COL.
template <bool TWO_BOX, bool SCORES>
__device__ __forceinline__ void issue_phase_a(uint32_t tmem_base, uint64_t desc0, uint32_t stage16, uint32_t u16, int KA, int nA,
                                              int u_box_rows, int e_pad, uint64_t *bar_full, uint64_t *bar_empty, int32_t *status) {
  const uint32_t idescH = umma_idesc_bf16(TM, u_box_rows);
  const uint32_t idescS = umma_idesc_bf16(TM, e_pad);
  constexpr uint32_t xtile16 = X_TILE_BYTES >> 4;
  uint32_t sA = 0, phA = 0;
#pragma unroll 1
  for (int pass = 0; pass < (TWO_BOX ? 2 : 1); ++pass) {
    const uint32_t d_h = tmem_base + pass * 256;
    for (int kb = 0; kb < KA; ++kb) {
      mbar_wait_or_exit(smem_u32(&bar_full[sA]), phA, status, kKernelInCore, 1);
      const uint64_t dx = desc0 + sA * stage16, du = dx + xtile16, dw = du + u16;
      const uint32_t acc0 = kb != 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t acc = acc0 | (uint32_t)(k != 0);
        umma_bf16(d_h, dx + 2 * k, du + 2 * k, idescH, acc);
        if (SCORES) umma_bf16(tmem_base + SCORE_COL, dx + 2 * k, dw + 2 * k, idescS, acc);
      }
      umma_commit(smem_u32(&bar_empty[sA]));
      if (++sA == (uint32_t)nA) { sA = 0; phA ^= 1; }
    }
  }
}

// R1: Tucker rank r1 (core slices per r2 tile); RK: capacity of the in-kernel top-k list (>= top_k)
template <int R1, int RK>
__global__ void __launch_bounds__(IC_THREADS, 1)
tc_in_core_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmU1,
                  const __grid_constant__ CUtensorMap tmW1, const __grid_constant__ CUtensorMap tmG1,
                  const __grid_constant__ InCoreParams pa, const __grid_constant__ CUtensorMap tmU2,
                  const __grid_constant__ CUtensorMap tmW2, const __grid_constant__ CUtensorMap tmG2,
                  const __grid_constant__ InCoreParams pb) {
  constexpr int N2 = 256 / R1;
  extern __shared__ uint8_t smem_raw[];
  // Two layers on one input (pa.pair: the FFN's gate and up projections, model.py:337-339): CTA 2m works on token tile m
  // for the first layer, CTA 2m + 1 on the same tile for the second -- neighbours in launch order, so the tile of x that one
  // of them brings in from HBM is in L2 for the other.  Everything below runs on this CTA's own copy of the parameters.
  const bool second = pa.pair && (blockIdx.x & 1u);
  const InCoreParams p = second ? pb : pa;
  const CUtensorMap *const tU = second ? &tmU2 : &tmU1;
  const CUtensorMap *const tW = second ? &tmW2 : &tmW1;
  const CUtensorMap *const tG = second ? &tmG2 : &tmG1;
  const int bid = pa.pair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  // every CTA of this grid is running once the last one has said this: the next kernel of the stream (the out-projection)
  // may then take SMs as they free up -- to do its set-up while this grid drains or, with the tile-by-tile hand-over, to
  // start on the token tiles that are already finished
  griddep_launch_dependents();
  __shared__ __align__(8) uint64_t bar_fullA[A_STAGES_MAX], bar_emptyA[A_STAGES_MAX], bar_fullB[G_STAGES_MAX],
      bar_emptyB[G_STAGES_MAX], bar_accA, bar_hready, bar_pfull[2], bar_pempty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ float inv_rms_s[TM];
  __shared__ __align__(16) bf16 wnorm_s[512];  // inner_norm weight; the layer is bf16, so this copy is exact

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int sp = p.j_split > 1 ? bid % p.j_split : 0;
  const int m0 = (p.j_split > 1 ? bid / p.j_split : bid) * TM;
  const int jn = p.n_tiles2 / p.j_split, j0 = sp * jn;   // this CTA's core tiles [j0, j0 + jn)
  float *const c_work = p.c_work + (p.j_split > 1 ? (int64_t)(sp + 1) * p.T * R1 : 0);

  const int u_boxes = (p.r3 + 255) / 256;         // U_in^T is streamed in pieces of <= 256 rows, one pass over K per piece
  const int u_box_rows = p.r3 / u_boxes;
  const int u_bytes = u_box_rows * 128, w_bytes = p.e_pad * 128;
  const int stageA_bytes = X_TILE_BYTES + u_bytes + w_bytes;
  int nA = IC_RING_BYTES / stageA_bytes;
  nA = nA > A_STAGES_MAX ? A_STAGES_MAX : nA;
  const int KA = p.d_in / 64;
  const int KH = p.r3 / 64;                       // 64-wide k blocks of h
  const int h_bytes = KH * H_KBLOCK_BYTES;        // 64 KB for r3 = 256, 128 KB for r3 = 512
  int nG = (IC_RING_BYTES - h_bytes) / G_STAGE_BYTES;
  nG = nG > G_STAGES_MAX ? G_STAGES_MAX : nG;

  for (int i = threadIdx.x; i < p.r3; i += blockDim.x) wnorm_s[i] = __float2bfloat16_rn(p.normw[i]);
  if (threadIdx.x == 0) {
    // a phase-A stage is free once its MMAs have retired and, with the in-kernel pre-norm, the four secondary
    // warps have read its x tile for the row statistics
    for (int s = 0; s < A_STAGES_MAX; ++s) { mbar_init(smem_u32(&bar_fullA[s]), 1); mbar_init(smem_u32(&bar_emptyA[s]), p.pre_norm ? 5 : 1); }
    for (int s = 0; s < G_STAGES_MAX; ++s) { mbar_init(smem_u32(&bar_fullB[s]), 1); mbar_init(smem_u32(&bar_emptyB[s]), 1); }
    mbar_init(smem_u32(&bar_accA), 1);
    // h is staged (and its TMEM columns free) once all eight warps have said so (each stages half of a row's columns); the score columns, which lie in
    // accumulator slot 1, are released through bar_pempty[1] (see the MMA thread's wait).  An accumulator slot is handed
    // back by all eight warps: the four that read it, and the four that only watched its 'full' barrier, so that the MMA
    // thread can never complete that barrier twice before a slow watcher has seen the first completion
    mbar_init(smem_u32(&bar_hready), IC_EPI_WARPS);
    for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&bar_pfull[s]), 1); mbar_init(smem_u32(&bar_pempty[s]), IC_EPI_WARPS); }
    fence_mbar_init();
    prefetch_tmap(&tmX);
    prefetch_tmap(tU);
    prefetch_tmap(tG);
    if (p.e_pad) prefetch_tmap(tW);
  }
  if (warp == 2) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }  // an epilogue warp: its lanes never retire early
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t ringB = ring + h_bytes;
  // this kernel may have been started while its predecessor in the stream drains: nothing above depends on that kernel,
  // everything below may (x, and the z / c rows this kernel overwrites may still be read by it)
  griddep_wait();
  if (p.queue && bid == 0 && !second && threadIdx.x == 0) {
    // tile queue of the out-projection that follows: this forward's epoch, no tile handed out yet.  No CTA of that kernel
    // can run before every CTA of this grid has started, and those of the last wave start only when CTAs that are past
    // this point have finished.
    *reinterpret_cast<volatile unsigned long long *>(p.queue) = (unsigned long long)p.epoch << 32;
    *reinterpret_cast<volatile unsigned long long *>(p.queue + 1) = (unsigned long long)p.epoch << 32;   // CTAs of this grid that are done
    __threadfence();
  }
#ifdef TMOE_TRACE
  const long long trace_t0 = clock64();
  unsigned long long trace_ns0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(trace_ns0));
#endif

  if (warp == 0) {
    // ------------------------------- TMA producer -------------------------------
    if (lane == 0) {
      bool ok = true;
      uint32_t sA = 0, phA = 0, sB = 0, phB = 0;
      // x is read once (with r3 = 512 twice, the second time from L2: no hint then): its lines are the first to go, so that
      // z -- which the out-projection reads next -- and the factors stay in L2 (200.9 -> 198.4 us per forward at the prefill
      // configuration; marking the z stores or the factor tiles evict-last on top of that changed nothing)
      const uint64_t pol_x = u_boxes == 1 ? l2_policy_evict_first() : l2_policy_evict_normal();
      for (int pass = 0; pass < u_boxes && ok; ++pass) {
        for (int kb = 0; kb < KA && ok; ++kb) {
          const uint32_t s = sA, ph = phA;
          if (++sA == (uint32_t)nA) { sA = 0; phA ^= 1; }  // ring position kept incrementally: no division in this loop
          if (!(ok = mbar_wait(smem_u32(&bar_emptyA[s]), ph ^ 1, p.status, kKernelInCore, 2))) break;
          const uint32_t full = smem_u32(&bar_fullA[s]);
          mbar_arrive_expect_tx(full, stageA_bytes);
          const uint32_t sa = ring + s * stageA_bytes;
          tma_load_2d_hint(sa, &tmX, kb * 64, m0, full, pol_x);
          tma_load_2d(sa + X_TILE_BYTES, tU, kb * 64, pass * u_box_rows, full);
          if (p.e_pad) tma_load_2d(sa + X_TILE_BYTES + u_bytes, tW, kb * 64, 0, full);
        }
      }
      // ring A aliases h and the core-tile ring: wait until every phase-A MMA has retired
      if (ok) ok = mbar_wait(smem_u32(&bar_accA), 0, p.status, kKernelInCore, 3);
      const int total = jn * KH;
      int j = j0, kbB = 0;
      for (int it = 0; it < total && ok; ++it) {
        const uint32_t s = sB, ph = phB;
        if (++sB == (uint32_t)nG) { sB = 0; phB ^= 1; }
        const int kb = kbB;
        const int row0 = j * 256;
        if (++kbB == KH) { kbB = 0; ++j; }
        if (!(ok = mbar_wait(smem_u32(&bar_emptyB[s]), ph ^ 1, p.status, kKernelInCore, 6))) break;
        const uint32_t full = smem_u32(&bar_fullB[s]);
        mbar_arrive_expect_tx(full, G_STAGE_BYTES);
        tma_load_2d(ringB + s * G_STAGE_BYTES, tG, kb * 64, row0, full);
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      // This thread is the serial path of the kernel (see mbar_wait_or_exit): the loops below have fixed trip
      // counts and no side exits, ring positions and descriptors are kept incrementally, and the shape variants of
      // phase A are separate loops so that no MMA sits behind a run-time condition (each of those was measured in a
      // replica of this loop: a conditional MMA costs ~43 cycles even when skipped, a `break` ~100 per k block).
      // No tcgen05 fence after a "tiles landed" wait: the mbarrier completion orders the TMA writes before the MMA
      // reads; the fence is only needed where another thread's tcgen05.ld preceded (accumulator / h hand-offs).
      const uint64_t desc0 = umma_desc_k_sw128(ring);          // descriptor of the ring base; tiles add (bytes >> 4)
      const uint32_t stageA16 = (uint32_t)stageA_bytes >> 4;
      if (p.e_pad)
        issue_phase_a<false, true>(tmem_base, desc0, stageA16, (uint32_t)u_bytes >> 4, KA, nA, u_box_rows, p.e_pad, bar_fullA, bar_emptyA, p.status);
      else if (u_boxes == 2)
        issue_phase_a<true, false>(tmem_base, desc0, stageA16, (uint32_t)u_bytes >> 4, KA, nA, u_box_rows, 16, bar_fullA, bar_emptyA, p.status);
      else
        issue_phase_a<false, false>(tmem_base, desc0, stageA16, (uint32_t)u_bytes >> 4, KA, nA, u_box_rows, 16, bar_fullA, bar_emptyA, p.status);
      umma_commit(smem_u32(&bar_accA));
      TMOE_STAMP(0);  // last phase-A MMA issued
      mbar_wait_or_exit(smem_u32(&bar_hready), 0, p.status, kKernelInCore, 4);
      tc_fence_after();
      TMOE_STAMP(1);  // MMA thread saw h ready
      const uint32_t idescP = umma_idesc_bf16(TM, 256);
      const uint64_t descB0 = desc0 + ((uint32_t)h_bytes >> 4);
      uint32_t sB = 0, phB = 0;
      for (int j = 0; j < jn; ++j) {
        const uint32_t slot = j & 1, pph = (j >> 1) & 1;
        // slot 0 is free from the start (parity trick); slot 1 holds the router scores first, so its first wait is for a
        // real arrival of the routing warps and its parity runs one phase ahead of slot 0's
        mbar_wait_or_exit(smem_u32(&bar_pempty[slot]), pph ^ 1 ^ slot, p.status, kKernelInCore, 8);
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + slot * 256;
        for (int kb = 0; kb < KH; ++kb) {
          mbar_wait_or_exit(smem_u32(&bar_fullB[sB]), phB, p.status, kKernelInCore, 5);
          const uint64_t dh = desc0 + kb * (H_KBLOCK_BYTES >> 4);
          const uint64_t dg = descB0 + sB * (G_STAGE_BYTES >> 4);
          const uint32_t acc0 = kb != 0;
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(d_tmem, dh + 2 * k, dg + 2 * k, idescP, acc0 | (uint32_t)(k != 0));
          umma_commit(smem_u32(&bar_emptyB[sB]));
          if (++sB == (uint32_t)nG) { sB = 0; phB ^= 1; }
        }
        umma_commit(smem_u32(&bar_pfull[slot]));
      }
    }
  } else {
    // ------------------------------- epilogue warps -------------------------------
    // Eight warps: warp w may read TMEM lanes 32*(w%4)..+31, so each row quadrant has a "primary" warp
    // (2-5) and a "secondary" warp (6-9); thread = token row in both.
    //   epilogue A: both warps of a row stage half of its h columns each (sum of squares, h*w -> bf16 -> shared
    //               memory); then primary = routing (scores -> top-k -> gates -> c) while the first core tile runs; they
    //               meet at a named barrier, the primary scales c by the row's 1/rms and publishes it through the
    //               workspace for its secondary twin.
    //   epilogue B: the 64-column units of z alternate between the two groups, so each group has two MMA
    //               tile times per unit; each thread stores its row's columns as 16-byte pieces.
    const int quad = warp & 3;
    const int grp = (warp - 2) >> 2;  // 0 primary, 1 secondary
    const int row = quad * 32 + lane;
    const int64_t grow = (int64_t)m0 + row;
    const bool live = grow < p.T;
    const uint32_t t_lane = tmem_base + ((uint32_t)(quad * 32) << 16);
    float c[R1];
    bool ok = true;
    float inv_x = 1.f;  // 1 / rms(x row) when the callers' pre-norm is applied here
    float ss_half = 0.f;  // this warp's half of the row's sum of squares of h
    if (p.pre_norm && grp == 1) {
      // The secondary warps are idle during phase A: they follow the x tiles through the ring and accumulate
      // each row's sum of squares (the swizzle permutes 16-byte chunks inside a row, which a sum does not see).
      float ssx = 0.f;
      uint32_t sA = 0, phA = 0;
      for (int kb = 0; kb < KA && ok; ++kb) {
        const uint32_t s = sA, ph = phA;
        if (++sA == (uint32_t)nA) { sA = 0; phA ^= 1; }
        ok = mbar_wait(smem_u32(&bar_fullA[s]), ph, p.status, kKernelInCore, 9);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint32_t xrow = ring + s * stageA_bytes + row * 128;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          uint32_t w0, w1, w2, w3;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3)
                       : "r"(xrow + (uint32_t)((i ^ (row & 7)) * 16)));
          const uint32_t w[4] = {w0, w1, w2, w3};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float lo = __uint_as_float(w[q] << 16), hi = __uint_as_float(w[q] & 0xffff0000u);
            ssx = fmaf(lo, lo, ssx);
            ssx = fmaf(hi, hi, ssx);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_emptyA[s]));
      }
      inv_x = 1.f / sqrtf(ssx / (float)p.d_in + p.pre_norm_eps);
    }
    if (ok) ok = mbar_wait(smem_u32(&bar_accA), 0, p.status, kKernelInCore, 3);
    ok = named_bar_and(2, 256, ok);  // the eight epilogue warps continue or leave together
    if (ok) {
      tc_fence_after();
      if (threadIdx.x == 64) TMOE_STAMP(2);  // phase A complete (accumulators readable)
      if (p.pre_norm) {  // hand 1/rms(x) from the secondary warp of each row to its primary twin (through the workspace)
        if (grp == 1 && live) c_work[grow * R1] = inv_x;
        named_bar_sync(5, 256);
        if (grp == 0) inv_x = live ? c_work[grow * R1] : 1.f;
      }
      // h rows: both warps of a row quadrant stage half of the r3 columns each (statistics, weight, bf16, swizzled store:
      // 16-byte chunk index XOR row % 8 inside 128-byte rows), so that phase B can start after half the time one warp
      // would need; the primary warps do the routing afterwards, while the first core tile is already running.
      {
        const int ncc = p.r3 / 32, cc_lo = grp * (ncc / 2), cc_hi = cc_lo + ncc / 2;
        float ss = 0.f;
        for (int cc = cc_lo; cc < cc_hi; ++cc) {
          uint32_t r[32];
          tmem_ld32(t_lane + cc * 32, r);
          tmem_ld_wait(r);
          const uint32_t kblk_base = ring + (cc >> 1) * H_KBLOCK_BYTES + row * 128;
          // the 32 weights of this column group as four 16-byte broadcast loads, all ahead of the stores
          uint4 wq[4];
#pragma unroll
          for (int g = 0; g < 4; ++g) wq[g] = *reinterpret_cast<const uint4 *>(&wnorm_s[cc * 32 + g * 8]);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
            const uint32_t ww[4] = {wq[g].x, wq[g].y, wq[g].z, wq[g].w};
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float a = __uint_as_float(r[g * 8 + q]);
              ss = fmaf(a, a, ss);
              v[q] = a * __uint_as_float((q & 1) ? (ww[q >> 1] & 0xffff0000u) : (ww[q >> 1] << 16));
            }
            const uint32_t chunk = (uint32_t)((cc & 1) * 4 + g) ^ (uint32_t)(row & 7);
            const uint32_t addr = kblk_base + chunk * 16;
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pack_bf16x2(v[0], v[1])),
                         "r"(pack_bf16x2(v[2], v[3])), "r"(pack_bf16x2(v[4], v[5])), "r"(pack_bf16x2(v[6], v[7])));
            // no "memory" clobber: nothing the compiler sees touches the h tile, and the proxy fence below orders it
          }
        }
        ss_half = ss;
        if (grp == 1) inv_rms_s[row] = ss;   // the secondary warp's half of the sum of squares, for its primary twin
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(smem_u32(&bar_hready));   // 8 arrivals: h is in shared memory, its TMEM columns are free
          if (grp == 1) mbar_arrive(smem_u32(&bar_pempty[1]));  // this warp does not read the score columns
        }
      }
      if (grp == 0) {
        if (p.fuse_router) {
          // Running top-k over the score columns, branch-free.  A score rounded to bf16 has 16 significant
          // bits, so (order-preserving map of those bits) << 16 | (0xFFFF - expert) is a 32-bit key whose
          // unsigned order is "higher score first, equal scores -> lower expert index first"; the sorted
          // list is then maintained with integer max/min only (no data-dependent branches, independent
          // scores pipeline through the levels).
          uint32_t key[RK];
          const bool rule1 = p.rc.mode == 1;   // the top-k then orders by the tempered capped logit (RouterCfg::order_value)
#pragma unroll
          for (int j = 0; j < RK; ++j) key[j] = 0u;
          for (int cc = 0; cc < p.e_pad / 16; ++cc) {
            uint32_t r[16];
            tmem_ld16(t_lane + SCORE_COL + cc * 16, r);
            tmem_ld_wait(r);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              const int e = cc * 16 + q;
              uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(__uint_as_float(r[q]) * inv_x));
              if (rule1) b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(p.rc.logit(__uint_as_float(b << 16))));
              b = (b == 0x8000u) ? 0u : b;                                   // -0 and +0 compare equal
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
          float sv[RK]; int si[RK];
#pragma unroll
          for (int j = 0; j < RK; ++j) {
            const uint32_t u = key[j] >> 16;
            const uint32_t b = (u & 0x8000u) ? (u & 0x7fffu) : (~u & 0xffffu);
            sv[j] = __uint_as_float(b << 16);
            si[j] = (int)(0xffffu - (key[j] & 0xffffu));
          }
          if (threadIdx.x == 64) TMOE_STAMP(6);  // score scan done
          // capped-softmax rule only: denominator over ALL experts, relative to the top logit.  Kept out of the
          // scan above (a second pass over the score columns) so that the default rule's loop stays branch-free.
          float z_all = 1.f;
          if (p.rc.mode == 1) {
            const float l0 = sv[0];   // the list holds logits under this rule
            z_all = 0.f;
            for (int cc = 0; cc < p.e_pad / 16; ++cc) {
              uint32_t r[16];
              tmem_ld16(t_lane + SCORE_COL + cc * 16, r);
              tmem_ld_wait(r);
#pragma unroll
              for (int q = 0; q < 16; ++q) {
                const float sc = round_to<bf16>(__uint_as_float(r[q]) * inv_x);
                if (cc * 16 + q < p.E) z_all += expf(p.rc.logit(sc) - l0);
              }
            }
          }
          // last read of the score columns: accumulator slot 1 may be overwritten from here on
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[1]));
          float gate[RK];
          gates_of<bf16, RK>(sv, p.top_k, p.rc, z_all, gate);
#pragma unroll
          for (int a = 0; a < R1; ++a) c[a] = 0.f;
#pragma unroll
          for (int j = 0; j < RK; ++j) {
            if (j < p.top_k) {
              const int e = min(max(si[j], 0), p.E - 1);
#pragma unroll
              for (int a = 0; a < R1; ++a) {
                const float ue = __ldg(p.uexp + e * R1 + a);
                c[a] = fmaf(gate[j], ue, c[a]);
              }
              if (live && sp == 0) {
                if (p.idx_out) p.idx_out[grow * p.top_k + j] = si[j];
                if (p.gates_out) p.gates_out[grow * p.top_k + j] = gate[j];
              }
            }
          }
          if (threadIdx.x == 64) TMOE_STAMP(7);  // gates and c done
          if (live && p.c_out && sp == 0) {
#pragma unroll
            for (int a = 0; a < R1; ++a) p.c_out[grow * R1 + a] = c[a];
          }
        } else {
          if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[1]));   // no scores in TMEM: slot 1 is free at once
#pragma unroll
          for (int a = 0; a < R1; ++a) c[a] = live ? __ldg(p.c_in + grow * R1 + a) : 0.f;
        }
        if (threadIdx.x == 64) TMOE_STAMP(3);  // routing done
        tc_fence_before();                      // score columns are free for the core-tile accumulators
        named_bar_sync(3, 256);                 // the secondary warps have written their halves of the sums of squares
        // h = inv_x * h_raw: RMSNorm(h) = h_raw * inv_x / sqrt(inv_x^2 * mean(h_raw^2) + eps)
        const float ss_row = ss_half + inv_rms_s[row];
        const float inv_rms = inv_x / sqrtf(inv_x * inv_x * ss_row / (float)p.r3 + p.eps);
#pragma unroll
        for (int a = 0; a < R1; ++a) c[a] *= inv_rms;
        if (live) {
#pragma unroll
          for (int a = 0; a < R1; ++a) c_work[grow * R1 + a] = c[a];
        }
      } else {
        named_bar_sync(3, 256);
      }
      if (threadIdx.x == 64) TMOE_STAMP(4);  // epilogue A done
      named_bar_sync(4, 256);                // c_work of every row is written
      if (grp == 1) {
#pragma unroll
        for (int a = 0; a < R1; ++a) c[a] = live ? c_work[grow * R1 + a] : 0.f;
      }

      // epilogue B: tile j belongs to group (j / JPU) & 1, JPU = tiles per 64-column unit of z
      constexpr int JPU = (N2 >= 64) ? 1 : 64 / N2;
      [[maybe_unused]] uint4 held = make_uint4(0, 0, 0, 0);   // N2 = 8: the even tile's half of a 32-byte store
      for (int jl = 0; jl < jn && ok; ++jl) {
        // every warp waits for every tile, also the ones its group does not own: a parity wait is only
        // meaningful for a waiter that has seen the barrier's previous phase complete
        const int j = j0 + jl;
        const uint32_t slot = jl & 1, pph = (jl >> 1) & 1;
        ok = mbar_wait(smem_u32(&bar_pfull[slot]), pph, p.status, kKernelInCore, 7);
        ok = __all_sync(0xffffffffu, ok);  // TMEM loads are warp-collective
        if (!ok) break;
        if (((jl / JPU) & 1) != grp) {  // not this group's tile: seen, nothing to read
          if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[slot]));
          continue;
        }
        tc_fence_after();
        const uint32_t t_p = t_lane + slot * 256;
        if constexpr (N2 >= 16) {
#pragma unroll 1
        for (int sc = 0; sc < N2 / 16; ++sc) {
          const int zc = j * N2 + sc * 16;  // first z column of this 16-column group
          float acc[16];
#pragma unroll
          for (int q = 0; q < 16; ++q) acc[q] = 0.f;
#pragma unroll
          for (int a = 0; a < R1; a += 2) {
            uint32_t r0[16], r1v[16];
            tmem_ld16(t_p + a * N2 + sc * 16, r0);
            tmem_ld16(t_p + (a + 1) * N2 + sc * 16, r1v);
            tmem_ld_wait(r0, r1v);
#pragma unroll
            for (int q = 0; q < 16; ++q) {
              acc[q] = fmaf(c[a], __uint_as_float(r0[q]), acc[q]);
              acc[q] = fmaf(c[a + 1], __uint_as_float(r1v[q]), acc[q]);
            }
          }
          if (sc == N2 / 16 - 1) {  // last TMEM read of this tile by this warp: hand the accumulator back
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[slot]));
          }
          if (live) {
            // 32 bytes of this thread's z row straight from registers, as ONE 256-bit store where the alignment allows:
            // a whole 32-byte sector per request instead of two halves (82 us against 87 us per launch at the prefill
            // configuration; without any z store the kernel takes 79 us).  The bytes in flight of the core-tile ring
            // matter more to this kernel than coalesced stores (measured), so no staging tile is kept.
            bf16 *dst = p.z + grow * p.r2 + zc;
            uint4 o0, o1;
            o0.x = pack_bf16x2(acc[0], acc[1]); o0.y = pack_bf16x2(acc[2], acc[3]);
            o0.z = pack_bf16x2(acc[4], acc[5]); o0.w = pack_bf16x2(acc[6], acc[7]);
            o1.x = pack_bf16x2(acc[8], acc[9]); o1.y = pack_bf16x2(acc[10], acc[11]);
            o1.z = pack_bf16x2(acc[12], acc[13]); o1.w = pack_bf16x2(acc[14], acc[15]);
            if (p.z_wide) {
              st_global_256(dst, o0, o1);
            } else {
              *reinterpret_cast<uint4 *>(dst) = o0;
              *reinterpret_cast<uint4 *>(dst + 8) = o1;
            }
          }
        }
        } else {
          // N2 = 8 (r1 = 32): one 16-column load covers two adjacent slices; 8 columns of z per tile and thread.  The 64-column
          // unit a group owns is JPU = 8 consecutive tiles: an even tile's 16 bytes wait in registers for the odd tile after
          // it, and the pair leaves as one 32-byte store.
          static_assert(N2 >= 16 || (N2 == 8 && R1 % 4 == 0), "slice widths below 8 columns are not covered");
          float acc[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) acc[q] = 0.f;
#pragma unroll
          for (int a = 0; a < R1; a += 4) {
            uint32_t r0[16], r1v[16];
            tmem_ld16(t_p + a * 8, r0);
            tmem_ld16(t_p + (a + 2) * 8, r1v);
            tmem_ld_wait(r0, r1v);
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              acc[q] = fmaf(c[a], __uint_as_float(r0[q]), acc[q]);
              acc[q] = fmaf(c[a + 1], __uint_as_float(r0[8 + q]), acc[q]);
              acc[q] = fmaf(c[a + 2], __uint_as_float(r1v[q]), acc[q]);
              acc[q] = fmaf(c[a + 3], __uint_as_float(r1v[8 + q]), acc[q]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_pempty[slot]));
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
          // pairs are (even j, j + 1) in global tile numbers: j0 and jn are multiples of JPU, so both are this CTA's
          const bool pair_up = p.z_wide && (jn & 1) == 0 && (j0 & 1) == 0;
          if (pair_up && (jl & 1) == 0) {
            held = o;
          } else if (live) {
            bf16 *dst = p.z + grow * p.r2 + j * 8;
            if (pair_up) st_global_256(dst - 8, held, o);
            else *reinterpret_cast<uint4 *>(dst) = o;
          }
        }
      }
      if (p.ready && ok) {
        // this warp's z rows are written: make them visible device-wide, then raise the warp's hand-off word
        __threadfence();
        __syncwarp();
        if (lane == 0) *reinterpret_cast<volatile uint32_t *>(p.ready + (size_t)bid * 8 + (warp - 2)) = p.epoch;
      }
      if (threadIdx.x == 64) TMOE_STAMP(5);  // z stored
#ifdef TMOE_TRACE
      if (threadIdx.x == 64 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {
        unsigned long long ns1;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns1));
        p.status[32 + (blockIdx.x == 0 ? 0 : 1)] = (int32_t)(ns1 - trace_ns0);  // wall time of the same span in ns
      }
#endif
    }
  }
  tc_fence_before();
  __syncthreads();
  if (p.queue && threadIdx.x == 0) {
    // every epilogue warp of this CTA has fenced its z rows and raised its word: count the CTA as done (a CTA of the
    // out-projection that finds all of them done skips the per-tile words)
    __threadfence();
    atomicAdd(p.queue + 1, 1ull);
  }
  if (warp == 2) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int launch_tc_in_core(const tmoe_layer_t &L, const void *x, const void *prepared, const PreparedLayout &P, int64_t T_,
                      int pre_norm, float pre_norm_eps, int fuse_router, const float *c_in, float *c_work, int c_work_blocks, int32_t *idx_out, float *gates_out, float *c_out,
                      void *z, int32_t *status, cudaStream_t st, const OutFlags *flags, const InCoreTwin *twin) {
  if (fuse_router && (P.e_pad > 256 || L.top_k > 8 || L.r3 > 256)) return TMOE_ERR_UNSUPPORTED;
  if ((!fuse_router && !c_in) || !c_work) return TMOE_ERR_NULL;
  if (pre_norm && !fuse_router) return TMOE_ERR_UNSUPPORTED;
  if (twin && (!fuse_router || !twin->prepared || !twin->c_work || !twin->z || flags)) return TMOE_ERR_UNSUPPORTED;
  if (X_TILE_BYTES + (L.r3 > 256 ? 256 : L.r3) * 128 + (fuse_router ? P.e_pad : 0) * 128 > IC_RING_BYTES) return TMOE_ERR_UNSUPPORTED;
  CUtensorMap tmX, tmU, tmW, tmG, tmU2, tmW2, tmG2;
  int rc = encode_tmap_bf16_2d(&tmX, x, (uint64_t)T_, (uint64_t)L.d_in, TM);
  if (rc) return rc;
  // tensor maps and parameter block of one layer's factor set
  auto fill = [&](const void *prep, float *cw, void *zz, int32_t *io, float *go, float *co, CUtensorMap *mU, CUtensorMap *mW,
                  CUtensorMap *mG, InCoreParams *q) -> int {
    const char *base = reinterpret_cast<const char *>(prep);
    int r = encode_tmap_bf16_2d(mU, base + P.uin_t, (uint64_t)L.r3, (uint64_t)L.d_in, (uint32_t)(L.r3 / ((L.r3 + 255) / 256)));
    if (r) return r;
    // the router tile is only loaded when the scores are computed in-kernel (e_pad <= 256 checked above)
    if ((r = encode_tmap_bf16_2d(mW, base + P.wr_b, (uint64_t)P.e_pad, (uint64_t)L.d_in, fuse_router ? (uint32_t)P.e_pad : 16u))) return r;
    if ((r = encode_tmap_bf16_2d(mG, base + P.g_t, (uint64_t)L.r1 * L.r2, (uint64_t)L.r3, 256))) return r;
    *q = InCoreParams{};
    q->T = T_; q->d_in = L.d_in; q->r3 = L.r3; q->r2 = L.r2; q->E = L.n_experts; q->top_k = L.top_k;
    q->e_pad = fuse_router ? P.e_pad : 0;
    q->n_tiles2 = P.n_tiles2; q->eps = L.eps; q->fuse_router = fuse_router; q->rc = router_cfg(L);
    q->pre_norm = pre_norm; q->pre_norm_eps = pre_norm_eps;
    q->normw = reinterpret_cast<const float *>(base + P.normw);
    q->uexp = reinterpret_cast<const float *>(base + P.uexp);
    q->c_in = c_in; q->c_work = cw; q->idx_out = io; q->gates_out = go; q->c_out = co;
    q->z = (bf16 *)zz; q->status = status;
    q->z_wide = (reinterpret_cast<uintptr_t>(zz) & 31) == 0;
    return TMOE_OK;
  };
  InCoreParams p, p2;
  if ((rc = fill(prepared, c_work, z, idx_out, gates_out, c_out, &tmU, &tmW, &tmG, &p))) return rc;
  if (twin) {
    if ((rc = fill(twin->prepared, twin->c_work, twin->z, nullptr, nullptr, nullptr, &tmU2, &tmW2, &tmG2, &p2))) return rc;
  } else {
    tmU2 = tmU; tmW2 = tmW; tmG2 = tmG; p2 = p;
  }

  unsigned grid = (unsigned)((T_ + TM - 1) / TM);
  const unsigned layers = twin ? 2u : 1u;
  // Few token tiles: share each tile between j_split CTAs (every one repeats phase A, then takes its share of the core
  // tiles).  j_split is the largest divisor of n_tiles2 that fits the SM count and the scratch blocks and keeps whole
  // 64-column units of z per CTA.
  p.j_split = 1;
  {
    const int sms = current_device_sms();
    const int n2 = 256 / L.r1, jpu = n2 >= 64 ? 1 : 64 / n2;
    int cap = sms > 0 ? sms / (int)(grid * layers) : 1;
    if (cap > c_work_blocks - 1) cap = c_work_blocks - 1;
    if (cap > kMaxJSplit) cap = kMaxJSplit;
    static const int env_split = [] { const char *s = getenv("TMOE_JSPLIT"); return s ? atoi(s) : -1; }();
    if (env_split >= 0 && cap > env_split) cap = env_split;
    for (int d = cap; d >= 2; --d)
      if (P.n_tiles2 % d == 0 && (P.n_tiles2 / d) % jpu == 0) { p.j_split = d; break; }
  }
  p2.j_split = p.j_split;
  grid *= (unsigned)p.j_split * layers;
  p.pair = p2.pair = twin ? 1 : 0;
  if (flags && flags->ready) {
    if (p.j_split != 1) return TMOE_ERR_UNSUPPORTED;   // the hand-over is for calls with more token tiles than SMs
    p.ready = flags->ready; p.epoch = flags->epoch; p.queue = flags->queue;
  }
  cudaError_t e = cudaSuccess;
#define TMOE_IC(R, K)                                                                                              \
  do {                                                                                                             \
    e = cudaFuncSetAttribute(tc_in_core_kernel<R, K>, cudaFuncAttributeMaxDynamicSharedMemorySize, IC_SMEM_BYTES); \
    if (e == cudaSuccess) e = launch_pdl(tc_in_core_kernel<R, K>, dim3(grid), dim3(IC_THREADS), (size_t)IC_SMEM_BYTES, st, tmX, tmU, tmW, tmG, p, tmU2, tmW2, tmG2, p2); \
  } while (0)
  const bool small_k = L.top_k <= 2;
  if (L.r1 == 2) { if (small_k) TMOE_IC(2, 2); else TMOE_IC(2, 8); }
  else if (L.r1 == 4) { if (small_k) TMOE_IC(4, 2); else TMOE_IC(4, 8); }
  else if (L.r1 == 8) { if (small_k) TMOE_IC(8, 2); else TMOE_IC(8, 8); }
  else if (L.r1 == 16) { if (small_k) TMOE_IC(16, 2); else TMOE_IC(16, 8); }
  else if (L.r1 == 32) { if (small_k) TMOE_IC(32, 2); else TMOE_IC(32, 8); }
  else return TMOE_ERR_UNSUPPORTED;
#undef TMOE_IC
  if (e != cudaSuccess) return TMOE_ERR_CUDA;
  count_launch();
  return launch_status();
}


}  // namespace tmoe
