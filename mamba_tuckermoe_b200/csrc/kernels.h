// Internal launcher declarations shared by the translation units of the library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>

#include "tmoe_b200.h"

namespace tmoe {

// SM count of the calling thread's current device, looked up once per device (0 on error).
inline int current_device_sms() {
  static std::atomic<int> cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  if (dev >= 0 && dev < 64) cache[dev].store(sms, std::memory_order_relaxed);
  return sms;
}


// Optional element-wise tail of the out-projection, applied in fp32 to v = acc + bias, in this order:
//   silu_gate   v = silu(g[t, n]) * v                      (the FFN's silu(gate) * up, model.py:340)
//   residual    v = residual[t, n] + layer_scale[n] * v    (model.py:260, 341)
// Pointers are in the layer dtype; nullptr = not applied.
struct OutEpilogue {
  const void *residual = nullptr;
  const void *layer_scale = nullptr;
  const void *silu_gate = nullptr;
  int n_peers = 0;                      // tensor-core out-projection only: every tile is also stored to peer_y[i]
  void *peer_y[TMOE_MAX_PEERS] = {};
};

// ---- router.cu ----
int launch_router_fused(const tmoe_layer_t &L, const void *x, const void *wr, const void *uexp, int64_t T,
                        int32_t *idx, float *gates, float *c, cudaStream_t st);
int launch_select(const tmoe_layer_t &L, const float *scores, const void *uexp, int64_t T, int32_t *idx,
                  float *gates, float *c, cudaStream_t st);
// same selection from bf16 scores [T, ld] (ld >= E: row pitch), bf16 layer
int launch_select_bf16_scores(const tmoe_layer_t &L, const void *scores, int ld, const void *uexp, int64_t T,
                              int32_t *idx, float *gates, float *c, cudaStream_t st);

// ---- simt_gemm.cu ----
// scores[T, E] (fp32) = x @ router_w^T
int launch_simt_scores(const tmoe_layer_t &L, const void *x, const void *wr, int64_t T, float *scores, cudaStream_t st);
// h[T, r3] (fp32) = x @ U_in, then in-place inner RMSNorm with weight w (layer dtype)
int launch_simt_inproj_norm(const tmoe_layer_t &L, const void *x, const void *U_in, const void *w, int64_t T, float *h,
                            cudaStream_t st);
// z[T, r2] (fp32) = sum_a c[:, a] * (h @ core[a])
int launch_simt_core(const tmoe_layer_t &L, const float *h, const float *c, const void *core, int64_t T, float *z,
                     cudaStream_t st);
// y[T, d_out] (layer dtype) = z @ U_out + bias, optionally residual + layer_scale * (...)
int launch_simt_out(const tmoe_layer_t &L, const float *z, const void *U_out, const void *bias, const OutEpilogue &epi,
                    int64_t T, void *y, cudaStream_t st);
// y[T, d] = x / sqrt(mean(x^2) + eps) * w, fp32 arithmetic, one rounding to the storage type (model.py:25-27)
int launch_rms_norm(int dtype, const void *x, const void *w, float eps, int64_t T, int d, void *y, cudaStream_t st);

// ---- prepare.cu ----
struct PreparedLayout {
  int64_t uin_t, wr_b, g_t, uout_t, normw, bias, uexp, total;  // byte offsets
  int e_pad, n2, n_tiles2;
};
bool prepared_covers(const tmoe_layer_t &L);     // prepared layout + decode kernels (r1 in {2,...,32})
bool tensor_path_covers(const tmoe_layer_t &L);  // tcgen05 kernels
PreparedLayout prepared_layout(const tmoe_layer_t &L);
// pre_norm_w (optional, [d_in], layer dtype): folded into the U_in and router copies (see prepare.cu)
int launch_prepare(const tmoe_layer_t &L, const tmoe_factors_t &F, const void *pre_norm_w, void *prepared, cudaStream_t st);

// ---- tc_out_gemm.cu ----
// Tile-by-tile hand-over of z from the in/core kernel to the out-projection (used when the token tiles need more than one
// wave of CTAs: the out-projection's CTA pairs then start on the SMs the last wave leaves free instead of waiting for the
// whole in/core grid).  ready: 8 words per 128-token tile in the workspace, each set to `epoch` by one epilogue warp of the
// CTA that stored the tile's z rows; queue: the 64-bit word {epoch, tiles handed out} the pairs draw their tiles from.
// Nothing is ever cleared: a forward's epoch supersedes the previous one's.
struct OutFlags {
  uint32_t *ready = nullptr;
  uint32_t epoch = 0;
  unsigned long long *queue = nullptr;
};
// Whether a forward of T tokens on a device with `sms` SMs uses the hand-over.
bool plan_out_handoff(const tmoe_layer_t &L, int64_t T, int sms);
bool tc_gemm_uses_pairs(int64_t M, int N, int sms);

// y[T, N] = z[T, K] (bf16) @ W_t[N, K]^T (bf16, K-major) + bias (fp32) on tcgen05 tensor cores.
int launch_tc_out(const tmoe_layer_t &L, const void *z, const void *uout_t, const float *bias, const OutEpilogue &epi,
                  int64_t T, void *y, int32_t *status, cudaStream_t st, const OutFlags *flags = nullptr);

// General form of the same kernel (used for the router scores when E is too large for the in-kernel router).
int launch_tc_gemm_bf16(const void *A, const void *B_t, const float *bias, const OutEpilogue &epi, int64_t M, int N,
                        int K, void *y, int32_t *status, cudaStream_t st, const OutFlags *flags = nullptr);

// ---- tc_in_core.cu ----
// Fused x@U_in (+ router scores) -> RMS statistics -> h@G tiles with c-weighted epilogue -> z bf16.
// fuse_router != 0: scores/top-k/softmax/c are computed inside (c_in ignored, taps optional);
// otherwise c_in [T, r1] is read.  c_work [T, r1] is scratch in both cases.
// pre_norm != 0: `prepared` carries the pre-norm weight folded into U_in / router rows; the kernel then computes every
// row's 1/rms(x) from the x tiles passing through shared memory and applies it to the scores and to the RMS statistics.
// c_work holds c_work_blocks blocks of [T, r1] floats.  With in_core_c_blocks(T) blocks and few token tiles, each tile
// is shared by several CTAs that split the core tiles between them (block 0 may alias c_in / c_out, the others may not).
constexpr int kMaxJSplit = 16;
inline int in_core_c_blocks(int64_t T) {
  const int64_t tiles = (T + 127) / 128;   // sized for up to 160 SMs, whatever device the sizing query runs on
  if (tiles < 1 || tiles * 2 > 160) return 1;
  const int per_tile = (int)(160 / tiles);
  return 1 + (per_tile < kMaxJSplit ? per_tile : kMaxJSplit);
}
// `twin` (optional): a second layer of the same sizes applied to the same x in the same launch (the FFN's gate and up
// projections): its prepared set, its own c scratch and its own z.  In-kernel router only, no taps, no hand-over.
struct InCoreTwin {
  const void *prepared;
  float *c_work;
  void *z;
};
int launch_tc_in_core(const tmoe_layer_t &L, const void *x, const void *prepared, const PreparedLayout &P, int64_t T,
                      int pre_norm, float pre_norm_eps, int fuse_router, const float *c_in, float *c_work, int c_work_blocks, int32_t *idx_out, float *gates_out, float *c_out,
                      void *z, int32_t *status, cudaStream_t st, const OutFlags *flags = nullptr, const InCoreTwin *twin = nullptr);

// Stand-alone router for bf16 layers on the tensor cores (tc_router.cu, persistent): idx / gates / c from x and
// the layer's own router_w / U_expert.  TMOE_ERR_UNSUPPORTED for E > 256 (padded), top_k > 8 or d_in % 64 != 0.
int launch_tc_router(const tmoe_layer_t &L, const void *x, const void *router_w, const void *uexp_bf16, int64_t T, int32_t *idx,
                     float *gates, float *c, int32_t *status, cudaStream_t st);

// ---- decode.cu ----
// Whole forward for T <= 64 bf16 tokens on the prepared (K-major) factors: split-K in-projection with
// fp32 atomics into h_raw/scores (adjacent in memory, cleared here), norm + routing + core, out-projection.
int launch_decode(const tmoe_layer_t &L, const void *x, const void *prepared, const PreparedLayout &P, int64_t T,
                  float *h_raw, float *scores, void *z, int32_t *idx_out, float *gates_out, float *c_out,
                  const OutEpilogue &epi, void *y, cudaStream_t st, int pre_norm = 0, float pre_norm_eps = 0.f);


// ---- decode_fused.cu ----
// The same forward for T <= kFusedDecodeMaxTokens in one launch of thread-block clusters (above that the per-token arithmetic
// it repeats in every cluster outweighs the launches it saves: measured 36 us against 17 us at T = 8).  partial: [kMaxDecodeClusters, T, d_out] floats of
// scratch; counters: kDecodeCounterWords zeroed words that the kernel leaves zeroed.  TMOE_ERR_UNSUPPORTED when the shape
// does not fit its shared-memory plan (the caller then uses launch_decode).
constexpr int kMaxDecodeClusters = 24;
constexpr int kFusedDecodeMaxTokens = 4;
constexpr int kDecodeCounterWords = 16;
int launch_decode_fused(const tmoe_layer_t &L, const void *x, const void *prepared, const PreparedLayout &P, int64_t T,
                        float *partial, unsigned int *counters, int32_t *idx_out, float *gates_out, float *c_out,
                        const OutEpilogue &epi, void *y, cudaStream_t st, int pre_norm = 0, float pre_norm_eps = 0.f);

}  // namespace tmoe
