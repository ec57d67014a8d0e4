// extern "C" entry points declared in include/tmoe_b200.h: validation, workspace carving and
// dispatch between the CUDA-core path and the tcgen05 tensor-core path.
#include "common.cuh"
#include "kernels.h"
#include "ptx.cuh"
#include <atomic>
#include <cmath>

namespace tmoe {

unsigned long long g_launch_count = 0;

namespace {

struct WsLayout {
  int64_t idx, gates, c, scores, h, z, partial, ready, total;
  bool simt_router_fused;  // CUDA-core path: warp-per-token router (else tiled scores + select)
  bool tc_router_fused;    // tensor-core path: scores and selection inside the in/core kernel
};

int check_layer(const tmoe_layer_t *L) {
  if (!L) return TMOE_ERR_NULL;
  if (L->dtype != TMOE_F32 && L->dtype != TMOE_BF16) return TMOE_ERR_DTYPE;
  if (L->d_in <= 0 || L->d_out <= 0 || L->n_experts <= 0 || L->top_k <= 0 || L->r1 <= 0 || L->r2 <= 0 || L->r3 <= 0)
    return TMOE_ERR_SHAPE;
  if (L->top_k > L->n_experts || L->top_k > TMOE_MAX_TOPK || L->r1 > TMOE_MAX_R1) return TMOE_ERR_SHAPE;
  if ((L->d_in | L->d_out | L->r2 | L->r3) & 7) return TMOE_ERR_SHAPE;
  if (L->router_mode != TMOE_ROUTER_TOPK_SOFTMAX && L->router_mode != TMOE_ROUTER_CAPPED_SOFTMAX) return TMOE_ERR_UNSUPPORTED;
  if (L->router_mode == TMOE_ROUTER_CAPPED_SOFTMAX) {
    // the cap divides the scores and the temperature divides the logits: both must be finite and positive
    if (!(L->router_cap > 0.f) || !(L->router_temperature > 0.f) || std::isinf(L->router_cap) ||
        std::isinf(L->router_temperature))
      return TMOE_ERR_SHAPE;
  }
  return TMOE_OK;
}

// Token counts are carried as 32-bit row indices by the CUDA-core kernels and as tensor-map extents by the others.
constexpr int64_t kMaxTokens = (int64_t)1 << 30;
inline int check_tokens(int64_t T) { return (T < 0 || T > kMaxTokens) ? (int)TMOE_ERR_SHAPE : (int)TMOE_OK; }

// allow_decode: tmoe_forward (and the sizing queries) may pick the decode kernels; the stage entry
// points cannot, so for them AUTO means the tensor-core path when it covers the shape, else the CUDA-core path.
constexpr int kDecodeAutoTokens = 8;

int resolve(const tmoe_layer_t &L, int64_t T, int path, bool allow_decode = true) {
  if (path == TMOE_PATH_SIMT) return TMOE_PATH_SIMT;
  const bool tensor_ok = tensor_path_covers(L), decode_ok = prepared_covers(L) && allow_decode && T <= 64;
  if (path == TMOE_PATH_TENSOR) return tensor_ok ? (int)TMOE_PATH_TENSOR : (int)TMOE_ERR_UNSUPPORTED;
  if (path == TMOE_PATH_DECODE) return decode_ok ? (int)TMOE_PATH_DECODE : (int)TMOE_ERR_UNSUPPORTED;
  if (path != TMOE_PATH_AUTO) return TMOE_ERR_UNSUPPORTED;
  // Up to 8 tokens the decode-shaped kernels win (16-18 us per call on the decode configuration); from there the
  // tensor-core kernels do: one 128-token tile shared by up to 16 CTAs costs the same 32 us for any T, the decode kernels
  // 47 us at T = 9 growing to 67 us at T = 64, and unlike their split-K in-projection the tensor path is run-to-run
  // reproducible.
  if (T > 64) return tensor_ok ? TMOE_PATH_TENSOR : TMOE_PATH_SIMT;
  if (T > kDecodeAutoTokens && tensor_ok) return TMOE_PATH_TENSOR;
  return decode_ok ? TMOE_PATH_DECODE : (tensor_ok ? TMOE_PATH_TENSOR : TMOE_PATH_SIMT);
}

WsLayout ws_layout(const tmoe_layer_t &L, int64_t T, int rpath) {
  WsLayout W{};
  int64_t off = kHeaderBytes;
  auto take = [&](int64_t bytes) { int64_t o = off; off = align_up(off + bytes, 256); return o; };
  W.idx = take(T * L.top_k * 4);
  W.gates = take(T * L.top_k * 4);
  // the tensor-core in/core kernel keeps extra [T, r1] blocks for small T (tiles shared between CTAs)
  W.c = take(T * L.r1 * 4 * (rpath == TMOE_PATH_TENSOR ? in_core_c_blocks(T) : 1));
  W.simt_router_fused = (L.n_experts <= 32) || (T <= 256);
  W.tc_router_fused = (align_up(L.n_experts, 16) <= 256) && (L.top_k <= 8) && (L.r3 <= 256);
  if (rpath == TMOE_PATH_SIMT) {
    W.scores = W.simt_router_fused ? 0 : take(T * L.n_experts * 4);
    W.h = take(T * L.r3 * 4);
    W.z = take(T * L.r2 * 4);
  } else if (rpath == TMOE_PATH_DECODE) {
    // h_raw and scores back to back (no padding in between): cleared together before the split-K atomics
    W.h = take(T * (L.r3 + L.n_experts) * 4);
    W.scores = W.h + T * L.r3 * 4;
    W.z = take(T * L.r2 * 2);
    // one-launch kernel for the smallest calls: per-cluster partial sums of y
    W.partial = T <= kFusedDecodeMaxTokens ? take((int64_t)kMaxDecodeClusters * T * L.d_out * 4) : 0;
  } else {
    W.scores = W.tc_router_fused ? 0 : take(T * align_up(L.n_experts, 16) * 2);  // bf16 [T, e_pad], made by the GEMM kernel
    W.h = 0;
    W.z = take(T * L.r2 * 2);
    W.ready = take(((T + 127) / 128) * 8 * 4);   // hand-over words, 8 per 128-token tile
  }
  W.total = off;
  return W;
}

bool misaligned(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

int check_factors(const tmoe_factors_t *F) {
  if (!F) return TMOE_ERR_NULL;
  const void *ps[7] = {F->router_w, F->U_in, F->inner_norm_w, F->U_expert, F->core, F->U_out, F->bias};
  for (const void *p : ps) {
    if (!p) return TMOE_ERR_NULL;
    if (misaligned(p)) return TMOE_ERR_ALIGN;
  }
  return TMOE_OK;
}

// Validates the optional epilogue inputs of `extras` and copies them into an OutEpilogue.
int epilogue_from(const tmoe_extras_t *extras, OutEpilogue *epi) {
  if (!extras) return TMOE_OK;
  if ((extras->residual == nullptr) != (extras->layer_scale == nullptr)) return TMOE_ERR_NULL;
  const void *ps[3] = {extras->residual, extras->layer_scale, extras->silu_gate};
  for (const void *q : ps)
    if (q && misaligned(q)) return TMOE_ERR_ALIGN;
  epi->residual = extras->residual;
  epi->layer_scale = extras->layer_scale;
  epi->silu_gate = extras->silu_gate;
  if (extras->n_peer_y < 0 || extras->n_peer_y > TMOE_MAX_PEERS) return TMOE_ERR_SHAPE;
  epi->n_peers = extras->n_peer_y;
  for (int i = 0; i < extras->n_peer_y; ++i) {
    if (!extras->peer_y[i]) return TMOE_ERR_NULL;
    if (misaligned(extras->peer_y[i])) return TMOE_ERR_ALIGN;
    epi->peer_y[i] = extras->peer_y[i];
  }
  return TMOE_OK;
}

int router_simt(const tmoe_layer_t &L, const tmoe_factors_t &F, const void *x, int64_t T, bool fused, float *scores,
                int32_t *idx, float *gates, float *c, cudaStream_t st) {
  if (fused) return launch_router_fused(L, x, F.router_w, F.U_expert, T, idx, gates, c, st);
  int rc = launch_simt_scores(L, x, F.router_w, T, scores, st);
  if (rc) return rc;
  return launch_select(L, scores, F.U_expert, T, idx, gates, c, st);
}

}  // namespace
}  // namespace tmoe

using namespace tmoe;

extern "C" {

int tmoe_version(void) { return TMOE_ABI_VERSION; }

const char *tmoe_status_string(int status) {
  switch (status) {
    case TMOE_OK: return "ok";
    case TMOE_ERR_NULL: return "a required pointer is NULL";
    case TMOE_ERR_SHAPE: return "invalid layer shape (sizes must be positive, d_in/d_out/r2/r3 multiples of 8, top_k <= n_experts)";
    case TMOE_ERR_DTYPE: return "unsupported dtype (fp32 and bf16 only)";
    case TMOE_ERR_ALIGN: return "a device pointer is not 16-byte aligned";
    case TMOE_ERR_WORKSPACE: return "workspace or prepared-factor buffer too small";
    case TMOE_ERR_UNSUPPORTED: return "the requested path does not cover this shape/dtype";
    case TMOE_ERR_CUDA: return "a CUDA runtime call or kernel launch failed";
    case TMOE_ERR_DRIVER: return "tensor-map encoding unavailable or failed";
    case TMOE_ERR_DEVICE_WAIT: return "a bounded wait inside a kernel expired";
    default: return "unknown status";
  }
}

int tmoe_resolve_path(const tmoe_layer_t *layer, int64_t T, int path) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  return resolve(*layer, T, path);
}

int64_t tmoe_prepared_bytes(const tmoe_layer_t *layer) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if (!prepared_covers(*layer)) return 0;
  return prepared_layout(*layer).total;
}

int tmoe_prepare_factors(const tmoe_layer_t *layer, const tmoe_factors_t *factors, void *prepared,
                         int64_t prepared_bytes, void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if ((rc = check_factors(factors))) return rc;
  if (!prepared) return TMOE_ERR_NULL;
  if (!prepared_covers(*layer)) return TMOE_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(prepared) & 255) return TMOE_ERR_ALIGN;
  if (prepared_bytes < prepared_layout(*layer).total) return TMOE_ERR_WORKSPACE;
  return launch_prepare(*layer, *factors, nullptr, prepared, (cudaStream_t)stream);
}

int tmoe_prepare_factors_prenorm(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *pre_norm_w,
                                 void *prepared, int64_t prepared_bytes, void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if ((rc = check_factors(factors))) return rc;
  if (!prepared || !pre_norm_w) return TMOE_ERR_NULL;
  if (!prepared_covers(*layer)) return TMOE_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(prepared) & 255) || misaligned(pre_norm_w)) return TMOE_ERR_ALIGN;
  if (prepared_bytes < prepared_layout(*layer).total) return TMOE_ERR_WORKSPACE;
  return launch_prepare(*layer, *factors, pre_norm_w, prepared, (cudaStream_t)stream);
}

int64_t tmoe_workspace_bytes(const tmoe_layer_t *layer, int64_t T, int path) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  int rp = resolve(*layer, T, path);
  if (rp < 0) return rp;
  return ws_layout(*layer, T, rp).total;
}

int tmoe_router(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *x, int64_t T, int32_t *idx,
                float *gates, float *c, void *workspace, int64_t workspace_bytes, void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if ((rc = check_factors(factors))) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  if (T == 0) return TMOE_OK;
  if (!x || !idx || !gates || !c || !workspace) return TMOE_ERR_NULL;
  if (misaligned(x) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return TMOE_ERR_ALIGN;
  WsLayout W = ws_layout(*layer, T, TMOE_PATH_SIMT);
  if (workspace_bytes < W.total) return TMOE_ERR_WORKSPACE;
  char *ws = reinterpret_cast<char *>(workspace);
  const tmoe_layer_t &L = *layer;
  // bf16 layers with enough tokens: the scores are a [T, d_in] x [d_in, E] contraction whose only HBM traffic is one read of
  // x, but at E >= 16 its FMA count exceeds what the CUDA cores do in that time.  router_w [E, d_in] is already the K-major
  // operand the tensor-core GEMM kernel wants, its bf16 output is the reference's rounding of the scores, and the keyed
  // select kernel finishes the job.  Needs E % 8 == 0 (16-byte rows of scores) and room for [T, E] bf16 in the workspace.
  const int64_t sc_off = kHeaderBytes;
  if (L.dtype == TMOE_BF16 && T >= 512) {
    // up to 1024 experts and top-8: one launch that accumulates the scores in TMEM and selects from there
    rc = launch_tc_router(L, x, factors->router_w, factors->U_expert, T, idx, gates, c, reinterpret_cast<int32_t *>(ws),
                          (cudaStream_t)stream);
    if (rc != TMOE_ERR_UNSUPPORTED) return rc;
  }
  if (L.dtype == TMOE_BF16 && T >= 512 && L.n_experts % 8 == 0 && L.n_experts <= 1024 &&
      workspace_bytes >= sc_off + T * L.n_experts * 2) {
    void *scores = ws + sc_off;
    if ((rc = launch_tc_gemm_bf16(x, factors->router_w, nullptr, OutEpilogue{}, T, L.n_experts, L.d_in, scores,
                                  reinterpret_cast<int32_t *>(ws), (cudaStream_t)stream)))
      return rc;
    return launch_select_bf16_scores(L, scores, L.n_experts, factors->U_expert, T, idx, gates, c, (cudaStream_t)stream);
  }
  return router_simt(L, *factors, x, T, W.simt_router_fused, reinterpret_cast<float *>(ws + W.scores), idx, gates,
                     c, (cudaStream_t)stream);
}

int tmoe_in_core(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *prepared, const void *x,
                 int64_t T, const float *c, void *z, void *workspace, int64_t workspace_bytes, int path, void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if ((rc = check_factors(factors))) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  if (T == 0) return TMOE_OK;
  if (!x || !c || !z || !workspace) return TMOE_ERR_NULL;
  if (misaligned(x) || misaligned(z) || misaligned(c) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return TMOE_ERR_ALIGN;
  int rp = resolve(*layer, T, path, false);
  if (rp < 0) return rp;
  WsLayout W = ws_layout(*layer, T, rp);
  if (workspace_bytes < W.total) return TMOE_ERR_WORKSPACE;
  char *ws = reinterpret_cast<char *>(workspace);
  cudaStream_t st = (cudaStream_t)stream;
  if (rp == TMOE_PATH_SIMT) {
    float *h = reinterpret_cast<float *>(ws + W.h);
    if ((rc = launch_simt_inproj_norm(*layer, x, factors->U_in, factors->inner_norm_w, T, h, st))) return rc;
    return launch_simt_core(*layer, h, c, factors->core, T, reinterpret_cast<float *>(z), st);
  }
  if (!prepared) return TMOE_ERR_NULL;
  return launch_tc_in_core(*layer, x, prepared, prepared_layout(*layer), T, 0, 0.f, 0, c,
                           reinterpret_cast<float *>(ws + W.c), in_core_c_blocks(T), nullptr, nullptr, nullptr, z,
                           reinterpret_cast<int32_t *>(ws), st);
}

int tmoe_out(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *prepared, const void *z, int64_t T,
             void *y, const tmoe_extras_t *extras, void *workspace, int64_t workspace_bytes, int path, void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if ((rc = check_factors(factors))) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  if (T == 0) return TMOE_OK;
  if (!z || !y || !workspace) return TMOE_ERR_NULL;
  if (misaligned(z) || misaligned(y) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return TMOE_ERR_ALIGN;
  if (workspace_bytes < kStatusBytes) return TMOE_ERR_WORKSPACE;
  OutEpilogue epi;
  if ((rc = epilogue_from(extras, &epi))) return rc;
  int rp = resolve(*layer, T, path, false);
  if (rp < 0) return rp;
  if (epi.n_peers && rp != TMOE_PATH_TENSOR) return TMOE_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  if (rp == TMOE_PATH_SIMT)
    return launch_simt_out(*layer, reinterpret_cast<const float *>(z), factors->U_out, factors->bias, epi, T, y, st);
  if (!prepared) return TMOE_ERR_NULL;
  PreparedLayout P = prepared_layout(*layer);
  const char *pb = reinterpret_cast<const char *>(prepared);
  return launch_tc_out(*layer, z, pb + P.uout_t, reinterpret_cast<const float *>(pb + P.bias), epi, T, y,
                       reinterpret_cast<int32_t *>(workspace), st);
}

int tmoe_forward(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *prepared, const void *x,
                 int64_t T, void *y, const tmoe_extras_t *extras, void *workspace, int64_t workspace_bytes, int path,
                 void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if ((rc = check_factors(factors))) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  if (T == 0) return TMOE_OK;
  if (!x || !y || !workspace) return TMOE_ERR_NULL;
  if (misaligned(x) || misaligned(y) || (reinterpret_cast<uintptr_t>(workspace) & 255)) return TMOE_ERR_ALIGN;
  OutEpilogue epi;
  if ((rc = epilogue_from(extras, &epi))) return rc;
  const int pre_norm = (extras && extras->pre_norm) ? 1 : 0;
  int rp = resolve(*layer, T, path);
  if (rp < 0) return rp;
  if (epi.n_peers && rp != TMOE_PATH_TENSOR) return TMOE_ERR_UNSUPPORTED;
  const tmoe_layer_t &L = *layer;
  WsLayout W = ws_layout(L, T, rp);
  if (workspace_bytes < W.total) return TMOE_ERR_WORKSPACE;
  // the in-kernel pre-norm exists on the tensor-core path with the in-kernel router and on the decode path
  if (pre_norm && !((rp == TMOE_PATH_TENSOR && W.tc_router_fused) || rp == TMOE_PATH_DECODE)) return TMOE_ERR_UNSUPPORTED;
  char *ws = reinterpret_cast<char *>(workspace);
  cudaStream_t st = (cudaStream_t)stream;
  int32_t *idx = (extras && extras->idx_out) ? extras->idx_out : reinterpret_cast<int32_t *>(ws + W.idx);
  float *gates = (extras && extras->gates_out) ? extras->gates_out : reinterpret_cast<float *>(ws + W.gates);
  float *c = (extras && extras->c_out) ? extras->c_out : reinterpret_cast<float *>(ws + W.c);
  float *scores = reinterpret_cast<float *>(ws + W.scores);

  if (rp == TMOE_PATH_SIMT) {
    float *h = reinterpret_cast<float *>(ws + W.h);
    float *z = reinterpret_cast<float *>(ws + W.z);
    if ((rc = router_simt(L, *factors, x, T, W.simt_router_fused, scores, idx, gates, c, st))) return rc;
    if ((rc = launch_simt_inproj_norm(L, x, factors->U_in, factors->inner_norm_w, T, h, st))) return rc;
    if ((rc = launch_simt_core(L, h, c, factors->core, T, z, st))) return rc;
    return launch_simt_out(L, z, factors->U_out, factors->bias, epi, T, y, st);
  }
  if (!prepared) return TMOE_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(prepared) & 255) return TMOE_ERR_ALIGN;
  PreparedLayout P = prepared_layout(L);
  const char *pb = reinterpret_cast<const char *>(prepared);
  void *z = ws + W.z;
  int32_t *status = reinterpret_cast<int32_t *>(ws);
  if (rp == TMOE_PATH_DECODE) {
    const bool taps = extras && (extras->idx_out || extras->gates_out || extras->c_out);
    if (T <= kFusedDecodeMaxTokens) {
      rc = launch_decode_fused(L, x, prepared, P, T, reinterpret_cast<float *>(ws + W.partial),
                               reinterpret_cast<unsigned int *>(ws + kStatusBytes + kHandoffBytes),
                               taps ? extras->idx_out : nullptr, taps ? extras->gates_out : nullptr,
                               taps ? extras->c_out : nullptr, epi, y, st, pre_norm, pre_norm ? extras->pre_norm_eps : 0.f);
      if (rc != TMOE_ERR_UNSUPPORTED) return rc;   // shapes outside its shared-memory plan take the three-kernel form
    }
    return launch_decode(L, x, prepared, P, T, reinterpret_cast<float *>(ws + W.h), scores, z,
                         taps ? extras->idx_out : nullptr, taps ? extras->gates_out : nullptr,
                         taps ? extras->c_out : nullptr, epi, y, st, pre_norm, pre_norm ? extras->pre_norm_eps : 0.f);
  }
  // more token tiles than SMs: the out-projection's CTA pairs take finished token tiles while the last wave still runs
  OutFlags flags{};
  {
    const int sms = current_device_sms();
    if (sms <= 0) return TMOE_ERR_CUDA;
    if (plan_out_handoff(L, T, sms)) {
      static std::atomic<uint32_t> epoch_counter{1};
      uint32_t e = epoch_counter.fetch_add(1, std::memory_order_relaxed);
      if (e == 0) e = epoch_counter.fetch_add(1, std::memory_order_relaxed);   // 0 is what a zeroed word holds
      flags.epoch = e;
      flags.ready = reinterpret_cast<uint32_t *>(ws + W.ready);
      flags.queue = reinterpret_cast<unsigned long long *>(ws + kStatusBytes + kHandoffBytes + 128);
    }
  }
  const OutFlags *fp = flags.ready ? &flags : nullptr;
  if (W.tc_router_fused) {
    const bool taps = extras && (extras->idx_out || extras->gates_out || extras->c_out);
    rc = launch_tc_in_core(L, x, prepared, P, T, pre_norm, pre_norm ? extras->pre_norm_eps : 0.f, 1, nullptr,
                           reinterpret_cast<float *>(ws + W.c), in_core_c_blocks(T),
                           taps ? extras->idx_out : nullptr,
                           taps ? extras->gates_out : nullptr, taps ? extras->c_out : nullptr, z, status, st, fp);
  } else {
    // the router as a kernel of its own (layers whose r3 = 512 leaves no TMEM columns for the scores next to h, or with more
    // than 256 experts).  Up to 1024 experts and top-8: the persistent router kernel, scores never leave the SM.  Beyond that: scores = x @ router_w^T as
    // a GEMM (bf16 out = the reference's rounding), then the select kernel.
    rc = launch_tc_router(L, x, factors->router_w, factors->U_expert, T, idx, gates, c, status, st);
    if (rc == TMOE_ERR_UNSUPPORTED) {
      if ((rc = launch_tc_gemm_bf16(x, pb + P.wr_b, nullptr, OutEpilogue{}, T, P.e_pad, L.d_in, scores, status, st)))
        return rc;
      rc = launch_select_bf16_scores(L, scores, P.e_pad, factors->U_expert, T, idx, gates, c, st);
    }
    if (rc) return rc;
    // c_work may alias c: every row is read by its own thread before that thread overwrites it
    rc = launch_tc_in_core(L, x, prepared, P, T, 0, 0.f, 0, c, reinterpret_cast<float *>(ws + W.c), in_core_c_blocks(T), nullptr, nullptr, nullptr, z,
                           status, st, fp);
  }
  if (rc) return rc;
  return launch_tc_out(L, z, pb + P.uout_t, reinterpret_cast<const float *>(pb + P.bias), epi, T, y, status, st, fp);
}

int tmoe_ffn_gate_up(const tmoe_layer_t *layer, const void *prepared_gate, const void *prepared_up, const void *x, int64_t T,
                     void *gate_y, void *act_y, const tmoe_extras_t *extras, void *workspace, int64_t workspace_bytes,
                     void *stream) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if (check_tokens(T)) return TMOE_ERR_SHAPE;
  if (T == 0) return TMOE_OK;
  if (!prepared_gate || !prepared_up || !x || !gate_y || !act_y || !workspace) return TMOE_ERR_NULL;
  if (misaligned(x) || misaligned(gate_y) || misaligned(act_y) || (reinterpret_cast<uintptr_t>(workspace) & 255) ||
      (reinterpret_cast<uintptr_t>(prepared_gate) & 255) || (reinterpret_cast<uintptr_t>(prepared_up) & 255))
    return TMOE_ERR_ALIGN;
  const tmoe_layer_t &L = *layer;
  if (!tensor_path_covers(L)) return TMOE_ERR_UNSUPPORTED;
  const WsLayout W = ws_layout(L, T, TMOE_PATH_TENSOR);
  if (!W.tc_router_fused) return TMOE_ERR_UNSUPPORTED;       // the paired launch needs the in-kernel router
  const int64_t half = align_up(W.total, 256);
  if (workspace_bytes < 2 * half) return TMOE_ERR_WORKSPACE;
  if (extras && (extras->residual || extras->layer_scale || extras->silu_gate || extras->idx_out || extras->gates_out ||
                 extras->c_out || extras->n_peer_y))
    return TMOE_ERR_UNSUPPORTED;                             // only the pre-norm applies here
  const int pre_norm = (extras && extras->pre_norm) ? 1 : 0;
  const float pn_eps = pre_norm ? extras->pre_norm_eps : 0.f;
  char *ws = reinterpret_cast<char *>(workspace);
  char *ws2 = ws + half;                                     // the up layer's c and z (status words are the first half's)
  int32_t *status = reinterpret_cast<int32_t *>(ws);
  cudaStream_t st = (cudaStream_t)stream;
  const PreparedLayout P = prepared_layout(L);
  const char *pg = reinterpret_cast<const char *>(prepared_gate), *pu = reinterpret_cast<const char *>(prepared_up);
  InCoreTwin twin{prepared_up, reinterpret_cast<float *>(ws2 + W.c), ws2 + W.z};
  if ((rc = launch_tc_in_core(L, x, prepared_gate, P, T, pre_norm, pn_eps, 1, nullptr, reinterpret_cast<float *>(ws + W.c),
                              in_core_c_blocks(T), nullptr, nullptr, nullptr, ws + W.z, status, st, nullptr, &twin)))
    return rc;
  if ((rc = launch_tc_out(L, ws + W.z, pg + P.uout_t, reinterpret_cast<const float *>(pg + P.bias), OutEpilogue{}, T, gate_y,
                          status, st)))
    return rc;
  OutEpilogue epi;
  epi.silu_gate = gate_y;
  return launch_tc_out(L, ws2 + W.z, pu + P.uout_t, reinterpret_cast<const float *>(pu + P.bias), epi, T, act_y, status, st);
}

int tmoe_rms_norm(int dtype, const void *x, const void *weight, float eps, int64_t T, int32_t d, void *y, void *stream) {
  if (dtype != TMOE_F32 && dtype != TMOE_BF16) return TMOE_ERR_DTYPE;
  if (T < 0 || d <= 0 || (d & 7)) return TMOE_ERR_SHAPE;
  if (T == 0) return TMOE_OK;
  if (!x || !weight || !y) return TMOE_ERR_NULL;
  if (misaligned(x) || misaligned(weight) || misaligned(y)) return TMOE_ERR_ALIGN;
  return launch_rms_norm(dtype, x, weight, eps, T, d, y, (cudaStream_t)stream);
}

int tmoe_read_device_status(void *workspace, int32_t *device_status, void *stream) {
  if (!workspace || !device_status) return TMOE_ERR_NULL;
  if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return TMOE_ERR_CUDA;
  int32_t words[4] = {0, 0, 0, 0};
  if (cudaMemcpy(words, workspace, sizeof(words), cudaMemcpyDeviceToHost) != cudaSuccess) return TMOE_ERR_CUDA;
  for (int i = 0; i < 4; ++i) device_status[i] = words[i];
  // after a reported wait the flags and counters behind the status words may be left mid-protocol: clear them all
  if (words[0] != 0 && cudaMemset(workspace, 0, kHeaderBytes) != cudaSuccess) return TMOE_ERR_CUDA;
  return TMOE_OK;
}

namespace tmoe {
namespace {
constexpr int kKernelSelfTest = 9;
// One warp; lane 0 waits on a barrier that nobody arrives on and lets the bounded wait run out.
__global__ void selftest_wait_kernel(int32_t *status, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bar;
  if (threadIdx.x == 0) {
    ptx::mbar_init(ptx::smem_u32(&bar), 1);
    ptx::fence_mbar_init();
    (void)ptx::mbar_wait_slow(ptx::smem_u32(&bar), 0, status, kKernelSelfTest, 42, limit_cycles);
  }
}
}  // namespace
}  // namespace tmoe

int tmoe_selftest_bounded_wait(void *workspace, int64_t limit_cycles, void *stream) {
  if (!workspace) return TMOE_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return TMOE_ERR_ALIGN;
  long long lim = limit_cycles < 10000 ? 10000 : (limit_cycles > 200000000 ? 200000000 : (long long)limit_cycles);
  tmoe::selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(reinterpret_cast<int32_t *>(workspace), lim);
  count_launch();
  return launch_status();
}

int tmoe_handoff_plan(const tmoe_layer_t *layer, int64_t T, int32_t *n_early_sms, int32_t *n_token_tiles) {
  int rc = check_layer(layer);
  if (rc) return rc;
  if (!n_early_sms || !n_token_tiles) return TMOE_ERR_NULL;
  *n_early_sms = 0; *n_token_tiles = 0;
  if (T <= 0 || check_tokens(T) || resolve(*layer, T, TMOE_PATH_AUTO) != TMOE_PATH_TENSOR) return TMOE_OK;
  const int sms = current_device_sms();
  if (sms <= 0) return TMOE_ERR_CUDA;
  if (!plan_out_handoff(*layer, T, sms)) return TMOE_OK;
  const int64_t tiles = (T + 127) / 128;
  const int tail = (int)(tiles % sms);
  *n_early_sms = tail ? sms - tail : 0;                 // SMs the last wave of token tiles leaves to the out-projection
  *n_token_tiles = (int32_t)(tiles - (tail ? tail : sms));   // token tiles of the complete waves before it
  return TMOE_OK;
}

int64_t tmoe_launch_count(void) { return (int64_t)__atomic_load_n(&g_launch_count, __ATOMIC_RELAXED); }

}  // extern "C"
