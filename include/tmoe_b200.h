/*
 * tmoe_b200.h -- C ABI of the B200 (sm_100a) Tucker-MoE layer forward.
 *
 * The reference project has no native/FFI interface: its boundary for this path is the
 * Python class TuckerMoE(d_in, d_out, cfg) with forward(x) (pure_torch_mlx/model.py:41-102).
 * The entry points below are what a binding for that forward needs; each comment names the
 * reference lines the entry point replaces.
 *
 * Conventions
 *  - plain C: pointers, integers, floats; no torch / C++ types.  `stream` is a cudaStream_t
 *    passed as void* (NULL = the legacy default stream).
 *  - every pointer named "device" is a CUDA device pointer on the current device.
 *  - functions return 0 (TMOE_OK) or a negative tmoe_status_t; they never throw, never call
 *    exit(), never synchronise the device (except tmoe_read_device_status) and never allocate
 *    device memory: the caller passes a workspace sized by tmoe_workspace_bytes().  (The tmoe_peer_*
 *    functions at the end are the exception: allocating and mapping buffers is their job.)
 *  - all work is enqueued on `stream`; buffers are borrowed until that work has finished.
 *  - tensors are dense row-major.  x, y and the seven factors share one dtype (tmoe_dtype_t).
 */
#ifndef TMOE_B200_H_
#define TMOE_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* 2: tmoe_extras_t grew (n_peer_y, peer_y); the tmoe_peer_* entry points */
#define TMOE_ABI_VERSION 2
#define TMOE_MAX_TOPK 16
#define TMOE_MAX_R1 64

typedef enum tmoe_status {
  TMOE_OK = 0,
  TMOE_ERR_NULL = -1,        /* a required pointer is NULL                               */
  TMOE_ERR_SHAPE = -2,       /* a size is <= 0 or not a multiple of 8, top_k > n_experts (top_k is NOT clamped
                                to n_experts as the trained-checkpoint module does: pass min(top_k, E)), T out of
                                range, or a non-positive / non-finite router cap or temperature in mode 1 */
  TMOE_ERR_DTYPE = -3,       /* dtype is neither TMOE_F32 nor TMOE_BF16                   */
  TMOE_ERR_ALIGN = -4,       /* a device pointer is not 16-byte aligned                   */
  TMOE_ERR_WORKSPACE = -5,   /* workspace / prepared buffer too small                     */
  TMOE_ERR_UNSUPPORTED = -6, /* the requested path does not cover this shape / dtype, or router_mode is unknown */
  TMOE_ERR_CUDA = -7,        /* a CUDA runtime call or kernel launch failed               */
  TMOE_ERR_DRIVER = -8,      /* tensor-map encoding is unavailable or failed              */
  TMOE_ERR_DEVICE_WAIT = -9  /* a bounded wait inside a kernel expired (device status)    */
} tmoe_status_t;

typedef enum tmoe_dtype { TMOE_F32 = 0, TMOE_BF16 = 1 } tmoe_dtype_t;

/* Which kernels run.
 *  SIMT    CUDA-core fp32-FMA kernels: any shape, fp32 or bf16 (the accuracy path).
 *  TENSOR  tcgen05 tensor-core kernels: bf16, r1 in {2,4,8,16,32}, r3 in {64,128,192,256,512},
 *          d_in and r2 multiples of 64.  Needs the prepared factor set.
 *  DECODE  bandwidth-shaped kernels for T <= 64 tokens on the same shapes, same prepared set (tmoe_forward only).
 *  AUTO    DECODE up to 8 tokens, TENSOR above, when the shape is covered; else SIMT. */
typedef enum tmoe_path {
  TMOE_PATH_AUTO = 0, TMOE_PATH_SIMT = 1, TMOE_PATH_TENSOR = 2, TMOE_PATH_DECODE = 3
} tmoe_path_t;

/* Gate rule.
 *  TOPK_SOFTMAX    top-k of the raw scores, softmax over the k winners (pure_torch_mlx/model.py:75-77).
 *  CAPPED_SOFTMAX  the trained checkpoints' rule (sft_cot_bundle/scripts/model.py:318-329,
 *                  mamba3_mlx/mlx_model/tucker_moe.py:107-114): l = cap * tanh(score / cap) / temperature,
 *                  p = softmax(l) over all experts, top-k of l, gate_k = p_k / (sum of the k selected p + 1e-6). */
typedef enum tmoe_router_mode { TMOE_ROUTER_TOPK_SOFTMAX = 0, TMOE_ROUTER_CAPPED_SOFTMAX = 1 } tmoe_router_mode_t;

/* Sizes of one layer; mirrors the constructor arguments TuckerMoE(d_in, d_out, cfg) with
 * cfg.kmoe_num_experts, kmoe_top_k, kmoe_r1, kmoe_r2, kmoe_r3, rms_norm_eps
 * (pure_torch_mlx/model.py:54-62). */
typedef struct tmoe_layer {
  int32_t d_in, d_out;
  int32_t n_experts, top_k;
  int32_t r1, r2, r3;
  int32_t dtype;  /* tmoe_dtype_t */
  float eps;      /* inner_norm epsilon */
  int32_t router_mode;      /* tmoe_router_mode_t; 0 = the pure-PyTorch module's rule */
  float router_cap;         /* TMOE_ROUTER_CAPPED_SOFTMAX: soft cap of the scores (reference: 10); finite, > 0 */
  float router_temperature; /* TMOE_ROUTER_CAPPED_SOFTMAX: softmax temperature (reference at inference: 0.5); finite, > 0 */
} tmoe_layer_t;

/* The seven parameters in the reference's own layouts (pure_torch_mlx/model.py:60-66,
 * filled by pure_torch_mlx/weights.py:74-81).  Device pointers. */
typedef struct tmoe_factors {
  const void *router_w;     /* [n_experts, d_in] */
  const void *U_in;         /* [d_in, r3]        */
  const void *inner_norm_w; /* [r3]              */
  const void *U_expert;     /* [n_experts, r1]   */
  const void *core;         /* [r1, r3, r2]      */
  const void *U_out;        /* [r2, d_out]       */
  const void *bias;         /* [d_out]           */
} tmoe_factors_t;

/* Optional inputs/outputs; a zeroed struct (or NULL) means "plain module forward".
 *  - residual/layer_scale: y = residual + layer_scale * (acc @ U_out + bias), the callers'
 *    epilogue (pure_torch_mlx/model.py:260, 341).  Both or neither; dtype of x; [T,d_out]/[d_out].
 *  - idx_out/gates_out/c_out: per-token routing results for inspection:
 *    expert indices [T, top_k] (descending score), gate weights [T, top_k] and the
 *    coefficient vector c[T, r1] = sum_k gate_k * U_expert[idx_k] (times 1/rms on the
 *    tensor-core path, see tmoe_in_core). */
typedef struct tmoe_extras {
  const void *residual;
  const void *layer_scale;
  int32_t *idx_out;
  float *gates_out;
  float *c_out;
  const void *silu_gate; /* [T, d_out], dtype of x: y = silu(silu_gate) * (acc @ U_out + bias), the FFN's
                            silu(gate) * up (pure_torch_mlx/model.py:338-340) fused into the `up` layer;
                            applied before the residual epilogue */
  int32_t pre_norm;      /* 1: the callers' RMSNorm of x (norm_out_proj / norm_ffn, model.py:258, 337) is applied
                            inside the in-projection kernel.  `prepared` must then come from
                            tmoe_prepare_factors_prenorm (the norm weight is folded into it).  Tensor-core path with
                            the in-kernel router only (n_experts <= 256, top_k <= 8, r3 <= 256); other
                            combinations return TMOE_ERR_UNSUPPORTED -- use tmoe_rms_norm in front instead. */
  float pre_norm_eps;    /* epsilon of that RMSNorm */
  int32_t n_peer_y;      /* 0 .. TMOE_MAX_PEERS.  Tensor-core path only (TMOE_ERR_UNSUPPORTED elsewhere): the out-projection
                            stores every finished output tile to y AND to peer_y[i], i < n_peer_y, each a [T, d_out]
                            row-major buffer of x's dtype, 16-byte aligned, with rows d_out elements apart -- typically
                            this rank's rows inside the result buffers of the other GPUs (tmoe_peer_open), so that the
                            all-gather of y leaves the GPU tile by tile from inside the GEMM; no reference counterpart */
  int32_t reserved0;
  void *peer_y[7];
} tmoe_extras_t;
#define TMOE_MAX_PEERS 7

/* ABI version of the loaded library (== TMOE_ABI_VERSION of the header it was built from). */
int tmoe_version(void);

/* Static, human-readable text for a status code. */
const char *tmoe_status_string(int status);

/* Path that tmoe_forward would run for T tokens when asked for `path` (for TMOE_PATH_AUTO one of
 * SIMT / TENSOR / DECODE), or a negative status for an invalid layer or an uncovered request. */
int tmoe_resolve_path(const tmoe_layer_t *layer, int64_t T, int path);

/* Bytes of the re-laid-out factor set used by the tensor-core path (0 when the layer's
 * shape/dtype is not covered by it), or a negative status. */
int64_t tmoe_prepared_bytes(const tmoe_layer_t *layer);

/* Re-layout of the factors for the tensor-core path: K-major bf16 copies of U_in, the router
 * weight, the core (slices interleaved per r2 tile) and U_out, plus fp32 copies of
 * inner_norm_w, U_expert and bias.  One-time cost per set of parameter values, the analogue
 * of loading a checkpoint into the module (pure_torch_mlx/weights.py:74-81).  `prepared`
 * must be 256-byte aligned and tmoe_prepared_bytes() large. */
int tmoe_prepare_factors(const tmoe_layer_t *layer, const tmoe_factors_t *factors, void *prepared,
                         int64_t prepared_bytes, void *stream);

/* Same re-layout with the callers' pre-norm weight ([d_in], layer dtype) folded into the U_in and router copies:
 * RMSNorm(x) @ W = (x @ (diag(w) W)) / rms(x), so a forward with tmoe_extras_t.pre_norm = 1 only has to find
 * 1/rms(x) per row, which it does from the x tiles on their way through shared memory. */
int tmoe_prepare_factors_prenorm(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *pre_norm_w,
                                 void *prepared, int64_t prepared_bytes, void *stream);

/* Bytes of scratch that tmoe_forward / tmoe_router / tmoe_in_core / tmoe_out need for T
 * tokens on `path`, or a negative status.  The workspace must be 256-byte aligned.  Its first 256 bytes hold
 * device status words and the 4096 bytes after them hold flags and counters that the kernels of one forward hand
 * to one another and leave cleared or superseded: zero the whole workspace once after allocation (stale non-zero
 * words there can release a waiting CTA early).  A workspace serves one forward at a time: calls that may overlap
 * on the GPU (different streams) need a workspace each.  T is limited to 2^30 tokens. */
int64_t tmoe_workspace_bytes(const tmoe_layer_t *layer, int64_t T, int path);

/* Router: scores = x @ router_w^T, top-k of the raw scores, softmax over the k winners
 * (pure_torch_mlx/model.py:75-77), and c = sum_k gate_k * U_expert[idx_k] (the gather of
 * model.py:93 folded through the linear core mixing of model.py:95-98).
 * Outputs (device): idx [T, top_k] int32, gates [T, top_k] fp32, c [T, r1] fp32. */
int tmoe_router(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *x, int64_t T,
                int32_t *idx, float *gates, float *c, void *workspace, int64_t workspace_bytes,
                void *stream);

/* In-projection, inner RMSNorm and core contraction:
 * h = RMSNorm(x @ U_in) (model.py:80-81), z[t] = sum_a c[t,a] * (h[t] @ core[a]) which equals
 * the per-expert accumulation of model.py:90-98.
 * SIMT path: c is read, z is fp32 [T, r2].  Tensor-core path (needs `prepared`): c is read,
 * the row's 1/rms is folded into the coefficients instead of into h, z is bf16 [T, r2]. */
int tmoe_in_core(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *prepared,
                 const void *x, int64_t T, const float *c, void *z, void *workspace,
                 int64_t workspace_bytes, int path, void *stream);

/* Out-projection: y = z @ U_out + bias (model.py:101), optionally
 * y = residual + layer_scale * (...) (model.py:260, 341).  z as written by tmoe_in_core on the
 * same path; y has the layer dtype, [T, d_out]. */
int tmoe_out(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *prepared,
             const void *z, int64_t T, void *y, const tmoe_extras_t *extras, void *workspace,
             int64_t workspace_bytes, int path, void *stream);

/* The whole forward of TuckerMoE.forward (pure_torch_mlx/model.py:68-102) on one stream:
 * x [T, d_in] -> y [T, d_out].  `prepared` may be NULL when the resolved path is SIMT.
 * The stage entry points above serve SIMT and TENSOR; for them AUTO never resolves to DECODE (TENSOR when the shape is
 * covered, else SIMT).
 * T == 0 is valid and enqueues nothing. */
int tmoe_forward(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *prepared,
                 const void *x, int64_t T, void *y, const tmoe_extras_t *extras, void *workspace,
                 int64_t workspace_bytes, int path, void *stream);

/* The gate and up projections of the reference's feed-forward block on one input (pure_torch_mlx/model.py:337-340):
 *     act = silu(ffn_gate(x_f)) * ffn_up(x_f),      x_f = x, or RMSNorm(x) with extras->pre_norm as in tmoe_forward,
 * for two layers of the same sizes (`layer`), given by their prepared factor sets.  Tensor-core path with the in-kernel
 * router only (bf16, n_experts <= 256, top_k <= 8, r3 <= 256; TMOE_ERR_UNSUPPORTED otherwise -- use two tmoe_forward
 * calls).  Three launches instead of four: the two layers' in-projection / core stages run as ONE launch whose CTAs
 * alternate between the layers, so each tile of x comes from HBM once; then the gate layer's out-projection into `gate_y`
 * ([T, d_out], caller-provided scratch) and the up layer's with silu(gate) * up in its epilogue into `act_y`.  Results are
 * bit-identical to tmoe_forward(gate) followed by tmoe_forward(up, extras.silu_gate = gate_y).
 * `workspace`: 2 * tmoe_workspace_bytes(layer, T, TMOE_PATH_TENSOR) bytes (rounded up to 256 each).  Of `extras` only
 * pre_norm / pre_norm_eps apply (both prepared sets then come from tmoe_prepare_factors_prenorm with the same weight). */
int tmoe_ffn_gate_up(const tmoe_layer_t *layer, const void *prepared_gate, const void *prepared_up, const void *x, int64_t T,
                     void *gate_y, void *act_y, const tmoe_extras_t *extras, void *workspace, int64_t workspace_bytes,
                     void *stream);

/* RMSNorm of typed rows: y[t] = x[t] / sqrt(mean(x[t]^2) + eps) * weight (pure_torch_mlx/model.py:25-27),
 * the callers' pre-norms in front of the layer (model.py:258, 337).  x, weight, y of `dtype`; d % 8 == 0;
 * fp32 arithmetic with one rounding to the storage type.  y may equal x. */
int tmoe_rms_norm(int dtype, const void *x, const void *weight, float eps, int64_t T, int32_t d, void *y,
                  void *stream);

/* Synchronises `stream`, reads the workspace's device status word into *device_status
 * (0, or TMOE_ERR_DEVICE_WAIT with details in the following words) and clears it. */
int tmoe_read_device_status(void *workspace, int32_t *device_status, void *stream);

/* Forward on the CUDA-core kernels with NO caller-provided workspace and no allocation of any kind.
 * (This entry point has no counterpart in the reference; it exists for hosts that cannot allocate.)
 * For callers that cannot call cudaMalloc when the layer runs -- a server whose arena already owns all
 * device memory, or a decode loop that cannot afford the device-wide synchronisation an allocation
 * implies -- the scratch lives in a fixed array of TMOE_STATIC_SCRATCH_BYTES inside the library, held by
 * every GPU that loads it until the process exits.
 *  - same arguments and results as tmoe_forward(..., path = TMOE_PATH_SIMT) minus workspace/prepared;
 *  - returns TMOE_ERR_WORKSPACE when tmoe_workspace_bytes(layer, T, TMOE_PATH_SIMT) exceeds
 *    TMOE_STATIC_SCRATCH_BYTES (T is then too large for the array; size a call with tmoe_workspace_bytes, which
 *    gives about 4 * (r3 + r2) bytes per token: some 800 tokens for r3 = 256, r2 = 1024 and some 370 for r3 = 512,
 *    r2 = 2048);
 *  - arguments are validated as by tmoe_forward before anything is enqueued, also when T == 0;
 *  - the first call on each device looks the array's device address up (a one-time host-side step);
 *    make that first call outside of any stream capture;
 *  - all calls on a device share the one array: two calls whose kernels overlap on the GPU (different
 *    streams, or different host threads on different streams) race.  Serialise them on one stream. */
#define TMOE_STATIC_SCRATCH_BYTES (4u << 20)
int tmoe_forward_static_scratch(const tmoe_layer_t *layer, const tmoe_factors_t *factors, const void *x,
                                int64_t T, void *y, const tmoe_extras_t *extras, void *stream);

/* Self-test of the bounded-wait reporting: launches one small CTA that waits on an mbarrier nobody arrives on, with a
 * limit of `limit_cycles` SM clock cycles (clamped to [1e4, 2e8], i.e. at most ~0.1 s) instead of the production
 * second.  The kernel gives up by itself, writes {TMOE_ERR_DEVICE_WAIT, kernel id 9, tag 42, block 0} to the
 * workspace's status words and exits; nothing is ever left waiting.  Read the words back with
 * tmoe_read_device_status.  No reference counterpart. */
int tmoe_selftest_bounded_wait(void *workspace, int64_t limit_cycles, void *stream);

/* Number of kernels the library has launched in this process (monotonic counter). */
int64_t tmoe_launch_count(void);

/* Scheduling detail of tmoe_forward on the tensor-core path, for diagnostics.  With TMOE_HANDOFF=1 in the environment, a
 * call with more 128-token tiles than the device has SMs does not make the out-projection wait for the whole
 * in-projection/core kernel: its CTAs start on the SMs that kernel's last, partial wave of token tiles leaves free and
 * take the token tiles that are already finished.  Writes the number of such SMs (0: the hand-over is not used for this
 * call) and the number of token tiles of the waves before the last.  No reference counterpart. */
int tmoe_handoff_plan(const tmoe_layer_t *layer, int64_t T, int32_t *n_early_sms, int32_t *n_token_tiles);

/* ---- Peer buffers: the all-gather of y across the GPUs of one node (one process per GPU) -------------------------
 * No reference counterpart (the reference runs on one device).  Every rank allocates its [n_tokens, d_out] result
 * buffer with tmoe_peer_alloc, the ranks exchange the 64-byte handles through any host channel, each rank opens the
 * other ranks' buffers with tmoe_peer_open, and after the layer has written a token block into the rank's own buffer
 * tmoe_peer_push copies that block to the same offset of every peer buffer with the copy engines over NVLink (no SM is
 * used, so the copies run beside the kernels of the next token block).  Ordering across ranks (every push has landed;
 * nobody still reads the previous contents) is the caller's: mamba_tuckermoe_b200/sharding.py brackets the pushes
 * with two one-element NCCL all-reduces.  These four are the only entry points that allocate or map device memory. */
#define TMOE_PEER_HANDLE_BYTES 64
/* cudaMalloc of `bytes` (rounded up to 2 MiB) on the current device + its inter-process handle. */
int tmoe_peer_alloc(int64_t bytes, void **device_ptr, unsigned char handle[TMOE_PEER_HANDLE_BYTES]);
/* Maps another process's tmoe_peer_alloc buffer (any GPU of the node that the current device can reach over NVLink /
 * PCIe peer access) into this process; *device_ptr is its base. */
int tmoe_peer_open(const unsigned char handle[TMOE_PEER_HANDLE_BYTES], void **device_ptr);
int tmoe_peer_close(void *device_ptr);   /* unmaps a tmoe_peer_open pointer   */
int tmoe_peer_free(void *device_ptr);    /* frees a tmoe_peer_alloc pointer; synchronises the device */
/* Enqueues, for i < n_dst, one device-to-device copy of `bytes` bytes from src to dst[i] on streams[i] (cudaStream_t as
 * void*; the same stream may be given more than once).  Neither waits for nor signals anything else. */
int tmoe_peer_push(void *const *dst, int32_t n_dst, const void *src, int64_t bytes, void *const *streams);

#ifdef __cplusplus
}
#endif
#endif /* TMOE_B200_H_ */
