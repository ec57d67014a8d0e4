// CUDA-core (fp32 FMA) contractions: the accuracy path for fp32 layers and the general-shape
// path for everything the tensor-core kernels do not cover.
//
// One tiled kernel, C[M,N] = A[M,K] * B, 64x64x16 tiles, 256 threads, 4x4 outputs per thread,
// fp32 accumulation, inputs fp32 or bf16.  It serves the four contractions of the layer
// (pure_torch_mlx/model.py:75, 80, 95-98, 101):
//   scores = x @ router_w^T                     (B stored [N,K])
//   h      = x @ U_in                           (B stored [K,N]) followed by rmsnorm_rows_kernel
//   z      = sum_a c_a * (h @ core[a])          A[t, a*r3 + r] = c[t,a] * h[t,r] is formed while the
//                                               A tile is staged; B = core viewed as [r1*r3, r2]
//   y      = z @ U_out + bias  (+ residual/layer-scale epilogue)
#include "common.cuh"
#include "kernels.h"

namespace tmoe {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

struct GemmP {
  const void *A;
  const void *B;
  int M, N, K;
  int64_t lda, ldb;
  const float *cvec;  // A_CORE only
  int r1, r3;
};

struct EpiF32 {
  float *C;
  int64_t ldc;
  __device__ __forceinline__ void operator()(int m, int n, float v) const { C[(int64_t)m * ldc + n] = v; }
};

template <typename T>
struct EpiOut {
  T *y;
  int64_t ldc;
  const T *bias;
  const T *residual;
  const T *gamma;
  const T *silu_gate;
  __device__ __forceinline__ void operator()(int m, int n, float v) const {
    if (bias) v += to_f32(bias[n]);
    if (silu_gate) {
      const float g = to_f32(silu_gate[(int64_t)m * ldc + n]);
      v *= g / (1.f + expf(-g));
    }
    if (residual) v = to_f32(residual[(int64_t)m * ldc + n]) + to_f32(gamma[n]) * v;
    y[(int64_t)m * ldc + n] = from_f32<T>(v);
  }
};

template <typename T>
__device__ __forceinline__ void load4(const T *p, float (&o)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float *p, float (&o)[4]) {
  float4 v = __ldg(reinterpret_cast<const float4 *>(p));
  o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
}
template <>
__device__ __forceinline__ void load4<bf16>(const bf16 *p, float (&o)[4]) {
  uint2 v = __ldg(reinterpret_cast<const uint2 *>(p));
  o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
  o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
}

// Requires K % 4 == 0, lda % 4 == 0, ldb % 4 == 0 and 16-byte aligned bases (checked by the callers).
template <typename TA, typename TB, bool B_NK, bool A_CORE, typename Epi>
__global__ void __launch_bounds__(256) simt_gemm_kernel(GemmP p, Epi epi) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Bs[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;   // token tiles on grid.x: no 65535 limit on them
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int a_row = tid >> 2, a_kq = (tid & 3) * 4;
  const int b_kr = tid >> 4, b_nq = (tid & 15) * 4;

  for (int k0 = 0; k0 < p.K; k0 += BK) {
    {  // stage A
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      const int m = m0 + a_row, k = k0 + a_kq;
      if (m < p.M && k < p.K) {
        if constexpr (A_CORE) {
          const int a = k / p.r3, r = k - a * p.r3;
          load4<float>(reinterpret_cast<const float *>(p.A) + (int64_t)m * p.r3 + r, v);
          const float cw = p.cvec[(int64_t)m * p.r1 + a];
#pragma unroll
          for (int i = 0; i < 4; ++i) v[i] *= cw;
        } else {
          load4<TA>(reinterpret_cast<const TA *>(p.A) + (int64_t)m * p.lda + k, v);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) As[a_kq + i][a_row] = v[i];
    }
    if constexpr (B_NK) {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      const int n = n0 + a_row, k = k0 + a_kq;
      if (n < p.N && k < p.K) load4<TB>(reinterpret_cast<const TB *>(p.B) + (int64_t)n * p.ldb + k, v);
#pragma unroll
      for (int i = 0; i < 4; ++i) Bs[a_kq + i][a_row] = v[i];
    } else {
      float v[4] = {0.f, 0.f, 0.f, 0.f};
      const int k = k0 + b_kr, n = n0 + b_nq;
      if (k < p.K && n < p.N) load4<TB>(reinterpret_cast<const TB *>(p.B) + (int64_t)k * p.ldb + n, v);
      *reinterpret_cast<float4 *>(&Bs[b_kr][b_nq]) = make_float4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      const float4 av = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      const float a[4] = {av.x, av.y, av.z, av.w};
      const float b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < p.N) epi(m, n, acc[i][j]);
    }
  }
}

// In-place inner RMSNorm of fp32 rows: h / sqrt(mean(h^2) + eps) * w (model.py:25-27).
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(float *__restrict__ h, const T *__restrict__ w, int64_t Tn,
                                                           int r3, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  float *row = h + t * r3;
  float ss = 0.f;
  for (int i = lane; i < r3; i += 32) ss = fmaf(row[i], row[i], ss);
  ss = warp_sum(ss);
  const float den = sqrtf(ss / (float)r3 + eps);
  for (int i = lane; i < r3; i += 32) row[i] = row[i] / den * to_f32(w[i]);
}

static dim3 gemm_grid(int64_t M, int N) { return dim3((unsigned)((M + BM - 1) / BM), (unsigned)((N + BN - 1) / BN)); }

template <typename T>
static int scores_t(const tmoe_layer_t &L, const void *x, const void *wr, int64_t T_, float *scores, cudaStream_t st) {
  GemmP p{x, wr, (int)T_, L.n_experts, L.d_in, L.d_in, L.d_in, nullptr, 0, 0};
  simt_gemm_kernel<T, T, true, false, EpiF32><<<gemm_grid(T_, L.n_experts), 256, 0, st>>>(p, EpiF32{scores, L.n_experts});
  count_launch();
  return launch_status();
}
int launch_simt_scores(const tmoe_layer_t &L, const void *x, const void *wr, int64_t T_, float *scores, cudaStream_t st) {
  return L.dtype == TMOE_F32 ? scores_t<float>(L, x, wr, T_, scores, st) : scores_t<bf16>(L, x, wr, T_, scores, st);
}

template <typename T>
static int inproj_t(const tmoe_layer_t &L, const void *x, const void *U_in, const void *w, int64_t T_, float *h,
                    cudaStream_t st) {
  GemmP p{x, U_in, (int)T_, L.r3, L.d_in, L.d_in, L.r3, nullptr, 0, 0};
  simt_gemm_kernel<T, T, false, false, EpiF32><<<gemm_grid(T_, L.r3), 256, 0, st>>>(p, EpiF32{h, L.r3});
  rmsnorm_rows_kernel<T><<<(unsigned)((T_ + 7) / 8), 256, 0, st>>>(h, (const T *)w, T_, L.r3, L.eps);
  count_launch(2);
  return launch_status();
}
int launch_simt_inproj_norm(const tmoe_layer_t &L, const void *x, const void *U_in, const void *w, int64_t T_, float *h,
                            cudaStream_t st) {
  return L.dtype == TMOE_F32 ? inproj_t<float>(L, x, U_in, w, T_, h, st) : inproj_t<bf16>(L, x, U_in, w, T_, h, st);
}

template <typename T>
static int core_t(const tmoe_layer_t &L, const float *h, const float *c, const void *core, int64_t T_, float *z,
                  cudaStream_t st) {
  GemmP p{h, core, (int)T_, L.r2, L.r1 * L.r3, L.r3, L.r2, c, L.r1, L.r3};
  simt_gemm_kernel<float, T, false, true, EpiF32><<<gemm_grid(T_, L.r2), 256, 0, st>>>(p, EpiF32{z, L.r2});
  count_launch();
  return launch_status();
}
int launch_simt_core(const tmoe_layer_t &L, const float *h, const float *c, const void *core, int64_t T_, float *z,
                     cudaStream_t st) {
  return L.dtype == TMOE_F32 ? core_t<float>(L, h, c, core, T_, z, st) : core_t<bf16>(L, h, c, core, T_, z, st);
}

template <typename T>
static int out_t(const tmoe_layer_t &L, const float *z, const void *U_out, const void *bias, const OutEpilogue &epi,
                 int64_t T_, void *y, cudaStream_t st) {
  GemmP p{z, U_out, (int)T_, L.d_out, L.r2, L.r2, L.d_out, nullptr, 0, 0};
  EpiOut<T> e{(T *)y, L.d_out, (const T *)bias, (const T *)epi.residual, (const T *)epi.layer_scale,
              (const T *)epi.silu_gate};
  simt_gemm_kernel<float, T, false, false, EpiOut<T>><<<gemm_grid(T_, L.d_out), 256, 0, st>>>(p, e);
  count_launch();
  return launch_status();
}
int launch_simt_out(const tmoe_layer_t &L, const float *z, const void *U_out, const void *bias, const OutEpilogue &epi,
                    int64_t T_, void *y, cudaStream_t st) {
  return L.dtype == TMOE_F32 ? out_t<float>(L, z, U_out, bias, epi, T_, y, st) : out_t<bf16>(L, z, U_out, bias, epi, T_, y, st);
}

// Stand-alone RMSNorm of typed rows (the callers' pre-norms, model.py:258, 337): one warp per row,
// 128-bit loads, the row stays in registers between the two passes when it fits.
template <typename T>
__global__ void __launch_bounds__(256) rms_norm_kernel(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ y,
                                                       int64_t Tn, int d, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= Tn) return;
  const T *xr = x + t * d;
  T *yr = y + t * d;
  float ss = 0.f;
  for (int i = lane * 4; i < d; i += 128) {
    float v[4];
    load4<T>(xr + i, v);
#pragma unroll
    for (int q = 0; q < 4; ++q) ss = fmaf(v[q], v[q], ss);
  }
  ss = warp_sum(ss);
  const float den = sqrtf(ss / (float)d + eps);
  for (int i = lane * 4; i < d; i += 128) {
    float v[4], g[4];
    load4<T>(xr + i, v);
    load4<T>(w + i, g);
#pragma unroll
    for (int q = 0; q < 4; ++q) yr[i + q] = from_f32<T>(v[q] / den * g[q]);
  }
}

int launch_rms_norm(int dtype, const void *x, const void *w, float eps, int64_t T_, int d, void *y, cudaStream_t st) {
  const unsigned grid = (unsigned)((T_ + 7) / 8);
  if (dtype == TMOE_F32) rms_norm_kernel<float><<<grid, 256, 0, st>>>((const float *)x, (const float *)w, (float *)y, T_, d, eps);
  else rms_norm_kernel<bf16><<<grid, 256, 0, st>>>((const bf16 *)x, (const bf16 *)w, (bf16 *)y, T_, d, eps);
  count_launch();
  return launch_status();
}

}  // namespace tmoe
