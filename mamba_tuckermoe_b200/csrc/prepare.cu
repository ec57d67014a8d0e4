// Factor re-layout for the tensor-core path.
//
// tcgen05.mma reads both operands from shared memory as K-major tiles (the contraction index
// is the contiguous one).  The reference stores U_in [d_in, r3], core [r1, r3, r2] and
// U_out [r2, d_out] with the contraction index outermost (pure_torch_mlx/model.py:61-65), so
// each is transposed once into a bf16 buffer the TMA unit can tile directly:
//   uin_t  [r3, d_in]            uin_t[n][k]  = U_in[k][n]
//   wr_b   [e_pad, d_in]         router_w rows, zero rows up to a multiple of 16
//   g_t    [r1*r2, r3]           row (j*r1 + a)*n2 + s = core[a][:, j*n2 + s]: the r1 slices of one
//                                r2 tile (n2 = 256/r1 columns) are adjacent, so one N=256 MMA
//                                produces every slice of that tile in one TMEM accumulator
//   uout_t [d_out, r2]           uout_t[n][k] = U_out[k][n]
// plus fp32 copies of inner_norm_w, bias and U_expert.
#include "common.cuh"
#include "kernels.h"

namespace tmoe {

// Shapes the prepared (K-major bf16) factor layout and the decode kernels handle.
bool prepared_covers(const tmoe_layer_t &L) {
  if (L.dtype != TMOE_BF16) return false;
  if (!(L.r1 == 2 || L.r1 == 4 || L.r1 == 8 || L.r1 == 16 || L.r1 == 32)) return false;
  if (L.r3 % 64 != 0 || L.r3 > 512 || (L.r3 > 256 && L.r3 % 256 != 0)) return false;
  if (L.d_in % 64 != 0 || L.r2 % 64 != 0) return false;
  if (L.r2 % (256 / L.r1) != 0) return false;
  if (L.d_out % 8 != 0) return false;
  return true;
}

// Shapes the tcgen05 kernels handle: every prepared shape (a slice of the 256-column accumulator has 256 / r1 >= 8
// columns; the epilogue reads 16 columns per load, two adjacent slices at r1 = 32).
bool tensor_path_covers(const tmoe_layer_t &L) { return prepared_covers(L); }

PreparedLayout prepared_layout(const tmoe_layer_t &L) {
  PreparedLayout P{};
  P.e_pad = (int)align_up(L.n_experts, 16);
  P.n2 = 256 / L.r1;
  P.n_tiles2 = L.r2 / P.n2;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = align_up(off + bytes, 1024); return o; };
  P.uin_t = take((int64_t)L.r3 * L.d_in * 2);
  P.wr_b = take((int64_t)P.e_pad * L.d_in * 2);
  P.g_t = take((int64_t)L.r1 * L.r2 * L.r3 * 2);
  P.uout_t = take((int64_t)L.d_out * L.r2 * 2);
  P.normw = take((int64_t)L.r3 * 4);
  P.bias = take((int64_t)L.d_out * 4);
  P.uexp = take((int64_t)L.n_experts * L.r1 * 4);
  P.total = off;
  return P;
}

// `kscale` (optional, [K]): a weight per contraction index folded into the copy -- the callers' pre-norm weight,
// so that RMSNorm(x) @ W becomes (x @ (diag(w_pre) W)) / rms(x) and only the per-row 1/rms is left for the kernel.
template <typename T>
__global__ void transpose_to_bf16_kernel(const T *__restrict__ src, bf16 *__restrict__ dst, int K, int N,
                                         const T *__restrict__ kscale) {
  // src [K, N] -> dst [N, K]; 32x32 tiles through shared memory
  __shared__ float tile[32][33];
  const int k0 = blockIdx.y * 32, n0 = blockIdx.x * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int k = k0 + i, n = n0 + threadIdx.x;
    tile[i][threadIdx.x] = (k < K && n < N) ? to_f32(src[(int64_t)k * N + n]) * (kscale ? to_f32(kscale[k]) : 1.f) : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    int n = n0 + i, k = k0 + threadIdx.x;
    if (n < N && k < K) dst[(int64_t)n * K + k] = __float2bfloat16_rn(tile[threadIdx.x][i]);
  }
}

template <typename T>
__global__ void router_rows_kernel(const T *__restrict__ wr, bf16 *__restrict__ dst, int E, int e_pad, int d_in,
                                   const T *__restrict__ kscale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t total = (int64_t)e_pad * d_in;
  if (i >= total) return;
  int e = (int)(i / d_in);
  const float sc = kscale ? to_f32(kscale[i - (int64_t)e * d_in]) : 1.f;
  dst[i] = (e < E) ? __float2bfloat16_rn(to_f32(wr[i]) * sc) : __float2bfloat16_rn(0.f);
}

template <typename T>
__global__ void core_tiles_kernel(const T *__restrict__ core, bf16 *__restrict__ dst, int r1, int r3, int r2, int n2) {
  // dst row = (j*r1 + a)*n2 + s, col = r ; source core[a][r][j*n2 + s]
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // enumerates (row, r) with s fastest inside a warp
  int64_t total = (int64_t)r1 * r2 * r3;
  if (i >= total) return;
  // choose the enumeration so that reads are coalesced: i = ((j*r1 + a)*r3 + r)*n2 + s
  int s = (int)(i % n2);
  int64_t q = i / n2;
  int r = (int)(q % r3);
  q /= r3;
  int a = (int)(q % r1);
  int j = (int)(q / r1);
  int64_t row = ((int64_t)j * r1 + a) * n2 + s;
  dst[row * r3 + r] = __float2bfloat16_rn(to_f32(core[((int64_t)a * r3 + r) * r2 + (int64_t)j * n2 + s]));
}

template <typename T>
__global__ void to_f32_kernel(const T *__restrict__ src, float *__restrict__ dst, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = to_f32(src[i]);
}

template <typename T>
static int prepare_t(const tmoe_layer_t &L, const tmoe_factors_t &F, const void *pre_w, void *prepared, cudaStream_t st) {
  PreparedLayout P = prepared_layout(L);
  char *base = reinterpret_cast<char *>(prepared);
  dim3 tb(32, 8);
  transpose_to_bf16_kernel<T><<<dim3((L.r3 + 31) / 32, (L.d_in + 31) / 32), tb, 0, st>>>(
      (const T *)F.U_in, (bf16 *)(base + P.uin_t), L.d_in, L.r3, (const T *)pre_w);
  transpose_to_bf16_kernel<T><<<dim3((L.d_out + 31) / 32, (L.r2 + 31) / 32), tb, 0, st>>>(
      (const T *)F.U_out, (bf16 *)(base + P.uout_t), L.r2, L.d_out, (const T *)nullptr);
  {
    int64_t n = (int64_t)P.e_pad * L.d_in;
    router_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const T *)F.router_w, (bf16 *)(base + P.wr_b),
                                                                      L.n_experts, P.e_pad, L.d_in, (const T *)pre_w);
  }
  {
    int64_t n = (int64_t)L.r1 * L.r2 * L.r3;
    core_tiles_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const T *)F.core, (bf16 *)(base + P.g_t), L.r1,
                                                                     L.r3, L.r2, P.n2);
  }
  to_f32_kernel<T><<<(L.r3 + 255) / 256, 256, 0, st>>>((const T *)F.inner_norm_w, (float *)(base + P.normw), L.r3);
  to_f32_kernel<T><<<(L.d_out + 255) / 256, 256, 0, st>>>((const T *)F.bias, (float *)(base + P.bias), L.d_out);
  {
    int64_t n = (int64_t)L.n_experts * L.r1;
    to_f32_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>((const T *)F.U_expert, (float *)(base + P.uexp), n);
  }
  count_launch(7);
  return launch_status();
}

int launch_prepare(const tmoe_layer_t &L, const tmoe_factors_t &F, const void *pre_norm_w, void *prepared, cudaStream_t st) {
  return L.dtype == TMOE_F32 ? prepare_t<float>(L, F, pre_norm_w, prepared, st) : prepare_t<bf16>(L, F, pre_norm_w, prepared, st);
}

}  // namespace tmoe
