// Updates of the residual stream that are no mixer and no feed-forward.
//
// token_gated_update (a block per TOK tokens): a per-token input enters the stream through a small gated
// bottleneck,
//   x = h + sa * a + sb * b                      the stream with its waiting branches folded in
//   g = gelu_tanh(Wg x) * e[token]               Wg [R, D]; e the token's R entries of a table row
//   y = Wp g                                     Wp [D, R]
//   h = x + y / sqrt(mean(y^2) + eps) * w
// The stream, the fold, the products' sums, the activation, the root mean square and the final sum are
// float in both storage types; the matrices and the table are read in the storage type.
//
// cast_rows: out[t, :D] (storage type, row stride ld) = h[t] (+ waiting branches, which are folded into h
// as well): the stream as an operand of a matrix product.
//
// relu_squared: out = max(x, 0)^2, element-wise.
#include "common.cuh"

namespace pmm {

__device__ __forceinline__ float gelu_tanh_f(float z) {
  const float c = 0.7978845608028654f;  // sqrt(2 / pi)
  return 0.5f * z * (1.f + tanhf(c * (z + 0.044715f * z * z * z)));
}

constexpr int kSideThreads = 256;

template <typename S, int TOK>
__global__ void __launch_bounds__(kSideThreads)
    token_gated_update_kernel(float* __restrict__ h, const S* __restrict__ a, float sa, const S* __restrict__ b, float sb,
                              const int* __restrict__ tokens, const S* __restrict__ table, long long ld_table, int col0,
                              const S* __restrict__ w_gate, const S* __restrict__ w_proj, const float* __restrict__ norm_w,
                              float eps, int T, int D, int R) {
  extern __shared__ __align__(16) float side_smem[];  // x [TOK][D] | y [TOK][D] | g [TOK][R]
  __shared__ float red[32];
  float* xs = side_smem;
  float* ys = xs + static_cast<size_t>(TOK) * D;
  float* gs = ys + static_cast<size_t>(TOK) * D;
  pdl_launch_dependents();
  pdl_wait();
  const int t0 = blockIdx.x * TOK;
  const int nt = min(TOK, T - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int r = 0; r < nt; ++r) {
    const size_t row = static_cast<size_t>(t0 + r) * D;
    for (int i = threadIdx.x; i < D; i += kSideThreads) {
      float v = h[row + i];
      if (a) v += sa * ldf(a + row + i);
      if (b) v += sb * ldf(b + row + i);
      xs[r * D + i] = v;
    }
  }
  __syncthreads();
  // g[r][j] = gelu(Wg[j] . x_r) * e_r[j]: a warp per row of Wg, read once for the block's tokens
  for (int j = warp; j < R; j += kSideThreads / 32) {
    const S* wr = w_gate + static_cast<size_t>(j) * D;
    float acc[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) acc[r] = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float wv = ldf(wr + i);
#pragma unroll
      for (int r = 0; r < TOK; ++r)
        if (r < nt) acc[r] += wv * xs[r * D + i];
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r) {
      const float sum = warp_sum(acc[r]);
      if (lane == 0 && r < nt) {
        const float e = ldf(table + static_cast<long long>(tokens[t0 + r]) * ld_table + col0 + j);
        gs[r * R + j] = gelu_tanh_f(sum) * e;
      }
    }
  }
  __syncthreads();
  // y[r][i] = Wp[i] . g_r: a thread per row of Wp
  float sq[TOK];
#pragma unroll
  for (int r = 0; r < TOK; ++r) sq[r] = 0.f;
  for (int i = threadIdx.x; i < D; i += kSideThreads) {
    const S* wr = w_proj + static_cast<size_t>(i) * R;
    float acc[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) acc[r] = 0.f;
    for (int j = 0; j < R; ++j) {
      const float wv = ldf(wr + j);
#pragma unroll
      for (int r = 0; r < TOK; ++r)
        if (r < nt) acc[r] += wv * gs[r * R + j];
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r)
      if (r < nt) {
        ys[r * D + i] = acc[r];
        sq[r] += acc[r] * acc[r];
      }
  }
#pragma unroll
  for (int r = 0; r < TOK; ++r) {
    const float total = block_sum(sq[r], red);  // (syncs the block)
    if (r >= nt) continue;
    const float inv = 1.f / sqrtf(total / static_cast<float>(D) + eps);
    const size_t row = static_cast<size_t>(t0 + r) * D;
    for (int i = threadIdx.x; i < D; i += kSideThreads) h[row + i] = xs[r * D + i] + ys[r * D + i] * inv * norm_w[i];
  }
}

template <typename S>
__global__ void __launch_bounds__(256)
    cast_rows_kernel(float* __restrict__ h, const S* __restrict__ a, float sa, const S* __restrict__ b, float sb,
                     S* __restrict__ out, long long ld_out, int D) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const size_t row = static_cast<size_t>(t) * D;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < D; i += gridDim.y * blockDim.x) {
    float v = h[row + i];
    if (a || b) {
      if (a) v += sa * ldf(a + row + i);
      if (b) v += sb * ldf(b + row + i);
      h[row + i] = v;
    }
    stf(out + static_cast<long long>(t) * ld_out + i, v);
  }
}

template <typename S>
__global__ void __launch_bounds__(256)
    relu_squared_kernel(const S* __restrict__ x, long long ld_x, S* __restrict__ out, long long ld_out, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < F; i += gridDim.y * blockDim.x) {
    const float v = fmaxf(ldf(x + static_cast<long long>(t) * ld_x + i), 0.f);
    stf(out + static_cast<long long>(t) * ld_out + i, v * v);
  }
}

template <typename S, int TOK>
int launch_token_gated_update(float* h, const void* a, float sa, const void* b, float sb, const int* tokens,
                              const void* table, long long ld_table, int col0, const void* w_gate, const void* w_proj,
                              const float* norm_w, float eps, int T, int D, int R, cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>(2) * TOK * D + static_cast<size_t>(TOK) * R) * sizeof(float);
  auto kern = token_gated_update_kernel<S, TOK>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  launch_pdl(kern, dim3((T + TOK - 1) / TOK), dim3(kSideThreads), smem, stream, h, static_cast<const S*>(a), sa,
             static_cast<const S*>(b), sb, tokens, static_cast<const S*>(table), ld_table, col0,
             static_cast<const S*>(w_gate), static_cast<const S*>(w_proj), norm_w, eps, T, D, R);
  return launch_status();
}

}  // namespace pmm

// How many floats of shared memory a block of `tok` tokens needs; the launcher takes 4 tokens a block where
// the step has many tokens and they fit, else 1.
PMM_EXPORT int pmm_token_gated_update_fits(int D, int R) {
  return (static_cast<size_t>(2) * D + R) * sizeof(float) <= 200 * 1024 ? 1 : 0;
}

PMM_EXPORT int pmm_token_gated_update(float* h, const void* a, float sa, const void* b, float sb, const int* tokens,
                                      const void* table, long long ld_table, int col0, const void* w_gate,
                                      const void* w_proj, const float* norm_w, float eps, int T, int D, int R, int dtype,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || R <= 0 || col0 < 0 || !pmm_token_gated_update_fits(D, R)) return PMM_ERR_BAD_ARGUMENT;
  const bool four = T >= 1024 && (static_cast<size_t>(8) * D + 4 * static_cast<size_t>(R)) * sizeof(float) <= 200 * 1024;
  PMM_DISPATCH_DTYPE(dtype, S, {
    if (four)
      return pmm::launch_token_gated_update<S, 4>(h, a, sa, b, sb, tokens, table, ld_table, col0, w_gate, w_proj, norm_w,
                                                  eps, T, D, R, stream);
    return pmm::launch_token_gated_update<S, 1>(h, a, sa, b, sb, tokens, table, ld_table, col0, w_gate, w_proj, norm_w, eps,
                                                T, D, R, stream);
  });
  return 0;
}

PMM_EXPORT int pmm_cast_rows(float* h, const void* a, float sa, const void* b, float sb, void* out, long long ld_out, int T,
                             int D, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (D + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::cast_rows_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream, h,
                                               static_cast<const S*>(a), sa, static_cast<const S*>(b), sb,
                                               static_cast<S*>(out), ld_out, D));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_relu_squared(const void* x, long long ld_x, void* out, long long ld_out, int T, int F, int dtype,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (F + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::relu_squared_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream,
                                               static_cast<const S*>(x), ld_x, static_cast<S*>(out), ld_out, F));
  return pmm::launch_status();
}
