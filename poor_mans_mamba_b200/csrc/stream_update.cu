// Updates of the residual stream that are no mixer and no feed-forward.
//
// token_gated_update (a block per TOK tokens): a per-token input enters the stream through a small gated
// bottleneck,
//   x = h + sa * a + sb * b                      the stream with its waiting branches folded in
//   g = gelu_tanh(Wg x) * e[token]               Wg [R, D]; e the token's R entries of a table row
//   y = Wp g                                     Wp [D, R], given transposed: Wp^T [R, D]
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

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
  const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

// VEC: D and R are multiples of 4 and every row starts on a 16-byte boundary; rows are then read four entries
// at a time, and every thread keeps four neighbouring columns of y for the block's tokens in registers while it
// walks the rows of Wp^T (read coalesced, once for the block's tokens).
template <typename S, int TOK, bool VEC>
__global__ void __launch_bounds__(kSideThreads)
    token_gated_update_kernel(float* __restrict__ h, const S* __restrict__ a, float sa, const S* __restrict__ b, float sb,
                              const int* __restrict__ tokens, const S* __restrict__ table, long long ld_table, int col0,
                              const S* __restrict__ w_gate, const S* __restrict__ w_proj_t, const float* __restrict__ norm_w,
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
  // x = h + sa * a + sb * b; the rows of a short last block that have no token are zero
  if (VEC) {
    const int per_row = D >> 2;
    for (int idx = threadIdx.x; idx < TOK * per_row; idx += kSideThreads) {
      const int r = idx / per_row, i = (idx - r * per_row) << 2;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r < nt) {
        const size_t at = static_cast<size_t>(t0 + r) * D + i;
        v = ld4(h + at);
        if (a) {
          const float4 u = ld4(a + at);
          v.x += sa * u.x, v.y += sa * u.y, v.z += sa * u.z, v.w += sa * u.w;
        }
        if (b) {
          const float4 u = ld4(b + at);
          v.x += sb * u.x, v.y += sb * u.y, v.z += sb * u.z, v.w += sb * u.w;
        }
      }
      *reinterpret_cast<float4*>(xs + r * D + i) = v;
    }
  } else {
    for (int r = 0; r < TOK; ++r) {
      const size_t row = static_cast<size_t>(t0 + r) * D;
      for (int i = threadIdx.x; i < D; i += kSideThreads) {
        float v = 0.f;
        if (r < nt) {
          v = h[row + i];
          if (a) v += sa * ldf(a + row + i);
          if (b) v += sb * ldf(b + row + i);
        }
        xs[r * D + i] = v;
      }
    }
  }
  __syncthreads();
  // g[r][j] = gelu(Wg[j] . x_r) * e_r[j]: a warp per row of Wg, read once for the block's tokens
  for (int j = warp; j < R; j += kSideThreads / 32) {
    const S* wr = w_gate + static_cast<size_t>(j) * D;
    float acc[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) acc[r] = 0.f;
    if (VEC) {
      for (int i = lane << 2; i < D; i += 128) {
        const float4 w = ld4(wr + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) {
          const float4 x = *reinterpret_cast<const float4*>(xs + r * D + i);
          acc[r] += w.x * x.x + w.y * x.y + w.z * x.z + w.w * x.w;
        }
      }
    } else {
      for (int i = lane; i < D; i += 32) {
        const float wv = ldf(wr + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) acc[r] += wv * xs[r * D + i];
      }
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r) {
      const float sum = warp_sum(acc[r]);
      if (lane == 0) {
        float g = 0.f;
        if (r < nt)
          g = gelu_tanh_f(sum) * ldf(table + static_cast<long long>(tokens[t0 + r]) * ld_table + col0 + j);
        gs[r * R + j] = g;
      }
    }
  }
  __syncthreads();
  // y[r][i] = sum_j Wp^T[j][i] g_r[j]
  float sq[TOK];
#pragma unroll
  for (int r = 0; r < TOK; ++r) sq[r] = 0.f;
  if (VEC) {
    for (int i = threadIdx.x << 2; i < D; i += kSideThreads * 4) {
      float4 acc[TOK];
#pragma unroll
      for (int r = 0; r < TOK; ++r) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < R; j += 4) {
        float4 w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) w[k] = ld4(w_proj_t + static_cast<size_t>(j + k) * D + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) {
          const float4 g = *reinterpret_cast<const float4*>(gs + r * R + j);
          acc[r].x += w[0].x * g.x + w[1].x * g.y + w[2].x * g.z + w[3].x * g.w;
          acc[r].y += w[0].y * g.x + w[1].y * g.y + w[2].y * g.z + w[3].y * g.w;
          acc[r].z += w[0].z * g.x + w[1].z * g.y + w[2].z * g.z + w[3].z * g.w;
          acc[r].w += w[0].w * g.x + w[1].w * g.y + w[2].w * g.z + w[3].w * g.w;
        }
      }
#pragma unroll
      for (int r = 0; r < TOK; ++r) {
        *reinterpret_cast<float4*>(ys + r * D + i) = acc[r];
        sq[r] += acc[r].x * acc[r].x + acc[r].y * acc[r].y + acc[r].z * acc[r].z + acc[r].w * acc[r].w;
      }
    }
  } else {
    for (int i = threadIdx.x; i < D; i += kSideThreads) {
      float acc[TOK];
#pragma unroll
      for (int r = 0; r < TOK; ++r) acc[r] = 0.f;
      for (int j = 0; j < R; ++j) {
        const float wv = ldf(w_proj_t + static_cast<size_t>(j) * D + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) acc[r] += wv * gs[r * R + j];
      }
#pragma unroll
      for (int r = 0; r < TOK; ++r) {
        ys[r * D + i] = acc[r];
        sq[r] += acc[r] * acc[r];
      }
    }
  }
  float inv[TOK];
#pragma unroll
  for (int r = 0; r < TOK; ++r)  // (block_sum syncs the block)
    inv[r] = 1.f / sqrtf(block_sum(sq[r], red) / static_cast<float>(D) + eps);
#pragma unroll
  for (int r = 0; r < TOK; ++r) {
    if (r >= nt) continue;
    const size_t row = static_cast<size_t>(t0 + r) * D;
    if (VEC) {
      for (int i = threadIdx.x << 2; i < D; i += kSideThreads * 4) {
        const float4 x = *reinterpret_cast<const float4*>(xs + r * D + i);
        const float4 y = *reinterpret_cast<const float4*>(ys + r * D + i);
        const float4 w = ld4(norm_w + i);
        *reinterpret_cast<float4*>(h + row + i) =
            make_float4(x.x + y.x * inv[r] * w.x, x.y + y.y * inv[r] * w.y, x.z + y.z * inv[r] * w.z, x.w + y.w * inv[r] * w.w);
      }
    } else {
      for (int i = threadIdx.x; i < D; i += kSideThreads) h[row + i] = xs[r * D + i] + ys[r * D + i] * inv[r] * norm_w[i];
    }
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

template <typename S, int TOK, bool VEC>
int launch_token_gated_update(float* h, const void* a, float sa, const void* b, float sb, const int* tokens,
                              const void* table, long long ld_table, int col0, const void* w_gate, const void* w_proj,
                              const float* norm_w, float eps, int T, int D, int R, cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>(2) * TOK * D + static_cast<size_t>(TOK) * R) * sizeof(float);
  auto kern = token_gated_update_kernel<S, TOK, VEC>;
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
  auto aligned = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = D % 4 == 0 && R % 4 == 0 && aligned(h) && aligned(a) && aligned(b) && aligned(w_gate) &&
                   aligned(w_proj) && aligned(norm_w);
#define PMM_SIDE_LAUNCH(TOK, VEC)                                                                                     \
  return pmm::launch_token_gated_update<S, TOK, VEC>(h, a, sa, b, sb, tokens, table, ld_table, col0, w_gate, w_proj, \
                                                     norm_w, eps, T, D, R, stream)
  PMM_DISPATCH_DTYPE(dtype, S, {
    if (four && vec) PMM_SIDE_LAUNCH(4, true);
    if (four) PMM_SIDE_LAUNCH(4, false);
    if (vec) PMM_SIDE_LAUNCH(1, true);
    PMM_SIDE_LAUNCH(1, false);
  });
#undef PMM_SIDE_LAUNCH
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
