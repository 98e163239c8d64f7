// Embedding gather and the fused "residual add + RMSNorm" kernel.
//
// The residual stream is float in every mode.  Branch outputs (mixer / feed-forward
// results in the storage type) are folded into it by the same kernel that produces
// the next normalised activation, so the stream is read and written once per norm.
//
// Formulas: h[t] = mult * E[tok[t]]  (reference src/ops/gpu/embed.cu:5-16);
// y = x * (1/sqrt(mean(x^2)+eps)) * w  (reference src/ops/gpu/rms_norm.cu:6-26).
#include "common.cuh"

namespace pmm {

// norm_w != nullptr: the row is divided by its root mean square and multiplied by norm_w,
//   h[t] = r / sqrt(mean(r^2) + eps) * norm_w with r = mult * E[tok[t]], all in float.
template <typename S>
__global__ void embed_kernel(float* __restrict__ out, const S* __restrict__ table,
                             const int* __restrict__ tokens, float mult, int D, int V,
                             const float* __restrict__ norm_w, float eps) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = tokens[t];
  const bool ok = id >= 0 && id < V;  // the host rejects such ids before launching
  if (!ok) id = 0;
  const S* row = table + static_cast<size_t>(id) * D;
  float* o = out + static_cast<size_t>(t) * D;
  if (!norm_w) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = ok ? mult * ldf(row + i) : 0.f;
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float v = ok ? mult * ldf(row + i) : 0.f;
    ss += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(D) + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = ok ? mult * ldf(row + i) * inv * norm_w[i] : 0.f;
}

// One block per output row.  h' = (h + sa*a) + sb*b ; out = h' * rsqrt(mean(h'^2)+eps) * w.
// rows == nullptr: row r of h is updated in place and out[r] written.
// rows != nullptr: h is left untouched, out[r] is computed from row rows[r].
template <typename S>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const S* __restrict__ a, float sa,
                                   const S* __restrict__ b, float sb, const float* __restrict__ w,
                                   float eps, S* __restrict__ out, const int* __restrict__ rows,
                                   int D) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = h[src + i];
    if (a) v = v + sa * ldf(a + src + i);
    if (b) v = v + sb * ldf(b + src + i);
    buf[i] = v;
    ss += v * v;
    if (!rows && (a || b)) h[src + i] = v;
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
  S* o = out + static_cast<size_t>(r) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) stf(o + i, buf[i] * inv * w[i]);
}

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}

// The same for widths that are a multiple of 4: four elements per thread and access.
template <typename S>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const S* __restrict__ a, float sa,
                                       const S* __restrict__ b, float sb, const float* __restrict__ w,
                                       float eps, S* __restrict__ out, const int* __restrict__ rows,
                                       int D) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
    float4 v = ld4(h + src + i);
    if (a) {
      const float4 x = ld4(a + src + i);
      v.x += sa * x.x; v.y += sa * x.y; v.z += sa * x.z; v.w += sa * x.w;
    }
    if (b) {
      const float4 x = ld4(b + src + i);
      v.x += sb * x.x; v.y += sb * x.y; v.z += sb * x.z; v.w += sb * x.w;
    }
    *reinterpret_cast<float4*>(buf + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    if (!rows && (a || b)) st4(h + src + i, v);
  }
  if (!out) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
  S* o = out + static_cast<size_t>(r) * D;
  for (int i = threadIdx.x * 4; i < D; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(buf + i);
    const float4 g = ld4(w + i);
    st4(o + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
  }
}

// A sublayer's result is normed once more before it joins the stream, and the stream is normed for the
// next sublayer, in one launch (a block per row, the row kept in shared memory, float throughout):
//   s   = sa * a + sb * b
//   u   = s / sqrt(mean(s^2) + post_eps) * post_w
//   v   = h + u                      (h absent: v = u);  h = v when rows == nullptr
//   out = v / sqrt(mean(v^2) + eps) * w          (when out is given; w absent: out = v)
// rows != nullptr: h is left untouched and out[r] comes from row rows[r] of h, a and b.
template <typename S>
__global__ void add_postnorm_rmsnorm_kernel(float* __restrict__ h, const S* __restrict__ a, float sa,
                                            const S* __restrict__ b, float sb, const float* __restrict__ post_w,
                                            float post_eps, const float* __restrict__ w, float eps,
                                            S* __restrict__ out, const int* __restrict__ rows, int D) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  float ss = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = sa * ldf(a + src + i);
    if (b) s = s + sb * ldf(b + src + i);
    buf[i] = s;
    ss += s * s;
  }
  const float inv_p = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(D) + post_eps);
  float sv = 0.f;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float v = buf[i] * inv_p * post_w[i];
    if (h) {
      v = h[src + i] + v;
      if (!rows) h[src + i] = v;
    }
    buf[i] = v;
    sv += v * v;
  }
  if (!out) return;
  S* o = out + static_cast<size_t>(r) * D;
  if (!w) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) stf(o + i, buf[i]);
    return;
  }
  const float inv = 1.0f / sqrtf(block_sum(sv, red) / static_cast<float>(D) + eps);
  for (int i = threadIdx.x; i < D; i += blockDim.x) stf(o + i, buf[i] * inv * w[i]);
}

// The same for widths that are a multiple of 4: four elements per thread and access.  A thread's first P pieces
// (the launcher takes the smallest P of 1, 2, 4 that covers the row) stay in registers from the first read to the
// last write; with P = 4 pieces beyond wait in shared memory.
template <typename S, int P>
__global__ void add_postnorm_rmsnorm_vec_kernel(float* __restrict__ h, const S* __restrict__ a, float sa,
                                                const S* __restrict__ b, float sb, const float* __restrict__ post_w,
                                                float post_eps, const float* __restrict__ w, float eps,
                                                S* __restrict__ out, const int* __restrict__ rows, int D) {
  extern __shared__ float buf[];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  const int step = blockDim.x * 4;
  auto branches = [&](int i) {
    float4 s = ld4(a + src + i);
    s.x *= sa; s.y *= sa; s.z *= sa; s.w *= sa;
    if (b) {
      const float4 x = ld4(b + src + i);
      s.x += sb * x.x; s.y += sb * x.y; s.z += sb * x.z; s.w += sb * x.w;
    }
    return s;
  };
  auto sq = [](float4 v) { return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; };
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 v[P], hv[P];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < P; ++c) {
    const int i = threadIdx.x * 4 + c * step;
    v[c] = i < D ? branches(i) : zero;
    // (the stream's row is asked for before the reduction, so that its latency hides behind it)
    hv[c] = (h && i < D) ? ld4(h + src + i) : zero;
    ss += sq(v[c]);
  }
  if (P == 4) {
    for (int i = threadIdx.x * 4 + 4 * step; i < D; i += step) {
      const float4 s = branches(i);
      *reinterpret_cast<float4*>(buf + i) = s;
      ss += sq(s);
    }
  }
  const float inv_p = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(D) + post_eps);
  float sv = 0.f;
  auto join = [&](int i, float4 s, float4 x) {
    const float4 g = ld4(post_w + i);
    float4 y = make_float4(s.x * inv_p * g.x + x.x, s.y * inv_p * g.y + x.y, s.z * inv_p * g.z + x.z, s.w * inv_p * g.w + x.w);
    if (h && !rows) st4(h + src + i, y);
    sv += sq(y);
    return y;
  };
#pragma unroll
  for (int c = 0; c < P; ++c) {
    const int i = threadIdx.x * 4 + c * step;
    if (i < D) v[c] = join(i, v[c], hv[c]);
  }
  if (P == 4) {
    for (int i = threadIdx.x * 4 + 4 * step; i < D; i += step)
      *reinterpret_cast<float4*>(buf + i) = join(i, *reinterpret_cast<const float4*>(buf + i), h ? ld4(h + src + i) : zero);
  }
  if (!out) return;
  S* o = out + static_cast<size_t>(r) * D;
  float inv = 1.f;
  if (w) inv = 1.0f / sqrtf(block_sum(sv, red) / static_cast<float>(D) + eps);
  auto write = [&](int i, float4 y) {
    if (w) {
      const float4 g = ld4(w + i);
      y = make_float4(y.x * inv * g.x, y.y * inv * g.y, y.z * inv * g.z, y.w * inv * g.w);
    }
    st4(o + i, y);
  };
#pragma unroll
  for (int c = 0; c < P; ++c) {
    const int i = threadIdx.x * 4 + c * step;
    if (i < D) write(i, v[c]);
  }
  if (P == 4) {
    for (int i = threadIdx.x * 4 + 4 * step; i < D; i += step) write(i, *reinterpret_cast<const float4*>(buf + i));
  }
}

__global__ void scale_f32_kernel(float* __restrict__ x, float s, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] *= s;
}

template <typename S>
__global__ void cast_scale_kernel(float* __restrict__ out, const S* __restrict__ in, float s, size_t n) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = s * ldf(in + i);
}

}  // namespace pmm

PMM_EXPORT int pmm_embed(void* out, const void* table, const int* tokens, float mult, int T, int D,
                         int V, int dtype, const float* norm_w, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::embed_kernel<S>, dim3(T), dim3(256), 0, stream,
                                               static_cast<float*>(out), static_cast<const S*>(table), tokens,
                                               mult, D, V, norm_w, eps));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_add_rmsnorm(void* h, const void* a, float sa, const void* b, float sb,
                               const float* w, float eps, void* out, const int* rows, int R, int D,
                               int dtype, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (out && !w) return PMM_ERR_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(D) * sizeof(float);
  if (smem > 200 * 1024) return PMM_ERR_BAD_ARGUMENT;  // width beyond one block's shared memory
  const int threads = D >= 1024 ? 256 : 128;
  const bool vec = D % 4 == 0 && reinterpret_cast<uintptr_t>(h) % 16 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(b) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(w) % 16 == 0;
  PMM_DISPATCH_DTYPE(dtype, S, {
    auto kern = vec ? pmm::add_rmsnorm_vec_kernel<S> : pmm::add_rmsnorm_kernel<S>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    pmm::launch_pdl(kern, dim3(R), dim3(threads), smem, stream, static_cast<float*>(h), static_cast<const S*>(a), sa,
                    static_cast<const S*>(b), sb, w, eps, static_cast<S*>(out), rows, D);
  });
  return pmm::launch_status();
}

// h [T, D] float or nullptr; a (and b or nullptr) [T, D] storage type; post_w, w float [D]; out [R, D] storage
// type or nullptr; rows [R] or nullptr (then R = T).
PMM_EXPORT int pmm_add_postnorm_rmsnorm(void* h, const void* a, float sa, const void* b, float sb, const float* post_w,
                                        float post_eps, const float* w, float eps, void* out, const int* rows, int R,
                                        int D, int dtype, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || !a || !post_w || (rows && !out) || (!h && !out)) return PMM_ERR_BAD_ARGUMENT;
  const size_t smem = static_cast<size_t>(D) * sizeof(float);
  if (smem > 200 * 1024) return PMM_ERR_BAD_ARGUMENT;
  const int threads = D >= 1024 ? 256 : 128;
  auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = D % 4 == 0 && aligned(h) && aligned(a) && aligned(b) && aligned(out) && aligned(w) && aligned(post_w);
  PMM_DISPATCH_DTYPE(dtype, S, {
    const int pieces = (D + threads * 4 - 1) / (threads * 4);
    auto kern = !vec ? pmm::add_postnorm_rmsnorm_kernel<S>
              : pieces <= 1 ? pmm::add_postnorm_rmsnorm_vec_kernel<S, 1>
              : pieces <= 2 ? pmm::add_postnorm_rmsnorm_vec_kernel<S, 2> : pmm::add_postnorm_rmsnorm_vec_kernel<S, 4>;
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    pmm::launch_pdl(kern, dim3(R), dim3(threads), smem, stream, static_cast<float*>(h), static_cast<const S*>(a), sa,
                    static_cast<const S*>(b), sb, post_w, post_eps, w, eps, static_cast<S*>(out), rows, D);
  });
  return pmm::launch_status();
}

PMM_EXPORT int pmm_scale_f32(float* x, float s, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  pmm::scale_f32_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
      x, s, static_cast<size_t>(n));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_cast_scale(float* out, const void* in, float s, long long n, int dtype,
                              cudaStream_t stream) {
  if (n <= 0) return 0;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::cast_scale_kernel<S><<<static_cast<unsigned>((n + 255) / 256), 256,
                                                          0, stream>>>(
                                   out, static_cast<const S*>(in), s, static_cast<size_t>(n)));
  return pmm::launch_status();
}
