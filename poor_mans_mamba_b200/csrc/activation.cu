// SwiGLU activation on the output of the fused [gate; up] projection.
//   act[t,f] = silu(gu[t,f] * gate_mult) * gu[t,F+f]
// (reference src/ops/cuda_backend.cu:311-338: scale, silu, mul as three launches).
#include "common.cuh"

namespace pmm {

template <typename S>
__global__ void silu_mul_kernel(const S* __restrict__ gu, long long ld, float gate_mult,
                                S* __restrict__ out, int F) {
  const int t = blockIdx.x;
  const S* row = gu + static_cast<long long>(t) * ld;
  S* o = out + static_cast<size_t>(t) * F;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < F; f += gridDim.y * blockDim.x) {
    const float g = ldf(row + f) * gate_mult;
    stf(o + f, silu_f(g) * ldf(row + F + f));
  }
}

// bfloat16, F and ld multiples of 8, 16-byte aligned rows: eight elements per thread.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, float gate_mult,
                                       __nv_bfloat16* __restrict__ out, int F) {
  const int t = blockIdx.x;
  const __nv_bfloat16* row = gu + static_cast<long long>(t) * ld;
  __nv_bfloat16* o = out + static_cast<size_t>(t) * F;
  for (int f = (blockIdx.y * blockDim.x + threadIdx.x) * 8; f < F; f += gridDim.y * blockDim.x * 8) {
    const uint4 gv = *reinterpret_cast<const uint4*>(row + f);
    const uint4 uv = *reinterpret_cast<const uint4*>(row + F + f);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = __bfloat1622float2(g2[i]);
      const float2 u = __bfloat1622float2(u2[i]);
      o2[i] = __floats2bfloat162_rn(silu_fast(g.x * gate_mult) * u.x, silu_fast(g.y * gate_mult) * u.y);
    }
    *reinterpret_cast<uint4*>(o + f) = ov;
  }
}

// The tanh form of GELU: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// act[t, f] = gelu_tanh(gu[t, f] * gate_mult) * gu[t, F + f]
template <typename S>
__global__ void gelu_tanh_mul_kernel(const S* __restrict__ gu, long long ld, float gate_mult,
                                     S* __restrict__ out, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const S* row = gu + static_cast<long long>(t) * ld;
  S* o = out + static_cast<size_t>(t) * F;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < F; f += gridDim.y * blockDim.x)
    stf(o + f, gelu_tanh_f(ldf(row + f) * gate_mult) * ldf(row + F + f));
}

// bfloat16, F and ld multiples of 8, 16-byte aligned rows: eight elements per thread.
__global__ void gelu_tanh_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, long long ld, float gate_mult,
                                            __nv_bfloat16* __restrict__ out, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const __nv_bfloat16* row = gu + static_cast<long long>(t) * ld;
  __nv_bfloat16* o = out + static_cast<size_t>(t) * F;
  for (int f = (blockIdx.y * blockDim.x + threadIdx.x) * 8; f < F; f += gridDim.y * blockDim.x * 8) {
    const uint4 gv = *reinterpret_cast<const uint4*>(row + f);
    const uint4 uv = *reinterpret_cast<const uint4*>(row + F + f);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = __bfloat1622float2(g2[i]);
      const float2 u = __bfloat1622float2(u2[i]);
      o2[i] = __floats2bfloat162_rn(gelu_tanh_f(g.x * gate_mult) * u.x, gelu_tanh_f(g.y * gate_mult) * u.y);
    }
    *reinterpret_cast<uint4*>(o + f) = ov;
  }
}

}  // namespace pmm

PMM_EXPORT int pmm_gelu_tanh_mul(const void* gu, long long ld, float gate_mult, void* out, int T, int F,
                                 int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0) return PMM_ERR_BAD_ARGUMENT;
  if (dtype == PMM_DTYPE_BF16 && F % 8 == 0 && ld % 8 == 0 &&
      reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    int yt = (F / 8 + 255) / 256;
    if (yt > 64) yt = 64;
    pmm::launch_pdl(pmm::gelu_tanh_mul_bf16x8_kernel, dim3(T, yt), dim3(256), 0, stream,
                    static_cast<const __nv_bfloat16*>(gu), ld, gate_mult, static_cast<__nv_bfloat16*>(out), F);
    return pmm::launch_status();
  }
  int ytiles = (F + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::gelu_tanh_mul_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream,
                                               static_cast<const S*>(gu), ld, gate_mult, static_cast<S*>(out), F));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_silu_mul(const void* gu, long long ld, float gate_mult, void* out, int T, int F,
                            int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0) return PMM_ERR_BAD_ARGUMENT;
  if (dtype == PMM_DTYPE_BF16 && F % 8 == 0 && ld % 8 == 0 &&
      reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
    int yt = (F / 8 + 255) / 256;
    if (yt > 64) yt = 64;
    pmm::silu_mul_bf16x8_kernel<<<dim3(T, yt), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(gu), ld, gate_mult, static_cast<__nv_bfloat16*>(out), F);
    return pmm::launch_status();
  }
  int ytiles = (F + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  dim3 grid(T, ytiles);
  PMM_DISPATCH_DTYPE(dtype, S, pmm::silu_mul_kernel<S><<<grid, 256, 0, stream>>>(
                                   static_cast<const S*>(gu), ld, gate_mult, static_cast<S*>(out), F));
  return pmm::launch_status();
}

namespace pmm {
template <typename S>
__global__ void add_row_bias_kernel(S* __restrict__ x, const float* __restrict__ bias, int D) {
  S* row = x + static_cast<size_t>(blockIdx.x) * D;
  for (int i = threadIdx.x; i < D; i += blockDim.x) stf(row + i, ldf(row + i) + bias[i]);
}
}  // namespace pmm

// x[t, :] += bias for a contiguous [T, D] activation (projection biases).
PMM_EXPORT int pmm_add_row_bias(void* x, const float* bias, int T, int D, int dtype,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  PMM_DISPATCH_DTYPE(dtype, S,
                     pmm::add_row_bias_kernel<S><<<T, 256, 0, stream>>>(static_cast<S*>(x), bias, D));
  return pmm::launch_status();
}

namespace pmm {
// out[t, h*dv + i] = scale * a[t, h*da + i] * sigmoid(g[t, h*dv + i]) for i < dv: an output gate per
// channel on heads that may be stored wider (da >= dv) than they are used.
template <typename S>
__global__ void sigmoid_gate_kernel(const S* __restrict__ a, long long ld_a, const S* __restrict__ g, long long ld_g,
                                    float scale, S* __restrict__ out, long long ld_o, int H, int da, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n = H * dv;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    const int h = c / dv, i = c - h * dv;
    const float gv = ldf(g + static_cast<long long>(t) * ld_g + c);
    const float av = ldf(a + static_cast<long long>(t) * ld_a + h * da + i);
    stf(out + static_cast<long long>(t) * ld_o + c, scale * av / (1.f + expf(-gv)));
  }
}

// The clamped gated activation of a [gate | up] projection:
//   g = min(gu[t, f], limit); u = clamp(gu[t, F + f], -limit, limit); out = g * sigmoid(alpha * g) * (u + shift)
template <typename S>
__global__ void clamped_glu_kernel(const S* __restrict__ gu, long long ld, float limit, float alpha, float shift,
                                   S* __restrict__ out, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const S* row = gu + static_cast<long long>(t) * ld;
  S* o = out + static_cast<size_t>(t) * F;
  for (int f = blockIdx.y * blockDim.x + threadIdx.x; f < F; f += gridDim.y * blockDim.x) {
    const float g = fminf(ldf(row + f), limit);
    const float u = fminf(fmaxf(ldf(row + F + f), -limit), limit);
    stf(o + f, g / (1.f + expf(-alpha * g)) * (u + shift));
  }
}
}  // namespace pmm

PMM_EXPORT int pmm_sigmoid_gate(const void* a, long long ld_a, const void* g, long long ld_g, float scale, void* out,
                                long long ld_o, int T, int H, int da, int dv, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dv <= 0 || da < dv) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (H * dv + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::sigmoid_gate_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream,
                                               static_cast<const S*>(a), ld_a, static_cast<const S*>(g), ld_g, scale,
                                               static_cast<S*>(out), ld_o, H, da, dv));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_clamped_glu(const void* gu, long long ld, float limit, float alpha, float shift, void* out, int T,
                               int F, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (F <= 0) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (F + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::clamped_glu_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream,
                                               static_cast<const S*>(gu), ld, limit, alpha, shift,
                                               static_cast<S*>(out), F));
  return pmm::launch_status();
}
