// Rotation on part of every head, and the write into the cache pages, for heads whose key size d and
// value size dv differ.
//
// The first rot_dims entries of every query and key head are rotated in pairs (x, y): at position p they
// become (x cos a - y sin a, y cos a + x sin a) with a = p * inv_freq[i].  Pair i is entries (2i, 2i+1)
// (neighbouring pairs) or entries (i, i + rot_dims/2) (half layout: the first half of the rotated
// part against its second half); entries from rot_dims on pass unchanged; values are not rotated.
// A bias per channel (float, optional) is added to q, k and v as they are read.  Positions, angles, sines and cosines are
// float.  Queries go to q_out [T, H*Dp], keys and values into their page
// [page, plane, page_size, G*Dp]: all heads are laid out Dp = max(d, dv) rounded up wide, padded
// with zeros, so that one attention kernel of head size Dp serves both sizes (zeros add nothing to
// a score, and the padded value columns come out zero and are dropped by the output projection's
// operand view).
#include "common.cuh"

namespace pmm {

constexpr int kRopeMaxPairs = 128;  // rot_dims <= 256

// `sn`, `cs`: the token's sines and cosines per rotated pair (shared memory, made once a token).
template <typename S>
__device__ __forceinline__ float rotated(const S* __restrict__ head, const float* __restrict__ bias, int i, int rot_dims,
                                         const float* __restrict__ sn_t, const float* __restrict__ cs_t, int half_layout,
                                         const float* __restrict__ norm_w = nullptr, float inv = 1.f) {
  const float x = (ldf(head + i) + (bias ? bias[i] : 0.f)) * (norm_w ? inv * norm_w[i] : 1.f);
  if (i >= rot_dims) return x;
  const int half = rot_dims >> 1;
  const bool second = half_layout ? i >= half : (i & 1);
  const int j = half_layout ? (second ? i - half : i + half) : (i ^ 1);
  const int f = half_layout ? (second ? i - half : i) : (i >> 1);
  const float other = (ldf(head + j) + (bias ? bias[j] : 0.f)) * (norm_w ? inv * norm_w[j] : 1.f);
  const float sn = sn_t[f], cs = cs_t[f];
  return second ? x * cs + other * sn : x * cs - other * sn;
}

template <typename S>
__global__ void __launch_bounds__(256)
    rope_pairs_store_kernel(const S* __restrict__ q, long long ld_q, const S* __restrict__ k, long long ld_k,
                            const S* __restrict__ v, long long ld_v, const float* __restrict__ inv_freq,
                            const int* __restrict__ positions, const int* __restrict__ seq_of,
                            const int* __restrict__ block_table, int max_blocks, S* __restrict__ pool,
                            int page_size, S* __restrict__ q_out, int H, int G, int d, int dv, int Dp,
                            int rot_dims, int half_layout, const float* __restrict__ q_bias,
                            const float* __restrict__ k_bias, const float* __restrict__ v_bias,
                            const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float norm_eps) {
  __shared__ float sn_t[kRopeMaxPairs], cs_t[kRopeMaxPairs];
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = static_cast<float>(pos);
  for (int f = threadIdx.x; f < rot_dims / 2; f += blockDim.x) sincosf(fpos * inv_freq[f], &sn_t[f], &cs_t[f]);
  // q_norm_w / k_norm_w: all query rows of the token, and all its key rows, are divided by their root mean
  // square (over the whole projection, before it is cut into heads) and multiplied by the weight, before rotation
  float inv_q = 1.f, inv_k = 1.f;
  if (q_norm_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < H * d; i += blockDim.x) {
      const float x = ldf(q + static_cast<long long>(t) * ld_q + i) + (q_bias ? q_bias[i] : 0.f);
      ss += x * x;
    }
    inv_q = 1.f / sqrtf(block_sum(ss, red) / static_cast<float>(H * d) + norm_eps);
  }
  if (k_norm_w) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < G * d; i += blockDim.x) {
      const float x = ldf(k + static_cast<long long>(t) * ld_k + i) + (k_bias ? k_bias[i] : 0.f);
      ss += x * x;
    }
    inv_k = 1.f / sqrtf(block_sum(ss, red) / static_cast<float>(G * d) + norm_eps);
  }
  __syncthreads();
  const int n_q = H * Dp, n_kv = G * Dp;
  const int page = block_table[static_cast<size_t>(seq_of[t]) * max_blocks + pos / page_size];
  S* k_row = pool + (static_cast<size_t>(page) * 2 * page_size + pos % page_size) * n_kv;
  S* v_row = k_row + static_cast<size_t>(page_size) * n_kv;
  for (int e = threadIdx.x; e < n_q + 2 * n_kv; e += blockDim.x) {
    if (e < n_q) {
      const int h = e / Dp, i = e - h * Dp;
      const float val = i < d ? rotated(q + static_cast<long long>(t) * ld_q + h * d, q_bias ? q_bias + h * d : nullptr, i, rot_dims,
                                        sn_t, cs_t, half_layout, q_norm_w ? q_norm_w + h * d : nullptr, inv_q) : 0.f;
      stf(q_out + static_cast<size_t>(t) * n_q + e, val);
    } else if (e < n_q + n_kv) {
      const int c = e - n_q, g = c / Dp, i = c - g * Dp;
      const float val = i < d ? rotated(k + static_cast<long long>(t) * ld_k + g * d, k_bias ? k_bias + g * d : nullptr, i, rot_dims,
                                        sn_t, cs_t, half_layout, k_norm_w ? k_norm_w + g * d : nullptr, inv_k) : 0.f;
      stf(k_row + c, val);
    } else {
      const int c = e - n_q - n_kv, g = c / Dp, i = c - g * Dp;
      stf(v_row + c, i < dv ? ldf(v + static_cast<long long>(t) * ld_v + g * dv + i) + (v_bias ? v_bias[g * dv + i] : 0.f) : 0.f);
    }
  }
}

}  // namespace pmm

// q [T, H*d], k [T, G*d], v [T, G*dv] rows of stride ld; inv_freq [rot_dims/2] floats (may be nullptr when
// rot_dims is 0); pool [pages, 2, page_size, G*Dp]; q_out [T, H*Dp]; q_bias [H*d], k_bias [G*d], v_bias [G*dv]
// floats or nullptr; q_norm_w [H*d], k_norm_w [G*d] floats or nullptr: an RMS norm over the token's whole query
// (key) projection before rotation, eps inside the root.  Values are never normed.
PMM_EXPORT int pmm_rope_pairs_store(const void* q, long long ld_q, const void* k, long long ld_k, const void* v,
                                    long long ld_v, const float* inv_freq, const int* positions, const int* seq_of,
                                    const int* block_table, int max_blocks, void* pool, int page_size, void* q_out,
                                    int T, int H, int G, int d, int dv, int Dp, int rot_dims, int half_layout,
                                    const float* q_bias, const float* k_bias, const float* v_bias,
                                    const float* q_norm_w, const float* k_norm_w, float norm_eps, int dtype,
                                    cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || d <= 0 || dv <= 0 || Dp < d || Dp < dv || rot_dims < 0 || rot_dims > d || rot_dims % 2 ||
      rot_dims > 2 * pmm::kRopeMaxPairs || (rot_dims > 0 && !inv_freq) || page_size <= 0)
    return PMM_ERR_BAD_ARGUMENT;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::rope_pairs_store_kernel<S>, dim3(T), dim3(256), 0, stream,
                                               static_cast<const S*>(q), ld_q, static_cast<const S*>(k), ld_k,
                                               static_cast<const S*>(v), ld_v, inv_freq, positions, seq_of,
                                               block_table, max_blocks, static_cast<S*>(pool), page_size,
                                               static_cast<S*>(q_out), H, G, d, dv, Dp, rot_dims, half_layout, q_bias,
                                               k_bias, v_bias, q_norm_w, k_norm_w, norm_eps));
  return pmm::launch_status();
}
