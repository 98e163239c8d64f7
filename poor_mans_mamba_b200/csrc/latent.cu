// Latent attention: what stands between the stacked input projection and the attention kernels, and
// the per-head output gate.
//
// A token's keys and values of all heads are made from one latent row c (kv_rank entries) and, where
// the heads have a rotated part, one rotated key part r (rot_dim entries) shared by all heads:
//   k_h = [W_uk,h c | rot(r)],  v_h = W_uv,h c.
// Only [c | rot(r)] is cached.  The up-projections move to the queries and to the output:
//   score_h = q_h . k_h = (W_uk,h^T q_h,unrotated) . c + rot(q_h,rotated) . rot(r)
//   out_h   = W_uv,h (sum_j p_j c_j)
// so the attention kernels see H query heads of size Dp = kv_rank + rot_dim (rounded up to a multiple
// of 16, zeros beyond) over ONE key/value head: key row [c | rot(r) | 0], value row [c | 0].
//
// latent_norm_store (a block per token): the query latent and the key/value latent are divided by
// their root mean squares (float; x / sqrt(mean(x^2) + eps) * w; q_rank 0: the queries have no latent),
// the rotated key part turns in neighbouring pairs (2i, 2i+1), or with ``half`` in pairs (i, i + rot_dims/2),
// by the angle p * inv_freq[i], and the key and value rows go into their cache page.  latent_query_rot (a block per token): the rotated part of every query head turns the
// same way and is written behind the head's latent part.  Positions, angles, sines, cosines and both
// norms are float in both storage types.
#include "common.cuh"

namespace pmm {

constexpr int kLatentMaxPairs = 128;  // rot_dims <= 256

// Entry j (< rot_dims) of a rotated part turns together with its partner: neighbours (2i, 2i+1), or with
// ``half`` entries (i, i + rot_dims/2); the angle is that of pair i.
__device__ __forceinline__ void rot_partner(int j, int rot_dims, int half, int* partner, int* pair, bool* second) {
  if (half) {
    const int hd = rot_dims >> 1;
    *second = j >= hd;
    *pair = *second ? j - hd : j;
    *partner = *second ? j - hd : j + hd;
  } else {
    *second = (j & 1) != 0;
    *pair = j >> 1;
    *partner = j ^ 1;
  }
}

// x [T, >= q_rank] and kv [T, >= kv_rank + rot_dim]: rows of the stacked projection (strides ld_x, ld_kv).
// cq [T, q_rank] contiguous.  pool [pages, planes, page_size, Dp]; planes 2: keys in plane 0, values in plane 1.
template <typename S>
__global__ void __launch_bounds__(256)
    latent_norm_store_kernel(const S* __restrict__ x, long long ld_x, const S* __restrict__ kv, long long ld_kv,
                             const float* __restrict__ q_w, const float* __restrict__ kv_w, float eps,
                             const float* __restrict__ inv_freq, const int* __restrict__ positions,
                             const int* __restrict__ seq_of, const int* __restrict__ block_table, int max_blocks,
                             S* __restrict__ pool, int page_size, S* __restrict__ cq, int q_rank, int kv_rank,
                             int rot_dim, int rot_dims, int Dp, int half, const S* __restrict__ q, long long ld_q,
                             S* __restrict__ q_out, int H, int dim) {
  __shared__ float red[32];
  __shared__ float sn_t[kLatentMaxPairs], cs_t[kLatentMaxPairs];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const float fpos = static_cast<float>(pos);
  for (int f = threadIdx.x; f < rot_dims / 2; f += blockDim.x) sincosf(fpos * inv_freq[f], &sn_t[f], &cs_t[f]);
  const S* xr = x + static_cast<long long>(t) * ld_x;
  const S* kr = kv + static_cast<long long>(t) * ld_kv;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = ldf(xr + i); sq += v * v; }
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = ldf(kr + i); sk += v * v; }
  const float inv_q = q_rank > 0 ? 1.f / sqrtf(block_sum(sq, red) / static_cast<float>(q_rank) + eps) : 0.f;
  const float inv_k = 1.f / sqrtf(block_sum(sk, red) / static_cast<float>(kv_rank) + eps);  // (block_sum syncs: sn_t, cs_t are ready)
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) stf(cq + static_cast<size_t>(t) * q_rank + i, ldf(xr + i) * inv_q * q_w[i]);
  const int page = block_table[static_cast<size_t>(seq_of[t]) * max_blocks + pos / page_size];
  S* k_row = pool + (static_cast<size_t>(page) * 2 * page_size + pos % page_size) * Dp;
  S* v_row = k_row + static_cast<size_t>(page_size) * Dp;
  for (int i = threadIdx.x; i < Dp; i += blockDim.x) {
    float kval = 0.f, vval = 0.f;
    if (i < kv_rank) {
      // (rounded to the storage type first, so that key and value rows hold the same number)
      kval = vval = ldf(kr + i) * inv_k * kv_w[i];
    } else if (i < kv_rank + rot_dim) {
      const int j = i - kv_rank;
      const float a = ldf(kr + i);
      if (j < rot_dims) {
        int partner, pair;
        bool second;
        rot_partner(j, rot_dims, half, &partner, &pair, &second);
        const float b = ldf(kr + kv_rank + partner);
        const float sn = sn_t[pair], cs = cs_t[pair];
        kval = second ? a * cs + b * sn : a * cs - b * sn;
      } else {
        kval = a;
      }
    }
    stf(k_row + i, kval);
    stf(v_row + i, vval);
  }
  // q != nullptr (queries that need no latent, q [T, H * (dim + rot_dim)]): latent_query_rot's work in the same
  // launch, the rotated part of every head turned into q_out[t, h, kv_rank .. kv_rank + rot_dim), zeros up to Dp
  if (q != nullptr) {
    const int tail = Dp - kv_rank;
    const S* qr = q + static_cast<long long>(t) * ld_q;
    for (int e = threadIdx.x; e < H * tail; e += blockDim.x) {
      const int h = e / tail, j = e - h * tail;
      float val = 0.f;
      if (j < rot_dim) {
        const S* part = qr + static_cast<size_t>(h) * (dim + rot_dim) + dim;
        const float a = ldf(part + j);
        val = a;
        if (j < rot_dims) {
          int partner, pair;
          bool second;
          rot_partner(j, rot_dims, half, &partner, &pair, &second);
          const float b = ldf(part + partner);
          const float sn = sn_t[pair], cs = cs_t[pair];
          val = second ? a * cs + b * sn : a * cs - b * sn;
        }
      }
      stf(q_out + (static_cast<size_t>(t) * H + h) * Dp + kv_rank + j, val);
    }
  }
}

// q [T, H*(dim + rot_dim)] rows of stride ld_q: the rotated part of head h turns and goes to
// q_out[t, h, kv_rank .. kv_rank + rot_dim); the entries from there to Dp become zero.  The first kv_rank
// entries of every head are left alone (the per-head product W_uk^T q writes them).
template <typename S>
__global__ void __launch_bounds__(256)
    latent_query_rot_kernel(const S* __restrict__ q, long long ld_q, const float* __restrict__ inv_freq,
                            const int* __restrict__ positions, S* __restrict__ q_out, int H, int dim, int rot_dim,
                            int rot_dims, int kv_rank, int Dp, int half) {
  __shared__ float sn_t[kLatentMaxPairs], cs_t[kLatentMaxPairs];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float fpos = static_cast<float>(positions[t]);
  for (int f = threadIdx.x; f < rot_dims / 2; f += blockDim.x) sincosf(fpos * inv_freq[f], &sn_t[f], &cs_t[f]);
  __syncthreads();
  const int tail = Dp - kv_rank;
  const S* qr = q + static_cast<long long>(t) * ld_q;
  for (int e = threadIdx.x; e < H * tail; e += blockDim.x) {
    const int h = e / tail, j = e - h * tail;
    float val = 0.f;
    if (j < rot_dim) {
      const S* part = qr + static_cast<size_t>(h) * (dim + rot_dim) + dim;
      const float a = ldf(part + j);
      if (j < rot_dims) {
        int partner, pair;
        bool second;
        rot_partner(j, rot_dims, half, &partner, &pair, &second);
        const float b = ldf(part + partner);
        const float sn = sn_t[pair], cs = cs_t[pair];
        val = second ? a * cs + b * sn : a * cs - b * sn;
      } else {
        val = a;
      }
    }
    stf(q_out + (static_cast<size_t>(t) * H + h) * Dp + kv_rank + j, val);
  }
}

// out[t, h*dv + i] = scale * a[t, h*dv + i] * sigmoid(g[t, h]): one gate per head (g == nullptr: scale only).
template <typename S>
__global__ void head_gate_kernel(const S* __restrict__ a, long long ld_a, const S* __restrict__ g, long long ld_g,
                                 float scale, S* __restrict__ out, long long ld_o, int H, int dv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int n = H * dv;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    const int h = c / dv;
    const float gv = g ? 1.f / (1.f + expf(-ldf(g + static_cast<long long>(t) * ld_g + h))) : 1.f;
    stf(out + static_cast<long long>(t) * ld_o + c, scale * gv * ldf(a + static_cast<long long>(t) * ld_a + c));
  }
}

}  // namespace pmm

PMM_EXPORT int pmm_latent_norm_store(const void* x, long long ld_x, const void* kv, long long ld_kv, const float* q_w,
                                     const float* kv_w, float eps, const float* inv_freq, const int* positions,
                                     const int* seq_of, const int* block_table, int max_blocks, void* pool,
                                     int page_size, void* cq, int T, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                                     int Dp, int half, const void* q, long long ld_q, void* q_out, int H, int dim,
                                     int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank < 0 || (q_rank > 0 && (!x || !q_w || !cq)) || kv_rank <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2 ||
      rot_dims > 2 * pmm::kLatentMaxPairs || (rot_dims > 0 && !inv_freq) || Dp < kv_rank + rot_dim || page_size <= 0)
    return PMM_ERR_BAD_ARGUMENT;
  if (q && (!q_out || H <= 0 || dim <= 0)) return PMM_ERR_BAD_ARGUMENT;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::latent_norm_store_kernel<S>, dim3(T), dim3(256), 0, stream,
                                               static_cast<const S*>(x), ld_x, static_cast<const S*>(kv), ld_kv, q_w,
                                               kv_w, eps, inv_freq, positions, seq_of, block_table, max_blocks,
                                               static_cast<S*>(pool), page_size, static_cast<S*>(cq), q_rank, kv_rank,
                                               rot_dim, rot_dims, Dp, half, static_cast<const S*>(q), ld_q,
                                               static_cast<S*>(q_out), H, dim));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_latent_query_rot(const void* q, long long ld_q, const float* inv_freq, const int* positions,
                                    void* q_out, int T, int H, int dim, int rot_dim, int rot_dims, int kv_rank, int Dp,
                                    int half, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dim <= 0 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || rot_dims % 2 ||
      rot_dims > 2 * pmm::kLatentMaxPairs || (rot_dims > 0 && !inv_freq) || Dp < kv_rank + rot_dim)
    return PMM_ERR_BAD_ARGUMENT;
  if (Dp == kv_rank) return 0;  // nothing behind the latent part
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::latent_query_rot_kernel<S>, dim3(T), dim3(256), 0, stream,
                                               static_cast<const S*>(q), ld_q, inv_freq, positions,
                                               static_cast<S*>(q_out), H, dim, rot_dim, rot_dims, kv_rank, Dp, half));
  return pmm::launch_status();
}

PMM_EXPORT int pmm_head_gate(const void* a, long long ld_a, const void* g, long long ld_g, float scale, void* out,
                             long long ld_o, int T, int H, int dv, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dv <= 0) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (H * dv + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::head_gate_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream,
                                               static_cast<const S*>(a), ld_a, static_cast<const S*>(g), ld_g, scale,
                                               static_cast<S*>(out), ld_o, H, dv));
  return pmm::launch_status();
}
