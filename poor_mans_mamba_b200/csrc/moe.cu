// Routed feed-forward (mixture of experts): router with top-k choice, the plan that sorts the
// (token, choice) pairs by expert, grouped products over the sorted rows, and the weighted sum.
//
//   z = x Wr^T + br (float; Wr, br float);  the `top` largest z are chosen (the lower index wins a tie),
//   p = softmax over the chosen z only;
//   pairs (t, j) are sorted by expert: offsets[e] .. offsets[e+1] are expert e's rows of `perm`,
//   perm[i] = t * top + j;
//   act[i]  = glu(x[perm[i] / top] Wgu_e^T)        [gate | up] rows of expert e, clamped gated activation
//   y[perm[i]] = act[i] Wd_e^T                     storage type
//   out[t] = sum_j p[t, j] y[t * top + j] (+ shared[t])
//
// Everything stays on the device: the grouped products are launched for an upper bound of row
// tiles, sum_e ceil(n_e / TM) <= floor(A / TM) + min(E, A) with A = T * top, and a block beyond the
// last tile leaves.  A row's result does not depend on which other rows share its tile.
#include "common.cuh"
#include "mma_helpers.cuh"

namespace pmm {

// A block routes TOK tokens: their rows wait in shared memory as floats, every warp takes the experts
// e = warp, warp + 8, ... and reads a router row once (16 bytes a lane and access) for all TOK dot
// products; then a warp per token picks the `top` largest logits and norms their exponentials.
constexpr int kRouteWarps = 8;

template <typename S, int TOK>
__global__ void __launch_bounds__(kRouteWarps * 32)
    moe_route_kernel(const S* __restrict__ x, long long ld_x, const float* __restrict__ w,
                     const float* __restrict__ bias, int* __restrict__ ids, float* __restrict__ weights, int T, int D,
                     int E, int top, int scored, const float* __restrict__ correction, int groups, int keep,
                     float scale, const float* __restrict__ gate_w, float* __restrict__ gate_out) {
  extern __shared__ __align__(16) float route_smem[];  // rows [TOK][Dpad] | logits [TOK][E] (scored: | scores, group scores [TOK][2E])
  const int Dpad = (D + 3) & ~3;
  float* rows = route_smem;
  float* logits = route_smem + TOK * Dpad;
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.x * TOK;
  const int nt = min(TOK, T - t0);
  for (int r = 0; r < TOK; ++r)
    for (int i = threadIdx.x; i < Dpad; i += blockDim.x)
      rows[r * Dpad + i] = (r < nt && i < D) ? ldf(x + static_cast<long long>(t0 + r) * ld_x + i) : 0.f;
  __syncthreads();
  const bool vec = (D & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(gate_w) & 15) == 0;
  // (gate_w: one more row, whose product goes through a sigmoid into gate_out[t]: a gate per token that reads the
  // router's input, such as a shared expert's)
  const int n_rows = E + (gate_w ? 1 : 0);
  for (int e = warp; e < n_rows; e += kRouteWarps) {
    float acc[TOK];
#pragma unroll
    for (int r = 0; r < TOK; ++r) acc[r] = 0.f;
    const float* wr = e < E ? w + static_cast<size_t>(e) * D : gate_w;
    if (vec) {
      for (int i = lane * 4; i < D; i += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(wr + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) {
          const float4 xv = *reinterpret_cast<const float4*>(rows + r * Dpad + i);
          acc[r] += xv.x * wv.x + xv.y * wv.y + xv.z * wv.z + xv.w * wv.w;
        }
      }
    } else {
      for (int i = lane; i < D; i += 32) {
        const float wv = wr[i];
#pragma unroll
        for (int r = 0; r < TOK; ++r) acc[r] += rows[r * Dpad + i] * wv;
      }
    }
#pragma unroll
    for (int r = 0; r < TOK; ++r) {
      const float sum = warp_sum(acc[r]);
      if (lane == 0) {
        if (e < E) logits[r * E + e] = sum + (bias ? bias[e] : 0.f);
        else if (r < nt) gate_out[t0 + r] = 1.f / (1.f + expf(-sum));
      }
    }
  }
  __syncthreads();
  if (scored) {
    // Scores s = sigmoid(z) (scored == 2: s = softmax(z) over all experts, a group's score is its largest choice
    // score, and the weights are the chosen s times scale, not divided by their sum).  The choice runs on s + correction, among the experts of the `keep` groups (of `groups`
    // equal groups of neighbours) whose two largest choice scores sum highest; every other expert's choice score is
    // -inf.  The weights are the chosen s over their sum (+ 1e-20), times scale.  The lower index wins a tie.
    float* extra = logits + TOK * E;
    for (int r = warp; r < nt; r += kRouteWarps) {
      float* z = logits + r * E;         // becomes the choice scores
      float* sc = extra + r * 2 * E;     // s
      float* gs = sc + E;                // group scores
      if (scored == 2) {
        // scores: the softmax of z over all experts
        float zmax = -INFINITY;
        for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
        zmax = warp_max(zmax);
        float zsum = 0.f;
        for (int e = lane; e < E; e += 32) {
          const float ev = expf(z[e] - zmax);
          sc[e] = ev;
          zsum += ev;
        }
        const float zinv = 1.f / warp_sum(zsum);
        for (int e = lane; e < E; e += 32) {
          const float sv = sc[e] * zinv;
          sc[e] = sv;
          z[e] = sv + (correction ? correction[e] : 0.f);
        }
      } else {
        for (int e = lane; e < E; e += 32) {
          const float sv = 1.f / (1.f + expf(-z[e]));
          sc[e] = sv;
          z[e] = sv + (correction ? correction[e] : 0.f);
        }
      }
      __syncwarp();
      if (groups > 1) {
        const int per = E / groups;
        for (int g = lane; g < groups; g += 32) {
          float a = -INFINITY, b = -INFINITY;  // the largest and the second largest
          for (int e = g * per; e < (g + 1) * per; ++e) {
            const float v = z[e];
            if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
          }
          gs[g] = (per > 1 && scored != 2) ? a + b : a;
        }
        __syncwarp();
        // the `keep` best groups are marked by +inf in gs; then the others' experts drop out
        for (int j = 0; j < keep; ++j) {
          float best = -INFINITY;
          int arg = 0x7fffffff;
          for (int g = lane; g < groups; g += 32) {
            const float v = gs[g];
            if (v != INFINITY && (v > best || (v == best && g < arg) || arg == 0x7fffffff)) { best = v; arg = g; }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (oa != 0x7fffffff && (arg == 0x7fffffff || ob > best || (ob == best && oa < arg))) { best = ob; arg = oa; }
          }
          if (lane == 0 && arg < groups) gs[arg] = INFINITY;
          __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
          if (gs[e / per] != INFINITY) z[e] = -INFINITY;
        __syncwarp();
      }
      float denom = 0.f;
      for (int j = 0; j < top; ++j) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
          const float v = z[e];
          if (v > best || (v == best && e < arg)) { best = v; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ob = __shfl_xor_sync(0xffffffffu, best, o);
          const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
          if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= E) arg = j;  // nothing left to choose from: keep the indices valid
        const float p = sc[arg];
        denom += p;
        if (lane == 0) {
          ids[static_cast<size_t>(t0 + r) * top + j] = arg;
          weights[static_cast<size_t>(t0 + r) * top + j] = p;
          z[arg] = -INFINITY;
        }
        __syncwarp();
      }
      const float inv = scored == 2 ? scale : scale / (denom + 1e-20f);
      for (int j = lane; j < top; j += 32) weights[static_cast<size_t>(t0 + r) * top + j] *= inv;
    }
    return;
  }
  for (int r = warp; r < nt; r += kRouteWarps) {
    float* z = logits + r * E;
    float first = 0.f, denom = 0.f;
    for (int j = 0; j < top; ++j) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
      for (int e = lane; e < E; e += 32) {
        const float v = z[e];
        if (v > best || (v == best && e < arg)) { best = v; arg = e; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
      }
      if (arg >= E) arg = j;  // every logit left is NaN or -inf: keep the indices valid
      if (j == 0) first = best;
      const float p = expf(best - first);
      denom += p;
      if (lane == 0) {
        ids[static_cast<size_t>(t0 + r) * top + j] = arg;
        weights[static_cast<size_t>(t0 + r) * top + j] = p;
        z[arg] = -INFINITY;
      }
      __syncwarp();
    }
    const float inv = 1.f / denom;
    for (int j = lane; j < top; j += 32) weights[static_cast<size_t>(t0 + r) * top + j] *= inv;
  }
}

// One block: rows per expert, their exclusive sums, and the exclusive sums of the row tiles.
__global__ void __launch_bounds__(1024)
    moe_plan_kernel(const int* __restrict__ ids, int A, int E, int tile_rows, int* __restrict__ offsets,
                    int* __restrict__ tile_start) {
  extern __shared__ int plan_counts[];  // [E]
  pdl_launch_dependents();
  for (int e = threadIdx.x; e < E; e += blockDim.x) plan_counts[e] = 0;
  pdl_wait();
  __syncthreads();
  for (int i = threadIdx.x; i < A; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&plan_counts[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = rows;
      tile_start[e] = tiles;
      rows += plan_counts[e];
      tiles += (plan_counts[e] + tile_rows - 1) / tile_rows;
    }
    offsets[E] = rows;
    tile_start[E] = tiles;
  }
}

// One block per expert: its pairs in the order of their index (stable, so the plan is the same every time).
// A thread owns a run of consecutive pairs: it counts its matches, the block sums the counts before each
// thread, and the thread writes its matches from there.
__global__ void __launch_bounds__(1024)
    moe_fill_kernel(const int* __restrict__ ids, int A, const int* __restrict__ offsets, int* __restrict__ perm) {
  __shared__ int warp_total[32];
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int base = offsets[e];
  if (offsets[e + 1] == base) return;
  const int run = (A + blockDim.x - 1) / blockDim.x;
  const int i0 = min(A, static_cast<int>(threadIdx.x) * run), i1 = min(A, i0 + run);
  int mine = 0;
  for (int i = i0; i < i1; ++i) mine += ids[i] == e;
  int incl = mine;  // inclusive sum over the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  if (lane == 31) warp_total[warp] = incl;
  __syncthreads();
  int before = base + incl - mine;
  for (int w2 = 0; w2 < warp; ++w2) before += warp_total[w2];
  for (int i = i0; i < i1; ++i)
    if (ids[i] == e) perm[before++] = i;
}

// The whole plan of a step with few pairs (a decode step) in one block and one launch: a thread per expert
// counts its pairs, one thread sums, then every expert's thread writes its pairs in their order.
constexpr int kPlanSmallPairs = 512;

__global__ void __launch_bounds__(256)
    moe_plan_small_kernel(const int* __restrict__ ids, int A, int E, int tile_rows, int* __restrict__ offsets,
                          int* __restrict__ tile_start, int* __restrict__ perm) {
  extern __shared__ int plan_small[];  // ids [A] | counts, then starts [E]
  int* ids_s = plan_small;
  int* cnt = plan_small + A;
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < A; i += blockDim.x) ids_s[i] = ids[i];
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int c = 0;
    for (int i = 0; i < A; ++i) c += ids_s[i] == e;
    cnt[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int rows = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      offsets[e] = rows;
      tile_start[e] = tiles;
      cnt[e] = rows;
      rows += c;
      tiles += (c + tile_rows - 1) / tile_rows;
    }
    offsets[E] = rows;
    tile_start[E] = tiles;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int pos = cnt[e];
    for (int i = 0; i < A; ++i)
      if (ids_s[i] == e) perm[pos++] = i;
  }
}

__device__ __forceinline__ float clamped_glu(float g, float u, float limit, float alpha, float shift) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + expf(-alpha * g)) * (u + shift);
}

// The ungated experts' activation: max(z, 0)^2.
__device__ __forceinline__ float relu_squared(float z) {
  z = fmaxf(z, 0.f);
  return z * z;
}

// Finds the expert and the rows of row tile `tile`; false when there is no such tile.
__device__ __forceinline__ bool moe_tile(int tile, const int* __restrict__ offsets, const int* __restrict__ tile_start,
                                         int E, int tile_rows, int& e, int& row0, int& row1) {
  if (tile >= tile_start[E]) return false;
  int lo = 0, hi = E - 1;  // the last e with tile_start[e] <= tile (experts without rows share a start)
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tile_start[mid] <= tile) lo = mid; else hi = mid - 1;
  }
  e = lo;
  row0 = offsets[e] + (tile - tile_start[e]) * tile_rows;
  row1 = min(offsets[e + 1], row0 + tile_rows);
  return true;
}

// The grouped product in float arithmetic on the CUDA cores, for any sizes and both storage types.
// UP (the [gate | up] product with the activation): a = x [T, K], row i reads x[perm[i] / top]; w [E, 2N, K];
// out = act [A, N] in the storage type.  Otherwise (the down product): a = act [A, K]; w [E, N, K];
// out = y [A, N] in the storage type, row perm[i].
constexpr int kGenRows = 32, kGenCols = 32, kGenK = 32;

template <typename S, bool UP>
__global__ void __launch_bounds__(256)
    moe_gemm_generic_kernel(const S* __restrict__ a, long long ld_a, const S* __restrict__ w,
                            const int* __restrict__ perm, const int* __restrict__ offsets,
                            const int* __restrict__ tile_start, int E, int top, int K, int N, float limit, float alpha,
                            float shift, int ungated, void* __restrict__ out) {
  __shared__ float As[kGenRows][kGenK + 1];
  __shared__ float Bs[UP ? 2 : 1][kGenCols][kGenK + 1];
  __shared__ int src_row[kGenRows];
  pdl_launch_dependents();
  pdl_wait();
  int e, row0, row1;
  if (!moe_tile(blockIdx.y, offsets, tile_start, E, kGenRows, e, row0, row1)) return;
  const int n0 = blockIdx.x * kGenCols;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  if (threadIdx.x < kGenRows) {
    const int i = row0 + threadIdx.x;
    src_row[threadIdx.x] = i < row1 ? ((UP || ungated) ? perm[i] / top : i) : -1;
  }
  __syncthreads();
  const S* we = w + static_cast<size_t>(e) * (UP ? 2 : 1) * N * K;
  float acc[UP ? 2 : 1][4];
#pragma unroll
  for (int m = 0; m < (UP ? 2 : 1); ++m)
#pragma unroll
    for (int r = 0; r < 4; ++r) acc[m][r] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kGenK) {
    for (int idx = threadIdx.x; idx < kGenRows * kGenK; idx += 256) {
      const int r = idx / kGenK, k = idx - r * kGenK;
      const int src = src_row[r];
      As[r][k] = (src >= 0 && k0 + k < K) ? ldf(a + static_cast<long long>(src) * ld_a + k0 + k) : 0.f;
    }
    for (int idx = threadIdx.x; idx < kGenCols * kGenK; idx += 256) {
      const int c = idx / kGenK, k = idx - c * kGenK;
      const bool ok = n0 + c < N && k0 + k < K;
      Bs[0][c][k] = ok ? ldf(we + static_cast<size_t>(n0 + c) * K + k0 + k) : 0.f;
      if (UP) Bs[UP ? 1 : 0][c][k] = ok ? ldf(we + static_cast<size_t>(N + n0 + c) * K + k0 + k) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kGenK; ++k) {
      const float b0 = Bs[0][tx][k];
      const float b1 = UP ? Bs[UP ? 1 : 0][tx][k] : 0.f;
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const float av = As[ty * 4 + r][k];
        acc[0][r] += av * b0;
        if (UP) acc[UP ? 1 : 0][r] += av * b1;
      }
    }
    __syncthreads();
  }
  if (n0 + tx >= N) return;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = row0 + ty * 4 + r;
    if (i >= row1) continue;
    if (UP) {
      stf(static_cast<S*>(out) + static_cast<size_t>(i) * N + n0 + tx,
          clamped_glu(acc[0][r], acc[UP ? 1 : 0][r], limit, alpha, shift));
    } else {
      // (ungated: the activation's rows stay in the order of the sorted pairs, like the gated form's)
      stf(static_cast<S*>(out) + static_cast<size_t>(ungated ? i : perm[i]) * N + n0 + tx,
          ungated ? relu_squared(acc[0][r]) : acc[0][r]);
    }
  }
}

// The grouped product on the tensor cores (mma.sync m16n8k16, bfloat16 operands, float accumulation):
// tiles of 64 rows x 64 columns (UP: 64 gate and 64 up columns), K in slices of 32 through a
// two-stage ring of 16-byte asynchronous copies.  Needs K % 8 == 0 and 16-byte aligned rows.
constexpr int kMmaRows = 64, kMmaCols = 64, kMmaK = 32, kMmaPad = 8;

template <bool UP>
__global__ void __launch_bounds__(128)
    moe_gemm_mma_kernel(const bf16* __restrict__ a, long long ld_a, const bf16* __restrict__ w,
                        const int* __restrict__ perm, const int* __restrict__ offsets,
                        const int* __restrict__ tile_start, int E, int top, int K, int N, float limit, float alpha,
                        float shift, int ungated, void* __restrict__ out) {
  constexpr int BROWS = UP ? 2 * kMmaCols : kMmaCols;
  constexpr int LD = kMmaK + kMmaPad;  // 40 elements = 80 bytes: ldmatrix rows fall into different banks
  __shared__ __align__(16) bf16 As[2][kMmaRows][LD];
  __shared__ __align__(16) bf16 Bs[2][BROWS][LD];
  __shared__ int src_row[kMmaRows];
  __shared__ int dst_row[kMmaRows];
  pdl_launch_dependents();
  pdl_wait();
  int e, row0, row1;
  if (!moe_tile(blockIdx.y, offsets, tile_start, E, kMmaRows, e, row0, row1)) return;
  const int n0 = blockIdx.x * kMmaCols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < kMmaRows) {
    const int i = row0 + threadIdx.x;
    const int p = i < row1 ? perm[i] : -1;
    src_row[threadIdx.x] = i < row1 ? ((UP || ungated) ? p / top : i) : -1;
    dst_row[threadIdx.x] = p;
  }
  __syncthreads();
  const bf16* we = w + static_cast<size_t>(e) * (UP ? 2 : 1) * N * K;

  auto stage = [&](int buf, int k0) {
    // 64 rows x 4 pieces of 8 elements for A; BROWS x 4 for B
    for (int idx = threadIdx.x; idx < kMmaRows * 4; idx += 128) {
      const int r = idx >> 2, c = (idx & 3) * 8;
      const int src = src_row[r];
      const bool ok = src >= 0 && k0 + c < K;
      cp_async16(&As[buf][r][c], ok ? a + static_cast<long long>(src) * ld_a + k0 + c : a, ok);
    }
    for (int idx = threadIdx.x; idx < BROWS * 4; idx += 128) {
      const int r = idx >> 2, c = (idx & 3) * 8;
      const int col = UP ? (r < kMmaCols ? n0 + r : N + n0 + (r - kMmaCols)) : n0 + r;
      const bool ok = (UP ? (r < kMmaCols ? n0 + r : n0 + r - kMmaCols) : n0 + r) < N && k0 + c < K;
      cp_async16(&Bs[buf][r][c], ok ? we + static_cast<size_t>(col) * K + k0 + c : we, ok);
    }
    cp_async_commit();
  };

  float acc[BROWS / 8][4];
#pragma unroll
  for (int j = 0; j < BROWS / 8; ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[j][q] = 0.f;

  const int n_slices = (K + kMmaK - 1) / kMmaK;
  stage(0, 0);
  for (int s = 0; s < n_slices; ++s) {
    if (s + 1 < n_slices) {
      stage((s + 1) & 1, (s + 1) * kMmaK);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int buf = s & 1;
#pragma unroll
    for (int kk = 0; kk < kMmaK; kk += 16) {
      unsigned af[4];
      // the warp's 16 rows: matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
      ldmatrix_x4(af[0], af[1], af[2], af[3], &As[buf][warp * 16 + (lane & 15)][kk + ((lane >> 4) << 3)]);
#pragma unroll
      for (int j = 0; j < BROWS / 16; ++j) {
        unsigned b0, b1, b2, b3;
        // 16 weight rows (two groups of 8 columns of the result) x 16 k
        ldmatrix_x4(b0, b1, b2, b3, &Bs[buf][j * 16 + (lane & 7) + ((lane >> 4) << 3)][kk + (((lane >> 3) & 1) << 3)]);
        mma_bf16(acc[2 * j], af, b0, b1);
        mma_bf16(acc[2 * j + 1], af, b2, b3);
      }
    }
    __syncthreads();
  }

  // accumulator layout: acc[j][0..1] row lane/4, columns j*8 + (lane%4)*2 + {0,1}; acc[j][2..3] row lane/4 + 8
  const int r_lo = warp * 16 + (lane >> 2), c_in = (lane & 3) * 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = r_lo + half * 8;
    const int i = row0 + r;
    if (i >= row1) continue;
#pragma unroll
    for (int j = 0; j < kMmaCols / 8; ++j) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int col = n0 + j * 8 + c_in + q;
        if (col >= N) continue;
        if (UP) {
          const float g = acc[j][half * 2 + q], u = acc[UP ? j + kMmaCols / 8 : j][half * 2 + q];
          static_cast<bf16*>(out)[static_cast<size_t>(i) * N + col] = __float2bfloat16_rn(clamped_glu(g, u, limit, alpha, shift));
        } else {
          const float val = acc[j][half * 2 + q];
          static_cast<bf16*>(out)[static_cast<size_t>(ungated ? i : dst_row[r]) * N + col] =
              __float2bfloat16_rn(ungated ? relu_squared(val) : val);
        }
      }
    }
  }
}

// The same product for steps of few pairs (decode steps), where an expert has a handful of rows and the
// launch is a read of the chosen experts' matrices: tiles of 16 rows x 64 columns, the four warps share the
// columns, K in slices of 64 through a four-stage ring, so that a block keeps three slices in flight.
constexpr int kFewRows = 16, kFewCols = 64, kFewK = 64, kFewStages = 4, kFewLd = kFewK + 8;

template <bool UP>
__global__ void __launch_bounds__(128)
    moe_gemm_few_kernel(const bf16* __restrict__ a, long long ld_a, const bf16* __restrict__ w,
                        const int* __restrict__ perm, const int* __restrict__ offsets,
                        const int* __restrict__ tile_start, int E, int top, int K, int N, float limit, float alpha,
                        float shift, int ungated, bf16* __restrict__ out) {
  constexpr int BROWS = UP ? 2 * kFewCols : kFewCols;
  constexpr int kStageElems = (kFewRows + BROWS) * kFewLd;
  extern __shared__ __align__(16) unsigned char few_smem[];
  bf16* ring = reinterpret_cast<bf16*>(few_smem);
  __shared__ int src_row[kFewRows];
  __shared__ int dst_row[kFewRows];
  pdl_launch_dependents();
  pdl_wait();
  int e, row0, row1;
  if (!moe_tile(blockIdx.y, offsets, tile_start, E, kFewRows, e, row0, row1)) return;
  const int n0 = blockIdx.x * kFewCols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < kFewRows) {
    const int i = row0 + threadIdx.x;
    const int p = i < row1 ? perm[i] : -1;
    src_row[threadIdx.x] = i < row1 ? ((UP || ungated) ? p / top : i) : -1;
    dst_row[threadIdx.x] = p;
  }
  __syncthreads();
  const bf16* we = w + static_cast<size_t>(e) * (UP ? 2 : 1) * N * K;

  auto stage = [&](int buf, int k0) {
    bf16* As = ring + static_cast<size_t>(buf) * kStageElems;
    bf16* Bs = As + kFewRows * kFewLd;
    {  // 16 rows x 8 pieces of 8 elements: one a thread
      const int r = threadIdx.x >> 3, c = (threadIdx.x & 7) * 8;
      const int src = src_row[r];
      const bool ok = src >= 0 && k0 + c < K;
      cp_async16(As + r * kFewLd + c, ok ? a + static_cast<long long>(src) * ld_a + k0 + c : a, ok);
    }
    for (int idx = threadIdx.x; idx < BROWS * 8; idx += 128) {
      const int r = idx >> 3, c = (idx & 7) * 8;
      const int col = UP ? (r < kFewCols ? n0 + r : n0 + r - kFewCols) : n0 + r;
      const bool ok = col < N && k0 + c < K;
      const size_t wrow = UP && r >= kFewCols ? static_cast<size_t>(N) + col : col;
      cp_async16(Bs + r * kFewLd + c, ok ? we + wrow * K + k0 + c : we, ok);
    }
    cp_async_commit();
  };

  float acc[UP ? 4 : 2][4];
#pragma unroll
  for (int j = 0; j < (UP ? 4 : 2); ++j)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[j][q] = 0.f;

  const int n_slices = (K + kFewK - 1) / kFewK;
#pragma unroll
  for (int s = 0; s < kFewStages - 1; ++s) {
    if (s < n_slices) stage(s, s * kFewK);
    else cp_async_commit();
  }
  for (int s = 0; s < n_slices; ++s) {
    cp_async_wait<kFewStages - 2>();  // slice s has landed
    __syncthreads();                  // ... for every thread, and slice s - 1's buffer is free
    if (s + kFewStages - 1 < n_slices) stage((s + kFewStages - 1) % kFewStages, (s + kFewStages - 1) * kFewK);
    else cp_async_commit();
    const bf16* As = ring + static_cast<size_t>(s % kFewStages) * kStageElems;
    const bf16* Bs = As + kFewRows * kFewLd;
#pragma unroll
    for (int kk = 0; kk < kFewK; kk += 16) {
      unsigned af[4];
      ldmatrix_x4(af[0], af[1], af[2], af[3], As + (lane & 15) * kFewLd + kk + ((lane >> 4) << 3));
#pragma unroll
      for (int part = 0; part < (UP ? 2 : 1); ++part) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3,
                    Bs + (part * kFewCols + warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * kFewLd + kk + (((lane >> 3) & 1) << 3));
        mma_bf16(acc[2 * part], af, b0, b1);
        mma_bf16(acc[2 * part + 1], af, b2, b3);
      }
    }
  }

  const int c_in = (lane & 3) * 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = (lane >> 2) + half * 8;
    const int i = row0 + r;
    if (i >= row1) continue;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int col = n0 + warp * 16 + j * 8 + c_in + q;
        if (col >= N) continue;
        if (UP) {
          out[static_cast<size_t>(i) * N + col] =
              __float2bfloat16_rn(clamped_glu(acc[j][half * 2 + q], acc[UP ? 2 + j : j][half * 2 + q], limit, alpha, shift));
        } else {
          const float val = acc[j][half * 2 + q];
          out[static_cast<size_t>(ungated ? i : dst_row[r]) * N + col] = __float2bfloat16_rn(ungated ? relu_squared(val) : val);
        }
      }
    }
  }
}

// out[t] = sum_j p[t, j] y[t * top + j] (+ shared[t], times shared_gate[t] where there is one); y, shared and out in the storage type, the sum in float.
template <typename S>
__global__ void __launch_bounds__(256)
    moe_combine_kernel(const S* __restrict__ y, const float* __restrict__ weights, const S* __restrict__ shared,
                       const float* __restrict__ shared_gate, S* __restrict__ out, int D, int top) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < D; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j)
      acc += weights[static_cast<size_t>(t) * top + j] * ldf(y + (static_cast<size_t>(t) * top + j) * D + i);
    if (shared) acc += (shared_gate ? shared_gate[t] : 1.f) * ldf(shared + static_cast<size_t>(t) * D + i);
    stf(out + static_cast<size_t>(t) * D + i, acc);
  }
}

}  // namespace pmm

namespace pmm {
template <typename S, int TOK>
int launch_route(const void* x, long long ld_x, const float* w, const float* bias, int* ids, float* weights, int T, int D,
                 int E, int top, int scored, const float* correction, int groups, int keep, float scale,
                 const float* gate_w, float* gate_out, cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>(TOK) * ((D + 3) & ~3) + static_cast<size_t>(TOK) * E * (scored ? 3 : 1)) * sizeof(float);
  if (smem > 200 * 1024) return PMM_ERR_BAD_ARGUMENT;
  auto kern = moe_route_kernel<S, TOK>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  launch_pdl(kern, dim3((T + TOK - 1) / TOK), dim3(kRouteWarps * 32), smem, stream, static_cast<const S*>(x), ld_x, w, bias,
             ids, weights, T, D, E, top, scored, correction, groups, keep, scale, gate_w, gate_out);
  return launch_status();
}
}  // namespace pmm

// scored == 0: the `top` largest logits, weights their softmax.  scored != 0: scores sigmoid(z); the choice runs on
// score + correction (may be null) within the `keep` best of `groups` groups of neighbours; weights are the chosen
// scores over their sum, times scale.  scored == 2: scores softmax(z) over all experts; groups are ranked by their
// largest choice score; weights are the chosen scores times scale.
PMM_EXPORT int pmm_moe_route(const void* x, long long ld_x, const float* w, const float* bias, int* ids, float* weights,
                             int T, int D, int E, int top, int scored, const float* correction, int groups, int keep,
                             float scale, const float* gate_w, float* gate_out, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || E <= 0 || top <= 0 || top > E || (gate_w && !gate_out)) return PMM_ERR_BAD_ARGUMENT;
  if (scored && (groups <= 0 || E % groups || keep <= 0 || keep > groups || top > keep * (E / groups)))
    return PMM_ERR_BAD_ARGUMENT;
  // few tokens: a block each, so that the step's few rows still spread over the GPU; many: four a block, which
  // reads the router a quarter as often
  const bool four = T >= 512 && (static_cast<size_t>(4) * (((D + 3) & ~3) + 3 * E)) * sizeof(float) <= 96 * 1024;
  PMM_DISPATCH_DTYPE(dtype, S, {
    if (four)
      return pmm::launch_route<S, 4>(x, ld_x, w, bias, ids, weights, T, D, E, top, scored, correction, groups, keep, scale,
                                     gate_w, gate_out, stream);
    return pmm::launch_route<S, 1>(x, ld_x, w, bias, ids, weights, T, D, E, top, scored, correction, groups, keep, scale,
                                   gate_w, gate_out, stream);
  });
  return 0;
}

// ids [A] -> offsets [E + 1], tile_start [E + 1] (row tiles of `tile_rows`), perm [A].  One launch for up to
// kPlanSmallPairs pairs, else two.
PMM_EXPORT int pmm_moe_plan(const int* ids, int A, int E, int tile_rows, int* offsets, int* tile_start, int* perm,
                            cudaStream_t stream) {
  if (A <= 0) return 0;
  if (E <= 0 || E > 4096 || tile_rows <= 0) return PMM_ERR_BAD_ARGUMENT;
  if (A <= pmm::kPlanSmallPairs) {
    pmm::launch_pdl(pmm::moe_plan_small_kernel, dim3(1), dim3(256), static_cast<size_t>(A + E) * sizeof(int), stream, ids,
                    A, E, tile_rows, offsets, tile_start, perm);
    return pmm::launch_status();
  }
  pmm::launch_pdl(pmm::moe_plan_kernel, dim3(1), dim3(1024), static_cast<size_t>(E) * sizeof(int), stream, ids, A, E,
                  tile_rows, offsets, tile_start);
  int rc = pmm::launch_status();
  if (rc != 0) return rc;
  pmm::launch_pdl(pmm::moe_fill_kernel, dim3(E), dim3(1024), 0, stream, ids, A, static_cast<const int*>(offsets), perm);
  return pmm::launch_status();
}

// 0: float products on the CUDA cores, 1: mma.sync tiles, 2: mma.sync tiles for few pairs
PMM_EXPORT int pmm_moe_tile_rows(int tensor_cores) {
  return tensor_cores == 2 ? pmm::kFewRows : tensor_cores ? pmm::kMmaRows : pmm::kGenRows;
}

// up == 1: a = x [T, K] (ld_a), w [E, 2N, K], out act [A, N] (storage type).  up == 0: a = act [A, K], w [E, N, K],
// out y [A, N] in the storage type.  up == 2 (ungated experts): a = x [T, K], w [E, N, K], out act [A, N] = max(x W^T, 0)^2
// in the order of the sorted pairs.  tensor_cores != 0 needs bfloat16, K % 8 == 0, ld_a % 8 == 0 and 16-byte aligned a, w; the
// plan must have been made with pmm_moe_tile_rows(tensor_cores) rows a tile.
PMM_EXPORT int pmm_moe_gemm(const void* a, long long ld_a, const void* w, const int* perm, const int* offsets,
                            const int* tile_start, int A, int E, int top, int K, int N, int up, float limit, float alpha,
                            float shift, void* out, int tensor_cores, int dtype, cudaStream_t stream) {
  if (A <= 0) return 0;
  if (E <= 0 || top <= 0 || K <= 0 || N <= 0 || up < 0 || up > 2) return PMM_ERR_BAD_ARGUMENT;
  const int ungated = up == 2 ? 1 : 0;
  if (ungated) up = 0;
  const int tile_rows = pmm_moe_tile_rows(tensor_cores);
  const int row_tiles = A / tile_rows + (E < A ? E : A);
  if (row_tiles > 65535) return PMM_ERR_BAD_ARGUMENT;
  if (tensor_cores) {
    if (dtype != PMM_DTYPE_BF16 || K % 8 || ld_a % 8 || reinterpret_cast<uintptr_t>(a) % 16 ||
        reinterpret_cast<uintptr_t>(w) % 16)
      return PMM_ERR_BAD_ARGUMENT;
    if (tensor_cores == 2) {
      const dim3 grid((N + pmm::kFewCols - 1) / pmm::kFewCols, row_tiles);
      const size_t smem = static_cast<size_t>(pmm::kFewStages) * (pmm::kFewRows + (up ? 2 : 1) * pmm::kFewCols) *
                          pmm::kFewLd * sizeof(pmm::bf16);
      cudaError_t err;
      if (up) {
        auto kern = pmm::moe_gemm_few_kernel<true>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return static_cast<int>(err);
        pmm::launch_pdl(kern, grid, dim3(128), smem, stream, static_cast<const pmm::bf16*>(a), ld_a,
                        static_cast<const pmm::bf16*>(w), perm, offsets, tile_start, E, top, K, N, limit, alpha, shift,
                        ungated, static_cast<pmm::bf16*>(out));
      } else {
        auto kern = pmm::moe_gemm_few_kernel<false>;
        err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        if (err != cudaSuccess) return static_cast<int>(err);
        pmm::launch_pdl(kern, grid, dim3(128), smem, stream, static_cast<const pmm::bf16*>(a), ld_a,
                        static_cast<const pmm::bf16*>(w), perm, offsets, tile_start, E, top, K, N, limit, alpha, shift,
                        ungated, static_cast<pmm::bf16*>(out));
      }
      return pmm::launch_status();
    }
    const dim3 grid((N + pmm::kMmaCols - 1) / pmm::kMmaCols, row_tiles);
    if (up)
      pmm::launch_pdl(pmm::moe_gemm_mma_kernel<true>, grid, dim3(128), 0, stream, static_cast<const pmm::bf16*>(a), ld_a,
                      static_cast<const pmm::bf16*>(w), perm, offsets, tile_start, E, top, K, N, limit, alpha, shift, ungated, out);
    else
      pmm::launch_pdl(pmm::moe_gemm_mma_kernel<false>, grid, dim3(128), 0, stream, static_cast<const pmm::bf16*>(a), ld_a,
                      static_cast<const pmm::bf16*>(w), perm, offsets, tile_start, E, top, K, N, limit, alpha, shift, ungated, out);
    return pmm::launch_status();
  }
  const dim3 grid((N + pmm::kGenCols - 1) / pmm::kGenCols, row_tiles);
  PMM_DISPATCH_DTYPE(dtype, S, {
    if (up)
      pmm::launch_pdl(pmm::moe_gemm_generic_kernel<S, true>, grid, dim3(256), 0, stream, static_cast<const S*>(a), ld_a,
                      static_cast<const S*>(w), perm, offsets, tile_start, E, top, K, N, limit, alpha, shift, ungated, out);
    else
      pmm::launch_pdl(pmm::moe_gemm_generic_kernel<S, false>, grid, dim3(256), 0, stream, static_cast<const S*>(a), ld_a,
                      static_cast<const S*>(w), perm, offsets, tile_start, E, top, K, N, limit, alpha, shift, ungated, out);
  });
  return pmm::launch_status();
}

PMM_EXPORT int pmm_moe_combine(const void* y, const float* weights, const void* shared, const float* shared_gate, void* out,
                               int T, int D, int top, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || top <= 0) return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (D + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::moe_combine_kernel<S>, dim3(T, ytiles), dim3(256), 0, stream,
                                               static_cast<const S*>(y), weights, static_cast<const S*>(shared), shared_gate,
                                               static_cast<S*>(out), D, top));
  return pmm::launch_status();
}
