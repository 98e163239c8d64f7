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
#include "mma_helpers.cuh"

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
  extern __shared__ __align__(16) float side_smem[];  // x [TOK][D] | y [TOK][D] | g [TOK][R] | e [TOK][R]
  __shared__ float red[TOK * (kSideThreads / 32)];
  float* xs = side_smem;
  float* ys = xs + static_cast<size_t>(TOK) * D;
  float* gs = ys + static_cast<size_t>(TOK) * D;
  float* es = gs + TOK * R;
  pdl_launch_dependents();
  const int t0 = blockIdx.x * TOK;
  const int nt = min(TOK, T - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // What does not depend on the launch before this one is asked for while that one still runs: the two matrices
  // towards the L2 (the blocks share out their 128-byte lines) and the tokens' table entries (two dependent
  // reads a token, all in flight at once).
  {
    const int lines = static_cast<int>((static_cast<size_t>(R) * D * sizeof(S)) >> 7);  // per matrix
    const int each = min(kSideThreads, (lines + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
    if (static_cast<int>(threadIdx.x) < each) {
      const size_t line = static_cast<size_t>((blockIdx.x * each + threadIdx.x) % lines) << 7;
      asm volatile("prefetch.global.L2 [%0];\n" ::"l"(reinterpret_cast<const char*>(w_gate) + line));
      asm volatile("prefetch.global.L2 [%0];\n" ::"l"(reinterpret_cast<const char*>(w_proj_t) + line));
    }
  }
  for (int idx = threadIdx.x; idx < TOK * R; idx += kSideThreads) {
    const int r = idx / R, j = idx - r * R;
    es[idx] = r < nt ? ldf(table + static_cast<long long>(tokens[t0 + r]) * ld_table + col0 + j) : 0.f;
  }
  pdl_wait();
  // x = h + sa * a + sb * b; the rows of a short last block that have no token are zero
  if (VEC) {
    const int per_row = D >> 2;
#pragma unroll 4
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
  // g[r][j] = gelu(Wg[j] . x_r) * e_r[j]: the rows of Wg are read once for the block's tokens; a warp takes four
  // rows at a time (VEC), so that their reads are in flight together and a piece of x serves four rows
  if (VEC) {
    for (int j0 = warp << 2; j0 < R; j0 += (kSideThreads / 32) << 2) {
      float acc[4][TOK];
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int r = 0; r < TOK; ++r) acc[q][r] = 0.f;
      const S* wr = w_gate + static_cast<size_t>(j0) * D;
#pragma unroll(TOK == 1 ? 4 : 2)
      for (int i = lane << 2; i < D; i += 128) {
        float4 w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = ld4(wr + static_cast<size_t>(q) * D + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) {
          const float4 x = *reinterpret_cast<const float4*>(xs + r * D + i);
#pragma unroll
          for (int q = 0; q < 4; ++q) acc[q][r] += w[q].x * x.x + w[q].y * x.y + w[q].z * x.z + w[q].w * x.w;
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int r = 0; r < TOK; ++r) {
          const float sum = warp_sum(acc[q][r]);
          if (lane == 0) gs[r * R + j0 + q] = gelu_tanh_f(sum) * es[r * R + j0 + q];
        }
    }
  } else {
    for (int j = warp; j < R; j += kSideThreads / 32) {
      const S* wr = w_gate + static_cast<size_t>(j) * D;
      float acc[TOK];
#pragma unroll
      for (int r = 0; r < TOK; ++r) acc[r] = 0.f;
      for (int i = lane; i < D; i += 32) {
        const float wv = ldf(wr + i);
#pragma unroll
        for (int r = 0; r < TOK; ++r) acc[r] += wv * xs[r * D + i];
      }
#pragma unroll
      for (int r = 0; r < TOK; ++r) {
        const float sum = warp_sum(acc[r]);
        if (lane == 0) gs[r * R + j] = gelu_tanh_f(sum) * es[r * R + j];
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
#pragma unroll 2
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
  for (int r = 0; r < TOK; ++r) {
    sq[r] = warp_sum(sq[r]);
    if (lane == 0) red[r * (kSideThreads / 32) + warp] = sq[r];
  }
  __syncthreads();  // (also: every thread's part of ys is written)
#pragma unroll
  for (int r = 0; r < TOK; ++r) {
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < kSideThreads / 32; ++k) total += red[r * (kSideThreads / 32) + k];
    inv[r] = 1.f / sqrtf(total / static_cast<float>(D) + eps);
  }
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

// The same update on the tensor cores (bfloat16 storage, mma.sync m16n8k16 with float accumulation): a block
// per 16 tokens, R = 16 * RK.  x enters the gate product rounded to bfloat16 and g the projection likewise; the
// sums, the activation, the root mean square and the new stream are float, and x itself is read again from the
// float stream and its branches for the final sum.  Wg x: the warps split D and their partial sums meet in
// shared memory.  Wp g: the warps split the columns; the tiles are made twice (K is only R), first for the
// sum of squares and then for the stream, so that no row of y waits anywhere, whatever D is.
constexpr int kSideMmaThreads = 512, kSideMmaWarps = kSideMmaThreads / 32, kSideMmaTok = 16;
constexpr int kSideStage = 33;  // floats a row of a warp's staged 16 x 32 piece of y
constexpr int kSideMmaFromTokens = 1024;  // below, a block per token on the CUDA cores fills the SMs better

inline size_t side_mma_smem_bytes(int D, int R) {
  const size_t per_warp = static_cast<size_t>(R > kSideStage ? R : kSideStage) * kSideMmaTok;
  return static_cast<size_t>(kSideMmaTok) * (D + 32) * 2 + static_cast<size_t>(kSideMmaWarps) * per_warp * 4 +
         static_cast<size_t>(kSideMmaTok) * R * 4 + static_cast<size_t>(kSideMmaWarps) * kSideMmaTok * 4 +
         static_cast<size_t>(kSideMmaTok) * 4 + static_cast<size_t>(kSideMmaTok) * (R + 8) * 2;
}

template <int RK>
__global__ void __launch_bounds__(kSideMmaThreads)  // (64 registers for two blocks an SM, and 256 threads a block, measured slower)
    token_gated_update_mma_kernel(float* __restrict__ h, const bf16* __restrict__ a, float sa, const bf16* __restrict__ b,
                                  float sb, const int* __restrict__ tokens, const bf16* __restrict__ table,
                                  long long ld_table, int col0, const bf16* __restrict__ w_gate,
                                  const bf16* __restrict__ w_proj, const float* __restrict__ norm_w, float eps, int T, int D) {
  constexpr int R = 16 * RK, NT1 = 2 * RK, GS = R + 8, PW = (R > kSideStage ? R : kSideStage) * kSideMmaTok;
  extern __shared__ __align__(16) unsigned char side_mma_smem[];
  const int XS = D + 32;                                            // row stride of xb: neighbouring rows 64 bytes apart in the banks
  bf16* xb = reinterpret_cast<bf16*>(side_mma_smem);                // [16][D + 32]
  float* part = reinterpret_cast<float*>(xb + kSideMmaTok * XS);    // [warps][16][R], later [warps][16][33] (a warp's staged tiles)
  float* es = part + kSideMmaWarps * PW;                            // [16][R]
  float* sqs = es + kSideMmaTok * R;                                // [warps][16]
  float* invs = sqs + kSideMmaWarps * kSideMmaTok;                  // [16]
  bf16* gb = reinterpret_cast<bf16*>(invs + kSideMmaTok);           // [16][R + 8]
  pdl_launch_dependents();
  const int t0 = blockIdx.x * kSideMmaTok;
  const int nt = min(kSideMmaTok, T - t0);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  // What does not depend on the launch before this one is asked for while that one still runs: the two matrices
  // towards the L2 (every block a slice of their 128-byte lines, all blocks together all of them) and the
  // tokens' table entries.
  {
    const int lines = (R * D * 2) >> 7;  // per matrix
    const int mine = blockIdx.x * 16 + static_cast<int>(threadIdx.x);
    if (threadIdx.x < 16 && lines > 0) {
      const char* p0 = reinterpret_cast<const char*>(w_gate) + (static_cast<size_t>(mine % lines) << 7);
      const char* p1 = reinterpret_cast<const char*>(w_proj) + (static_cast<size_t>(mine % lines) << 7);
      asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p0));
      asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p1));
    }
  }
  for (int idx = threadIdx.x; idx < kSideMmaTok * R; idx += kSideMmaThreads) {
    const int r = idx / R, j = idx - r * R;
    es[idx] = r < nt ? ldf(table + static_cast<long long>(tokens[t0 + r]) * ld_table + col0 + j) : 0.f;
  }
  pdl_wait();
  const int per_row = D >> 2;
#pragma unroll 4
  for (int idx = threadIdx.x; idx < kSideMmaTok * per_row; idx += kSideMmaThreads) {
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
    *reinterpret_cast<uint2*>(xb + r * XS + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  }
  __syncthreads();
  // In both products a lane reads its operands in 16-byte pieces of one row, so the order of the summed index
  // inside a product step differs from the instruction's own; it is the same on both sides, which is all a sum
  // needs.  Slices of 32 of D here: lane (g, t) holds entries t * 8 .. t * 8 + 7 of its rows of x and of Wg.
  {  // part[warp] = x[:, this warp's slices of D] Wg[:, the same]^T
    float acc[NT1][4];
#pragma unroll
    for (int n = 0; n < NT1; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll 2
    for (int k0 = warp * 32; k0 < D; k0 += kSideMmaWarps * 32) {
      const bf16* xr = xb + g * XS + k0 + t * 8;
      const uint4 lo = *reinterpret_cast<const uint4*>(xr);
      const uint4 hi = *reinterpret_cast<const uint4*>(xr + 8 * XS);
      const unsigned a0[4] = {lo.x, hi.x, lo.y, hi.y}, a1[4] = {lo.z, hi.z, lo.w, hi.w};
      uint4 bw[NT1];
#pragma unroll
      for (int n = 0; n < NT1; ++n)
        bw[n] = *reinterpret_cast<const uint4*>(w_gate + static_cast<size_t>(n * 8 + g) * D + k0 + t * 8);
#pragma unroll
      for (int n = 0; n < NT1; ++n) {
        mma_bf16(acc[n], a0, bw[n].x, bw[n].y);
        mma_bf16(acc[n], a1, bw[n].z, bw[n].w);
      }
    }
    float* mine = part + warp * PW;
#pragma unroll
    for (int n = 0; n < NT1; ++n) {
      *reinterpret_cast<float2*>(mine + g * R + n * 8 + 2 * t) = make_float2(acc[n][0], acc[n][1]);
      *reinterpret_cast<float2*>(mine + (g + 8) * R + n * 8 + 2 * t) = make_float2(acc[n][2], acc[n][3]);
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kSideMmaTok * R; idx += kSideMmaThreads) {
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kSideMmaWarps; ++w) sum += part[w * PW + idx];
    const int r = idx / R, j = idx - r * R;
    gb[r * GS + j] = __float2bfloat16_rn(gelu_tanh_f(sum) * es[idx]);
  }
  __syncthreads();
  // Wp g: a tile's eight rows of Wp are 16 R bytes in a row; lane L reads bytes L * R / 2 .. of them, which are
  // entries t * 4 RK .. of row g, and takes the same entries of g_r on the other side.
  unsigned ga[RK][4];
#pragma unroll
  for (int kk = 0; kk < RK; ++kk) {
    const bf16* gr = gb + g * GS + t * 4 * RK + 4 * kk;
    ga[kk][0] = *reinterpret_cast<const unsigned*>(gr);
    ga[kk][1] = *reinterpret_cast<const unsigned*>(gr + 8 * GS);
    ga[kk][2] = *reinterpret_cast<const unsigned*>(gr + 2);
    ga[kk][3] = *reinterpret_cast<const unsigned*>(gr + 8 * GS + 2);
  }
  auto y_tile = [&](int tile, float* c) {
    c[0] = c[1] = c[2] = c[3] = 0.f;
    const bf16* wr = w_proj + static_cast<size_t>(tile) * 8 * R + lane * 4 * RK;
    unsigned bw[2 * RK];
    if (RK == 1) {
      const uint2 v = *reinterpret_cast<const uint2*>(wr);
      bw[0] = v.x, bw[1] = v.y;
    } else {
#pragma unroll
      for (int q = 0; q < RK / 2; ++q) {
        const uint4 v = reinterpret_cast<const uint4*>(wr)[q];
        bw[4 * q] = v.x, bw[4 * q + 1] = v.y, bw[4 * q + 2] = v.z, bw[4 * q + 3] = v.w;
      }
    }
#pragma unroll
    for (int kk = 0; kk < RK; ++kk) mma_bf16(c, ga[kk], bw[2 * kk], bw[2 * kk + 1]);
  };
  const int blocks32 = D >> 5;  // a warp takes blocks of 32 columns: four tiles
  float sq_lo = 0.f, sq_hi = 0.f;
  for (int cb = warp; cb < blocks32; cb += kSideMmaWarps) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float c[4];
      y_tile(cb * 4 + u, c);
      sq_lo += c[0] * c[0] + c[1] * c[1];
      sq_hi += c[2] * c[2] + c[3] * c[3];
    }
  }
  sq_lo += __shfl_xor_sync(0xffffffffu, sq_lo, 1);
  sq_lo += __shfl_xor_sync(0xffffffffu, sq_lo, 2);
  sq_hi += __shfl_xor_sync(0xffffffffu, sq_hi, 1);
  sq_hi += __shfl_xor_sync(0xffffffffu, sq_hi, 2);
  if (t == 0) {
    sqs[warp * kSideMmaTok + g] = sq_lo;
    sqs[warp * kSideMmaTok + g + 8] = sq_hi;
  }
  __syncthreads();
  if (threadIdx.x < kSideMmaTok) {
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < kSideMmaWarps; ++w) total += sqs[w * kSideMmaTok + threadIdx.x];
    invs[threadIdx.x] = 1.f / sqrtf(total / static_cast<float>(D) + eps);
  }
  __syncthreads();
  // The tiles once more, staged in shared memory so that the stream is read and written in whole rows of 32
  // columns; eight rows' reads are asked for before the first of their writes (the writes go to the array the
  // reads come from, so the compiler keeps their order).
  float* st = part + warp * PW;  // [16][33]
  for (int cb = warp; cb < blocks32; cb += kSideMmaWarps) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float c[4];
      y_tile(cb * 4 + u, c);
      st[g * kSideStage + u * 8 + 2 * t] = c[0];
      st[g * kSideStage + u * 8 + 2 * t + 1] = c[1];
      st[(g + 8) * kSideStage + u * 8 + 2 * t] = c[2];
      st[(g + 8) * kSideStage + u * 8 + 2 * t + 1] = c[3];
    }
    __syncwarp();
    const int col = cb * 32 + lane;
    const float w = norm_w[col];
#pragma unroll
    for (int r0 = 0; r0 < kSideMmaTok; r0 += 8) {
      float x[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        x[r] = 0.f;
        if (r0 + r < nt) {
          const size_t at = static_cast<size_t>(t0 + r0 + r) * D + col;
          x[r] = h[at];
          if (a) x[r] += sa * __bfloat162float(a[at]);
          if (b) x[r] += sb * __bfloat162float(b[at]);
        }
      }
#pragma unroll
      for (int r = 0; r < 8; ++r)
        if (r0 + r < nt)
          h[static_cast<size_t>(t0 + r0 + r) * D + col] = x[r] + st[(r0 + r) * kSideStage + lane] * invs[r0 + r] * w;
    }
    __syncwarp();
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
  const size_t smem = (static_cast<size_t>(2) * TOK * D + static_cast<size_t>(2) * TOK * R) * sizeof(float);
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

template <int RK>
int launch_token_gated_update_mma(float* h, const void* a, float sa, const void* b, float sb, const int* tokens,
                                  const void* table, long long ld_table, int col0, const void* w_gate, const void* w_proj,
                                  const float* norm_w, float eps, int T, int D, cudaStream_t stream) {
  const size_t smem = side_mma_smem_bytes(D, 16 * RK);
  auto kern = token_gated_update_mma_kernel<RK>;
  if (smem > 48 * 1024) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return static_cast<int>(err);
  }
  launch_pdl(kern, dim3((T + kSideMmaTok - 1) / kSideMmaTok), dim3(kSideMmaThreads), smem, stream, h,
             static_cast<const bf16*>(a), sa, static_cast<const bf16*>(b), sb, tokens, static_cast<const bf16*>(table),
             ld_table, col0, static_cast<const bf16*>(w_gate), static_cast<const bf16*>(w_proj), norm_w, eps, T, D);
  return launch_status();
}

}  // namespace pmm

// How many floats of shared memory a block of `tok` tokens needs; the launcher takes 4 tokens a block where
// the step has many tokens and they fit, else 1.
PMM_EXPORT int pmm_token_gated_update_fits(int D, int R) {
  return (static_cast<size_t>(2) * D + 2 * static_cast<size_t>(R)) * sizeof(float) <= 200 * 1024 ? 1 : 0;
}

// w_proj: Wp^T [R, D].  w_proj_rows: Wp [D, R] as stored, or null; with it, bfloat16 steps of many tokens whose
// sizes the tensor-core form takes (D a multiple of 32, R 16, 32 or 64) run that form.
PMM_EXPORT int pmm_token_gated_update(float* h, const void* a, float sa, const void* b, float sb, const int* tokens,
                                      const void* table, long long ld_table, int col0, const void* w_gate,
                                      const void* w_proj, const void* w_proj_rows, const float* norm_w, float eps, int T,
                                      int D, int R, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D <= 0 || R <= 0 || col0 < 0 || !pmm_token_gated_update_fits(D, R)) return PMM_ERR_BAD_ARGUMENT;
  {
    auto al = [](const void* p) { return p == nullptr || reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    if (dtype == PMM_DTYPE_BF16 && w_proj_rows != nullptr && T >= pmm::kSideMmaFromTokens && D % 32 == 0 &&
        (R == 16 || R == 32 || R == 64) && al(h) && al(a) && al(b) && al(w_gate) && al(w_proj_rows) && al(norm_w) &&
        pmm::side_mma_smem_bytes(D, R) <= 200 * 1024) {
#define PMM_SIDE_MMA(RK)                                                                                               \
  return pmm::launch_token_gated_update_mma<RK>(h, a, sa, b, sb, tokens, table, ld_table, col0, w_gate, w_proj_rows, \
                                                norm_w, eps, T, D, stream)
      if (R == 16) PMM_SIDE_MMA(1);
      if (R == 32) PMM_SIDE_MMA(2);
      PMM_SIDE_MMA(4);
#undef PMM_SIDE_MMA
    }
  }
  const bool four = T >= 1024 && (static_cast<size_t>(8) * D + 8 * static_cast<size_t>(R)) * sizeof(float) <= 200 * 1024;
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
