// The grouped products of the routed feed-forward on the fifth-generation tensor cores, for steps of
// many tokens (bfloat16).  The rows are the (token, choice) pairs sorted by expert (see moe.cu); a row
// tile of 128 rows belongs to one expert and may be ragged at its end.
//
//   up:    act[i, f] = glu((xs W_gate,e^T)[i, f], (xs W_up,e^T)[i, f])     xs = the token rows in sorted order
//   down:  y[perm[i], :] = act[i] W_down,e^T
//
// One block computes 128 rows x 256 accumulator columns (up: 128 gate columns beside their 128 up
// columns; down: 256 output columns).  Structure as in tc_gemm.cu: a TMA producer warp fills a ring
// of 64-wide K slices (A: one box of 128 sorted rows; B: two boxes of 128 weight rows of the tile's
// expert out of the stacked matrix), one thread issues tcgen05.mma (M = 128, N = 256, K = 16) into
// tensor memory, four epilogue warps read the accumulator a lane quarter each, apply the
// activation and store whole row pieces.  Rows of a tile that lie beyond the expert's last row are
// computed (they belong to the next expert, or are zero past the end) and not stored; weight rows
// beyond the expert's block are loaded and their columns not stored.  Every mbarrier wait is
// bounded; a wait that gives up records a code in *status and the block leaves.  No cluster
// multicast is used.
#include "tcgen05.cuh"

namespace pmm {

using bf16 = __nv_bfloat16;

constexpr int kGM = 128;         // rows per tile
constexpr int kGN = 256;         // accumulator columns per tile
constexpr int kGK = 64;          // K per stage: one 128-byte swizzle row of bfloat16
constexpr int kGStages = 4;
constexpr int kGThreads = 192;   // warp 0: TMA producer, warp 1: tensor memory and MMA, warps 2..5: epilogue
constexpr int kGABytes = kGM * kGK * 2;  // 16 KB
constexpr int kGBBytes = kGN * kGK * 2;  // 32 KB
constexpr size_t kGSmem = static_cast<size_t>(kGStages) * (kGABytes + kGBBytes) + 1024 /*alignment*/;
constexpr unsigned kGIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((kGN >> 3) << 17) | ((kGM >> 4) << 24);

__device__ __forceinline__ bool moe_tc_tile(int tile, const int* __restrict__ offsets, const int* __restrict__ tile_start,
                                            int E, int& e, int& row0, int& row1) {
  if (tile >= tile_start[E]) return false;
  int lo = 0, hi = E - 1;  // the last e with tile_start[e] <= tile
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (tile_start[mid] <= tile) lo = mid; else hi = mid - 1;
  }
  e = lo;
  row0 = offsets[e] + (tile - tile_start[e]) * kGM;
  row1 = min(offsets[e + 1], row0 + kGM);
  return true;
}

template <bool UP>
__global__ void __launch_bounds__(kGThreads)
    moe_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                  const int* __restrict__ perm, const int* __restrict__ offsets, const int* __restrict__ tile_start, int E,
                  int K, int N, float limit, float alpha, float shift, int ungated, void* __restrict__ out,
                  int* __restrict__ status) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ unsigned char smem_raw[];
  __shared__ __align__(8) unsigned long long bar_full[kGStages], bar_empty[kGStages], bar_accum;
  __shared__ unsigned s_tmem_base;
  __shared__ int s_abort;

  int e, row0, row1;
  if (!moe_tc_tile(blockIdx.x, offsets, tile_start, E, e, row0, row1)) return;  // the whole block leaves together

  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sA = tiles;
  unsigned char* sB = tiles + kGStages * kGABytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * (UP ? kGN / 2 : kGN);      // first output column of the tile
  const int w_row = e * (UP ? 2 * N : N) + n0;           // first weight row of the tile in the stacked matrix
  const int k_blocks = (K + kGK - 1) / kGK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], 1);
    }
    mbar_init(&bar_accum, 1);
    s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&s_tmem_base)), "r"(kGN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const unsigned tmem_base = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int issued = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int s = kb % kGStages;
        const unsigned use = kb / kGStages;
        if (!mbar_wait(&bar_empty[s], (use & 1) ^ 1, abort_flag)) {
          if (!*abort_flag) atomicExch(status, 11);
          s_abort = 1;
          break;
        }
        mbar_expect_tx(&bar_full[s], kGABytes + kGBBytes);
        tma_load_2d(sA + s * kGABytes, &map_a, kb * kGK, row0, &bar_full[s]);
        tma_load_2d(sB + s * kGBBytes, &map_w, kb * kGK, w_row, &bar_full[s]);
        tma_load_2d(sB + s * kGBBytes + kGBBytes / 2, &map_w, kb * kGK, w_row + (UP ? N : kGN / 2), &bar_full[s]);
        issued = kb + 1;
      }
      if (s_abort) {
        // copies already requested still write into this block's shared memory: wait for them
        for (int kb = issued > kGStages ? issued - kGStages : 0; kb < issued; ++kb) {
          const int s = kb % kGStages;
          for (unsigned i = 0; i < kSpinLimit && !mbar_try_wait(&bar_full[s], (kb / kGStages) & 1); ++i) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = true;
      for (int kb = 0; kb < k_blocks && ok; ++kb) {
        const int s = kb % kGStages;
        if (!mbar_wait(&bar_full[s], (kb / kGStages) & 1, abort_flag)) {
          if (!*abort_flag) atomicExch(status, 12);
          s_abort = 1;
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const unsigned long long a_desc = umma_desc(sA + s * kGABytes);
        const unsigned long long b_desc = umma_desc(sB + s * kGBBytes);
#pragma unroll
        for (int k = 0; k < kGK / 16; ++k)
          umma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kGIdesc, (kb > 0 || k > 0) ? 1u : 0u);
        umma_commit(&bar_empty[s]);
      }
      if (ok) umma_commit(&bar_accum);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quad = warp & 3;  // a warp may only read tensor-memory lanes 32 * (warp % 4) ...
    bool ok = mbar_wait(&bar_accum, 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) {
      if (lane == 0 && !*abort_flag) atomicExch(status, 13);
      s_abort = 1;
    } else {
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const int i = row0 + quad * 32 + lane;  // this thread's row among the sorted pairs
      const bool row_ok = i < row1;
      const unsigned lane_base = tmem_base + (static_cast<unsigned>(quad * 32) << 16);
      if (UP) {
        bf16* dst_row = static_cast<bf16*>(out) + static_cast<size_t>(row_ok ? i : 0) * N;
#pragma unroll 1
        for (int c = 0; c < kGN / 64; ++c) {
          unsigned g[32], u[32];
          tmem_ld32(lane_base + c * 32, g);
          tmem_ld32(lane_base + kGN / 2 + c * 32, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n0 + c * 32 + j;
              if (col < N) {  // N is a multiple of 8
                uint4 pack;
                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pack);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  float r[2];
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
                    const float gv = fminf(__uint_as_float(g[j + 2 * q + h]), limit);
                    const float uv = fminf(fmaxf(__uint_as_float(u[j + 2 * q + h]), -limit), limit);
                    r[h] = __fdividef(gv, 1.f + __expf(-alpha * gv)) * (uv + shift);
                  }
                  p2[q] = __floats2bfloat162_rn(r[0], r[1]);
                }
                *reinterpret_cast<uint4*>(dst_row + col) = pack;
              }
            }
          }
        }
      } else {
        // (ungated experts' up product: rows stay in the order of the sorted pairs, values become max(z, 0)^2)
        bf16* dst_row = static_cast<bf16*>(out) + static_cast<size_t>(row_ok ? (ungated ? i : perm[i]) : 0) * N;
#pragma unroll 1
        for (int q = 0; q < kGN / 32; ++q) {
          unsigned v[32];
          tmem_ld32(lane_base + q * 32, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              const int col = n0 + q * 32 + j;
              if (col < N) {  // N is a multiple of 8
                uint4 pack;
                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pack);
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                  float v0 = __uint_as_float(v[j + 2 * h]), v1 = __uint_as_float(v[j + 2 * h + 1]);
                  if (ungated) {
                    v0 = fmaxf(v0, 0.f), v1 = fmaxf(v1, 0.f);
                    v0 *= v0, v1 *= v1;
                  }
                  p2[h] = __floats2bfloat162_rn(v0, v1);
                }
                *reinterpret_cast<uint4*>(dst_row + col) = pack;
              }
            }
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kGN) : "memory");
  }
}

// bfloat16 matrix [rows, cols] with row stride ld (elements); box = 64 columns x 128 rows, 128-byte swizzle,
// zeros outside.
inline bool moe_make_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {kGK, kGM};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// xs[i, :] = x[perm[i] / top, :]: the token rows in the order of the sorted pairs (16-byte pieces).
__global__ void __launch_bounds__(256)
    moe_gather_rows_kernel(const bf16* __restrict__ x, long long ld_x, const int* __restrict__ perm, int top,
                           bf16* __restrict__ xs, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(perm[i] / top) * ld_x);
  uint4* dst = reinterpret_cast<uint4*>(xs + static_cast<size_t>(i) * K);
  for (int c = threadIdx.x; c < K / 8; c += blockDim.x) dst[c] = src[c];
}

}  // namespace pmm

PMM_EXPORT int pmm_moe_tc_tile_rows() { return pmm::kGM; }

// K a multiple of 64 (whole swizzle rows), N a multiple of 8 (whole 16-byte pieces), 16-byte aligned rows.
PMM_EXPORT int pmm_moe_tc_supported(int K, int N, long long ld_a) {
  return K > 0 && K % pmm::kGK == 0 && N > 0 && N % 8 == 0 && ld_a % 8 == 0;
}

PMM_EXPORT int pmm_moe_gather_rows(const void* x, long long ld_x, const int* perm, int A, int top, void* xs, int K,
                                   cudaStream_t stream) {
  if (A <= 0) return 0;
  if (K <= 0 || K % 8 || ld_x % 8 || top <= 0 || reinterpret_cast<uintptr_t>(x) % 16 || reinterpret_cast<uintptr_t>(xs) % 16)
    return PMM_ERR_BAD_ARGUMENT;
  pmm::launch_pdl(pmm::moe_gather_rows_kernel, dim3(A), dim3(K / 8 < 256 ? ((K / 8 + 31) / 32) * 32 : 256), 0, stream,
                  static_cast<const pmm::bf16*>(x), ld_x, perm, top, static_cast<pmm::bf16*>(xs), K);
  return pmm::launch_status();
}

// a [A, K] bfloat16 rows in the order of the sorted pairs (row stride ld_a); w the experts' stacked matrices
// [E * (up ? 2N : N), K]; the plan made with rows of pmm_moe_tc_tile_rows().  up: out = act [A, N] bfloat16;
// else out = y [A, N] bfloat16, row perm[i].  status: one int, stays 0 unless a bounded wait gave up.
PMM_EXPORT int pmm_moe_tc_gemm(const void* a, long long ld_a, const void* w, const int* perm, const int* offsets,
                               const int* tile_start, int A, int E, int K, int N, int up, float limit, float alpha,
                               float shift, void* out, int* status, cudaStream_t stream) {
  if (A <= 0) return 0;
  if (E <= 0 || !pmm_moe_tc_supported(K, N, ld_a) || !status || up < 0 || up > 2) return PMM_ERR_BAD_ARGUMENT;
  const int ungated = up == 2 ? 1 : 0;  // up == 2: w [E * N, K], out = max(a W^T, 0)^2 in the order of the sorted pairs
  if (ungated) up = 0;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(w) % 16 || reinterpret_cast<uintptr_t>(out) % 16)
    return PMM_ERR_BAD_ARGUMENT;
  CUtensorMap map_a, map_w;
  const long long w_rows = static_cast<long long>(E) * (up ? 2LL * N : N);
  if (!pmm::moe_make_map(&map_a, a, A, K, ld_a) || !pmm::moe_make_map(&map_w, w, w_rows, K, K)) return PMM_ERR_BAD_ARGUMENT;
  const int row_tiles = A / pmm::kGM + (E < A ? E : A);
  const int cols_per_block = up ? pmm::kGN / 2 : pmm::kGN;
  dim3 grid(row_tiles, (N + cols_per_block - 1) / cols_per_block);
  if (grid.y > 65535) return PMM_ERR_BAD_ARGUMENT;
  cudaError_t err;
  if (up) {
    auto kern = pmm::moe_tc_kernel<true>;
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pmm::kGSmem));
    if (err != cudaSuccess) return static_cast<int>(err);
    pmm::launch_pdl(kern, grid, dim3(pmm::kGThreads), pmm::kGSmem, stream, map_a, map_w, perm, offsets, tile_start, E, K, N,
                    limit, alpha, shift, ungated, out, status);
  } else {
    auto kern = pmm::moe_tc_kernel<false>;
    err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(pmm::kGSmem));
    if (err != cudaSuccess) return static_cast<int>(err);
    pmm::launch_pdl(kern, grid, dim3(pmm::kGThreads), pmm::kGSmem, stream, map_a, map_w, perm, offsets, tile_start, E, K, N,
                    limit, alpha, shift, ungated, out, status);
  }
  return pmm::launch_status();
}
