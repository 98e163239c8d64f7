// Launchers of attention_mma.cu that other sources of the library call: declared once, so that a
// changed argument list fails to compile instead of being called with the old one.
#pragma once
#include <cuda_runtime.h>

extern "C" int pmm_flash_supported(int Hq, int Hkv, int Dh);
extern "C" int pmm_flash_paged_attention(const void* q, const void* pool, const int* block_table,
                                         int max_blocks, const int* positions, const int* cu, void* out,
                                         float* part_o, float* part_ml, float scale, int window,
                                         int split_len, int n_splits, int page_size, int n_seq, int n_tiles,
                                         int tile_rows, int Hq, int Hkv, int Dh, int* split_counter,
                                         const float* sink, float* lse, cudaStream_t stream);
extern "C" int pmm_flash_combine(const float* part_o, const float* part_ml, void* out, int n_rows,
                                 int n_splits, int Dh, int dtype, cudaStream_t stream);
