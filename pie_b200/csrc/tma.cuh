// Tensor-map construction (host) and TMA issue helpers (device).
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace piekv {

// Pool [P, 2, 16, Hkv, 128] of 16-bit elements seen as the 5-D tensor
// {64 d, 16 tokens, 2 d-halves, Hkv, 2P (page, K|V)} with 128-byte swizzle; the box is
// {64, 16, box_halves, box_heads, box_kv}.  Shared memory receives [kv][head][half][token][64 d].
int make_page_tensor_map(CUtensorMap *tm, const void *pool, int num_pages, int hkv, int dtype, int box_halves,
                         int box_heads, int box_kv);

// q [n, Hq, 128] (strides in elements) seen as {64 d, n tokens, 2 d-halves, Hq}; box {64, rows, 2, heads}.
int make_q_tensor_map(CUtensorMap *tm, const void *q, int64_t nnz, int hq, int64_t q_sn, int64_t q_sh, int dtype,
                      int box_rows, int box_heads = 1);

// Row-major matrix [rows, cols] of 16-bit elements (row stride in elements) seen as {cols, rows}; box
// {box_cols (64: one 128-byte swizzled row), box_rows}: shared memory receives [box_rows][64], K-major.
int make_matrix_tensor_map(CUtensorMap *tm, const void *ptr, int64_t rows, int64_t cols, int64_t row_stride, int dtype,
                           int box_rows, int box_cols);

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, int c0, int c1, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *tmap, int c0, int c1, int c2, int c3,
                                            int c4, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *tmap, int c0, int c1, int c2, int c3,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}

}  // namespace piekv
