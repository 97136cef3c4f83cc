// Host-side construction of TMA tensor maps.  The driver entry point is resolved at run time
// through the runtime API, so the library has no link-time dependency on the driver library.
#include "tma.cuh"

namespace piekv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void *sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

static CUtensorMapDataType tm_dtype(int dtype) {
  return dtype == PIEKV_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

int make_page_tensor_map(CUtensorMap *tm, const void *pool, int num_pages, int hkv, int dtype, int box_halves,
                         int box_heads, int box_kv) {
  EncodeTiledFn enc = get_encode_fn();
  PIEKV_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t row = (cuuint64_t)hkv * 128 * 2;  // bytes of one token row (all heads)
  cuuint64_t gdim[5] = {64, 16, 2, (cuuint64_t)hkv, (cuuint64_t)num_pages * 2};
  cuuint64_t gstr[4] = {row, 128, 256, 16 * row};
  cuuint32_t box[5] = {64, 16, (cuuint32_t)box_halves, (cuuint32_t)box_heads, (cuuint32_t)box_kv};
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = enc(tm, tm_dtype(dtype), 5, const_cast<void *>(pool), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PIEKV_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (pages) failed with CUresult %d", (int)r);
  return 0;
}

int make_q_tensor_map(CUtensorMap *tm, const void *q, int64_t nnz, int hq, int64_t q_sn, int64_t q_sh, int dtype,
                      int box_rows, int box_heads) {
  EncodeTiledFn enc = get_encode_fn();
  PIEKV_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[4] = {64, (cuuint64_t)nnz, 2, (cuuint64_t)hq};
  cuuint64_t gstr[3] = {(cuuint64_t)q_sn * 2, 128, (cuuint64_t)q_sh * 2};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 2, (cuuint32_t)box_heads};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, tm_dtype(dtype), 4, const_cast<void *>(q), gdim, gstr, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PIEKV_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (q) failed with CUresult %d", (int)r);
  return 0;
}


int make_matrix_tensor_map(CUtensorMap *tm, const void *ptr, int64_t rows, int64_t cols, int64_t row_stride, int dtype,
                           int box_rows, int box_cols) {
  EncodeTiledFn enc = get_encode_fn();
  PIEKV_REQUIRE(enc != nullptr, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t gstr[1] = {(cuuint64_t)row_stride * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, tm_dtype(dtype), 2, const_cast<void *>(ptr), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PIEKV_REQUIRE(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (matrix) failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace piekv
