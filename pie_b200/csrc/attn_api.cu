// C ABI of the attention entry points: argument checks and kernel selection.
#include "attn.cuh"
#include "common.cuh"

namespace piekv {
int64_t decode_tma_workspace_bytes(int batch, int hq, int hkv);
int64_t prefill_tc_workspace_bytes(int batch, int nnz, int hq);
}  // namespace piekv

using namespace piekv;

static int check_common(const AttnArgs &a, int dtype, const char *who) {
  PIEKV_REQUIRE(dtype >= PIEKV_F32 && dtype <= PIEKV_BF16, "%s: unknown dtype %d", who, dtype);
  PIEKV_REQUIRE(a.batch >= 0 && a.nnz >= 0, "%s: negative batch / nnz", who);
  PIEKV_REQUIRE(a.hq > 0 && a.hkv > 0 && a.hq % a.hkv == 0, "%s: num_qo_heads %d not a multiple of num_kv_heads %d",
                who, a.hq, a.hkv);
  PIEKV_REQUIRE(a.dim > 0 && a.page_size > 0 && a.num_pages > 0, "%s: bad head_dim / page_size / num_pages", who);
  if (a.nnz > 0) {
    PIEKV_REQUIRE(a.q && a.pool && a.out && a.kv_indptr && a.kv_indices && a.kv_last_page_len, "%s: null pointer", who);
  }
  return 0;
}

extern "C" int64_t piekv_decode_counter_bytes(int32_t batch) {
  (void)batch;
  return 65536;
}

extern "C" int64_t piekv_decode_workspace_bytes(int32_t batch, int32_t num_qo_heads, int32_t num_kv_heads,
                                                int32_t head_dim) {
  (void)head_dim;
  if (batch < 0 || num_qo_heads <= 0 || num_kv_heads <= 0) return 0;
  return decode_tma_workspace_bytes(batch, num_qo_heads, num_kv_heads);
}

extern "C" int piekv_decode_run(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool, void *out,
                                float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                                const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                                int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes, int32_t *err,
                                void *stream) {
  AttnArgs a{};
  a.q = q;
  a.q_sn = q_stride_n;
  a.q_sh = q_stride_h;
  a.pool = pool;
  a.out = out;
  a.lse = lse;
  a.qo_indptr = nullptr;
  a.kv_indptr = kv_indptr;
  a.kv_indices = kv_indices;
  a.kv_last_page_len = kv_last_page_len;
  a.mask = nullptr;
  a.causal = 0;
  a.batch = batch;
  a.nnz = batch;
  a.hq = num_qo_heads;
  a.hkv = num_kv_heads;
  a.dim = head_dim;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.sm_scale = sm_scale;
  a.err = err;
  if (int rc = check_common(a, dtype, "decode_run")) return rc;
  if (batch == 0) return 0;
  if (decode_tma_supported(a, dtype)) return launch_decode_tma(a, dtype, workspace, workspace_bytes, (cudaStream_t)stream);
  return launch_attn_generic(a, dtype, (cudaStream_t)stream);
}

extern "C" int64_t piekv_prefill_workspace_bytes(int32_t batch, int32_t nnz, int32_t num_qo_heads, int32_t head_dim) {
  (void)head_dim;
  if (batch < 0 || nnz < 0 || num_qo_heads <= 0) return 0;
  return prefill_tc_workspace_bytes(batch, nnz, num_qo_heads);
}

extern "C" int piekv_prefill_run(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool, void *out,
                                 float *lse, const int32_t *qo_indptr, const int32_t *kv_indptr,
                                 const int32_t *kv_indices, const int32_t *kv_last_page_len,
                                 const uint8_t *custom_mask, int32_t causal, int32_t batch, int32_t nnz,
                                 int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim, int32_t page_size,
                                 int32_t num_pages, int32_t dtype, float sm_scale, void *workspace,
                                 int64_t workspace_bytes, int32_t *err, void *stream) {
  AttnArgs a{};
  a.q = q;
  a.q_sn = q_stride_n;
  a.q_sh = q_stride_h;
  a.pool = pool;
  a.out = out;
  a.lse = lse;
  a.qo_indptr = qo_indptr;
  a.kv_indptr = kv_indptr;
  a.kv_indices = kv_indices;
  a.kv_last_page_len = kv_last_page_len;
  a.mask = custom_mask;
  a.causal = causal;
  a.batch = batch;
  a.nnz = nnz;
  a.hq = num_qo_heads;
  a.hkv = num_kv_heads;
  a.dim = head_dim;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.sm_scale = sm_scale;
  a.err = err;
  if (int rc = check_common(a, dtype, "prefill_run")) return rc;
  PIEKV_REQUIRE(nnz == 0 || qo_indptr != nullptr, "prefill_run: qo_indptr is null");
  if (batch == 0 || nnz == 0) return 0;
  if (prefill_tc_supported(a, dtype)) return launch_prefill_tc(a, dtype, workspace, workspace_bytes, (cudaStream_t)stream);
  return launch_attn_generic(a, dtype, (cudaStream_t)stream);
}
