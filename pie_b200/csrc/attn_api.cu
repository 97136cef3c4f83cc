// C ABI of the attention entry points: argument checks and kernel selection.
#include "attn.cuh"
#include "common.cuh"
#include "rope.cuh"

namespace piekv {
int64_t decode_tma_workspace_bytes(int batch, int hq, int hkv);
bool decode_fused_tma_supported(const AttnArgs &a, int dtype, const void *k, const void *v, int64_t k_sn,
                                int64_t k_sh, int64_t v_sn, int64_t v_sh);
int launch_decode_fused_tma(const AttnArgs &a, int dtype, const void *k, const void *v, int64_t k_sn, int64_t k_sh,
                            int64_t v_sn, int64_t v_sh, const int32_t *pos_ids, const RopeDev &rope, void *workspace,
                            int64_t workspace_bytes, cudaStream_t st, const PeerOut *peer = nullptr);
int launch_decode_append_general(void *q_out, const void *q, const void *k, const void *v, int64_t q_sn, int64_t q_sh,
                                 int64_t k_sn, int64_t k_sh, int64_t v_sn, int64_t v_sh, const int32_t *pos_ids,
                                 int32_t *bi_scratch, int32_t *pos_scratch, void *pool, const int32_t *kv_indices,
                                 const int32_t *kv_indptr, const int32_t *kv_last_page_len, int batch, int hq, int hkv,
                                 int dim, int page_size, int num_pages, int dtype, const RopeDev &rp, int32_t *err,
                                 cudaStream_t st);
}  // namespace piekv

static const int64_t kCounterBytes = 65536;
// scratch of the fused step's general path: batch_indices, positions, rotated q (fp32-sized upper bound)
static int64_t general_fused_bytes(int batch, int hq, int dim) {
  return kCounterBytes + ((int64_t)batch * 8 + 255) / 256 * 256 + (int64_t)batch * hq * dim * 4 + 256;
}

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
  const int64_t a = decode_tma_workspace_bytes(batch, num_qo_heads, num_kv_heads);
  const int64_t b = general_fused_bytes(batch, num_qo_heads, head_dim);
  return a > b ? a : b;
}

static int apply_options(AttnArgs &a, const piekv_attn_options *opt, const char *who) {
  if (opt == nullptr) return 0;
  PIEKV_REQUIRE(opt->window_left >= -1, "%s: window_left %d (use -1 for no window)", who, opt->window_left);
  a.window_left = opt->window_left;
  a.sinks = opt->sinks;
  return 0;
}

extern "C" int piekv_decode_run_opt(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                                    void *out, float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                                    const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                    int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                                    int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes,
                                    int32_t *err, void *stream, const piekv_attn_options *opt) {
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
  if (int rc = apply_options(a, opt, "decode_run")) return rc;
  if (batch == 0) return 0;
  if (decode_tma_supported(a, dtype)) return launch_decode_tma(a, dtype, workspace, workspace_bytes, (cudaStream_t)stream);
  return launch_attn_generic(a, dtype, (cudaStream_t)stream);
}

extern "C" int piekv_decode_run(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool, void *out,
                                float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                                const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                                int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes, int32_t *err,
                                void *stream) {
  return piekv_decode_run_opt(q, q_stride_n, q_stride_h, pool, out, lse, kv_indptr, kv_indices, kv_last_page_len, batch,
                              num_qo_heads, num_kv_heads, head_dim, page_size, num_pages, dtype, sm_scale, workspace,
                              workspace_bytes, err, stream, nullptr);
}

static int decode_step_fused_impl(const void *q, const void *k, const void *v, int64_t q_stride_n, int64_t q_stride_h,
                                  int64_t k_stride_n, int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h,
                                  const int32_t *pos_ids, void *pool, void *out, float *lse, const int32_t *kv_indptr,
                                  const int32_t *kv_indices, const int32_t *kv_last_page_len, int32_t batch,
                                  int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim, int32_t page_size,
                                  int32_t num_pages, int32_t dtype, const piekv_rope_params *rope, float sm_scale,
                                  void *workspace, int64_t workspace_bytes, int32_t *err, void *stream,
                                  const piekv::PeerOut *peer, const piekv_attn_options *opt = nullptr) {
  AttnArgs a{};
  a.q = q;
  a.q_sn = q_stride_n;
  a.q_sh = q_stride_h;
  a.pool = pool;
  a.out = out;
  a.lse = lse;
  a.kv_indptr = kv_indptr;
  a.kv_indices = kv_indices;
  a.kv_last_page_len = kv_last_page_len;
  a.batch = batch;
  a.nnz = batch;
  a.hq = num_qo_heads;
  a.hkv = num_kv_heads;
  a.dim = head_dim;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.sm_scale = sm_scale;
  a.err = err;
  if (int rc = check_common(a, dtype, "decode_step_fused")) return rc;
  if (int rc = apply_options(a, opt, "decode_step_fused")) return rc;
  if (int rc = check_rope(rope, head_dim, "decode_step_fused")) return rc;
  if (batch == 0) return 0;
  PIEKV_REQUIRE(k && v, "decode_step_fused: null k / v");
  const bool do_rope = rope && rope->mode != PIEKV_ROPE_NONE;
  PIEKV_REQUIRE(!do_rope || pos_ids, "decode_step_fused: pos_ids required when rope is on");
  RopeDev rp;
  fill_inv_freq(rope, head_dim, &rp);
  cudaStream_t st = (cudaStream_t)stream;
  if (decode_fused_tma_supported(a, dtype, k, v, k_stride_n, k_stride_h, v_stride_n, v_stride_h))
    return launch_decode_fused_tma(a, dtype, k, v, k_stride_n, k_stride_h, v_stride_n, v_stride_h, pos_ids, rp,
                                   workspace, workspace_bytes, st, peer);
  PIEKV_REQUIRE(peer == nullptr, "decode_step_fused_peer: needs the tuned kernel (fp16/bf16, head_dim 128, page size 16, "
                                 "1/2/4/8 kv heads, 16-byte aligned buffers)");
  // general path: metadata -> RoPE + append (rotated q into scratch) -> general attention
  const int64_t need = general_fused_bytes(batch, num_qo_heads, head_dim);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= need,
                "decode_step_fused: workspace too small (%lld < %lld bytes)", (long long)workspace_bytes,
                (long long)need);
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0,
                "decode_step_fused: workspace must be 256-byte aligned");
  uint8_t *ws = reinterpret_cast<uint8_t *>(workspace) + kCounterBytes;
  int32_t *bi = reinterpret_cast<int32_t *>(ws);
  int32_t *pos = bi + batch;
  void *q_rot = ws + ((int64_t)batch * 8 + 255) / 256 * 256;
  if (int rc = launch_decode_append_general(q_rot, q, k, v, q_stride_n, q_stride_h, k_stride_n, k_stride_h,
                                            v_stride_n, v_stride_h, pos_ids, bi, pos, pool, kv_indices, kv_indptr,
                                            kv_last_page_len, batch, num_qo_heads, num_kv_heads, head_dim, page_size,
                                            num_pages, dtype, rp, err, st))
    return rc;
  if (do_rope) {
    a.q = q_rot;
    a.q_sn = (int64_t)num_qo_heads * head_dim;
    a.q_sh = head_dim;
  }
  return launch_attn_generic(a, dtype, st);
}

extern "C" int piekv_decode_step_fused(const void *q, const void *k, const void *v, int64_t q_stride_n,
                                       int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                                       int64_t v_stride_n, int64_t v_stride_h, const int32_t *pos_ids, void *pool,
                                       void *out, float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                                       const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                       int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                                       int32_t dtype, const piekv_rope_params *rope, float sm_scale, void *workspace,
                                       int64_t workspace_bytes, int32_t *err, void *stream) {
  return decode_step_fused_impl(q, k, v, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h,
                                pos_ids, pool, out, lse, kv_indptr, kv_indices, kv_last_page_len, batch, num_qo_heads,
                                num_kv_heads, head_dim, page_size, num_pages, dtype, rope, sm_scale, workspace,
                                workspace_bytes, err, stream, nullptr);
}

extern "C" int piekv_decode_step_fused_opt(const void *q, const void *k, const void *v, int64_t q_stride_n,
                                           int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                                           int64_t v_stride_n, int64_t v_stride_h, const int32_t *pos_ids, void *pool,
                                           void *out, float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                                           const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                           int32_t num_kv_heads, int32_t head_dim, int32_t page_size,
                                           int32_t num_pages, int32_t dtype, const piekv_rope_params *rope,
                                           float sm_scale, void *workspace, int64_t workspace_bytes, int32_t *err,
                                           void *stream, const piekv_attn_options *opt) {
  return decode_step_fused_impl(q, k, v, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h,
                                pos_ids, pool, out, lse, kv_indptr, kv_indices, kv_last_page_len, batch, num_qo_heads,
                                num_kv_heads, head_dim, page_size, num_pages, dtype, rope, sm_scale, workspace,
                                workspace_bytes, err, stream, nullptr, opt);
}

extern "C" int piekv_decode_step_fused_peer(const void *q, const void *k, const void *v, int64_t q_stride_n,
                                            int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                                            int64_t v_stride_n, int64_t v_stride_h, const int32_t *pos_ids,
                                            void *pool, const piekv_peer_outputs *peers, const int32_t *kv_indptr,
                                            const int32_t *kv_indices, const int32_t *kv_last_page_len, int32_t batch,
                                            int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim,
                                            int32_t page_size, int32_t num_pages, int32_t dtype,
                                            const piekv_rope_params *rope, float sm_scale, void *workspace,
                                            int64_t workspace_bytes, int32_t *err, void *stream) {
  PIEKV_REQUIRE(peers != nullptr, "decode_step_fused_peer: null peer description");
  PIEKV_REQUIRE(peers->world >= 1 && peers->world <= PIEKV_MAX_PEERS && peers->rank >= 0 && peers->rank < peers->world,
                "decode_step_fused_peer: world %d / rank %d", peers->world, peers->rank);
  PIEKV_REQUIRE(peers->row_heads >= num_qo_heads * peers->world, "decode_step_fused_peer: rows of %d heads cannot hold %d x %d",
                peers->row_heads, peers->world, num_qo_heads);
  piekv::PeerOut po{};
  po.n = peers->world;
  po.row_heads = peers->row_heads;
  po.head_off = peers->rank * num_qo_heads;
  po.step = peers->step;
  po.step_ptr = peers->step_counter;
  for (int d = 0; d < peers->world; ++d) {
    if (peers->step_counter != nullptr) {
      PIEKV_REQUIRE(peers->out_alt[d] != nullptr && (reinterpret_cast<uintptr_t>(peers->out_alt[d]) & 15) == 0,
                    "decode_step_fused_peer: out_alt of rank %d is null or not 16-byte aligned", d);
      po.dst_alt[d] = peers->out_alt[d];
    }
    PIEKV_REQUIRE(peers->out[d] != nullptr && peers->flags[d] != nullptr, "decode_step_fused_peer: null pointer for rank %d", d);
    PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(peers->out[d]) & 15) == 0, "decode_step_fused_peer: output of rank %d not 16-byte aligned", d);
    po.dst[d] = peers->out[d];
    po.flag[d] = peers->flags[d] + peers->rank;
  }
  // the tuned kernel checks a.out for alignment only; results go to the peers' buffers
  return decode_step_fused_impl(q, k, v, q_stride_n, q_stride_h, k_stride_n, k_stride_h, v_stride_n, v_stride_h,
                                pos_ids, pool, peers->out[peers->rank], nullptr, kv_indptr, kv_indices,
                                kv_last_page_len, batch, num_qo_heads, num_kv_heads, head_dim, page_size, num_pages,
                                dtype, rope, sm_scale, workspace, workspace_bytes, err, stream, &po);
}

static void fill_prefill_args(AttnArgs &a, const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                              void *out, float *lse, const int32_t *qo_indptr, const int32_t *kv_indptr,
                              const int32_t *kv_indices, const int32_t *kv_last_page_len, const uint8_t *custom_mask,
                              int32_t causal, int32_t batch, int32_t nnz, int32_t num_qo_heads, int32_t num_kv_heads,
                              int32_t head_dim, int32_t page_size, int32_t num_pages, float sm_scale, int32_t *err) {
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
  a.causal = custom_mask ? 0 : causal;  // a mask alone decides, as in the reference
  a.batch = batch;
  a.nnz = nnz;
  a.hq = num_qo_heads;
  a.hkv = num_kv_heads;
  a.dim = head_dim;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.sm_scale = sm_scale;
  a.err = err;
}

extern "C" int64_t piekv_prefill_workspace_bytes(int32_t batch, int32_t nnz, int32_t num_qo_heads, int32_t head_dim,
                                                 int32_t num_pages, int64_t mask_bytes) {
  (void)head_dim;
  (void)num_qo_heads;
  if (batch < 0 || nnz < 0 || num_pages < 0 || mask_bytes < 0) return 0;
  return prefill_tc_workspace_bytes(batch, nnz, num_pages, mask_bytes);
}

extern "C" int piekv_prefill_plan(const int32_t *qo_indptr, const int32_t *kv_indptr, const int32_t *kv_last_page_len,
                                  const uint8_t *custom_mask, int64_t mask_bytes, int32_t causal, int32_t batch,
                                  int32_t nnz, int32_t page_size, int32_t num_pages, void *workspace,
                                  int64_t workspace_bytes, int32_t *err, void *stream) {
  PIEKV_REQUIRE(batch >= 0 && nnz >= 0 && page_size > 0 && num_pages > 0, "prefill_plan: bad sizes");
  PIEKV_REQUIRE(nnz == 0 || (qo_indptr && kv_indptr && kv_last_page_len), "prefill_plan: null pointer");
  PIEKV_REQUIRE(custom_mask == nullptr || mask_bytes >= 0, "prefill_plan: negative mask size");
  if (page_size != 16) return 0;  // the general kernel needs no plan
  AttnArgs a{};
  fill_prefill_args(a, nullptr, 0, 0, nullptr, nullptr, nullptr, qo_indptr, kv_indptr, nullptr, kv_last_page_len,
                    custom_mask, causal, batch, nnz, 1, 1, 128, page_size, num_pages, 1.f, err);
  return launch_prefill_plan(a, mask_bytes, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" int piekv_prefill_plan_brle(const int32_t *qo_indptr, const int32_t *kv_indptr,
                                       const int32_t *kv_last_page_len, const uint32_t *brle_runs,
                                       const int32_t *brle_indptr, int64_t mask_bits, int32_t batch, int32_t nnz,
                                       int32_t page_size, int32_t num_pages, void *workspace, int64_t workspace_bytes,
                                       int32_t *err, void *stream) {
  PIEKV_REQUIRE(batch >= 0 && nnz >= 0 && page_size > 0 && num_pages > 0 && mask_bits >= 0, "prefill_plan_brle: bad sizes");
  PIEKV_REQUIRE(page_size == 16, "prefill_plan_brle: page size %d (the tensor-core path needs 16)", page_size);
  PIEKV_REQUIRE(nnz == 0 || (qo_indptr && kv_indptr && kv_last_page_len && brle_indptr),
                "prefill_plan_brle: null pointer");
  AttnArgs a{};
  fill_prefill_args(a, nullptr, 0, 0, nullptr, nullptr, nullptr, qo_indptr, kv_indptr, nullptr, kv_last_page_len,
                    nullptr, 0, batch, nnz, 1, 1, 128, page_size, num_pages, 1.f, err);
  return launch_prefill_plan(a, mask_bits, workspace, workspace_bytes, (cudaStream_t)stream, brle_runs, brle_indptr);
}

extern "C" int piekv_prefill_plan_opt(const int32_t *qo_indptr, const int32_t *kv_indptr,
                                      const int32_t *kv_last_page_len, const uint8_t *custom_mask,
                                      const uint32_t *brle_runs, const int32_t *brle_indptr, int64_t mask_entries,
                                      int32_t causal, int32_t window_left, int32_t batch, int32_t nnz,
                                      int32_t page_size, int32_t num_pages, void *workspace, int64_t workspace_bytes,
                                      int32_t *err, void *stream) {
  PIEKV_REQUIRE(batch >= 0 && nnz >= 0 && page_size > 0 && num_pages > 0 && mask_entries >= 0,
                "prefill_plan_opt: bad sizes");
  PIEKV_REQUIRE(window_left >= -1, "prefill_plan_opt: window_left %d (use -1 for no window)", window_left);
  PIEKV_REQUIRE(nnz == 0 || (qo_indptr && kv_indptr && kv_last_page_len), "prefill_plan_opt: null pointer");
  const bool brle = brle_runs != nullptr || brle_indptr != nullptr;
  PIEKV_REQUIRE(!(brle && custom_mask), "prefill_plan_opt: pass the mask either as bytes or as run lengths");
  PIEKV_REQUIRE(!brle || brle_indptr != nullptr, "prefill_plan_opt: brle_indptr is null");
  if (page_size != 16) {
    PIEKV_REQUIRE(!brle, "prefill_plan_opt: page size %d (a run-length mask needs the tensor-core path: 16)", page_size);
    return 0;  // the general kernel needs no plan; it applies the window itself
  }
  AttnArgs a{};
  fill_prefill_args(a, nullptr, 0, 0, nullptr, nullptr, nullptr, qo_indptr, kv_indptr, nullptr, kv_last_page_len,
                    custom_mask, (custom_mask || brle) ? 0 : causal, batch, nnz, 1, 1, 128, page_size, num_pages, 1.f,
                    err);
  a.window_left = window_left;
  return launch_prefill_plan(a, mask_entries, workspace, workspace_bytes, (cudaStream_t)stream, brle_runs, brle_indptr);
}

extern "C" int piekv_prefill_run(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool, void *out,
                                 float *lse, const int32_t *qo_indptr, const int32_t *kv_indptr,
                                 const int32_t *kv_indices, const int32_t *kv_last_page_len,
                                 const uint8_t *custom_mask, int64_t mask_bytes, int32_t causal, int32_t planned,
                                 int32_t batch, int32_t nnz, int32_t num_qo_heads, int32_t num_kv_heads,
                                 int32_t head_dim, int32_t page_size, int32_t num_pages, int32_t dtype, float sm_scale,
                                 void *workspace, int64_t workspace_bytes, int32_t *err, void *stream) {
  return piekv_prefill_run_opt(q, q_stride_n, q_stride_h, pool, out, lse, qo_indptr, kv_indptr, kv_indices,
                               kv_last_page_len, custom_mask, mask_bytes, causal, planned, batch, nnz, num_qo_heads,
                               num_kv_heads, head_dim, page_size, num_pages, dtype, sm_scale, workspace, workspace_bytes,
                               err, stream, nullptr);
}

extern "C" int piekv_prefill_run_opt(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                                     void *out, float *lse, const int32_t *qo_indptr, const int32_t *kv_indptr,
                                     const int32_t *kv_indices, const int32_t *kv_last_page_len,
                                     const uint8_t *custom_mask, int64_t mask_bytes, int32_t causal, int32_t planned,
                                     int32_t batch, int32_t nnz, int32_t num_qo_heads, int32_t num_kv_heads,
                                     int32_t head_dim, int32_t page_size, int32_t num_pages, int32_t dtype,
                                     float sm_scale, void *workspace, int64_t workspace_bytes, int32_t *err,
                                     void *stream, const piekv_attn_options *opt) {
  AttnArgs a{};
  fill_prefill_args(a, q, q_stride_n, q_stride_h, pool, out, lse, qo_indptr, kv_indptr, kv_indices, kv_last_page_len,
                    custom_mask, causal, batch, nnz, num_qo_heads, num_kv_heads, head_dim, page_size, num_pages,
                    sm_scale, err);
  if (int rc = check_common(a, dtype, "prefill_run")) return rc;
  if (int rc = apply_options(a, opt, "prefill_run")) return rc;
  PIEKV_REQUIRE(nnz == 0 || qo_indptr != nullptr, "prefill_run: qo_indptr is null");
  if (batch == 0 || nnz == 0) return 0;
  if (planned == 2) {
    PIEKV_REQUIRE(prefill_tc_supported(a, dtype),
                  "prefill_run: a BRLE plan needs the tensor-core path (fp16/bf16, head_dim 128, page size 16)");
    a.mask = reinterpret_cast<const uint8_t *>(workspace);  // marks "masked"; the packed form is what is read
    a.causal = 0;
  }
  if (prefill_tc_supported(a, dtype)) {
    if (!planned) {
      if (int rc = launch_prefill_plan(a, mask_bytes, workspace, workspace_bytes, (cudaStream_t)stream)) return rc;
    }
    // with a window the plan holds a packed mask even when the caller passed none
    if (a.window_left >= 0 && a.mask == nullptr && mask_bytes > 0) a.mask = reinterpret_cast<const uint8_t *>(workspace);
    return launch_prefill_tc(a, dtype, mask_bytes, workspace, workspace_bytes, (cudaStream_t)stream);
  }
  return launch_attn_generic(a, dtype, (cudaStream_t)stream);
}
