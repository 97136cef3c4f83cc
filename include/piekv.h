/*
 * piekv.h - C ABI of libpiekv.so, the B200 (sm_100a) paged KV-cache hot path.
 *
 * The reference (zyma98/pie) has no C FFI at this seam: its Python worker calls a
 * module-level operator API (`ops.<name>`; the list of names a replacement must
 * export is pie/src/flashinfer_metal/__init__.py:14-37).  Each entry point below
 * names the reference call site it stands behind.  `pie_b200/ops.py` is the thin
 * Python shim that keeps the reference's names and keyword arguments and forwards
 * raw device pointers to these functions.
 *
 * Conventions
 *   - every pointer named q/k/v/pool/out/indptr/... is a DEVICE pointer unless the
 *     comment says "host";
 *   - `stream` is a cudaStream_t passed as void*; every call is stream-ordered,
 *     performs no device allocation and no synchronisation;
 *   - strides are in ELEMENTS; the innermost (head_dim) axis is contiguous;
 *   - `dtype` is one of PIEKV_F32 / PIEKV_F16 / PIEKV_BF16;
 *   - return value: 0 ok; >0 invalid argument (checked on the host, nothing was
 *     launched; text via piekv_last_error_string()); <0 is -(cudaError_t);
 *   - `err` (nullable) is a device int32[4] "error word": a kernel that meets an
 *     out-of-range index or gives up a bounded wait writes
 *     {code, kernel id, index, value} there with an atomic compare-and-swap on
 *     err[0] (first error wins) and skips the access.  Kernels never trap.
 *   - KV pool layout (one layer): [num_pages, 2, page_size, num_kv_heads, head_dim],
 *     "NHD", K at [:,0], V at [:,1]  (pie/src/pie_worker/model/llama3.py:959-979).
 */
#ifndef PIEKV_H_
#define PIEKV_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PIEKV_VERSION 103

/* element types */
#define PIEKV_F32 0
#define PIEKV_F16 1
#define PIEKV_BF16 2

/* RoPE modes */
#define PIEKV_ROPE_NONE 0    /* no rotation: pure append                                  */
#define PIEKV_ROPE_PLAIN 1   /* f_i = theta^(-2i/D)                                       */
#define PIEKV_ROPE_LLAMA31 2 /* plain + Llama-3.1 wavelength-dependent frequency scaling   */
#define PIEKV_ROPE_TABLE 3   /* cos/sin read from a caller-supplied fp32 table            */

/* device error-word codes (err[0]) */
#define PIEKV_ERR_NONE 0
#define PIEKV_ERR_BATCH_INDEX 1   /* batch_indices[i] outside [0,B)                         */
#define PIEKV_ERR_PAGE_SLOT 2     /* position / page_size beyond the request's page list    */
#define PIEKV_ERR_PAGE_ID 3       /* physical page id outside [0,num_pages)                 */
#define PIEKV_ERR_LAST_PAGE_LEN 4 /* kv_last_page_len outside [1,page_size]                 */
#define PIEKV_ERR_WAIT_TIMEOUT 5  /* a bounded on-chip wait ran out                         */
#define PIEKV_ERR_TABLE_RANGE 6   /* RoPE table position outside [0,table_len)              */
#define PIEKV_ERR_INDPTR 7        /* non-monotone indptr                                    */
#define PIEKV_ERR_NO_FREE_PAGE 8  /* device page table: fewer free pages than the call needs */
#define PIEKV_ERR_PAGE_CAPACITY 9 /* device page table: a request outgrew its row, or too many pages in one call */
#define PIEKV_ERR_SLOT 10         /* device page table: bad request slot / fork into a used slot */

/* RoPE parameters.  Reference arguments: apply_llama31_rope_pos_ids_inplace(q, k,
 * pos_ids, rope_scale, rope_theta, low_freq_factor, high_freq_factor, old_context_len)
 * at pie/src/pie_worker/model/llama3.py:660-669; arithmetic restated in
 * pie/src/flashinfer_metal/kernels/metal_rope.metal:58-106. */
typedef struct piekv_rope_params {
  int32_t mode;             /* PIEKV_ROPE_*                                               */
  int32_t interleave;       /* 0: pairs (i, i+D/2)  (reference default); 1: pairs (2i,2i+1) */
  float theta;              /* rope_theta                                                 */
  float scale;              /* rope_scale / rope_factor (LLAMA31 only)                    */
  float low_freq_factor;    /* LLAMA31 only                                               */
  float high_freq_factor;   /* LLAMA31 only                                               */
  float old_context_len;    /* LLAMA31 only                                               */
  int32_t table_len;        /* rows of cos_sin_table (TABLE only)                         */
  const float *cos_sin_table; /* device [table_len, D] fp32: cos in [:, :D/2], sin in [:, D/2:] */
} piekv_rope_params;

/* ---- library ------------------------------------------------------------------- */

/* Version of this ABI (PIEKV_VERSION of the build). No reference counterpart. */
int piekv_version(void);

/* Text of the last >0 / <0 status returned on the calling thread. Reference: Python
 * exceptions raised by the op library (pie/src/flashinfer_metal/ops.py:208-209). */
const char *piekv_last_error_string(void);

/* Process-wide options.  PIEKV_OPT_PDL: launch the tuned decode kernel with programmatic dependent
 * launch so that its prologue overlaps the tail of the kernel before it on the stream.
 *   0 off (default); 1 on, the kernel waits for the previous kernel before reading anything;
 *   2 on, and the caller guarantees that kv_indptr is not written by the kernel immediately before
 *     (the reference uploads the page tables once per step ahead of the layer loop,
 *     pie/src/pie_worker/batching.py:196-239): the offsets are read before the wait;
 *   3 as 2, and the caller also guarantees that the kernel immediately before wrote at most into the last
 *     two pages of any request of this batch (true when it is the previous decode step of the same
 *     requests, which appended one token each; false after a prefill, a refill or a page copy): the first
 *     pages of every SM's share are then requested before the wait, so that the launch and its first
 *     memory round trip hide behind the tail of the kernel before.
 * No reference counterpart. */
#define PIEKV_OPT_PDL 0
/* PIEKV_OPT_WORK_STEALING: 0 (default) - in the tuned decode kernel every SM keeps to its own page range
 * and equal inputs give bit-identical outputs; 1 - SMs that finish early take over page ranges of slower
 * ones, so how a request's pages are grouped before the partial results are merged (and with it the last
 * bits of the output) can differ from launch to launch.  It pays when the per-SM work is very uneven in
 * time; on the benchmark configurations it does not.  No reference counterpart. */
#define PIEKV_OPT_WORK_STEALING 1
int piekv_set_option(int32_t key, int32_t value);

/* ---- metadata (device-resident) ------------------------------------------------- */

/* seq_lens[b] = max(npages_b - 1, 0) * page_size + last_page_len[b]  (a request without pages
 * keeps last_page_len, as in pie/src/pie_worker/batching.py:104-111).
 * Replaces ops.get_seq_lens (call: llama3.py:745-749; restated ops.py:392-407). */
int piekv_get_seq_lens(const int32_t *kv_indptr, const int32_t *kv_last_page_len, int32_t batch,
                       int32_t page_size, int32_t *seq_lens_out, void *stream);

/* For token i of request b: batch_indices[i] = b,
 * positions[i] = seq_lens[b] - (indptr[b+1]-indptr[b]) + (i - indptr[b]).
 * Replaces ops.get_batch_indices_positions (call: llama3.py:751-755; ops.py:410-436). */
int piekv_get_batch_indices_positions(const int32_t *append_indptr, const int32_t *seq_lens,
                                      int32_t batch, int32_t nnz, int32_t *batch_indices_out,
                                      int32_t *positions_out, void *stream);

/* Both of the above in one launch (seq_lens_out may be NULL). */
int piekv_metadata(const int32_t *qo_indptr, const int32_t *kv_indptr,
                   const int32_t *kv_last_page_len, int32_t batch, int32_t nnz, int32_t page_size,
                   int32_t *seq_lens_out, int32_t *batch_indices_out, int32_t *positions_out,
                   void *stream);

/* ---- RoPE and append ------------------------------------------------------------- */

/* In-place rotary embedding of q [n,Hq,D] and k [n,Hkv,D] (either may be NULL).
 * Replaces ops.apply_llama31_rope_pos_ids_inplace (llama3.py:660-669) and
 * ops.apply_rope_pos_ids_inplace (qwen3.py:665-670). */
int piekv_rope_inplace(void *q, void *k, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                       int64_t k_stride_h, const int32_t *pos_ids, int32_t nnz, int32_t num_qo_heads,
                       int32_t num_kv_heads, int32_t head_dim, int32_t dtype,
                       const piekv_rope_params *rope, int32_t *err, void *stream);

/* Write k,v [n,Hkv,D] into the pool at page = kv_indices[kv_indptr[b] + pos/page_size],
 * slot pos % page_size.  With rope->mode != NONE, k is rotated on the way (one
 * rounding to the storage type) and, if q != NULL, q is rotated in place; with
 * `rotate_k_in_place` != 0 the rotated k is also stored back over k (so the caller
 * sees what the reference's two separate ops would leave behind).
 * rope == NULL or mode NONE: exactly ops.append_paged_kv_cache (llama3.py:675-685;
 * addressing restated in metal_append_paged_kv_cache.metal:45-105). */
int piekv_rope_append(void *q, void *k, const void *v, int64_t q_stride_n, int64_t q_stride_h,
                      int64_t k_stride_n, int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h,
                      const int32_t *pos_ids, const int32_t *batch_indices, const int32_t *positions,
                      void *pool, const int32_t *kv_indices, const int32_t *kv_indptr,
                      const int32_t *kv_last_page_len, int32_t nnz, int32_t batch,
                      int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim, int32_t page_size,
                      int32_t num_pages, int32_t dtype, const piekv_rope_params *rope,
                      int32_t rotate_k_in_place, int32_t *err, void *stream);

/* The projection in front of the path, fused with it: qkv = x . w_qkv^T for `nnz` token rows
 * (x [nnz, hidden], w_qkv [(Hq + 2 Hkv) * 128, hidden], both row-major 16-bit with row strides in elements),
 * q heads rotated and written to q_out [nnz, Hq, 128] (contiguous), k heads rotated and v heads copied
 * straight into each token's slot of the paged pool; the [nnz, (Hq + 2 Hkv) * 128] projection output never
 * exists in memory, and the fp32 accumulator is rounded once, after the rotation.  head_dim 128, hidden a
 * multiple of 64, pairs (i, i + 64) only.  Stands for the sequence linear -> split -> RoPE -> append of
 * ForwardPass.attention (pie/src/pie_worker/model/llama3.py:627-685) when no adapter edits q / k / v in
 * between. */
int piekv_qkv_rope_append(const void *x, int64_t x_stride_n, const void *w_qkv, int64_t w_stride_n, void *q_out,
                          const int32_t *pos_ids, const int32_t *batch_indices, const int32_t *positions,
                          void *pool, const int32_t *kv_indices, const int32_t *kv_indptr, int32_t nnz,
                          int32_t batch, int32_t hidden, int32_t num_qo_heads, int32_t num_kv_heads,
                          int32_t head_dim, int32_t page_size, int32_t num_pages, int32_t dtype,
                          const piekv_rope_params *rope, int32_t *err, void *stream);

/* Optional terms between the projection and the rotation, as other model families have them: a bias on the
 * whole projection (pie/src/pie_worker/model/qwen2.py:596-603) and a per-head RMSNorm of q and of k with a
 * [128] weight each (qwen3.py:651-662: x * rsqrt(mean(x^2) + eps) * weight over the head's 128 elements), all
 * evaluated on the fp32 accumulator.  NULL pointers switch a term off. */
typedef struct piekv_qkv_options {
  const void *bias;          /* [(Hq + 2 Hkv) * 128], storage type */
  const void *q_norm_weight; /* [128], storage type */
  const void *k_norm_weight; /* [128], storage type */
  float rms_eps;
  int32_t reserved;
} piekv_qkv_options;

int piekv_qkv_rope_append_opt(const void *x, int64_t x_stride_n, const void *w_qkv, int64_t w_stride_n, void *q_out,
                              const int32_t *pos_ids, const int32_t *batch_indices, const int32_t *positions,
                              void *pool, const int32_t *kv_indices, const int32_t *kv_indptr, int32_t nnz,
                              int32_t batch, int32_t hidden, int32_t num_qo_heads, int32_t num_kv_heads,
                              int32_t head_dim, int32_t page_size, int32_t num_pages, int32_t dtype,
                              const piekv_rope_params *rope, int32_t *err, void *stream,
                              const piekv_qkv_options *opt);

/* ---- attention ------------------------------------------------------------------- */

/* Bytes of scratch piekv_decode_run needs at least for `batch` requests (split-KV partials and the
 * counters and tables of its work partition); given more (up to about three times as much) the kernel
 * rebalances more freely between SMs.  The first `piekv_decode_counter_bytes(batch)` bytes hold the
 * counters and tables and must be zero before the first run; runs leave them zero.
 * Reference: the 128 MiB workspace handed to the wrappers (llama3.py:230-232). */
int64_t piekv_decode_workspace_bytes(int32_t batch, int32_t num_qo_heads, int32_t num_kv_heads,
                                     int32_t head_dim);
int64_t piekv_decode_counter_bytes(int32_t batch);

/* out[b,h,:] = softmax(q[b,h,:] . K_b^T * sm_scale) V_b over all cached tokens of request
 * b, kv head = h / (Hq/Hkv).  `lse` (nullable) receives natural-log-sum-exp [batch,Hq] fp32.
 * The work partition is computed on the device from kv_indptr, so there is no host plan
 * step and the call can be captured in a CUDA graph whose index buffers change between
 * replays.  Replaces BatchDecodeWithPagedKVCacheWrapper.plan/run
 * (llama3.py:293-300,766-777,689). */
int piekv_decode_run(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                     void *out, float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                     const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                     int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                     int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes,
                     int32_t *err, void *stream);

/* Same computation as piekv_decode_run for callers that cannot supply scratch memory and must not
 * trigger an allocation: a runtime that has already given every free byte to the KV pool, a
 * binding that can only forward its own tensors, or code running where cudaMalloc is forbidden.
 * It has no counterpart in the reference.  The split-KV scratch is a fixed
 * piekv_decode_noalloc_max_bytes() (8 MiB) array inside the library, held by every GPU that loads
 * the library until the process exits.  Calls whose batch / head count need more are rejected with
 * a >0 status and a message; nothing is launched.  The call never allocates (no cudaMalloc /
 * cudaFree, no allocating library routine); it issues one small cudaMemsetAsync (the counters and
 * tables at the head of the array) and the kernel.  The first call on each device looks the array's device address up
 * (cudaGetSymbolAddress) and should therefore happen before any stream capture.  All calls on a
 * device share the one array: calls that may overlap on the GPU (different streams) race. */
int64_t piekv_decode_noalloc_max_bytes(void);
int piekv_decode_run_noalloc(const void *q, int64_t q_stride_n, int64_t q_stride_h,
                             const void *pool, void *out, float *lse, const int32_t *kv_indptr,
                             const int32_t *kv_indices, const int32_t *kv_last_page_len,
                             int32_t batch, int32_t num_qo_heads, int32_t num_kv_heads,
                             int32_t head_dim, int32_t page_size, int32_t num_pages, int32_t dtype,
                             float sm_scale, int32_t *err, void *stream);

/* One decode step in a single launch: rotate q and the new token's k (RoPE at pos_ids[b]), write
 * k,v into slot kv_last_page_len[b]-1 of request b's last page, and attend over all of the
 * request's pages including the new token.  The page table must already include the new token
 * (the reference grows the page list before the forward pass,
 * sdk/rust/inferlet/src/context.rs:489).  q, k and v are read only: unlike the three separate
 * ops, q and k are NOT rotated in place.  Replaces the op sequence
 * get_seq_lens / get_batch_indices_positions / apply_llama31_rope_pos_ids_inplace /
 * append_paged_kv_cache / BatchDecodeWithPagedKVCacheWrapper.run of one decode layer
 * (llama3.py:745-755,660-689). */
int piekv_decode_step_fused(const void *q, const void *k, const void *v, int64_t q_stride_n,
                            int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                            int64_t v_stride_n, int64_t v_stride_h, const int32_t *pos_ids, void *pool,
                            void *out, float *lse, const int32_t *kv_indptr,
                            const int32_t *kv_indices, const int32_t *kv_last_page_len, int32_t batch,
                            int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim,
                            int32_t page_size, int32_t num_pages, int32_t dtype,
                            const piekv_rope_params *rope, float sm_scale, void *workspace,
                            int64_t workspace_bytes, int32_t *err, void *stream);

/* Bytes of scratch the prefill entry points need for `batch` requests with `nnz` query tokens over
 * a pool of `num_pages` pages; `mask_bytes` = number of entries of the flat boolean mask (0: none). */
int64_t piekv_prefill_workspace_bytes(int32_t batch, int32_t nnz, int32_t num_qo_heads,
                                      int32_t head_dim, int32_t num_pages, int64_t mask_bytes);

/* Once per batch (stream-ordered, no host synchronisation): builds in the workspace the work
 * list of query tiles and, for a custom mask, its bit-packed form with a per-tile "any allowed"
 * summary, so that the per-layer runs read 1 bit per pair instead of 1 byte and skip kv tiles no
 * query of the tile may see.  Replaces BatchPrefillWithPagedKVCacheWrapper.plan
 * (llama3.py:779-791), which the reference calls once per step before the layer loop. */
int piekv_prefill_plan(const int32_t *qo_indptr, const int32_t *kv_indptr,
                       const int32_t *kv_last_page_len, const uint8_t *custom_mask,
                       int64_t mask_bytes, int32_t causal, int32_t batch, int32_t nnz,
                       int32_t page_size, int32_t num_pages, void *workspace,
                       int64_t workspace_bytes, int32_t *err, void *stream);

/* The same plan built from the wire form of the mask: per query token a list of run lengths that
 * alternate attend / skip starting with attend (BRLE, sdk/rust/inferlet/src/brle.rs:4-21), runs of
 * token i at brle_runs[brle_indptr[i] .. brle_indptr[i+1]), and only the first position + 1 entries
 * of a row can be set (position = kv_len_b - qo_len_b + index of the token in its request).  The
 * bit-packed mask is produced on the device, so neither the host expansion to one byte per pair
 * nor its upload happens.  `mask_bits` = sum over requests of qo_len_b * kv_len_b (sizes the
 * packed mask; the same number piekv_prefill_workspace_bytes takes as mask_bytes).  Run the batch
 * with piekv_prefill_run(custom_mask = NULL, mask_bytes = mask_bits, planned = 2).  Needs the
 * tensor-core path (fp16 / bf16, head_dim 128, page size 16).
 * Replaces Batch.__init__'s decode_brle_batch (pie/src/pie_worker/batching.py:113-135,337-389)
 * followed by the `custom_mask` upload (batching.py:196-239). */
int piekv_prefill_plan_brle(const int32_t *qo_indptr, const int32_t *kv_indptr,
                            const int32_t *kv_last_page_len, const uint32_t *brle_runs,
                            const int32_t *brle_indptr, int64_t mask_bits, int32_t batch,
                            int32_t nnz, int32_t page_size, int32_t num_pages, void *workspace,
                            int64_t workspace_bytes, int32_t *err, void *stream);

/* Packed variable-length attention over paged K/V: query token j of request b (rows
 * qo_indptr[b]..qo_indptr[b+1]) attends to cached token t of that request when
 *   custom_mask != NULL:  custom_mask[off_b + j*kv_len_b + t] != 0,
 *                         off_b = sum_{b'<b} qo_len_b' * kv_len_b'
 *                         (flat bool layout of pie/src/pie_worker/batching.py:113-135);
 *   otherwise:            !causal || t <= kv_len_b - qo_len_b + j.
 * `planned` 1: piekv_prefill_plan was already called on this workspace with the same metadata
 * and mask (one plan, many layers); 2: piekv_prefill_plan_brle was (the mask lives in the
 * workspace only; custom_mask is ignored); 0: the plan is built inside this call.
 * Replaces BatchPrefillWithPagedKVCacheWrapper.run (llama3.py:307-309,689). */
int piekv_prefill_run(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                      void *out, float *lse, const int32_t *qo_indptr, const int32_t *kv_indptr,
                      const int32_t *kv_indices, const int32_t *kv_last_page_len,
                      const uint8_t *custom_mask, int64_t mask_bytes, int32_t causal,
                      int32_t planned, int32_t batch, int32_t nnz, int32_t num_qo_heads,
                      int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                      int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes,
                      int32_t *err, void *stream);

/* ---- the wire form of a batch, decoded on the device ------------------------------------------------
 *
 * The reference's runtime sends a step's metadata as little-endian uint32 arrays
 * (BatchedForwardPassRequest, runtime/src/model/request.rs:250-298); its worker decodes them with numpy,
 * derives per-token arrays, expands the run-length masks on the CPU and uploads each array
 * (pie/src/pie_worker/batching.py:28-135,196-239).  With these entry points the arrays are uploaded as
 * they arrive - concatenated in ONE device buffer `wire`, each field at the word offset `piekv_wire_batch`
 * names - and the per-token work happens on the device.  The index arrays are used in place:
 * `(const int32_t *)(wire + layout.kv_page_indptr)` etc. are what the attention entry points take, and
 * (wire + flattened_masks, wire + mask_indptr) is the `brle_runs` / `brle_indptr` pair of
 * piekv_prefill_plan_opt. */
typedef struct piekv_wire_batch {
  int64_t token_ids, position_ids, kv_page_indices, kv_page_indptr, kv_last_page_lens, qo_indptr,
      flattened_masks, mask_indptr; /* offsets of the fields in `wire`, in 32-bit words            */
  int32_t nnz;                      /* tokens: entries of token_ids / position_ids                 */
  int32_t batch;                    /* requests: kv_page_indptr and qo_indptr hold batch + 1 words  */
  int32_t total_pages;              /* entries of kv_page_indices                                   */
  int32_t num_runs;                 /* entries of flattened_masks; mask_indptr holds nnz + 1 words  */
} piekv_wire_batch;

/* Outputs (each nullable): token_ids_out int64 [nnz] (batching.py:206-208); seq_lens_out [batch];
 * batch_indices_out / positions_out [nnz] (both or neither) - request and kv position of every token,
 * the latter also being the position the reference derives for the mask rows (batching.py:113-122);
 * token_acc_seq_lens_out int64 [nnz + 1], the reference's per-token offsets into the flat mask
 * (batching.py:124-126; at most 4096 requests).  `lay` is a host struct. */
int piekv_batch_from_wire(const uint32_t *wire, const piekv_wire_batch *lay, int32_t page_size,
                          int64_t *token_ids_out, int32_t *seq_lens_out, int32_t *batch_indices_out,
                          int32_t *positions_out, int64_t *token_acc_seq_lens_out, void *stream);

/* The mask a prefill plan holds in `workspace` (built from bytes, run lengths and / or a window) written
 * out in the reference's flat form: one byte per (query, key) pair, rows of kv_len_b entries, requests
 * end to end (`custom_mask` of batching.py:113-135,228-230).  For callers that still want that tensor,
 * and for checking the device-built mask against the reference's.  `mask_entries` as given to the plan. */
int piekv_prefill_export_mask(const int32_t *qo_indptr, const int32_t *kv_indptr,
                              const int32_t *kv_last_page_len, int64_t mask_entries, int32_t batch,
                              int32_t nnz, int32_t page_size, int32_t num_pages, const void *workspace,
                              int64_t workspace_bytes, uint8_t *flat_out, void *stream);

/* ---- sliding window and attention sinks ----------------------------------------------------------
 *
 * Other model families of the reference plan their wrappers with `window_left` (a different one per
 * layer: pie/src/pie_worker/model/olmo3.py:976-1013, decode and prefill, the prefill together with
 * `custom_mask`) or run a wrapper that takes per-head attention sinks
 * (BatchAttentionWithAttentionSinkWrapper.run(q, kv, sinks, scaling),
 * pie/src/pie_worker/model/gpt_oss.py:418-439,693-697,840-870).  The `_opt` entry points are the plain
 * ones with this block appended; `opt == NULL` is exactly the plain call.
 *
 *   window_left  -1: none.  >= 0: the query at kv position p (= kv_len - qo_len + index of the query in
 *                its request; for decode p = kv_len - 1) sees keys p - window_left .. only, on top of
 *                whatever the causal flag or the mask allows.  The decode kernel then streams only the
 *                pages that hold such keys.
 *   sinks        nullable device fp32 [num_qo_heads]: softmax is taken over the scaled scores AND the
 *                head's sink logit (not scaled); the sink has no value row, so it only takes
 *                probability mass: out = sum_t exp(s_t) v_t / (sum_t exp(s_t) + exp(sink_h)).
 *                `lse` then includes the sink term.  A query without any visible key gives zeros. */
typedef struct piekv_attn_options {
  int32_t window_left;
  int32_t reserved; /* 0 */
  const float *sinks;
} piekv_attn_options;

int piekv_decode_run_opt(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                         void *out, float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                         const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                         int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                         int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes,
                         int32_t *err, void *stream, const piekv_attn_options *opt);

int piekv_decode_step_fused_opt(const void *q, const void *k, const void *v, int64_t q_stride_n,
                                int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                                int64_t v_stride_n, int64_t v_stride_h, const int32_t *pos_ids, void *pool,
                                void *out, float *lse, const int32_t *kv_indptr,
                                const int32_t *kv_indices, const int32_t *kv_last_page_len, int32_t batch,
                                int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim,
                                int32_t page_size, int32_t num_pages, int32_t dtype,
                                const piekv_rope_params *rope, float sm_scale, void *workspace,
                                int64_t workspace_bytes, int32_t *err, void *stream,
                                const piekv_attn_options *opt);

/* piekv_prefill_plan and piekv_prefill_plan_brle in one call, plus the window: the mask comes as bytes
 * (`custom_mask`), as run lengths (`brle_runs` / `brle_indptr`) or not at all, and `window_left` >= 0 is
 * ANDed into it on the device; a window without a mask is turned into one (causal or not, as `causal`
 * says).  `mask_entries` = sum over requests of qo_len_b * kv_len_b whenever a mask or a window is
 * given (it sizes the packed mask; also the `mask_bytes` of piekv_prefill_workspace_bytes and of the
 * run call).  Run with piekv_prefill_run_opt(planned = 2 for run lengths, else 1) and the same window. */
int piekv_prefill_plan_opt(const int32_t *qo_indptr, const int32_t *kv_indptr,
                           const int32_t *kv_last_page_len, const uint8_t *custom_mask,
                           const uint32_t *brle_runs, const int32_t *brle_indptr, int64_t mask_entries,
                           int32_t causal, int32_t window_left, int32_t batch, int32_t nnz,
                           int32_t page_size, int32_t num_pages, void *workspace, int64_t workspace_bytes,
                           int32_t *err, void *stream);

int piekv_prefill_run_opt(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                          void *out, float *lse, const int32_t *qo_indptr, const int32_t *kv_indptr,
                          const int32_t *kv_indices, const int32_t *kv_last_page_len,
                          const uint8_t *custom_mask, int64_t mask_bytes, int32_t causal,
                          int32_t planned, int32_t batch, int32_t nnz, int32_t num_qo_heads,
                          int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                          int32_t dtype, float sm_scale, void *workspace, int64_t workspace_bytes,
                          int32_t *err, void *stream, const piekv_attn_options *opt);

/* ---- head-sharded decode over the GPUs of one node: results stored straight to every GPU ----
 *
 * The reference's tensor parallelism (llama3.py:607-610,963-965) gives every GPU Hkv/G kv heads and
 * their query heads with identical page tables, and joins the GPUs with an NCCL collective per
 * layer (all_reduce after o_proj, llama3.py:705-706).  On a path that ends at the attention output
 * the join is an all-gather of [batch, Hq/G * D] slices.  These entry points remove the separate
 * collective: the decode kernel stores its slice into the output buffer of every GPU over NVLink
 * (plain peer stores from the same kernel that computes the rows) and, when its last row is out,
 * raises this GPU's flag on every GPU; a consumer waits for all G flags (bounded) and reads the full
 * rows locally.  One process per GPU; buffers are cudaMalloc'd here and mapped into the other
 * processes with CUDA IPC handles that the host exchanges (e.g. torch.distributed
 * all_gather_object).  No counterpart in the reference. */
#define PIEKV_MAX_PEERS 8
#define PIEKV_PEER_HANDLE_BYTES 64

/* cudaMalloc `bytes` (zero-filled) on the current device and export its IPC handle (64 bytes). */
int piekv_peer_alloc(int64_t bytes, void **ptr, void *handle);
/* Map another process's buffer (handle from its piekv_peer_alloc); enables peer access lazily. */
int piekv_peer_open(const void *handle, void **ptr);
int piekv_peer_close(void *ptr); /* unmap a pointer from piekv_peer_open   */
int piekv_peer_free(void *ptr);  /* free a pointer from piekv_peer_alloc    */

typedef struct piekv_peer_outputs {
  void *out[PIEKV_MAX_PEERS];      /* out[r]: this step's output rows [batch, row_heads, head_dim] on rank r */
  int32_t *flags[PIEKV_MAX_PEERS]; /* flags[r]: int32[world] on rank r; word i is raised by rank i           */
  int32_t world, rank;
  int32_t row_heads;               /* query heads per output row (>= world * num_qo_heads of the call)       */
  int32_t step;                    /* published in the flags; must grow from call to call                     */
  /* Graph replays: when step_counter is not NULL the kernel reads the step number from that device
   * word instead of `step`, and stores to out[r] on odd and out_alt[r] on even step numbers;
   * piekv_peer_wait_counted increments the word when the step is complete.  Start it at 1. */
  const int32_t *step_counter;
  void *out_alt[PIEKV_MAX_PEERS];
} piekv_peer_outputs;

/* piekv_decode_step_fused with the results of this rank's heads written to columns
 * [rank * num_qo_heads, (rank + 1) * num_qo_heads) of out[r] for every r, then flags[r][rank] = step.
 * Use two alternating output buffers: a rank may start step s + 1 while another still reads step s.
 * batch == 0 launches nothing and raises no flag: do not consume a step number or wait for it. */
int piekv_decode_step_fused_peer(const void *q, const void *k, const void *v, int64_t q_stride_n,
                                 int64_t q_stride_h, int64_t k_stride_n, int64_t k_stride_h,
                                 int64_t v_stride_n, int64_t v_stride_h, const int32_t *pos_ids,
                                 void *pool, const piekv_peer_outputs *peers,
                                 const int32_t *kv_indptr, const int32_t *kv_indices,
                                 const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t page_size,
                                 int32_t num_pages, int32_t dtype, const piekv_rope_params *rope,
                                 float sm_scale, void *workspace, int64_t workspace_bytes, int32_t *err,
                                 void *stream);

/* Stream-ordered wait until flags[0..world) (this rank's own flag array) have all reached `step`;
 * gives up after 2 s with PIEKV_ERR_WAIT_TIMEOUT in the error word.  Work queued behind it on the
 * stream sees every rank's rows of that step. */
int piekv_peer_wait(const int32_t *flags, int32_t world, int32_t step, int32_t *err, void *stream);
/* The same wait with the step number taken from the device word `step_counter`, which is incremented
 * afterwards: [piekv_decode_step_fused_peer with step_counter, piekv_peer_wait_counted] can be captured
 * in a CUDA graph once and replayed for every step. */
int piekv_peer_wait_counted(const int32_t *flags, int32_t world, int32_t *step_counter, int32_t *err,
                            void *stream);

/* ---- output projection with the sum over the ranks in its epilogue ---------------------------------
 *
 * Replaces, for a head-sharded (tensor-parallel) layer, the three steps after the attention in
 * pie/src/pie_worker/model/llama3.py:693-709: the row-parallel o_proj on the local shard
 * (fun.linear(attn_output, proj_o)), dist.all_reduce of the partial result, and residual + attn_proj.
 * One launch per rank and step; the partial sums travel as fp32 over NVLink (plain peer stores) and
 * the result is rounded once.  Every rank gets the same bits.
 *
 * Buffers of all ranks are mapped into every process (piekv_peer_alloc / piekv_peer_open):
 *   out[r]     the result rows [n, hidden] (row stride `hidden`) on rank r.  Alternate between two
 *              buffers from step to step: a rank may run one step ahead of a rank that still reads.
 *   stage[r]   staging for the partial sums of the tiles rank r owns; stage_bytes each
 *   arrive[r]  int32[arrive_words], done[r] int32[done_words] flag words on rank r, zero at the start
 * Sizes for n <= n_max from piekv_oproj_allreduce_sizes: sizes[0] staging bytes, [1] arrival words,
 * [2] completion words.  `step` must grow by one from call to call (start at 1) and be the same on
 * every rank, as must n, k_local and hidden.  world == 1 needs only out[0].
 * A rank that waits 2 s for another gives up with PIEKV_ERR_WAIT_TIMEOUT in the error word. */
/* flags: the partial sums cross NVLink rounded to the 16-bit storage type (what an all-reduce of 16-bit
 * tensors does) instead of fp32: half the bytes, for large n where the link is the limit. */
#define PIEKV_REDUCE_PARTIALS_16BIT 1
typedef struct piekv_peer_reduce {
  void *out[PIEKV_MAX_PEERS];
  void *stage[PIEKV_MAX_PEERS];
  int32_t *arrive[PIEKV_MAX_PEERS];
  int32_t *done[PIEKV_MAX_PEERS];
  int64_t stage_bytes, arrive_words, done_words;
  int32_t world, rank;
  int32_t step;
  int32_t flags; /* PIEKV_REDUCE_* bits; the same on every rank */
} piekv_peer_reduce;

int piekv_oproj_allreduce_sizes(int32_t n_max, int32_t hidden, int32_t world, int64_t *sizes);
/* Hidden columns per tile (256, 128 or 64) that piekv_oproj_allreduce uses for n rows; 0 for sizes it
 * rejects.  Tiles are 128 rows high, numbered row tile * (hidden / cols) + column tile; tile t belongs to
 * rank t % world and is staged in slot t / world of its owner.  For tools that inspect the staging. */
int32_t piekv_oproj_tile_cols(int32_t n, int32_t hidden);

/* out[r][i, :] = residual[i, :] + sum over ranks of a[i, :k_local] . w_o[:, :k_local]^T for every r.
 * a: [n, k_local] this rank's attention rows (k_local = local heads x head_dim, a multiple of 64);
 * w_o: [hidden, k_local] this rank's columns of the projection weight (rows = output features, as
 * torch.nn.functional.linear takes it); residual: NULL or [n, hidden], the same values on every rank;
 * hidden a multiple of 64; 16-bit types; strides in elements.  n == 0 launches nothing: do not consume a
 * step number for it. */
int piekv_oproj_allreduce(const void *a, int64_t a_stride_n, const void *w_o, int64_t w_stride_n,
                          const void *residual, int64_t residual_stride_n, int32_t n, int32_t k_local,
                          int32_t hidden, int32_t dtype, const piekv_peer_reduce *peers, int32_t *err,
                          void *stream);

/* sizeof of the structs that cross this boundary, for bindings to check their mirrors against:
 * which = 0: piekv_rope_params, 1: piekv_peer_outputs, 2: piekv_attn_options, 3: piekv_wire_batch,
 * 4: piekv_qkv_options, 5: piekv_peer_reduce; anything else: -1. */
int32_t piekv_abi_sizeof(int32_t which);

/* ---- page copy (fork with copy-on-write of a partial page) ----------------------- */

/* For every pair j and every layer l: pool_l[dst[j], :, :valid_j] = pool_l[src[j], :, :valid_j]
 * (valid_len == NULL copies whole pages).  `pools` is a HOST array of `num_layers` device
 * pointers.  The reference never copies a page: Context::fork drops the partial last page
 * and recomputes it (sdk/rust/inferlet/src/context.rs:147-225); this entry point is the
 * copy-on-write that replaces that recomputation. */
int piekv_copy_pages(void *const *pools, int32_t num_layers, const int32_t *src_pages,
                     const int32_t *dst_pages, const int32_t *valid_len, int32_t count,
                     int32_t page_size, int32_t num_kv_heads, int32_t head_dim, int32_t num_pages,
                     int32_t dtype, int32_t *err, void *stream);

/* ---- page tables, reference counts and the free list on the device -------------------------------
 *
 * The reference keeps page ownership on the host: an id pool that hands out the smallest free id
 * (runtime/src/utils.rs:42-158), contexts that grow by whole pages as tokens arrive (adjust_kv_pages,
 * sdk/rust/inferlet/src/context.rs:356-399), forks that share full pages (context.rs:147-225) and pages
 * that return to the pool with their last holder (sdk/rust/inferlet/src/forward.rs:28-55); every step
 * the page tables are rebuilt and uploaded (pie/src/pie_worker/batching.py:196-239).  These entry points
 * keep the same bookkeeping in device memory, advanced by small stream-ordered kernels, so a decode loop
 * or a beam search runs (and can be captured in a CUDA graph) without host page tables.
 *
 * `state` is a caller-owned device buffer of piekv_pagestate_bytes() bytes holding, for `max_requests`
 * request slots of up to `pages_per_request` pages each: page rows, page counts, last-page fill, one
 * reference count per physical page and the free bitmap.  The four size arguments must be the same in
 * every call on one state.  Slot lists are DEVICE int32 arrays; a slot appears at most once per call.
 * Requests are served in list order and the i-th page a call needs is the i-th smallest free id - what
 * a host loop over the same list does with the reference's id pool.  Problems (no free page, a row
 * that is full, a bad slot) are reported through the error word and the call changes nothing further.
 * No counterpart in the reference as device code. */
int64_t piekv_pagestate_bytes(int32_t num_pages, int32_t max_requests, int32_t pages_per_request);
/* every page free, every slot empty */
int piekv_pagestate_init(void *state, int64_t state_bytes, int32_t num_pages, int32_t max_requests,
                         int32_t pages_per_request, int32_t page_size, void *stream);
/* Grow (delta > 0) or shrink (delta < 0) the listed requests by deltas[i] tokens, or by delta_all when
 * deltas == NULL (a decode step: 1); shrinks release their pages before any page is handed out.
 * At most 1024 requests and 4096 new pages per call.  Optional outputs (NULL: skip), the CSR page table
 * of exactly this batch as the attention entry points take it: kv_indptr [count + 1], kv_indices
 * [kv_indptr[count]], kv_last_page_len [count], and pos_ids [count] = tokens held before the call
 * (the RoPE position of the first new token). */
int piekv_pagestate_adjust(void *state, int32_t num_pages, int32_t max_requests, int32_t pages_per_request,
                           int32_t page_size, const int32_t *slots, const int32_t *deltas,
                           int32_t delta_all, int32_t count, int32_t *kv_indptr, int32_t *kv_indices,
                           int32_t *kv_last_page_len, int32_t *pos_ids, int32_t *err, void *stream);
/* The listed requests let go of all their pages; pages without a holder return to the free list. */
int piekv_pagestate_release(void *state, int32_t num_pages, int32_t max_requests, int32_t pages_per_request,
                            int32_t page_size, const int32_t *slots, int32_t count, int32_t *err,
                            void *stream);
/* children[i] (an empty slot, not a parent of this call) becomes a copy-on-write fork of parents[i]:
 * full pages shared by reference count, a partly filled last page replaced by a fresh page.  Outputs
 * (device, [count]): the page copies that complete the forks, to be passed to piekv_copy_pages with the
 * same `count` (entries with nothing to copy have valid 0 and src == dst).  At most 1024 forks per call. */
int piekv_pagestate_fork(void *state, int32_t num_pages, int32_t max_requests, int32_t pages_per_request,
                         int32_t page_size, const int32_t *parents, const int32_t *children, int32_t count,
                         int32_t *copy_src, int32_t *copy_dst, int32_t *copy_valid, int32_t *err,
                         void *stream);

/* ---- page bookkeeping on the host (no GPU work) ---------------------------------------------
 *
 * Native counterpart of the reference's id pool (runtime/src/utils.rs:42-158: smallest free id
 * first, tail compaction above 1000 free ids) and of its resource manager for KV pages of one
 * device group (runtime/src/model/resource.rs:62-463): instances own pages; an allocation that
 * does not fit terminates instances that started after the requester, newest first, and fails
 * with PIEKV_STATUS_OUT_OF_PAGES if that is not enough; export moves pages to a name, import
 * reads them, release_exported frees them.  Reference counts (piekv_pages_share) are an addition
 * for forked contexts that keep full pages in common: a page returns to the pool when its last
 * holder lets go.  Calls return 0, 1 (invalid argument, see piekv_last_error_string) or
 * PIEKV_STATUS_OUT_OF_PAGES.  One manager per pool, driven from one thread. */
#define PIEKV_STATUS_OUT_OF_PAGES 8
typedef struct piekv_page_manager piekv_page_manager;
piekv_page_manager *piekv_pages_create(int32_t num_pages);
void piekv_pages_destroy(piekv_page_manager *m);
int32_t piekv_pages_available(const piekv_page_manager *m);
int32_t piekv_pages_refcount(const piekv_page_manager *m, int32_t page);   /* -1: no such page */
int32_t piekv_pages_owned(const piekv_page_manager *m, uint64_t instance); /* pages the instance holds */
/* `count` pages for `instance` (allocate_with_oom, resource.rs:112-175); the instances terminated
 * to make room are reported by piekv_pages_last_victims. */
int piekv_pages_alloc(piekv_page_manager *m, uint64_t instance, int32_t count, int32_t *out);
int32_t piekv_pages_last_victims(const piekv_page_manager *m, uint64_t *out, int32_t max_count);
/* deallocate (resource.rs:225-254): pages the instance does not hold are skipped */
int piekv_pages_free(piekv_page_manager *m, uint64_t instance, const int32_t *pages, int32_t count);
/* the instance becomes a co-holder of pages that are already allocated (fork of full pages) */
int piekv_pages_share(piekv_page_manager *m, uint64_t instance, const int32_t *pages, int32_t count);
/* everything the instance holds (cleanup, resource.rs:321-354) */
int piekv_pages_cleanup(piekv_page_manager *m, uint64_t instance);
int piekv_pages_export(piekv_page_manager *m, uint64_t instance, const int32_t *pages, int32_t count,
                       const char *name);
/* number of pages under `name` (-1: not found); up to max_count ids are written to `out` */
int32_t piekv_pages_import(const piekv_page_manager *m, const char *name, int32_t *out, int32_t max_count);
int piekv_pages_release_exported(piekv_page_manager *m, const char *name);

#ifdef __cplusplus
}
#endif
#endif /* PIEKV_H_ */
