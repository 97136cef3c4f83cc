// Wire form of a batched forward pass -> device metadata.
//
// The reference ships a step's metadata from its Rust runtime to the Python worker as little-endian
// uint32 arrays (BatchedForwardPassRequest, runtime/src/model/request.rs:250-298: token_ids,
// position_ids, kv_page_indices, kv_page_indptr, kv_last_page_lens, qo_indptr, flattened_masks,
// mask_indptr).  The worker decodes them with numpy, derives per-request sequence lengths, per-token
// positions and mask bit offsets, expands the run-length masks with a Numba loop and uploads every
// array separately (pie/src/pie_worker/batching.py:28-135,196-239).
//
// Here the byte strings are uploaded as they are (one buffer, one copy) and everything per token or
// per (query, key) pair is derived on the device.  The index arrays need no conversion at all: the
// attention entry points read them in place (uint32 values below 2^31 are the same bits as int32).
#include "attn.cuh"
#include "common.cuh"

namespace piekv {
namespace {

constexpr int kWireMaxBatch = 4096;

// token ids widened to int64 (the embedding lookup of the reference takes torch.long,
// batching.py:206-208) and, optionally, the reference's per-token bit offsets into the flat mask
// (token_acc_seq_lens, batching.py:124-126): offset of request b + j * kv_len_b.  One block.
__global__ void __launch_bounds__(1024)
    wire_derive_kernel(const uint32_t *__restrict__ token_ids, const int32_t *__restrict__ qo_indptr,
                       const int32_t *__restrict__ kv_indptr, const int32_t *__restrict__ last, int batch, int nnz,
                       int page_size, int64_t *token_ids_out, int64_t *token_acc_seq_lens) {
  __shared__ long long req_off[kWireMaxBatch + 1];
  __shared__ long long sh[33];
  __shared__ long long carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (token_ids_out != nullptr)
    for (int i = threadIdx.x; i < nnz; i += blockDim.x) token_ids_out[i] = (int64_t)token_ids[i];
  if (token_acc_seq_lens == nullptr) return;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < batch; base += 1024) {
    const int b = base + threadIdx.x;
    long long v = 0;
    if (b < batch) {
      const long long np = kv_indptr[b + 1] - kv_indptr[b];
      const long long kv = (np > 0 ? (np - 1) * page_size : 0) + last[b];
      v = kv * (qo_indptr[b + 1] - qo_indptr[b]);
    }
    long long x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const long long y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) sh[warp] = x;
    __syncthreads();
    if (warp == 0) {
      long long w = sh[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const long long y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      sh[lane] = w;
    }
    __syncthreads();
    const long long excl = carry + (warp > 0 ? sh[warp - 1] : 0) + x - v;
    if (b < batch) req_off[b] = excl;
    __syncthreads();
    if (threadIdx.x == 1023) carry = excl + v;
    __syncthreads();
  }
  if (threadIdx.x == 0) req_off[batch] = carry;
  __syncthreads();
  for (int i = threadIdx.x; i <= nnz; i += blockDim.x) {
    if (i == nnz) {
      token_acc_seq_lens[i] = req_off[batch];
      break;
    }
    int lo = 0, hi = batch;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (qo_indptr[mid + 1] > i)
        hi = mid;
      else
        lo = mid + 1;
    }
    const int b = lo < batch ? lo : batch - 1;
    const long long np = kv_indptr[b + 1] - kv_indptr[b];
    const long long kv = (np > 0 ? (np - 1) * page_size : 0) + last[b];
    token_acc_seq_lens[i] = req_off[b] + (long long)(i - qo_indptr[b]) * kv;
  }
}

}  // namespace
}  // namespace piekv

using namespace piekv;

extern "C" int piekv_batch_from_wire(const uint32_t *wire, const piekv_wire_batch *lay, int32_t page_size,
                                     int64_t *token_ids_out, int32_t *seq_lens_out, int32_t *batch_indices_out,
                                     int32_t *positions_out, int64_t *token_acc_seq_lens_out, void *stream) {
  PIEKV_REQUIRE(wire != nullptr && lay != nullptr, "batch_from_wire: null pointer");
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(wire) & 3) == 0, "batch_from_wire: wire buffer not 4-byte aligned");
  PIEKV_REQUIRE(lay->batch >= 0 && lay->nnz >= 0 && page_size > 0, "batch_from_wire: bad sizes");
  PIEKV_REQUIRE(token_acc_seq_lens_out == nullptr || lay->batch <= kWireMaxBatch,
                "batch_from_wire: %d requests (token_acc_seq_lens is built for at most %d)", lay->batch, kWireMaxBatch);
  const int64_t offs[8] = {lay->token_ids, lay->position_ids, lay->kv_page_indices, lay->kv_page_indptr,
                           lay->kv_last_page_lens, lay->qo_indptr, lay->flattened_masks, lay->mask_indptr};
  for (int i = 0; i < 8; ++i) PIEKV_REQUIRE(offs[i] >= 0, "batch_from_wire: negative offset of field %d", i);
  if (lay->batch == 0) return 0;
  const int32_t *qo = reinterpret_cast<const int32_t *>(wire + lay->qo_indptr);
  const int32_t *kvp = reinterpret_cast<const int32_t *>(wire + lay->kv_page_indptr);
  const int32_t *last = reinterpret_cast<const int32_t *>(wire + lay->kv_last_page_lens);
  PIEKV_REQUIRE((batch_indices_out == nullptr) == (positions_out == nullptr),
                "batch_from_wire: batch_indices and positions go together");
  if (batch_indices_out != nullptr) {
    if (int rc = piekv_metadata(qo, kvp, last, lay->batch, lay->nnz, page_size, seq_lens_out, batch_indices_out,
                                positions_out, stream))
      return rc;
  } else if (seq_lens_out != nullptr) {
    if (int rc = piekv_get_seq_lens(kvp, last, lay->batch, page_size, seq_lens_out, stream)) return rc;
  }
  if (token_ids_out != nullptr || token_acc_seq_lens_out != nullptr) {
    wire_derive_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(wire + lay->token_ids, qo, kvp, last, lay->batch, lay->nnz,
                                                             page_size, token_ids_out, token_acc_seq_lens_out);
    PIEKV_LAUNCH_CHECK("wire_derive_kernel");
  }
  return 0;
}

extern "C" int piekv_prefill_export_mask(const int32_t *qo_indptr, const int32_t *kv_indptr,
                                         const int32_t *kv_last_page_len, int64_t mask_entries, int32_t batch,
                                         int32_t nnz, int32_t page_size, int32_t num_pages, const void *workspace,
                                         int64_t workspace_bytes, uint8_t *flat_out, void *stream) {
  PIEKV_REQUIRE(batch >= 0 && nnz >= 0 && page_size == 16 && num_pages > 0 && mask_entries >= 0,
                "prefill_export_mask: bad sizes (the packed mask exists for page size 16 only)");
  PIEKV_REQUIRE(nnz == 0 || (qo_indptr && kv_indptr && kv_last_page_len && flat_out), "prefill_export_mask: null pointer");
  AttnArgs a{};
  a.qo_indptr = qo_indptr;
  a.kv_indptr = kv_indptr;
  a.kv_last_page_len = kv_last_page_len;
  a.batch = batch;
  a.nnz = nnz;
  a.page_size = page_size;
  a.num_pages = num_pages;
  return launch_prefill_export_mask(a, mask_entries, const_cast<void *>(workspace), workspace_bytes, flat_out,
                                    (cudaStream_t)stream);
}
