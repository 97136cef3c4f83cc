// Argument block shared by the attention kernels and their launchers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace piekv {

struct AttnArgs {
  const void *q;  // [nnz, Hq, D], strides q_sn / q_sh (elements)
  int64_t q_sn, q_sh;
  const void *pool;            // [num_pages, 2, page_size, Hkv, D]
  void *out;                   // [nnz, Hq, D] contiguous
  float *lse;                  // nullable [nnz, Hq]
  const int32_t *qo_indptr;    // nullable: decode (one row per request)
  const int32_t *kv_indptr;    // [batch+1]
  const int32_t *kv_indices;   // [kv_indptr[batch]]
  const int32_t *kv_last_page_len;  // [batch]
  const uint8_t *mask;         // nullable flat bool mask
  int causal;
  int batch, nnz, hq, hkv, dim, page_size, num_pages;
  float sm_scale;
  int32_t *err;
  // Sliding window: the query at kv position p (= kv_len - qo_len + row index) sees keys p - window_left .. ;
  // -1: no window.  The decode and generic kernels apply it themselves; the tensor-core prefill kernels
  // get it through the packed mask their plan builds.
  int window_left = -1;
  // Attention sinks: nullable fp32 [Hq].  The head's sink logit joins the softmax normaliser (it takes
  // probability mass) but has no value row.
  const float *sinks = nullptr;
};

// Destinations of a head-sharded decode step on several GPUs: the same output buffer on every GPU
// (own GPU included), mapped into this process; `flag[d]` is this GPU's word in GPU d's flag array.
struct PeerOut {
  void *dst[8];
  void *dst_alt[8];     // used for even step numbers when the step is read from `step_ptr`
  const int *step_ptr;  // nullable: device word holding the step number (graph replays), else `step`
  int *flag[8];
  int n;          // 0: not used
  int row_heads;  // query heads per output row at the destinations (all GPUs' heads)
  int head_off;   // first head of this GPU inside a row
  int step;       // value published in the flags when every result of the launch has been stored
  int *done;      // device counter, zero between launches
};

// any dtype / shape
int launch_attn_generic(const AttnArgs &a, int dtype, cudaStream_t st);

// tuned decode (16-bit, D=128, page 16): returns 0 on launch, >0 / <0 on error
bool decode_tma_supported(const AttnArgs &a, int dtype);
int launch_decode_tma(const AttnArgs &a, int dtype, void *workspace, int64_t workspace_bytes, cudaStream_t st);

// tuned prefill (tcgen05): 16-bit, D=128, page 16.  plan builds the work list (and packs a custom
// mask) into the workspace; launch_prefill_tc consumes that plan.
bool prefill_tc_supported(const AttnArgs &a, int dtype);
int64_t prefill_tc_workspace_bytes(int batch, int nnz, int num_pages, int64_t mask_bytes);
// brle_runs / brle_indptr (both or neither): build the packed mask from per-token run lengths
// instead of a.mask
// a.window_left >= 0 is ANDed into whichever mask form is given; without any mask it becomes one
// (mask_bytes must then still name sum qo_len * kv_len, which sizes the packed mask)
int launch_prefill_plan(const AttnArgs &a, int64_t mask_bytes, void *workspace, int64_t workspace_bytes,
                        cudaStream_t st, const uint32_t *brle_runs = nullptr, const int32_t *brle_indptr = nullptr);
// the planned packed mask written out as one byte per (query, key) pair (the reference's flat layout)
int launch_prefill_export_mask(const AttnArgs &a, int64_t mask_bytes, void *workspace, int64_t workspace_bytes,
                               uint8_t *flat, cudaStream_t st);
int launch_prefill_tc(const AttnArgs &a, int dtype, int64_t mask_bytes, void *workspace, int64_t workspace_bytes,
                      cudaStream_t st);

}  // namespace piekv
