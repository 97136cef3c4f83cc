// Rotary-embedding parameters as the kernels receive them.
#pragma once
#include "common.cuh"

namespace piekv {

constexpr int kMaxHalfDim = 128;  // head_dim <= 256

struct RopeDev {
  int mode;
  int interleave;
  int table_len;
  const float *table;           // [table_len, D]: cos | sin
  float inv_freq[kMaxHalfDim];  // final per-pair frequency (plain or Llama-3.1 scaled), fp32
};

// Per-pair frequencies evaluated in double and rounded once to fp32 (host).
void fill_inv_freq(const piekv_rope_params *rope, int head_dim, RopeDev *out);
// Host-side validation shared by the entry points; 0 or a >0 status with the error text set.
int check_rope(const piekv_rope_params *rope, int head_dim, const char *who);

// cos / sin of pair `pair` at position `pos` (device).
__device__ __forceinline__ void rope_cos_sin1(const RopeDev &rp, int pos, int pair, int half_dim, float &c, float &s) {
  if (rp.mode == PIEKV_ROPE_TABLE) {
    const float *row = rp.table + (size_t)pos * (2 * half_dim);
    c = __ldg(row + pair);
    s = __ldg(row + half_dim + pair);
  } else {
    sincosf(__fmul_rn((float)pos, rp.inv_freq[pair]), &s, &c);
  }
}

// x' = x*c - y*s ; y' = x*s + y*c with separately rounded products and sums.
__device__ __forceinline__ void rope_rotate(float x, float y, float c, float s, float &xo, float &yo) {
  xo = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s));
  yo = __fadd_rn(__fmul_rn(x, s), __fmul_rn(y, c));
}

}  // namespace piekv
