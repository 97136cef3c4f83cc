// Definitions shared by the prefill attention kernels: tile constants, the device-built plan and the
// kernel parameter block.
#pragma once
#include <cuda.h>

#include "attn.cuh"
#include "common.cuh"

namespace piekv {
namespace prefill {

constexpr int kDim = 128;
constexpr int kPage = 16;
constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 128;  // kv tokens per tile (8 pages)
constexpr int kKStages = 3;  // K tiles in flight (needed early, by S = Q K^T)
constexpr int kVStages = 2;  // V tiles in flight (needed a softmax later, by O += P V)
constexpr int kSoftmaxWarps = 8;  // two threads per query row: each owns 64 of the 128 kv columns
constexpr int kProducerWarp = kSoftmaxWarps, kMmaWarp = kSoftmaxWarps + 1;
constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
constexpr int kTileBytes = 32768;  // one 128 x 128 16-bit operand tile
constexpr int kHalfBytes = 16384;  // one 128 x 64 half of it
constexpr int kSmemBytes = kTileBytes * (1 + kKStages + kVStages + 1) + 1024;
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256;
constexpr int kCounterBytes = 65536;
constexpr int kSortBins = 1024;

// Plan of one batch, built on the device into the workspace (after the counter area):
//   header | tile_base[B+1] | poff[B+1] | moff[B+1] | tiles[max_tiles] | summary[max_tiles][sw] | packed mask
struct PlanView {
  int *ntiles;             // header word 0
  int32_t *tile_base;      // first q-tile index of every request (prefix of ceil(qo_len / 128))
  long long *poff;         // packed-mask offset of every request, in 16-byte units
  long long *moff;         // byte offset of every request in the flat boolean mask
  int2 *tiles;             // (request, first row within the request), heaviest first
  uint32_t *summary;       // bit j of row t: kv tile j of q tile t has at least one allowed pair
  uint4 *packed;           // per query row ceil(kv_len/128) x 128 mask bits
  int sw;                  // words per summary row
  int max_tiles;
  int64_t bytes;           // total workspace bytes including the counter area
};

struct PrefillParams {
  AttnArgs a;
  const int2 *tiles;
  const int *ntiles;
  const int32_t *tile_base;
  const long long *poff;
  const uint32_t *summary;
  const uint4 *packed;
  int sw;
  int has_mask;
};

// bounded wait that also gives up when another role has already aborted
__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (global_timer_ns() - t0 > 2000000000ull) return false;
  }
}

}  // namespace prefill
}  // namespace piekv
