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
//   header (word 0: tiles, words 2-3: items claimed / CTAs finished) | tile_base[B+1] | poff[B+1] | moff[B+1] | tiles[max_tiles] | summary[max_tiles][sw] | packed mask
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
  int *claim;              // [0] items handed out, [1] CTAs that ran out of items; zero between launches
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

// Zero the rows of a staged V tile that belong to the request's last page but lie beyond its last
// token (rows [first, end) of the 128-token tile; a row is 128 bytes in each 64-column half,
// whatever the swizzle does inside it).  Their probabilities are zero, but 0 x NaN is NaN, and a
// recycled page may hold anything there.  Executed by one full warp after the tile has landed.
__device__ __forceinline__ void zero_v_rows(uint32_t v_tile_smem, int first, int end, int lane) {
  for (int x = lane; x < (end - first) * 16; x += 32) {
    const int row = first + (x >> 4), half = (x >> 3) & 1, ch = x & 7;
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(v_tile_smem + half * kHalfBytes + row * 128 + ch * 16),
                 "r"(0)
                 : "memory");
  }
}

}  // namespace prefill
}  // namespace piekv
