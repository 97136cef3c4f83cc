// Paged decode attention for 16-bit K/V, head_dim 128, page_size 16 on sm_100a.
//
// Work partition (on the device, no host plan).  The flat list of all requests' pages
// (kv_indices[0 .. kv_indptr[B])) is cut into small equal CHUNKS (a few pages each, at most kMaxChunks of
// them).  Every CTA (one per SM) owns a contiguous run of chunks and walks it front to back.  Optionally
// (PIEKV_OPT_WORK_STEALING) a CTA that runs out takes chunks from the BACK of the CTA with the most work
// left: HBM bandwidth is not the same for every SM of the two-die part (some finish an equal share 10 %
// later than others), and with stealing all SMs stop streaming within a chunk of each other - but every
// stolen piece is a run of its own with a partial to merge, and measured on config 2 the two effects
// cancel (99.7 us either way), so the default is the static split, whose results are reproducible bit for
// bit.
//
// A CTA accumulates a request's pages in registers for as long as the chunks it takes are consecutive:
// such a RUN of chunk pieces ends at a request boundary, at the end of the CTA's chunks, or (long
// requests) at a group boundary.  A run that holds a whole request is normalised and stored directly;
// otherwise the run's (max, sum, accumulator) triple goes to a scratch slot taken from a counter, the
// slot number is entered in a table at the run's first chunk, and the run adds its number of pieces to
// the request's arrival counter.  Whoever completes the count merges the request's runs.  A request
// spread over many chunks is merged in two levels (groups of chunk pieces fold concurrently on different
// SMs, the last group folds the groups).  Counters and tables are left zero by the CTAs that consume them.
//
// Data path: a producer warp gathers pages with TMA.  A page holds K [16, Hkv, 128] then
// V [16, Hkv, 128]; one 5-D tensor-map box {64 d, 16 tokens, 2 d-halves, Hkv heads, K|V}
// moves the whole page (Hkv * 8 KiB) and lands it in shared memory regrouped per head as
// 128-byte-swizzled [token][64 d] tiles, which is the layout ldmatrix wants.  A stage is
// always 64 KiB = 8 (page, head) tiles: 8/Hkv pages for Hkv heads.  Three stages keep
// 128-192 KiB per SM in flight.  The producer decides everything about the schedule and describes each
// stage to the consumers in a small shared-memory record (pages, request, run start / end).
//
// Math: consumer warp w owns tile (page w / Hkv, head w % Hkv).  The GQA group's query
// heads (<= 16) are the M rows of m16n8k16 tensor-core MMAs: S = Q K^T (16 x 16 tokens),
// fp32 online softmax in the base-2 domain with quad shuffles, O += P V.
#include <cuda.h>

#include "attn.cuh"
#include "common.cuh"
#include "rope.cuh"
#include "tma.cuh"

namespace piekv {

namespace {

constexpr int kDim = 128;
constexpr int kPage = 16;
constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
// Three warpgroups: two of consumer warps, one that holds the producer warp (its other three warps leave at
// once).  The third gives most of its registers to the consumers, whose accumulators (a [16 x 128] fp32 tile
// per warp) plus the bookkeeping of the work partition do not fit the 168 registers a 384-thread CTA starts with.
constexpr int kThreads = 384;
constexpr int kRegsLaunch = 168, kRegsConsumer = 224, kRegsProducer = 56;
static_assert(kConsumers * kRegsConsumer + 128 * kRegsProducer <= kThreads * kRegsLaunch, "registers the CTA owns");
static_assert(kRegsConsumer % 8 == 0 && kRegsProducer % 8 == 0, "setmaxnreg takes multiples of 8");
constexpr int kStages = 3;
constexpr int kTileBytes = 8192;               // one (page, head): K 4 KiB + V 4 KiB
constexpr int kStageBytes = 8 * kTileBytes;    // 64 KiB
constexpr int kMaxGrid = 256;                  // CTAs (SMs) the steal table holds

// The first 64 KiB of the workspace: everything that must be zero when a launch starts and is zero again
// when it ends (other users of the same workspace leave this block alone).
//   req_cnt  [kMaxBatch]            arrival counters of the requests (chunk pieces, or groups)
//   ctl      [16]                   0: scratch slots handed out  1: CTAs finished  2: peer completion
//   steal    [kMaxGrid] x 64 bit    (hi << 32) | lo of every CTA's remaining chunk range
//   grp_cnt  [kTable]               arrival counters of the groups of long requests
//   run_tab  [kTable] x 16 bit      slot + 1 of the run that starts at (chunk + request)
//   grp_tab  [kTable] x 16 bit      slot + 1 of a folded group, at (first chunk of the group + request)
constexpr int kCounterBytes = 65536;
constexpr int kMaxBatch = 2048;
constexpr int kMaxChunks = 4096;
constexpr int kTable = kMaxChunks + kMaxBatch;
constexpr int kCtlWord0 = kMaxBatch;
constexpr int kStealByte0 = (kMaxBatch + 16) * 4;
constexpr int kGrpCntByte0 = kStealByte0 + kMaxGrid * 8;
constexpr int kRunTabByte0 = kGrpCntByte0 + kTable * 4;
constexpr int kGrpTabByte0 = kRunTabByte0 + kTable * 2;
static_assert(kGrpTabByte0 + kTable * 2 <= kCounterBytes, "zero-state block of the decode kernel");
constexpr int kMaxSlots = 65534;               // slot + 1 must fit the 16-bit tables
constexpr int kMergeList = 1024;               // runs (or groups) one merge can fold

struct DecodeParams {
  AttnArgs a;
  float *part_o;    // [slot][subs][Hq][128]
  float2 *part_ml;  // [slot][subs][Hq]  (running max in log2 domain, running sum)
  int subs;         // partials per slot: 1, or the pages per stage when the warps of a stage cannot fold theirs on chip
  int *counters;    // the zero-state block
  int num_slots;    // scratch slots part_o / part_ml hold
  int steal;        // 0: every CTA keeps to its own chunks (results reproducible bit for bit)
  int pdl;          // programmatic dependent launch: 0 off, 1 wait first, 2 wait after the page-table offsets,
                    // 3 as 2 and the producer's first pages before the wait
  PeerOut peer;     // n == 0: results go to a.out only
  // Sliding window (a.window_left >= 0): the kernel streams only the pages that hold keys inside each
  // request's window.  win_indptr [B+1] is the prefix sum of those page counts (it takes kv_indptr's place
  // in the work partition), win_meta[b] = (shift, first): flat windowed page g of request b is
  // kv_indices[g + shift], and tokens before `first` of the request's first streamed page are outside
  // the window.  Both are written by decode_window_kernel just before the launch; nullptr: no window.
  const int32_t *win_indptr;
  const int2 *win_meta;
};

// Extra inputs of the fused step (RoPE + append + attention in one launch): the new token's
// un-rotated k / v rows and RoPE position per request.  q in AttnArgs is then un-rotated too.
struct FusedArgs {
  const void *k_new;  // [batch, Hkv, 128]
  const void *v_new;  // [batch, Hkv, 128]
  int64_t k_sn, k_sh, v_sn, v_sh;
  const int32_t *pos_ids;  // [batch]
  RopeDev rope;
};

constexpr int kSmemBatch = 1024;  // kv_indptr is staged in shared memory up to this batch size

// Optional per-CTA time stamps (builds with -DPIEKV_TRACE only): kernel entry, first page consumed, last
// page consumed, exit; read back with piekv_trace_read.
#ifdef PIEKV_TRACE
__device__ unsigned long long g_trace[256 * 16];
#define PIEKV_STAMP(slot)                                                               \
  do {                                                                                  \
    if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 0) g_trace[blockIdx.x * 16 + (slot)] = global_timer_ns(); \
  } while (0)
#define PIEKV_ACC_BEGIN() const unsigned long long acc_t0__ = global_timer_ns()
#define PIEKV_ACC_END(slot)                                                                              \
  do {                                                                                                   \
    if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 0) {                                            \
      g_trace[blockIdx.x * 16 + (slot)] += global_timer_ns() - acc_t0__;                                 \
      g_trace[blockIdx.x * 16 + (slot) + 1] += 1;                                                        \
    }                                                                                                    \
  } while (0)
#define PIEKV_ACC_RESET()                                                                                \
  do {                                                                                                   \
    if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 0)                                              \
      for (int z__ = 8; z__ < 16; ++z__) g_trace[blockIdx.x * 16 + z__] = 0;                             \
  } while (0)
#else
#define PIEKV_STAMP(slot) \
  do {                    \
  } while (0)
#define PIEKV_ACC_BEGIN() \
  do {                    \
  } while (0)
#define PIEKV_ACC_END(slot) \
  do {                      \
  } while (0)
#define PIEKV_ACC_RESET() \
  do {                    \
  } while (0)
#endif

__device__ __forceinline__ void tma_load_page(uint32_t dst, const CUtensorMap *tmap, int coord4, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(tmap)), "r"(0), "r"(0), "r"(0), "r"(0), "r"(coord4), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void consumer_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers)); }

// last request whose first page index is <= g, skipping empty requests after it
__device__ __forceinline__ int request_of_page(const int32_t *indptr, int batch, int g) {
  int lo = 0, hi = batch;  // first b with indptr[b+1] > g
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (indptr[mid + 1] > g)
      hi = mid;
    else
      lo = mid + 1;
  }
  return lo;
}

// Windowed page ranges of a decode batch.  One block; a request keeps the pages from the one that holds
// key (seq_len - 1 - window_left) to its last.
__global__ void __launch_bounds__(1024) decode_window_kernel(const int32_t *__restrict__ kv_indptr,
                                                             const int32_t *__restrict__ last_page_len, int batch,
                                                             int window_left, int32_t *win_indptr, int2 *win_meta) {
  __shared__ int sh[32];
  __shared__ int carry;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (int base = 0; base < batch; base += 1024) {
    const int b = base + threadIdx.x;
    int eff = 0, skip = 0, first = 0, p0 = 0;
    if (b < batch) {
      p0 = kv_indptr[b];
      const int np = kv_indptr[b + 1] - p0;
      if (np > 0) {
        int last = last_page_len[b];
        last = last < 1 ? 1 : (last > kPage ? kPage : last);  // the attention kernel reports a bad value
        const int seq = (np - 1) * kPage + last;
        const int first_tok = max(0, seq - 1 - window_left);
        skip = first_tok / kPage;
        first = first_tok % kPage;
        eff = np - skip;
      }
    }
    int x = eff;  // inclusive scan over the block
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int y = __shfl_up_sync(0xffffffffu, x, d);
      if (lane >= d) x += y;
    }
    if (lane == 31) sh[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int w = sh[lane];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, w, d);
        if (lane >= d) w += y;
      }
      sh[lane] = w;
    }
    __syncthreads();
    const int excl = carry + (warp > 0 ? sh[warp - 1] : 0) + x - eff;
    if (b < batch) {
      win_indptr[b] = excl;
      win_meta[b] = make_int2(p0 + skip - excl, first);
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry = excl + eff;
    __syncthreads();
  }
  if (threadIdx.x == 0) win_indptr[batch] = carry;
}

// Run header: what the consumers need to open a run (the request's query rows and, for the fused step,
// its new k / v rows and RoPE position), brought into shared memory by the producer ahead of time with
// bulk copies, so that opening a run costs no trip to global memory while the page pipeline drains.
constexpr int kHdrQBytes = 8192;   // up to 32 query heads
constexpr int kHdrKOff = kHdrQBytes, kHdrVOff = kHdrKOff + 2048, kHdrMetaOff = kHdrVOff + 2048;
constexpr int kHdrBytes = kHdrMetaOff + 32;
constexpr int kHdrSlots = 2;

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t *bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// What the producer tells the consumers about a stage (written before the stage's barrier is armed).
struct StageDesc {
  int g;            // flat index of the stage's first page; -1: no more work
  int b;            // request
  int npg;          // pages in the stage
  int flags;        // kRunStart | kRunEnd
  int first_chunk;  // chunk the run started in (meaningful with kRunEnd)
  int pieces;       // chunk pieces of the request the run covered (meaningful with kRunEnd)
  int hdr;          // run header: slot | phase << 1, or -1 when the consumers load the rows themselves
  int pad;
  int page[8];      // physical ids of the stage's pages
};
constexpr int kRunStart = 1, kRunEnd = 2;

// 64-bit steal word: (hi << 32) | lo, chunks [lo, hi) are still untaken.  The owner takes from the front
// (add 1), others from the back (subtract k << 32); the word only ever shrinks the range, so whoever's
// atomic comes first gets the chunk.
__device__ __forceinline__ unsigned long long steal_pack(int lo, int hi) {
  return ((unsigned long long)(unsigned int)hi << 32) | (unsigned int)lo;
}
__device__ __forceinline__ int steal_lo(unsigned long long w) { return (int)(unsigned int)(w & 0xffffffffull); }
__device__ __forceinline__ int steal_hi(unsigned long long w) { return (int)(unsigned int)(w >> 32); }

// The non-zero entries of tab[first .. first + count) in index order -> list (slot numbers); the entries
// are zeroed on the way.  All consumer threads; returns how many (at most kMergeList).
__device__ __noinline__ int collect_slots(unsigned short *tab, int first, int count, unsigned short *list,
                                          int *nlist, int *wsum) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int done = 0;  // entries found so far (the same in every thread)
  for (int base = 0; base < count; base += kConsumers) {
    const int i = base + tid;
    unsigned short v = 0;
    if (i < count) {
      v = __ldcg(tab + first + i);
      if (v != 0) tab[first + i] = 0;
    }
    const unsigned m = __ballot_sync(0xffffffffu, v != 0);
    if (lane == 0) wsum[warp] = __popc(m);
    consumer_bar_sync();
    int off = done, all = done;
#pragma unroll
    for (int w = 0; w < kConsumerWarps; ++w) {
      const int n = wsum[w];
      if (w < warp) off += n;
      all += n;
    }
    off += __popc(m & ((1u << lane) - 1u));
    if (v != 0 && off < kMergeList) list[off] = (unsigned short)(v - 1);
    done = all;
    consumer_bar_sync();  // the list is complete (and wsum free) before anybody goes on
  }
  (void)nlist;
  return min(done, kMergeList);
}

// Fold the partials of the slots in list[0 .. n) (`subs` sub-slots each) for the HW query heads
// q0, q0 + 8, ... of this warp; lanes own 4 consecutive d.  One pass with a running maximum, 16 / HW partials
// at a time: all of a batch's loads are issued before any value is used, so a typical merge is a single trip
// to L2 - which, while the other SMs are still streaming, takes microseconds.  The result is the request's
// output row (normalised) or again a partial (maximum, sum, unnormalised accumulator) written to sub-slot 0
// of `to_slot`.
template <typename T, int HW>
__device__ __forceinline__ void merge_heads(const DecodeParams &p, const unsigned short *list, int np, int subs, int b,
                                            int to_slot, int peer_step, int q0) {
  constexpr int PB = 16 / HW;  // partials per batch
  const AttnArgs &a = p.a;
  const int lane = threadIdx.x & 31;
  const int d4 = lane * 4;
  float M[HW], L[HW];
  float4 acc[HW];
#pragma unroll
  for (int u = 0; u < HW; ++u) {
    M[u] = -INFINITY;
    L[u] = 0.f;
    acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int p0 = 0; p0 < np; p0 += PB) {
    float2 ml[PB][HW];
    float4 po[PB][HW];
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      const int pp = min(p0 + j, np - 1);  // (a slot read twice at the end of the list gets weight 0)
      const size_t base = ((size_t)list[pp / subs] * p.subs + pp % subs) * a.hq;
#pragma unroll
      for (int u = 0; u < HW; ++u) {
        const int qh = min(q0 + u * kConsumerWarps, a.hq - 1);
        ml[j][u] = __ldcg(p.part_ml + base + qh);
        po[j][u] = __ldcg(reinterpret_cast<const float4 *>(p.part_o + (base + qh) * kDim + d4));
      }
    }
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      const bool live = p0 + j < np;
#pragma unroll
      for (int u = 0; u < HW; ++u) {
        if (live && ml[j][u].y > 0.f) {  // (a warp that saw no page contributes nothing)
          const float mn = fmaxf(M[u], ml[j][u].x);
          const float so = fast_exp2(M[u] - mn);  // M = -inf at first: 0
          const float w = fast_exp2(ml[j][u].x - mn);
          M[u] = mn;
          L[u] = fmaf(L[u], so, ml[j][u].y * w);
          acc[u].x = fmaf(acc[u].x, so, po[j][u].x * w);
          acc[u].y = fmaf(acc[u].y, so, po[j][u].y * w);
          acc[u].z = fmaf(acc[u].z, so, po[j][u].z * w);
          acc[u].w = fmaf(acc[u].w, so, po[j][u].w * w);
        }
      }
    }
  }
  const int n_dst = p.peer.n > 0 ? p.peer.n : 1;
  const int row_heads = p.peer.n > 0 ? p.peer.row_heads : a.hq;
  const int head_off = p.peer.n > 0 ? p.peer.head_off : 0;
  const bool use_alt = p.peer.n > 0 && p.peer.step_ptr != nullptr && (peer_step & 1) == 0;
#pragma unroll
  for (int u = 0; u < HW; ++u) {
    const int qh = q0 + u * kConsumerWarps;
    if (qh >= a.hq) continue;
    if (to_slot >= 0) {
      __syncwarp();  // every lane has read this head's partials before one of them is overwritten
      const size_t idx = (size_t)to_slot * p.subs * a.hq + qh;
      *reinterpret_cast<float4 *>(p.part_o + idx * kDim + d4) = acc[u];
      if (lane == 0) p.part_ml[idx] = make_float2(M[u], L[u]);
      continue;
    }
    const float Ls = add_sink(L[u], M[u], a.sinks, qh);
    const float inv = Ls > 0.f ? 1.f / Ls : 0.f;
    uint2 pk;
    pk.x = pack2<T>(acc[u].x * inv, acc[u].y * inv);
    pk.y = pack2<T>(acc[u].z * inv, acc[u].w * inv);
    for (int d = 0; d < n_dst; ++d) {
      void *pb = a.out;
      if (p.peer.n > 0) pb = use_alt ? p.peer.dst_alt[d] : p.peer.dst[d];
      T *row = reinterpret_cast<T *>(pb) + ((size_t)b * row_heads + head_off + qh) * kDim;
      *reinterpret_cast<uint2 *>(row + d4) = pk;
    }
    if (a.lse != nullptr && lane == 0)
      a.lse[(size_t)b * a.hq + qh] = Ls > 0.f ? (M[u] + log2f(Ls)) * 0.6931471805599453f : -INFINITY;
  }
}

// All consumer threads: warp w folds heads w, w + 8, ... (up to four at a time; with few heads per warp more
// partials are in flight per batch instead).
template <typename T>
__device__ __noinline__ void merge_slots(const DecodeParams &p, const unsigned short *list, int n, int subs, int b,
                                         int to_slot, int peer_step) {
  const int warp = threadIdx.x >> 5;
  const int np = n * subs;
  const int hq = p.a.hq;
  for (int q0 = warp; q0 < hq; q0 += 4 * kConsumerWarps) {
    const int left = (hq - q0 + kConsumerWarps - 1) / kConsumerWarps;  // heads of this warp from q0 on
    if (left >= 3)
      merge_heads<T, 4>(p, list, np, subs, b, to_slot, peer_step, q0);
    else if (left == 2)
      merge_heads<T, 2>(p, list, np, subs, b, to_slot, peer_step, q0);
    else
      merge_heads<T, 1>(p, list, np, subs, b, to_slot, peer_step, q0);
  }
}

template <typename T, int HKV, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1)
    decode_tma_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ DecodeParams p,
                      const __grid_constant__ FusedArgs f) {
  constexpr int PG = 8 / HKV;  // pages per stage
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t desc_bar[kStages];  // the stage's record is written (its pages may still be in flight)
  __shared__ StageDesc sh_desc[kStages];
  __shared__ int sh_abort;
  __shared__ int sh_last;
  __shared__ int sh_slot;
  __shared__ int sh_nlist;
  __shared__ int sh_wsum[kConsumerWarps];
  __shared__ unsigned short sh_list[kMergeList];
  __shared__ int32_t sh_indptr[kSmemBatch + 1];
  __shared__ __align__(8) uint64_t hdr_full[kHdrSlots];
  __shared__ __align__(8) uint64_t hdr_empty[kHdrSlots];
  __shared__ __align__(128) uint8_t sh_hdr[kHdrSlots][kHdrBytes];
  __shared__ float2 sh_cs[kDim / 2];  // fused step: (cos, sin) of the open run's position, one entry per pair

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *stage0_ptr = smem_raw + (stage0 - smem_u32(smem_raw));

  const AttnArgs &a = p.a;
  const int B = a.batch;
  const int c = blockIdx.x;
  const int G = gridDim.x;
  PIEKV_STAMP(0);
  PIEKV_ACC_RESET();
  // Programmatic dependent launch: let the next kernel of the stream start its own prologue as SMs
  // free up, and do not touch anything an earlier kernel may still be producing before the wait.
  // Mode 2 is for callers whose page-table arrays are not written by the kernel just before this one
  // (the reference uploads them once per step, ahead of the layer loop): the offsets are then read
  // before the wait.  Both instructions do nothing in a launch without the attribute.
  if (p.pdl) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (p.pdl == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
  // one coalesced read of the page-table offsets instead of a chain of dependent searches in L2
  const bool windowed = p.win_indptr != nullptr;
  const int32_t *ip = windowed ? p.win_indptr : a.kv_indptr;  // the windowed prefix takes the offsets' place
  if (B <= kSmemBatch) {
    const int32_t *src = ip;
    for (int x = threadIdx.x; x <= B; x += kThreads) sh_indptr[x] = __ldg(src + x);
    ip = sh_indptr;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kConsumerWarps);
      mbar_init(&desc_bar[s], 1);
    }
    for (int s = 0; s < kHdrSlots; ++s) {
      mbar_init(&hdr_full[s], FUSED ? 2 : 1);  // the bulk copies' arming arrival (+ the position's copy)
      mbar_init(&hdr_empty[s], kConsumerWarps);
    }
    sh_abort = 0;
    sh_last = 0;
    mbar_fence_init();
  }
  __syncthreads();
  // Mode 3 adds to mode 2 the promise that the kernel just before wrote at most into the LAST TWO pages of any
  // request (a decode step appends one token: the page it wrote is the next step's last or last but one):
  // the producer warp then starts bringing in its first pages before it waits, everybody else waits here.
  if (p.pdl == 2 || (p.pdl == 3 && warp != kConsumerWarps)) asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- chunk geometry, the same on every CTA
  const int total_pages = ip[B];
  const int stages_total = (total_pages + PG - 1) / PG;
  // pages per chunk: at most kMaxChunks chunks, and two stages or more once there is enough work, so that a
  // chunk's first loads are in flight while the producer finds out what it will do next
  const int cp = PG * max(stages_total >= 8 * G ? 2 : 1, (stages_total + kMaxChunks - 1) / kMaxChunks);
  const int n_chunks = (total_pages + cp - 1) / cp;
  // Every CTA owns a contiguous range of chunks of about equal cost: opening and closing a run costs about as
  // much as streaming one stage, so a share that holds many short requests gets fewer pages.  bound(i) is the
  // chunk at which CTA i starts: where pages + kRunCost * (requests passed) reaches i / G of the total.
  constexpr int kRunCost = PG;  // pages (weights of 2 and 3 stages measured the same within noise)
  auto bound = [&](int i) -> int {
    if (i <= 0) return 0;
    if (i >= G) return n_chunks;
    const long long target = ((long long)total_pages + (long long)kRunCost * B) * i / G;
    int lo = 0, hi = B;  // first request b with ip[b + 1] + PG * (b + 1) > target
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if ((long long)ip[mid + 1] + (long long)kRunCost * (mid + 1) > target)
        hi = mid;
      else
        lo = mid + 1;
    }
    if (lo >= B) return n_chunks;
    long long g = target - (long long)kRunCost * lo;
    g = g < ip[lo] ? ip[lo] : (g > ip[lo + 1] ? ip[lo + 1] : g);
    const int ch = (int)((g + cp / 2) / cp);
    return ch < n_chunks ? ch : n_chunks;
  };
  const int my_lo = bound(c);
  const int my_hi = bound(c + 1);
  // chunk pieces per merge group of a long request: about what 16 CTAs own
  const int gsz = 16 * max(1, n_chunks / G);
  const int group = a.hq / HKV;
  // several pages per stage and a GQA group that fits a warp's own tile: the warps of a stage fold their
  // partials through shared memory when a run ends (p.subs == 1), instead of each writing its own to scratch
  const bool fold_on_chip = PG > 1 && group <= 8;

  // Run headers need the rows contiguous and 16-byte aligned for bulk copies, and at most 32 query heads.
  bool use_hdr = a.hq * kDim * (int)sizeof(T) <= kHdrQBytes && a.q_sh == kDim &&
                 (reinterpret_cast<uintptr_t>(a.q) & 15) == 0 && ((a.q_sn * (int64_t)sizeof(T)) & 15) == 0;
  if (FUSED)
    use_hdr = use_hdr && f.k_sh == kDim && f.v_sh == kDim && (reinterpret_cast<uintptr_t>(f.k_new) & 15) == 0 &&
              (reinterpret_cast<uintptr_t>(f.v_new) & 15) == 0 && ((f.k_sn * (int64_t)sizeof(T)) & 15) == 0 &&
              ((f.v_sn * (int64_t)sizeof(T)) & 15) == 0 && f.pos_ids != nullptr;

  int *req_cnt = p.counters;
  int *ctl = p.counters + kCtlWord0;
  unsigned long long *steal_tab =
      reinterpret_cast<unsigned long long *>(reinterpret_cast<uint8_t *>(p.counters) + kStealByte0);
  int *grp_cnt = reinterpret_cast<int *>(reinterpret_cast<uint8_t *>(p.counters) + kGrpCntByte0);
  unsigned short *run_tab = reinterpret_cast<unsigned short *>(reinterpret_cast<uint8_t *>(p.counters) + kRunTabByte0);
  unsigned short *grp_tab = reinterpret_cast<unsigned short *>(reinterpret_cast<uint8_t *>(p.counters) + kGrpTabByte0);

  if (warp >= kConsumerWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsProducer));
    if (warp > kConsumerWarps) return;  // idle warps of the third warpgroup
    // ------------------------------------------------------------------ producer
    int armed = 0;  // stages armed so far
    bool ok = true;
    // publish one stage: wait for the slot, describe it, arm the barrier, issue the page loads
    auto publish = [&](const StageDesc &d, int page_of_lane) -> bool {
      const int s = armed % kStages;
      const uint32_t ph = (armed / kStages) & 1;
      if (*(volatile int *)&sh_abort) return false;
      if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
        if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, 100 + s);
        if (lane == 0) atomicExch(&sh_abort, 1);
        return false;
      }
      if (lane == 0) {
        sh_desc[s].g = d.g;
        sh_desc[s].b = d.b;
        sh_desc[s].npg = d.npg;
        sh_desc[s].flags = d.flags;
        sh_desc[s].first_chunk = d.first_chunk;
        sh_desc[s].pieces = d.pieces;
        sh_desc[s].hdr = d.hdr;
      }
      if (lane < d.npg) sh_desc[s].page[lane] = page_of_lane;
      __syncwarp();
      // the record first: the consumers open a run (query loads, rotation) while the pages are in flight
      if (lane == 0) mbar_arrive(&desc_bar[s]);
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], (uint32_t)(d.npg * HKV * kTileBytes));
      __syncwarp();
      if (lane < d.npg)
        tma_load_page(stage0 + s * kStageBytes + lane * (HKV * kTileBytes), &tmap, page_of_lane * 2, &full_bar[s]);
      ++armed;
      return true;
    };

    // ---- which chunks: the own range front to back, then the back of whoever has most left.
    // The first part of the own range is private (walked without any atomic, like a static split); the
    // rest is shared: the owner claims it chunk by chunk with an atomic issued one chunk ahead (so that the
    // answer is there when it is needed), others may take chunks from its back.
    const int my_n = my_hi - my_lo;
    const int priv = p.steal ? max(min(my_n, 1), my_n - max(2, my_n / 3)) : my_n;
    int cur_lo = my_lo, cur_hi = my_lo + priv;  // interval of chunks in hand
    // ---- mode 3: the first stages of the own range go out before the wait (never a piece's last stage, which
    // may have to say that the run ends, and never one of a request's last two pages)
    int resume_g = -1, resume_b = 0;
    if (p.pdl == 3) {
      if (cur_lo < cur_hi) {
        const int b0 = request_of_page(ip, B, cur_lo * cp);
        int g = cur_lo * cp;
        const int seg_end = min(min(total_pages, g + cp), ip[b0 + 1]);
        const int safe_end = ip[b0 + 1] - 2;
        int n = 0;
        while (n < kStages && g + min(PG, seg_end - g) < seg_end && g + min(PG, seg_end - g) <= safe_end) {
          const int npg = min(PG, seg_end - g);
          int page = lane < npg ? __ldg(a.kv_indices + g + lane) : 0;
          if (lane < npg && (page < 0 || page >= a.num_pages)) {
            report_error(a.err, PIEKV_ERR_PAGE_ID, KID_DECODE, g + lane, page);
            page = a.num_pages;
          }
          StageDesc d;
          d.g = g;
          d.b = b0;
          d.npg = npg;
          d.flags = n == 0 ? kRunStart : 0;
          d.first_chunk = cur_lo;
          d.pieces = 1;
          d.hdr = use_hdr ? 0 : -1;  // the first header is slot 0, phase 0; its copies follow the wait
          if (!publish(d, page)) {
            ok = false;
            break;
          }
          g += npg;
          ++n;
        }
        if (n > 0) {
          resume_g = g;
          resume_b = b0;
        }
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    if (lane == 0) atomicExch(&steal_tab[c], steal_pack(my_lo + priv, my_hi));  // nothing else is published with it
    unsigned long long claim = 0;                // lane 0: answer of the claim in flight
    bool claim_out = false;                      // a claim has been issued and not yet looked at
    auto issue_claim = [&]() {
      if (lane == 0) claim = atomicAdd(&steal_tab[c], 1ull);
      claim_out = true;
    };
    auto next_interval = [&](int &lo_out, int &hi_out) -> bool {
      unsigned long long got = 0;
      bool have = false;
      if (!claim_out) issue_claim();
      claim_out = false;
      if (lane == 0 && steal_lo(claim) < steal_hi(claim)) {
        got = steal_pack(steal_lo(claim), steal_lo(claim) + 1);
        have = true;
      }
      have = __shfl_sync(0xffffffffu, have ? 1 : 0, 0) != 0;
      if (!have && p.steal) {
        for (int attempt = 0; attempt < 4 && !have; ++attempt) {
          int best = 0, who = -1;
          for (int v = lane; v < G; v += 32) {
            const unsigned long long w = __ldcg(&steal_tab[v]);
            const int rem = steal_hi(w) - steal_lo(w);
            if (v != c && rem > best) {
              best = rem;
              who = v;
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const int ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int ow = __shfl_xor_sync(0xffffffffu, who, o);
            if (ob > best || (ob == best && ow > who)) {
              best = ob;
              who = ow;
            }
          }
          if (best < 2) break;  // a last chunk is finished sooner by its owner than taken over
          int stop = 0;
          if (lane == 0) {
            // scratch slots are finite and every stolen interval is a run of its own
            if (__ldcg(&ctl[0]) + 2 * G + B + 8 < p.num_slots) {
              // small bites: everybody is about to finish, and what is taken here cannot be taken back
              const int k = best >= 8 ? 2 : 1;
              const unsigned long long old = atomicAdd(&steal_tab[who], 0ull - ((unsigned long long)k << 32));
              const int lo_v = steal_lo(old), hi_v = steal_hi(old);
              if (lo_v < hi_v) {
                got = steal_pack(max(lo_v, hi_v - k), hi_v);
                have = true;
              }
            } else {
              stop = 1;
            }
          }
          have = __shfl_sync(0xffffffffu, have ? 1 : 0, 0) != 0;
          if (__shfl_sync(0xffffffffu, stop, 0)) break;
        }
      }
      got = __shfl_sync(0xffffffffu, got, 0);
      lo_out = steal_lo(got);
      hi_out = steal_hi(got);
      return have;
    };

    // ---- walk the chunks in hand; a run continues while the next chunk is the next one of the same request
    bool have = cur_lo < cur_hi;
    if (!have) have = next_interval(cur_lo, cur_hi);
    bool run_open = false;
    int run_first = 0, run_pieces = 0;
    int hdr_n = 0, run_hdr = -1;  // headers started so far; the open run's header word
    // bring request b_'s rows into the next header slot (asynchronously) and return its header word
    auto start_header = [&](int b_) -> int {
      if (!use_hdr) return -1;
      const int hs = hdr_n % kHdrSlots;
      const int hph = (hdr_n / kHdrSlots) & 1;
      if (!mbar_wait(&hdr_empty[hs], hph ^ 1)) {
        if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, 300 + hs);
        if (lane == 0) atomicExch(&sh_abort, 1);
        return -2;
      }
      if (lane == 0) {
        const uint32_t dst = smem_u32(&sh_hdr[hs][0]);
        const uint32_t qbytes = (uint32_t)(a.hq * kDim * sizeof(T));
        const uint32_t kbytes = FUSED ? (uint32_t)(HKV * kDim * sizeof(T)) : 0u;
        mbar_arrive_expect_tx(&hdr_full[hs], qbytes + 2 * kbytes);
        bulk_copy_g2s(dst, reinterpret_cast<const T *>(a.q) + (size_t)b_ * a.q_sn, qbytes, &hdr_full[hs]);
        if (FUSED) {
          bulk_copy_g2s(dst + kHdrKOff, reinterpret_cast<const T *>(f.k_new) + (size_t)b_ * f.k_sn, kbytes, &hdr_full[hs]);
          bulk_copy_g2s(dst + kHdrVOff, reinterpret_cast<const T *>(f.v_new) + (size_t)b_ * f.v_sn, kbytes, &hdr_full[hs]);
          cp_async_4(dst + kHdrMetaOff, f.pos_ids + b_);
          cp_async_arrive_noinc(&hdr_full[hs]);
        }
      }
      __syncwarp();
      ++hdr_n;
      return hs | (hph << 1);
    };
    if (resume_g >= 0 && ok) {  // the run opened before the wait: its rows can be fetched now
      run_open = true;
      run_first = cur_lo;
      run_pieces = 1;
      run_hdr = start_header(resume_b);
      if (run_hdr == -2) ok = false;
    }
    while (have && ok) {
      int b = request_of_page(ip, B, cur_lo * cp);
      int nx_lo = 0, nx_hi = 0;
      bool have_next = false;
      for (int ck = cur_lo; ck < cur_hi && ok; ++ck) {
        // What follows this chunk decides whether the run goes on, which only the chunk's LAST stage has to
        // say.  For the last chunk in hand the claim of the next one is issued now and looked at then.
        bool next_known = ck + 1 < cur_hi;
        int next_ck = ck + 1;
        if (!next_known && !claim_out) issue_claim();
        int g = ck * cp;
        const int chunk_end = min(total_pages, g + cp);
        while (g < chunk_end && ok) {
          const bool resumed = resume_g >= 0;  // (only the very first piece can be one begun before the wait)
          if (resumed) g = resume_g;
          resume_g = -1;
          while (b < B - 1 && ip[b + 1] <= g) ++b;
          const int req_begin = ip[b], req_end = ip[b + 1];
          const int seg_end = min(chunk_end, req_end);
          if (seg_end <= g) {  // non-monotone indptr: give up cleanly
            if (lane == 0) report_error(a.err, PIEKV_ERR_INDPTR, KID_DECODE, b, g);
            if (lane == 0) atomicExch(&sh_abort, 1);
            ok = false;
            break;
          }
          const int c_first = req_begin / cp, c_last = (req_end - 1) / cp;
          const bool two_level = c_last - c_first + 1 > gsz;
          if (!run_open) {
            run_open = true;
            run_first = ck;
            run_pieces = 0;
            run_hdr = start_header(b);
            if (run_hdr == -2) {
              ok = false;
              break;
            }
          }
          if (!resumed) ++run_pieces;
          const int shift = windowed ? __ldg(&p.win_meta[b].x) : 0;
          const bool starts = run_pieces == 1;
          bool first_stage = !resumed;
          bool goes_on = false;
          // the piece's page ids, 32 at a time in one coalesced load (lane l holds page id_base + l)
          int id_base = g;
          int ids = g + lane < seg_end ? __ldg(a.kv_indices + g + shift + lane) : 0;
          while (g < seg_end) {
            const int npg = min(PG, seg_end - g);
            if (g + npg > id_base + 32) {
              id_base = g;
              ids = g + lane < seg_end ? __ldg(a.kv_indices + g + shift + lane) : 0;
            }
            int page = __shfl_sync(0xffffffffu, ids, (g - id_base + lane) & 31);
            if (lane < npg && (page < 0 || page >= a.num_pages)) {
              report_error(a.err, PIEKV_ERR_PAGE_ID, KID_DECODE, g + lane, page);
              page = a.num_pages;  // outside the tensor map: the box is zero-filled
            }
            const bool last_stage = g + npg >= seg_end;
            if (last_stage && seg_end < req_end) {
              // the piece ends with the chunk, not with the request: does the run go on?
              if (!next_known) {
                have_next = next_interval(nx_lo, nx_hi);
                next_ck = have_next ? nx_lo : -1;
                next_known = true;
              }
              goes_on = next_ck == ck + 1 && !(two_level && (ck + 1 - c_first) % gsz == 0);
            }
            StageDesc d;
            d.g = g;
            d.b = b;
            d.npg = npg;
            d.flags = ((starts && first_stage) ? kRunStart : 0) | ((last_stage && !goes_on) ? kRunEnd : 0);
            d.first_chunk = run_first;
            d.pieces = run_pieces;
            d.hdr = run_hdr;
            if (!publish(d, page)) {
              ok = false;
              break;
            }
            first_stage = false;
            g += npg;
          }
          if (!goes_on) run_open = false;
        }
        if (!next_known && ok) {  // the chunk ended with a request: still need to know what comes next
          have_next = next_interval(nx_lo, nx_hi);
          next_known = true;
        }
      }
      have = have_next;
      cur_lo = nx_lo;
      cur_hi = nx_hi;
    }
    if (ok) {  // tell the consumers that nothing follows
      StageDesc d;
      d.g = -1;
      d.b = 0;
      d.npg = 0;
      d.flags = 0;
      d.first_chunk = 0;
      d.pieces = 0;
      d.hdr = -1;
      publish(d, 0);
    }
    // Drain: do not let the CTA retire while a bulk copy may still be landing.
    __syncwarp();
    if (lane == 0) {
      const int first = armed > kStages ? armed - kStages : 0;
      for (int it = first; it < armed; ++it) {
        mbar_wait(&full_bar[it % kStages], (it / kStages) & 1, 200000000ull);
      }
      for (int hn = hdr_n > kHdrSlots ? hdr_n - kHdrSlots : 0; hn < hdr_n; ++hn)
        mbar_wait(&hdr_full[hn % kHdrSlots], (hn / kHdrSlots) & 1, 200000000ull);
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsConsumer));
  const int tid = threadIdx.x;   // 0..255
  const int pslot = warp / HKV;  // page slot within a stage
  const int h = warp % HKV;      // kv head
  const int quad = lane >> 2;    // MMA row (and row + 8)
  const int qlane = lane & 3;
  const float scale_log2 = a.sm_scale * 1.4426950408889634f;
  // Where results go: a.out, or (head-sharded run over several GPUs) the same rows of an output
  // buffer on every GPU, this GPU's heads at column head_off of rows that hold row_heads heads.
  T *out = reinterpret_cast<T *>(a.out);
  const int n_dst = p.peer.n > 0 ? p.peer.n : 1;
  const int row_heads = p.peer.n > 0 ? p.peer.row_heads : a.hq;
  const int head_off = p.peer.n > 0 ? p.peer.head_off : 0;
  // The step number either came with the launch or sits in device memory, where the wait that closes
  // a step bumps it: a captured graph can then be replayed step after step.  Odd steps use dst, even
  // steps dst_alt.  Read once per thread here: every input of this kernel is final by now (the
  // programmatic-dependent-launch waits are above).
  int peer_step = p.peer.step;
  if (p.peer.n > 0 && p.peer.step_ptr != nullptr) peer_step = ld_global_relaxed_sys(p.peer.step_ptr);
  const bool use_alt = p.peer.n > 0 && p.peer.step_ptr != nullptr && (peer_step & 1) == 0;
  auto dst_row = [&](int d, int b_, int qh) -> T * {
    void *pb = a.out;
    if (p.peer.n > 0) pb = use_alt ? p.peer.dst_alt[d] : p.peer.dst[d];
    return reinterpret_cast<T *>(pb) + ((size_t)b_ * row_heads + head_off + qh) * kDim;
  };
  // Every CTA passes here exactly once after its last result store.  The CTA that arrives last tidies the
  // zero-state block (scratch-slot counter, steal words) and, on a head-sharded run, publishes this step's
  // number in every GPU's flag array: all stores of this launch, fenced at system scope by their threads,
  // are ordered before it.
  auto finish = [&]() {
    if (p.peer.n > 0) __threadfence_system();
    consumer_bar_sync();
    if (tid == 0) {
      if (p.peer.n > 0) __threadfence_system();
      sh_last = atomicAdd(&ctl[1], 1) == G - 1 ? 1 : 0;
    }
    consumer_bar_sync();
    if (sh_last == 0) return;
    for (int v = tid; v < G; v += kConsumers) steal_tab[v] = 0ull;
    if (tid == 0) {
#ifdef PIEKV_TRACE
      g_trace[255 * 16] = (unsigned long long)ctl[0];  // scratch slots (= merged runs) this launch used
#endif
      ctl[0] = 0;
      ctl[1] = 0;  // ready for the next launch
      if (p.peer.n > 0) {
        __threadfence_system();
        for (int d = 0; d < p.peer.n; ++d)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.peer.flag[d]), "r"(peer_step) : "memory");
      }
    }
  };

  // requests without any page: softmax over nothing -> zeros
  for (int b = c; b < B; b += G) {
    if (ip[b + 1] == ip[b]) {
      for (int d = 0; d < n_dst; ++d) {
        T *row = dst_row(d, b, 0);
        for (int x = tid; x < a.hq * kDim; x += kConsumers) row[x] = Elem<T>::from_f32(0.f);
      }
      if (a.lse != nullptr)
        for (int x = tid; x < a.hq; x += kConsumers) a.lse[(size_t)b * a.hq + x] = -INFINITY;
    }
  }

  // Publish this run (or folded group) and count it in.  Every thread's stores come before the barrier;
  // thread 0 then writes the table entry, fences once (the fence covers what it has synchronised with) and
  // adds to the counter.  Whoever completes a count sees everybody else's partials (read through L2).
  auto arrive = [&](unsigned short *tab_entry, int slot_, int *counter, int add, int expected) -> bool {
    consumer_bar_sync();
    if (tid == 0) {
      *tab_entry = (unsigned short)(slot_ + 1);
      __threadfence();
      const int old = atomicAdd(counter, add);
      sh_last = (old + add == expected) ? 1 : 0;
      if (sh_last) {
        *counter = 0;  // ready for the next launch (nobody else touches it any more)
        __threadfence();
      }
    }
    consumer_bar_sync();
    return sh_last != 0;
  };
  auto collect = [&](unsigned short *tab, int first, int count) -> int {
    return collect_slots(tab, first, count, sh_list, &sh_nlist, sh_wsum);
  };
  auto merge_list = [&](int n, int subs, int b_, int to_slot) {
    merge_slots<T>(p, sh_list, n, subs, b_, to_slot, peer_step);
  };

  int b = 0, req_begin = 0, req_end = 0, last_len = kPage, rope_pos = 0, win_first = 0;
  int my_slot = 0;  // thread 0: the open run's scratch slot
  int cur_hdr = -1; // the open run's header word (-1: rows are read from global memory)
  bool aborted = false, finished = false;
  int it = 0, s = 0, g = 0, npg = 0, flags = 0, run_first = 0, run_pieces = 0, my_page = -1;
  uint32_t ph = 0;
  // Wait for the record of stage `it` and read it: 1 a stage, 0 nothing follows, -1 given up.
  auto fetch = [&]() -> int {
    s = it % kStages;
    ph = (it / kStages) & 1;
    if (*(volatile int *)&sh_abort) return -1;
    if (!mbar_wait(&desc_bar[s], ph)) {
      if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, 200 + s);
      if (lane == 0) atomicExch(&sh_abort, 1);
      return -1;
    }
    g = sh_desc[s].g;
    if (g < 0) return 0;  // (the closing record is armed without pages; nobody waits for its slot)
    npg = sh_desc[s].npg;
    flags = sh_desc[s].flags;
    run_first = sh_desc[s].first_chunk;
    run_pieces = sh_desc[s].pieces;
    my_page = pslot < npg ? sh_desc[s].page[pslot] : -1;
    return 1;
  };

  // One iteration per run: the accumulators live inside it, so nothing of a finished run is kept (or saved
  // around the merge calls) once its partial is written.
  while (true) {
    {
      const int r = fetch();
      if (r <= 0) {
        aborted = r < 0;
        break;
      }
    }
    if (it == 0) PIEKV_STAMP(1);
    uint32_t qa[8][4];
    float o[16][4];
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    {
      // ================= open a run of request b
      // (a scratch slot is asked for now so that its number is there when the run closes; a run that turns
      // out to hold a whole request leaves its slot unused)
      if (tid == 0) my_slot = atomicAdd(&ctl[0], 1);
      b = sh_desc[s].b;
      req_begin = ip[b];
      req_end = ip[b + 1];
      m0 = m1 = -INFINITY;
      l0 = l1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
      cur_hdr = sh_desc[s].hdr;
      last_len = __ldg(a.kv_last_page_len + b);  // (used, and checked, at the request's last page)
      win_first = windowed ? __ldg(&p.win_meta[b].y) : 0;
      if (cur_hdr >= 0) {
        // the rows are (or are about to be) in shared memory: no trip to global memory here
        if (!mbar_wait(&hdr_full[cur_hdr & 1], (uint32_t)(cur_hdr >> 1))) {
          if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, 310);
          if (lane == 0) atomicExch(&sh_abort, 1);
          aborted = true;
          break;
        }
        const T *qb = reinterpret_cast<const T *>(&sh_hdr[cur_hdr & 1][0]) + (size_t)(h * group) * kDim;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int col = ks * 16 + qlane * 2;
          const uint32_t *r0 = reinterpret_cast<const uint32_t *>(qb + (size_t)quad * kDim + col);
          const uint32_t *r1 = reinterpret_cast<const uint32_t *>(qb + (size_t)(quad + 8) * kDim + col);
          qa[ks][0] = quad < group ? *r0 : 0u;
          qa[ks][1] = quad + 8 < group ? *r1 : 0u;
          qa[ks][2] = quad < group ? *(r0 + 4) : 0u;
          qa[ks][3] = quad + 8 < group ? *(r1 + 4) : 0u;
        }
      } else {
        // query fragments of this head's group (rows beyond the group are zero)
        const T *qb = reinterpret_cast<const T *>(a.q) + (size_t)b * a.q_sn + (size_t)(h * group) * a.q_sh;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int col = ks * 16 + qlane * 2;
          const uint32_t *r0 = reinterpret_cast<const uint32_t *>(qb + (size_t)quad * a.q_sh + col);
          const uint32_t *r1 = reinterpret_cast<const uint32_t *>(qb + (size_t)(quad + 8) * a.q_sh + col);
          qa[ks][0] = quad < group ? __ldg(r0) : 0u;
          qa[ks][1] = quad + 8 < group ? __ldg(r1) : 0u;
          qa[ks][2] = quad < group ? __ldg(r0 + 4) : 0u;
          qa[ks][3] = quad + 8 < group ? __ldg(r1 + 4) : 0u;
        }
      }
      if (FUSED) {
        rope_pos = cur_hdr >= 0 ? *reinterpret_cast<const int *>(&sh_hdr[cur_hdr & 1][kHdrMetaOff]) : f.pos_ids[b];
        if (f.rope.mode == PIEKV_ROPE_TABLE && (rope_pos < 0 || rope_pos >= f.rope.table_len)) {
          if (lane == 0) report_error(a.err, PIEKV_ERR_TABLE_RANGE, KID_DECODE, b, rope_pos);
          rope_pos = 0;
        }
        // rotate the query fragments in registers (one rounding to T, as the in-place op does); the 64
        // (cos, sin) pairs of the position are evaluated once for the CTA, not once per warp and quad
        if (f.rope.mode != PIEKV_ROPE_NONE) {
          consumer_bar_sync();  // nobody still reads the previous run's pairs
          if (tid < kDim / 2) {
            float cc, ss;
            rope_cos_sin1(f.rope, rope_pos, tid, 64, cc, ss);
            sh_cs[tid] = make_float2(cc, ss);
          }
          consumer_bar_sync();
          if (!f.rope.interleave) {
            // element d pairs with d + 64: fragments ks and ks + 4 of the same thread
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
              for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int i0 = ks * 16 + hi8 * 8 + qlane * 2;
                const float2 cs0 = sh_cs[i0], cs1 = sh_cs[i0 + 1];
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                  const int j = hi8 * 2 + rr;
                  const float2 x = unpack2<T>(qa[ks][j]);
                  const float2 y = unpack2<T>(qa[ks + 4][j]);
                  float xa, ya, xb, yb;
                  rope_rotate(x.x, y.x, cs0.x, cs0.y, xa, ya);
                  rope_rotate(x.y, y.y, cs1.x, cs1.y, xb, yb);
                  qa[ks][j] = pack2<T>(xa, xb);
                  qa[ks + 4][j] = pack2<T>(ya, yb);
                }
              }
            }
          } else {
            // pairs (2i, 2i+1) sit in one register
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
              for (int hi8 = 0; hi8 < 2; ++hi8) {
                const int pair = (ks * 16 + hi8 * 8 + qlane * 2) >> 1;
                const float2 cs0 = sh_cs[pair];
#pragma unroll
                for (int rr = 0; rr < 2; ++rr) {
                  const int j = hi8 * 2 + rr;
                  const float2 x = unpack2<T>(qa[ks][j]);
                  float xa, ya;
                  rope_rotate(x.x, x.y, cs0.x, cs0.y, xa, ya);
                  qa[ks][j] = pack2<T>(xa, ya);
                }
              }
            }
          }
        }
      }
    }

    for (;;) {
    // ================= the stage's pages
    if (!mbar_wait(&full_bar[s], ph)) {
      if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, s);
      if (lane == 0) atomicExch(&sh_abort, 1);
      aborted = true;
      break;
    }
    if (pslot < npg) {
      if (g + pslot == req_end - 1 && (last_len < 1 || last_len > kPage)) {
        if (lane == 0) report_error(a.err, PIEKV_ERR_LAST_PAGE_LEN, KID_DECODE, b, last_len);
        last_len = last_len < 1 ? 1 : kPage;
      }
      const int valid = (g + pslot == req_end - 1) ? last_len : kPage;
      const int tok_lo = (g + pslot == req_begin) ? win_first : 0;  // window start inside the first page
      const uint32_t page_base = stage0 + s * kStageBytes + pslot * (HKV * kTileBytes);
      const uint32_t ktile = page_base + h * 4096;
      const uint32_t vtile = page_base + HKV * 4096 + h * 4096;
      if (FUSED && g + pslot == req_end - 1) {
        // This warp owns (last page, head h): rotate the new token's k, copy its v, store both
        // into the pool for later steps and patch them into the staged tile for this one.
        const int row = last_len - 1;
        const int last_phys = my_page;
        uint8_t *kp = stage0_ptr + s * kStageBytes + pslot * (HKV * kTileBytes) + h * 4096;
        uint8_t *vp = kp + HKV * 4096;
        const T *ksrc = cur_hdr >= 0 ? reinterpret_cast<const T *>(&sh_hdr[cur_hdr & 1][kHdrKOff]) + h * kDim
                                     : reinterpret_cast<const T *>(f.k_new) + (size_t)b * f.k_sn + (size_t)h * f.k_sh;
        const T *vsrc = cur_hdr >= 0 ? reinterpret_cast<const T *>(&sh_hdr[cur_hdr & 1][kHdrVOff]) + h * kDim
                                     : reinterpret_cast<const T *>(f.v_new) + (size_t)b * f.v_sn + (size_t)h * f.v_sh;
        const bool page_ok = last_phys >= 0 && last_phys < a.num_pages;
        T *pool = reinterpret_cast<T *>(const_cast<void *>(a.pool));
        T *kdst = pool + ((size_t)last_phys * 2 * kPage + row) * (HKV * kDim) + h * kDim;
        T *vdst = kdst + (size_t)kPage * HKV * kDim;
        // smem byte offset of element d of `row` inside a [2][16][64] swizzled tile
        auto tile_off = [&](int d) { return (d >> 6) * 2048 + row * 128 + ((((d & 63) >> 3) ^ (row & 7)) << 4) + (d & 7) * 2; };
        if (f.rope.mode == PIEKV_ROPE_NONE) {
          const int d = lane * 4;
          const uint2 kv = *reinterpret_cast<const uint2 *>(ksrc + d);
          *reinterpret_cast<uint2 *>(kp + tile_off(d)) = kv;
          if (page_ok) *reinterpret_cast<uint2 *>(kdst + d) = kv;
        } else if (!f.rope.interleave) {
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int i = lane + 32 * rr;
            float xo, yo;
            const float2 cs = sh_cs[i];
            rope_rotate(Elem<T>::to_f32(ksrc[i]), Elem<T>::to_f32(ksrc[i + 64]), cs.x, cs.y, xo, yo);
            const T xt = Elem<T>::from_f32(xo), yt = Elem<T>::from_f32(yo);
            *reinterpret_cast<T *>(kp + tile_off(i)) = xt;
            *reinterpret_cast<T *>(kp + tile_off(i + 64)) = yt;
            if (page_ok) {
              kdst[i] = xt;
              kdst[i + 64] = yt;
            }
          }
        } else {
#pragma unroll
          for (int rr = 0; rr < 2; ++rr) {
            const int i = lane + 32 * rr;  // pair (2i, 2i+1)
            float xo, yo;
            const float2 cs = sh_cs[i];
            rope_rotate(Elem<T>::to_f32(ksrc[2 * i]), Elem<T>::to_f32(ksrc[2 * i + 1]), cs.x, cs.y, xo, yo);
            const uint32_t pk = pack2<T>(xo, yo);
            *reinterpret_cast<uint32_t *>(kp + tile_off(2 * i)) = pk;
            if (page_ok) *reinterpret_cast<uint32_t *>(kdst + 2 * i) = pk;
          }
        }
        {
          const int d = lane * 4;
          const uint2 vv = *reinterpret_cast<const uint2 *>(vsrc + d);
          *reinterpret_cast<uint2 *>(vp + tile_off(d)) = vv;
          if (page_ok) *reinterpret_cast<uint2 *>(vdst + d) = vv;
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      if (valid < kPage) {
        // rows past the end of the context may hold anything: zero the V rows so that
        // 0 * garbage cannot produce NaN (their scores are masked to -inf below)
        uint8_t *vptr = stage0_ptr + s * kStageBytes + pslot * (HKV * kTileBytes) + HKV * 4096 + h * 4096;
        for (int x = lane; x < (kPage - valid) * 16; x += 32) {
          const int row = valid + (x >> 4);
          const int hf = (x >> 3) & 1;
          const int ch = x & 7;
          *reinterpret_cast<uint4 *>(vptr + hf * 2048 + row * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async_smem();
        __syncwarp();
      }
      // ---- S = Q K^T : 16 rows x 16 tokens
      float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      {
        const int mi = lane >> 3, r = lane & 7;
        const int t = (mi >> 1) * 8 + r;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const int hf = ks >> 2;
          const int ch = (ks & 3) * 2 + (mi & 1);
          uint32_t kb[4];
          ldmatrix_x4(kb, ktile + hf * 2048 + t * 128 + ((ch ^ r) << 4));
          mma_16816<T>(sc[0], qa[ks], kb[0], kb[1]);
          mma_16816<T>(sc[1], qa[ks], kb[2], kb[3]);
        }
      }
      // ---- online softmax (base 2); rows quad and quad+8, tokens nt*8 + qlane*2 + {0,1}
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int tok = nt * 8 + qlane * 2 + e;
          const bool okt = tok < valid && tok >= tok_lo;
          sc[nt][e] = okt ? sc[nt][e] * scale_log2 : -INFINITY;
          sc[nt][2 + e] = okt ? sc[nt][2 + e] * scale_log2 : -INFINITY;
          mx0 = fmaxf(mx0, sc[nt][e]);
          mx1 = fmaxf(mx1, sc[nt][2 + e]);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0;
      const float mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = fast_exp2(m0 - mu0), al1 = fast_exp2(m1 - mu1);
      m0 = mn0;
      m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          sc[nt][e] = fast_exp2(sc[nt][e] - mu0);
          sc[nt][2 + e] = fast_exp2(sc[nt][2 + e] - mu1);
          ps0 += sc[nt][e];
          ps1 += sc[nt][2 + e];
        }
      }
      l0 = l0 * al0 + ps0;
      l1 = l1 * al1 + ps1;
      if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          o[nt][0] *= al0;
          o[nt][1] *= al0;
          o[nt][2] *= al1;
          o[nt][3] *= al1;
        }
      }
      // ---- O += P V
      uint32_t pa[4];
      pa[0] = pack2<T>(sc[0][0], sc[0][1]);
      pa[1] = pack2<T>(sc[0][2], sc[0][3]);
      pa[2] = pack2<T>(sc[1][0], sc[1][1]);
      pa[3] = pack2<T>(sc[1][2], sc[1][3]);
      {
        const int mi = lane >> 3, r = lane & 7;
        const int t = (mi & 1) * 8 + r;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int hf = i >> 2;
          const int ch = (i & 3) * 2 + (mi >> 1);
          uint32_t vb[4];
          ldmatrix_x4_trans(vb, vtile + hf * 2048 + t * 128 + ((ch ^ r) << 4));
          mma_16816<T>(o[2 * i], pa, vb[0], vb[1]);
          mma_16816<T>(o[2 * i + 1], pa, vb[2], vb[3]);
        }
      }
    }
    __syncwarp();
    // (with several pages per stage the run's last stage is kept a little longer: its tiles carry the warps'
    // partial results to each other, below)
    if (lane == 0 && !(fold_on_chip && (flags & kRunEnd))) mbar_arrive(&empty_bar[s]);
    ++it;
    if (flags & kRunEnd) break;
    {
      const int r = fetch();
      if (r <= 0) {  // (a run always ends with a stage that says so; this is the way out after a fault)
        aborted = r < 0;
        finished = r == 0;
        break;
      }
    }
    }  // stages of the run
    if (aborted || finished) break;
    if (cur_hdr >= 0 && lane == 0) mbar_arrive(&hdr_empty[cur_hdr & 1]);  // the run's rows are no longer needed

    // ================= close the run: publish the result or the partial
    PIEKV_STAMP(2);
    const int c_first = req_begin / cp;
    const int c_last = (req_end - 1) / cp;
    const int nseg = c_last - c_first + 1;  // chunk pieces of the request
    float ls0 = l0, ls1 = l1;  // quad-reduce the running sums
    ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
    ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
    ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
    ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
    int slot = -1;  // the run's scratch slot, if it needs one
    if (fold_on_chip) {
      // ---- several pages per stage: the warps of a stage hold partials of the same heads.  Each writes its
      // rows (unnormalised accumulator, maximum, sum) over its own K / V tile of the run's last stage, which
      // nobody else reads; then all threads fold them, four consecutive d of one head at a time, into the
      // request's output rows or into ONE partial of the run.
      const bool whole = run_pieces == nseg;
      uint8_t *page0 = stage0_ptr + s * kStageBytes;  // page slot ps at + ps * HKV * kTileBytes: K tiles, then V tiles
      if (quad < group) {
        float2 *orow = reinterpret_cast<float2 *>(page0 + pslot * (HKV * kTileBytes) + h * 4096 + quad * 512);
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) orow[nt * 4 + qlane] = make_float2(o[nt][0], o[nt][1]);
        if (qlane == 0)
          reinterpret_cast<float2 *>(page0 + pslot * (HKV * kTileBytes) + HKV * 4096 + h * 4096)[quad] =
              make_float2(m0, ls0);
      }
      if (tid == 0) sh_slot = my_slot;
      consumer_bar_sync();
      slot = sh_slot;
      if (!whole && slot >= p.num_slots) {
        if (tid == 0) report_error(a.err, PIEKV_ERR_PAGE_CAPACITY, KID_DECODE, c, slot);
        if (tid == 0) atomicExch(&sh_abort, 1);
        aborted = true;
        break;
      }
      for (int e = tid * 4; e < a.hq * kDim; e += kConsumers * 4) {
        const int qh = e >> 7, d = e & (kDim - 1);
        const int hh = qh / group, row = qh - hh * group;
        float2 ml[PG];
        float M = -INFINITY;
#pragma unroll
        for (int ps = 0; ps < PG; ++ps) {
          ml[ps] = reinterpret_cast<const float2 *>(page0 + ps * (HKV * kTileBytes) + HKV * 4096 + hh * 4096)[row];
          if (ml[ps].y > 0.f) M = fmaxf(M, ml[ps].x);  // (a warp that saw no page contributes nothing)
        }
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int ps = 0; ps < PG; ++ps) {
          if (ml[ps].y > 0.f) {
            const float w = fast_exp2(ml[ps].x - M);
            const float4 v =
                *reinterpret_cast<const float4 *>(page0 + ps * (HKV * kTileBytes) + hh * 4096 + row * 512 + d * 4);
            L = fmaf(ml[ps].y, w, L);
            acc.x = fmaf(v.x, w, acc.x);
            acc.y = fmaf(v.y, w, acc.y);
            acc.z = fmaf(v.z, w, acc.z);
            acc.w = fmaf(v.w, w, acc.w);
          }
        }
        if (whole) {
          const float lsum = add_sink(L, M, a.sinks, qh);
          const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
          uint2 pk;
          pk.x = pack2<T>(acc.x * inv, acc.y * inv);
          pk.y = pack2<T>(acc.z * inv, acc.w * inv);
          for (int dd = 0; dd < n_dst; ++dd) *reinterpret_cast<uint2 *>(dst_row(dd, b, qh) + d) = pk;
          if (a.lse != nullptr && d == 0)
            a.lse[(size_t)b * a.hq + qh] = lsum > 0.f ? (M + log2f(lsum)) * 0.6931471805599453f : -INFINITY;
        } else {
          const size_t idx = (size_t)slot * a.hq + qh;  // one partial per slot
          *reinterpret_cast<float4 *>(p.part_o + idx * kDim + d) = acc;
          if (d == 0) p.part_ml[idx] = make_float2(M, L);
        }
      }
      fence_proxy_async_smem();  // these tiles are next written by bulk copies
      consumer_bar_sync();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
      if (whole) continue;
    } else if (PG == 1 && run_pieces == nseg) {
      // the whole request lived in this run: normalise and store
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = quad + half * 8;
        if (row < group) {
          const int qh = h * group + row;
          const float lsum = add_sink(half ? ls1 : ls0, half ? m1 : m0, a.sinks, qh);
          const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
          if (p.peer.n == 0) {  // the usual case keeps its own straight-line stores
            uint32_t *orow = reinterpret_cast<uint32_t *>(out + ((size_t)b * a.hq + qh) * kDim);
#pragma unroll
            for (int nt = 0; nt < 16; ++nt)
              orow[nt * 4 + qlane] = pack2<T>(o[nt][half * 2] * inv, o[nt][half * 2 + 1] * inv);
          } else {
            for (int d = 0; d < n_dst; ++d) {
              uint32_t *orow = reinterpret_cast<uint32_t *>(dst_row(d, b, qh));
#pragma unroll
              for (int nt = 0; nt < 16; ++nt)
                orow[nt * 4 + qlane] = pack2<T>(o[nt][half * 2] * inv, o[nt][half * 2 + 1] * inv);
            }
          }
          if (a.lse != nullptr && qlane == 0) {
            const float mm = half ? m1 : m0;
            a.lse[(size_t)b * a.hq + qh] = lsum > 0.f ? (mm + log2f(lsum)) * 0.6931471805599453f : -INFINITY;
          }
        }
      }
      continue;
    }
    if (!fold_on_chip) {
      // the run's scratch slot
      if (tid == 0) sh_slot = my_slot;
      consumer_bar_sync();
      slot = sh_slot;
      if (slot >= p.num_slots) {
        if (tid == 0) report_error(a.err, PIEKV_ERR_PAGE_CAPACITY, KID_DECODE, c, slot);
        if (tid == 0) atomicExch(&sh_abort, 1);
        aborted = true;
        break;
      }
      const size_t pidx = (size_t)slot * p.subs + pslot;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int row = quad + half * 8;
        if (row < group) {
          const int qh = h * group + row;
          float2 *orow = reinterpret_cast<float2 *>(p.part_o + (pidx * a.hq + qh) * kDim);
#pragma unroll
          for (int nt = 0; nt < 16; ++nt) orow[nt * 4 + qlane] = make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
          if (qlane == 0) p.part_ml[pidx * a.hq + qh] = make_float2(half ? m1 : m0, half ? ls1 : ls0);
        }
      }
    }
    const int tab_idx = run_first + b;  // unique per (chunk piece, request)
    if (nseg <= gsz) {
      PIEKV_STAMP(4);
      if (!arrive(&run_tab[tab_idx], slot, &req_cnt[b], run_pieces, nseg)) continue;
      PIEKV_STAMP(5);
      const int n = collect(run_tab, c_first + b, nseg);
      PIEKV_STAMP(6);
      merge_list(n, p.subs, b, -1);
      PIEKV_STAMP(7);
      continue;
    }
    // A request spread over many chunks (one long context): merging 100+ partials in a single CTA would sit
    // on the critical path of the whole launch.  Its chunk pieces are grouped gsz at a time (runs end at
    // group boundaries); whoever completes a group folds it into one partial (groups fold concurrently on
    // different SMs), and whoever completes the last group folds the groups.
    const int gi = (run_first - c_first) / gsz;
    const int g_first = c_first + gi * gsz;
    const int g_size = min(gsz, c_last + 1 - g_first);
    const int n_groups = (nseg + gsz - 1) / gsz;
    if (!arrive(&run_tab[tab_idx], slot, &grp_cnt[g_first + b], run_pieces, g_size)) continue;
    {
      const int n = collect(run_tab, g_first + b, g_size);
      merge_list(n, p.subs, b, slot);  // into sub-slot 0 of this run's own slot
    }
    if (!arrive(&grp_tab[g_first + b], slot, &req_cnt[b], 1, n_groups)) continue;
    {
      const int n = collect(grp_tab, c_first + b, nseg);
      merge_list(n, 1, b, -1);
    }
  }
  PIEKV_STAMP(3);
  if (aborted && tid == 0) steal_tab[c] = 0ull;  // nothing of an abandoned range may look stealable later
  finish();
}

template <typename T, int HKV, bool FUSED>
int launch_t(const CUtensorMap &tm, const DecodeParams &p, const FusedArgs &f, cudaStream_t st) {
  static unsigned char configured[kMaxDevices] = {0};  // per instantiation and device
  const int smem = kStages * kStageBytes + 1024;
  if (int rc = opt_in_dynamic_smem(decode_tma_kernel<T, HKV, FUSED>, smem, configured, "decode: cudaFuncSetAttribute"))
    return rc;
  if (p.pdl == 0) {
    decode_tma_kernel<T, HKV, FUSED><<<sm_count(), kThreads, smem, st>>>(tm, p, f);
    PIEKV_LAUNCH_CHECK("decode_tma_kernel");
    return 0;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sm_count());
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_tma_kernel<T, HKV, FUSED>, tm, p, f);
  if (e != cudaSuccess) return cuda_status(e, "decode_tma_kernel (programmatic dependent launch)");
  return 0;
}

template <typename T, bool FUSED>
int launch_h(const CUtensorMap &tm, const DecodeParams &p, const FusedArgs &f, cudaStream_t st) {
  switch (p.a.hkv) {
    case 1:
      return launch_t<T, 1, FUSED>(tm, p, f, st);
    case 2:
      return launch_t<T, 2, FUSED>(tm, p, f, st);
    case 4:
      return launch_t<T, 4, FUSED>(tm, p, f, st);
    case 8:
      return launch_t<T, 8, FUSED>(tm, p, f, st);
  }
  set_error("decode: unsupported num_kv_heads %d", p.a.hkv);
  return 1;
}

}  // namespace

bool decode_tma_supported(const AttnArgs &a, int dtype) {
  if (dtype != PIEKV_BF16 && dtype != PIEKV_F16) return false;
  if (a.dim != kDim || a.page_size != kPage) return false;
  if (!(a.hkv == 1 || a.hkv == 2 || a.hkv == 4 || a.hkv == 8)) return false;
  if (a.hq % a.hkv != 0 || a.hq / a.hkv > 16) return false;
  if (a.batch > kMaxBatch) return false;
  if ((reinterpret_cast<uintptr_t>(a.pool) & 15) || (reinterpret_cast<uintptr_t>(a.q) & 3) ||
      (reinterpret_cast<uintptr_t>(a.out) & 15))
    return false;
  if ((a.q_sn & 1) || (a.q_sh & 1)) return false;
  return true;
}

// Scratch slots (one per run that has to be merged): the least a launch can need when every CTA keeps to its
// own chunks - a run per CTA, per request boundary and per group boundary - and what lets idle CTAs take
// over other CTAs' chunks freely (every stolen interval is a run of its own).
static int64_t min_slots(int batch) { return 2ll * sm_count() + batch + 64; }
static int64_t full_slots(int batch) { return 6ll * sm_count() + 2ll * batch + 64; }
// Partials per scratch slot.  With several pages per stage (fewer than 8 kv heads) the warps of a stage each
// hold a partial of the same heads; they fold them through shared memory when a run ends (a GQA group of up to
// 8 rows fits a warp's own tile), otherwise every warp writes its own.
static int sub_slots(int hq, int hkv) {
  const int pg = (hkv == 1 || hkv == 2 || hkv == 4 || hkv == 8) ? 8 / hkv : 1;
  return (pg > 1 && hq / hkv <= 8) ? 1 : pg;
}
static int64_t slot_bytes(int hq, int hkv) { return (int64_t)sub_slots(hq, hkv) * hq * (kDim * 4 + 8); }
static int64_t window_meta_bytes(int batch) { return (((int64_t)batch + 1) * 12 + 255) / 256 * 256; }

int64_t decode_tma_workspace_bytes(int batch, int hq, int hkv) {
  return kCounterBytes + min_slots(batch) * slot_bytes(hq, hkv) + 512 + window_meta_bytes(batch);
}

static int prepare(const AttnArgs &a, int dtype, void *workspace, int64_t workspace_bytes, DecodeParams *p,
                   CUtensorMap *tm, cudaStream_t st) {
  const int pg = sub_slots(a.hq, a.hkv);
  const int64_t need = decode_tma_workspace_bytes(a.batch, a.hq, a.hkv);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= need, "decode: workspace too small (%lld < %lld bytes)",
                (long long)workspace_bytes, (long long)need);
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "decode: workspace must be 256-byte aligned");
  PIEKV_REQUIRE(sm_count() <= kMaxGrid, "decode: %d SMs, the steal table holds %d", sm_count(), kMaxGrid);
  // as many scratch slots as the workspace holds, up to what free stealing can use
  int64_t slots = (workspace_bytes - kCounterBytes - 512 - window_meta_bytes(a.batch)) / slot_bytes(a.hq, a.hkv);
  if (slots > full_slots(a.batch)) slots = full_slots(a.batch);
  if (slots > kMaxSlots) slots = kMaxSlots;
  p->a = a;
  p->peer = PeerOut{};
  p->pdl = get_option(PIEKV_OPT_PDL);
  p->steal = get_option(PIEKV_OPT_WORK_STEALING) ? 1 : 0;
  p->num_slots = (int)slots;
  p->subs = pg;
  uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
  p->counters = reinterpret_cast<int *>(ws);
  p->part_ml = reinterpret_cast<float2 *>(ws + kCounterBytes);
  const int64_t ml_bytes = ((slots * pg * a.hq * 8 + 255) / 256) * 256;
  p->part_o = reinterpret_cast<float *>(ws + kCounterBytes + ml_bytes);
  p->win_indptr = nullptr;
  p->win_meta = nullptr;
  if (a.window_left >= 0) {
    // windowed page ranges, computed on the device right before the launch (stream-ordered, no host work)
    const int64_t o_bytes = ((slots * pg * a.hq * kDim * 4 + 255) / 256) * 256;
    int32_t *wi = reinterpret_cast<int32_t *>(ws + kCounterBytes + ml_bytes + o_bytes);
    int2 *wm = reinterpret_cast<int2 *>(wi + ((a.batch + 1 + 1) & ~1));  // 8-byte aligned
    decode_window_kernel<<<1, 1024, 0, st>>>(a.kv_indptr, a.kv_last_page_len, a.batch, a.window_left, wi, wm);
    PIEKV_LAUNCH_CHECK("decode_window_kernel");
    p->win_indptr = wi;
    p->win_meta = wm;
    if (p->pdl > 1) p->pdl = 1;  // the offsets the kernel partitions by were written by the launch before it
  }
  return make_page_tensor_map(tm, a.pool, a.num_pages, a.hkv, dtype, /*box_halves=*/2, /*box_heads=*/a.hkv,
                              /*box_kv=*/2);
}

int launch_decode_tma(const AttnArgs &a, int dtype, void *workspace, int64_t workspace_bytes, cudaStream_t st) {
  if (a.batch == 0) return 0;
  DecodeParams p;
  CUtensorMap tm;
  if (int rc = prepare(a, dtype, workspace, workspace_bytes, &p, &tm, st)) return rc;
  FusedArgs f{};
  if (dtype == PIEKV_BF16) return launch_h<__nv_bfloat16, false>(tm, p, f, st);
  return launch_h<__half, false>(tm, p, f, st);
}

bool decode_fused_tma_supported(const AttnArgs &a, int dtype, const void *k, const void *v, int64_t k_sn,
                                int64_t k_sh, int64_t v_sn, int64_t v_sh) {
  if (!decode_tma_supported(a, dtype)) return false;
  if ((reinterpret_cast<uintptr_t>(k) & 7) || (reinterpret_cast<uintptr_t>(v) & 7)) return false;
  if ((k_sn & 3) || (k_sh & 3) || (v_sn & 3) || (v_sh & 3)) return false;
  return true;
}

int launch_decode_fused_tma(const AttnArgs &a, int dtype, const void *k, const void *v, int64_t k_sn, int64_t k_sh,
                            int64_t v_sn, int64_t v_sh, const int32_t *pos_ids, const RopeDev &rope, void *workspace,
                            int64_t workspace_bytes, cudaStream_t st, const PeerOut *peer) {
  if (a.batch == 0) return 0;
  DecodeParams p;
  CUtensorMap tm;
  if (int rc = prepare(a, dtype, workspace, workspace_bytes, &p, &tm, st)) return rc;
  if (peer != nullptr && peer->n > 0) {
    p.peer = *peer;
    p.peer.done = nullptr;  // completion is counted in the zero-state block
  }
  FusedArgs f;
  f.k_new = k;
  f.v_new = v;
  f.k_sn = k_sn;
  f.k_sh = k_sh;
  f.v_sn = v_sn;
  f.v_sh = v_sh;
  f.pos_ids = pos_ids;
  f.rope = rope;
  if (dtype == PIEKV_BF16) return launch_h<__nv_bfloat16, true>(tm, p, f, st);
  return launch_h<__half, true>(tm, p, f, st);
}

}  // namespace piekv

// =====================================================================================
// Decode attention without any allocation by the caller or by the library
// =====================================================================================
// Some hosts of this library cannot hand over a workspace: an inference runtime whose memory
// pool is fully committed to the KV cache at start-up (the reference sizes its pool from all free
// memory, pie/src/pie_worker/model/llama3.py:177-202), a plugin called from a stream callback or
// from inside a captured region where cudaMalloc is not allowed, or a foreign-language binding that
// only passes its own tensors through.  For those, the split-KV scratch of the tuned decode kernel
// lives in a fixed array inside the library image.  Every GPU that loads the library keeps these
// bytes until the process exits.
namespace piekv {
namespace {
constexpr int64_t kStaticScratchBytes = 8ll << 20;  // 8 MiB: counters + partial (max, sum, acc) triples
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

// The array's name is only a host-side handle; the device address is looked up once per device
// (with that device current) and cached.
int static_scratch_ptr(void **out) {
  static void *cached[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_status(e, "decode_run_noalloc: cudaGetDevice");
  PIEKV_REQUIRE(dev >= 0 && dev < 64, "decode_run_noalloc: device index %d out of range", dev);
  if (cached[dev] == nullptr) {
    void *ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_scratch);
    if (e != cudaSuccess) return cuda_status(e, "decode_run_noalloc: cudaGetSymbolAddress");
    PIEKV_REQUIRE(ptr != nullptr, "decode_run_noalloc: scratch symbol has no device address");
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return 0;
}
}  // namespace
}  // namespace piekv

#ifdef PIEKV_TRACE
extern "C" int piekv_trace_read(unsigned long long *host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, piekv::g_trace, sizeof(unsigned long long) * 256 * 16);
}
#endif

extern "C" int64_t piekv_decode_noalloc_max_bytes(void) { return piekv::kStaticScratchBytes; }

extern "C" int piekv_decode_run_noalloc(const void *q, int64_t q_stride_n, int64_t q_stride_h, const void *pool,
                                        void *out, float *lse, const int32_t *kv_indptr, const int32_t *kv_indices,
                                        const int32_t *kv_last_page_len, int32_t batch, int32_t num_qo_heads,
                                        int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                                        int32_t dtype, float sm_scale, int32_t *err, void *stream) {
  using namespace piekv;
  PIEKV_REQUIRE(dtype >= PIEKV_F32 && dtype <= PIEKV_BF16, "decode_run_noalloc: unknown dtype %d", dtype);
  PIEKV_REQUIRE(batch >= 0 && num_qo_heads > 0 && num_kv_heads > 0 && num_qo_heads % num_kv_heads == 0 &&
                    head_dim > 0 && page_size > 0 && num_pages > 0,
                "decode_run_noalloc: bad sizes");
  if (batch == 0) return 0;
  PIEKV_REQUIRE(q && pool && out && kv_indptr && kv_indices && kv_last_page_len, "decode_run_noalloc: null pointer");
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
  cudaStream_t st = (cudaStream_t)stream;
  // The size limit is checked before a kernel is chosen, so that which sizes are accepted does not depend
  // on the dtype or alignment of a call (the general kernel below happens to need no scratch).
  const int64_t need = decode_tma_workspace_bytes(batch, num_qo_heads, num_kv_heads);
  PIEKV_REQUIRE(need <= kStaticScratchBytes,
                "decode_run_noalloc: batch %d with %d query heads needs %lld bytes of scratch, the built-in "
                "scratch holds %lld; use piekv_decode_run with a caller workspace",
                batch, num_qo_heads, (long long)need, (long long)kStaticScratchBytes);
  if (!decode_tma_supported(a, dtype)) return launch_attn_generic(a, dtype, st);
  void *scratch = nullptr;
  if (int rc = static_scratch_ptr(&scratch)) return rc;
  // the zero-state block (counters, tables) must be zero when the kernel starts, whatever an earlier call
  // left behind
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)kCounterBytes, st);
  if (e != cudaSuccess) return cuda_status(e, "decode_run_noalloc: cudaMemsetAsync");
  return launch_decode_tma(a, dtype, scratch, kStaticScratchBytes, st);
}
