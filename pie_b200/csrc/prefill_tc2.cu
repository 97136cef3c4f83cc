// Prefill attention, two query heads per CTA, persistent CTAs (sm_100a tcgen05 / TMEM).
//
// A work item is one (request, 128-token query tile) for TWO query heads of the same GQA group,
// so both 128 x 128 problems share every K and V tile brought into shared memory: half the K/V
// fill and twice the tensor work per tile compared with one head per item.  The two heads
// ("A" and "B") overlap: while the softmax warps of one head work on its scores, the tensor pipe
// runs the other head's MMAs.
//
// One CTA per SM stays resident and takes items, heaviest first, from a device-side counter: TMEM
// and the barriers are set up once, and the streams of the roles run across item boundaries - the
// K / V rings keep filling with the next item's tiles, a head's query tile is replaced as soon as
// its last score MMA has run, and the first scores of the next item are issued in the slot where
// the current item would have issued its next tile, while the softmax warps write the finished
// item's output.
//
//   TMEM (512 columns): S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,384)  O_B [384,512)
//   smem: Q_A, Q_B (32 KiB each, a TMA box per head), K ring (3 x 32 KiB), V ring (2 x 32 KiB)
//
// P never goes through shared memory: a softmax thread owns a whole row (one TMEM lane), reads the
// row's 128 scores, and writes the probabilities back over the same columns as packed 16-bit pairs
// (64 columns); O += P V then takes its A operand from TMEM.  S is therefore single-buffered per
// head.  One thread issues every MMA, in the order
//     S_A(0) S_B(0)   then per kv tile t:   O_A(t) S_A(next)   O_B(t) S_B(next)
// where "next" is tile t + 1 of the item or tile 0 of the following item.  The tensor pipe executes
// MMAs in issue order, hence S_x(next) follows O_x(t), which consumed P_x(t) in the same columns, and
// O_x is stable whenever S_x has been committed.  O_x of the following item is first written after the
// softmax warps of head x have delivered that item's first probabilities, i.e. after they have read
// the finished item's O_x.
//
// What bounds the kernel: a 128 x 128 tile needs 16384 exponentials, and the SM's special-function
// units deliver 16 per clock, i.e. 1024 clocks - as long as the tile's two MMAs (2 x 512 clocks at
// 8192 flop/clk).  Measured on B200, one softmax pass of a tile takes ~1.8k clocks when it has the
// SM to itself, the MMAs run at 64 clocks each once queued, and the pipe accepts only about two
// MMAs ahead of the running one, so every wait of the issuing thread shows as idle tensor time.
//
// Roles (384 threads, three warpgroups): warps 0-3 softmax of head A (thread = row), warps 4-7
// softmax of head B, warp 8 TMA producer of K tiles, warp 9 MMA issuer and TMEM owner, warp 10
// scheduler (claims items and publishes their description in a small shared-memory ring that every
// role reads on entering an item) and producer of the query tiles, warp 11 TMA producer of V tiles.
// The third warpgroup gives registers to the softmax warps (setmaxnreg).  Masking, the device-built work list, the
// packed custom mask and the bounded waits are those of the one-head kernel (prefill_tc.cu).
#include <type_traits>

#include "prefill_common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace piekv {

using namespace prefill;

namespace {

constexpr int k2SmemBytes = kTileBytes * (2 + kKStages + kVStages) + 1024;
// Three warpgroups: two of softmax warps and one holding the producer, MMA and scheduler warps (its
// fourth warp idles).  The third gives most of its registers to the softmax warps, which keep a whole
// row of 128 scores in registers.
constexpr int k2Threads = 384;
constexpr int k2RegsLaunch = 168;  // what __launch_bounds__(384, 1) gives every thread at launch
constexpr int k2RegsSoftmax = 200, k2RegsOther = 96;
// setmaxnreg.inc waits until the registers exist: the CTA owns 384 * 168 and not one more
static_assert(256 * k2RegsSoftmax + 128 * k2RegsOther <= k2Threads * k2RegsLaunch, "registers the CTA owns");
static_assert(k2RegsSoftmax % 8 == 0 && k2RegsOther % 8 == 0, "setmaxnreg takes multiples of 8");
constexpr int k2ColS = 0;    // + 128 * head
constexpr int k2ColO = 256;  // + 128 * head
constexpr int kSchedWarp = kMmaWarp + 1, kVWarp = kMmaWarp + 2;
constexpr int kItemSlots = 4;  // how many items the scheduler may describe ahead of the slowest reader
// every reader copies an item's description once: 8 softmax warps, the MMA thread, the K, V and query-tile cursors
constexpr int kItemReaders = kSoftmaxWarps + 1 + 3;

// One work item as the scheduler warp publishes it.
struct Item {
  int valid;         // 0: the list is exhausted
  int b, r0, rows;   // request, first row of the query tile within it, rows that exist
  int h0, hk;        // first of the two query heads, their kv head
  int q_row;         // first row of the tile in the packed query tensor
  int p0, np;        // the request's slice of the page list
  int kv_len, qo_len;
  int n_tiles;       // kv tiles a row of this query tile can see (causal bound applied)
  int n_active;      // of those, tiles with at least one allowed pair (all of them without a mask)
  int groups;        // 128-bit groups per row of the packed mask
  int srow;          // row of the (query tile, kv tile) summary
  int pad;
  long long poff;    // the request's first 128-bit group in the packed mask
};

// not volatile: the scheduler may interleave these with the surrounding arithmetic
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
// A poll that never suspends the warp (the producer has other barriers to look at), made uniform: the
// lanes of a warp may see a phase complete at different moments, and a phase that one lane saw complete
// is complete.
__device__ __forceinline__ bool warp_poll(uint64_t *bar, uint32_t parity) {
  return __any_sync(0xffffffffu, mbar_test_wait(bar, parity));
}

// The MMA batches.  Inlined on purpose: the issuing thread's own instructions sit on the critical path
// between one softmax pass of a head and the next, and a call per batch measured 10 % slower.
// S = Q K^T: eight K = 16 steps over the two 64-element halves of head_dim, then the commit that wakes
// the softmax warps of the head.
__device__ __forceinline__ void issue_scores(uint32_t d_tmem, uint64_t q_desc, uint64_t k_desc, uint32_t idesc,
                                             uint64_t *s_full_bar) {
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const uint64_t off = (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
    tc::mma_ss(d_tmem, q_desc + off, k_desc + off, idesc, ks > 0 ? 1u : 0u);
  }
  tc::commit(s_full_bar);
}
// O (+)= P V for 64 kv tokens (four K = 16 steps); P is read from TMEM, two 16-bit values per column
__device__ __forceinline__ void issue_pv_half(uint32_t d_tmem, uint32_t p_tmem, uint64_t v_desc, uint32_t idesc,
                                              uint32_t accumulate_first) {
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    tc::mma_ts(d_tmem, p_tmem + ks * 8, v_desc + (uint64_t)((ks * 2048) >> 4), idesc, (accumulate_first || ks > 0) ? 1u : 0u);
}

template <typename T>
__global__ void __launch_bounds__(k2Threads, 1)
    prefill_tc2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                       const __grid_constant__ PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full[2], q_empty[2], k_full[kKStages], k_empty[kKStages], v_full[kVStages],
      v_empty[kVStages], v_land, s_full[2], p_full[2][2], o_done[2], item_full[kItemSlots], item_empty[kItemSlots];
  __shared__ __align__(16) Item sh_item[kItemSlots];
  __shared__ uint32_t tmem_slot;
  __shared__ int sh_abort;

  const AttnArgs &a = p.a;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const bool has_mask = p.has_mask != 0;
  T *out = reinterpret_cast<T *>(a.out);

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;                                    // head A at +0, head B at +32K
  const uint32_t k_smem0 = base + 2 * kTileBytes;                  // K stage s at + s * 32K
  const uint32_t v_smem0 = base + (2 + kKStages) * kTileBytes;     // V stage s at + s * 32K

  if (threadIdx.x == 0) {
    mbar_init(&v_land, 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&q_full[x], 1);
      mbar_init(&q_empty[x], 1);
      mbar_init(&s_full[x], 1);
      mbar_init(&p_full[x][0], 4);  // one arrival per softmax warp
      mbar_init(&p_full[x][1], 4);
      mbar_init(&o_done[x], 1);
    }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(&item_full[s], 1);
      mbar_init(&item_empty[s], kItemReaders);
    }
    sh_abort = 0;
    mbar_fence_init();
  }
  if (warp == kMmaWarp) {
    tc::tmem_alloc(&tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int *abort_flag = &sh_abort;
  constexpr bool kBf16 = !std::is_same<T, __half>::value;

  // kv tile j of the query tile whose summary row is `srow` has at least one allowed pair
  auto tile_active = [&](const uint32_t *srow, int j) {
    return !has_mask || ((__ldg(srow + (j >> 5)) >> (j & 31)) & 1u) != 0;
  };
  auto give_up = [&](int where) {
    if (lane == 0 && !*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, where);
    if (lane == 0) atomicExch(&sh_abort, 1);
  };

  if (warp >= kSoftmaxWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(k2RegsOther));
  if (warp == kSchedWarp) {
    // ================================================================== scheduler and query tiles
    // Claims the next item of the list (heaviest first) and describes it for the other roles; also
    // replaces a head's query tile as soon as the current item's last S of that head has run.  Neither
    // is urgent (descriptions run up to four items ahead, a query tile is needed a tile period after it
    // can be requested), so this warp polls and sleeps instead of occupying issue slots.
    const int pairs = a.hq >> 1;
    const int group = a.hq / a.hkv;
    const int total = *p.ntiles * pairs;
    int n = 0, sched_done = 0;                                              // scheduler
    int qn = 0, q_loaded = 0, q_done = 0, q_x = 0, q_row = 0, q_h0 = 0, q_cnt = 0;  // query-tile cursor
    uint64_t idle_since = 0;
    while (!(sched_done && q_done)) {
      bool progressed = false;
      if (!sched_done && warp_poll(&item_empty[n % kItemSlots], ((n / kItemSlots) & 1) ^ 1)) {
        const int slot = n % kItemSlots;
        int idx = 0;
        if (lane == 0) idx = atomicAdd(p.claim, 1);
        idx = __shfl_sync(0xffffffffu, idx, 0);
        Item it;
        it.valid = idx < total ? 1 : 0;
        if (it.valid) {
          const int tile = idx / pairs;
          it.h0 = (idx % pairs) * 2;  // heads h0 and h0 + 1 share a kv head (even GQA group)
          it.hk = it.h0 / group;
          const int2 tr = p.tiles[tile];
          it.b = tr.x;
          it.r0 = tr.y;
          const int q0 = a.qo_indptr[it.b];
          it.qo_len = a.qo_indptr[it.b + 1] - q0;
          it.q_row = q0 + it.r0;
          it.p0 = a.kv_indptr[it.b];
          it.np = a.kv_indptr[it.b + 1] - it.p0;
          int last_len = it.np > 0 ? a.kv_last_page_len[it.b] : 0;
          if (it.np > 0 && (last_len < 1 || last_len > kPage)) {
            if (lane == 0) report_error(a.err, PIEKV_ERR_LAST_PAGE_LEN, KID_PREFILL, it.b, last_len);
            last_len = last_len < 1 ? 1 : kPage;
          }
          it.kv_len = it.np > 0 ? (it.np - 1) * kPage + last_len : 0;
          it.rows = min(kBM, it.qo_len - it.r0);
          const int kv_hi = (a.causal && !has_mask) ? min(it.kv_len, it.kv_len - it.qo_len + it.r0 + kBM) : it.kv_len;
          it.n_tiles = kv_hi > 0 ? (kv_hi + kBN - 1) / kBN : 0;
          it.groups = (it.kv_len + kBN - 1) / kBN;
          it.srow = has_mask ? p.tile_base[it.b] + it.r0 / kBM : 0;
          it.poff = has_mask ? p.poff[it.b] : 0;
          it.pad = 0;
          it.n_active = it.n_tiles;
          if (has_mask) {
            const uint32_t *srow = p.summary + (size_t)it.srow * p.sw;
            int cnt = 0;
            for (int w = lane; w < (it.n_tiles + 31) / 32; w += 32) cnt += __popc(__ldg(srow + w));
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, d);
            it.n_active = cnt;
          }
        }
        if (lane == 0) {
          if (it.valid) sh_item[slot] = it;
          else sh_item[slot].valid = 0;
          mbar_arrive(&item_full[slot]);  // release: the description is visible to whoever sees the phase
        }
        __syncwarp();
        if (it.valid) ++n;
        else sched_done = 1;
        progressed = true;
      }
      if (!q_done) {
        if (!q_loaded) {
          const int slot = qn % kItemSlots;
          if (warp_poll(&item_full[slot], (qn / kItemSlots) & 1)) {
            const int valid = sh_item[slot].valid, act = sh_item[slot].n_active;
            q_row = sh_item[slot].q_row;
            q_h0 = sh_item[slot].h0;
            __syncwarp();
            if (lane == 0) mbar_arrive(&item_empty[slot]);
            progressed = true;
            if (!valid) {
              q_done = 1;
            } else if (act == 0) {
              ++qn;
            } else {
              q_loaded = 1;
              q_x = 0;
            }
          }
        } else if (warp_poll(&q_empty[q_x], (q_cnt & 1) ^ 1)) {
          if (lane == 0) {
            mbar_arrive_expect_tx(&q_full[q_x], kTileBytes);
            tma_load_4d(q_smem + q_x * kTileBytes, &tmap_q, 0, q_row, 0, q_h0 + q_x, &q_full[q_x]);
          }
          progressed = true;
          if (++q_x == 2) {
            q_loaded = 0;
            ++q_cnt;
            ++qn;
          }
        }
      }
      if (progressed) {
        idle_since = 0;
      } else {
        __nanosleep(200);
        if (*abort_flag) break;
        const uint64_t now = global_timer_ns();
        if (idle_since == 0) idle_since = now;
        if (now - idle_since > 2000000000ull) {
          give_up(400);
          break;
        }
      }
    }
    // The last scheduler to run out of items puts the counters back to zero for the next launch: every
    // CTA has made its final claim by then.
    if (sched_done && lane == 0 && atomicAdd(p.claim + 1, 1) == (int)gridDim.x - 1) {
      p.claim[0] = 0;
      p.claim[1] = 0;
    }
    // drain: the CTA must not retire while a bulk copy may still be landing
    if (lane == 0) {
      const int q_issued = q_cnt * 2 + (q_loaded ? q_x : 0);  // head A loads: ceil, head B loads: floor
      if (q_issued > 0) mbar_wait(&q_full[0], (((q_issued + 1) / 2) - 1) & 1, 200000000ull);
      if (q_issued > 1) mbar_wait(&q_full[1], ((q_issued / 2) - 1) & 1, 200000000ull);
    }
  } else if (warp == kProducerWarp || warp == kVWarp) {
    // ================================================================== TMA producers: K tiles / V tiles
    // Two warps walk the same item sequence, one filling the K ring, the other the V ring; each blocks on
    // its own ring only.
    const bool is_v = warp == kVWarp;
    const uint32_t ring0 = is_v ? v_smem0 : k_smem0;
    const int stages = is_v ? kVStages : kKStages;
    uint64_t *full = is_v ? v_full : k_full, *empty = is_v ? v_empty : k_empty;
    int armed = 0, lands = 0;  // tiles issued so far (all items), uses of v_land
    bool ok = true;
    for (int n = 0; ok; ++n) {
      const int slot = n % kItemSlots;
      if (!wait_or_abort(&item_full[slot], (n / kItemSlots) & 1, abort_flag)) {
        give_up(is_v ? 120 : 100);
        break;
      }
      const int valid = sh_item[slot].valid, left0 = sh_item[slot].n_active;
      const int p0 = sh_item[slot].p0, np = sh_item[slot].np, hk = sh_item[slot].hk, kv_len = sh_item[slot].kv_len;
      const uint32_t *srow = p.summary + (size_t)sh_item[slot].srow * p.sw;
      __syncwarp();
      if (lane == 0) mbar_arrive(&item_empty[slot]);
      if (!valid) break;
      int j = 0;
      for (int left = left0; left > 0; --left) {
        const int st = armed % stages;
        if (!wait_or_abort(&empty[st], ((armed / stages) & 1) ^ 1, abort_flag)) {
          give_up(is_v ? 121 : 101);
          ok = false;
          break;
        }
        while (!tile_active(srow, j)) ++j;
        const int pi = j * 8 + lane;
        int page = (lane < 8 && pi < np) ? __ldg(a.kv_indices + p0 + pi) : a.num_pages;
        if (lane < 8 && pi < np && (page < 0 || page >= a.num_pages)) {
          report_error(a.err, PIEKV_ERR_PAGE_ID, KID_PREFILL, p0 + pi, page);
          page = a.num_pages;  // outside the tensor map: zero fill
        }  // pages beyond the request's list are out of range too: their rows are zero-filled
        // The V tile that holds a partly filled last page lands on a barrier of its own, has its stale
        // rows zeroed, and only then is handed to the MMA warp (at most once per item).
        const bool partial = is_v && (kv_len & (kPage - 1)) != 0 && j == (kv_len - 1) / kBN;
        uint64_t *land = partial ? &v_land : &full[st];
        if (lane == 0) mbar_arrive_expect_tx(land, kTileBytes);
        __syncwarp();
        if (lane < 8) {
          const uint32_t dst = ring0 + st * kTileBytes + lane * 2048;
          tma_load_5d(dst, &tmap_kv, 0, 0, 0, hk, page * 2 + (is_v ? 1 : 0), land);
          tma_load_5d(dst + kHalfBytes, &tmap_kv, 0, 0, 1, hk, page * 2 + (is_v ? 1 : 0), land);
        }
        ++armed;
        if (partial) {
          if (!wait_or_abort(&v_land, lands & 1, abort_flag)) {
            give_up(110);
            ok = false;
            break;
          }
          ++lands;
          const int first = kv_len - j * kBN;
          zero_v_rows(ring0 + st * kTileBytes, first, min(kBN, (first + kPage - 1) / kPage * kPage), lane);
          fence_proxy_async_smem();  // generic-proxy stores before the tensor core's reads
          __syncwarp();
          if (lane == 0) mbar_arrive(&full[st]);
        }
        ++j;
      }
    }
    // drain: the CTA must not retire while a bulk copy may still be landing
    __syncwarp();
    if (lane == 0)
      for (int x = armed > stages ? armed - stages : 0; x < armed; ++x)
        mbar_wait(&full[x % stages], (x / stages) & 1, 200000000ull);
  } else if (warp == kMmaWarp) {
    // ================================================================== MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::instr_desc(kBf16, false, false, kBM, kBN);
      constexpr uint32_t idesc_pv = tc::instr_desc(kBf16, false, true, kBM, kDim);
      // Descriptors are built once; per MMA only the 14-bit start-address field (bytes >> 4) moves, by
      // amounts known at compile time.
      const uint64_t q_desc[2] = {tc::desc_k_major(q_smem), tc::desc_k_major(q_smem + kTileBytes)};
      const uint64_t k_desc0 = tc::desc_k_major(k_smem0);
      const uint64_t v_desc0 = tc::desc_mn_major(v_smem0, kHalfBytes);
      int kt = 0, vt = 0;  // K / V tiles consumed so far (all items): ring positions and phases
      int qi = 0;          // items (with work) started so far: phase of the query barriers
      // S_x = Q_x K^T into the head's score columns; the K tile is number `kt` of the stream
      auto issue_qk = [&](int x) {
        issue_scores(tmem + k2ColS + x * 128, q_desc[x], k_desc0 + (uint64_t)(((kt % kKStages) * kTileBytes) >> 4),
                     idesc_qk, &s_full[x]);
      };
      // O_x (+)= P_x V for V tile number `vt` of the stream; P_x is read from TMEM (two 16-bit values per
      // column) and arrives in two halves of 64 kv tokens
      auto issue_pv = [&](int x, bool accumulate) -> bool {
        const uint64_t vd = v_desc0 + (uint64_t)(((vt % kVStages) * kTileBytes) >> 4);
        const uint32_t d = tmem + k2ColO + x * 128;
        const uint32_t pa = tmem + k2ColS + x * 128;
        if (!wait_or_abort(&p_full[x][0], vt & 1, abort_flag)) return false;
        tc::fence_after_sync();
        issue_pv_half(d, pa, vd, idesc_pv, accumulate ? 1u : 0u);
        if (!wait_or_abort(&p_full[x][1], vt & 1, abort_flag)) return false;
        tc::fence_after_sync();
        issue_pv_half(d, pa + 32, vd + (uint64_t)((4 * 2048) >> 4), idesc_pv, 1u);
        return true;
      };
      // the next item of the sequence that has work (n_active > 0); -1 when the list is exhausted, -2 on failure
      int n = 0;
      auto next_item = [&]() -> int {
        for (;;) {
          const int slot = n % kItemSlots;
          if (!wait_or_abort(&item_full[slot], (n / kItemSlots) & 1, abort_flag)) return -2;
          const int valid = sh_item[slot].valid, act = sh_item[slot].n_active;
          mbar_arrive(&item_empty[slot]);
          ++n;
          if (!valid) return -1;
          if (act > 0) return act;
        }
      };
      // first scores of an item whose query tiles are phase `qi` and whose first K tile is number `kt`
      // (head x); `tiles` is the item's tile count: with a single tile the query tile is free again at once
      auto first_scores = [&](int x, int tiles) -> bool {
        if (!wait_or_abort(&q_full[x], qi & 1, abort_flag)) return false;
        if (x == 0 && !wait_or_abort(&k_full[kt % kKStages], (kt / kKStages) & 1, abort_flag)) return false;
        tc::fence_after_sync();
        issue_qk(x);
        if (tiles == 1) tc::commit(&q_empty[x]);
        return true;
      };
      // Issue order: S_A(0) S_B(0), then per tile t:  O_A(t) S_A(next)  O_B(t) S_B(next), where next is
      // tile t + 1 or the first tile of the following item.  A head's next scores follow its O += P V
      // immediately, so the time from the end of one softmax to the start of the next is one and a half
      // MMA batches; the softmax of a 128 x 128 tile (bound by the 16 exp/clk of the SM) takes about
      // twice as long as the two MMAs, so that turnaround, not tensor time, is what the order has to
      // keep short.
      int tiles = next_item();
      bool ok = tiles != -2;
      if (ok && tiles > 0) {
        ok = first_scores(0, tiles) && first_scores(1, tiles);
        if (ok) {
          tc::commit(&k_empty[kt % kKStages]);
          ++kt;
        }
      }
      while (ok && tiles > 0) {
        int following = 0;  // tile count of the following item, fetched when this item's last tile comes up
        for (int t = 0; ok && t < tiles; ++t) {
          const bool last = t + 1 == tiles;
          if (last) {
            following = next_item();
            if (following == -2) {
              ok = false;
              break;
            }
          }
          ok = wait_or_abort(&v_full[vt % kVStages], (vt / kVStages) & 1, abort_flag) && issue_pv(0, t > 0);
          if (!ok) break;
          if (!last) {
            ok = wait_or_abort(&k_full[kt % kKStages], (kt / kKStages) & 1, abort_flag);
            if (!ok) break;
            tc::fence_after_sync();
            issue_qk(0);
            if (t + 2 == tiles) tc::commit(&q_empty[0]);  // that was head A's last use of its query tile
          } else {
            tc::commit(&o_done[0]);  // all of head A's MMAs of this item
            if (following > 0) {
              ++qi;
              ok = first_scores(0, following);
              if (!ok) break;
            }
          }
          ok = issue_pv(1, t > 0);
          if (!ok) break;
          tc::commit(&v_empty[vt % kVStages]);  // both heads are done with this V tile
          ++vt;
          if (!last) {
            issue_qk(1);
            tc::commit(&k_empty[kt % kKStages]);  // and with this K tile
            ++kt;
            if (t + 2 == tiles) tc::commit(&q_empty[1]);
          } else {
            tc::commit(&o_done[1]);
            if (following > 0) {
              ok = first_scores(1, following);
              if (!ok) break;
              tc::commit(&k_empty[kt % kKStages]);
              ++kt;
            }
          }
        }
        tiles = following;
      }
      if (!ok) give_up(200);
    }
  }
  } else {
    // ================================================ softmax of head x (thread = row = TMEM lane)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(k2RegsSoftmax));
    const int x = warp >> 2;   // 0: head A, 1: head B
    const int q4 = warp & 3;   // TMEM lane quarter of this warp
    const int row = q4 * 32 + lane;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const uint32_t s_addr = tmem + lane_base + k2ColS + x * 128;  // scores in, packed probabilities out
    const uint32_t o_addr = tmem + lane_base + k2ColO + x * 128;
    const float c = a.sm_scale * 1.4426950408889634f;
    int sc = 0;  // score tiles of this head consumed so far (all items): phase of s_full
    int oc = 0;  // items (with work) finished so far: phase of o_done
    bool ok = true;

    for (int n = 0; ok; ++n) {
      const int slot = n % kItemSlots;
      if (!wait_or_abort(&item_full[slot], (n / kItemSlots) & 1, abort_flag)) {
        ok = false;
        break;
      }
      const Item it = sh_item[slot];
      __syncwarp();
      if (lane == 0) mbar_arrive(&item_empty[slot]);
      if (!it.valid) break;
      const int head = it.h0 + x;
      const bool row_valid = row < it.rows;
      T *orow = out + ((size_t)(it.q_row + row) * a.hq + head) * kDim;
      if (it.n_active == 0) {  // nothing to attend to: zeros
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < kDim / 8; ++i) reinterpret_cast<uint4 *>(orow)[i] = make_uint4(0, 0, 0, 0);
          if (a.lse != nullptr) a.lse[(size_t)(it.q_row + row) * a.hq + head] = -INFINITY;
        }
        continue;
      }
      const int kv_len = it.kv_len;
      const int limit =
          row_valid ? ((a.causal && !has_mask) ? min(kv_len - 1, kv_len - it.qo_len + it.r0 + row) : kv_len - 1) : -1;
      const uint32_t *srow = p.summary + (size_t)it.srow * p.sw;
      const uint4 *mrow = has_mask ? p.packed + it.poff + (long long)(it.r0 + (row_valid ? row : 0)) * it.groups : nullptr;
      const int n_tiles = it.n_tiles;
      float m_ref = -INFINITY, l = 0.f;
      int done = 0;  // tiles of this item consumed

      for (int j = 0; j < n_tiles; ++j) {
        if (!tile_active(srow, j)) continue;
        uint4 mw = make_uint4(0, 0, 0, 0);
        if (has_mask && row_valid) mw = __ldg(mrow + j);  // in flight while we wait for S
        ok = wait_or_abort(&s_full[x], sc & 1, abort_flag);
        if (!ok) break;
        ++sc;
        tc::fence_after_sync();
        const int t0 = j * kBN;
        const bool full_tile = has_mask ? (mw.x & mw.y & mw.z & mw.w) == 0xffffffffu : t0 + kBN - 1 <= limit;

        // ---- pass 1: running maximum, 64 columns at a time (rolled: the unrolled body of a whole row is
        // ~10 KB of code per softmax warp, which evicts the MMA thread's code from the instruction cache)
        float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t sr[64];
          tc::tmem_ld32(s_addr + h * 64, sr);
          tc::tmem_ld32(s_addr + h * 64 + 32, sr + 32);
          tc::tmem_wait_ld();
          if (!full_tile) {
            const uint32_t w0 = h ? mw.z : mw.x, w1 = h ? mw.w : mw.y;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const bool allow = has_mask ? (((i < 32 ? w0 : w1) >> (i & 31)) & 1u) != 0 : t0 + h * 64 + i <= limit;
              sr[i] = allow ? sr[i] : 0xff800000u;
            }
          }
#pragma unroll
          for (int i = 0; i < 32; ++i)
            mxa[i & 3] = max3(mxa[i & 3], __uint_as_float(sr[2 * i]), __uint_as_float(sr[2 * i + 1]));
        }
        float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * c;  // c > 0
        float alpha = 1.f;
        bool rescale = false;
        if (mx > m_ref + 8.f) {
          alpha = exp2_approx(m_ref - mx);  // m_ref = -inf on the first hit: 0
          l *= alpha;
          m_ref = mx;
          rescale = done > 0;
        }
        // O_x is stable here: S_x of this tile was committed after O_x of the previous one in issue order
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int ch = 0; ch < 4; ++ch) {
            uint32_t oreg[32];
            tc::tmem_ld32(o_addr + ch * 32, oreg);
            tc::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
            tc::tmem_st32(o_addr + ch * 32, oreg);
          }
        }
        // ---- pass 2: probabilities, packed two per column, written back over the row's first 64 score
        // columns; the MMA warp is released after each half (64 kv tokens) so that O += P V starts while
        // the second half is still being exponentiated.  Half h reads score columns [64h, 64h + 64) and
        // writes packed columns [32h, 32h + 32), which only cover scores already consumed.
        const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
        float suma[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          uint32_t sr[64];
          uint32_t pk[32];
          tc::tmem_ld32(s_addr + h * 64, sr);
          tc::tmem_ld32(s_addr + h * 64 + 32, sr + 32);
          tc::tmem_wait_ld();
          if (!full_tile) {
            const uint32_t w0 = h ? mw.z : mw.x, w1 = h ? mw.w : mw.y;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
              const bool allow = has_mask ? (((i < 32 ? w0 : w1) >> (i & 31)) & 1u) != 0 : t0 + h * 64 + i <= limit;
              sr[i] = allow ? sr[i] : 0xff800000u;
            }
          }
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float p0v = exp2_approx(fmaf(__uint_as_float(sr[2 * i]), c, neg_m));
            const float p1v = exp2_approx(fmaf(__uint_as_float(sr[2 * i + 1]), c, neg_m));
            suma[i & 3] += p0v + p1v;
            pk[i] = pack2<T>(p0v, p1v);  // tokens 64h + 2i (low half) and + 2i + 1 (high half)
          }
          tc::tmem_st16(s_addr + h * 32, pk);
          tc::tmem_st16(s_addr + h * 32 + 16, pk + 16);
          tc::tmem_wait_st();
          tc::fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&p_full[x][h]);
        }
        l += (suma[0] + suma[1]) + (suma[2] + suma[3]);
        ++done;
      }

      // ---- epilogue: O_x / l -> out, head h0 + x.  The next item's O_x is not written before this warp
      // has delivered that item's first probabilities, so the accumulator is ours until then.
      if (ok) ok = wait_or_abort(&o_done[x], oc & 1, abort_flag);  // committed once per item, after the last tile
      if (!ok) break;
      ++oc;
      tc::fence_after_sync();
      l = add_sink(l, m_ref, a.sinks, head);
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        uint32_t oreg[32];
        tc::tmem_ld32(o_addr + ch * 32, oreg);
        tc::tmem_wait_ld();
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2<T>(__uint_as_float(oreg[i * 8 + 0]) * inv, __uint_as_float(oreg[i * 8 + 1]) * inv);
            v.y = pack2<T>(__uint_as_float(oreg[i * 8 + 2]) * inv, __uint_as_float(oreg[i * 8 + 3]) * inv);
            v.z = pack2<T>(__uint_as_float(oreg[i * 8 + 4]) * inv, __uint_as_float(oreg[i * 8 + 5]) * inv);
            v.w = pack2<T>(__uint_as_float(oreg[i * 8 + 6]) * inv, __uint_as_float(oreg[i * 8 + 7]) * inv);
            *reinterpret_cast<uint4 *>(orow + ch * 32 + i * 8) = v;
          }
        }
      }
      if (a.lse != nullptr && row_valid)
        a.lse[(size_t)(it.q_row + row) * a.hq + head] =
            l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
    if (!ok) give_up(300 + warp);
  }

  // ---- teardown: every thread arrives here on every path
  tc::fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

template <typename T>
int launch_t(const AttnArgs &a, const CUtensorMap &tq, const CUtensorMap &tkv, const PrefillParams &p, int max_tiles,
             cudaStream_t st) {
  static unsigned char configured[kMaxDevices] = {0};
  if (int rc = opt_in_dynamic_smem(prefill_tc2_kernel<T>, k2SmemBytes, configured,
                                   "prefill (two heads): cudaFuncSetAttribute"))
    return rc;
  const long long items = (long long)max_tiles * (a.hq / 2);
  PIEKV_REQUIRE(items < (1ll << 31), "prefill: too many tiles");
  const int sms = sm_count();
  PIEKV_REQUIRE(sms > 0, "prefill: cannot read the multiprocessor count");
  const unsigned grid = (unsigned)(items < sms ? items : sms);
  prefill_tc2_kernel<T><<<grid, k2Threads, k2SmemBytes, st>>>(tq, tkv, p);
  PIEKV_LAUNCH_CHECK("prefill_tc2_kernel");
  return 0;
}

}  // namespace

// heads are processed in pairs that must share a kv head
bool prefill_tc2_supported(const AttnArgs &a) { return a.hq % a.hkv == 0 && ((a.hq / a.hkv) % 2) == 0; }

int launch_prefill_tc2(const AttnArgs &a, int dtype, const PrefillParams &p, int max_tiles, cudaStream_t st) {
  CUtensorMap tq, tkv;
  if (int rc = make_q_tensor_map(&tq, a.q, a.nnz, a.hq, a.q_sn, a.q_sh, dtype, kBM, 1)) return rc;
  if (int rc = make_page_tensor_map(&tkv, a.pool, a.num_pages, a.hkv, dtype, 1, 1, 1)) return rc;
  if (dtype == PIEKV_BF16) return launch_t<__nv_bfloat16>(a, tq, tkv, p, max_tiles, st);
  return launch_t<__half>(a, tq, tkv, p, max_tiles, st);
}

}  // namespace piekv
