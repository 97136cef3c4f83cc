// Prefill attention, two query tiles per CTA (sm_100a tcgen05 / TMEM).
//
// A CTA works on one (request, 128-token query tile) for TWO query heads of the same GQA group,
// so both 128 x 128 problems share every K and V tile brought into shared memory: half the K/V
// fill and twice the tensor work per tile compared with one head per CTA.  The two heads
// ("A" and "B") overlap: while the softmax warps of one head work on its scores, the tensor pipe
// runs the other head's MMAs.
//
//   TMEM (512 columns): S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,384)  O_B [384,512)
//   smem: Q_A, Q_B (64 KiB, one TMA box), K ring (3 x 32 KiB), V ring (2 x 32 KiB)
//
// P never goes through shared memory: a softmax thread owns a whole row (one TMEM lane), reads the
// row's 128 scores, and writes the probabilities back over the same columns as packed 16-bit pairs
// (64 columns); O += P V then takes its A operand from TMEM.  S is therefore single-buffered per
// head.  One thread issues every MMA, in the order
//     S_A(0) S_B(0)   then per kv tile t:   O_A(t) S_A(t+1)   O_B(t) S_B(t+1)
// The tensor pipe executes MMAs in issue order, hence S_x(t+1) follows O_x(t), which consumed P_x(t)
// in the same columns, and O_x is stable whenever S_x has been committed.
//
// What bounds the kernel: a 128 x 128 tile needs 16384 exponentials, and the SM's special-function
// units deliver 16 per clock, i.e. 1024 clocks - as long as the tile's two MMAs (2 x 512 clocks at
// 8192 flop/clk).  Measured on B200, one softmax pass of a tile takes ~1.8k clocks when it has the
// SM to itself, the MMAs run at 64 clocks each once queued, and the pipe accepts only about two
// MMAs ahead of the running one, so every wait of the issuing thread shows as idle tensor time.
//
// Roles (384 threads, three warpgroups): warps 0-3 softmax of head A (thread = row), warps 4-7
// softmax of head B, warp 8 TMA producer, warp 9 MMA issuer and TMEM owner, warps 10-11 idle.  The
// third warpgroup gives registers to the softmax warps (setmaxnreg).  Masking, the device-built work
// list, the packed custom mask and the bounded waits are those of the one-head kernel
// (prefill_tc.cu).
#include <type_traits>

#include "prefill_common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace piekv {

using namespace prefill;

namespace {

constexpr int k2SmemBytes = kTileBytes * (2 + kKStages + kVStages) + 1024;
// Three warpgroups: two of softmax warps and one holding the producer and MMA warps (its other two
// warps idle).  The third gives most of its registers to the softmax warps, which keep a whole row
// of 128 scores in registers.
constexpr int k2Threads = 384;
constexpr int k2RegsLaunch = 168;  // what __launch_bounds__(384, 1) gives every thread at launch
constexpr int k2RegsSoftmax = 200, k2RegsOther = 96;
// setmaxnreg.inc waits until the registers exist: the CTA owns 384 * 168 and not one more
static_assert(256 * k2RegsSoftmax + 128 * k2RegsOther <= k2Threads * k2RegsLaunch, "register budget of the CTA");
static_assert(k2RegsSoftmax % 8 == 0 && k2RegsOther % 8 == 0, "setmaxnreg takes multiples of 8");
constexpr int k2ColS = 0;    // + 128 * head
constexpr int k2ColO = 256;  // + 128 * head

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

template <typename T>
__global__ void __launch_bounds__(k2Threads, 1)
    prefill_tc2_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                       const __grid_constant__ PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages], v_land,
      s_full[2], p_full[2][2], o_done[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int sh_abort;

  const AttnArgs &a = p.a;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work item: (q tile, pair of heads) -------------------------------------------------------
  const int pairs = a.hq >> 1;
  const int tile = blockIdx.x / pairs;
  const int h0 = (blockIdx.x % pairs) * 2;  // heads h0 and h0 + 1 share a kv head (even GQA group)
  if (tile >= *p.ntiles) return;
  const int2 item = p.tiles[tile];
  const int b = item.x, r0 = item.y;
  const int group = a.hq / a.hkv;
  const int hk = h0 / group;
  const int q0 = a.qo_indptr[b];
  const int qo_len = a.qo_indptr[b + 1] - q0;
  const int p0 = a.kv_indptr[b];
  const int np = a.kv_indptr[b + 1] - p0;
  int last_len = np > 0 ? a.kv_last_page_len[b] : 0;
  if (np > 0 && (last_len < 1 || last_len > kPage)) {
    if (threadIdx.x == 0) report_error(a.err, PIEKV_ERR_LAST_PAGE_LEN, KID_PREFILL, b, last_len);
    last_len = last_len < 1 ? 1 : kPage;
  }
  const int kv_len = np > 0 ? (np - 1) * kPage + last_len : 0;
  const int rows = min(kBM, qo_len - r0);
  const bool has_mask = p.has_mask != 0;
  const int kv_hi = (a.causal && !has_mask) ? min(kv_len, kv_len - qo_len + r0 + kBM) : kv_len;
  const int n_tiles = kv_hi > 0 ? (kv_hi + kBN - 1) / kBN : 0;
  const int groups = (kv_len + kBN - 1) / kBN;
  const uint32_t *srow = has_mask ? p.summary + (size_t)(p.tile_base[b] + r0 / kBM) * p.sw : nullptr;
  auto active = [&](int j) { return !has_mask || ((__ldg(srow + (j >> 5)) >> (j & 31)) & 1u) != 0; };
  int n_active = n_tiles;
  if (has_mask) {
    n_active = 0;
    for (int w = 0; w < (n_tiles + 31) / 32; ++w) n_active += __popc(__ldg(srow + w));
  }
  T *out = reinterpret_cast<T *>(a.out);

  if (n_active == 0) {  // nothing to attend to: zeros for both heads
    for (int x = threadIdx.x; x < rows * (2 * kDim / 8); x += k2Threads) {
      const int r = x / (2 * kDim / 8), c8 = x % (2 * kDim / 8);
      *reinterpret_cast<uint4 *>(out + ((size_t)(q0 + r0 + r) * a.hq + h0) * kDim + c8 * 8) = make_uint4(0, 0, 0, 0);
    }
    if (a.lse != nullptr)
      for (int x = threadIdx.x; x < rows * 2; x += k2Threads)
        a.lse[(size_t)(q0 + r0 + (x >> 1)) * a.hq + h0 + (x & 1)] = -INFINITY;
    return;
  }

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = base;                                    // head A at +0, head B at +32K
  const uint32_t k_smem0 = base + 2 * kTileBytes;                  // K stage s at + s * 32K
  const uint32_t v_smem0 = base + (2 + kKStages) * kTileBytes;     // V stage s at + s * 32K

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
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
      mbar_init(&s_full[x], 1);
      mbar_init(&p_full[x][0], 4);  // one arrival per softmax warp
      mbar_init(&p_full[x][1], 4);
      mbar_init(&o_done[x], 1);
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

  if (warp >= kSoftmaxWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(k2RegsOther));
  if (warp > kMmaWarp) {
    // idle warps of the third warpgroup
  } else if (warp == kProducerWarp) {
    // ================================================================== TMA producer
    int k_armed = 0, v_armed = 0;  // K / V tiles issued so far
    int jk = 0, jv = 0;            // next kv tile index to consider for K / for V
    if (lane == 0) {
      mbar_arrive_expect_tx(&q_full, 2 * kTileBytes);
      tma_load_4d(q_smem, &tmap_q, 0, q0 + r0, 0, h0, &q_full);  // box of two heads: A then B
    }
    auto page_of = [&](int j) {
      const int pi = j * 8 + lane;
      int page = (lane < 8 && pi < np) ? __ldg(a.kv_indices + p0 + pi) : a.num_pages;
      if (lane < 8 && pi < np && (page < 0 || page >= a.num_pages)) {
        report_error(a.err, PIEKV_ERR_PAGE_ID, KID_PREFILL, p0 + pi, page);
        page = a.num_pages;  // outside the tensor map: zero fill
      }
      return page;  // pages beyond the request's list are out of range too: their rows are zero-filled
    };
    uint64_t idle_since = 0;
    while (k_armed < n_active || v_armed < n_active) {
      bool progressed = false;
      if (k_armed < n_active) {
        const int ks = k_armed % kKStages;
        if (mbar_try_wait(&k_empty[ks], ((k_armed / kKStages) & 1) ^ 1)) {
          while (!active(jk)) ++jk;
          const int page = page_of(jk);
          if (lane == 0) mbar_arrive_expect_tx(&k_full[ks], kTileBytes);
          __syncwarp();
          if (lane < 8) {
            const uint32_t kdst = k_smem0 + ks * kTileBytes + lane * 2048;
            tma_load_5d(kdst, &tmap_kv, 0, 0, 0, hk, page * 2, &k_full[ks]);
            tma_load_5d(kdst + kHalfBytes, &tmap_kv, 0, 0, 1, hk, page * 2, &k_full[ks]);
          }
          ++jk;
          ++k_armed;
          progressed = true;
        }
      }
      if (v_armed < n_active && v_armed < k_armed) {
        const int vs = v_armed % kVStages;
        if (mbar_try_wait(&v_empty[vs], ((v_armed / kVStages) & 1) ^ 1)) {
          while (!active(jv)) ++jv;
          const int page = page_of(jv);
          // The tile that holds a partly filled last page lands on a barrier of its own, has its stale
          // rows zeroed, and only then is handed to the MMA warp (at most once per CTA).
          const bool partial = (kv_len & (kPage - 1)) != 0 && jv == (kv_len - 1) / kBN;
          uint64_t *land = partial ? &v_land : &v_full[vs];
          if (lane == 0) mbar_arrive_expect_tx(land, kTileBytes);
          __syncwarp();
          if (lane < 8) {
            const uint32_t vdst = v_smem0 + vs * kTileBytes + lane * 2048;
            tma_load_5d(vdst, &tmap_kv, 0, 0, 0, hk, page * 2 + 1, land);
            tma_load_5d(vdst + kHalfBytes, &tmap_kv, 0, 0, 1, hk, page * 2 + 1, land);
          }
          if (partial) {
            if (!wait_or_abort(&v_land, 0, abort_flag)) {
              if (lane == 0 && !*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 110);
              if (lane == 0) atomicExch(&sh_abort, 1);
              break;
            }
            const int first = kv_len - jv * kBN;
            zero_v_rows(v_smem0 + vs * kTileBytes, first, min(kBN, (first + kPage - 1) / kPage * kPage), lane);
            fence_proxy_async_smem();  // generic-proxy stores before the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&v_full[vs]);
          }
          ++jv;
          ++v_armed;
          progressed = true;
        }
      }
      if (progressed) {
        idle_since = 0;
      } else {
        if (*abort_flag) break;
        const uint64_t now = global_timer_ns();
        if (idle_since == 0) idle_since = now;
        if (now - idle_since > 2000000000ull) {
          if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 100);
          if (lane == 0) atomicExch(&sh_abort, 1);
          break;
        }
      }
    }
    // drain: the CTA must not retire while a bulk copy may still be landing
    __syncwarp();
    if (lane == 0) {
      mbar_wait(&q_full, 0, 200000000ull);
      for (int x = k_armed > kKStages ? k_armed - kKStages : 0; x < k_armed; ++x)
        mbar_wait(&k_full[x % kKStages], (x / kKStages) & 1, 200000000ull);
      for (int x = v_armed > kVStages ? v_armed - kVStages : 0; x < v_armed; ++x)
        mbar_wait(&v_full[x % kVStages], (x / kVStages) & 1, 200000000ull);
    }
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
      // S_x = Q_x K^T into the head's score columns; K tile number t has landed
      auto issue_qk = [&](int x, int t) {
        const uint64_t kd = k_desc0 + (uint64_t)(((t % kKStages) * kTileBytes) >> 4);
        const uint64_t qd = q_desc[x];
        const uint32_t d = tmem + k2ColS + x * 128;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t off = (uint64_t)(((ks >> 2) * kHalfBytes + (ks & 3) * 32) >> 4);
          tc::mma_ss(d, qd + off, kd + off, idesc_qk, ks > 0 ? 1u : 0u);
        }
        tc::commit(&s_full[x]);
      };
      // O_x += P_x V for tile number t (V tile t has landed); P_x is read from TMEM (two 16-bit values
      // per column) and arrives in two halves of 64 kv tokens
      auto issue_pv = [&](int x, int t) -> bool {
        const uint64_t vd = v_desc0 + (uint64_t)(((t % kVStages) * kTileBytes) >> 4);
        const uint32_t d = tmem + k2ColO + x * 128;
        const uint32_t pa = tmem + k2ColS + x * 128;
        if (!wait_or_abort(&p_full[x][0], t & 1, abort_flag)) return false;
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          tc::mma_ts(d, pa + ks * 8, vd + (uint64_t)((ks * 2048) >> 4), idesc_pv, (t > 0 || ks > 0) ? 1u : 0u);
        if (!wait_or_abort(&p_full[x][1], t & 1, abort_flag)) return false;
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 4; ks < 8; ++ks)
          tc::mma_ts(d, pa + ks * 8, vd + (uint64_t)((ks * 2048) >> 4), idesc_pv, 1u);
        return true;
      };
      // Issue order: S_A(0) S_B(0), then per tile t:  O_A(t) S_A(t+1)  O_B(t) S_B(t+1).
      // A head's next scores follow its O += P V immediately, so the time from the end of one softmax
      // to the start of the next is one and a half MMA batches; the softmax of a 128 x 128 tile (bound
      // by the 16 exp/clk of the SM) takes about twice as long as the two MMAs, so that turnaround, not
      // tensor time, is what the order has to keep short.  The pipe executes in issue order, hence
      // S_x(t+1) follows O_x(t), which consumed P_x(t) in the same columns, and O_x is stable whenever
      // S_x has been committed.
      bool ok = wait_or_abort(&q_full, 0, abort_flag) && wait_or_abort(&k_full[0], 0, abort_flag);
      if (ok) {
        issue_qk(0, 0);
        issue_qk(1, 0);
        tc::commit(&k_empty[0]);
      }
      for (int t = 0; ok && t < n_active; ++t) {
        const bool more = t + 1 < n_active;
        ok = wait_or_abort(&v_full[t % kVStages], (t / kVStages) & 1, abort_flag) && issue_pv(0, t);
        if (!ok) break;
        if (more) {
          ok = wait_or_abort(&k_full[(t + 1) % kKStages], ((t + 1) / kKStages) & 1, abort_flag);
          if (!ok) break;
          issue_qk(0, t + 1);
        } else {
          tc::commit(&o_done[0]);  // all of head A's MMAs
        }
        ok = issue_pv(1, t);
        if (!ok) break;
        tc::commit(&v_empty[t % kVStages]);  // both heads are done with V tile t
        if (more) {
          issue_qk(1, t + 1);
          tc::commit(&k_empty[(t + 1) % kKStages]);  // and with K tile t + 1
        } else {
          tc::commit(&o_done[1]);
        }
      }
      if (!ok) {
        if (!*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 200);
        atomicExch(&sh_abort, 1);
      }
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
    const bool row_valid = row < rows;
    const int limit = row_valid ? ((a.causal && !has_mask) ? min(kv_len - 1, kv_len - qo_len + r0 + row) : kv_len - 1) : -1;
    const uint4 *mrow = has_mask ? p.packed + p.poff[b] + (long long)(r0 + (row_valid ? row : 0)) * groups : nullptr;
    const float c = a.sm_scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    int it = 0;

    for (int j = 0; j < n_tiles; ++j) {
      if (!active(j)) continue;
      uint4 mw = make_uint4(0, 0, 0, 0);
      if (has_mask && row_valid) mw = __ldg(mrow + j);  // in flight while we wait for S
      ok = wait_or_abort(&s_full[x], it & 1, abort_flag);
      if (!ok) break;
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
        rescale = it > 0;
      }
      // O_x is stable here: S_x(it) was committed after O_x(it-1) in the pipe's issue order
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
      ++it;
    }

    // ---- epilogue: O_x / l -> out, head h0 + x
    if (ok) ok = wait_or_abort(&o_done[x], 0, abort_flag);  // committed once, after the last tile
    if (ok) {
      tc::fence_after_sync();
      l = add_sink(l, m_ref, a.sinks, h0 + x);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T *orow = out + ((size_t)(q0 + r0 + row) * a.hq + h0 + x) * kDim;
#pragma unroll
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
        a.lse[(size_t)(q0 + r0 + row) * a.hq + h0 + x] = l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    } else {
      if (lane == 0 && !*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 300 + warp);
      if (lane == 0) atomicExch(&sh_abort, 1);
    }
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
  const long long blocks = (long long)max_tiles * (a.hq / 2);
  PIEKV_REQUIRE(blocks < (1ll << 31), "prefill: too many tiles");
  prefill_tc2_kernel<T><<<(unsigned)blocks, k2Threads, k2SmemBytes, st>>>(tq, tkv, p);
  PIEKV_LAUNCH_CHECK("prefill_tc2_kernel");
  return 0;
}

}  // namespace

// heads are processed in pairs that must share a kv head
bool prefill_tc2_supported(const AttnArgs &a) { return a.hq % a.hkv == 0 && ((a.hq / a.hkv) % 2) == 0; }

int launch_prefill_tc2(const AttnArgs &a, int dtype, const PrefillParams &p, int max_tiles, cudaStream_t st) {
  CUtensorMap tq, tkv;
  if (int rc = make_q_tensor_map(&tq, a.q, a.nnz, a.hq, a.q_sn, a.q_sh, dtype, kBM, 2)) return rc;
  if (int rc = make_page_tensor_map(&tkv, a.pool, a.num_pages, a.hkv, dtype, 1, 1, 1)) return rc;
  if (dtype == PIEKV_BF16) return launch_t<__nv_bfloat16>(a, tq, tkv, p, max_tiles, st);
  return launch_t<__half>(a, tq, tkv, p, max_tiles, st);
}

}  // namespace piekv
