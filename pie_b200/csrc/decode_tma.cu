// Paged decode attention for 16-bit K/V, head_dim 128, page_size 16 on sm_100a.
//
// Work partition (on the device, no host plan): the flat list of all requests' pages
// (kv_indices[0 .. kv_indptr[B])) is cut into gridDim.x equal contiguous ranges, one per
// CTA (one CTA per SM).  A CTA therefore streams the same number of pages whatever the
// mix of context lengths; where a range crosses a request boundary the CTA closes one
// "segment" and opens the next.  A request cut across CTAs is finished by whichever CTA
// delivers its last segment (per-request arrival counter), which merges the partial
// (max, sum, accumulator) triples from scratch memory.
//
// Data path: a producer warp gathers pages with TMA.  A page holds K [16, Hkv, 128] then
// V [16, Hkv, 128]; one 5-D tensor-map box {64 d, 16 tokens, 2 d-halves, Hkv heads, K|V}
// moves the whole page (Hkv * 8 KiB) and lands it in shared memory regrouped per head as
// 128-byte-swizzled [token][64 d] tiles, which is the layout ldmatrix wants.  A stage is
// always 64 KiB = 8 (page, head) tiles: 8/Hkv pages for Hkv heads.  Three stages keep
// 128-192 KiB per SM in flight.
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
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr int kStages = 3;
constexpr int kTileBytes = 8192;               // one (page, head): K 4 KiB + V 4 KiB
constexpr int kStageBytes = 8 * kTileBytes;    // 64 KiB
constexpr int kCounterBytes = 65536;           // head of the workspace: arrival counters
constexpr int kMergeGroup = 16;                // partials folded by one CTA at a time
constexpr int kGroupCounters = 256;            // group counters, indexed by the group's first CTA (grid <= 256)
constexpr int kMaxBatch = kCounterBytes / 4 - kGroupCounters - 1;  // request counters; then the group counters; then one word
constexpr int kGroupCounter0 = kMaxBatch;

struct DecodeParams {
  AttnArgs a;
  float *part_o;    // [slot][PG][Hq][128]
  float2 *part_ml;  // [slot][PG][Hq]  (running max in log2 domain, running sum)
  int *counters;    // [batch], zero between launches
  int pdl;          // programmatic dependent launch: 0 off, 1 wait first, 2 wait after the page-table offsets
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
__device__ unsigned long long g_trace[256 * 4];
#define PIEKV_STAMP(slot)                                                               \
  do {                                                                                  \
    if ((threadIdx.x & 31) == 0 && (threadIdx.x >> 5) == 0) g_trace[blockIdx.x * 4 + (slot)] = global_timer_ns(); \
  } while (0)
#else
#define PIEKV_STAMP(slot) \
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

__device__ __forceinline__ void consumer_bar_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32)); }

// CTA that owns flat page g when T pages are cut into G ranges [c*T/G, (c+1)*T/G).
__device__ __forceinline__ int cta_of_page(long long g, long long T, long long G) {
  return (int)(((g + 1) * G - 1) / T);
}

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

template <typename T, int HKV, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1)
    decode_tma_kernel(const __grid_constant__ CUtensorMap tmap, const __grid_constant__ DecodeParams p,
                      const __grid_constant__ FusedArgs f) {
  constexpr int PG = 8 / HKV;  // pages per stage
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ int sh_abort;
  __shared__ int sh_last;
  __shared__ int32_t sh_indptr[kSmemBatch + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *stage0_ptr = smem_raw + (stage0 - smem_u32(smem_raw));

  const AttnArgs &a = p.a;
  const int B = a.batch;
  const int c = blockIdx.x;
  PIEKV_STAMP(0);
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
    }
    sh_abort = 0;
    sh_last = 0;
    mbar_fence_init();
  }
  __syncthreads();
  if (p.pdl == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
  const int total_pages = ip[B];
  // With fewer pages than CTAs only the first `total_pages` CTAs take part, so that every
  // participating range is non-empty (the segment count of a request relies on that).
  const int G = min((int)gridDim.x, max(total_pages, 1));
  const int lo = c < G ? (int)((long long)c * total_pages / G) : 0;
  const int hi = c < G ? (int)((long long)(c + 1) * total_pages / G) : 0;
  const int group = a.hq / HKV;

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------------ producer
    int armed = 0;  // stages armed so far
    if (lo < hi) {
      int b = request_of_page(ip, B, lo);
      int g = lo;
      bool stop = false;
      while (g < hi && !stop) {
        while (b < B - 1 && ip[b + 1] <= g) ++b;
        const int seg_end = min(hi, ip[b + 1]);
        if (seg_end <= g) {  // non-monotone indptr: give up cleanly
          if (lane == 0) report_error(a.err, PIEKV_ERR_INDPTR, KID_DECODE, b, g);
          if (lane == 0) atomicExch(&sh_abort, 1);
          break;
        }
        const int shift = windowed ? __ldg(&p.win_meta[b].x) : 0;
        while (g < seg_end) {
          const int npg = min(PG, seg_end - g);
          // page ids first, so the load is in flight while we wait for the stage
          int page = lane < npg ? __ldg(a.kv_indices + g + shift + lane) : 0;
          const int s = armed % kStages;
          const uint32_t ph = (armed / kStages) & 1;
          if (*(volatile int *)&sh_abort) {
            stop = true;
            break;
          }
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, 100 + s);
            if (lane == 0) atomicExch(&sh_abort, 1);
            stop = true;
            break;
          }
          if (lane < npg && (page < 0 || page >= a.num_pages)) {
            report_error(a.err, PIEKV_ERR_PAGE_ID, KID_DECODE, g + lane, page);
            page = a.num_pages;  // outside the tensor map: the box is zero-filled
          }
          if (lane == 0) mbar_arrive_expect_tx(&full_bar[s], (uint32_t)(npg * HKV * kTileBytes));
          __syncwarp();
          if (lane < npg) {
            tma_load_page(stage0 + s * kStageBytes + lane * (HKV * kTileBytes), &tmap, page * 2, &full_bar[s]);
          }
          g += npg;
          ++armed;
        }
      }
    }
    // Drain: do not let the CTA retire while a bulk copy may still be landing.
    __syncwarp();
    if (lane == 0) {
      const int first = armed > kStages ? armed - kStages : 0;
      for (int it = first; it < armed; ++it) {
        mbar_wait(&full_bar[it % kStages], (it / kStages) & 1, 200000000ull);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumers
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
  // Every CTA passes here exactly once after its last result store.  The CTA that arrives last
  // publishes this step's number in every GPU's flag array: all stores of this launch, fenced at
  // system scope by their threads, are ordered before it.
  auto finish = [&]() {
    if (p.peer.n == 0) return;
    __threadfence_system();
    consumer_bar_sync();
    if (tid == 0) {
      __threadfence_system();
      const int old = atomicAdd(p.peer.done, 1);
      if (old == (int)gridDim.x - 1) {
        atomicExch(p.peer.done, 0);  // ready for the next launch
        __threadfence_system();
        for (int d = 0; d < p.peer.n; ++d)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.peer.flag[d]), "r"(peer_step) : "memory");
      }
    }
  };

  // requests without any page: softmax over nothing -> zeros
  for (int b = c; b < B; b += gridDim.x) {
    if (ip[b + 1] == ip[b]) {
      for (int d = 0; d < n_dst; ++d) {
        T *row = dst_row(d, b, 0);
        for (int x = tid; x < a.hq * kDim; x += kConsumerWarps * 32) row[x] = Elem<T>::from_f32(0.f);
      }
      if (a.lse != nullptr)
        for (int x = tid; x < a.hq; x += kConsumerWarps * 32) a.lse[(size_t)b * a.hq + x] = -INFINITY;
    }
  }
  if (lo >= hi) {
    finish();
    return;
  }

  uint32_t qa[8][4];
  float o[16][4];
  int b = request_of_page(ip, B, lo);
  int g = lo;
  int it = 0;
  bool aborted = false;

  while (g < hi) {
    // ================= open the segment of request b that starts at flat page g
    while (b < B - 1 && ip[b + 1] <= g) ++b;
    const int req_begin = ip[b];
    const int req_end = ip[b + 1];
    const int seg_end = min(hi, req_end);
    if (seg_end <= g) break;  // non-monotone indptr (the producer reports it)
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
    {
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
    int last_len = a.kv_last_page_len[b];
    if (last_len < 1 || last_len > kPage) {
      if (lane == 0) report_error(a.err, PIEKV_ERR_LAST_PAGE_LEN, KID_DECODE, b, last_len);
      last_len = last_len < 1 ? 1 : kPage;
    }
    int shift = 0, win_first = 0;
    if (windowed) {
      const int2 wm = __ldg(p.win_meta + b);
      shift = wm.x;
      win_first = wm.y;
    }
    int rope_pos = 0;
    int last_phys = -1;  // physical id of the request's last page when this segment contains it
    if (FUSED) {
      rope_pos = f.pos_ids[b];
      if (f.rope.mode == PIEKV_ROPE_TABLE && (rope_pos < 0 || rope_pos >= f.rope.table_len)) {
        if (lane == 0) report_error(a.err, PIEKV_ERR_TABLE_RANGE, KID_DECODE, b, rope_pos);
        rope_pos = 0;
      }
      if (seg_end == req_end) last_phys = __ldg(a.kv_indices + req_end - 1 + shift);
      // rotate the query fragments in registers (one rounding to T, as the in-place op does)
      if (f.rope.mode != PIEKV_ROPE_NONE) {
        if (!f.rope.interleave) {
          // element d pairs with d + 64: fragments ks and ks + 4 of the same thread
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
            for (int hi8 = 0; hi8 < 2; ++hi8) {
              const int i0 = ks * 16 + hi8 * 8 + qlane * 2;
              float c0, s0, c1, s1;
              rope_cos_sin1(f.rope, rope_pos, i0, 64, c0, s0);
              rope_cos_sin1(f.rope, rope_pos, i0 + 1, 64, c1, s1);
#pragma unroll
              for (int rr = 0; rr < 2; ++rr) {
                const int j = hi8 * 2 + rr;
                const float2 x = unpack2<T>(qa[ks][j]);
                const float2 y = unpack2<T>(qa[ks + 4][j]);
                float xa, ya, xb, yb;
                rope_rotate(x.x, y.x, c0, s0, xa, ya);
                rope_rotate(x.y, y.y, c1, s1, xb, yb);
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
              float c0, s0;
              rope_cos_sin1(f.rope, rope_pos, pair, 64, c0, s0);
#pragma unroll
              for (int rr = 0; rr < 2; ++rr) {
                const int j = hi8 * 2 + rr;
                const float2 x = unpack2<T>(qa[ks][j]);
                float xa, ya;
                rope_rotate(x.x, x.y, c0, s0, xa, ya);
                qa[ks][j] = pack2<T>(xa, ya);
              }
            }
          }
        }
      }
    }

    // ================= stream the segment's pages
    while (g < seg_end) {
      const int npg = min(PG, seg_end - g);
      const int s = it % kStages;
      const uint32_t ph = (it / kStages) & 1;
      if (!aborted && *(volatile int *)&sh_abort) aborted = true;
      if (!aborted && !mbar_wait(&full_bar[s], ph)) {
        if (lane == 0) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_DECODE, c, s);
        if (lane == 0) atomicExch(&sh_abort, 1);
        aborted = true;
      }
      if (it == 0) PIEKV_STAMP(1);
      if (!aborted && pslot < npg) {
        const int valid = (g + pslot == req_end - 1) ? last_len : kPage;
        const int tok_lo = (g + pslot == req_begin) ? win_first : 0;  // window start inside the first page
        const uint32_t page_base = stage0 + s * kStageBytes + pslot * (HKV * kTileBytes);
        const uint32_t ktile = page_base + h * 4096;
        const uint32_t vtile = page_base + HKV * 4096 + h * 4096;
        if (FUSED && g + pslot == req_end - 1) {
          // This warp owns (last page, head h): rotate the new token's k, copy its v, store both
          // into the pool for later steps and patch them into the staged tile for this one.
          const int row = last_len - 1;
          uint8_t *kp = stage0_ptr + s * kStageBytes + pslot * (HKV * kTileBytes) + h * 4096;
          uint8_t *vp = kp + HKV * 4096;
          const T *ksrc = reinterpret_cast<const T *>(f.k_new) + (size_t)b * f.k_sn + (size_t)h * f.k_sh;
          const T *vsrc = reinterpret_cast<const T *>(f.v_new) + (size_t)b * f.v_sn + (size_t)h * f.v_sh;
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
              float cc, ss, xo, yo;
              rope_cos_sin1(f.rope, rope_pos, i, 64, cc, ss);
              rope_rotate(Elem<T>::to_f32(ksrc[i]), Elem<T>::to_f32(ksrc[i + 64]), cc, ss, xo, yo);
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
              float cc, ss, xo, yo;
              rope_cos_sin1(f.rope, rope_pos, i, 64, cc, ss);
              rope_rotate(Elem<T>::to_f32(ksrc[2 * i]), Elem<T>::to_f32(ksrc[2 * i + 1]), cc, ss, xo, yo);
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
            const bool ok = tok < valid && tok >= tok_lo;
            sc[nt][e] = ok ? sc[nt][e] * scale_log2 : -INFINITY;
            sc[nt][2 + e] = ok ? sc[nt][2 + e] * scale_log2 : -INFINITY;
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
      if (lane == 0 && !aborted) mbar_arrive(&empty_bar[s]);
      g += npg;
      ++it;
    }

    // ================= close the segment: publish the result or the partial
    if (g >= hi) PIEKV_STAMP(2);
    const int c_first = cta_of_page(req_begin, total_pages, G);
    const int c_last = cta_of_page(req_end - 1, total_pages, G);
    const int nseg = c_last - c_first + 1;
    float ls0 = l0, ls1 = l1;  // quad-reduce the running sums
    ls0 += __shfl_xor_sync(0xffffffffu, ls0, 1);
    ls0 += __shfl_xor_sync(0xffffffffu, ls0, 2);
    ls1 += __shfl_xor_sync(0xffffffffu, ls1, 1);
    ls1 += __shfl_xor_sync(0xffffffffu, ls1, 2);
    if (PG == 1 && nseg == 1) {
      // the whole request lived in this CTA: normalise and store
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
    const size_t pidx = (size_t)(c + b) * PG + pslot;
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
    // Combine `n` partials of request b, `stride` slots apart starting at slot `first`: thread ->
    // (query head tid/32 + 8k, 4 consecutive d).  Two passes so that the loads of a pass are
    // independent of one another and stay in flight together: first the global maximum, then the
    // weighted sums.  The result is either the request's output row (normalised) or again a partial
    // (maximum, sum, unnormalised accumulator) written over slot `first`.
    auto merge_parts = [&](size_t first, size_t stride, int n, bool to_partial) {
      const int d4 = (tid & 31) * 4;
      for (int qh = tid >> 5; qh < a.hq; qh += kConsumerWarps) {
        float M = -INFINITY;
#pragma unroll 8
        for (int pp = 0; pp < n; ++pp) {
          const float2 ml = __ldcg(p.part_ml + (first + pp * stride) * a.hq + qh);
          M = ml.y > 0.f ? fmaxf(M, ml.x) : M;
        }
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
        for (int pp = 0; pp < n; ++pp) {
          const size_t idx = (first + pp * stride) * a.hq + qh;
          const float2 ml = __ldcg(p.part_ml + idx);
          const float4 po = __ldcg(reinterpret_cast<const float4 *>(p.part_o + idx * kDim + d4));
          const float w = ml.y > 0.f ? fast_exp2(ml.x - M) : 0.f;  // a warp that saw no page: weight 0
          L = fmaf(ml.y, w, L);
          acc.x = fmaf(po.x, w, acc.x);
          acc.y = fmaf(po.y, w, acc.y);
          acc.z = fmaf(po.z, w, acc.z);
          acc.w = fmaf(po.w, w, acc.w);
        }
        if (to_partial) {
          __syncwarp();  // every lane has read slot `first` of this head before it is overwritten
          const size_t idx = first * a.hq + qh;
          *reinterpret_cast<float4 *>(p.part_o + idx * kDim + d4) = acc;
          if ((tid & 31) == 0) p.part_ml[idx] = make_float2(M, L);
          continue;
        }
        L = add_sink(L, M, a.sinks, qh);
        const float inv = L > 0.f ? 1.f / L : 0.f;
        uint2 pk;
        pk.x = pack2<T>(acc.x * inv, acc.y * inv);
        pk.y = pack2<T>(acc.z * inv, acc.w * inv);
        if (p.peer.n == 0) {
          *reinterpret_cast<uint2 *>(out + ((size_t)b * a.hq + qh) * kDim + d4) = pk;
        } else {
          for (int d = 0; d < n_dst; ++d) *reinterpret_cast<uint2 *>(dst_row(d, b, qh) + d4) = pk;
        }
        if (a.lse != nullptr && (tid & 31) == 0)
          a.lse[(size_t)b * a.hq + qh] = L > 0.f ? (M + log2f(L)) * 0.6931471805599453f : -INFINITY;
      }
    };
    // whoever arrives last on a counter sees everybody else's partials
    auto arrive_last = [&](int *counter, int expected) -> bool {
      __threadfence();
      consumer_bar_sync();
      if (tid == 0) {
        const int old = atomicAdd(counter, 1);
        sh_last = (old == expected - 1) ? 1 : 0;
        if (sh_last) *counter = 0;  // ready for the next launch (nobody else touches it any more)
      }
      consumer_bar_sync();
      const bool last = sh_last != 0;
      consumer_bar_sync();  // everyone has read sh_last before it is rewritten
      if (last) __threadfence();
      return last;
    };
    if (nseg <= kMergeGroup) {
      if (!arrive_last(&p.counters[b], nseg)) continue;
      merge_parts((size_t)(c_first + b) * PG, 1, nseg * PG, false);
      continue;
    }
    // A request cut over many CTAs (one long context): merging 100+ partials in a single CTA would sit
    // on the critical path of the whole launch.  Segments are grouped kMergeGroup at a time; the last
    // CTA of a group folds the group into one partial (groups fold concurrently on different SMs), and
    // the last group to finish folds the groups.
    const int gi = (c - c_first) / kMergeGroup;
    const int g_first = c_first + gi * kMergeGroup;
    const int g_size = min(kMergeGroup, c_last + 1 - g_first);
    const int n_groups = (nseg + kMergeGroup - 1) / kMergeGroup;
    if (!arrive_last(&p.counters[kGroupCounter0 + g_first], g_size)) continue;
    merge_parts((size_t)(g_first + b) * PG, 1, g_size * PG, true);
    if (!arrive_last(&p.counters[b], n_groups)) continue;
    merge_parts((size_t)(c_first + b) * PG, (size_t)kMergeGroup * PG, n_groups, false);
  }
  PIEKV_STAMP(3);
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

int64_t decode_tma_workspace_bytes(int batch, int hq, int hkv) {
  const int pg = (hkv == 1 || hkv == 2 || hkv == 4 || hkv == 8) ? 8 / hkv : 1;
  const int64_t slots = (int64_t)sm_count() + batch;
  const int64_t window_meta = (((int64_t)batch + 1) * 12 + 255) / 256 * 256;  // win_indptr + win_meta
  return kCounterBytes + slots * pg * hq * (kDim * 4 + 8) + 512 + window_meta;
}

static int prepare(const AttnArgs &a, int dtype, void *workspace, int64_t workspace_bytes, DecodeParams *p,
                   CUtensorMap *tm, cudaStream_t st) {
  const int pg = 8 / a.hkv;
  const int64_t slots = (int64_t)sm_count() + a.batch;
  const int64_t need = decode_tma_workspace_bytes(a.batch, a.hq, a.hkv);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= need, "decode: workspace too small (%lld < %lld bytes)",
                (long long)workspace_bytes, (long long)need);
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "decode: workspace must be 256-byte aligned");
  PIEKV_REQUIRE(sm_count() <= kGroupCounters, "decode: %d SMs, the group counters hold %d", sm_count(), kGroupCounters);
  p->a = a;
  p->peer = PeerOut{};
  p->pdl = get_option(PIEKV_OPT_PDL);
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
    p.peer.done = p.counters + (kCounterBytes / 4 - 1);  // last word of the counter block
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
  return (int)cudaMemcpyFromSymbol(host_out, piekv::g_trace, sizeof(unsigned long long) * 256 * 4);
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
  // the arrival counters must be zero when the kernel starts, whatever an earlier call left behind
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)batch * sizeof(int), st);
  if (e != cudaSuccess) return cuda_status(e, "decode_run_noalloc: cudaMemsetAsync");
  // and the group counters of the two-level merge, at the tail of the counter block
  e = cudaMemsetAsync(reinterpret_cast<uint8_t *>(scratch) + (size_t)kGroupCounter0 * sizeof(int), 0,
                      (size_t)(kGroupCounters + 1) * sizeof(int), st);
  if (e != cudaSuccess) return cuda_status(e, "decode_run_noalloc: cudaMemsetAsync");
  return launch_decode_tma(a, dtype, scratch, kStaticScratchBytes, st);
}
