// Prefill / chunked-prefill attention over paged K/V on the sm_100a tensor cores.
//
// One CTA works on one (request, 128-row query tile, query head).  S = Q K^T and O += P V are
// tcgen05 MMAs (M = 128, N = 128, K = 16) with fp32 accumulators in tensor memory:
//   TMEM columns [0,128) and [128,256): two S buffers, [256,384): O.
// Operands are staged in shared memory with 128-byte swizzle:
//   Q   [2 d-halves][128 rows][64 d]      K-major A operand            (one TMA box)
//   K_j [2 d-halves][128 tokens][64 d]    K-major B operand            (2 TMA boxes per page)
//   V_j [2 d-halves][128 tokens][64 d]    MN-major B operand           (2 TMA boxes per page)
//   P_j [2 token-halves][128 rows][64 t]  K-major A operand, written by the softmax threads
// Warp roles: warps 0-7 softmax (two threads per query row, 64 kv columns each), warp 8 TMA
// producer (K ring of 3 tiles, V ring of 2, independent cursors), warp 9 MMA issuer and TMEM owner.  The MMA warp runs one tile ahead on S (S is double buffered), the
// softmax threads keep the running maximum lazily (O in TMEM is only rescaled when the maximum
// grows by more than 2^8), so tile j's softmax overlaps QK of tile j+1 and PV of tile j-1.
//
// Masking: causal with offset (token t allowed iff t <= kv_len - qo_len + row), none, or a custom
// mask.  The flat boolean mask of the reference is bit-packed once per batch by the plan kernels
// (128 bits per query row and kv tile) together with a per-(query tile, kv tile) "any allowed"
// summary; kv tiles no row of the query tile may see are skipped by every role.
//
// Every wait is bounded; on a timeout the CTA records PIEKV_ERR_WAIT_TIMEOUT, all roles leave
// their loops, outstanding bulk copies are drained and TMEM is released before the CTA exits.
#include <cuda.h>

#include <type_traits>

#include "attn.cuh"
#include "common.cuh"
#include "tcgen05.cuh"
#include "prefill_common.cuh"
#include "tma.cuh"

namespace piekv {

using namespace prefill;

namespace {

PlanView plan_view(void *workspace, int batch, int nnz, int num_pages, int64_t mask_bytes) {
  PlanView v;
  v.max_tiles = (nnz + kBM - 1) / kBM + batch;
  v.sw = mask_bytes > 0 ? ((num_pages + 7) / 8 + 31) / 32 : 0;
  uint8_t *ws = reinterpret_cast<uint8_t *>(workspace);
  int64_t off = kCounterBytes;
  auto take = [&](int64_t bytes) {
    int64_t o = off;
    off += (bytes + 255) / 256 * 256;
    return ws ? ws + o : nullptr;
  };
  v.ntiles = reinterpret_cast<int *>(take(256));
  v.tile_base = reinterpret_cast<int32_t *>(take((int64_t)(batch + 1) * 4));
  v.poff = reinterpret_cast<long long *>(take((int64_t)(batch + 1) * 8));
  v.moff = reinterpret_cast<long long *>(take((int64_t)(batch + 1) * 8));
  v.tiles = reinterpret_cast<int2 *>(take((int64_t)v.max_tiles * 8));
  v.summary = reinterpret_cast<uint32_t *>(take((int64_t)v.max_tiles * v.sw * 4));
  // every row is padded to whole 128-bit groups: at most 16 bytes more than its share of mask_bytes / 8
  v.packed = reinterpret_cast<uint4 *>(take(mask_bytes > 0 ? mask_bytes / 8 + (int64_t)nnz * 16 + 16 : 0));
  v.bytes = off;
  return v;
}

__device__ __forceinline__ int kv_len_of(const int32_t *kv_indptr, const int32_t *last, int b, int page_size) {
  const int np = kv_indptr[b + 1] - kv_indptr[b];
  return np > 0 ? (np - 1) * page_size + last[b] : 0;
}

// per-request prefix sums: q tiles, packed-mask rows (16-byte units), flat-mask bytes.  One block.
__global__ void prefill_scan_kernel(const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                                    const int32_t *__restrict__ last, int batch, int page_size, int32_t *tile_base,
                                    long long *poff, long long *moff) {
  __shared__ long long sh[3][32];
  __shared__ long long carry[3];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  if (threadIdx.x < 3) carry[threadIdx.x] = 0;
  __syncthreads();
  for (int base = 0; base < batch; base += blockDim.x) {
    const int b = base + threadIdx.x;
    long long v[3] = {0, 0, 0};
    if (b < batch) {
      const long long qo = qo_indptr[b + 1] - qo_indptr[b];
      const long long kv = kv_len_of(kv_indptr, last, b, page_size);
      v[0] = (qo + kBM - 1) / kBM;
      v[1] = qo * ((kv + 127) / 128);
      v[2] = qo * kv;
    }
    long long incl[3];
#pragma unroll
    for (int q = 0; q < 3; ++q) {
      long long x = v[q];
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        long long y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      incl[q] = x;
      if (lane == 31) sh[q][warp] = x;
    }
    __syncthreads();
    if (warp == 0) {
#pragma unroll
      for (int q = 0; q < 3; ++q) {
        long long x = lane < nw ? sh[q][lane] : 0;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          long long y = __shfl_up_sync(0xffffffffu, x, d);
          if (lane >= d) x += y;
        }
        sh[q][lane] = x;  // inclusive over warps
      }
    }
    __syncthreads();
    long long excl[3];
#pragma unroll
    for (int q = 0; q < 3; ++q) excl[q] = carry[q] + (warp > 0 ? sh[q][warp - 1] : 0) + incl[q] - v[q];
    if (b < batch) {
      tile_base[b] = (int32_t)excl[0];
      poff[b] = excl[1];
      moff[b] = excl[2];
    }
    __syncthreads();
    if (threadIdx.x == blockDim.x - 1) {
#pragma unroll
      for (int q = 0; q < 3; ++q) carry[q] = excl[q] + v[q];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    tile_base[batch] = (int32_t)carry[0];
    poff[batch] = carry[1];
    moff[batch] = carry[2];
  }
}

// flat boolean mask -> 128-bit groups per (query row, kv tile) + per-(q tile, kv tile) "any" bits.
// One warp per query row.
__global__ void prefill_pack_mask_kernel(const uint8_t *__restrict__ mask, const int32_t *__restrict__ qo_indptr,
                                         const int32_t *__restrict__ kv_indptr, const int32_t *__restrict__ last,
                                         int batch, int nnz, int page_size, const int32_t *__restrict__ tile_base,
                                         const long long *__restrict__ poff, const long long *__restrict__ moff,
                                         uint4 *packed, uint32_t *summary, int sw, int window_left) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= nnz) return;
  int lo = 0, hi = batch;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (qo_indptr[mid + 1] > i)
      hi = mid;
    else
      lo = mid + 1;
  }
  const int b = lo < batch ? lo : batch - 1;
  const int j = i - qo_indptr[b];
  const int kv = kv_len_of(kv_indptr, last, b, page_size);
  const int groups = (kv + 127) / 128;
  // a sliding window is ANDed into the mask: keys before (position of the query) - window_left are dropped
  const int t_first = window_left >= 0 ? max(0, kv - (qo_indptr[b + 1] - qo_indptr[b]) + j - window_left) : 0;
  const uint8_t *src = mask + moff[b] + (long long)j * kv;
  uint32_t *dst = reinterpret_cast<uint32_t *>(packed + poff[b] + (long long)j * groups);
  uint32_t *srow = summary + (size_t)(tile_base[b] + j / kBM) * sw;
  for (int g = 0; g < groups; ++g) {
    uint32_t any = 0;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const int t = g * 128 + w * 32 + lane;
      const uint32_t word = __ballot_sync(0xffffffffu, t < kv && t >= t_first && src[t] != 0);
      if (lane == w) dst[g * 4 + w] = word;
      any |= word;
    }
    if (lane == 0 && any != 0) {
      uint32_t *sp = srow + (g >> 5);
      const uint32_t bit = 1u << (g & 31);
      if ((*(volatile uint32_t *)sp & bit) == 0) atomicOr(sp, bit);
    }
  }
}

// BRLE runs -> the same 128-bit groups and "any" bits, without the flat boolean mask ever existing.
// Semantics of the reference's host expansion (pie/src/pie_worker/batching.py:337-389): the runs of a
// query token alternate attend / skip starting with attend, lie end to end from kv position 0, and
// only the first position + 1 entries of the row can be set, position = kv_len - qo_len + index of
// the token in its request.  One warp per query row: the row is cleared, then every attend run ORs
// its clipped interval into the words it touches (word w belongs to lane w % 32, so the read-modify-
// writes of a row never collide), then the groups are summarised.
__global__ void prefill_brle_mask_kernel(const uint32_t *__restrict__ runs, const int32_t *__restrict__ run_indptr,
                                         const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                                         const int32_t *__restrict__ last, int batch, int nnz, int page_size,
                                         const int32_t *__restrict__ tile_base, const long long *__restrict__ poff,
                                         uint4 *packed, uint32_t *summary, int sw, int window_left) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= nnz) return;
  int lo = 0, hi = batch;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (qo_indptr[mid + 1] > i)
      hi = mid;
    else
      lo = mid + 1;
  }
  const int b = lo < batch ? lo : batch - 1;
  const int j = i - qo_indptr[b];
  const int qo = qo_indptr[b + 1] - qo_indptr[b];
  const int kv = kv_len_of(kv_indptr, last, b, page_size);
  const int groups = (kv + 127) / 128;
  const int words = groups * 4;
  const long long valid = max(0, min(kv, kv - qo + j + 1));
  // a sliding window clips every attend run from below
  const long long t_first = window_left >= 0 ? max(0, kv - qo + j - window_left) : 0;
  uint32_t *dst = reinterpret_cast<uint32_t *>(packed + poff[b] + (long long)j * groups);
  for (int w = lane; w < words; w += 32) dst[w] = 0;
  const int r0 = run_indptr[i], r1 = run_indptr[i + 1];
  long long carry = 0;  // kv position where the next run starts
  for (int base = r0; base < r1 && carry < valid; base += 32) {
    const int r = base + lane;
    const long long len = r < r1 ? (long long)runs[r] : 0;
    long long end = len;  // inclusive scan of the run lengths of this chunk
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long up = __shfl_up_sync(0xffffffffu, end, o);
      if (lane >= o) end += up;
    }
    end += carry;
    const long long start = end - len;
    const int n_here = min(32, r1 - base);
    for (int k = 0; k < n_here; k += 2) {  // attend runs: even index within the token (r0 is index 0)
      const int src_lane = k;  // chunks start 32 runs apart, so even lanes hold the even-numbered runs
      long long s = __shfl_sync(0xffffffffu, start, src_lane);
      long long e = __shfl_sync(0xffffffffu, end, src_lane);
      if (s >= valid) break;
      e = min(e, valid);
      s = max(s, t_first);
      if (e <= s) continue;
      const int w_first = (int)(s >> 5), w_last = (int)((e - 1) >> 5);
      // lane's first owned word at or after w_first
      int w = w_first + ((lane - w_first) & 31);
      for (; w <= w_last; w += 32) {
        const long long wb = (long long)w << 5;
        const uint32_t lo_mask = s > wb ? 0xffffffffu << (int)(s - wb) : 0xffffffffu;
        const uint32_t hi_mask = e < wb + 32 ? 0xffffffffu >> (int)(wb + 32 - e) : 0xffffffffu;
        dst[w] |= lo_mask & hi_mask;
      }
    }
    carry = __shfl_sync(0xffffffffu, end, 31);
  }
  __syncwarp();
  uint32_t *srow = summary + (size_t)(tile_base[b] + j / kBM) * sw;
  for (int g = lane; g < groups; g += 32) {
    const uint4 v = reinterpret_cast<const uint4 *>(dst)[g];
    if ((v.x | v.y | v.z | v.w) != 0) {
      uint32_t *sp = srow + (g >> 5);
      const uint32_t bit = 1u << (g & 31);
      if ((*(volatile uint32_t *)sp & bit) == 0) atomicOr(sp, bit);
    }
  }
}

// A sliding window without any other mask, in the same packed form: the query at position
// p = kv_len - qo_len + j sees keys [max(0, p - window_left), causal ? p : kv_len - 1].  One warp per
// query row; lane w writes words w, w + 32, ... of the row.
__global__ void prefill_window_mask_kernel(const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                                           const int32_t *__restrict__ last, int batch, int nnz, int page_size,
                                           const int32_t *__restrict__ tile_base, const long long *__restrict__ poff,
                                           uint4 *packed, uint32_t *summary, int sw, int window_left, int causal) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= nnz) return;
  int lo = 0, hi = batch;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (qo_indptr[mid + 1] > i)
      hi = mid;
    else
      lo = mid + 1;
  }
  const int b = lo < batch ? lo : batch - 1;
  const int j = i - qo_indptr[b];
  const int qo = qo_indptr[b + 1] - qo_indptr[b];
  const int kv = kv_len_of(kv_indptr, last, b, page_size);
  const int groups = (kv + 127) / 128;
  const int pos = kv - qo + j;
  const long long s = max(0, pos - window_left);
  const long long e = causal ? max(0, min(kv, pos + 1)) : kv;  // exclusive
  uint32_t *dst = reinterpret_cast<uint32_t *>(packed + poff[b] + (long long)j * groups);
  uint32_t *srow = summary + (size_t)(tile_base[b] + j / kBM) * sw;
  for (int w = lane; w < groups * 4; w += 32) {
    const long long wb = (long long)w << 5;
    uint32_t bits = 0;
    if (e > s && wb < e && wb + 32 > s) {
      const uint32_t lo_mask = s > wb ? 0xffffffffu << (int)(s - wb) : 0xffffffffu;
      const uint32_t hi_mask = e < wb + 32 ? 0xffffffffu >> (int)(wb + 32 - e) : 0xffffffffu;
      bits = lo_mask & hi_mask;
    }
    dst[w] = bits;
    if (bits != 0) {
      const int g = w >> 2;
      uint32_t *sp = srow + (g >> 5);
      const uint32_t bit = 1u << (g & 31);
      if ((*(volatile uint32_t *)sp & bit) == 0) atomicOr(sp, bit);
    }
  }
}

// The packed mask of a planned batch written back in the reference's flat form (one byte per
// (query, key) pair, rows of kv_len entries, requests end to end; pie/src/pie_worker/batching.py:113-135).
// One warp per query row.
__global__ void prefill_unpack_mask_kernel(const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                                           const int32_t *__restrict__ last, int batch, int nnz, int page_size,
                                           const long long *__restrict__ poff, const long long *__restrict__ moff,
                                           const uint4 *__restrict__ packed, uint8_t *flat) {
  const int lane = threadIdx.x & 31;
  const int i = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= nnz) return;
  int lo = 0, hi = batch;
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (qo_indptr[mid + 1] > i)
      hi = mid;
    else
      lo = mid + 1;
  }
  const int b = lo < batch ? lo : batch - 1;
  const int j = i - qo_indptr[b];
  const int kv = kv_len_of(kv_indptr, last, b, page_size);
  const int groups = (kv + 127) / 128;
  const uint32_t *src = reinterpret_cast<const uint32_t *>(packed + poff[b] + (long long)j * groups);
  uint8_t *dst = flat + moff[b] + (long long)j * kv;
  for (int t = lane; t < kv; t += 32) dst[t] = (uint8_t)((src[t >> 5] >> (t & 31)) & 1u);
}

// ------------------------------------------------------------------------------------------------
// work list: one entry per (request, 128-row tile), ordered by decreasing number of kv tiles
// ------------------------------------------------------------------------------------------------
__global__ void prefill_plan_kernel(const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                                    const int32_t *__restrict__ kv_last_page_len, int batch, int page_size, int causal,
                                    const int32_t *__restrict__ tile_base, const uint32_t *__restrict__ summary, int sw,
                                    int has_mask, int2 *tiles, int *ntiles, int max_tiles) {
  __shared__ int hist[kSortBins];
  for (int i = threadIdx.x; i < kSortBins; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  auto key_of = [&](int b, int qo_len, int kv_len, int r0) {
    int nt;
    if (has_mask) {
      nt = 0;
      const uint32_t *srow = summary + (size_t)(tile_base[b] + r0 / kBM) * sw;
      const int words = ((kv_len + kBN - 1) / kBN + 31) / 32;
      for (int w = 0; w < words; ++w) nt += __popc(srow[w]);
    } else {
      int hi = causal ? min(kv_len, kv_len - qo_len + r0 + kBM) : kv_len;
      nt = hi > 0 ? (hi + kBN - 1) / kBN : 0;
    }
    nt = nt < kSortBins ? nt : kSortBins - 1;
    return kSortBins - 1 - nt;  // bin 0 = most work
  };
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    int qo_len = qo_indptr[b + 1] - qo_indptr[b];
    int kv_len = kv_len_of(kv_indptr, kv_last_page_len, b, page_size);
    for (int r0 = 0; r0 < qo_len; r0 += kBM) atomicAdd(&hist[key_of(b, qo_len, kv_len, r0)], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < kSortBins; ++i) {
      int c = hist[i];
      hist[i] = acc;
      acc += c;
    }
    *ntiles = acc < max_tiles ? acc : max_tiles;
    ntiles[2] = 0;  // items claimed and CTAs finished: the persistent kernel's counters, which every
    ntiles[3] = 0;  // launch leaves at zero again
  }
  __syncthreads();
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    int qo_len = qo_indptr[b + 1] - qo_indptr[b];
    int kv_len = kv_len_of(kv_indptr, kv_last_page_len, b, page_size);
    for (int r0 = 0; r0 < qo_len; r0 += kBM) {
      int pos = atomicAdd(&hist[key_of(b, qo_len, kv_len, r0)], 1);
      if (pos < max_tiles) tiles[pos] = make_int2(b, r0);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                      const __grid_constant__ PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages], v_land,
      s_full[2], s_empty[2], p_full, pv_done, pair_bar[4];
  __shared__ uint32_t tmem_slot;
  __shared__ int sh_abort;
  __shared__ float xch_sum[2][kBM];  // [column half][row]: partial softmax denominators (epilogue)

  const AttnArgs &a = p.a;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- work item ------------------------------------------------------------------------------
  const int tile = blockIdx.x / a.hq;
  const int h = blockIdx.x % a.hq;
  if (tile >= *p.ntiles) return;
  const int2 item = p.tiles[tile];
  const int b = item.x, r0 = item.y;
  const int group = a.hq / a.hkv;
  const int hk = h / group;
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
  const int rows = min(kBM, qo_len - r0);  // valid query rows of this tile
  const bool has_mask = p.has_mask != 0;
  const int kv_hi = (a.causal && !has_mask) ? min(kv_len, kv_len - qo_len + r0 + kBM) : kv_len;
  const int n_tiles = kv_hi > 0 ? (kv_hi + kBN - 1) / kBN : 0;
  const int groups = (kv_len + kBN - 1) / kBN;  // 128-bit mask groups per query row
  // with a custom mask, kv tiles without a single allowed pair are skipped by every role
  const uint32_t *srow = has_mask ? p.summary + (size_t)(p.tile_base[b] + r0 / kBM) * p.sw : nullptr;
  auto active = [&](int j) { return !has_mask || ((__ldg(srow + (j >> 5)) >> (j & 31)) & 1u) != 0; };
  int n_active = n_tiles;
  if (has_mask) {
    n_active = 0;
    for (int w = 0; w < (n_tiles + 31) / 32; ++w) n_active += __popc(__ldg(srow + w));
  }
  T *out = reinterpret_cast<T *>(a.out);

  if (n_active == 0) {  // nothing to attend to: zeros (uniform for the whole CTA, before any allocation)
    for (int x = threadIdx.x; x < rows * (kDim / 8); x += kThreads) {
      const int r = x / (kDim / 8), c8 = x % (kDim / 8);
      *reinterpret_cast<uint4 *>(out + ((size_t)(q0 + r0 + r) * a.hq + h) * kDim + c8 * 8) = make_uint4(0, 0, 0, 0);
    }
    if (a.lse != nullptr)
      for (int r = threadIdx.x; r < rows; r += kThreads) a.lse[(size_t)(q0 + r0 + r) * a.hq + h] = -INFINITY;
    return;
  }

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t q_smem = base;
  const uint32_t k_smem0 = base + kTileBytes;                   // K stage s at + s * 32K
  const uint32_t v_smem0 = base + kTileBytes * (1 + kKStages);  // V stage s at + s * 32K
  const uint32_t p_smem = base + kTileBytes * (1 + kKStages + kVStages);
  uint8_t *p_ptr = base_ptr + kTileBytes * (1 + kKStages + kVStages);

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
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], kSoftmaxWarps * 32);
    }
    mbar_init(&p_full, kSoftmaxWarps * 32);
    for (int s = 0; s < 4; ++s) mbar_init(&pair_bar[s], 64);
    mbar_init(&pv_done, 1);
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

  if (warp == kProducerWarp) {
    // ================================================================== TMA producer
    // K and V have their own rings and cursors, so K runs ahead of V by the depth of its ring
    int k_armed = 0, v_armed = 0;  // K / V tiles issued so far
    int jk = 0, jv = 0;            // next kv tile index to consider for K / for V
    if (lane == 0) {
      mbar_arrive_expect_tx(&q_full, kTileBytes);
      tma_load_4d(q_smem, &tmap_q, 0, q0 + r0, 0, h, &q_full);
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
      // O += P V for the it-th processed tile
      auto issue_pv = [&](int jj) -> bool {
        const int vs = jj % kVStages;
        if (!wait_or_abort(&v_full[vs], (jj / kVStages) & 1, abort_flag)) return false;
        if (!wait_or_abort(&p_full, jj & 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t v_smem = v_smem0 + vs * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          tc::mma_ss(tmem + kColO, tc::desc_k_major(p_smem + (ks >> 2) * kHalfBytes + (ks & 3) * 32),
                     tc::desc_mn_major(v_smem + ks * 2048, kHalfBytes), idesc_pv, (jj > 0 || ks > 0) ? 1u : 0u);
        }
        tc::commit(&pv_done);
        tc::commit(&v_empty[vs]);
        return true;
      };
      bool ok = wait_or_abort(&q_full, 0, abort_flag);
      int it = 0;  // S tiles issued so far
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (!active(j)) continue;
        const int kst = it % kKStages, sb = it & 1;
        ok = wait_or_abort(&k_full[kst], (it / kKStages) & 1, abort_flag) &&
             wait_or_abort(&s_empty[sb], ((it >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc::fence_after_sync();
        const uint32_t k_smem = k_smem0 + kst * kTileBytes;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          tc::mma_ss(tmem + kColS + sb * kBN, tc::desc_k_major(q_smem + off), tc::desc_k_major(k_smem + off), idesc_qk,
                     ks > 0 ? 1u : 0u);
        }
        tc::commit(&k_empty[kst]);
        tc::commit(&s_full[sb]);
        if (it >= 1) ok = issue_pv(it - 1);
        ++it;
      }
      if (ok && it >= 1) ok = issue_pv(it - 1);
      if (!ok) {
        if (!*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 200);
        atomicExch(&sh_abort, 1);
      }
    }
  } else {
    // ============================================== softmax (two threads per row, 64 columns each)
    const int q4 = warp & 3;    // TMEM lane quarter this warp may access
    const int hh = warp >> 2;   // column half of the S tile (and token half of the P tile) it owns
    const int row = q4 * 32 + lane;  // row of the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const bool row_valid = row < rows;
    // last allowed token of this row (inclusive)
    const int limit = row_valid ? ((a.causal && !has_mask) ? min(kv_len - 1, kv_len - qo_len + r0 + row) : kv_len - 1) : -1;
    const uint4 *mrow = has_mask ? p.packed + p.poff[b] + (long long)(r0 + (row_valid ? row : 0)) * groups : nullptr;
    const float c = a.sm_scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t sreg[64];
    int it = 0;
    // the two warps that share a lane quarter meet at their own mbarrier (bounded, abort-aware)
    uint32_t pair_phase = 0;
    auto pair_sync = [&]() -> bool {
      mbar_arrive(&pair_bar[q4]);
      const bool r = wait_or_abort(&pair_bar[q4], pair_phase & 1, abort_flag);
      ++pair_phase;
      return r;
    };

    for (int j = 0; j < n_tiles; ++j) {
      if (!active(j)) continue;
      const int sb = it & 1;
      uint4 mw4 = make_uint4(0, 0, 0, 0);
      if (has_mask && row_valid) mw4 = __ldg(mrow + j);  // in flight while we wait for S
      ok = wait_or_abort(&s_full[sb], (it >> 1) & 1, abort_flag);
      if (!ok) break;
      tc::fence_after_sync();
      // own half of the row stays in registers; the other half is read only for the row maximum,
      // so the two threads of a row agree on it without exchanging anything
      const uint32_t s_row = tmem + lane_base + kColS + sb * kBN;
      uint32_t oth[64];
      tc::tmem_ld32(s_row + hh * 64, sreg);
      tc::tmem_ld32(s_row + hh * 64 + 32, sreg + 32);
      tc::tmem_ld32(s_row + (hh ^ 1) * 64, oth);
      tc::tmem_ld32(s_row + (hh ^ 1) * 64 + 32, oth + 32);
      tc::tmem_wait_ld();
      tc::fence_before_sync();
      mbar_arrive(&s_empty[sb]);  // S is in registers: the MMA warp may overwrite this buffer

      // ---- running maximum (lazy) and probabilities
      const int t0 = j * kBN + hh * 64;       // first token of the own half
      const int t1 = j * kBN + (hh ^ 1) * 64;  // first token of the other half
      const uint32_t mown[2] = {hh ? mw4.z : mw4.x, hh ? mw4.w : mw4.y};
      const uint32_t moth[2] = {hh ? mw4.x : mw4.z, hh ? mw4.y : mw4.w};
      const bool full_own = has_mask ? (mown[0] & mown[1]) == 0xffffffffu : t0 + 63 <= limit;
      const bool full_oth = has_mask ? (moth[0] & moth[1]) == 0xffffffffu : t1 + 63 <= limit;
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (full_own) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mxa[i & 3] = fmaxf(mxa[i & 3], __uint_as_float(sreg[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const bool allow = has_mask ? ((mown[i >> 5] >> (i & 31)) & 1u) != 0 : t0 + i <= limit;
          const float v = allow ? __uint_as_float(sreg[i]) : -INFINITY;
          sreg[i] = __float_as_uint(v);
          mxa[i & 3] = fmaxf(mxa[i & 3], v);
        }
      }
      if (full_oth) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mxa[i & 3] = fmaxf(mxa[i & 3], __uint_as_float(oth[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const bool allow = has_mask ? ((moth[i >> 5] >> (i & 31)) & 1u) != 0 : t1 + i <= limit;
          mxa[i & 3] = fmaxf(mxa[i & 3], allow ? __uint_as_float(oth[i]) : -INFINITY);
        }
      }
      float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
      mx *= c;  // c > 0
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_ref + 8.f) {
        alpha = fast_exp2(m_ref - mx);  // m_ref = -inf on the first hit: 0
        l *= alpha;
        m_ref = mx;
        rescale = it > 0;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      float suma[4] = {0.f, 0.f, 0.f, 0.f};
      const float neg_m = -m_use;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float p0v = fast_exp2(fmaf(__uint_as_float(sreg[2 * i]), c, neg_m));
        const float p1v = fast_exp2(fmaf(__uint_as_float(sreg[2 * i + 1]), c, neg_m));
        suma[i & 3] += p0v + p1v;
        sreg[i] = pack2<T>(p0v, p1v);  // tokens 2i, 2i+1 of this half
      }
      l += (suma[0] + suma[1]) + (suma[2] + suma[3]);
      // ---- P buffer free and O stable once PV of the previous tile has completed
      if (it > 0) {
        ok = wait_or_abort(&pv_done, (it - 1) & 1, abort_flag);
        if (!ok) break;
        tc::fence_after_sync();
      }
      if (__any_sync(0xffffffffu, rescale)) {
        const uint32_t o_addr = tmem + lane_base + kColO + hh * 64;
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          uint32_t oreg[32];
          tc::tmem_ld32(o_addr + ch * 32, oreg);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
          tc::tmem_st32(o_addr + ch * 32, oreg);
        }
        tc::tmem_wait_st();
      }
      // ---- P -> shared memory, K-major with 128-byte swizzle: row r, token half hh, 16-byte chunk cc
      {
        uint8_t *prow = p_ptr + hh * kHalfBytes + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          *reinterpret_cast<uint4 *>(prow + ((cc ^ (row & 7)) << 4)) =
              make_uint4(sreg[cc * 4], sreg[cc * 4 + 1], sreg[cc * 4 + 2], sreg[cc * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc::fence_before_sync();
      mbar_arrive(&p_full);
      ++it;
    }

    // ---- epilogue: O / l -> out (each thread stores its 64 of the row's 128 values)
    if (ok) ok = wait_or_abort(&pv_done, (n_active - 1) & 1, abort_flag);
    xch_sum[hh][row] = l;
    if (ok) ok = pair_sync();
    if (ok) {
      tc::fence_after_sync();
      const float lsum = add_sink(l + xch_sum[hh ^ 1][row], m_ref, a.sinks, h);
      const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
      T *orow = out + ((size_t)(q0 + r0 + row) * a.hq + h) * kDim + hh * 64;
      const uint32_t o_addr = tmem + lane_base + kColO + hh * 64;
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
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
      if (a.lse != nullptr && row_valid && hh == 0)
        a.lse[(size_t)(q0 + r0 + row) * a.hq + h] = lsum > 0.f ? (m_ref + log2f(lsum)) * 0.6931471805599453f : -INFINITY;
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

}  // namespace

bool prefill_tc_supported(const AttnArgs &a, int dtype) {
  if (dtype != PIEKV_BF16 && dtype != PIEKV_F16) return false;
  if (a.dim != kDim || a.page_size != kPage) return false;
  if (a.hq % a.hkv != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.pool) & 15) || (reinterpret_cast<uintptr_t>(a.q) & 15) ||
      (reinterpret_cast<uintptr_t>(a.out) & 15))
    return false;
  if ((a.q_sn & 7) || (a.q_sh & 7)) return false;
  return true;
}

int64_t prefill_tc_workspace_bytes(int batch, int nnz, int num_pages, int64_t mask_bytes) {
  return plan_view(nullptr, batch, nnz, num_pages, mask_bytes).bytes;
}

// Build the plan of a batch in the workspace: per-request offsets, the bit-packed mask with its
// tile summary (custom mask only) and the work list.  Stream-ordered, no host synchronisation.
int launch_prefill_plan(const AttnArgs &a, int64_t mask_bytes, void *workspace, int64_t workspace_bytes,
                        cudaStream_t st, const uint32_t *brle_runs, const int32_t *brle_indptr) {
  if (a.nnz == 0 || a.batch == 0) return 0;
  const bool brle = brle_runs != nullptr || brle_indptr != nullptr;
  const bool window_only = a.window_left >= 0 && a.mask == nullptr && !brle && mask_bytes > 0;
  const bool masked = a.mask != nullptr || brle || window_only;
  const PlanView v = plan_view(workspace, a.batch, a.nnz, a.num_pages, masked ? mask_bytes : 0);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= v.bytes, "prefill: workspace too small (%lld < %lld bytes)",
                (long long)workspace_bytes, (long long)v.bytes);
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "prefill: workspace must be 256-byte aligned");
  prefill_scan_kernel<<<1, 1024, 0, st>>>(a.qo_indptr, a.kv_indptr, a.kv_last_page_len, a.batch, a.page_size,
                                          v.tile_base, v.poff, v.moff);
  PIEKV_LAUNCH_CHECK("prefill_scan_kernel");
  if (masked) {
    cudaError_t e = cudaMemsetAsync(v.summary, 0, (size_t)v.max_tiles * v.sw * 4, st);
    if (e != cudaSuccess) return cuda_status(e, "prefill: cudaMemsetAsync");
  }
  if (brle) {
    prefill_brle_mask_kernel<<<(a.nnz + 7) / 8, 256, 0, st>>>(brle_runs, brle_indptr, a.qo_indptr, a.kv_indptr,
                                                               a.kv_last_page_len, a.batch, a.nnz, a.page_size,
                                                               v.tile_base, v.poff, v.packed, v.summary, v.sw,
                                                               a.window_left);
    PIEKV_LAUNCH_CHECK("prefill_brle_mask_kernel");
  } else if (a.mask != nullptr) {
    prefill_pack_mask_kernel<<<(a.nnz + 7) / 8, 256, 0, st>>>(a.mask, a.qo_indptr, a.kv_indptr, a.kv_last_page_len,
                                                               a.batch, a.nnz, a.page_size, v.tile_base, v.poff, v.moff,
                                                               v.packed, v.summary, v.sw, a.window_left);
    PIEKV_LAUNCH_CHECK("prefill_pack_mask_kernel");
  } else if (window_only) {
    prefill_window_mask_kernel<<<(a.nnz + 7) / 8, 256, 0, st>>>(a.qo_indptr, a.kv_indptr, a.kv_last_page_len, a.batch,
                                                                 a.nnz, a.page_size, v.tile_base, v.poff, v.packed,
                                                                 v.summary, v.sw, a.window_left, a.causal);
    PIEKV_LAUNCH_CHECK("prefill_window_mask_kernel");
  }
  prefill_plan_kernel<<<1, 1024, 0, st>>>(a.qo_indptr, a.kv_indptr, a.kv_last_page_len, a.batch, a.page_size, a.causal,
                                          v.tile_base, v.summary, v.sw, masked ? 1 : 0, v.tiles, v.ntiles, v.max_tiles);
  PIEKV_LAUNCH_CHECK("prefill_plan_kernel");
  return 0;
}

int launch_prefill_export_mask(const AttnArgs &a, int64_t mask_bytes, void *workspace, int64_t workspace_bytes,
                               uint8_t *flat, cudaStream_t st) {
  if (a.nnz == 0 || a.batch == 0 || mask_bytes == 0) return 0;
  const PlanView v = plan_view(workspace, a.batch, a.nnz, a.num_pages, mask_bytes);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= v.bytes, "prefill: workspace too small (%lld < %lld bytes)",
                (long long)workspace_bytes, (long long)v.bytes);
  prefill_unpack_mask_kernel<<<(a.nnz + 7) / 8, 256, 0, st>>>(a.qo_indptr, a.kv_indptr, a.kv_last_page_len, a.batch,
                                                               a.nnz, a.page_size, v.poff, v.moff, v.packed, flat);
  PIEKV_LAUNCH_CHECK("prefill_unpack_mask_kernel");
  return 0;
}

template <typename T>
static int launch_prefill_t(const AttnArgs &a, const CUtensorMap &tq, const CUtensorMap &tkv, const PrefillParams &p,
                            int max_tiles, cudaStream_t st) {
  static unsigned char configured[kMaxDevices] = {0};
  if (int rc = opt_in_dynamic_smem(prefill_tc_kernel<T>, kSmemBytes, configured, "prefill: cudaFuncSetAttribute"))
    return rc;
  const long long blocks = (long long)max_tiles * a.hq;
  PIEKV_REQUIRE(blocks < (1ll << 31), "prefill: too many tiles");
  prefill_tc_kernel<T><<<(unsigned)blocks, kThreads, kSmemBytes, st>>>(tq, tkv, p);
  PIEKV_LAUNCH_CHECK("prefill_tc_kernel");
  return 0;
}

bool prefill_tc2_supported(const AttnArgs &a);
int launch_prefill_tc2(const AttnArgs &a, int dtype, const PrefillParams &p, int max_tiles, cudaStream_t st);

// Attention over a batch whose plan is already in the workspace.
int launch_prefill_tc(const AttnArgs &a, int dtype, int64_t mask_bytes, void *workspace, int64_t workspace_bytes,
                      cudaStream_t st) {
  if (a.nnz == 0 || a.batch == 0) return 0;
  const PlanView v = plan_view(workspace, a.batch, a.nnz, a.num_pages, a.mask ? mask_bytes : 0);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= v.bytes, "prefill: workspace too small (%lld < %lld bytes)",
                (long long)workspace_bytes, (long long)v.bytes);
  PrefillParams p;
  p.a = a;
  p.ntiles = v.ntiles;
  p.claim = v.ntiles + 2;
  p.tiles = v.tiles;
  p.tile_base = v.tile_base;
  p.poff = v.poff;
  p.summary = v.summary;
  p.packed = v.packed;
  p.sw = v.sw;
  p.has_mask = a.mask != nullptr ? 1 : 0;
  if (prefill_tc2_supported(a)) return launch_prefill_tc2(a, dtype, p, v.max_tiles, st);
  CUtensorMap tq, tkv;
  if (int rc = make_q_tensor_map(&tq, a.q, a.nnz, a.hq, a.q_sn, a.q_sh, dtype, kBM)) return rc;
  if (int rc = make_page_tensor_map(&tkv, a.pool, a.num_pages, a.hkv, dtype, 1, 1, 1)) return rc;
  if (dtype == PIEKV_BF16) return launch_prefill_t<__nv_bfloat16>(a, tq, tkv, p, v.max_tiles, st);
  return launch_prefill_t<__half>(a, tq, tkv, p, v.max_tiles, st);
}

}  // namespace piekv
