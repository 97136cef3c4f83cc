// Device-resident page bookkeeping: page tables, reference counts and the free list live in HBM and are
// advanced by small kernels, so that a decode loop (and a beam search that forks and drops contexts)
// runs without the host touching a page table between steps.
//
// Semantics restated from the reference's host code:
//   * which id a new page gets: always the smallest free one (runtime/src/utils.rs:42-158; the host
//     pool's "free set + next counter" is the same set of ids as the free bitmap kept here);
//   * growing a context by n tokens (adjust_kv_pages, sdk/rust/inferlet/src/context.rs:356-399):
//     pages = ceil(tokens / page_size), last_page_len = tokens mod page_size (page_size when it divides);
//   * fork (context.rs:147-225): the child shares every FULL page by reference count; the partly
//     filled last page gets a private copy here (the reference drops and recomputes it);
//   * a page returns to the free list when its last holder lets go
//     (sdk/rust/inferlet/src/forward.rs:28-55, runtime/src/model/resource.rs:225-254); its contents stay.
// Requests are processed in the order they are listed: the i-th page needed by a call gets the i-th
// smallest free id, which is what a host loop over the same list does with the host pool.
//
// State (all int32, in one caller-owned buffer): header | npages[R] | last_len[R] | table[R][C] |
// refs[P] | free bitmap.  Every mutating kernel is a single block on the caller's stream, so calls are
// ordered by the stream and need no locking.
#include "common.cuh"

namespace piekv {
namespace {

constexpr int kPsThreads = 1024;
constexpr int kPsMaxList = 1024;   // slots per call
constexpr int kPsMaxAlloc = 4096;  // pages allocated per call
constexpr int kHdrWords = 16;      // [0] free pages, [1] P, [2] R, [3] C, [4] page_size

struct PageState {
  int32_t *hdr;
  int32_t *npages;
  int32_t *last_len;
  int32_t *table;
  int32_t *refs;
  uint32_t *free_bits;
  int P, R, C, W, page_size;
};

int64_t state_words(int P, int R, int C) {
  const int64_t W = (P + 31) / 32;
  return kHdrWords + 2ll * R + (int64_t)R * C + P + W;
}

PageState view(int32_t *buf, int P, int R, int C, int page_size) {
  PageState s;
  s.P = P;
  s.R = R;
  s.C = C;
  s.W = (P + 31) / 32;
  s.page_size = page_size;
  s.hdr = buf;
  s.npages = buf + kHdrWords;
  s.last_len = s.npages + R;
  s.table = s.last_len + R;
  s.refs = s.table + (size_t)R * C;
  s.free_bits = reinterpret_cast<uint32_t *>(s.refs + P);
  return s;
}

__global__ void __launch_bounds__(kPsThreads) ps_init_kernel(PageState s) {
  const int64_t words = kHdrWords + 2ll * s.R + (int64_t)s.R * s.C + s.P;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (int64_t)gridDim.x * blockDim.x)
    s.hdr[i] = 0;
  for (int w = blockIdx.x * blockDim.x + threadIdx.x; w < s.W; w += gridDim.x * blockDim.x) {
    const int left = s.P - w * 32;
    s.free_bits[w] = left >= 32 ? 0xffffffffu : (1u << left) - 1u;
  }
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    s.hdr[0] = s.P;
    s.hdr[1] = s.P;
    s.hdr[2] = s.R;
    s.hdr[3] = s.C;
    s.hdr[4] = s.page_size;
  }
}

// block-wide exclusive scan of one int per thread; returns the exclusive prefix, *total = sum
__device__ int block_scan(int v, int *total, int *sh /* [33] */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  __syncthreads();  // sh may still be read from an earlier scan
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
    if (lane == 31) sh[32] = w;
  }
  __syncthreads();
  *total = sh[32];
  return (warp > 0 ? sh[warp - 1] : 0) + x - v;
}

// The `total` smallest free page ids, ids[r] = the r-th smallest, taken off the free list (reference
// count 1).  Whole block; `pref` [kPsThreads] and `sh` [33] are shared scratch.  Returns false (and takes
// nothing) when fewer than `total` pages are free.
__device__ bool take_smallest(const PageState &s, int total, int *ids /* shared [kPsMaxAlloc] */, int *pref, int *sh) {
  const int tid = threadIdx.x;
  const int wpt = (s.W + kPsThreads - 1) / kPsThreads;
  const int w0 = min(s.W, tid * wpt), w1 = min(s.W, w0 + wpt);
  int cnt = 0;
  for (int w = w0; w < w1; ++w) cnt += __popc(s.free_bits[w]);
  int total_free;
  const int excl = block_scan(cnt, &total_free, sh);
  pref[tid] = excl;
  __syncthreads();
  if (total > total_free) return false;
  for (int r = tid; r < total; r += kPsThreads) {
    int lo = 0, hi = kPsThreads - 1;  // last thread whose exclusive prefix is <= r
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (pref[mid] <= r)
        lo = mid;
      else
        hi = mid - 1;
    }
    int k = r - pref[lo];
    int w = min(s.W, lo * wpt);
    uint32_t word = s.free_bits[w];
    while (k >= __popc(word)) {  // ends inside this thread's words: its count exceeds k
      k -= __popc(word);
      word = s.free_bits[++w];
    }
    ids[r] = w * 32 + (int)__fns(word, 0, k + 1);
  }
  __syncthreads();  // every rank has been located before any bit changes
  for (int r = tid; r < total; r += kPsThreads) {
    const int id = ids[r];
    atomicAnd(&s.free_bits[id >> 5], ~(1u << (id & 31)));
    s.refs[id] = 1;
  }
  if (tid == 0) s.hdr[0] -= total;
  __syncthreads();
  return true;
}

// one reference of `page` goes away; the page returns to the free list with the last one
__device__ __forceinline__ void drop_ref(const PageState &s, int page, int *freed) {
  if (page < 0 || page >= s.P) return;
  if (atomicSub(&s.refs[page], 1) == 1) {
    atomicOr(&s.free_bits[page >> 5], 1u << (page & 31));
    atomicAdd(freed, 1);
  }
}

// Grow (or shrink) the listed requests by deltas[i] tokens (delta_all when deltas == nullptr), then write
// the batch's CSR header: kv_indptr, kv_last_page_len and pos_ids (= tokens held before the call, the
// position of the first new token).  Shrinks are applied before any page is handed out.
__global__ void __launch_bounds__(kPsThreads)
    ps_adjust_kernel(PageState s, const int32_t *__restrict__ slots, const int32_t *__restrict__ deltas, int delta_all,
                     int n, int32_t *kv_indptr, int32_t *kv_last_page_len, int32_t *pos_ids, int32_t *err) {
  __shared__ int ids[kPsMaxAlloc];
  __shared__ int pref[kPsThreads];
  __shared__ int base[kPsMaxList + 1];
  __shared__ int old_np[kPsMaxList];
  __shared__ int sh[33];
  __shared__ int freed, bad;
  const int tid = threadIdx.x;
  if (tid == 0) freed = bad = 0;
  __syncthreads();
  int slot = -1, np = 0, need = 0, required = 0, new_total = 0, old_total = 0;
  if (tid < n) {
    slot = slots[tid];
    if (slot < 0 || slot >= s.R) {
      report_error(err, PIEKV_ERR_SLOT, KID_PAGES, tid, slot);
      atomicExch(&bad, 1);
      slot = -1;
    } else {
      np = s.npages[slot];
      old_total = np > 0 ? (np - 1) * s.page_size + s.last_len[slot] : 0;
      new_total = max(0, old_total + (deltas != nullptr ? deltas[tid] : delta_all));
      required = (new_total + s.page_size - 1) / s.page_size;
      if (required > s.C) {
        report_error(err, PIEKV_ERR_PAGE_CAPACITY, KID_PAGES, slot, required);
        atomicExch(&bad, 1);
      }
      need = max(0, required - np);
      for (int j = required; j < np; ++j) drop_ref(s, s.table[(size_t)slot * s.C + j], &freed);  // shrink
    }
  }
  int total;
  const int b0 = block_scan(need, &total, sh);
  if (tid < n) {
    base[tid] = b0;
    old_np[tid] = np;
  }
  if (tid == 0) base[n] = total;
  __syncthreads();
  if (tid == 0 && freed) s.hdr[0] += freed;
  if (total > kPsMaxAlloc) {
    if (tid == 0) report_error(err, PIEKV_ERR_PAGE_CAPACITY, KID_PAGES, -1, total);
    return;
  }
  if (bad) return;
  if (!take_smallest(s, total, ids, pref, sh)) {
    if (tid == 0) report_error(err, PIEKV_ERR_NO_FREE_PAGE, KID_PAGES, total, s.hdr[0]);
    return;
  }
  for (int r = tid; r < total; r += kPsThreads) {
    int lo = 0, hi = n - 1;  // request whose range [base[i], base[i+1]) holds r
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (base[mid] <= r)
        lo = mid;
      else
        hi = mid - 1;
    }
    s.table[(size_t)slots[lo] * s.C + old_np[lo] + (r - base[lo])] = ids[r];
  }
  int last = 0;
  if (slot >= 0) {
    const int rem = new_total % s.page_size;
    last = (rem == 0 && new_total > 0) ? s.page_size : rem;
    s.npages[slot] = required;
    s.last_len[slot] = last;
  }
  if (kv_indptr != nullptr) {
    int tot_pages;
    const int off = block_scan(slot >= 0 ? required : 0, &tot_pages, sh);
    if (tid < n) {
      kv_indptr[tid] = off;
      if (kv_last_page_len) kv_last_page_len[tid] = last;
      if (pos_ids) pos_ids[tid] = old_total;
    }
    if (tid == 0) kv_indptr[n] = tot_pages;
  }
}

// kv_indices of the batch from the per-request rows.  One block per request.
__global__ void ps_gather_kernel(PageState s, const int32_t *__restrict__ slots, const int32_t *__restrict__ kv_indptr,
                                 int32_t *kv_indices) {
  const int i = blockIdx.x;
  const int slot = slots[i];
  if (slot < 0 || slot >= s.R) return;
  const int o = kv_indptr[i], np = kv_indptr[i + 1] - o;
  const int32_t *row = s.table + (size_t)slot * s.C;
  for (int j = threadIdx.x; j < np; j += blockDim.x) kv_indices[o + j] = row[j];
}

// The listed requests let go of all their pages.
__global__ void __launch_bounds__(kPsThreads)
    ps_release_kernel(PageState s, const int32_t *__restrict__ slots, int n, int32_t *err) {
  __shared__ int freed;
  if (threadIdx.x == 0) freed = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = warp; i < n; i += kPsThreads / 32) {
    const int slot = slots[i];
    if (slot < 0 || slot >= s.R) {
      if (lane == 0) report_error(err, PIEKV_ERR_SLOT, KID_PAGES, i, slot);
      continue;
    }
    const int np = s.npages[slot];
    for (int j = lane; j < np; j += 32) drop_ref(s, s.table[(size_t)slot * s.C + j], &freed);
    __syncwarp();
    if (lane == 0) {
      s.npages[slot] = 0;
      s.last_len[slot] = 0;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && freed) s.hdr[0] += freed;
}

// children[i] becomes a copy-on-write fork of parents[i]: full pages shared, a partly filled last page
// replaced by a fresh one; (copy_src, copy_dst, copy_valid)[i] is the page copy that completes the fork
// (valid 0 and src == dst when there is nothing to copy).  A child slot must be empty.
__global__ void __launch_bounds__(kPsThreads)
    ps_fork_kernel(PageState s, const int32_t *__restrict__ parents, const int32_t *__restrict__ children, int n,
                   int32_t *copy_src, int32_t *copy_dst, int32_t *copy_valid, int32_t *err) {
  __shared__ int ids[kPsMaxAlloc];
  __shared__ int pref[kPsThreads];
  __shared__ int sh[33];
  __shared__ int bad;
  const int tid = threadIdx.x;
  if (tid == 0) bad = 0;
  __syncthreads();
  int par = -1, chi = -1, np = 0, last = 0, need = 0;
  if (tid < n) {
    par = parents[tid];
    chi = children[tid];
    if (par < 0 || par >= s.R || chi < 0 || chi >= s.R || par == chi || s.npages[chi] != 0) {
      report_error(err, PIEKV_ERR_SLOT, KID_PAGES, tid, chi);
      atomicExch(&bad, 1);
      par = chi = -1;
    } else {
      np = s.npages[par];
      last = s.last_len[par];
      need = (np > 0 && last < s.page_size) ? 1 : 0;
    }
  }
  int total;
  const int rank = block_scan(need, &total, sh);
  __syncthreads();
  if (bad) return;
  if (!take_smallest(s, total, ids, pref, sh)) {
    if (tid == 0) report_error(err, PIEKV_ERR_NO_FREE_PAGE, KID_PAGES, total, s.hdr[0]);
    return;
  }
  if (tid < n) {
    s.npages[chi] = np;
    s.last_len[chi] = last;
    int src = 0, dst = 0, valid = 0;
    if (need) {
      src = s.table[(size_t)par * s.C + np - 1];
      dst = ids[rank];
      valid = last;
      s.table[(size_t)chi * s.C + np - 1] = dst;
    }
    copy_src[tid] = src;
    copy_dst[tid] = dst;
    copy_valid[tid] = valid;
  }
  __syncthreads();
  // shared pages: one warp per fork copies the row and takes a reference on every shared page
  const int warp = tid >> 5, lane = tid & 31;
  for (int i = warp; i < n; i += kPsThreads / 32) {
    const int p_ = parents[i], c_ = children[i];
    const int npp = s.npages[p_];
    const int shared = (npp > 0 && s.last_len[p_] < s.page_size) ? npp - 1 : npp;
    for (int j = lane; j < shared; j += 32) {
      const int page = s.table[(size_t)p_ * s.C + j];
      s.table[(size_t)c_ * s.C + j] = page;
      if (page >= 0 && page < s.P) atomicAdd(&s.refs[page], 1);
    }
  }
}

int check_state(const void *state, int P, int R, int C, int page_size, const char *who) {
  PIEKV_REQUIRE(state != nullptr && (reinterpret_cast<uintptr_t>(state) & 15) == 0, "%s: state is null or not 16-byte aligned", who);
  PIEKV_REQUIRE(P > 0 && R > 0 && C > 0 && page_size > 0, "%s: bad sizes", who);
  return 0;
}

}  // namespace
}  // namespace piekv

using namespace piekv;

extern "C" int64_t piekv_pagestate_bytes(int32_t num_pages, int32_t max_requests, int32_t pages_per_request) {
  if (num_pages <= 0 || max_requests <= 0 || pages_per_request <= 0) return 0;
  return state_words(num_pages, max_requests, pages_per_request) * 4;
}

extern "C" int piekv_pagestate_init(void *state, int64_t state_bytes, int32_t num_pages, int32_t max_requests,
                                    int32_t pages_per_request, int32_t page_size, void *stream) {
  if (int rc = check_state(state, num_pages, max_requests, pages_per_request, page_size, "pagestate_init")) return rc;
  PIEKV_REQUIRE(state_bytes >= piekv_pagestate_bytes(num_pages, max_requests, pages_per_request),
                "pagestate_init: %lld bytes given, %lld needed", (long long)state_bytes,
                (long long)piekv_pagestate_bytes(num_pages, max_requests, pages_per_request));
  PageState s = view(reinterpret_cast<int32_t *>(state), num_pages, max_requests, pages_per_request, page_size);
  ps_init_kernel<<<1, kPsThreads, 0, (cudaStream_t)stream>>>(s);
  PIEKV_LAUNCH_CHECK("ps_init_kernel");
  return 0;
}

extern "C" int piekv_pagestate_adjust(void *state, int32_t num_pages, int32_t max_requests, int32_t pages_per_request,
                                      int32_t page_size, const int32_t *slots, const int32_t *deltas,
                                      int32_t delta_all, int32_t count, int32_t *kv_indptr, int32_t *kv_indices,
                                      int32_t *kv_last_page_len, int32_t *pos_ids, int32_t *err, void *stream) {
  if (int rc = check_state(state, num_pages, max_requests, pages_per_request, page_size, "pagestate_adjust")) return rc;
  PIEKV_REQUIRE(count >= 0 && count <= kPsMaxList, "pagestate_adjust: %d requests (at most %d per call)", count, kPsMaxList);
  PIEKV_REQUIRE(count == 0 || slots != nullptr, "pagestate_adjust: null slot list");
  PIEKV_REQUIRE((kv_indices == nullptr) || (kv_indptr != nullptr), "pagestate_adjust: kv_indices needs kv_indptr");
  if (count == 0) return 0;
  PageState s = view(reinterpret_cast<int32_t *>(state), num_pages, max_requests, pages_per_request, page_size);
  ps_adjust_kernel<<<1, kPsThreads, 0, (cudaStream_t)stream>>>(s, slots, deltas, delta_all, count, kv_indptr,
                                                               kv_last_page_len, pos_ids, err);
  PIEKV_LAUNCH_CHECK("ps_adjust_kernel");
  if (kv_indices != nullptr) {
    ps_gather_kernel<<<count, 128, 0, (cudaStream_t)stream>>>(s, slots, kv_indptr, kv_indices);
    PIEKV_LAUNCH_CHECK("ps_gather_kernel");
  }
  return 0;
}

extern "C" int piekv_pagestate_release(void *state, int32_t num_pages, int32_t max_requests, int32_t pages_per_request,
                                       int32_t page_size, const int32_t *slots, int32_t count, int32_t *err,
                                       void *stream) {
  if (int rc = check_state(state, num_pages, max_requests, pages_per_request, page_size, "pagestate_release")) return rc;
  PIEKV_REQUIRE(count >= 0 && (count == 0 || slots != nullptr), "pagestate_release: bad slot list");
  if (count == 0) return 0;
  PageState s = view(reinterpret_cast<int32_t *>(state), num_pages, max_requests, pages_per_request, page_size);
  ps_release_kernel<<<1, kPsThreads, 0, (cudaStream_t)stream>>>(s, slots, count, err);
  PIEKV_LAUNCH_CHECK("ps_release_kernel");
  return 0;
}

extern "C" int piekv_pagestate_fork(void *state, int32_t num_pages, int32_t max_requests, int32_t pages_per_request,
                                    int32_t page_size, const int32_t *parents, const int32_t *children, int32_t count,
                                    int32_t *copy_src, int32_t *copy_dst, int32_t *copy_valid, int32_t *err,
                                    void *stream) {
  if (int rc = check_state(state, num_pages, max_requests, pages_per_request, page_size, "pagestate_fork")) return rc;
  PIEKV_REQUIRE(count >= 0 && count <= kPsMaxList, "pagestate_fork: %d forks (at most %d per call)", count, kPsMaxList);
  PIEKV_REQUIRE(count == 0 || (parents && children && copy_src && copy_dst && copy_valid), "pagestate_fork: null pointer");
  if (count == 0) return 0;
  PageState s = view(reinterpret_cast<int32_t *>(state), num_pages, max_requests, pages_per_request, page_size);
  ps_fork_kernel<<<1, kPsThreads, 0, (cudaStream_t)stream>>>(s, parents, children, count, copy_src, copy_dst,
                                                             copy_valid, err);
  PIEKV_LAUNCH_CHECK("ps_fork_kernel");
  return 0;
}
