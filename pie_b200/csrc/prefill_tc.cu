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
// Warp roles: warps 0-3 softmax (thread = query row = TMEM lane), warp 4 TMA producer, warp 5
// MMA issuer and TMEM owner.  The MMA warp runs one tile ahead on S (S is double buffered), the
// softmax threads keep the running maximum lazily (O in TMEM is only rescaled when the maximum
// grows by more than 2^8), so tile j's softmax overlaps QK of tile j+1 and PV of tile j-1.
//
// Masking: causal with offset (token t allowed iff t <= kv_len - qo_len + row) or none.  A flat
// boolean custom mask is handled by the general kernel (see attn_api.cu).
//
// Every wait is bounded; on a timeout the CTA records PIEKV_ERR_WAIT_TIMEOUT, all roles leave
// their loops, outstanding bulk copies are drained and TMEM is released before the CTA exits.
#include <cuda.h>

#include <type_traits>

#include "attn.cuh"
#include "common.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace piekv {

namespace {

constexpr int kDim = 128;
constexpr int kPage = 16;
constexpr int kBM = 128;  // query rows per CTA
constexpr int kBN = 128;  // kv tokens per tile (8 pages)
constexpr int kStages = 2;
constexpr int kThreads = 192;
constexpr int kTileBytes = 32768;  // one 128 x 128 16-bit operand tile
constexpr int kHalfBytes = 16384;  // one 128 x 64 half of it
constexpr int kSmemBytes = kTileBytes * (1 + 2 * kStages + 1) + 1024;
constexpr int kTmemCols = 512;
constexpr int kColS = 0, kColO = 256;
constexpr int kCounterBytes = 65536;
constexpr int kSortBins = 1024;

struct PrefillParams {
  AttnArgs a;
  const int2 *tiles;  // (request, first row of the tile within the request), heaviest first
  const int *ntiles;
};

// ------------------------------------------------------------------------------------------------
// work list: one entry per (request, 128-row tile), ordered by decreasing number of kv tiles
// ------------------------------------------------------------------------------------------------
__global__ void prefill_plan_kernel(const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                                    const int32_t *__restrict__ kv_last_page_len, int batch, int page_size, int causal,
                                    int2 *tiles, int *ntiles, int max_tiles) {
  __shared__ int hist[kSortBins];
  for (int i = threadIdx.x; i < kSortBins; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  auto key_of = [&](int qo_len, int kv_len, int r0) {
    int hi = causal ? min(kv_len, kv_len - qo_len + r0 + kBM) : kv_len;
    int nt = hi > 0 ? (hi + kBN - 1) / kBN : 0;
    nt = nt < kSortBins ? nt : kSortBins - 1;
    return kSortBins - 1 - nt;  // bin 0 = most work
  };
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    int qo_len = qo_indptr[b + 1] - qo_indptr[b];
    int np = kv_indptr[b + 1] - kv_indptr[b];
    int kv_len = np > 0 ? (np - 1) * page_size + kv_last_page_len[b] : 0;
    for (int r0 = 0; r0 < qo_len; r0 += kBM) atomicAdd(&hist[key_of(qo_len, kv_len, r0)], 1);
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
  }
  __syncthreads();
  for (int b = threadIdx.x; b < batch; b += blockDim.x) {
    int qo_len = qo_indptr[b + 1] - qo_indptr[b];
    int np = kv_indptr[b + 1] - kv_indptr[b];
    int kv_len = np > 0 ? (np - 1) * page_size + kv_last_page_len[b] : 0;
    for (int r0 = 0; r0 < qo_len; r0 += kBM) {
      int pos = atomicAdd(&hist[key_of(qo_len, kv_len, r0)], 1);
      if (pos < max_tiles) tiles[pos] = make_int2(b, r0);
    }
  }
}

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

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
    prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                      const __grid_constant__ PrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full[2], s_empty[2], p_full, pv_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int sh_abort;

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
  const int kv_hi = a.causal ? min(kv_len, kv_len - qo_len + r0 + kBM) : kv_len;
  const int n_tiles = kv_hi > 0 ? (kv_hi + kBN - 1) / kBN : 0;
  T *out = reinterpret_cast<T *>(a.out);

  if (n_tiles == 0) {  // nothing to attend to: zeros (uniform for the whole CTA, before any allocation)
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
  const uint32_t kv_smem = base + kTileBytes;                    // stage s: K at +s*64K, V at +s*64K+32K
  const uint32_t p_smem = base + kTileBytes * (1 + 2 * kStages);
  uint8_t *p_ptr = base_ptr + kTileBytes * (1 + 2 * kStages);

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 128);
    }
    mbar_init(&p_full, 128);
    mbar_init(&pv_done, 1);
    sh_abort = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tc::tmem_alloc(&tmem_slot, kTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int *abort_flag = &sh_abort;
  constexpr bool kBf16 = sizeof(T) == 2 && !std::is_same<T, __half>::value;

  if (warp == 4) {
    // ================================================================== TMA producer
    int armed = 0;
    if (lane == 0) {
      mbar_arrive_expect_tx(&q_full, kTileBytes);
      tma_load_4d(q_smem, &tmap_q, 0, q0 + r0, 0, h, &q_full);
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int s = j % kStages;
      const uint32_t k = j / kStages;
      // page id of this lane's page (lanes 0-7), loaded before the wait so it is in flight
      const int pi = j * 8 + lane;
      int page = (lane < 8 && pi < np) ? __ldg(a.kv_indices + p0 + pi) : a.num_pages;
      if (lane < 8 && pi < np && (page < 0 || page >= a.num_pages)) {
        report_error(a.err, PIEKV_ERR_PAGE_ID, KID_PREFILL, p0 + pi, page);
        page = a.num_pages;  // outside the tensor map: zero fill
      }
      if (!wait_or_abort(&kv_empty[s], (k & 1) ^ 1, abort_flag)) {
        if (lane == 0 && !*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 100 + s);
        if (lane == 0) atomicExch(&sh_abort, 1);
        break;
      }
      if (lane == 0) mbar_arrive_expect_tx(&kv_full[s], 2 * kTileBytes);
      __syncwarp();
      if (lane < 8) {
        // pages beyond the request's list use an out-of-range coordinate: the rows are zero-filled
        const uint32_t kdst = kv_smem + s * 2 * kTileBytes + lane * 2048;
        const uint32_t vdst = kdst + kTileBytes;
        tma_load_5d(kdst, &tmap_kv, 0, 0, 0, hk, page * 2, &kv_full[s]);
        tma_load_5d(kdst + kHalfBytes, &tmap_kv, 0, 0, 1, hk, page * 2, &kv_full[s]);
        tma_load_5d(vdst, &tmap_kv, 0, 0, 0, hk, page * 2 + 1, &kv_full[s]);
        tma_load_5d(vdst + kHalfBytes, &tmap_kv, 0, 0, 1, hk, page * 2 + 1, &kv_full[s]);
      }
      ++armed;
    }
    // drain: the CTA must not retire while a bulk copy may still be landing
    __syncwarp();
    if (lane == 0) {
      mbar_wait(&q_full, 0, 200000000ull);
      const int first = armed > kStages ? armed - kStages : 0;
      for (int j = first; j < armed; ++j) mbar_wait(&kv_full[j % kStages], (j / kStages) & 1, 200000000ull);
    }
  } else if (warp == 5) {
    // ================================================================== MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::instr_desc(kBf16, false, false, kBM, kBN);
      constexpr uint32_t idesc_pv = tc::instr_desc(kBf16, false, true, kBM, kDim);
      bool ok = wait_or_abort(&q_full, 0, abort_flag);
      for (int j = 0; ok && j <= n_tiles; ++j) {
        if (j < n_tiles) {
          const int s = j % kStages, sb = j & 1;
          ok = wait_or_abort(&kv_full[s], (j / kStages) & 1, abort_flag) &&
               wait_or_abort(&s_empty[sb], ((j >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc::fence_after_sync();
          const uint32_t k_smem = kv_smem + s * 2 * kTileBytes;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
            tc::mma_ss(tmem + kColS + sb * kBN, tc::desc_k_major(q_smem + off), tc::desc_k_major(k_smem + off),
                       idesc_qk, ks > 0 ? 1u : 0u);
          }
          tc::commit(&s_full[sb]);
        }
        if (j >= 1) {
          const int jj = j - 1, s = jj % kStages;
          ok = wait_or_abort(&p_full, jj & 1, abort_flag);
          if (!ok) break;
          tc::fence_after_sync();
          const uint32_t v_smem = kv_smem + s * 2 * kTileBytes + kTileBytes;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            tc::mma_ss(tmem + kColO, tc::desc_k_major(p_smem + (ks >> 2) * kHalfBytes + (ks & 3) * 32),
                       tc::desc_mn_major(v_smem + ks * 2048, kHalfBytes), idesc_pv, (jj > 0 || ks > 0) ? 1u : 0u);
          }
          tc::commit(&pv_done);
          tc::commit(&kv_empty[s]);
        }
      }
      if (!ok) {
        if (!*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 200);
        atomicExch(&sh_abort, 1);
      }
    }
  } else {
    // ================================================================== softmax (thread = row)
    const int row = warp * 32 + lane;             // row of the tile = TMEM lane
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const bool row_valid = row < rows;
    // last allowed token of this row (inclusive)
    const int limit = row_valid ? (a.causal ? min(kv_len - 1, kv_len - qo_len + r0 + row) : kv_len - 1) : -1;
    const float c = a.sm_scale * 1.4426950408889634f;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    uint32_t sreg[128];

    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      ok = wait_or_abort(&s_full[sb], (j >> 1) & 1, abort_flag);
      if (!ok) break;
      tc::fence_after_sync();
      const uint32_t s_addr = tmem + lane_base + kColS + sb * kBN;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) tc::tmem_ld32(s_addr + ch * 32, sreg + ch * 32);
      tc::tmem_wait_ld();
      tc::fence_before_sync();
      mbar_arrive(&s_empty[sb]);  // S is in registers: the MMA warp may overwrite this buffer

      // ---- running maximum (lazy) and probabilities
      const int t0 = j * kBN;
      const bool full_tile = t0 + kBN - 1 <= limit;  // no masking needed for this row
      float mx = -INFINITY;
      if (full_tile) {
#pragma unroll
        for (int i = 0; i < 128; ++i) mx = fmaxf(mx, __uint_as_float(sreg[i]));
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          const float v = (t0 + i <= limit) ? __uint_as_float(sreg[i]) : -INFINITY;
          sreg[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      }
      mx *= c;  // c > 0
      float alpha = 1.f;
      bool rescale = false;
      if (mx > m_ref + 8.f) {
        alpha = fast_exp2(m_ref - mx);  // m_ref = -inf on the first hit: 0
        l *= alpha;
        m_ref = mx;
        rescale = j > 0;
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const float p0v = fast_exp2(fmaf(__uint_as_float(sreg[2 * i]), c, -m_use));
        const float p1v = fast_exp2(fmaf(__uint_as_float(sreg[2 * i + 1]), c, -m_use));
        sum += p0v + p1v;
        sreg[i] = pack2<T>(p0v, p1v);  // tokens 2i, 2i+1
      }
      l += sum;

      // ---- P buffer free and O stable once PV of the previous tile has completed
      if (j > 0) {
        ok = wait_or_abort(&pv_done, (j - 1) & 1, abort_flag);
        if (!ok) break;
        tc::fence_after_sync();
      }
      if (__any_sync(0xffffffffu, rescale)) {
        const uint32_t o_addr = tmem + lane_base + kColO;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t oreg[32];
          tc::tmem_ld32(o_addr + ch * 32, oreg);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) oreg[i] = __float_as_uint(__uint_as_float(oreg[i]) * alpha);
          tc::tmem_st32(o_addr + ch * 32, oreg);
        }
        tc::tmem_wait_st();
      }
      // ---- P -> shared memory, K-major with 128-byte swizzle: row r, 16-byte chunk ch of token half hf
      {
        uint8_t *prow = p_ptr + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          const int hf = ch >> 3, cc = ch & 7;
          *reinterpret_cast<uint4 *>(prow + hf * kHalfBytes + ((cc ^ (row & 7)) << 4)) =
              make_uint4(sreg[ch * 4], sreg[ch * 4 + 1], sreg[ch * 4 + 2], sreg[ch * 4 + 3]);
        }
      }
      fence_proxy_async_smem();
      tc::fence_before_sync();
      mbar_arrive(&p_full);
    }

    // ---- epilogue: O / l -> out
    if (ok) ok = wait_or_abort(&pv_done, (n_tiles - 1) & 1, abort_flag);
    if (ok) {
      tc::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T *orow = out + ((size_t)(q0 + r0 + row) * a.hq + h) * kDim;
      const uint32_t o_addr = tmem + lane_base + kColO;
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
        a.lse[(size_t)(q0 + r0 + row) * a.hq + h] = l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    } else {
      if (lane == 0 && !*abort_flag) report_error(a.err, PIEKV_ERR_WAIT_TIMEOUT, KID_PREFILL, blockIdx.x, 300 + warp);
      if (lane == 0) atomicExch(&sh_abort, 1);
    }
  }

  // ---- teardown: every thread arrives here on every path
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 5) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace

bool prefill_tc_supported(const AttnArgs &a, int dtype) {
  if (dtype != PIEKV_BF16 && dtype != PIEKV_F16) return false;
  if (a.dim != kDim || a.page_size != kPage) return false;
  if (a.mask != nullptr) return false;
  if (a.hq % a.hkv != 0) return false;
  if ((reinterpret_cast<uintptr_t>(a.pool) & 15) || (reinterpret_cast<uintptr_t>(a.q) & 15) ||
      (reinterpret_cast<uintptr_t>(a.out) & 15))
    return false;
  if ((a.q_sn & 7) || (a.q_sh & 7)) return false;
  return true;
}

static int64_t max_tiles_of(int batch, int nnz) { return (int64_t)(nnz + kBM - 1) / kBM + batch; }

int64_t prefill_tc_workspace_bytes(int batch, int nnz, int hq) {
  (void)hq;
  return kCounterBytes + 256 + max_tiles_of(batch, nnz) * (int64_t)sizeof(int2);
}

template <typename T>
static int launch_prefill_t(const AttnArgs &a, const CUtensorMap &tq, const CUtensorMap &tkv, const PrefillParams &p,
                            int max_tiles, cudaStream_t st) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(prefill_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return cuda_status(e, "prefill: cudaFuncSetAttribute");
    configured = true;
  }
  const long long blocks = (long long)max_tiles * a.hq;
  PIEKV_REQUIRE(blocks < (1ll << 31), "prefill: too many tiles");
  prefill_tc_kernel<T><<<(unsigned)blocks, kThreads, kSmemBytes, st>>>(tq, tkv, p);
  PIEKV_LAUNCH_CHECK("prefill_tc_kernel");
  return 0;
}

int launch_prefill_tc(const AttnArgs &a, int dtype, void *workspace, int64_t workspace_bytes, cudaStream_t st) {
  if (a.nnz == 0 || a.batch == 0) return 0;
  const int64_t need = prefill_tc_workspace_bytes(a.batch, a.nnz, a.hq);
  PIEKV_REQUIRE(workspace != nullptr && workspace_bytes >= need, "prefill: workspace too small (%lld < %lld bytes)",
                (long long)workspace_bytes, (long long)need);
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, "prefill: workspace must be 256-byte aligned");
  const int max_tiles = (int)max_tiles_of(a.batch, a.nnz);
  uint8_t *ws = reinterpret_cast<uint8_t *>(workspace) + kCounterBytes;
  PrefillParams p;
  p.a = a;
  p.ntiles = reinterpret_cast<int *>(ws);
  p.tiles = reinterpret_cast<int2 *>(ws + 256);
  prefill_plan_kernel<<<1, 1024, 0, st>>>(a.qo_indptr, a.kv_indptr, a.kv_last_page_len, a.batch, a.page_size, a.causal,
                                          const_cast<int2 *>(p.tiles), const_cast<int *>(p.ntiles), max_tiles);
  PIEKV_LAUNCH_CHECK("prefill_plan_kernel");
  CUtensorMap tq, tkv;
  if (int rc = make_q_tensor_map(&tq, a.q, a.nnz, a.hq, a.q_sn, a.q_sh, dtype, kBM)) return rc;
  if (int rc = make_page_tensor_map(&tkv, a.pool, a.num_pages, a.hkv, dtype, 1, 1, 1)) return rc;
  if (dtype == PIEKV_BF16) return launch_prefill_t<__nv_bfloat16>(a, tq, tkv, p, max_tiles, st);
  return launch_prefill_t<__half>(a, tq, tkv, p, max_tiles, st);
}

}  // namespace piekv
