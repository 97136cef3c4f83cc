// QKV projection with the RoPE + append epilogue (sm_100a tcgen05 / TMEM).
//
//   qkv[n, (Hq + 2 Hkv) D] = x[n, hidden] . w[(Hq + 2 Hkv) D, hidden]^T        (D = 128)
//
// never reaches memory as such: the accumulator tile of 128 tokens x one or two heads stays in tensor
// memory in fp32, and the epilogue thread that owns a token row rotates it (q and k heads), rounds it
// ONCE to the storage type and writes it where the next kernel wants it - q rows to `q_out`, k / v rows
// straight into the token's slot of the paged pool.  This is the step before the paged-KV path in the
// reference's layer (pie/src/pie_worker/model/llama3.py:627-685: linear, split, RoPE in place, append).
//
// Persistent CTAs, one per SM; a tile is 128 tokens x NH heads (NH = 2 when the head count is even: an MMA
// with N = 256 does twice the work per instruction and per byte of x staged); tile t -> (token tile, head
// group) with the head group fastest, so the CTAs that run at the same time share their rows of x through L2.
// Per tile: hidden / 64 k-blocks; a k-block is one TMA box of x (128 x 64, K-major, 128-byte swizzle) and one
// of w (NH * 128 x 64), four tcgen05.mma (M128, N = NH * 128, K16) each.  Four stages of 32 or 48 KiB; two
// accumulators (2 x NH * 128 TMEM columns) so that the epilogue of a tile runs under the MMAs of the next.
// Roles: warps 0-7 epilogue (thread = token row = TMEM lane; the two warps of a lane quarter take one head
// each: the rotation's cos / sin are the epilogue's cost), warp 8 TMA producer, warp 9 MMA issuer and TMEM
// owner.  Every wait is bounded (2 s); on expiry the error word is set and all roles leave.
#include <type_traits>

#include "rope.cuh"
#include "tcgen05.cuh"
#include "tma.cuh"

namespace piekv {

namespace {

constexpr int kQDim = 128;
constexpr int kQBM = 128, kQBK = 64;
constexpr int kQStages = 4;
constexpr int kQTileBytes = kQBM * kQBK * 2;  // 128 rows x 64 16-bit elements
constexpr int kQEpiWarps = 8, kQProducerWarp = 8, kQMmaWarp = 9;
constexpr int kQThreads = 32 * (kQEpiWarps + 2);

struct QkvParams {
  int n, hidden, hq, hkv;
  void *q_out;  // [n, Hq, 128]
  void *pool;   // [P, 2, page, Hkv, 128]
  const int32_t *pos_ids, *batch_indices, *positions, *kv_indices, *kv_indptr;
  int batch, page_size, num_pages;
  int32_t *err;
  const void *bias;     // nullable: [(Hq + 2 Hkv) * 128], added to the projection
  const void *q_norm;   // nullable: [128] weight of a per-head RMSNorm of q, applied before the rotation
  const void *k_norm;   // the same for k
  float rms_eps;
};

template <typename T, int NH>
__global__ void __launch_bounds__(kQThreads, 1)
    qkv_rope_append_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                           const __grid_constant__ QkvParams p, const __grid_constant__ RopeDev rp) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full[kQStages], empty[kQStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_slot;
  __shared__ int sh_abort;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int kQStageBytes = (1 + NH) * kQTileBytes;  // x tile + w tile
  constexpr int kQTmemCols = 2 * NH * kQDim;
  const int heads = (p.hq + 2 * p.hkv) / NH;  // head groups
  const int m_tiles = (p.n + kQBM - 1) / kQBM;
  const int tiles = m_tiles * heads;
  const int kblocks = p.hidden / kQBK;
  constexpr bool kBf16 = !std::is_same<T, __half>::value;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], kQEpiWarps);
    }
    sh_abort = 0;
    mbar_fence_init();
  }
  if (warp == kQMmaWarp) {
    tc::tmem_alloc(&tmem_slot, kQTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int *abort_flag = &sh_abort;
  auto wait = [&](uint64_t *bar, uint32_t parity, int where) -> bool {
    if (*abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    if (lane == 0 || warp >= kQEpiWarps) report_error(p.err, PIEKV_ERR_WAIT_TIMEOUT, KID_APPEND, blockIdx.x, where);
    atomicExch(&sh_abort, 1);
    return false;
  };

  if (warp == kQProducerWarp) {
    if (lane == 0) {
      int it = 0;  // k-blocks issued so far (all tiles)
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int m = t / heads, h = t - m * heads;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kQStages;
          ok = wait(&empty[s], ((it / kQStages) & 1) ^ 1, 100);
          if (!ok) break;
          mbar_arrive_expect_tx(&full[s], kQStageBytes);
          const uint32_t dst = base + s * kQStageBytes;
          tma_load_2d(dst, &tmap_x, kb * kQBK, m * kQBM, &full[s]);
          tma_load_2d(dst + kQTileBytes, &tmap_w, kb * kQBK, h * NH * kQDim, &full[s]);
        }
        if (!ok) break;
      }
      // drain: nothing may still be landing when the CTA retires
      for (int x = it > kQStages ? it - kQStages : 0; x < it; ++x)
        mbar_wait(&full[x % kQStages], (x / kQStages) & 1, 200000000ull);
    }
  } else if (warp == kQMmaWarp) {
    if (lane == 0) {
      constexpr uint32_t idesc = tc::instr_desc(kBf16, false, false, kQBM, NH * kQDim);
      int it = 0, nt = 0;  // k-blocks / tiles consumed so far
      for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++nt) {
        const int buf = nt & 1;
        // the epilogue has read this accumulator's previous tile
        if (!wait(&acc_empty[buf], ((nt >> 1) & 1) ^ 1, 200)) break;
        tc::fence_after_sync();
        const uint32_t d = tmem + buf * NH * kQDim;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % kQStages;
          ok = wait(&full[s], (it / kQStages) & 1, 210);
          if (!ok) break;
          tc::fence_after_sync();
          const uint64_t a_desc = tc::desc_k_major(base + s * kQStageBytes);
          const uint64_t b_desc = tc::desc_k_major(base + s * kQStageBytes + kQTileBytes);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::mma_ss(d, a_desc + (uint64_t)((ks * 32) >> 4), b_desc + (uint64_t)((ks * 32) >> 4), idesc,
                       (kb > 0 || ks > 0) ? 1u : 0u);
          tc::commit(&empty[s]);
        }
        if (!ok) break;
        tc::commit(&acc_full[buf]);
      }
    }
  } else {
    // ================================================ epilogue: thread = token row; warps w and w + 4 own the
    // same 32 rows (TMEM lanes) and take one head of the tile each
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    T *q_out = reinterpret_cast<T *>(p.q_out);
    T *pool = reinterpret_cast<T *>(p.pool);
    const size_t half_page = (size_t)p.page_size * p.hkv * kQDim;
    int nt = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++nt) {
      const int m = t / heads, hg = t - m * heads;
      const int buf = nt & 1;
      const int tok = m * kQBM + r;
      const bool row_ok = tok < p.n;
      if (!wait(&acc_full[buf], (nt >> 1) & 1, 300 + warp)) break;
      __syncwarp();
      tc::fence_after_sync();
#pragma unroll 1
      for (int hh = warp >> 2; hh < NH; hh += 2) {
      const int h = hg * NH + hh;
      // where the row goes, and whether it is rotated
      T *dst = nullptr;
      const bool is_q = h < p.hq, is_k = !is_q && h < p.hq + p.hkv;
      int pos_id = 0;
      if (row_ok) {
        if (is_q) {
          dst = q_out + ((size_t)tok * p.hq + h) * kQDim;
        } else {
          const int hk = is_k ? h - p.hq : h - p.hq - p.hkv;
          const int b = p.batch_indices[tok];
          const int pos = p.positions[tok];
          if (b < 0 || b >= p.batch) {
            report_error(p.err, PIEKV_ERR_BATCH_INDEX, KID_APPEND, tok, b);
          } else {
            const int p0 = p.kv_indptr[b], p1 = p.kv_indptr[b + 1];
            const int slot = pos >= 0 ? pos / p.page_size : -1;
            if (slot < 0 || p0 + slot >= p1) {
              report_error(p.err, PIEKV_ERR_PAGE_SLOT, KID_APPEND, tok, pos);
            } else {
              const int page = p.kv_indices[p0 + slot];
              if (page < 0 || page >= p.num_pages)
                report_error(p.err, PIEKV_ERR_PAGE_ID, KID_APPEND, tok, page);
              else
                dst = pool + (size_t)page * 2 * half_page + (is_k ? 0 : half_page) +
                      (size_t)(pos % p.page_size) * p.hkv * kQDim + (size_t)hk * kQDim;
            }
          }
        }
        if (is_q || is_k) pos_id = p.pos_ids[tok];
      }
      bool rot = (is_q || is_k) && rp.mode != PIEKV_ROPE_NONE && row_ok;
      if (rot && rp.mode == PIEKV_ROPE_TABLE && (pos_id < 0 || pos_id >= rp.table_len)) {
        report_error(p.err, PIEKV_ERR_TABLE_RANGE, KID_ROPE, tok, pos_id);
        rot = false;  // the row is stored un-rotated, as the separate kernel does
      }
      const uint32_t acc = tmem + lane_base + (buf * NH + hh) * kQDim;
      const T *bias = p.bias != nullptr ? reinterpret_cast<const T *>(p.bias) + (size_t)h * kQDim : nullptr;
      const T *nw = is_q ? reinterpret_cast<const T *>(p.q_norm) : (is_k ? reinterpret_cast<const T *>(p.k_norm) : nullptr);
      float inv_rms = 1.f;
      if (nw != nullptr) {
        // per-head RMSNorm of the row (over its 128 elements) ahead of the rotation: a pass of its own
        // over the accumulator for the sum of squares
        float ss = 0.f;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t v[32];
          tc::tmem_ld32(acc + ch * 32, v);
          tc::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = __uint_as_float(v[i]) + (bias ? Elem<T>::to_f32(bias[ch * 32 + i]) : 0.f);
            ss = fmaf(x, x, ss);
          }
        }
        inv_rms = rsqrtf(ss * (1.f / kQDim) + p.rms_eps);
      }
      // element `col` of the row as the reference has it before the rotation
      auto value = [&](uint32_t raw, int col) {
        float x = __uint_as_float(raw);
        if (bias) x += Elem<T>::to_f32(bias[col]);
        if (nw) x = x * inv_rms * Elem<T>::to_f32(nw[col]);
        return x;
      };
      // pairs (i, i + 64): columns [32c, 32c + 32) with [64 + 32c, 64 + 32c + 32)
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t lo[32], hi[32];
        tc::tmem_ld32(acc + c * 32, lo);
        tc::tmem_ld32(acc + 64 + c * 32, hi);
        tc::tmem_wait_ld();
        if (dst != nullptr) {
          uint32_t olo[16], ohi[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0 = value(lo[i], c * 32 + i), x1 = value(lo[i + 1], c * 32 + i + 1);
            float y0 = value(hi[i], 64 + c * 32 + i), y1 = value(hi[i + 1], 64 + c * 32 + i + 1);
            if (rot) {
              float c0, s0, c1, s1, a0, b0, a1, b1;
              rope_cos_sin1(rp, pos_id, c * 32 + i, 64, c0, s0);
              rope_cos_sin1(rp, pos_id, c * 32 + i + 1, 64, c1, s1);
              rope_rotate(x0, y0, c0, s0, a0, b0);
              rope_rotate(x1, y1, c1, s1, a1, b1);
              x0 = a0, y0 = b0, x1 = a1, y1 = b1;
            }
            olo[i >> 1] = pack2<T>(x0, x1);
            ohi[i >> 1] = pack2<T>(y0, y1);
          }
          uint4 *d_lo = reinterpret_cast<uint4 *>(dst + c * 32);
          uint4 *d_hi = reinterpret_cast<uint4 *>(dst + 64 + c * 32);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            d_lo[v] = make_uint4(olo[4 * v], olo[4 * v + 1], olo[4 * v + 2], olo[4 * v + 3]);
            d_hi[v] = make_uint4(ohi[4 * v], ohi[4 * v + 1], ohi[4 * v + 2], ohi[4 * v + 3]);
          }
        }
      }
      }  // heads of the tile
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the accumulator may be overwritten
    }
  }

  tc::fence_before_sync();
  __syncthreads();
  if (warp == kQMmaWarp) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kQTmemCols);
  }
}

template <typename T, int NH>
int launch_qkv(const CUtensorMap &tx, const CUtensorMap &tw, const QkvParams &p, const RopeDev &rp, cudaStream_t st) {
  constexpr int kQSmemBytes = kQStages * (1 + NH) * kQTileBytes + 1024;
  static unsigned char configured[kMaxDevices] = {0};
  if (int rc = opt_in_dynamic_smem(qkv_rope_append_kernel<T, NH>, kQSmemBytes, configured, "qkv: cudaFuncSetAttribute"))
    return rc;
  const long long tiles = (long long)((p.n + kQBM - 1) / kQBM) * ((p.hq + 2 * p.hkv) / NH);
  const int sms = sm_count();
  PIEKV_REQUIRE(sms > 0, "qkv: cannot read the multiprocessor count");
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  qkv_rope_append_kernel<T, NH><<<grid, kQThreads, kQSmemBytes, st>>>(tx, tw, p, rp);
  PIEKV_LAUNCH_CHECK("qkv_rope_append_kernel");
  return 0;
}

}  // namespace
}  // namespace piekv

extern "C" int piekv_qkv_rope_append_opt(const void *x, int64_t x_stride_n, const void *w_qkv, int64_t w_stride_n,
                                         void *q_out, const int32_t *pos_ids, const int32_t *batch_indices,
                                         const int32_t *positions, void *pool, const int32_t *kv_indices,
                                         const int32_t *kv_indptr, int32_t nnz, int32_t batch, int32_t hidden,
                                         int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim,
                                         int32_t page_size, int32_t num_pages, int32_t dtype,
                                         const piekv_rope_params *rope, int32_t *err, void *stream,
                                         const piekv_qkv_options *opt) {
  using namespace piekv;
  PIEKV_REQUIRE(dtype == PIEKV_BF16 || dtype == PIEKV_F16, "qkv_rope_append: 16-bit types only (dtype %d)", dtype);
  PIEKV_REQUIRE(head_dim == kQDim, "qkv_rope_append: head_dim %d (only 128)", head_dim);
  PIEKV_REQUIRE(nnz >= 0 && batch >= 0 && num_qo_heads > 0 && num_kv_heads > 0 && page_size > 0 && num_pages >= 0,
                "qkv_rope_append: negative size");
  PIEKV_REQUIRE(hidden > 0 && hidden % kQBK == 0, "qkv_rope_append: hidden %d is not a multiple of %d", hidden, kQBK);
  if (nnz == 0) return 0;
  PIEKV_REQUIRE(x && w_qkv && q_out && pool && pos_ids && batch_indices && positions && kv_indices && kv_indptr,
                "qkv_rope_append: null pointer");
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w_qkv) & 15) == 0 &&
                    (x_stride_n * 2) % 16 == 0 && (w_stride_n * 2) % 16 == 0 && x_stride_n >= hidden &&
                    w_stride_n >= hidden,
                "qkv_rope_append: x and w_qkv rows must be 16-byte aligned and at least `hidden` long");
  PIEKV_REQUIRE((reinterpret_cast<uintptr_t>(q_out) & 15) == 0 && (reinterpret_cast<uintptr_t>(pool) & 15) == 0,
                "qkv_rope_append: q_out and the pool must be 16-byte aligned");
  if (int rc = check_rope(rope, head_dim, "qkv_rope_append")) return rc;
  PIEKV_REQUIRE(rope == nullptr || rope->mode == PIEKV_ROPE_NONE || !rope->interleave,
                "qkv_rope_append: interleaved pairs are not supported by the fused epilogue");
  RopeDev rp;
  fill_inv_freq(rope, head_dim, &rp);
  QkvParams p;
  p.n = nnz;
  p.hidden = hidden;
  p.hq = num_qo_heads;
  p.hkv = num_kv_heads;
  p.q_out = q_out;
  p.pool = pool;
  p.pos_ids = pos_ids;
  p.batch_indices = batch_indices;
  p.positions = positions;
  p.kv_indices = kv_indices;
  p.kv_indptr = kv_indptr;
  p.batch = batch;
  p.page_size = page_size;
  p.num_pages = num_pages;
  p.err = err;
  p.bias = opt ? opt->bias : nullptr;
  p.q_norm = opt ? opt->q_norm_weight : nullptr;
  p.k_norm = opt ? opt->k_norm_weight : nullptr;
  p.rms_eps = opt ? opt->rms_eps : 0.f;
  PIEKV_REQUIRE(!opt || opt->rms_eps >= 0.f, "qkv_rope_append: negative rms_eps");
  CUtensorMap tx, tw;
  const int64_t rows_w = (int64_t)(num_qo_heads + 2 * num_kv_heads) * head_dim;
  if (int rc = make_matrix_tensor_map(&tx, x, nnz, hidden, x_stride_n, dtype, kQBM, kQBK)) return rc;
  const int nh = (num_qo_heads + 2 * num_kv_heads) % 2 == 0 ? 2 : 1;  // heads per tile
  if (int rc = make_matrix_tensor_map(&tw, w_qkv, rows_w, hidden, w_stride_n, dtype, nh * kQDim, kQBK)) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == PIEKV_BF16)
    return nh == 2 ? launch_qkv<__nv_bfloat16, 2>(tx, tw, p, rp, st) : launch_qkv<__nv_bfloat16, 1>(tx, tw, p, rp, st);
  return nh == 2 ? launch_qkv<__half, 2>(tx, tw, p, rp, st) : launch_qkv<__half, 1>(tx, tw, p, rp, st);
}

extern "C" int piekv_qkv_rope_append(const void *x, int64_t x_stride_n, const void *w_qkv, int64_t w_stride_n,
                                     void *q_out, const int32_t *pos_ids, const int32_t *batch_indices,
                                     const int32_t *positions, void *pool, const int32_t *kv_indices,
                                     const int32_t *kv_indptr, int32_t nnz, int32_t batch, int32_t hidden,
                                     int32_t num_qo_heads, int32_t num_kv_heads, int32_t head_dim, int32_t page_size,
                                     int32_t num_pages, int32_t dtype, const piekv_rope_params *rope, int32_t *err,
                                     void *stream) {
  return piekv_qkv_rope_append_opt(x, x_stride_n, w_qkv, w_stride_n, q_out, pos_ids, batch_indices, positions, pool,
                                   kv_indices, kv_indptr, nnz, batch, hidden, num_qo_heads, num_kv_heads, head_dim,
                                   page_size, num_pages, dtype, rope, err, stream, nullptr);
}
