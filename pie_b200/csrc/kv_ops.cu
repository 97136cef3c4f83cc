// Metadata, RoPE, K/V append (optionally fused with RoPE) and page copy.
// All of these are index arithmetic plus data movement: HBM-bound, so the kernels use
// 16-byte vector accesses on contiguous head_dim rows and no shared memory.
#include <math.h>

#include "common.cuh"
#include "rope.cuh"

namespace piekv {

// =====================================================================================
// metadata
// =====================================================================================

// seq_lens / batch_indices / positions in one pass.  Reference semantics:
// pie/src/flashinfer_metal/ops.py:392-436; a request without pages keeps last_page_len as its
// length, as the CUDA dependency and the numpy twin do (pie/src/pie_worker/batching.py:104-111;
// the Metal twin returns 0 there).
__global__ void meta_kernel(const int32_t *__restrict__ qo_indptr, const int32_t *__restrict__ kv_indptr,
                            const int32_t *__restrict__ kv_last_page_len, const int32_t *__restrict__ seq_lens_in,
                            int batch, int nnz, int page_size, int32_t *__restrict__ seq_lens_out,
                            int32_t *__restrict__ batch_indices, int32_t *__restrict__ positions) {
  int tid = blockIdx.x * blockDim.x + threadIdx.x;
  if (seq_lens_out != nullptr && tid < batch) {
    int np = kv_indptr[tid + 1] - kv_indptr[tid];
    seq_lens_out[tid] = (np > 0 ? (np - 1) * page_size : 0) + kv_last_page_len[tid];
  }
  if (batch_indices != nullptr && tid < nnz) {
    if (qo_indptr == nullptr) {  // decode: token i belongs to request i
      int np = kv_indptr[tid + 1] - kv_indptr[tid];
      batch_indices[tid] = tid;
      positions[tid] = (np > 0 ? (np - 1) * page_size : 0) + kv_last_page_len[tid] - 1;
      return;
    }
    // first b with qo_indptr[b+1] > tid
    int lo = 0, hi = batch;  // answer in [0, batch)
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if (qo_indptr[mid + 1] > tid)
        hi = mid;
      else
        lo = mid + 1;
    }
    int b = lo < batch ? lo : batch - 1;
    int sl;
    if (seq_lens_in != nullptr) {
      sl = seq_lens_in[b];
    } else {
      int np = kv_indptr[b + 1] - kv_indptr[b];
      sl = (np > 0 ? (np - 1) * page_size : 0) + kv_last_page_len[b];
    }
    int q0 = qo_indptr[b], q1 = qo_indptr[b + 1];
    batch_indices[tid] = b;
    positions[tid] = sl - (q1 - q0) + (tid - q0);
  }
}

// =====================================================================================
// RoPE + append
// =====================================================================================

template <typename T, int VEC>
struct alignas(sizeof(T) * VEC) Vec {
  T v[VEC];
};

template <typename T, int VEC>
__device__ __forceinline__ Vec<T, VEC> load_vec(const T *p) {
  return *reinterpret_cast<const Vec<T, VEC> *>(p);
}
template <typename T, int VEC>
__device__ __forceinline__ void store_vec(T *p, const Vec<T, VEC> &x) {
  *reinterpret_cast<Vec<T, VEC> *>(p) = x;
}

// cos/sin of VEC consecutive pair indices starting at pair0 for one token.
template <int VEC>
__device__ __forceinline__ void rope_cos_sin(const RopeDev &rp, int pos, int pair0, int half_dim, float (&c)[VEC],
                                             float (&s)[VEC]) {
  if (rp.mode == PIEKV_ROPE_TABLE) {
    const float *row = rp.table + (size_t)pos * (2 * half_dim);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      c[j] = row[pair0 + j];
      s[j] = row[half_dim + pair0 + j];
    }
  } else {
    float p = (float)pos;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float ang = __fmul_rn(p, rp.inv_freq[pair0 + j]);
      sincosf(ang, &s[j], &c[j]);
    }
  }
}

// Rotate one head row in place / to a destination. x' = x*c - y*s ; y' = x*s + y*c with
// separately rounded products and sums (no FMA contraction), one rounding to T at the end.
template <typename T, int VEC>
__device__ __forceinline__ void rotate_chunk(const T *src, T *dst0, T *dst1, int chunk, int half_dim, bool interleave,
                                             const float *c, const float *s) {
  // non-interleaved: chunk covers pairs [chunk*VEC, +VEC): elements i and i + half_dim
  // interleaved:     chunk covers elements [chunk*VEC, +VEC) = pairs [chunk*VEC/2, +VEC/2)
  if (!interleave) {
    int i0 = chunk * VEC;
    Vec<T, VEC> lo = load_vec<T, VEC>(src + i0);
    Vec<T, VEC> hi = load_vec<T, VEC>(src + i0 + half_dim);
    Vec<T, VEC> olo, ohi;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      float x = Elem<T>::to_f32(lo.v[j]);
      float y = Elem<T>::to_f32(hi.v[j]);
      olo.v[j] = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x, c[j]), __fmul_rn(y, s[j])));
      ohi.v[j] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(x, s[j]), __fmul_rn(y, c[j])));
    }
    store_vec<T, VEC>(dst0 + i0, olo);
    store_vec<T, VEC>(dst0 + i0 + half_dim, ohi);
    if (dst1 != nullptr) {
      store_vec<T, VEC>(dst1 + i0, olo);
      store_vec<T, VEC>(dst1 + i0 + half_dim, ohi);
    }
  }
}

template <typename T>
__device__ __forceinline__ void rotate_pair_interleaved(const T *src, T *dst0, T *dst1, int pair, float c, float s) {
  float x = Elem<T>::to_f32(src[2 * pair]);
  float y = Elem<T>::to_f32(src[2 * pair + 1]);
  T ox = Elem<T>::from_f32(__fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s)));
  T oy = Elem<T>::from_f32(__fadd_rn(__fmul_rn(x, s), __fmul_rn(y, c)));
  dst0[2 * pair] = ox;
  dst0[2 * pair + 1] = oy;
  if (dst1 != nullptr) {
    dst1[2 * pair] = ox;
    dst1[2 * pair + 1] = oy;
  }
}

struct AppendArgs {
  void *q_out;    // nullable: rotated q goes here ([n, Hq, D] contiguous) instead of back into q
  void *q;        // nullable
  void *k;        // nullable (rope-only call may pass only q)
  const void *v;  // nullable (rope-only call)
  int64_t q_sn, q_sh, k_sn, k_sh, v_sn, v_sh;
  const int32_t *pos_ids;
  const int32_t *batch_indices;
  const int32_t *positions;
  void *pool;  // nullable: rope-only call
  const int32_t *kv_indices;
  const int32_t *kv_indptr;
  int nnz, batch, hq, hkv, dim, page_size, num_pages;
  int rotate_k_in_place;
  int32_t *err;
};

// One block per token.  threadIdx.x walks the vector chunks of a head row, threadIdx.y
// walks heads, so a warp's accesses are consecutive 16-byte pieces of contiguous rows.
// Work list per token: Hq q-heads (rotate in place), Hkv k-heads (rotate -> pool [and back]),
// Hkv v-heads (copy -> pool).
template <typename T, int VEC>
__global__ void rope_append_kernel(AppendArgs a, RopeDev rp) {
  const int tok = blockIdx.x;
  if (tok >= a.nnz) return;
  const int D = a.dim, half = D / 2;
  const bool do_rope = rp.mode != PIEKV_ROPE_NONE;

  T *kdst = nullptr, *vdst = nullptr;
  bool have_dst = false;
  if (a.pool != nullptr) {
    int b = a.batch_indices[tok];
    int pos = a.positions[tok];
    if (b < 0 || b >= a.batch) {
      if (threadIdx.x == 0 && threadIdx.y == 0) report_error(a.err, PIEKV_ERR_BATCH_INDEX, KID_APPEND, tok, b);
    } else {
      int p0 = a.kv_indptr[b], p1 = a.kv_indptr[b + 1];
      int slot = pos >= 0 ? pos / a.page_size : -1;
      if (slot < 0 || p0 + slot >= p1) {
        if (threadIdx.x == 0 && threadIdx.y == 0) report_error(a.err, PIEKV_ERR_PAGE_SLOT, KID_APPEND, tok, pos);
      } else {
        int page = a.kv_indices[p0 + slot];
        if (page < 0 || page >= a.num_pages) {
          if (threadIdx.x == 0 && threadIdx.y == 0) report_error(a.err, PIEKV_ERR_PAGE_ID, KID_APPEND, tok, page);
        } else {
          size_t half_page = (size_t)a.page_size * a.hkv * D;
          size_t row = (size_t)(pos % a.page_size) * a.hkv * D;
          kdst = reinterpret_cast<T *>(a.pool) + (size_t)page * 2 * half_page + row;
          vdst = kdst + half_page;
          have_dst = true;
        }
      }
    }
  }

  int pos_id = 0;
  bool rope_ok = do_rope;
  if (do_rope) {
    pos_id = a.pos_ids[tok];
    if (rp.mode == PIEKV_ROPE_TABLE && (pos_id < 0 || pos_id >= rp.table_len)) {
      if (threadIdx.x == 0 && threadIdx.y == 0) report_error(a.err, PIEKV_ERR_TABLE_RANGE, KID_ROPE, tok, pos_id);
      rope_ok = false;  // leave q/k un-rotated; k still lands in the pool un-rotated
    }
  }

  const int n_rot_heads = (a.q != nullptr ? a.hq : 0) + (a.k != nullptr ? a.hkv : 0);
  const int q_heads = a.q != nullptr ? a.hq : 0;

  if (rope_ok) {
    if (!rp.interleave) {
      const int chunks = half / VEC;  // chunks of pairs per head
      for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
        float c[VEC], s[VEC];
        rope_cos_sin<VEC>(rp, pos_id, ch * VEC, half, c, s);
        for (int h = threadIdx.y; h < n_rot_heads; h += blockDim.y) {
          if (h < q_heads) {
            T *row = reinterpret_cast<T *>(a.q) + (size_t)tok * a.q_sn + (size_t)h * a.q_sh;
            T *dst = a.q_out ? reinterpret_cast<T *>(a.q_out) + ((size_t)tok * a.hq + h) * D : row;
            rotate_chunk<T, VEC>(row, dst, nullptr, ch, half, false, c, s);
          } else {
            int hk = h - q_heads;
            T *row = reinterpret_cast<T *>(a.k) + (size_t)tok * a.k_sn + (size_t)hk * a.k_sh;
            if (have_dst) {
              rotate_chunk<T, VEC>(row, kdst + (size_t)hk * D, a.rotate_k_in_place ? row : nullptr, ch, half, false, c,
                                   s);
            } else if (a.pool == nullptr || a.rotate_k_in_place) {
              rotate_chunk<T, VEC>(row, row, nullptr, ch, half, false, c, s);
            }
          }
        }
      }
    } else {
      for (int pr = threadIdx.x; pr < half; pr += blockDim.x) {
        float c[1], s[1];
        rope_cos_sin<1>(rp, pos_id, pr, half, c, s);
        for (int h = threadIdx.y; h < n_rot_heads; h += blockDim.y) {
          if (h < q_heads) {
            T *row = reinterpret_cast<T *>(a.q) + (size_t)tok * a.q_sn + (size_t)h * a.q_sh;
            T *dst = a.q_out ? reinterpret_cast<T *>(a.q_out) + ((size_t)tok * a.hq + h) * D : row;
            rotate_pair_interleaved<T>(row, dst, nullptr, pr, c[0], s[0]);
          } else {
            int hk = h - q_heads;
            T *row = reinterpret_cast<T *>(a.k) + (size_t)tok * a.k_sn + (size_t)hk * a.k_sh;
            if (have_dst) {
              rotate_pair_interleaved<T>(row, kdst + (size_t)hk * D, a.rotate_k_in_place ? row : nullptr, pr, c[0],
                                         s[0]);
            } else if (a.pool == nullptr || a.rotate_k_in_place) {
              rotate_pair_interleaved<T>(row, row, nullptr, pr, c[0], s[0]);
            }
          }
        }
      }
    }
  }

  if (have_dst) {
    const int chunks = D / VEC;
    // V always; K here only when it was not written by the rotation above
    const bool copy_k = !rope_ok && a.k != nullptr;
    for (int h = threadIdx.y; h < a.hkv; h += blockDim.y) {
      const T *vrow = reinterpret_cast<const T *>(a.v) + (size_t)tok * a.v_sn + (size_t)h * a.v_sh;
      const T *krow = reinterpret_cast<const T *>(a.k) + (size_t)tok * a.k_sn + (size_t)h * a.k_sh;
      for (int ch = threadIdx.x; ch < chunks; ch += blockDim.x) {
        store_vec<T, VEC>(vdst + (size_t)h * D + ch * VEC, load_vec<T, VEC>(vrow + ch * VEC));
        if (copy_k) store_vec<T, VEC>(kdst + (size_t)h * D + ch * VEC, load_vec<T, VEC>(krow + ch * VEC));
      }
    }
  }
}

// The same operation for the common case (16-byte vectors, non-interleaved pairs, head_dim <= 256),
// laid out for bandwidth: a block takes kTokPerBlock tokens; their cos / sin values are computed once
// (one pair per thread) and shared through shared memory instead of once per head, the page lookup of a
// token (three dependent loads) is done by one thread while the others compute, and afterwards every
// thread moves 16-byte pieces of a flat work list (token, head, chunk) so that all 256 threads carry
// loads in flight whatever the head count.  Arithmetic and rounding are those of rotate_chunk.
constexpr int kTokPerBlock = 4;

template <typename T>
__global__ void __launch_bounds__(256) rope_append_tokens_kernel(AppendArgs a, RopeDev rp) {
  constexpr int VEC = 16 / sizeof(T);
  __shared__ float sh_c[kTokPerBlock][kMaxHalfDim], sh_s[kTokPerBlock][kMaxHalfDim];
  __shared__ T *sh_kdst[kTokPerBlock];
  __shared__ int sh_rope_ok[kTokPerBlock];
  const int tok0 = blockIdx.x * kTokPerBlock;
  const int ntok = min(kTokPerBlock, a.nnz - tok0);
  const int D = a.dim, half = D / 2;
  const bool do_rope = rp.mode != PIEKV_ROPE_NONE;
  const int tid = threadIdx.x;

  if (tid < ntok) {  // destination rows in the pool
    const int tok = tok0 + tid;
    T *kdst = nullptr;
    if (a.pool != nullptr) {
      const int b = a.batch_indices[tok];
      const int pos = a.positions[tok];
      if (b < 0 || b >= a.batch) {
        report_error(a.err, PIEKV_ERR_BATCH_INDEX, KID_APPEND, tok, b);
      } else {
        const int p0 = a.kv_indptr[b], p1 = a.kv_indptr[b + 1];
        const int slot = pos >= 0 ? pos / a.page_size : -1;
        if (slot < 0 || p0 + slot >= p1) {
          report_error(a.err, PIEKV_ERR_PAGE_SLOT, KID_APPEND, tok, pos);
        } else {
          const int page = a.kv_indices[p0 + slot];
          if (page < 0 || page >= a.num_pages) {
            report_error(a.err, PIEKV_ERR_PAGE_ID, KID_APPEND, tok, page);
          } else {
            const size_t half_page = (size_t)a.page_size * a.hkv * D;
            kdst = reinterpret_cast<T *>(a.pool) + (size_t)page * 2 * half_page + (size_t)(pos % a.page_size) * a.hkv * D;
          }
        }
      }
    }
    sh_kdst[tid] = kdst;
  }
  if (do_rope) {
    for (int x = tid; x < ntok * half; x += blockDim.x) {
      const int t = x / half, pr = x - t * half;
      const int pos_id = a.pos_ids[tok0 + t];
      const bool ok = !(rp.mode == PIEKV_ROPE_TABLE && (pos_id < 0 || pos_id >= rp.table_len));
      if (pr == 0) {
        sh_rope_ok[t] = ok ? 1 : 0;  // out of the table: q / k stay un-rotated, k still lands in the pool
        if (!ok) report_error(a.err, PIEKV_ERR_TABLE_RANGE, KID_ROPE, tok0 + t, pos_id);
      }
      float c = 1.f, sn = 0.f;
      if (ok) rope_cos_sin1(rp, pos_id, pr, half, c, sn);
      sh_c[t][pr] = c;
      sh_s[t][pr] = sn;
    }
  } else if (tid < ntok) {
    sh_rope_ok[tid] = 0;
  }
  __syncthreads();

  const int q_heads = a.q != nullptr ? a.hq : 0;
  const int k_heads = a.k != nullptr ? a.hkv : 0;
  const int rchunks = half / VEC;  // a rotation item covers VEC pairs: elements [i0, i0+VEC) and the same + half
  // ---- rotations: q heads (in place or to q_out) and k heads (to the pool and / or in place)
  const int rot_items = ntok * (q_heads + k_heads) * rchunks;
  for (int x = tid; x < rot_items; x += blockDim.x) {
    const int ch = x % rchunks;
    const int h = (x / rchunks) % (q_heads + k_heads);
    const int t = x / (rchunks * (q_heads + k_heads));
    const int tok = tok0 + t;
    const bool rot = sh_rope_ok[t] != 0;
    const T *src;
    T *dst0 = nullptr, *dst1 = nullptr;
    if (h < q_heads) {
      if (!rot) continue;  // nothing to do for q without a rotation
      T *row = reinterpret_cast<T *>(a.q) + (size_t)tok * a.q_sn + (size_t)h * a.q_sh;
      src = row;
      dst0 = a.q_out ? reinterpret_cast<T *>(a.q_out) + ((size_t)tok * a.hq + h) * D : row;
    } else {
      const int hk = h - q_heads;
      T *row = reinterpret_cast<T *>(a.k) + (size_t)tok * a.k_sn + (size_t)hk * a.k_sh;
      src = row;
      T *kd = sh_kdst[t];
      if (kd != nullptr) {
        dst0 = kd + (size_t)hk * D;
        dst1 = (rot && a.rotate_k_in_place) ? row : nullptr;
      } else if (rot && (a.pool == nullptr || a.rotate_k_in_place)) {
        dst0 = row;
      } else {
        continue;
      }
    }
    const int i0 = ch * VEC;
    const Vec<T, VEC> lo = load_vec<T, VEC>(src + i0);
    const Vec<T, VEC> hi = load_vec<T, VEC>(src + i0 + half);
    Vec<T, VEC> olo = lo, ohi = hi;
    if (rot) {
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        const float xv = Elem<T>::to_f32(lo.v[j]), yv = Elem<T>::to_f32(hi.v[j]);
        const float c = sh_c[t][i0 + j], sn = sh_s[t][i0 + j];
        olo.v[j] = Elem<T>::from_f32(__fsub_rn(__fmul_rn(xv, c), __fmul_rn(yv, sn)));
        ohi.v[j] = Elem<T>::from_f32(__fadd_rn(__fmul_rn(xv, sn), __fmul_rn(yv, c)));
      }
    }
    store_vec<T, VEC>(dst0 + i0, olo);
    store_vec<T, VEC>(dst0 + i0 + half, ohi);
    if (dst1 != nullptr) {
      store_vec<T, VEC>(dst1 + i0, olo);
      store_vec<T, VEC>(dst1 + i0 + half, ohi);
    }
  }
  // ---- v rows into the pool
  if (a.pool != nullptr && a.v != nullptr) {
    const int vchunks = D / VEC;
    const int v_items = ntok * a.hkv * vchunks;
    const size_t half_page = (size_t)a.page_size * a.hkv * D;
    for (int x = tid; x < v_items; x += blockDim.x) {
      const int ch = x % vchunks;
      const int h = (x / vchunks) % a.hkv;
      const int t = x / (vchunks * a.hkv);
      T *kd = sh_kdst[t];
      if (kd == nullptr) continue;
      const T *vrow = reinterpret_cast<const T *>(a.v) + (size_t)(tok0 + t) * a.v_sn + (size_t)h * a.v_sh;
      store_vec<T, VEC>(kd + half_page + (size_t)h * D + ch * VEC, load_vec<T, VEC>(vrow + ch * VEC));
    }
  }
}

// Append without a rotation (ops.append_paged_kv_cache): a warp per token, no block-wide step.  Every lane
// resolves the token's page itself (the three loads are the same addresses for the whole warp), then the
// lanes move the k row and the v row in 16-byte pieces with all of a lane's loads issued before its stores.
template <typename T>
__global__ void __launch_bounds__(256) append_tokens_warp_kernel(AppendArgs a) {
  constexpr int VEC = 16 / sizeof(T);
  const int tok = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (tok >= a.nnz) return;
  const int b = a.batch_indices[tok];
  const int pos = a.positions[tok];
  if (b < 0 || b >= a.batch) {
    if (lane == 0) report_error(a.err, PIEKV_ERR_BATCH_INDEX, KID_APPEND, tok, b);
    return;
  }
  const int p0 = a.kv_indptr[b], p1 = a.kv_indptr[b + 1];
  const int slot = pos >= 0 ? pos / a.page_size : -1;
  if (slot < 0 || p0 + slot >= p1) {
    if (lane == 0) report_error(a.err, PIEKV_ERR_PAGE_SLOT, KID_APPEND, tok, pos);
    return;
  }
  const int page = a.kv_indices[p0 + slot];
  if (page < 0 || page >= a.num_pages) {
    if (lane == 0) report_error(a.err, PIEKV_ERR_PAGE_ID, KID_APPEND, tok, page);
    return;
  }
  const int D = a.dim;
  const size_t half_page = (size_t)a.page_size * a.hkv * D;
  T *kdst = reinterpret_cast<T *>(a.pool) + (size_t)page * 2 * half_page + (size_t)(pos % a.page_size) * a.hkv * D;
  const int chunks = D / VEC;            // 16-byte pieces per head row
  const int items = a.hkv * chunks;      // per tensor
  constexpr int kU = 4;
  for (int x0 = lane; x0 < items; x0 += 32 * kU) {
    Vec<T, VEC> kv[kU], vv[kU];
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int x = x0 + u * 32;
      if (x < items) {
        const int h = x / chunks, ch = x - h * chunks;
        kv[u] = load_vec<T, VEC>(reinterpret_cast<const T *>(a.k) + (size_t)tok * a.k_sn + (size_t)h * a.k_sh + ch * VEC);
        vv[u] = load_vec<T, VEC>(reinterpret_cast<const T *>(a.v) + (size_t)tok * a.v_sn + (size_t)h * a.v_sh + ch * VEC);
      }
    }
#pragma unroll
    for (int u = 0; u < kU; ++u) {
      const int x = x0 + u * 32;
      if (x < items) {
        store_vec<T, VEC>(kdst + (size_t)x * VEC, kv[u]);
        store_vec<T, VEC>(kdst + half_page + (size_t)x * VEC, vv[u]);
      }
    }
  }
}

// Per-pair frequencies in double, rounded once to fp32.  Formula of
// pie/src/flashinfer_metal/kernels/metal_rope.metal:66-89 with the low/high/old_context
// parameters the reference passes at pie/src/pie_worker/model/llama3.py:660-669.
void fill_inv_freq(const piekv_rope_params *rope, int head_dim, RopeDev *out) {
  const int half = head_dim / 2;
  out->mode = rope ? rope->mode : PIEKV_ROPE_NONE;
  out->interleave = rope ? rope->interleave : 0;
  out->table_len = rope ? rope->table_len : 0;
  out->table = rope ? rope->cos_sin_table : nullptr;
  for (int i = 0; i < kMaxHalfDim; ++i) out->inv_freq[i] = 0.f;
  if (!rope || (rope->mode != PIEKV_ROPE_PLAIN && rope->mode != PIEKV_ROPE_LLAMA31)) return;
  const double two_pi = 6.283185307179586476925286766559;
  for (int i = 0; i < half; ++i) {
    double f = pow((double)rope->theta, -2.0 * (double)i / (double)head_dim);
    if (rope->mode == PIEKV_ROPE_PLAIN && rope->scale > 0.f) f = f / (double)rope->scale;
    if (rope->mode == PIEKV_ROPE_LLAMA31) {
      double scale = rope->scale, lowf = rope->low_freq_factor, highf = rope->high_freq_factor;
      double old = rope->old_context_len;
      double wavelen = two_pi / f;
      if (wavelen > old / lowf) {
        f = f / scale;
      } else if (wavelen < old / highf) {
        // unchanged
      } else {
        double smooth = (old / wavelen - lowf) / (highf - lowf);
        f = (1.0 - smooth) * (f / scale) + smooth * f;
      }
    }
    out->inv_freq[i] = (float)f;
  }
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T>
static int launch_rope_append_t(const AppendArgs &a, const RopeDev &rp, cudaStream_t st) {
  constexpr int VEC = 16 / sizeof(T);
  const size_t es = sizeof(T);
  bool vec_ok = (a.dim % (2 * VEC) == 0);
  auto stride_ok = [&](int64_t s) { return (s * (int64_t)es) % 16 == 0; };
  if (a.q) vec_ok = vec_ok && aligned16(a.q) && stride_ok(a.q_sn) && stride_ok(a.q_sh);
  if (a.q_out) vec_ok = vec_ok && aligned16(a.q_out);
  if (a.k) vec_ok = vec_ok && aligned16(a.k) && stride_ok(a.k_sn) && stride_ok(a.k_sh);
  if (a.v) vec_ok = vec_ok && aligned16(a.v) && stride_ok(a.v_sn) && stride_ok(a.v_sh);
  if (a.pool) vec_ok = vec_ok && aligned16(a.pool);
  if (a.nnz == 0) return 0;
  if (vec_ok && rp.mode == PIEKV_ROPE_NONE && a.q == nullptr && a.k != nullptr && a.v != nullptr && a.pool != nullptr) {
    append_tokens_warp_kernel<T><<<(a.nnz + 7) / 8, 256, 0, st>>>(a);
  } else if (vec_ok && !rp.interleave && a.dim <= 2 * kMaxHalfDim && (a.k != nullptr || a.pool == nullptr)) {
    rope_append_tokens_kernel<T><<<(a.nnz + kTokPerBlock - 1) / kTokPerBlock, 256, 0, st>>>(a, rp);
  } else if (vec_ok) {
    int tx = a.dim / VEC;  // chunks across a full row (V copy); rope uses half of them
    if (tx > 32) tx = 32;
    int heads = (a.q ? a.hq : 0) + a.hkv;
    int ty = 256 / tx;
    if (ty > heads) ty = heads;
    if (ty < 1) ty = 1;
    rope_append_kernel<T, VEC><<<a.nnz, dim3(tx, ty), 0, st>>>(a, rp);
  } else {
    int tx = 32;
    int ty = 4;
    rope_append_kernel<T, 1><<<a.nnz, dim3(tx, ty), 0, st>>>(a, rp);
  }
  PIEKV_LAUNCH_CHECK("rope_append_kernel");
  return 0;
}

static int launch_rope_append(const AppendArgs &a, const RopeDev &rp, int dtype, cudaStream_t st) {
  switch (dtype) {
    case PIEKV_F32:
      return launch_rope_append_t<float>(a, rp, st);
    case PIEKV_F16:
      return launch_rope_append_t<__half>(a, rp, st);
    case PIEKV_BF16:
      return launch_rope_append_t<__nv_bfloat16>(a, rp, st);
  }
  set_error("unknown dtype %d", dtype);
  return 1;
}

// =====================================================================================
// page copy
// =====================================================================================

constexpr int kMaxLayersPerLaunch = 32;
struct PoolPtrs {
  void *p[kMaxLayersPerLaunch];
};

// grid (pair * parts, K|V, layer).  The first `valid` rows of a page half are one contiguous run of
// valid * Hkv * D elements, so the copy is a flat 16-byte-vector memcpy; a half is cut into `parts`
// slices, one CTA each, so that a handful of pairs (a beam fork copies a few dozen pages) still
// spreads over all SMs.  Every thread keeps four 16-byte loads in flight.
__global__ void copy_pages_kernel(PoolPtrs pools, const int32_t *__restrict__ src, const int32_t *__restrict__ dst,
                                  const int32_t *__restrict__ valid_len, int page_size, size_t row_bytes,
                                  int num_pages, int parts, int32_t *err) {
  const int j = blockIdx.x / parts;
  const int part = blockIdx.x % parts;
  const int kv = blockIdx.y;
  char *base = reinterpret_cast<char *>(pools.p[blockIdx.z]);
  int s = src[j], d = dst[j];
  int valid = valid_len != nullptr ? valid_len[j] : page_size;
  if (s < 0 || s >= num_pages || d < 0 || d >= num_pages) {
    if (threadIdx.x == 0 && part == 0) report_error(err, PIEKV_ERR_PAGE_ID, KID_COPY, j, s < 0 || s >= num_pages ? s : d);
    return;
  }
  if (valid < 0 || valid > page_size) {
    if (threadIdx.x == 0 && part == 0) report_error(err, PIEKV_ERR_LAST_PAGE_LEN, KID_COPY, j, valid);
    return;
  }
  if (s == d || valid == 0) return;
  size_t half_bytes = (size_t)page_size * row_bytes;
  const char *sp = base + ((size_t)s * 2 + kv) * half_bytes;
  char *dp = base + ((size_t)d * 2 + kv) * half_bytes;
  size_t bytes = (size_t)valid * row_bytes;
  if ((row_bytes & 15) == 0 && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
    const uint4 *s4 = reinterpret_cast<const uint4 *>(sp);
    uint4 *d4 = reinterpret_cast<uint4 *>(dp);
    const size_t n = bytes >> 4;
    const size_t per = (n + parts - 1) / parts;
    const size_t lo = (size_t)part * per;
    const size_t hi = lo + per < n ? lo + per : n;
    size_t i = lo + threadIdx.x;
    const size_t step = blockDim.x;
    for (; i + 3 * step < hi; i += 4 * step) {
      const uint4 a0 = s4[i], a1 = s4[i + step], a2 = s4[i + 2 * step], a3 = s4[i + 3 * step];
      d4[i] = a0;
      d4[i + step] = a1;
      d4[i + 2 * step] = a2;
      d4[i + 3 * step] = a3;
    }
    for (; i < hi; i += step) d4[i] = s4[i];
  } else {
    const size_t per = (bytes + parts - 1) / parts;
    const size_t lo = (size_t)part * per;
    const size_t hi = lo + per < bytes ? lo + per : bytes;
    for (size_t i = lo + threadIdx.x; i < hi; i += blockDim.x) dp[i] = sp[i];
  }
}

int launch_decode_append_general(void *q_out, const void *q, const void *k, const void *v, int64_t q_sn, int64_t q_sh,
                                 int64_t k_sn, int64_t k_sh, int64_t v_sn, int64_t v_sh, const int32_t *pos_ids,
                                 int32_t *bi_scratch, int32_t *pos_scratch, void *pool, const int32_t *kv_indices,
                                 const int32_t *kv_indptr, const int32_t *kv_last_page_len, int batch, int hq, int hkv,
                                 int dim, int page_size, int num_pages, int dtype, const RopeDev &rp, int32_t *err,
                                 cudaStream_t st) {
  meta_kernel<<<(batch + 255) / 256, 256, 0, st>>>(nullptr, kv_indptr, kv_last_page_len, nullptr, batch, batch,
                                                   page_size, nullptr, bi_scratch, pos_scratch);
  PIEKV_LAUNCH_CHECK("meta_kernel");
  AppendArgs a{};
  const bool do_rope = rp.mode != PIEKV_ROPE_NONE;
  a.q_out = do_rope ? q_out : nullptr;
  a.q = do_rope ? const_cast<void *>(q) : nullptr;
  a.k = const_cast<void *>(k);
  a.v = v;
  a.q_sn = q_sn;
  a.q_sh = q_sh;
  a.k_sn = k_sn;
  a.k_sh = k_sh;
  a.v_sn = v_sn;
  a.v_sh = v_sh;
  a.pos_ids = pos_ids;
  a.batch_indices = bi_scratch;
  a.positions = pos_scratch;
  a.pool = pool;
  a.kv_indices = kv_indices;
  a.kv_indptr = kv_indptr;
  a.nnz = batch;
  a.batch = batch;
  a.hq = hq;
  a.hkv = hkv;
  a.dim = dim;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.rotate_k_in_place = 0;
  a.err = err;
  return launch_rope_append(a, rp, dtype, st);
}

}  // namespace piekv

using namespace piekv;

// =====================================================================================
// C ABI
// =====================================================================================

extern "C" int piekv_get_seq_lens(const int32_t *kv_indptr, const int32_t *kv_last_page_len, int32_t batch,
                                  int32_t page_size, int32_t *seq_lens_out, void *stream) {
  PIEKV_REQUIRE(batch >= 0 && page_size > 0, "get_seq_lens: bad batch %d / page_size %d", batch, page_size);
  PIEKV_REQUIRE(kv_indptr && kv_last_page_len && seq_lens_out, "get_seq_lens: null pointer");
  if (batch == 0) return 0;
  meta_kernel<<<(batch + 255) / 256, 256, 0, (cudaStream_t)stream>>>(nullptr, kv_indptr, kv_last_page_len, nullptr,
                                                                      batch, 0, page_size, seq_lens_out, nullptr,
                                                                      nullptr);
  PIEKV_LAUNCH_CHECK("meta_kernel");
  return 0;
}

extern "C" int piekv_get_batch_indices_positions(const int32_t *append_indptr, const int32_t *seq_lens, int32_t batch,
                                                 int32_t nnz, int32_t *batch_indices_out, int32_t *positions_out,
                                                 void *stream) {
  PIEKV_REQUIRE(batch >= 0 && nnz >= 0, "get_batch_indices_positions: bad batch %d / nnz %d", batch, nnz);
  PIEKV_REQUIRE(append_indptr && seq_lens && batch_indices_out && positions_out,
                "get_batch_indices_positions: null pointer");
  if (nnz == 0 || batch == 0) return 0;
  meta_kernel<<<(nnz + 255) / 256, 256, 0, (cudaStream_t)stream>>>(append_indptr, nullptr, nullptr, seq_lens, batch,
                                                                    nnz, 1, nullptr, batch_indices_out, positions_out);
  PIEKV_LAUNCH_CHECK("meta_kernel");
  return 0;
}

extern "C" int piekv_metadata(const int32_t *qo_indptr, const int32_t *kv_indptr, const int32_t *kv_last_page_len,
                              int32_t batch, int32_t nnz, int32_t page_size, int32_t *seq_lens_out,
                              int32_t *batch_indices_out, int32_t *positions_out, void *stream) {
  PIEKV_REQUIRE(batch >= 0 && nnz >= 0 && page_size > 0, "metadata: bad sizes");
  PIEKV_REQUIRE(qo_indptr && kv_indptr && kv_last_page_len && batch_indices_out && positions_out,
                "metadata: null pointer");
  int work = nnz > batch ? nnz : batch;
  if (work == 0) return 0;
  meta_kernel<<<(work + 255) / 256, 256, 0, (cudaStream_t)stream>>>(qo_indptr, kv_indptr, kv_last_page_len, nullptr,
                                                                     batch, nnz, page_size, seq_lens_out,
                                                                     batch_indices_out, positions_out);
  PIEKV_LAUNCH_CHECK("meta_kernel");
  return 0;
}

namespace piekv {
int check_rope(const piekv_rope_params *rope, int head_dim, const char *who) {
  PIEKV_REQUIRE(head_dim > 0 && head_dim % 2 == 0 && head_dim / 2 <= kMaxHalfDim, "%s: head_dim %d unsupported", who,
                head_dim);
  if (!rope) return 0;
  PIEKV_REQUIRE(rope->mode >= PIEKV_ROPE_NONE && rope->mode <= PIEKV_ROPE_TABLE, "%s: bad rope mode %d", who,
                rope->mode);
  if (rope->mode == PIEKV_ROPE_TABLE)
    PIEKV_REQUIRE(rope->cos_sin_table && rope->table_len > 0, "%s: rope table missing", who);
  if (rope->mode == PIEKV_ROPE_PLAIN || rope->mode == PIEKV_ROPE_LLAMA31)
    PIEKV_REQUIRE(rope->theta > 0.f, "%s: rope theta must be > 0", who);
  if (rope->mode == PIEKV_ROPE_LLAMA31)
    PIEKV_REQUIRE(rope->scale > 0.f && rope->high_freq_factor != rope->low_freq_factor && rope->low_freq_factor > 0.f &&
                      rope->high_freq_factor > 0.f && rope->old_context_len > 0.f,
                  "%s: bad llama31 rope parameters", who);
  return 0;
}
}  // namespace piekv

extern "C" int piekv_rope_inplace(void *q, void *k, int64_t q_stride_n, int64_t q_stride_h, int64_t k_stride_n,
                                  int64_t k_stride_h, const int32_t *pos_ids, int32_t nnz, int32_t num_qo_heads,
                                  int32_t num_kv_heads, int32_t head_dim, int32_t dtype,
                                  const piekv_rope_params *rope, int32_t *err, void *stream) {
  if (int rc = check_rope(rope, head_dim, "rope_inplace")) return rc;
  PIEKV_REQUIRE(rope && rope->mode != PIEKV_ROPE_NONE, "rope_inplace: rope mode NONE");
  PIEKV_REQUIRE(nnz >= 0 && pos_ids, "rope_inplace: bad nnz / pos_ids");
  PIEKV_REQUIRE(q || k, "rope_inplace: both q and k are null");
  AppendArgs a{};
  a.q = q;
  a.k = k;
  a.v = nullptr;
  a.q_sn = q_stride_n;
  a.q_sh = q_stride_h;
  a.k_sn = k_stride_n;
  a.k_sh = k_stride_h;
  a.pos_ids = pos_ids;
  a.pool = nullptr;
  a.nnz = nnz;
  a.hq = q ? num_qo_heads : 0;
  a.hkv = k ? num_kv_heads : 0;
  a.dim = head_dim;
  a.page_size = 1;
  a.rotate_k_in_place = 1;
  a.err = err;
  RopeDev rp;
  fill_inv_freq(rope, head_dim, &rp);
  return launch_rope_append(a, rp, dtype, (cudaStream_t)stream);
}

extern "C" int piekv_rope_append(void *q, void *k, const void *v, int64_t q_stride_n, int64_t q_stride_h,
                                 int64_t k_stride_n, int64_t k_stride_h, int64_t v_stride_n, int64_t v_stride_h,
                                 const int32_t *pos_ids, const int32_t *batch_indices, const int32_t *positions,
                                 void *pool, const int32_t *kv_indices, const int32_t *kv_indptr,
                                 const int32_t *kv_last_page_len, int32_t nnz, int32_t batch, int32_t num_qo_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t page_size, int32_t num_pages,
                                 int32_t dtype, const piekv_rope_params *rope, int32_t rotate_k_in_place, int32_t *err,
                                 void *stream) {
  (void)kv_last_page_len;  // part of the reference signature; addressing needs only positions
  if (int rc = check_rope(rope, head_dim, "rope_append")) return rc;
  PIEKV_REQUIRE(nnz >= 0 && batch >= 0 && num_kv_heads > 0 && page_size > 0 && num_pages > 0,
                "rope_append: bad sizes nnz=%d batch=%d Hkv=%d page_size=%d pages=%d", nnz, batch, num_kv_heads,
                page_size, num_pages);
  PIEKV_REQUIRE(k && v && pool && batch_indices && positions && kv_indices && kv_indptr, "rope_append: null pointer");
  const bool do_rope = rope && rope->mode != PIEKV_ROPE_NONE;
  PIEKV_REQUIRE(!do_rope || pos_ids, "rope_append: pos_ids required when rope is on");
  AppendArgs a{};
  a.q = do_rope ? q : nullptr;
  a.k = k;
  a.v = v;
  a.q_sn = q_stride_n;
  a.q_sh = q_stride_h;
  a.k_sn = k_stride_n;
  a.k_sh = k_stride_h;
  a.v_sn = v_stride_n;
  a.v_sh = v_stride_h;
  a.pos_ids = pos_ids;
  a.batch_indices = batch_indices;
  a.positions = positions;
  a.pool = pool;
  a.kv_indices = kv_indices;
  a.kv_indptr = kv_indptr;
  a.nnz = nnz;
  a.batch = batch;
  a.hq = num_qo_heads;
  a.hkv = num_kv_heads;
  a.dim = head_dim;
  a.page_size = page_size;
  a.num_pages = num_pages;
  a.rotate_k_in_place = rotate_k_in_place;
  a.err = err;
  RopeDev rp;
  fill_inv_freq(rope, head_dim, &rp);
  return launch_rope_append(a, rp, dtype, (cudaStream_t)stream);
}

extern "C" int piekv_copy_pages(void *const *pools, int32_t num_layers, const int32_t *src_pages,
                                const int32_t *dst_pages, const int32_t *valid_len, int32_t count, int32_t page_size,
                                int32_t num_kv_heads, int32_t head_dim, int32_t num_pages, int32_t dtype, int32_t *err,
                                void *stream) {
  PIEKV_REQUIRE(pools && num_layers > 0, "copy_pages: no layers");
  PIEKV_REQUIRE(count >= 0 && page_size > 0 && num_kv_heads > 0 && head_dim > 0 && num_pages > 0,
                "copy_pages: bad sizes");
  PIEKV_REQUIRE(dtype >= PIEKV_F32 && dtype <= PIEKV_BF16, "copy_pages: unknown dtype %d", dtype);
  PIEKV_REQUIRE(count == 0 || (src_pages && dst_pages), "copy_pages: null page lists");
  if (count == 0) return 0;
  size_t row_bytes = (size_t)num_kv_heads * head_dim * dtype_size(dtype);
  for (int l0 = 0; l0 < num_layers; l0 += kMaxLayersPerLaunch) {
    int nl = num_layers - l0 < kMaxLayersPerLaunch ? num_layers - l0 : kMaxLayersPerLaunch;
    PoolPtrs pp{};
    for (int i = 0; i < nl; ++i) {
      PIEKV_REQUIRE(pools[l0 + i] != nullptr, "copy_pages: pool %d is null", l0 + i);
      pp.p[i] = pools[l0 + i];
    }
    // enough CTAs for two waves over the SMs even when only a few pages are copied
    int parts = 1;
    while (parts < 8 && (long long)count * 2 * nl * parts < 2ll * sm_count()) parts *= 2;
    copy_pages_kernel<<<dim3((unsigned)count * parts, 2, nl), 256, 0, (cudaStream_t)stream>>>(
        pp, src_pages, dst_pages, valid_len, page_size, row_bytes, num_pages, parts, err);
    PIEKV_LAUNCH_CHECK("copy_pages_kernel");
  }
  return 0;
}
