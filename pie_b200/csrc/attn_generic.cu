// General paged attention: any element type, any head_dim <= 256, any page size, GQA,
// optional causal offset, optional flat boolean mask, optional sliding window and attention sinks.
// One warp per (query row, query
// head); lanes own head_dim elements d = lane, lane+32, ...; fp32 online softmax.
// It is the path for shapes the tuned kernels do not cover (fp32, odd head sizes, other page sizes).  Math follows the decode statement in
// pie/src/flashinfer_metal/kernels/metal_attention_simdgroup_opt.metal:1235-1330
// (scale 1/sqrt(D), kv_head = q_head / (Hq/Hkv), fp32 running max / sum).
#include "attn.cuh"
#include "common.cuh"

namespace piekv {

constexpr int kMaxEpl = 8;  // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(128) attn_generic_kernel(AttnArgs a) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)a.nnz * a.hq;
  if (w >= total) return;
  const int i = (int)(w / a.hq);
  const int h = (int)(w % a.hq);
  const int D = a.dim;
  const int group = a.hq / a.hkv;
  const int hk = h / group;

  // request of this row
  int b, q0, qo_len;
  if (a.qo_indptr != nullptr) {
    int lo = 0, hi = a.batch;
    while (lo < hi) {
      int mid = (lo + hi) >> 1;
      if (a.qo_indptr[mid + 1] > i)
        hi = mid;
      else
        lo = mid + 1;
    }
    b = lo < a.batch ? lo : a.batch - 1;
    q0 = a.qo_indptr[b];
    qo_len = a.qo_indptr[b + 1] - q0;
  } else {
    b = i;
    q0 = i;
    qo_len = 1;
  }
  const int j = i - q0;
  const int p0 = a.kv_indptr[b];
  const int np = a.kv_indptr[b + 1] - p0;
  int last = a.kv_last_page_len[b];
  if (np > 0 && (last < 1 || last > a.page_size)) {
    if (lane == 0) report_error(a.err, PIEKV_ERR_LAST_PAGE_LEN, KID_ATTN_GENERIC, b, last);
    last = last < 1 ? 1 : a.page_size;
  }
  const int kv_len = np > 0 ? (np - 1) * a.page_size + last : 0;
  int limit = kv_len;
  if (a.causal) {
    int c = kv_len - qo_len + j + 1;
    limit = c < limit ? c : limit;
  }
  // sliding window: keys before (position of this query) - window_left are not seen
  int t_first = 0;
  if (a.window_left >= 0) {
    const int first = kv_len - qo_len + j - a.window_left;
    t_first = first > 0 ? first : 0;
  }

  const uint8_t *mrow = nullptr;
  if (a.mask != nullptr) {
    long long off = 0;
    for (int bb = lane; bb < b; bb += 32) {
      int npb = a.kv_indptr[bb + 1] - a.kv_indptr[bb];
      long long kl = npb > 0 ? (long long)(npb - 1) * a.page_size + a.kv_last_page_len[bb] : 0;
      long long ql = a.qo_indptr != nullptr ? a.qo_indptr[bb + 1] - a.qo_indptr[bb] : 1;
      off += kl * ql;
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) off += __shfl_xor_sync(0xffffffffu, off, s);
    mrow = a.mask + off + (long long)j * kv_len;
  }

  const T *qrow = reinterpret_cast<const T *>(a.q) + (size_t)i * a.q_sn + (size_t)h * a.q_sh;
  float qv[kMaxEpl], acc[kMaxEpl];
#pragma unroll
  for (int e = 0; e < kMaxEpl; ++e) {
    int d = e * 32 + lane;
    qv[e] = d < D ? Elem<T>::to_f32(qrow[d]) : 0.f;
    acc[e] = 0.f;
  }
  const float scale_log2 = a.sm_scale * 1.4426950408889634f;
  float m = -INFINITY, l = 0.f;
  const size_t row_elems = (size_t)a.hkv * D;
  const size_t half_page = (size_t)a.page_size * row_elems;
  const T *pool = reinterpret_cast<const T *>(a.pool);

  for (int t = t_first; t < limit; ++t) {
    if (mrow != nullptr && mrow[t] == 0) continue;
    int page = a.kv_indices[p0 + t / a.page_size];
    if (page < 0 || page >= a.num_pages) {
      if (lane == 0) report_error(a.err, PIEKV_ERR_PAGE_ID, KID_ATTN_GENERIC, b, page);
      continue;
    }
    const T *krow = pool + (size_t)page * 2 * half_page + (size_t)(t % a.page_size) * row_elems + (size_t)hk * D;
    const T *vrow = krow + half_page;
    float dot = 0.f;
    float vv[kMaxEpl];
#pragma unroll
    for (int e = 0; e < kMaxEpl; ++e) {
      int d = e * 32 + lane;
      float kf = d < D ? Elem<T>::to_f32(krow[d]) : 0.f;
      vv[e] = d < D ? Elem<T>::to_f32(vrow[d]) : 0.f;
      dot = fmaf(qv[e], kf, dot);
    }
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
    float sc = dot * scale_log2;
    float m_new = fmaxf(m, sc);
    float alpha = exp2f(m - m_new);  // m = -inf on the first hit -> 0
    float p = exp2f(sc - m_new);
    l = l * alpha + p;
#pragma unroll
    for (int e = 0; e < kMaxEpl; ++e) acc[e] = acc[e] * alpha + p * vv[e];
    m = m_new;
  }

  T *orow = reinterpret_cast<T *>(a.out) + ((size_t)i * a.hq + h) * D;
  l = add_sink(l, m, a.sinks, h);
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int e = 0; e < kMaxEpl; ++e) {
    int d = e * 32 + lane;
    if (d < D) orow[d] = Elem<T>::from_f32(acc[e] * inv);
  }
  if (a.lse != nullptr && lane == 0) {
    a.lse[(size_t)i * a.hq + h] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
}

int launch_attn_generic(const AttnArgs &a, int dtype, cudaStream_t st) {
  long long total = (long long)a.nnz * a.hq;
  if (total == 0) return 0;
  PIEKV_REQUIRE(a.dim <= 32 * kMaxEpl, "attention: head_dim %d > %d unsupported", a.dim, 32 * kMaxEpl);
  long long blocks = (total + 3) / 4;
  PIEKV_REQUIRE(blocks < (1ll << 31), "attention: too many rows");
  switch (dtype) {
    case PIEKV_F32:
      attn_generic_kernel<float><<<(unsigned)blocks, 128, 0, st>>>(a);
      break;
    case PIEKV_F16:
      attn_generic_kernel<__half><<<(unsigned)blocks, 128, 0, st>>>(a);
      break;
    case PIEKV_BF16:
      attn_generic_kernel<__nv_bfloat16><<<(unsigned)blocks, 128, 0, st>>>(a);
      break;
    default:
      set_error("attention: unknown dtype %d", dtype);
      return 1;
  }
  PIEKV_LAUNCH_CHECK("attn_generic_kernel");
  return 0;
}

}  // namespace piekv
