// Shared helpers for the libpiekv.so translation units: status handling, the device
// error word, element-type traits and small PTX wrappers (mbarrier, TMA, ldmatrix, mma).
#pragma once
#include <string.h>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/piekv.h"

namespace piekv {

// ---- host side ---------------------------------------------------------------------
void set_error(const char *fmt, ...);
int cuda_status(cudaError_t e, const char *what);  // 0 or -(int)e, records text

#define PIEKV_REQUIRE(cond, ...)          \
  do {                                    \
    if (!(cond)) {                        \
      ::piekv::set_error(__VA_ARGS__);    \
      return 1;                           \
    }                                     \
  } while (0)

#define PIEKV_LAUNCH_CHECK(what)                                   \
  do {                                                             \
    cudaError_t e__ = cudaGetLastError();                          \
    if (e__ != cudaSuccess) return ::piekv::cuda_status(e__, what); \
  } while (0)

int sm_count();  // multiprocessors of the current device (cached per device)
int current_device_slot();  // ordinal of the current device if it is in [0, kMaxDevices), else -1
constexpr int kMaxDevices = 64;

// The dynamic-shared-memory opt-in of a kernel belongs to one device (context), so it is made once per
// device ordinal, not once per process.  `done` is the caller's static table for that kernel
// instantiation; atomic byte accesses keep two host threads from tearing a flag (a doubled opt-in is harmless).
template <typename Kernel>
int opt_in_dynamic_smem(Kernel kernel, int bytes, unsigned char *done, const char *what) {
  const int dev = current_device_slot();
  if (dev >= 0 && __atomic_load_n(&done[dev], __ATOMIC_ACQUIRE)) return 0;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return ::piekv::cuda_status(e, what);
  if (dev >= 0) __atomic_store_n(&done[dev], (unsigned char)1, __ATOMIC_RELEASE);
  return 0;
}
int get_option(int key);  // library options set through piekv_set_option

inline int dtype_size(int dtype) { return dtype == PIEKV_F32 ? 4 : 2; }

// kernel ids for err[1]
enum KernelId : int {
  KID_META = 1,
  KID_ROPE = 2,
  KID_APPEND = 3,
  KID_COPY = 4,
  KID_ATTN_GENERIC = 5,
  KID_DECODE = 6,
  KID_PREFILL = 7,
  KID_PEER = 8,
  KID_PAGES = 9,
};

// ---- device side -------------------------------------------------------------------
__device__ __forceinline__ void report_error(int32_t *err, int code, int kid, int index, int value) {
  if (err == nullptr) return;
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = kid;
    err[2] = index;
    err[3] = value;
  }
}

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float to_f32(float x) { return x; }
  static __device__ __forceinline__ float from_f32(float x) { return x; }
};
template <>
struct Elem<__half> {
  static __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
};

// pack two fp32 into one 32-bit register holding two 16-bit floats (low = a, high = b)
template <typename T>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t *>(&h);
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t v);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t v) {
  return __half22float2(*reinterpret_cast<__half2 *>(&v));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&v));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ----------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// non-blocking form: try_wait may suspend the thread for a while before it answers "not yet"
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: returns false once `timeout_ns` of wall time has passed without the phase
// completing (the caller records PIEKV_ERR_WAIT_TIMEOUT and unwinds; nothing spins forever).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint64_t timeout_ns = 2000000000ull) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (global_timer_ns() - t0 > timeout_ns) return false;
  }
}

// One 32-bit word of global memory that another kernel (or GPU) may just have written.  Always an
// explicit .global load inside the caller's own branch: folding "pointer or kernel parameter" into
// one generic volatile load would read parameter space through a generic address, which faults.
__device__ __forceinline__ int ld_global_relaxed_sys(const int *p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- warp-level tensor ops (decode path) -------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                          uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                   uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Softmax normaliser with an attention sink.  `l` is the running sum of exp2(score - m_log2); the sink's
// logit (natural units, not multiplied by sm_scale) adds exp(sink) in the same units.  A row without any
// key keeps l = 0 (its output is zero either way).
__device__ __forceinline__ float add_sink(float l, float m_log2, const float *sinks, int head) {
  if (sinks == nullptr || !(l > 0.f)) return l;
  return l + fast_exp2(fmaf(__ldg(sinks + head), 1.4426950408889634f, -m_log2));
}

}  // namespace piekv
