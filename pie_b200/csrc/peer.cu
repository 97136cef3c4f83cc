// Output buffers shared between the GPUs of one node (one process per GPU), and the wait that closes a
// head-sharded decode step.  Memory comes from cudaMalloc and is mapped into the other processes with
// the CUDA IPC calls; the kernels only ever use plain loads and stores on it (no TMA, no multicast).
#include "common.cuh"

namespace piekv {
namespace {

// step_ptr != nullptr: the step number is read from device memory and, once every flag has reached it,
// incremented for the next launch (so that a captured graph of [decode step, wait] can be replayed).
__global__ void peer_wait_kernel(const int32_t *flags, int world, int step_arg, int32_t *step_ptr, int32_t *err) {
  const int r = threadIdx.x;
  int step = step_arg;
  if (step_ptr != nullptr) step = ld_global_relaxed_sys(step_ptr);
  __syncwarp();  // every lane has read the counter before lane 0 rewrites it below
  if (r < world) {
    const uint64_t t0 = global_timer_ns();
    for (;;) {
      int32_t v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
      if (v - step >= 0) break;  // step numbers only grow (wrap-safe comparison)
      if (global_timer_ns() - t0 > 2000000000ull) {
        report_error(err, PIEKV_ERR_WAIT_TIMEOUT, KID_PEER, r, v);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncwarp();
  if (r == 0 && step_ptr != nullptr)
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(step_ptr), "r"(step + 1) : "memory");
}

}  // namespace
}  // namespace piekv

extern "C" int piekv_peer_alloc(int64_t bytes, void **ptr, void *handle) {
  PIEKV_REQUIRE(bytes > 0 && ptr != nullptr && handle != nullptr, "peer_alloc: bad arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == PIEKV_PEER_HANDLE_BYTES, "handle size");
  void *p = nullptr;
  if (int rc = piekv::cuda_status(cudaMalloc(&p, (size_t)bytes), "peer_alloc: cudaMalloc")) return rc;
  if (int rc = piekv::cuda_status(cudaMemset(p, 0, (size_t)bytes), "peer_alloc: cudaMemset")) {
    cudaFree(p);
    return rc;
  }
  cudaIpcMemHandle_t h;
  if (int rc = piekv::cuda_status(cudaIpcGetMemHandle(&h, p), "peer_alloc: cudaIpcGetMemHandle")) {
    cudaFree(p);
    return rc;
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return 0;
}

extern "C" int piekv_peer_open(const void *handle, void **ptr) {
  PIEKV_REQUIRE(handle != nullptr && ptr != nullptr, "peer_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void *p = nullptr;
  if (int rc = piekv::cuda_status(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "peer_open"))
    return rc;
  *ptr = p;
  return 0;
}

extern "C" int piekv_peer_close(void *ptr) {
  if (ptr == nullptr) return 0;
  return piekv::cuda_status(cudaIpcCloseMemHandle(ptr), "peer_close");
}

extern "C" int piekv_peer_free(void *ptr) {
  if (ptr == nullptr) return 0;
  return piekv::cuda_status(cudaFree(ptr), "peer_free");
}

extern "C" int piekv_peer_wait(const int32_t *flags, int32_t world, int32_t step, int32_t *err, void *stream) {
  PIEKV_REQUIRE(flags != nullptr && world >= 1 && world <= PIEKV_MAX_PEERS, "peer_wait: bad arguments");
  piekv::peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, world, step, nullptr, err);
  PIEKV_LAUNCH_CHECK("peer_wait_kernel");
  return 0;
}

extern "C" int piekv_peer_wait_counted(const int32_t *flags, int32_t world, int32_t *step_counter, int32_t *err,
                                       void *stream) {
  PIEKV_REQUIRE(flags != nullptr && step_counter != nullptr && world >= 1 && world <= PIEKV_MAX_PEERS,
                "peer_wait_counted: bad arguments");
  piekv::peer_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flags, world, 0, step_counter, err);
  PIEKV_LAUNCH_CHECK("peer_wait_kernel");
  return 0;
}
