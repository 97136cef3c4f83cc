// Library-level plumbing: version, per-thread error text, device property cache.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace piekv {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_status(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return 0;
  set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
  return -(int)e;
}

int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static int g_options[8] = {0};

int get_option(int key) { return key >= 0 && key < 8 ? g_options[key] : 0; }

}  // namespace piekv

extern "C" int piekv_set_option(int32_t key, int32_t value) {
  PIEKV_REQUIRE(key >= 0 && key < 8, "set_option: unknown key %d", key);
  if (key == PIEKV_OPT_PDL) PIEKV_REQUIRE(value >= 0 && value <= 3, "set_option: PDL mode %d not in 0..3", value);
  if (key == PIEKV_OPT_WORK_STEALING) PIEKV_REQUIRE(value == 0 || value == 1, "set_option: work stealing must be 0 or 1");
  piekv::g_options[key] = value;
  return 0;
}

extern "C" int piekv_version(void) { return PIEKV_VERSION; }

extern "C" int32_t piekv_abi_sizeof(int32_t which) {
  if (which == 0) return (int32_t)sizeof(piekv_rope_params);
  if (which == 1) return (int32_t)sizeof(piekv_peer_outputs);
  if (which == 2) return (int32_t)sizeof(piekv_attn_options);
  if (which == 3) return (int32_t)sizeof(piekv_wire_batch);
  if (which == 4) return (int32_t)sizeof(piekv_qkv_options);
  if (which == 5) return (int32_t)sizeof(piekv_peer_reduce);
  return -1;
}

extern "C" const char *piekv_last_error_string(void) { return piekv::g_err; }
