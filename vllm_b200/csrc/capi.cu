// Library-wide state of libb200pa: thread-local error text, launch counter,
// the device status word, and the small C-ABI utility entry points.
#include <cstring>

#include "common.cuh"

namespace b200pa {

__device__ int g_status_word = 0;

static thread_local char t_error[512] = "";
static thread_local int64_t t_launches = 0;

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

void count_launch(int n) { t_launches += n; }

int* device_status_ptr() {
  constexpr int kMaxDev = 64;
  static int* cache[kMaxDev] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
    set_error("cudaGetDevice failed or device index out of range");
    return nullptr;
  }
  int* p = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_status_word);
    if (e != cudaSuccess) {
      set_error("cudaGetSymbolAddress(g_status_word) failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    __atomic_store_n(&cache[dev], p, __ATOMIC_RELEASE);
  }
  return p;
}

}  // namespace b200pa

extern "C" const char* b200pa_last_error(void) { return b200pa::t_error; }

extern "C" int b200pa_version(void) { return B200PA_VERSION; }

extern "C" int64_t b200pa_launch_count(int reset) {
  const int64_t v = b200pa::t_launches;
  if (reset) b200pa::t_launches = 0;
  return v;
}

extern "C" int b200pa_kv_dtype_from_string(const char* s) {
  if (s == nullptr) return -1;
  if (!strcmp(s, "auto")) return B200PA_KV_AUTO;
  if (!strcmp(s, "fp8") || !strcmp(s, "fp8_e4m3") || !strcmp(s, "fp8_ds_mla"))
    return B200PA_KV_FP8_E4M3;
  if (!strcmp(s, "fp8_e5m2")) return B200PA_KV_FP8_E5M2;
  return -1;
}

extern "C" int b200pa_device_status(int32_t* status) {
  using namespace b200pa;
  B200PA_CHECK_ARG(status != nullptr, "status is NULL");
  int v = 0;
  B200PA_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)));
  if (v != 0) {
    const int zero = 0;
    B200PA_CHECK_CUDA(cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int)));
  }
  *status = v;
  return B200PA_OK;
}
