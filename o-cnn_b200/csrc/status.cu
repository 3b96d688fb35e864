// Error state of the C ABI (one message per calling thread) and the version queries.
#include <atomic>

#include "common.cuh"

namespace ocnn {

static thread_local char g_error[512] = "";
static std::atomic<long long> g_launches{0};

int sm_count() {
  static std::mutex mutex;
  static int cached[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return kSMs;
  std::lock_guard<std::mutex> lock(mutex);
  if (cached[device] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0)
      n = kSMs;
    cached[device] = n;
  }
  return cached[device];
}

void note_launches(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return status;
}

TapList taps_for_kernel(const int ks[3]) {
  TapList out;
  out.count = -1;
  auto set = [&](std::initializer_list<int> v) {
    out.count = 0;
    for (int t : v) out.tap[out.count++] = (signed char)t;
  };
  switch (ks[0] * 100 + ks[1] * 10 + ks[2]) {
    case 333:
      out.count = 27;
      for (int i = 0; i < 27; ++i) out.tap[i] = (signed char)i;
      break;
    case 111: set({13}); break;
    case 222: set({13, 14, 16, 17, 22, 23, 25, 26}); break;
    case 311: set({4, 13, 22}); break;
    case 131: set({10, 13, 16}); break;
    case 113: set({12, 13, 14}); break;
    case 331: set({1, 4, 7, 10, 13, 16, 19, 22, 25}); break;
    case 313: set({3, 4, 5, 12, 13, 14, 21, 22, 23}); break;
    case 133: set({9, 10, 11, 12, 13, 14, 15, 16, 17}); break;
    default: break;
  }
  return out;
}

}  // namespace ocnn

extern "C" {

const char* ocnn_last_error(void) { return ocnn::g_error; }
int ocnn_version(void) { return 100; }
int ocnn_compiled_arch(void) { return 100; }
long long ocnn_launch_count(void) { return ocnn::g_launches.load(std::memory_order_relaxed); }

}  // extern "C"
