// Process-wide runtime pieces shared by all kernels: the host-mapped status block
// that bounded waits report into, and device queries.

#include <mutex>

#include "common.cuh"
#include "tpb.h"

namespace tpb {

static int* g_status_host = nullptr;
static int* g_status_dev = nullptr;

int* status_block() {
  static std::once_flag once;
  std::call_once(once, [] {
    // Mapped pinned memory: kernels write it with system-scope atomics, the host
    // polls it without touching the device.
    if (cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), 4 * sizeof(int), cudaHostAllocMapped) ==
        cudaSuccess) {
      for (int i = 0; i < 4; ++i) g_status_host[i] = 0;
      cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_status_dev), g_status_host, 0);
    }
  });
  return g_status_dev;
}

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

}  // namespace tpb

extern "C" int tpb_status(int* out4) {
  tpb::status_block();
  if (!tpb::g_status_host) return -1;
  for (int i = 0; i < 4; ++i) out4[i] = reinterpret_cast<volatile int*>(tpb::g_status_host)[i];
  return 0;
}
extern "C" void tpb_status_clear(void) {
  tpb::status_block();
  if (tpb::g_status_host)
    for (int i = 0; i < 4; ++i) tpb::g_status_host[i] = 0;
}
extern "C" int tpb_sm_count(void) { return tpb::sm_count(); }
