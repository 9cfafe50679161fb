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

// A wait that is meant to run out: spins (bounded by `budget_cycles`) until *flag == expected and
// reports kTimeoutPeerFlag into the status block when the budget is exhausted.  Used by the
// failure-detection tests to show that a stuck wait ends with a status code, not with a hung GPU.
__global__ void bounded_wait_kernel(const unsigned* flag, unsigned expected, long long budget_cycles, int* status,
                                    int* result) {
  const long long t0 = clock64();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v == expected) {
      *result = 1;
      return;
    }
    if (clock64() - t0 > budget_cycles) {
      tpb::report(status, tpb::kTimeoutPeerFlag, 99);
      *result = -1;
      return;
    }
    __nanosleep(200);
  }
}

extern "C" int tpb_bounded_wait(const unsigned* flag, unsigned expected, long long budget_cycles, int* result,
                                void* stream) {
  bounded_wait_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, expected, budget_cycles,
                                                                           tpb::status_block(), result);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
