// Symmetric-memory runtime: device allocations that every rank of a group maps into its own address
// space, so that kernels can read, write and `red.add` into peers' buffers over NVLink.
//
// Each rank allocates a segment with cudaMalloc, exports it as a 64-byte inter-process handle, and
// opens the handles of its peers (the handles travel over the host-side process group).  A segment
// carries a small signal pad next to the payload; tpb_symm_barrier() is a device-side barrier on
// those pads: every rank stores the epoch into slot [rank] of every peer's pad and then waits, with
// a cycle budget, until all slots of its own pad have reached the epoch.  A wait that runs out
// reports kTimeoutPeerFlag into the status block and the kernel returns; nothing spins forever.
//
// A record of live segments lets tpb_symm_close_all() unmap peers before the owner frees.

#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "tpb.h"

namespace tpb {

constexpr size_t kPadBytes = 256;        // signal pad: 64 u32 slots in front of the payload
constexpr int kMaxRanks = 64;

struct Segment {
  void* base = nullptr;                  // cudaMalloc'd (owner) or mapped (peer) base, pad first
  size_t bytes = 0;
  bool mine = false;
};

static std::mutex g_mu;
static std::unordered_map<void*, Segment> g_segments;   // keyed by payload pointer

}  // namespace tpb

// Allocate `bytes` of zeroed payload (plus the pad) on the current device.  `payload` receives the
// payload pointer (256-byte aligned), `handle64` the exportable handle of the whole segment.
extern "C" int tpb_symm_alloc(long long bytes, void** payload, unsigned char* handle64) {
  if (bytes <= 0 || !payload || !handle64) return -2;
  void* base = nullptr;
  size_t total = tpb::kPadBytes + ((size_t)bytes + 255) / 256 * 256;
  cudaError_t e = cudaMalloc(&base, total);
  if (e != cudaSuccess) return 1000 + (int)e;
  e = cudaMemset(base, 0, total);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, base);
  if (e != cudaSuccess) {
    cudaFree(base);
    cudaGetLastError();
    return 1000 + (int)e;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  std::memcpy(handle64, &h, 64);
  *payload = static_cast<char*>(base) + tpb::kPadBytes;
  std::lock_guard<std::mutex> g(tpb::g_mu);
  tpb::g_segments[*payload] = {base, total, true};
  return 0;
}

// Map a peer's segment; `payload` receives the address of its payload in this process.
extern "C" int tpb_symm_open(const unsigned char* handle64, void** payload) {
  if (!handle64 || !payload) return -2;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  void* base = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 1000 + (int)e;
  }
  *payload = static_cast<char*>(base) + tpb::kPadBytes;
  std::lock_guard<std::mutex> g(tpb::g_mu);
  tpb::g_segments[*payload] = {base, 0, false};
  return 0;
}

// Unmap a peer segment or free an own one.  The caller orders this after a host barrier: an owner
// must not free while a peer still has the segment mapped.
extern "C" int tpb_symm_release(void* payload) {
  tpb::Segment s;
  {
    std::lock_guard<std::mutex> g(tpb::g_mu);
    auto it = tpb::g_segments.find(payload);
    if (it == tpb::g_segments.end()) return -2;
    s = it->second;
    tpb::g_segments.erase(it);
  }
  cudaError_t e = s.mine ? cudaFree(s.base) : cudaIpcCloseMemHandle(s.base);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return 1000 + (int)e;
  }
  return 0;
}

// Copy `bytes` from (or to) a mapped segment with the copy engine, ordered on `stream`.
extern "C" int tpb_symm_copy(void* dst, const void* src, long long bytes, void* stream) {
  cudaError_t e = cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToDevice,
                                  reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

extern "C" int tpb_symm_live_segments(void) {
  std::lock_guard<std::mutex> g(tpb::g_mu);
  return (int)tpb::g_segments.size();
}

namespace tpb {

struct BarrierPeers {
  unsigned* pad[kMaxRanks];
};

// One thread per peer.  Epochs only grow; the comparison is on the signed difference so that a
// wrapped counter still orders correctly.
__global__ void symm_barrier_kernel(BarrierPeers peers, int rank, int world, unsigned epoch, int* status) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.pad[t] + rank), "r"(epoch) : "memory");
  const unsigned* mine = peers.pad[rank] + t;
  const long long t0 = clock64();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - epoch) >= 0) break;
    if (clock64() - t0 > kSpinBudgetCycles) {
      report(status, kTimeoutPeerFlag, 90);
      break;
    }
    __nanosleep(100);
  }
}

}  // namespace tpb

// Device-side barrier over the ranks whose payload pointers are given (this rank's own included, at
// index `rank`).  Ordered on `stream`: work enqueued before it on every rank is complete and
// visible to all ranks' work enqueued after it.
extern "C" int tpb_symm_barrier(void* const* payloads, int rank, int world, unsigned epoch, void* stream) {
  if (world < 1 || world > tpb::kMaxRanks || rank < 0 || rank >= world) return -2;
  tpb::BarrierPeers peers;
  for (int i = 0; i < world; ++i)
    peers.pad[i] = reinterpret_cast<unsigned*>(static_cast<char*>(payloads[i]) - tpb::kPadBytes);
  tpb::symm_barrier_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(peers, rank, world, epoch,
                                                                                 tpb::status_block());
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
