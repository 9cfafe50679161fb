// L2 -> shared memory bulk-copy bandwidth and latency: every SM streams 16 KB chunks of an
// L2-resident buffer through a ring of 1..6 copies in flight.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o l2_to_smem bench/micro/l2_to_smem.cu -lcuda
//   ./l2_to_smem
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include "../../csrc/common.cuh"
using namespace tpb;

constexpr int STAGES = 6;
constexpr int CHUNK = 16384;

// pattern 0: every CTA reads the same 2 MB region; 1: CTA-private 1 MB regions (148 MB total > L2? no: use 64 MB total);
__global__ void __launch_bounds__(64, 1) l2_kernel(const uint8_t* buf, long long buf_bytes, int iters, int pattern, int inflight,
                                                   long long* out, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t full[STAGES];
  if (threadIdx.x == 0) { for (int i = 0; i < STAGES; ++i) mbar_init(&full[i], 1); fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x == 0) {
    const long long region = pattern == 0 ? (2LL << 20) : (buf_bytes / gridDim.x / CHUNK * CHUNK);
    const uint8_t* base = pattern == 0 ? buf : buf + region * blockIdx.x;
    const int nchunk = (int)(region / CHUNK);
    long long t0 = clock64();
    int issued = 0, done = 0;
    while (done < iters) {
      while (issued < iters && issued - done < inflight) {
        const int st = issued % STAGES;
        mbar_expect_tx(&full[st], CHUNK);
        const uint8_t* src = base + (long long)((issued * 7 + blockIdx.x) % nchunk) * CHUNK;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(smem + st * CHUNK)), "l"(src), "r"(CHUNK), "r"(smem_u32(&full[st])) : "memory");
        ++issued;
      }
      if (!mbar_wait(&full[done % STAGES], (done / STAGES) & 1, status, 1, 98)) break;
      ++done;
    }
    out[blockIdx.x] = clock64() - t0;
  }
}

int main() {
  const long long bytes = 64LL << 20;
  uint8_t* buf; cudaMalloc(&buf, bytes); cudaMemset(buf, 1, bytes);
  long long* d_out; int* d_status;
  cudaMalloc(&d_out, 148 * sizeof(long long));
  cudaMalloc(&d_status, 64); cudaMemset(d_status, 0, 64);
  cudaFuncSetAttribute(l2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, STAGES * CHUNK + 2048);
  const int iters = 4096;
  for (int pattern = 0; pattern < 2; ++pattern)
    for (int inflight = 1; inflight <= STAGES; inflight += (inflight < 2 ? 1 : 2)) {
      cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
      l2_kernel<<<148, 64, STAGES * CHUNK + 2048>>>(buf, bytes, iters, pattern, inflight, d_out, d_status);
      cudaEventRecord(e0);
      l2_kernel<<<148, 64, STAGES * CHUNK + 2048>>>(buf, bytes, iters, pattern, inflight, d_out, d_status);
      cudaEventRecord(e1);
      cudaError_t e = cudaDeviceSynchronize();
      float ms; cudaEventElapsedTime(&ms, e0, e1);
      long long h[148]; cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost);
      double avg = 0; for (int i = 0; i < 148; ++i) avg += h[i]; avg /= 148;
      printf("pattern=%d inflight=%d: %.1f B/clk/SM, latency-ish %.0f clk/chunk, %.2f TB/s aggregate (err=%d)\n", pattern, inflight,
             (double)iters * CHUNK / avg, avg / iters * inflight, 148.0 * iters * CHUNK / ms / 1e9, (int)e);
    }
  int hs[4]; cudaMemcpy(hs, d_status, 16, cudaMemcpyDeviceToHost);
  printf("status %d %d %d %d\n", hs[0], hs[1], hs[2], hs[3]);
  return 0;
}
