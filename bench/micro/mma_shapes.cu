// tcgen05.mma throughput by shape: clocks per MMA (issue and completion) for M=128 and
// N = 64/128/256, operands from shared memory (SS) or A from TMEM (TS), K-major or MN-major B.
// One CTA per SM issues 4096 MMAs back to back from one thread.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_shapes bench/micro/mma_shapes.cu -lcuda
//   ./mma_shapes
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include "../../csrc/common.cuh"
using namespace tpb;

// mode: 0 = SS K-major A,B ; 1 = TS (A tmem) B MN-major ; 2 = SS, B MN-major; 3 = TS B K-major
template <int N, int MODE>
__global__ void __launch_bounds__(128, 1) bench_kernel(long long* out, int iters, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_barrier_init(); }
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  // zero shared memory operands
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, N, false, MODE == 1 || MODE == 2);
    const uint32_t aA = smem_u32(smem), aB = smem_u32(smem + 64 * 1024);
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint64_t ad = make_smem_desc(aA + (k >> 2) * (128 * 128) + (k & 3) * 32, 16, 1024);
        uint64_t bd;
        if (MODE == 1 || MODE == 2) bd = make_smem_desc(aB + (k & 3) * 2048, 64 * 128, 1024);
        else bd = make_smem_desc(aB + (k >> 2) * (N * 128) + (k & 3) * 32, 16, 1024);
        if (MODE == 0 || MODE == 2) mma_ss(tm + ((N <= 128) ? (it & 1) * 256 : 0), ad, bd, idesc, 1);
        else mma_ts(tm + ((N <= 128) ? (it & 1) * 256 : 0), tm + 480 + (k & 3) * 8, bd, idesc, 1);
      }
    }
    long long t1 = clock64();
    tc_commit(&bar);
    mbar_wait(&bar, 0, status, 1, 99);
    long long t2 = clock64();
    out[blockIdx.x * 2] = t1 - t0;
    out[blockIdx.x * 2 + 1] = t2 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

template <int N, int MODE>
void run(const char* name, long long* d_out, int* d_status) {
  const int iters = 512;
  cudaFuncSetAttribute(bench_kernel<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  for (int rep = 0; rep < 2; ++rep) bench_kernel<N, MODE><<<148, 128, 200 * 1024>>>(d_out, iters, d_status);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[4];
  cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost);
  const double n = iters * 8.0;
  printf("%-28s N=%3d  issue %.1f clk/mma  complete %.1f clk/mma  (ideal %.0f)  err=%d\n", name, N, h[0] / n, h[1] / n,
         128.0 * N * 16 / 4096.0, (int)e);
}

int main() {
  long long* d_out; int* d_status;
  cudaMalloc(&d_out, 148 * 2 * sizeof(long long));
  cudaMalloc(&d_status, 64); cudaMemset(d_status, 0, 64);
  run<64, 0>("SS A,B K-major", d_out, d_status);
  run<128, 0>("SS A,B K-major", d_out, d_status);
  run<256, 0>("SS A,B K-major", d_out, d_status);
  run<64, 3>("TS B K-major", d_out, d_status);
  run<128, 3>("TS B K-major", d_out, d_status);
  run<128, 1>("TS B MN-major", d_out, d_status);
  run<256, 1>("TS B MN-major", d_out, d_status);
  run<128, 2>("SS B MN-major", d_out, d_status);
  int hs[4]; cudaMemcpy(hs, d_status, 16, cudaMemcpyDeviceToHost);
  printf("status %d %d %d %d\n", hs[0], hs[1], hs[2], hs[3]);
  return 0;
}
