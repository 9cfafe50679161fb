// Cost of the MMA-issuer <-> compute-warp handshake in an attention-style pipeline.
//
// One CTA per SM runs the tensor-core instruction stream of one attention-backward step
// (16 SS MMAs 128x64x16 into a double-buffered score tile, then 4 TS MMAs 128x128x16 that read
// their A operand from TMEM) 512 times, and features of the real kernel are switched on one
// at a time: compute warps doing the exp math, compute warps reading/writing TMEM, compute
// warps waiting on the commit barrier, arriving on the return barrier, and finally the MMA
// thread waiting on that barrier.  Prints clocks per step for every rung and, for the last
// one, the event times of four consecutive steps.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 --use_fast_math \
//        -o mma_handshake bench/micro/mma_handshake.cu -lcuda && ./mma_handshake
#include <cstdio>
#include <cstdint>
#include <cuda_runtime.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include "../../csrc/common.cuh"  // PTX wrappers of the framework
using namespace tpb;

// WAIT_MMA: MMA thread waits for ds_full.  WAIT_CMP: compute waits for sdp_full.  TMEM: compute touches TMEM.
// MATH: compute does the exp math.  ARRIVE: 0 none, 1 all threads, 2 one lane per warp.
template <int WAIT_MMA, bool WAIT_CMP, bool TMEM, bool MATH, int ARRIVE>
__global__ void __launch_bounds__(352, 1) skel(long long* out, int iters, int* status, float* sink, long long* ts) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ uint64_t sdp_full[2], ds_full[2], done_bar, dummy[2];
  __shared__ uint32_t slot;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&ds_full[i], ARRIVE == 2 ? 8 : 256); mbar_init(&dummy[i], 1); }
    mbar_init(&done_bar, 1);
    fence_barrier_init();
  }
  if (threadIdx.x < 32) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  for (int i = threadIdx.x; i < 160 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 32) {
    constexpr uint32_t id_s = make_idesc_bf16(128, 64, false, false);
    constexpr uint32_t id_dq = make_idesc_bf16(128, 128, false, true);
    const uint32_t aA = smem_u32(smem), aB = smem_u32(smem + 64 * 1024);
    auto scores = [&](int j) {
      const uint32_t tS = tm + 128 + (j & 1) * 128;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint64_t ad = make_smem_desc(aA + (k >> 2) * (128 * 128) + (k & 3) * 32, 16, 1024);
        uint64_t bd = make_smem_desc(aB + (k >> 2) * (64 * 128) + (k & 3) * 32, 16, 1024);
        mma_ss(tS, ad, bd, id_s, k != 0);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        uint64_t ad = make_smem_desc(aA + 32768 + (k >> 2) * (128 * 128) + (k & 3) * 32, 16, 1024);
        uint64_t bd = make_smem_desc(aB + 16384 + (k >> 2) * (64 * 128) + (k & 3) * 32, 16, 1024);
        mma_ss(tS + 64, ad, bd, id_s, k != 0);
      }
      tc_commit(&dummy[0]);
      tc_commit(&sdp_full[j & 1]);
    };
    long long t0 = clock64();
    scores(0);
    bool ok = true;
    if (WAIT_MMA == 5) {
      // two issuing threads: this one only issues the score MMAs; it may run one step ahead of
      // the compute warps (buffer (j+1)&1 is free once they arrived for step j-1)
      for (int j = 0; j < iters && ok; ++j) {
        if (j >= 1) { ok = mbar_wait(&ds_full[(j - 1) & 1], ((j - 1) >> 1) & 1, status, 2, 95); tc_fence_after(); }
        if (j + 1 < iters) scores(j + 1);
      }
      iters = 0;
    }
    for (int j = 0; j < iters && ok; ++j) {
      const bool rec = ts && blockIdx.x == 0 && j >= 100 && j < 104;
      if (rec) ts[(j - 100) * 8 + 0] = clock64() - t0;
      if (j + 1 < iters) scores(j + 1);
      if (rec) ts[(j - 100) * 8 + 1] = clock64() - t0;
      if (WAIT_MMA == 1 || WAIT_MMA == 2) ok = mbar_wait(&ds_full[j & 1], (j >> 1) & 1, status, 2, 97);
      if (WAIT_MMA == 1 || WAIT_MMA == 3) tc_fence_after();
      if (WAIT_MMA == 4) { while (!mbar_test(&ds_full[j & 1], (j >> 1) & 1)) {} tc_fence_after(); }
      if (rec) ts[(j - 100) * 8 + 2] = clock64() - t0;
      const uint32_t tDS = tm + 128 + (j & 1) * 128 + 64;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint64_t bd = make_smem_desc(aB + k * 2048, 64 * 128, 1024);
        mma_ts(tm, tDS + (k >> 1) * 32 + (k & 1) * 8, bd, id_dq, (j | k) != 0);
      }
      tc_commit(&dummy[1]);
      if (rec) ts[(j - 100) * 8 + 3] = clock64() - t0;
    }
    if (ts && blockIdx.x == 0) ts[63] = t0;
    if (WAIT_MMA != 5) {
      tc_commit(&done_bar);
      mbar_wait(&done_bar, 0, status, 1, 99);
      out[blockIdx.x] = clock64() - t0;
    }
  } else if (warp == 10) {
    if (WAIT_MMA == 5 && lane == 0) {
      constexpr uint32_t id_dq = make_idesc_bf16(128, 128, false, true);
      const uint32_t aB = smem_u32(smem + 64 * 1024);
      long long t0 = clock64();
      bool ok = true;
      for (int j = 0; j < iters && ok; ++j) {
        ok = mbar_wait(&ds_full[j & 1], (j >> 1) & 1, status, 2, 97);
        tc_fence_after();
        const uint32_t tDS = tm + 128 + (j & 1) * 128 + 64;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          uint64_t bd = make_smem_desc(aB + k * 2048, 64 * 128, 1024);
          mma_ts(tm, tDS + (k >> 1) * 32 + (k & 1) * 8, bd, id_dq, (j | k) != 0);
        }
        tc_commit(&dummy[1]);
      }
      tc_commit(&done_bar);
      mbar_wait(&done_bar, 0, status, 1, 99);
      out[blockIdx.x] = clock64() - t0;
    }
  } else if (warp >= 2) {
    const int half = (warp - 2) >> 2;
    const uint32_t tb = tm + ((uint32_t)((warp & 3) * 32) << 16);
    float lse2 = 3.f + lane * 0.01f, delta = 0.5f;
    bool ok = true;
    for (int j = 0; j < iters && ok; ++j) {
      const bool rec = ts && blockIdx.x == 0 && threadIdx.x == 64 && j >= 100 && j < 105;
      if (rec) ts[32 + (j - 100) * 4 + 0] = clock64();
      if (WAIT_CMP) { ok = mbar_wait(&sdp_full[j & 1], (j >> 1) & 1, status, 3, 96); tc_fence_after(); }
      if (rec) ts[32 + (j - 100) * 4 + 1] = clock64();
      const uint32_t tS = tb + 128 + (j & 1) * 128 + half * 32, tDP = tS + 64;
      uint32_t s[32], dp[32], pk[16];
      if (TMEM) {
        tmem_ld32(tS, s);
        tmem_ld32(tDP, dp);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) { s[c] = j + c; dp[c] = j - c; }
      }
      if (MATH) {
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          const float p0 = exp2f(fmaf(__uint_as_float(s[c]), 0.127f, -lse2));
          const float p1 = exp2f(fmaf(__uint_as_float(s[c + 1]), 0.127f, -lse2));
          pk[c / 2] = pack_bf16(p0 * (__uint_as_float(dp[c]) - delta), p1 * (__uint_as_float(dp[c + 1]) - delta));
        }
      } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) pk[c] = s[c] ^ dp[c];
      }
      if (TMEM) {
        tmem_st16(tDP, pk);
        tmem_wait_st();
        tc_fence_before();
      } else if (pk[3] == 0x12345) sink[1] = 1.f;
      if (ARRIVE == 1) mbar_arrive(&ds_full[j & 1]);
      if (ARRIVE == 2) { __syncwarp(); if (lane == 0) mbar_arrive(&ds_full[j & 1]); }
      if (rec) ts[32 + (j - 100) * 4 + 2] = clock64();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tm, 512); }
}

template <int A, bool B, bool C, bool D, int E>
void run(const char* name, long long* d_out, int* d_status, float* sink, long long* ts = nullptr) {
  cudaFuncSetAttribute(skel<A, B, C, D, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  int iters_unused = 0; (void)iters_unused;
  const int iters = 512;
  for (int rep = 0; rep < 2; ++rep) skel<A, B, C, D, E><<<148, 352, 200 * 1024>>>(d_out, iters, d_status, sink, ts);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[1];
  cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost);
  printf("%-60s %.0f clk/step (err=%d)\n", name, (double)h[0] / iters, (int)e);
  if (ts) {
    long long t[64]; cudaMemcpy(t, ts, sizeof(t), cudaMemcpyDeviceToHost);
    const long long t0 = t[63], base = t[0];
    for (int j = 0; j < 4; ++j)
      printf("  j=%d mma: begin %lld scores_issued %lld wait_done %lld dq_issued %lld | compute: wait_begin %lld woke %lld arrived %lld\n", 100 + j,
             t[j * 8] - base, t[j * 8 + 1] - base, t[j * 8 + 2] - base, t[j * 8 + 3] - base, t[32 + j * 4] - t0 - base, t[32 + j * 4 + 1] - t0 - base,
             t[32 + j * 4 + 2] - t0 - base);
  }
}

int main() {
  long long* d_out; int* d_status; float* sink;
  cudaMalloc(&d_out, 148 * sizeof(long long));
  cudaMalloc(&sink, 64);
  cudaMalloc(&d_status, 64); cudaMemset(d_status, 0, 64);
  long long* ts; cudaMalloc(&ts, 64 * 8); cudaMemset(ts, 0, 64 * 8);
  run<0, false, false, false, 0>("mma thread alone", d_out, d_status, sink);
  run<0, false, false, true, 0>("+ compute warps: exp math, free-running", d_out, d_status, sink);
  run<0, false, true, true, 0>("+ compute warps: tcgen05.ld/st, free-running", d_out, d_status, sink);
  run<0, true, true, true, 0>("+ compute warps wait for the score commit", d_out, d_status, sink);
  run<0, true, true, true, 1>("+ compute warps arrive (256 arrivals)", d_out, d_status, sink);
  run<1, true, true, true, 1>("+ mma thread waits for them (full handshake)", d_out, d_status, sink);
  run<1, true, true, true, 2>("full handshake, one arrival per warp", d_out, d_status, sink);
  run<1, true, false, false, 1>("full handshake, no math, no TMEM traffic", d_out, d_status, sink, ts);
  run<5, true, true, true, 1>("full handshake, two issuing threads (scores / dQ)", d_out, d_status, sink);
  int hs[4]; cudaMemcpy(hs, d_status, 16, cudaMemcpyDeviceToHost);
  printf("status %d %d %d %d\n", hs[0], hs[1], hs[2], hs[3]);
  return 0;
}
