// Bandwidth-bound kernels of the training step: RMSNorm (+residual) fwd/bwd, RoPE,
// SwiGLU, softmax cross-entropy (fused forward + gradient), embedding gather /
// scatter-add, fused AdamW and the gradient-norm reduction.  All of them move
// 16-byte vectors, keep a row in registers between its passes and run on grids
// sized from the SM count.

#include "common.cuh"
#include "tpb.h"

namespace tpb {

int sm_count();

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` is 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = lane < nw ? red[lane] : -INFINITY;
  return warp_max(t);
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
// bf16 rounding of a float (keeps fp32 type) so results match torch's bf16 ops
__device__ __forceinline__ float rbf(float x) { return __bfloat162float(__float2bfloat16(x)); }

// ----------------------------------------------------------------------------
// RMSNorm
// ----------------------------------------------------------------------------
constexpr int NORM_THREADS = 256;
constexpr int NORM_VPT = 4;  // most 16-byte vectors kept in registers per thread (dim <= 8192)
// The kernels are instantiated for 1, 2 and 4 vectors per thread: a 4096-wide row needs two, and
// the instantiation that holds exactly that many leaves registers for more resident CTAs, which
// is what a latency-bound row-per-CTA kernel needs to fill the memory pipe.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res, const uint4* __restrict__ w,
                   uint4* __restrict__ y, uint4* __restrict__ h_out, float* __restrict__ rstd_out, int rows,
                   int nvec, float eps) {
  __shared__ float red[32];
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = x + (size_t)row * nvec;
    float vals[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        unpack8(xr[i], vals[j]);
        if (res) {
          float r[8];
          unpack8(res[(size_t)row * nvec + i], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) vals[j][e] = rbf(vals[j][e] + r[e]);
          if (h_out) h_out[(size_t)row * nvec + i] = pack8(vals[j]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += vals[j][e] * vals[j][e];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)(nvec * 8) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float wv[8], o[8];
        unpack8(w[i], wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = wv[e] * rbf(vals[j][e] * rstd);
        y[(size_t)row * nvec + i] = pack8(o);
      }
    }
  }
}

template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x, const uint4* __restrict__ w,
                   const float* __restrict__ rstd, const uint4* __restrict__ dres, uint4* __restrict__ dx,
                   float* __restrict__ dw, int rows, int nvec) {
  __shared__ float red[32];
  float dw_acc[VPT][8];
  float wv[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int i = threadIdx.x + j * NORM_THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[j][e] = 0.f;
    if (i < nvec) unpack8(w[i], wv[j]);
  }
  const float inv_d = 1.0f / (float)(nvec * 8);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rs = rstd[row];
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float dyv[8], xv[8];
        unpack8(dy[(size_t)row * nvec + i], dyv);
        unpack8(x[(size_t)row * nvec + i], xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = xv[e] * rs;
          dw_acc[j][e] += dyv[e] * xh[j][e];
          g[j][e] = dyv[e] * wv[j][e];
          dot += g[j][e] * xh[j][e];
        }
      }
    }
    dot = block_sum(dot, red) * inv_d;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rs * (g[j][e] - xh[j][e] * dot);
        if (dres) {
          float r[8];
          unpack8(dres[(size_t)row * nvec + i], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += r[e];
        }
        dx[(size_t)row * nvec + i] = pack8(o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        // two 16-byte vector reductions instead of eight scalar atomics
        float* dst = dw + i * 8;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(dw_acc[j][0]), "f"(dw_acc[j][1]),
                     "f"(dw_acc[j][2]), "f"(dw_acc[j][3])
                     : "memory");
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(dw_acc[j][4]),
                     "f"(dw_acc[j][5]), "f"(dw_acc[j][6]), "f"(dw_acc[j][7])
                     : "memory");
      }
    }
  }
}

constexpr int NB_MAX_STAGES = 4;
__device__ __forceinline__ void bulk_row_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Forward with its input rows streamed through shared memory by bulk copies (see the streamed backward
// below for the scheme): stage = x row | residual row.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_bulk_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res, const uint4* __restrict__ w,
                        uint4* __restrict__ y, uint4* __restrict__ h_out, float* __restrict__ rstd_out, int rows,
                        int nvec, float eps, int stages, int* status) {
  extern __shared__ uint8_t nf_smem_raw[];
  uint8_t* smem = nf_smem_raw + ((128u - (smem_u32(nf_smem_raw) & 127u)) & 127u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);   // [NB_MAX_STAGES]
  uint8_t* ring = smem + 128;
  __shared__ float red[32];
  const uint32_t row_bytes = (uint32_t)nvec * 16u;
  const uint32_t stage_bytes = 2u * row_bytes;
  const int ntens = res ? 2 : 1;
  const int my_rows = (rows - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // grid <= rows
  if (threadIdx.x == 0) {
    for (int s = 0; s < NB_MAX_STAGES; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
  }
  __syncthreads();
  auto issue = [&](int k) {   // thread 0: request row k of this CTA
    const int s = k % stages;
    const size_t off = ((size_t)blockIdx.x + (size_t)k * gridDim.x) * nvec;
    uint8_t* dst = ring + (size_t)s * stage_bytes;
    mbar_expect_tx(&full[s], (uint32_t)ntens * row_bytes);
    bulk_row_load(dst, x + off, row_bytes, &full[s]);
    if (res) bulk_row_load(dst + row_bytes, res + off, row_bytes, &full[s]);
  };
  int issued = 0;
  if (threadIdx.x == 0)
    for (; issued < stages - 1 && issued < my_rows; ++issued) issue(issued);
  float wv[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int i = threadIdx.x + j * NORM_THREADS;
    if (i < nvec) unpack8(w[i], wv[j]);
  }
  bool ok = true;
  int k = 0, drain_from = -1;
  for (; k < my_rows; ++k) {
    ok = __syncthreads_and(ok);     // every thread is done with the stage the next request goes into
    if (!ok) break;
    if (threadIdx.x == 0 && issued < my_rows) {
      fence_proxy_async();
      issue(issued++);
    }
    const int s = k % stages;
    ok = mbar_wait(&full[s], (uint32_t)(k / stages) & 1u, status, kTimeoutTmaFull, 73);
    if (!ok && drain_from < 0) drain_from = k;
    const uint4* sx = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes);
    const uint4* sres = sx + nvec;
    const size_t row = (size_t)blockIdx.x + (size_t)k * gridDim.x;
    float vals[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        unpack8(sx[i], vals[j]);
        if (res) {
          float r[8];
          unpack8(sres[i], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) vals[j][e] = rbf(vals[j][e] + r[e]);
          if (h_out) h_out[row * nvec + i] = pack8(vals[j]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += vals[j][e] * vals[j][e];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)(nvec * 8) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = wv[j][e] * rbf(vals[j][e] * rstd);
        y[row * nvec + i] = pack8(o);
      }
    }
  }
  if (drain_from < 0 && k < my_rows) drain_from = k;
  if (drain_from >= 0 && threadIdx.x == 0)
    for (int kk = drain_from; kk < issued; ++kk)
      mbar_wait(&full[kk % stages], (uint32_t)(kk / stages) & 1u, status, kTimeoutTmaFull, 74);
}

// The same backward with its inputs streamed through shared memory by bulk copies.
//
// The kernel above is bound by latency, not by bandwidth: a CTA loads a row, reduces across the
// block, loads the residual gradient, stores, and only then asks for the next row, so an SM has a
// row or two in flight where HBM needs some 50 KB per SM to stay busy.  Here one thread issues
// `cp.async.bulk` copies of the rows `stages - 1` iterations ahead into a ring of shared-memory
// stages (dy | x | dres of one row each, completion counted on an mbarrier per stage); the 256
// threads read the rows from shared memory.  A stage is handed back by the block-wide barrier that
// opens every iteration, which also carries the give-up decision of a wait that ran out, so all
// threads leave the loop together.
template <int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_bulk_kernel(const uint4* __restrict__ dy, const uint4* __restrict__ x, const uint4* __restrict__ w,
                        const float* __restrict__ rstd, const uint4* __restrict__ dres, uint4* __restrict__ dx,
                        float* __restrict__ dw, int rows, int nvec, int stages, int* status) {
  extern __shared__ uint8_t nb_smem_raw[];
  uint8_t* smem = nb_smem_raw + ((128u - (smem_u32(nb_smem_raw) & 127u)) & 127u);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem);   // [NB_MAX_STAGES]
  uint8_t* ring = smem + 128;
  __shared__ float red[32];
  const uint32_t row_bytes = (uint32_t)nvec * 16u;
  const uint32_t stage_bytes = 3u * row_bytes;
  const int ntens = dres ? 3 : 2;
  const int my_rows = (rows - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // grid <= rows
  if (threadIdx.x == 0) {
    for (int s = 0; s < NB_MAX_STAGES; ++s) mbar_init(&full[s], 1);
    fence_barrier_init();
  }
  __syncthreads();
  auto issue = [&](int k) {   // thread 0: request row k of this CTA
    const int s = k % stages;
    const size_t off = ((size_t)blockIdx.x + (size_t)k * gridDim.x) * nvec;
    uint8_t* dst = ring + (size_t)s * stage_bytes;
    mbar_expect_tx(&full[s], (uint32_t)ntens * row_bytes);
    bulk_row_load(dst, dy + off, row_bytes, &full[s]);
    bulk_row_load(dst + row_bytes, x + off, row_bytes, &full[s]);
    if (dres) bulk_row_load(dst + 2 * row_bytes, dres + off, row_bytes, &full[s]);
  };
  int issued = 0;
  if (threadIdx.x == 0)
    for (; issued < stages - 1 && issued < my_rows; ++issued) issue(issued);

  float dw_acc[VPT][8];
  float wv[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    int i = threadIdx.x + j * NORM_THREADS;
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[j][e] = 0.f;
    if (i < nvec) unpack8(w[i], wv[j]);
  }
  const float inv_d = 1.0f / (float)(nvec * 8);
  bool ok = true;
  int k = 0, drain_from = -1;
  for (; k < my_rows; ++k) {
    // every thread is done with the stage the next request goes into (it was read in iteration k - 1)
    ok = __syncthreads_and(ok);
    if (!ok) break;
    if (threadIdx.x == 0 && issued < my_rows) {
      fence_proxy_async();
      issue(issued++);
    }
    const int s = k % stages;
    ok = mbar_wait(&full[s], (uint32_t)(k / stages) & 1u, status, kTimeoutTmaFull, 71);
    if (!ok && drain_from < 0) drain_from = k;
    const uint4* sdy = reinterpret_cast<const uint4*>(ring + (size_t)s * stage_bytes);
    const uint4* sx = sdy + nvec;
    const uint4* sres = sx + nvec;
    const size_t row = (size_t)blockIdx.x + (size_t)k * gridDim.x;
    const float rs = rstd[row];
    float g[VPT][8], xh[VPT][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float dyv[8], xv[8];
        unpack8(sdy[i], dyv);
        unpack8(sx[i], xv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] = xv[e] * rs;
          dw_acc[j][e] += dyv[e] * xh[j][e];
          g[j][e] = dyv[e] * wv[j][e];
          dot += g[j][e] * xh[j][e];
        }
      }
    }
    dot = block_sum(dot, red) * inv_d;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rs * (g[j][e] - xh[j][e] * dot);
        if (dres) {
          float r[8];
          unpack8(sres[i], r);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += r[e];
        }
        dx[row * nvec + i] = pack8(o);
      }
    }
  }
  // a wait ran out: the copies that were requested and not consumed still land in this CTA's shared
  // memory, so the CTA stays until they have (bounded again)
  if (drain_from < 0 && k < my_rows) drain_from = k;
  if (drain_from >= 0 && threadIdx.x == 0)
    for (int kk = drain_from; kk < issued; ++kk)
      mbar_wait(&full[kk % stages], (uint32_t)(kk / stages) & 1u, status, kTimeoutTmaFull, 72);
  if (dw) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      int i = threadIdx.x + j * NORM_THREADS;
      if (i < nvec) {
        float* dst = dw + i * 8;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(dw_acc[j][0]), "f"(dw_acc[j][1]),
                     "f"(dw_acc[j][2]), "f"(dw_acc[j][3])
                     : "memory");
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(dw_acc[j][4]),
                     "f"(dw_acc[j][5]), "f"(dw_acc[j][6]), "f"(dw_acc[j][7])
                     : "memory");
      }
    }
  }
}

// ----------------------------------------------------------------------------
// RoPE (rotate-half; optional interleaved-pair input layout), in place.
// One thread handles 8 consecutive elements of the first half and their partners.
// ----------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, long long ld, int col0, int heads, int dim, int head_stride,
                            const float* __restrict__ cosT, const float* __restrict__ sinT,
                            const int* __restrict__ pos, long long tokens, int seq_len, float sign,
                            int interleaved) {
  const int half = dim / 2;
  const int vec_per_head = half / 8;
  const long long total = tokens * heads * vec_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % vec_per_head);
    const long long th = idx / vec_per_head;
    const int h = (int)(th % heads);
    const long long t = th / heads;
    const int p = pos ? pos[t] : (int)(t % seq_len);
    __nv_bfloat16* base = x + t * ld + col0 + h * head_stride;
    const float* c = cosT + (size_t)p * half + v * 8;
    const float* s = sinT + (size_t)p * half + v * 8;
    float a[8], b[8];
    if (!interleaved) {
      unpack8(*reinterpret_cast<const uint4*>(base + v * 8), a);
      unpack8(*reinterpret_cast<const uint4*>(base + half + v * 8), b);
    } else {
      // pairs (2i, 2i+1): element i of the first half is x[2i], of the second half x[2i+1]
      float lo[8], hi[8];
      unpack8(*reinterpret_cast<const uint4*>(base + v * 16), lo);
      unpack8(*reinterpret_cast<const uint4*>(base + v * 16 + 8), hi);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        a[e] = lo[2 * e]; b[e] = lo[2 * e + 1];
        a[4 + e] = hi[2 * e]; b[4 + e] = hi[2 * e + 1];
      }
    }
    float oa[8], ob[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float cs = c[e], sn = s[e] * sign;
      oa[e] = a[e] * cs - b[e] * sn;
      ob[e] = b[e] * cs + a[e] * sn;
    }
    if (!interleaved) {
      *reinterpret_cast<uint4*>(base + v * 8) = pack8(oa);
      *reinterpret_cast<uint4*>(base + half + v * 8) = pack8(ob);
    }
    if (interleaved) {
      // The permuted (half-layout) result cannot be written in place by independent
      // threads without a race, so the interleaved variant keeps the pair layout:
      // attention scores are invariant to a fixed permutation applied to both q and k.
      float lo[8], hi[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        lo[2 * e] = oa[e]; lo[2 * e + 1] = ob[e];
        hi[2 * e] = oa[4 + e]; hi[2 * e + 1] = ob[4 + e];
      }
      *reinterpret_cast<uint4*>(base + v * 16) = pack8(lo);
      *reinterpret_cast<uint4*>(base + v * 16 + 8) = pack8(hi);
    }
  }
}

// ----------------------------------------------------------------------------
// SwiGLU
// ----------------------------------------------------------------------------
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ gu, uint4* __restrict__ act, long long rows, int fvec) {
  const long long total = rows * fvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / fvec;
    const int c = (int)(idx % fvec);
    float g[8], u[8], o[8];
    unpack8(gu[r * 2 * fvec + c], g);
    unpack8(gu[r * 2 * fvec + fvec + c], u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    act[idx] = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ dact, const uint4* __restrict__ gu,
                                  uint4* __restrict__ dgu, long long rows, int fvec) {
  const long long total = rows * fvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / fvec;
    const int c = (int)(idx % fvec);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(gu[r * 2 * fvec + c], g);
    unpack8(gu[r * 2 * fvec + fvec + c], u);
    unpack8(dact[idx], d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sg = 1.f / (1.f + __expf(-g[e]));
      const float silu = g[e] * sg;
      du[e] = d[e] * silu;
      dg[e] = d[e] * u[e] * (sg + silu * (1.f - sg));
    }
    dgu[r * 2 * fvec + c] = pack8(dg);
    dgu[r * 2 * fvec + fvec + c] = pack8(du);
  }
}

// ----------------------------------------------------------------------------
// Cross entropy: one CTA per row, online (max, sum) pass then gradient pass.
// ----------------------------------------------------------------------------
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
ce_kernel(__nv_bfloat16* __restrict__ logits, long long ld, const long long* __restrict__ targets,
          float* __restrict__ loss_sum, const float* __restrict__ grad_scale, int rows, int vocab) {
  __shared__ float red[32];
  const int nvec = vocab / 8;  // host guarantees vocab % 8 == 0
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    uint4* lr = reinterpret_cast<uint4*>(logits + (size_t)row * ld);
    const long long tgt = targets[row];
    if (tgt < 0) {
      for (int i = threadIdx.x; i < nvec; i += CE_THREADS) lr[i] = make_uint4(0, 0, 0, 0);
      continue;
    }
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      float f[8];
      unpack8(lr[i], f);
      float lm = f[0];
#pragma unroll
      for (int e = 1; e < 8; ++e) lm = fmaxf(lm, f[e]);
      if (lm > m) {
        s *= __expf(m - lm);
        m = lm;
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) s += __expf(f[e] - m);
    }
    const float gm = block_max(m, red);
    s *= (m == -INFINITY) ? 0.f : __expf(m - gm);
    const float gs = block_sum(s, red);
    const float lse = gm + __logf(gs);
    const float scale = grad_scale ? *grad_scale : 1.f;
    if (threadIdx.x == 0) {
      const float lt = __bfloat162float(logits[(size_t)row * ld + tgt]);
      atomicAdd(loss_sum, lse - lt);
    }
    __syncthreads();  // the target logit is read before it is overwritten below
    const float inv = 1.f / gs;
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
      float f[8];
      unpack8(lr[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float p = __expf(f[e] - gm) * inv;
        if ((long long)i * 8 + e == tgt) p -= 1.f;
        f[e] = p * scale;
      }
      lr[i] = pack8(f);
    }
  }
}

// ----------------------------------------------------------------------------
// Embedding
// ----------------------------------------------------------------------------
__global__ void embedding_fwd_kernel(const uint4* __restrict__ table, const long long* __restrict__ ids,
                                     uint4* __restrict__ out, long long tokens, int nvec, long long vocab,
                                     long long row0) {
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c = (int)(idx % nvec);
    const long long id = ids[t] - row0;
    out[idx] = (id >= 0 && id < vocab) ? table[id * nvec + c] : make_uint4(0, 0, 0, 0);
  }
}
template <bool F32>
__global__ void embedding_bwd_kernel(const __nv_bfloat162* __restrict__ dout, const long long* __restrict__ ids,
                                     void* __restrict__ dtable, long long tokens, int dim2, long long rows_local,
                                     long long row0) {
  const long long total = tokens * dim2;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / dim2;
    const int c = (int)(idx % dim2);
    const long long id = ids[t] - row0;
    if (id < 0 || id >= rows_local) continue;
    const __nv_bfloat162 g = dout[idx];
    if (F32) {
      float* d = reinterpret_cast<float*>(dtable) + (id * dim2 + c) * 2;
      atomicAdd(d, __low2float(g));
      atomicAdd(d + 1, __high2float(g));
    } else {
      atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable) + id * dim2 + c, g);
    }
  }
}

// ----------------------------------------------------------------------------
// Optimizer
// ----------------------------------------------------------------------------
template <bool GBF16>
__global__ void adamw_kernel(float4* __restrict__ p32, float4* __restrict__ m, float4* __restrict__ v,
                             const void* __restrict__ grad, uint2* __restrict__ p16, long long n4, float lr,
                             float b1, float b2, float eps, float wd, float inv_bc1, float inv_sqrt_bc2,
                             const float* __restrict__ clip) {
  const float gs = clip ? *clip : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float g[4];
    if (GBF16) {
      uint2 u = reinterpret_cast<const uint2*>(grad)[i];
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
      g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    } else {
      float4 u = reinterpret_cast<const float4*>(grad)[i];
      g[0] = u.x; g[1] = u.y; g[2] = u.z; g[3] = u.w;
    }
    float4 P = p32[i], M = m[i], V = v[i];
    float* pp = &P.x; float* mm = &M.x; float* vv = &V.x;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * gs;
      mm[e] = b1 * mm[e] + (1.f - b1) * ge;
      vv[e] = b2 * vv[e] + (1.f - b2) * ge * ge;
      const float denom = sqrtf(vv[e]) * inv_sqrt_bc2 + eps;
      pp[e] = pp[e] * (1.f - lr * wd) - lr * inv_bc1 * mm[e] / denom;
    }
    p32[i] = P; m[i] = M; v[i] = V;
    if (p16) p16[i] = make_uint2(pack_bf16(P.x, P.y), pack_bf16(P.z, P.w));
  }
}

template <bool BF16>
__global__ void sumsq_kernel(const void* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float acc = 0.f;
  if (BF16) {
    const long long nv = n / 8;
    const uint4* gv = reinterpret_cast<const uint4*>(g);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      float f[8];
      unpack8(gv[i], f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc += f[e] * f[e];
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      const __nv_bfloat16* gs = reinterpret_cast<const __nv_bfloat16*>(g);
      for (long long i = nv * 8; i < n; ++i) {
        float f = __bfloat162float(gs[i]);
        acc += f * f;
      }
    }
  } else {
    const long long nv = n / 4;
    const float4* gv = reinterpret_cast<const float4*>(g);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
      float4 f = gv[i];
      acc += f.x * f.x + f.y * f.y + f.z * f.z + f.w * f.w;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {
      const float* gs = reinterpret_cast<const float*>(g);
      for (long long i = nv * 4; i < n; ++i) acc += gs[i] * gs[i];
    }
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(out, acc);
}

__global__ void clip_coef_kernel(const float* sumsq, float max_norm, float* coef, float* norm_out) {
  const float n = sqrtf(*sumsq);
  if (norm_out) *norm_out = n;
  if (coef) *coef = (max_norm > 0.f) ? fminf(1.f, max_norm / (n + 1e-6f)) : 1.f;
}

__global__ void cast_kernel(const float4* __restrict__ src, uint2* __restrict__ dst, long long n4, float scale,
                            int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 s = src[i];
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    if (accumulate) {
      uint2 o = dst[i];
      float2 a = unpack_bf16(o.x), b = unpack_bf16(o.y);
      s.x += a.x; s.y += a.y; s.z += b.x; s.w += b.y;
    }
    dst[i] = make_uint2(pack_bf16(s.x, s.y), pack_bf16(s.z, s.w));
  }
}

inline int grid_for(long long work_items, int threads, int waves = 8) {
  long long blocks = (work_items + threads - 1) / threads;
  long long cap = (long long)sm_count() * waves;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}
inline int rc(cudaError_t e) { return e == cudaSuccess ? 0 : 1000 + (int)e; }

static void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx, float* dw_f32, int rows, int dim, cudaStream_t stream) {
  const int nvec = dim / 8;
  const int vpt = (nvec + NORM_THREADS - 1) / NORM_THREADS;
  const int per_sm = vpt <= 2 ? 4 : 2;
  const int grid = rows < sm_count() * per_sm ? rows : sm_count() * per_sm;
#define TPB_LAUNCH_NORM_BWD(V) rmsnorm_bwd_kernel<V><<<grid, NORM_THREADS, 0, stream>>>( \
      (const uint4*)dy, (const uint4*)x, (const uint4*)w, rstd, (const uint4*)dres, (uint4*)dx, dw_f32, rows, nvec)
  if (vpt <= 1) TPB_LAUNCH_NORM_BWD(1); else if (vpt == 2) TPB_LAUNCH_NORM_BWD(2); else TPB_LAUNCH_NORM_BWD(4);
#undef TPB_LAUNCH_NORM_BWD
}

}  // namespace tpb

using namespace tpb;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)

// Streamed form when the rows can be bulk-copied (16-byte aligned bases, enough rows to fill the rings) and no
// residual is added: 36 -> 30 us for 8192 x 4096.  With the residual (two reads, two writes per element, eight
// CTAs per SM) the thread-loaded kernel is already at 0.77 of copy bandwidth and the streamed one is no faster.
static bool launch_rmsnorm_fwd_bulk(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                                    int rows, int dim, float eps, cudaStream_t stream) {
  static const bool disabled = []() { const char* v = getenv("TPB_RMSNORM_FWD_BULK"); return v && v[0] == '0'; }();
  if (disabled || res) return false;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!aligned(x) || !aligned(y) || (h_out && !aligned(h_out))) return false;
  const int nvec = dim / 8;
  const int vpt = (nvec + NORM_THREADS - 1) / NORM_THREADS;
  const size_t stage_bytes = 2 * (size_t)nvec * 16;
  int stages = (int)((64 * 1024) / stage_bytes);
  if (stages > NB_MAX_STAGES) stages = NB_MAX_STAGES;
  if (stages < 2) return false;
  const size_t smem = 128 + 128 + stages * stage_bytes;
  int per_sm = (int)((220 * 1024) / (smem + 1024));
  if (per_sm > 3) per_sm = 3;
  if (per_sm < 1) return false;
  if (rows < sm_count() * per_sm * stages) return false;
  const int grid = sm_count() * per_sm;
  static bool configured[3] = {false, false, false};
#define TPB_LAUNCH_NORM_FWD_BULK(V, slot)                                                                             \
  do {                                                                                                                \
    if (!configured[slot]) {                                                                                          \
      if (cudaFuncSetAttribute(rmsnorm_fwd_bulk_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024) != \
          cudaSuccess)                                                                                                \
        return false;                                                                                                 \
      configured[slot] = true;                                                                                        \
    }                                                                                                                 \
    rmsnorm_fwd_bulk_kernel<V><<<grid, NORM_THREADS, smem, stream>>>((const uint4*)x, (const uint4*)res,             \
                                                                     (const uint4*)w, (uint4*)y, (uint4*)h_out, rstd, \
                                                                     rows, nvec, eps, stages, status_block());        \
  } while (0)
  if (vpt <= 1) TPB_LAUNCH_NORM_FWD_BULK(1, 0); else if (vpt == 2) TPB_LAUNCH_NORM_FWD_BULK(2, 1); else TPB_LAUNCH_NORM_FWD_BULK(4, 2);
#undef TPB_LAUNCH_NORM_FWD_BULK
  return true;
}

extern "C" int tpb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                               int rows, int dim, float eps, void* stream) {
  if (dim % 8 || dim > 8 * NORM_THREADS * NORM_VPT) return -2;
  if (rows <= 0) return 0;
  if (launch_rmsnorm_fwd_bulk(x, res, w, y, h_out, rstd, rows, dim, eps, STREAM(stream))) return rc(cudaGetLastError());
  const int nvec = dim / 8;
  const int vpt = (nvec + NORM_THREADS - 1) / NORM_THREADS;
  const int per_sm = vpt <= 2 ? 8 : 4;
  const int grid = rows < sm_count() * per_sm ? rows : sm_count() * per_sm;
#define TPB_LAUNCH_NORM_FWD(V) rmsnorm_fwd_kernel<V><<<grid, NORM_THREADS, 0, STREAM(stream)>>>( \
      (const uint4*)x, (const uint4*)res, (const uint4*)w, (uint4*)y, (uint4*)h_out, rstd, rows, nvec, eps)
  if (vpt <= 1) TPB_LAUNCH_NORM_FWD(1); else if (vpt == 2) TPB_LAUNCH_NORM_FWD(2); else TPB_LAUNCH_NORM_FWD(4);
#undef TPB_LAUNCH_NORM_FWD
  return rc(cudaGetLastError());
}

// Streamed form (rmsnorm_bwd_bulk_kernel) when the rows can be bulk-copied: 16-byte aligned bases (the
// row pitch is a multiple of 16 bytes already) and enough rows to fill the ring.
static bool launch_rmsnorm_bwd_bulk(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                                    void* dx, float* dw_f32, int rows, int dim, cudaStream_t stream) {
  static const bool disabled = []() { const char* v = getenv("TPB_RMSNORM_BWD_BULK"); return v && v[0] == '0'; }();
  if (disabled) return false;
  auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if (!aligned(dy) || !aligned(x) || !aligned(dx) || (dres && !aligned(dres))) return false;
  const int nvec = dim / 8;
  const int vpt = (nvec + NORM_THREADS - 1) / NORM_THREADS;
  const size_t stage_bytes = 3 * (size_t)nvec * 16;
  int stages = (int)((100 * 1024) / stage_bytes);
  if (stages > NB_MAX_STAGES) stages = NB_MAX_STAGES;
  if (stages < 2) return false;
  const size_t smem = 128 + 128 + stages * stage_bytes;
  const int per_sm = (int)((220 * 1024) / (smem + 1024)) < 2 ? 1 : 2;
  if (rows < sm_count() * per_sm * stages) return false;
  const int grid = sm_count() * per_sm;
  static bool configured[3] = {false, false, false};
#define TPB_LAUNCH_NORM_BWD_BULK(V, slot)                                                                              \
  do {                                                                                                                 \
    if (!configured[slot]) {                                                                                           \
      if (cudaFuncSetAttribute(rmsnorm_bwd_bulk_kernel<V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024) != \
          cudaSuccess)                                                                                                 \
        return false;                                                                                                  \
      configured[slot] = true;                                                                                         \
    }                                                                                                                  \
    rmsnorm_bwd_bulk_kernel<V><<<grid, NORM_THREADS, smem, stream>>>((const uint4*)dy, (const uint4*)x, (const uint4*)w, \
                                                                     rstd, (const uint4*)dres, (uint4*)dx, dw_f32,  \
                                                                     rows, nvec, stages, status_block());              \
  } while (0)
  if (vpt <= 1) TPB_LAUNCH_NORM_BWD_BULK(1, 0); else if (vpt == 2) TPB_LAUNCH_NORM_BWD_BULK(2, 1); else TPB_LAUNCH_NORM_BWD_BULK(4, 2);
#undef TPB_LAUNCH_NORM_BWD_BULK
  return true;
}

extern "C" int tpb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                               void* dx, float* dw_f32, int rows, int dim, void* stream) {
  if (dim % 8 || dim > 8 * NORM_THREADS * NORM_VPT) return -2;
  if (rows <= 0) return 0;
  if (!launch_rmsnorm_bwd_bulk(dy, x, w, rstd, dres, dx, dw_f32, rows, dim, STREAM(stream)))
    launch_rmsnorm_bwd(dy, x, w, rstd, dres, dx, dw_f32, rows, dim, STREAM(stream));
  return rc(cudaGetLastError());
}

extern "C" int tpb_rope_strided(void* x, long long ld, int col0, int heads, int dim, int head_stride,
                                const float* cos, const float* sin, const int* pos, int tokens, int seq_len,
                                int inverse, int interleaved, void* stream) {
  if (dim % 16 || ld % 8 || col0 % 8 || head_stride % 8 || head_stride < dim) return -2;
  if (tokens <= 0 || heads <= 0) return 0;
  long long total = (long long)tokens * heads * (dim / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, STREAM(stream)>>>((__nv_bfloat16*)x, ld, col0, heads, dim, head_stride,
                                                                cos, sin, pos, tokens, seq_len,
                                                                inverse ? -1.f : 1.f, interleaved);
  return rc(cudaGetLastError());
}

extern "C" int tpb_rope(void* x, long long ld, int col0, int heads, int dim, const float* cos, const float* sin,
                        const int* pos, int tokens, int seq_len, int inverse, int interleaved, void* stream) {
  return tpb_rope_strided(x, ld, col0, heads, dim, dim, cos, sin, pos, tokens, seq_len, inverse, interleaved, stream);
}

extern "C" int tpb_swiglu_fwd(const void* gu, void* act, int rows, int f, void* stream) {
  if (f % 8) return -2;
  if (rows <= 0) return 0;
  swiglu_fwd_kernel<<<grid_for((long long)rows * (f / 8), 256), 256, 0, STREAM(stream)>>>((const uint4*)gu,
                                                                                         (uint4*)act, rows, f / 8);
  return rc(cudaGetLastError());
}
extern "C" int tpb_swiglu_bwd(const void* dact, const void* gu, void* dgu, int rows, int f, void* stream) {
  if (f % 8) return -2;
  if (rows <= 0) return 0;
  swiglu_bwd_kernel<<<grid_for((long long)rows * (f / 8), 256), 256, 0, STREAM(stream)>>>(
      (const uint4*)dact, (const uint4*)gu, (uint4*)dgu, rows, f / 8);
  return rc(cudaGetLastError());
}

extern "C" int tpb_ce_fwd_bwd(void* logits, long long ld, const long long* targets, float* loss_sum,
                              const float* grad_scale, int rows, int vocab, void* stream) {
  if (vocab % 8 || ld % 8) return -2;
  if (rows <= 0) return 0;
  int grid = rows < sm_count() * 4 ? rows : sm_count() * 4;
  ce_kernel<<<grid, CE_THREADS, 0, STREAM(stream)>>>((__nv_bfloat16*)logits, ld, targets, loss_sum, grad_scale, rows,
                                                     vocab);
  return rc(cudaGetLastError());
}

extern "C" int tpb_adamw(float* p32, float* m, float* v, const void* grad, void* p16, long long n, float lr,
                         float beta1, float beta2, float eps, float wd, float bc1, float bc2, const float* clip_coef,
                         int grad_is_bf16, void* stream) {
  if (n % 4) return -2;
  if (n <= 0) return 0;
  const int grid = grid_for(n / 4, 256, 16);
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = 1.f / sqrtf(bc2);
  if (grad_is_bf16)
    adamw_kernel<true><<<grid, 256, 0, STREAM(stream)>>>((float4*)p32, (float4*)m, (float4*)v, grad, (uint2*)p16,
                                                         n / 4, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2,
                                                         clip_coef);
  else
    adamw_kernel<false><<<grid, 256, 0, STREAM(stream)>>>((float4*)p32, (float4*)m, (float4*)v, grad, (uint2*)p16,
                                                          n / 4, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2,
                                                          clip_coef);
  return rc(cudaGetLastError());
}

extern "C" int tpb_sumsq(const void* g, long long n, int is_bf16, float* out, void* stream) {
  if (n <= 0) return 0;
  const int grid = grid_for(n / 8 + 1, 512, 4);
  if (is_bf16) sumsq_kernel<true><<<grid, 512, 0, STREAM(stream)>>>(g, n, out);
  else sumsq_kernel<false><<<grid, 512, 0, STREAM(stream)>>>(g, n, out);
  return rc(cudaGetLastError());
}

extern "C" int tpb_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, STREAM(stream)>>>(sumsq, max_norm, coef, norm_out);
  return rc(cudaGetLastError());
}

extern "C" int tpb_embedding_fwd(const void* table, const long long* ids, void* out, int tokens, int dim,
                                 long long vocab, long long row0, void* stream) {
  if (dim % 8) return -2;
  if (tokens <= 0) return 0;
  embedding_fwd_kernel<<<grid_for((long long)tokens * (dim / 8), 256), 256, 0, STREAM(stream)>>>(
      (const uint4*)table, ids, (uint4*)out, tokens, dim / 8, vocab, row0);
  return rc(cudaGetLastError());
}
extern "C" int tpb_embedding_bwd(const void* dout, const long long* ids, void* dtable, int tokens, int dim,
                                 long long rows_local, long long row0, int dtable_is_f32, void* stream) {
  if (dim % 2) return -2;
  if (tokens <= 0) return 0;
  const int grid = grid_for((long long)tokens * (dim / 2), 256);
  if (dtable_is_f32)
    embedding_bwd_kernel<true><<<grid, 256, 0, STREAM(stream)>>>((const __nv_bfloat162*)dout, ids, dtable, tokens,
                                                                 dim / 2, rows_local, row0);
  else
    embedding_bwd_kernel<false><<<grid, 256, 0, STREAM(stream)>>>((const __nv_bfloat162*)dout, ids, dtable, tokens,
                                                                  dim / 2, rows_local, row0);
  return rc(cudaGetLastError());
}

extern "C" int tpb_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, int accumulate,
                                    void* stream) {
  if (n % 4) return -2;
  if (n <= 0) return 0;
  cast_kernel<<<grid_for(n / 4, 256), 256, 0, STREAM(stream)>>>((const float4*)src, (uint2*)dst, n / 4, scale,
                                                                accumulate);
  return rc(cudaGetLastError());
}

// ----------------------------------------------------------------------------
// Allocation-free variant of the RMSNorm backward (see tpb_noalloc.h).
// ----------------------------------------------------------------------------
#include "tpb_noalloc.h"

namespace tpb {
// fp32 weight-gradient accumulator shared by every call on this device.  In host code this
// name is only a handle; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_dw_scratch[TPB_NOALLOC_MAX_DIM];

constexpr int kMaxDevices = 64;
static float* g_noalloc_dw_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array for the current device (looked up once per device).
static float* noalloc_scratch_for_current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (g_noalloc_dw_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_dw_scratch) != cudaSuccess) return nullptr;
    g_noalloc_dw_ptr[dev] = ptr;
  }
  return g_noalloc_dw_ptr[dev];
}

__global__ void noalloc_store_dw_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ out, int dim) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x)
    out[i] = __float2bfloat16(acc[i]);
}
}  // namespace tpb

extern "C" int tpb_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                       const void* dres, void* dx, void* dw_bf16, int rows, int dim, void* stream) {
  if (dim <= 0 || dim % 8) return -2;
  if (dim > TPB_NOALLOC_MAX_DIM) return -6;
  float* scratch = noalloc_scratch_for_current_device();
  if (!scratch) return -7;
  cudaStream_t s = STREAM(stream);
  // the accumulator keeps the previous call's sums: clear what this call will add into
  cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(float) * dim, s);
  if (e != cudaSuccess) return 1000 + (int)e;
  if (rows > 0) {
    launch_rmsnorm_bwd(dy, x, w, rstd, dres, dx, scratch, rows, dim, s);
    e = cudaGetLastError();
    if (e != cudaSuccess) return 1000 + (int)e;
  }
  noalloc_store_dw_kernel<<<(dim + 255) / 256, 256, 0, s>>>(scratch, (__nv_bfloat16*)dw_bf16, dim);
  return rc(cudaGetLastError());
}

extern "C" const char* tpb_noalloc_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case -2: return "dim must be a positive multiple of 8";
    case -6: return "dim exceeds TPB_NOALLOC_MAX_DIM (8192): the built-in scratch accumulator is too small";
    case -7: return "could not resolve the device address of the built-in scratch (cudaGetSymbolAddress failed)";
    default: return code >= 1000 ? "CUDA launch failed (code - 1000 is the cudaError_t)" : "unknown error";
  }
}
