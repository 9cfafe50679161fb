// Mixture-of-experts support kernels: fused router top-k (softmax / sigmoid with
// group-limited selection), row gather into the expert-grouped layout, weighted combine
// back to token order and the routing-weight gradient.  The grouped GEMMs themselves are
// the grouped modes of gemm_sm100.cu.

#include "common.cuh"
#include "tpb.h"

namespace tpb {

int sm_count();

constexpr int ROUTER_MAX_PER_LANE = 8;  // experts per lane -> up to 256 experts

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax warp_argmax(float v, int i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
  return {v, i};
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per token.  Expert e lives in register e / 32 of lane e % 32.
//   mode 0: p = softmax(logits); top-k of p; weights renormalised to sum 1 (if norm_topk).
//   mode 1: s = sigmoid(logits); selection score = s + bias, restricted to the topk_group
//           groups with the largest (sum of top-2 selection scores); weights = s at the
//           selected experts, normalised (if norm_topk) and multiplied by `scale`.
template <typename T>
__global__ void router_topk_kernel(const T* __restrict__ logits, const float* __restrict__ bias,
                                   float* __restrict__ w_out, int* __restrict__ idx_out,
                                   float* __restrict__ scores_out, int tokens, int E, int K, int mode, int n_group,
                                   int topk_group, int norm_topk, float scale) {
  const int lane = threadIdx.x & 31;
  const int per_lane = (E + 31) / 32;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < tokens; t += (gridDim.x * blockDim.x) >> 5) {
    float s[ROUTER_MAX_PER_LANE], sel[ROUTER_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
      const int e = j * 32 + lane;
      float x = -INFINITY;
      if (j < per_lane && e < E) x = (float)logits[(long long)t * E + e];
      s[j] = x;
      mx = fmaxf(mx, x);
    }
    if (mode == 0) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        s[j] = (s[j] == -INFINITY) ? 0.f : __expf(s[j] - mx);
        sum += s[j];
      }
      sum = warp_sum_f(sum);
      const float inv = 1.f / sum;
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        s[j] *= inv;
        const int e = j * 32 + lane;
        sel[j] = (j < per_lane && e < E) ? s[j] : -INFINITY;
      }
    } else {
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        const int e = j * 32 + lane;
        const bool ok = j < per_lane && e < E;
        s[j] = ok ? 1.f / (1.f + __expf(-s[j])) : 0.f;
        sel[j] = ok ? s[j] + (bias ? bias[e] : 0.f) : -INFINITY;
      }
      if (n_group > 1) {
        const int gs = E / n_group;
        float gscore = -INFINITY;  // lane g keeps the score of group g
        for (int g = 0; g < n_group; ++g) {
          float best = -INFINITY;
          int besti = 0x7fffffff;
#pragma unroll
          for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
            const int e = j * 32 + lane;
            if (j < per_lane && e < E && e / gs == g && sel[j] > best) { best = sel[j]; besti = e; }
          }
          const ArgMax a1 = warp_argmax(best, besti);
          float second = -INFINITY;
          int secondi = 0x7fffffff;
#pragma unroll
          for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
            const int e = j * 32 + lane;
            if (j < per_lane && e < E && e / gs == g && e != a1.i && sel[j] > second) { second = sel[j]; secondi = e; }
          }
          const ArgMax a2 = warp_argmax(second, secondi);
          const float sc = a1.v + (gs > 1 ? a2.v : 0.f);
          if (lane == g) gscore = sc;
        }
        unsigned keep_groups = 0;
        for (int r = 0; r < topk_group; ++r) {
          const ArgMax a = warp_argmax(gscore, lane);
          keep_groups |= 1u << a.i;
          if (lane == a.i) gscore = -INFINITY;
        }
#pragma unroll
        for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
          const int e = j * 32 + lane;
          if (j < per_lane && e < E && !((keep_groups >> (e / gs)) & 1u)) sel[j] = 0.f;
        }
      }
    }
    if (scores_out) {
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        const int e = j * 32 + lane;
        if (j < per_lane && e < E) scores_out[(long long)t * E + e] = s[j];
      }
    }
    // top-k by repeated warp arg-max (ties go to the lower expert index)
    float wsum = 0.f;
    float my_w = 0.f;   // lane r keeps the r-th weight
    int my_i = 0;
    for (int r = 0; r < K; ++r) {
      float best = -INFINITY;
      int besti = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        const int e = j * 32 + lane;
        if (j < per_lane && e < E && (sel[j] > best || (sel[j] == best && e < besti))) { best = sel[j]; besti = e; }
      }
      const ArgMax a = warp_argmax(best, besti);
      float val = 0.f;
#pragma unroll
      for (int j = 0; j < ROUTER_MAX_PER_LANE; ++j) {
        const int e = j * 32 + lane;
        if (e == a.i) { val = s[j]; sel[j] = -INFINITY; }
      }
      val = warp_sum_f(val);   // only the owning lane contributed
      wsum += val;
      if (lane == r) { my_w = val; my_i = a.i; }
    }
    float norm = 1.f;
    if (norm_topk) norm = (mode == 0) ? 1.f / wsum : 1.f / (wsum + 1e-20f);
    if (lane < K) {
      w_out[(long long)t * K + lane] = my_w * norm * scale;
      idx_out[(long long)t * K + lane] = my_i;
    }
  }
}

// out[r, :] = (src_row[r] >= 0) ? scale[r] * x[src_row[r], :] : 0       (rows of 16-byte vectors)
__global__ void moe_gather_kernel(const uint4* __restrict__ x, const int* __restrict__ src_row,
                                  const float* __restrict__ row_scale, uint4* __restrict__ out, long long rows,
                                  int nvec) {
  const long long total = rows * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / nvec;
    const int c = (int)(i % nvec);
    const int src = src_row[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (src >= 0) {
      v = x[(long long)src * nvec + c];
      if (row_scale) {
        const float sc = row_scale[r];
        float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), d = unpack_bf16(v.w);
        v = make_uint4(pack_bf16(a.x * sc, a.y * sc), pack_bf16(b.x * sc, b.y * sc), pack_bf16(cc.x * sc, cc.y * sc),
                       pack_bf16(d.x * sc, d.y * sc));
      }
    }
    out[i] = v;
  }
}

// out[t, :] = sum_k w[t,k] * rows[dest[t,k], :]   (dest < 0: dropped pair; w null: weight 1)
__global__ void moe_combine_kernel(const uint4* __restrict__ rows, const int* __restrict__ dest,
                                   const float* __restrict__ w, uint4* __restrict__ out, long long tokens, int K,
                                   int nvec) {
  const long long total = tokens * nvec;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nvec;
    const int c = (int)(i % nvec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; ++k) {
      const int r = dest[t * K + k];
      if (r < 0) continue;
      const float wk = w ? w[t * K + k] : 1.f;
      const uint4 v = rows[(long long)r * nvec + c];
      float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), d = unpack_bf16(v.w);
      acc[0] += wk * a.x; acc[1] += wk * a.y; acc[2] += wk * b.x; acc[3] += wk * b.y;
      acc[4] += wk * cc.x; acc[5] += wk * cc.y; acc[6] += wk * d.x; acc[7] += wk * d.y;
    }
    out[i] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                        pack_bf16(acc[6], acc[7]));
  }
}

// dw[t,k] = <rows[dest[t,k], :], dout[t, :]>     (one warp per (t,k) pair)
__global__ void moe_combine_dw_kernel(const uint4* __restrict__ rows, const int* __restrict__ dest,
                                      const uint4* __restrict__ dout, float* __restrict__ dw, long long pairs, int K,
                                      int nvec) {
  const int lane = threadIdx.x & 31;
  for (long long pr = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; pr < pairs;
       pr += ((long long)gridDim.x * blockDim.x) >> 5) {
    const int r = dest[pr];
    float acc = 0.f;
    if (r >= 0) {
      const long long t = pr / K;
      for (int c = lane; c < nvec; c += 32) {
        const uint4 a = rows[(long long)r * nvec + c], b = dout[t * nvec + c];
        float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
        float2 b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y), b2 = unpack_bf16(b.z), b3 = unpack_bf16(b.w);
        acc += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x +
               a3.y * b3.y;
      }
    }
    acc = warp_sum_f(acc);
    if (lane == 0) dw[pr] = acc;
  }
}

static inline int grid_for_items(long long items, int threads, int waves = 8) {
  long long blocks = (items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * waves;
  if (blocks > cap) blocks = cap;
  return blocks < 1 ? 1 : (int)blocks;
}


// ----------------------------------------------------------------------------
// Variable-size all-to-all of rows over NVLink, done by this GPU's own stores (expert-parallel
// dispatch and return).  Rows [src_start[r], src_start[r+1]) of `src` go to rank r's receive buffer,
// starting at row dst_row0[r] there; plain 16-byte stores to peer memory (posted writes).  When the
// last CTA has finished, the flag "rank `me` has delivered" is raised in every rank's flag array.
// ----------------------------------------------------------------------------
struct A2APushParams {
  const uint4* src;
  int vec_per_row;
  int n_rows;
  int world, me;
  int src_start[9];
  long long dst_row0[8];
  uint4* dst[8];
  unsigned* flags[8];
  unsigned epoch;
  unsigned* done_counter;   // one zero-initialised word of local memory
};

__global__ void a2a_push_kernel(const A2APushParams p) {
  for (int row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
    int r = 0;
    while (r + 1 < p.world && row >= p.src_start[r + 1]) ++r;
    const uint4* s = p.src + (long long)row * p.vec_per_row;
    uint4* d = p.dst[r] + (p.dst_row0[r] + (row - p.src_start[r])) * p.vec_per_row;
    for (int i = threadIdx.x; i < p.vec_per_row; i += blockDim.x) d[i] = s[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {          // every CTA's stores are fenced: publish
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[r] + p.me), "r"(p.epoch) : "memory");
      *p.done_counter = 0;
    }
  }
}

// ----------------------------------------------------------------------------
// Dispatch plan: a stable counting sort of the (token, slot) pairs by expert into 128-row padded
// segments, in one CTA.  Every warp owns a contiguous range of pairs; sweep 1 counts per (warp,
// expert), a prefix over warps gives each warp its first row in every expert's segment, sweep 2
// walks the range again and hands out rows in order (match_any groups equal experts inside a
// warp, the lane order breaks ties), so the result does not depend on scheduling.
// Outputs: counts[E], k_offsets[E+1] (multiples of 128), dest[n] (row of each pair), src_row[M]
// (token feeding a row) and src_pair[M] (pair feeding a row), both pre-filled with -1 by the
// host, tile_expert[M/128] (pre-filled with -1).
// ----------------------------------------------------------------------------
constexpr int PLAN_THREADS = 1024;
constexpr int PLAN_MAX_E = 256;

__global__ void __launch_bounds__(PLAN_THREADS, 1)
moe_plan_kernel(const int* __restrict__ idx, int n, int K, int E, int align, int* __restrict__ counts,
                int* __restrict__ k_offsets, int* __restrict__ dest, int* __restrict__ src_row,
                long long* __restrict__ src_pair, int* __restrict__ tile_expert) {
  __shared__ int wcount[32][PLAN_MAX_E];     // sweep 1: pairs of (warp, expert); sweep 2: next row
  __shared__ int off_pad[PLAN_MAX_E + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * PLAN_MAX_E; i += PLAN_THREADS) (&wcount[0][0])[i] = 0;
  __syncthreads();
  const int per_warp = ((n + 31) / 32 + 31) / 32 * 32;      // multiple of 32 so that lanes stay aligned
  const int lo = warp * per_warp, hi = min(n, lo + per_warp);
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const int e = i < hi ? idx[i] : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned m = __match_any_sync(0xffffffffu, ok ? e : -1);
    if (ok && (m & ((1u << lane) - 1)) == 0) wcount[warp][e] += __popc(m);
    __syncwarp();
  }
  __syncthreads();
  if (threadIdx.x < E) {
    int total = 0;
    for (int w = 0; w < 32; ++w) total += wcount[w][threadIdx.x];
    counts[threadIdx.x] = total;
    off_pad[threadIdx.x + 1] = (total + align - 1) / align * align;
  }
  if (threadIdx.x == 0) off_pad[0] = 0;
  __syncthreads();
  if (threadIdx.x == 0)
    for (int e = 0; e < E; ++e) off_pad[e + 1] += off_pad[e];
  __syncthreads();
  if (threadIdx.x <= E) k_offsets[threadIdx.x] = off_pad[threadIdx.x];
  if (threadIdx.x < E) {
    int run = off_pad[threadIdx.x];
    for (int w = 0; w < 32; ++w) {
      const int c = wcount[w][threadIdx.x];
      wcount[w][threadIdx.x] = run;
      run += c;
    }
    for (int t = off_pad[threadIdx.x] / 128; t < off_pad[threadIdx.x + 1] / 128; ++t) tile_expert[t] = threadIdx.x;
  }
  __syncthreads();
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const int e = i < hi ? idx[i] : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned m = __match_any_sync(0xffffffffu, ok ? e : -1);
    int pos = -1;
    if (ok) pos = wcount[warp][e] + __popc(m & ((1u << lane) - 1));
    __syncwarp();
    if (ok && (m & ((1u << lane) - 1)) == 0) wcount[warp][e] += __popc(m);
    __syncwarp();
    if (i < hi) dest[i] = pos;
    if (ok) {
      src_row[pos] = i / K;
      src_pair[pos] = i;
    }
  }
}

// Block form of the push: the source rows are a sequence of `n_blocks` contiguous blocks, block b =
// rows [start[b], start[b+1]) going to rank dst_rank[b] at row dst_row0[b] of its receive buffer.
// The descriptors live in device memory as 64-bit words: start[n_blocks + 1], dst_rank[n_blocks],
// dst_row0[n_blocks].  One block per (destination rank, expert) lets rows land at the receiver
// already grouped by expert, whatever rank they came from.
struct A2ABlocksParams {
  const uint4* src;
  int vec_per_row;
  int n_rows;
  int n_blocks;
  int world, me;
  const long long* desc;
  uint4* dst[8];
  unsigned* flags[8];
  unsigned epoch;
  unsigned* done_counter;
};

__global__ void a2a_push_blocks_kernel(const A2ABlocksParams p) {
  extern __shared__ long long a2a_desc[];
  const int nd = 3 * p.n_blocks + 1;
  for (int i = threadIdx.x; i < nd; i += blockDim.x) a2a_desc[i] = p.desc[i];
  __syncthreads();
  const long long* start = a2a_desc;
  const long long* dst_rank = a2a_desc + p.n_blocks + 1;
  const long long* dst_row0 = dst_rank + p.n_blocks;
  for (int row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
    int lo = 0, hi = p.n_blocks - 1;                    // last block whose first row is <= row
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (start[mid] <= row) lo = mid; else hi = mid - 1;
    }
    const int r = (int)dst_rank[lo];
    if (r < 0 || r >= p.world) continue;
    const uint4* s = p.src + (long long)row * p.vec_per_row;
    uint4* d = p.dst[r] + (dst_row0[lo] + (row - start[lo])) * p.vec_per_row;
    for (int i = threadIdx.x; i < p.vec_per_row; i += blockDim.x) d[i] = s[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flags[r] + p.me), "r"(p.epoch) : "memory");
      *p.done_counter = 0;
    }
  }
}

// Stream-ordered wait (bounded) until every rank has delivered its rows for `epoch`.
__global__ void a2a_wait_kernel(const unsigned* flags, int world, unsigned epoch, int* status) {
  if (threadIdx.x != 0) return;
  for (int r = 0; r < world; ++r) {
    long long t0 = 0;
    int spins = 0;
    while (true) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + r) : "memory");
      if (v == epoch) break;
      if (++spins == 64) {
        spins = 0;
        if (t0 == 0) t0 = clock64();
        else if (clock64() - t0 > kSpinBudgetCycles) { report(status, kTimeoutPeerFlag, 61); return; }
        __nanosleep(200);
      }
    }
  }
}

}  // namespace tpb

using namespace tpb;
#define STREAM(s) reinterpret_cast<cudaStream_t>(s)
static inline int rc_of(cudaError_t e) { return e == cudaSuccess ? 0 : 1000 + (int)e; }

extern "C" int tpb_router_topk(const void* logits, int logits_is_bf16, const float* bias, float* w_out, int* idx_out,
                               float* scores_out, int tokens, int E, int K, int mode, int n_group, int topk_group,
                               int norm_topk, float scale, void* stream) {
  if (E > 32 * ROUTER_MAX_PER_LANE || K > 32 || K > E || E <= 0) return -2;
  if (mode == 1 && n_group > 1 && (E % n_group || n_group > 32 || topk_group > n_group)) return -2;
  if (tokens <= 0) return 0;
  const int grid = grid_for_items((long long)tokens * 32, 256);
  if (logits_is_bf16)
    router_topk_kernel<__nv_bfloat16><<<grid, 256, 0, STREAM(stream)>>>(
        (const __nv_bfloat16*)logits, bias, w_out, idx_out, scores_out, tokens, E, K, mode, n_group, topk_group,
        norm_topk, scale);
  else
    router_topk_kernel<float><<<grid, 256, 0, STREAM(stream)>>>((const float*)logits, bias, w_out, idx_out, scores_out,
                                                                tokens, E, K, mode, n_group, topk_group, norm_topk,
                                                                scale);
  return rc_of(cudaGetLastError());
}

extern "C" int tpb_moe_gather(const void* x, const int* src_row, const float* row_scale, void* out, long long rows,
                              int dim, void* stream) {
  if (dim % 8) return -2;
  if (rows <= 0) return 0;
  moe_gather_kernel<<<grid_for_items(rows * (dim / 8), 256), 256, 0, STREAM(stream)>>>(
      (const uint4*)x, src_row, row_scale, (uint4*)out, rows, dim / 8);
  return rc_of(cudaGetLastError());
}

extern "C" int tpb_moe_combine(const void* rows, const int* dest, const float* w, void* out, long long tokens, int K,
                               int dim, void* stream) {
  if (dim % 8) return -2;
  if (tokens <= 0) return 0;
  moe_combine_kernel<<<grid_for_items(tokens * (dim / 8), 256), 256, 0, STREAM(stream)>>>(
      (const uint4*)rows, dest, w, (uint4*)out, tokens, K, dim / 8);
  return rc_of(cudaGetLastError());
}

extern "C" int tpb_moe_combine_dw(const void* rows, const int* dest, const void* dout, float* dw, long long tokens,
                                  int K, int dim, void* stream) {
  if (dim % 8) return -2;
  if (tokens <= 0) return 0;
  moe_combine_dw_kernel<<<grid_for_items(tokens * K * 32, 256), 256, 0, STREAM(stream)>>>(
      (const uint4*)rows, dest, (const uint4*)dout, dw, tokens * K, K, dim / 8);
  return rc_of(cudaGetLastError());
}

// src: [n_rows, dim] bf16 rows sorted by destination rank; src_start[world + 1] row offsets of the
// blocks; dst_row0[r]: first row of this rank's block in rank r's receive buffer dst[r]; flags[r]:
// rank r's flag array (one word per source rank); done_counter: a zero-initialised local word.
extern "C" int tpb_a2a_push_rows(const void* src, int n_rows, int dim, int world, int me, const int* src_start,
                                 const long long* dst_row0, void* const* dst, unsigned* const* flags, unsigned epoch,
                                 unsigned* done_counter, void* stream) {
  if (dim % 8 || world < 1 || world > 8 || me < 0 || me >= world) return -2;
  A2APushParams p{};
  p.src = (const uint4*)src; p.vec_per_row = dim / 8; p.n_rows = n_rows; p.world = world; p.me = me;
  for (int r = 0; r <= world; ++r) p.src_start[r] = src_start[r];
  for (int r = 0; r < world; ++r) {
    p.dst_row0[r] = dst_row0[r];
    p.dst[r] = (uint4*)dst[r];
    p.flags[r] = flags[r];
  }
  p.epoch = epoch; p.done_counter = done_counter;
  int grid = n_rows < 1 ? 1 : (n_rows < 4 * sm_count() ? n_rows : 4 * sm_count());
  a2a_push_kernel<<<grid, 256, 0, STREAM(stream)>>>(p);
  return rc_of(cudaGetLastError());
}

// idx [tokens, K] int32 (entries outside [0, E) are dropped: dest = -1).  align: 128 or 256 rows per
// segment step.  rows = static row count of the padded layout (>= round_up(tokens * K, align) + align * E).  Everything is on the device; no host read.
extern "C" int tpb_moe_plan(const int* idx, int tokens, int K, int E, int rows, int align, int* counts, int* k_offsets,
                            int* dest, int* src_row, long long* src_pair, int* tile_expert, void* stream) {
  if (E < 1 || E > PLAN_MAX_E || K < 1 || tokens < 0 || (align != 128 && align != 256) || rows % align) return -2;
  const long long n = (long long)tokens * K;
  if (n > (1LL << 30) || rows < (n + align - 1) / align * align + (long long)align * E) return -2;
  cudaError_t e = cudaMemsetAsync(src_row, 0xFF, sizeof(int) * rows, STREAM(stream));
  if (e == cudaSuccess) e = cudaMemsetAsync(src_pair, 0xFF, sizeof(long long) * rows, STREAM(stream));
  if (e == cudaSuccess) e = cudaMemsetAsync(tile_expert, 0xFF, sizeof(int) * (rows / 128), STREAM(stream));
  if (e != cudaSuccess) return rc_of(e);
  moe_plan_kernel<<<1, PLAN_THREADS, 0, STREAM(stream)>>>(idx, (int)n, K, E, align, counts, k_offsets, dest, src_row, src_pair,
                                                          tile_expert);
  return rc_of(cudaGetLastError());
}

extern "C" int tpb_a2a_push_blocks(const void* src, int n_rows, int dim, int n_blocks, int world, int me,
                                   const long long* desc_dev, void* const* dst, unsigned* const* flags,
                                   unsigned epoch, unsigned* done_counter, void* stream) {
  if (dim % 8 || world < 1 || world > 8 || me < 0 || me >= world || n_blocks < 1 || n_blocks > 1024 || !desc_dev)
    return -2;
  A2ABlocksParams p{};
  p.src = (const uint4*)src; p.vec_per_row = dim / 8; p.n_rows = n_rows; p.n_blocks = n_blocks;
  p.world = world; p.me = me; p.desc = desc_dev;
  for (int r = 0; r < world; ++r) {
    p.dst[r] = (uint4*)dst[r];
    p.flags[r] = flags[r];
  }
  p.epoch = epoch; p.done_counter = done_counter;
  int grid = n_rows < 1 ? 1 : (n_rows < 4 * sm_count() ? n_rows : 4 * sm_count());
  a2a_push_blocks_kernel<<<grid, 256, (3 * n_blocks + 1) * sizeof(long long), STREAM(stream)>>>(p);
  return rc_of(cudaGetLastError());
}

extern "C" int tpb_a2a_wait(const unsigned* flags, int world, unsigned epoch, void* stream) {
  a2a_wait_kernel<<<1, 32, 0, STREAM(stream)>>>(flags, world, epoch, status_block());
  return rc_of(cudaGetLastError());
}
