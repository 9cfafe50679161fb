// bf16 GEMM for sm_100a: C[M,N] = alpha * A[M,K] * B[N,K]^T with fp32 accumulation.
//
// Structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: fills a 4-stage ring of {A 128x64, B 256x64} bf16
//               tiles in 128B-swizzled shared memory (non-multicast loads only).
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16 into one of
//               two 256-column TMEM accumulators and commits to mbarriers.
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (each warp owns a
//               32-lane quarter) and apply the fused epilogue while the next tile's
//               main loop already runs on the other accumulator.
//
// Either operand may be stored K-major ([rows][K]) or MN-major ([K][rows]); the
// three GEMMs of a linear layer map onto it without a transpose:
//   forward  Y = X W^T      A = X  (K-major)   B = W  (K-major)
//   dgrad    dX = dY W      A = dY (K-major)   B = W  (MN-major, contraction over W's rows)
//   wgrad    dW = dY^T X    A = dY (MN-major)  B = X  (MN-major), fp32 accumulate epilogue
//
// Every wait is bounded (common.cuh); on timeout the roles fall through to the
// common exit, TMEM is released and the status block tells the host what happened.

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tpb.h"

namespace tpb {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;                 // 16 KB
constexpr int B_BYTES = BN * BK * 2;                 // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;       // 48 KB
constexpr int EPI_SLAB_BYTES = 4 * 4096;              // one 32-row x 128-byte transpose slab per epilogue warp
constexpr int GEMM_SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + EPI_SLAB_BYTES;
static_assert(6 * 32768 + 64 <= STAGES * STAGE_BYTES + 256, "copier ring must fit the GEMM shared memory");
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  void* C;
  long long ldc;
  const void* aux;   // residual (EPI_BF16_RES)
  long long ldaux;
  void* c2;          // pre-activation output (EPI_SWIGLU, optional)
  long long ldc2;
  int b_split;       // EPI_SWIGLU: column of c2 where the "up" half starts (= F)
  int b2_off;        // EPI_SWIGLU: row/column offset of the "up" half inside the second B map
  float alpha;
  int epi;
  int group_m;       // rasterisation: m-tiles per group
  int* status;
  // Grouped (mixture-of-experts) modes.  0: dense.
  // 1: rows of A/C are grouped by expert in 128-row aligned segments; tile_expert[m_tile] is the
  //    expert whose weights (3rd coordinate of the B maps) that tile uses, -1 = tile unused.
  // 2: per-expert wgrad: E independent [M,N] outputs, expert e contracts over rows
  //    [k_offsets[e], k_offsets[e+1]) (multiples of 64) of A and B; C of expert e is at
  //    C + e * c_stride elements.
  int mode;
  int num_experts;
  const int* tile_expert;
  const int* k_offsets;
  long long c_stride;
  // All-gather fusion: the flat buffer that contains B is sharded over ag_world GPUs.  The
  // first ag_copiers CTAs pull every shard (peer memory, plain bulk copies) into the local
  // gathered buffer chunk by chunk and publish one flag per chunk; the TMA producer of a GEMM
  // CTA waits (bounded) for the chunks that hold its B tile before loading it locally.
  int ag_copiers;
  int ag_world;
  const void* ag_src[8];        // shard base of every rank (symmetric memory), bf16
  void* ag_dst;                 // local gathered buffer (ag_world * ag_shard_elems)
  long long ag_shard_elems;
  long long ag_chunk_elems;
  long long ag_b_offset;        // element offset of B inside the gathered buffer
  unsigned* ag_flags;           // [ag_world * chunks_per_shard], value = epoch when ready
  unsigned ag_epoch;
  int ag_local;                 // rank whose shard already sits in ag_dst (not copied, not waited for); -1: none
  // Push mode (ag_push != 0): the copier CTAs of rank ag_local read ITS OWN shard and store it into
  // every peer's gathered buffer with plain 16-byte stores (posted writes: nothing waits for a round
  // trip until the fence before a chunk's flags), then raise the flag in the peer's flag array; each
  // rank waits on flags in its own memory.  Measured on 2 GPUs: 11-12 GB/s per copier CTA, against
  // 7-8 GB/s for pulling (an SM keeps few peer reads in flight).
  int ag_push;
  void* ag_push_dst[8];         // gathered buffer of every rank (symmetric memory)
  unsigned* ag_push_flags[8];   // flag array of every rank (symmetric memory)
  void* ag_push_mc;             // NVSwitch multicast address of the gathered buffers (one store reaches every rank), or null
  // Reduce-scatter fusion (TPB_EPI_RS_BF16): the epilogue adds alpha * acc straight into the
  // owner's bf16 gradient shard over P2P with vector red.add.
  int rs_world;
  int tile_rot;                 // tiles are visited starting from this one (rotation by rank, see tpb_gemm_rs_bf16)
  int te_stride;                // tile_expert entries per m-tile (2 for CTA-pair tiles of 256 rows)
  void* rs_dst[8];              // gradient shard base of every rank (symmetric memory), bf16
  long long rs_shard_elems;
  long long rs_c_offset;        // element offset of C inside the sharded flat buffer
  int rs_store;                 // 1: plain 16-byte stores instead of red.add (each source writes its own staging
                                // slot at the owner, which adds the slots in rank order afterwards)
};

struct TileInfo {
  int tm, tn, e, kb0, kb1;
  bool skip;
};

__device__ __forceinline__ void tile_coords(int t, int m_tiles, int n_tiles, int group_m, int& tm,
                                            int& tn) {
  int per_group = group_m * n_tiles;
  int g = t / per_group;
  int first_m = g * group_m;
  int gsize = min(group_m, m_tiles - first_m);
  int within = t - g * per_group;
  tm = first_m + within % gsize;
  tn = within / gsize;
}

__device__ __forceinline__ TileInfo tile_info(const GemmParams& p, int t, int m_tiles, int n_tiles, int num_kb) {
  TileInfo ti;
  if (p.tile_rot) {
    const int total = m_tiles * n_tiles * (p.mode == 2 ? p.num_experts : 1);
    t += p.tile_rot;
    if (t >= total) t -= total;
  }
  ti.e = 0; ti.kb0 = 0; ti.kb1 = num_kb; ti.skip = false;
  if (p.mode == 2) {
    const int per = m_tiles * n_tiles;
    ti.e = t / per;
    tile_coords(t - ti.e * per, m_tiles, n_tiles, p.group_m, ti.tm, ti.tn);
    ti.kb0 = p.k_offsets[ti.e] / BK;
    ti.kb1 = p.k_offsets[ti.e + 1] / BK;
  } else {
    tile_coords(t, m_tiles, n_tiles, p.group_m, ti.tm, ti.tn);
    if (p.mode == 1) {
      ti.e = p.tile_expert[ti.tm * p.te_stride];   // entries are per 128 rows; a pair tile covers two
      ti.skip = ti.e < 0;
    }
  }
  return ti;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ long long ag_chunks_per_shard(const GemmParams& p) {
  return (p.ag_shard_elems + p.ag_chunk_elems - 1) / p.ag_chunk_elems;
}

// Wait until every chunk that overlaps flat elements [lo, hi] has been published.
__device__ __forceinline__ bool ag_wait_range(const GemmParams& p, long long lo, long long hi) {
  const long long cps = ag_chunks_per_shard(p);
  const long long total = p.ag_shard_elems * p.ag_world;
  if (hi >= total) hi = total - 1;
  long long e = lo;
  while (e <= hi) {
    const long long owner = e / p.ag_shard_elems;
    if (owner == p.ag_local) {
      e = (owner + 1) * p.ag_shard_elems;
      continue;
    }
    const long long j = (e - owner * p.ag_shard_elems) / p.ag_chunk_elems;
    const unsigned* f = p.ag_flags + owner * cps + j;
    unsigned v;
    long long t0 = 0;
    int spins = 0;
    while (true) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if ((int)(v - p.ag_epoch) >= 0) break;   // epochs only grow
      if (++spins == 64) {
        spins = 0;
        if (t0 == 0) t0 = clock64();
        else if (clock64() - t0 > kSpinBudgetCycles) { report(p.status, kTimeoutPeerFlag, 5); return false; }
        __nanosleep(100);
      }
    }
    const long long chunk_end = owner * p.ag_shard_elems + min(p.ag_shard_elems, (j + 1) * p.ag_chunk_elems);
    e = chunk_end;
  }
  asm volatile("fence.proxy.async;" ::: "memory");   // the data was written through the async proxy
  return true;
}

// Copier CTA: one thread drives a ring of bulk copies  peer shard -> shared memory -> local
// gathered buffer and publishes a flag per chunk.  Loads are plain (non-multicast) bulk copies.
__device__ void ag_copier(const GemmParams& p, uint8_t* smem) {
  constexpr int SLOTS = 6;
  const long long chunk_bytes_max = p.ag_chunk_elems * 2;   // <= 32 KB (host checks)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SLOTS * 32768);
  if (threadIdx.x != 0) return;
  for (int i = 0; i < SLOTS; ++i) mbar_init(&bars[i], 1);
  fence_barrier_init();
  const long long cps = ag_chunks_per_shard(p);
  const int n_owners = p.ag_local >= 0 ? p.ag_world - 1 : p.ag_world;   // the local shard is in place
  const long long n_chunks = cps * n_owners;
  const int G = p.ag_copiers, c = blockIdx.x;
  const long long mine = (n_chunks - c + G - 1) / G;   // chunks c, c+G, ... of the shards to copy
  auto chunk_geom = [&](long long k, const uint8_t*& src, uint8_t*& dst, uint32_t& bytes, long long& id) {
    const long long r = c + k * G;
    long long owner = r / cps;
    const long long j = r % cps;
    if (p.ag_local >= 0 && owner >= p.ag_local) ++owner;
    id = owner * cps + j;
    const long long off = j * p.ag_chunk_elems;
    const long long n = min(p.ag_chunk_elems, p.ag_shard_elems - off);
    src = reinterpret_cast<const uint8_t*>(p.ag_src[owner]) + off * 2;
    dst = reinterpret_cast<uint8_t*>(p.ag_dst) + (owner * p.ag_shard_elems + off) * 2;
    bytes = (uint32_t)(n * 2);
  };
  auto issue_load = [&](long long k) {
    const uint8_t* src; uint8_t* dst; uint32_t bytes; long long id;
    chunk_geom(k, src, dst, bytes, id);
    const int slot = (int)(k % SLOTS);
    mbar_expect_tx(&bars[slot], bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem + slot * 32768)),
                 "l"(src), "r"(bytes), "r"(smem_u32(&bars[slot]))
                 : "memory");
  };
  auto publish = [&](long long k) {
    const uint8_t* src; uint8_t* dst; uint32_t bytes; long long id;
    chunk_geom(k, src, dst, bytes, id);
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ag_flags + id), "r"(p.ag_epoch) : "memory");
  };
  (void)chunk_bytes_max;
  for (long long k = 0; k < mine && k < SLOTS; ++k) issue_load(k);
  for (long long k = 0; k < mine; ++k) {
    const int slot = (int)(k % SLOTS);
    if (!mbar_wait(&bars[slot], (uint32_t)((k / SLOTS) & 1), p.status, kTimeoutTmaFull, 6)) return;
    const uint8_t* src; uint8_t* dst; uint32_t bytes; long long id;
    chunk_geom(k, src, dst, bytes, id);
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst),
                 "r"(smem_u32(smem + slot * 32768)), "r"(bytes)
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (k >= 1) {
      asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");   // store of chunk k-1 is complete
      publish(k - 1);
      if (k - 1 + SLOTS < mine) issue_load(k - 1 + SLOTS);
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  if (mine > 0) publish(mine - 1);
}

// Push with plain stores: all threads of the copier CTA read 16-byte vectors of the local shard and
// store them into every peer's gathered buffer (posted writes, nothing waits for a round trip
// until the fence that precedes the chunk's flags).
__device__ void ag_pusher(const GemmParams& p) {
  const long long cps = ag_chunks_per_shard(p);
  const int G = p.ag_copiers, c = blockIdx.x;
  const int me = p.ag_local;
  for (long long j = c; j < cps; j += G) {
    const long long off = j * p.ag_chunk_elems;
    const long long n = min(p.ag_chunk_elems, p.ag_shard_elems - off);
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.ag_src[me]) + off);
    const int nvec = (int)(n / 8);
    for (int i = threadIdx.x; i < nvec; i += 16 * blockDim.x) {
      uint4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const int k = i + u * blockDim.x;
        if (k < nvec) v[u] = src[k];
      }
      if (p.ag_push_mc != nullptr) {
        // one multimem store per 16 bytes: the switch replicates it into every rank's gathered buffer
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.ag_push_mc) +
                                              (long long)me * p.ag_shard_elems + off);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int k = i + u * blockDim.x;
          if (k < nvec)
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + k),
                         "f"(__uint_as_float(v[u].x)), "f"(__uint_as_float(v[u].y)), "f"(__uint_as_float(v[u].z)),
                         "f"(__uint_as_float(v[u].w))
                         : "memory");
        }
        continue;
      }
      for (int r = 0; r < p.ag_world; ++r) {
        if (r == me) continue;
        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.ag_push_dst[r]) +
                                              (long long)me * p.ag_shard_elems + off);
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const int k = i + u * blockDim.x;
          if (k < nvec) dst[k] = v[u];
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int r = 0; r < p.ag_world; ++r) {
        if (r == me) continue;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.ag_push_flags[r] + me * cps + j), "r"(p.ag_epoch)
                     : "memory");
      }
    }
  }
}

// PAIR: the kernel runs as clusters of two CTAs on 256 x 256 output tiles.  Each CTA stages its
// 128 rows of A and ONE 128-row half of B per k-block (32 KB instead of 48 KB, in a 6-deep ring),
// the even CTA issues tcgen05.mma.cta_group::2 (M = 256) for both, and each CTA drains its own
// 128 accumulator rows.  Shared-memory traffic per FLOP drops by a third, which is what bounds
// the single-CTA kernel (TMA writes plus operand reads exceed 128 B/clk).  Dense mode only.
template <bool A_MN, bool B_MN, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmB2, const GemmParams p) {
  constexpr int NST = PAIR ? 6 : STAGES;                 // ring depth
  constexpr int SBYTES = PAIR ? 32768 : STAGE_BYTES;     // bytes per stage in this CTA
  constexpr int TM = PAIR ? 2 * BM : BM;                 // output rows per tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);   // == 6 * 32768
  uint64_t* empty = full + NST;
  uint64_t* acc_full = empty + NST;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  uint4* epi_stage = reinterpret_cast<uint4*>(smem + STAGES * STAGE_BYTES + 256);   // after the barrier block

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (!PAIR && (int)blockIdx.x < p.ag_copiers) {
    if (p.ag_push) ag_pusher(p); else ag_copier(p, smem);
    return;
  }
  const int rank = PAIR ? (int)cluster_ctarank() : 0;    // 0: issues the MMAs of the pair
  // tiles are dealt to CTAs (or to CTA pairs)
  const int cta = PAIR ? (int)blockIdx.x / 2 : (int)blockIdx.x - p.ag_copiers;
  const int n_ctas = PAIR ? (int)gridDim.x / 2 : (int)gridDim.x - p.ag_copiers;
  const bool swiglu = p.epi == TPB_EPI_SWIGLU;
  const int tile_n_out = swiglu ? BN / 2 : BN;  // output columns covered by one tile
  const int n_logical = swiglu ? p.N / 2 : p.N;
  const int m_tiles = (p.M + TM - 1) / TM;
  const int n_tiles = (n_logical + tile_n_out - 1) / tile_n_out;
  const int num_tiles = m_tiles * n_tiles * (p.mode == 2 ? p.num_experts : 1);
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], PAIR ? 8 : 4);   // one arrival per epilogue warp (of both CTAs)
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(tmem_slot, 512);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, 512);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      tma_prefetch_desc(&tmB2);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        const TileInfo ti = tile_info(p, t, m_tiles, n_tiles, num_kb);
        if (ti.skip) continue;
        const int m0 = ti.tm * TM + rank * BM, n0 = ti.tn * tile_n_out;
        const int ez = p.mode == 1 ? ti.e : 0;
        if (p.ag_world > 0) {
          // B rows [n0, n0 + BN) of a dense [N, ldb = K] matrix occupy one flat range; with the SwiGLU
          // epilogue a tile takes tile_n_out "gate" rows and the same rows of the "up" half
          const int r1 = swiglu ? min(n_logical, n0 + tile_n_out) : min(p.N, n0 + BN);
          const long long lo = p.ag_b_offset + (long long)n0 * p.K;
          const long long hi = p.ag_b_offset + (long long)r1 * p.K - 1;
          if (!ag_wait_range(p, lo, hi)) { ok = false; break; }
          if (swiglu) {
            const long long lo2 = p.ag_b_offset + (long long)(p.b2_off + n0) * p.K;
            const long long hi2 = p.ag_b_offset + (long long)(p.b2_off + r1) * p.K - 1;
            if (!ag_wait_range(p, lo2, hi2)) { ok = false; break; }
          }
        }
        for (int kb = ti.kb0; kb < ti.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1, p.status, kTimeoutStageFree, 1)) {
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * SBYTES;
          uint8_t* sB = sA + A_BYTES;
          const int k0 = kb * BK;
          if (PAIR) {
            // Both CTAs' bytes are counted on the even CTA's barrier, which alone expects them.
            const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
            if (rank == 0) mbar_expect_tx(&full[stage], 2 * SBYTES);
            if (!A_MN) {
              tma_load_2d_pair(sA, &tmA, bar, k0, m0);
            } else {
#pragma unroll
              for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sA + c * 8192, &tmA, bar, m0 + c * 64, k0);
            }
            // this CTA's half of B: rows/columns [n0 + rank * 128, +128) (for SwiGLU the odd CTA
            // takes the "up" half)
            const CUtensorMap* mb = (swiglu && rank == 1) ? &tmB2 : &tmB;
            const int nb = (swiglu && rank == 1) ? p.b2_off + n0 : n0 + rank * 128;
            if (!B_MN) {
              tma_load_3d_pair(sB, mb, bar, k0, nb, ez);
            } else {
#pragma unroll
              for (int c = 0; c < 2; ++c) tma_load_3d_pair(sB + c * 8192, mb, bar, nb + c * 64, k0, ez);
            }
          } else {
          mbar_expect_tx(&full[stage], STAGE_BYTES);
          if (!A_MN) {
            tma_load_2d(sA, &tmA, &full[stage], k0, m0);  // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)  // box {64 m, 64 k}
              tma_load_2d(sA + c * 8192, &tmA, &full[stage], m0 + c * 64, k0);
          }
          if (!B_MN) {
            // two boxes {64 k, 128 rows}; for SwiGLU the second one comes from the "up" half
            // (with two B maps the "up" half is the same rows of the second tensor)
            tma_load_3d(sB, &tmB, &full[stage], k0, n0, ez);
            tma_load_3d(sB + 16384, &tmB2, &full[stage], k0, swiglu ? p.b2_off + n0 : n0 + 128, ez);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) {
              if (swiglu && c >= 2)
                tma_load_3d(sB + c * 8192, &tmB2, &full[stage], p.b2_off + n0 + (c - 2) * 64, k0, ez);
              else
                tma_load_3d(sB + c * 8192, &tmB, &full[stage], n0 + c * 64, k0, ez);
            }
          }
          }
          if (++stage == NST) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(TM, BN, A_MN, B_MN);
      constexpr uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t smem_base = smem_u32(smem);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int local = 0;
      for (int t = cta; t < num_tiles && ok; t += n_ctas) {
        const TileInfo ti = tile_info(p, t, m_tiles, n_tiles, num_kb);
        if (ti.skip) continue;
        const int acc = local & 1;
        const uint32_t acc_phase = (local >> 1) & 1;
        ++local;
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, p.status, kTimeoutAccFree, 2)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        // The MMA queue is shallow: whatever this thread does between two MMAs is tensor idle
        // time.  So the wait for the next k-block's operands is placed before the last MMA of the
        // current one, where its latency hides behind the MMAs still in flight.
        bool prewaited = false;
        for (int kb = ti.kb0; kb < ti.kb1; ++kb) {
          if (!prewaited && !mbar_wait(&full[stage], phase, p.status, kTimeoutTmaFull, 3)) {
            ok = false;
            break;
          }
          prewaited = false;
          tc_fence_after();
          // Descriptors of one stage differ from the stage's first one only in the low word, by a
          // compile-time constant per k-step: one integer add per operand and MMA.
          const uint32_t sA = smem_base + stage * SBYTES;
          const uint32_t a_lo = smem_desc_lo(sA, A_MN ? 8192 : 16);
          const uint32_t b_lo = smem_desc_lo(sA + A_BYTES, B_MN ? 8192 : 16);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            if (k == BK / 16 - 1 && kb + 1 < ti.kb1) {
              const int ns = (stage + 1 == NST) ? 0 : stage + 1;
              const uint32_t np = (stage + 1 == NST) ? (phase ^ 1) : phase;
              if (!mbar_wait(&full[ns], np, p.status, kTimeoutTmaFull, 3)) {
                ok = false;
                break;
              }
              prewaited = true;
            }
            if (PAIR)
              mma_ss_pair_w(d_tmem, a_lo + (A_MN ? k * 128 : k * 2), desc_hi, b_lo + (B_MN ? k * 128 : k * 2), desc_hi,
                            idesc, ((kb - ti.kb0) | k) != 0);
            else
              mma_ss_w(d_tmem, a_lo + (A_MN ? k * 128 : k * 2), desc_hi, b_lo + (B_MN ? k * 128 : k * 2), desc_hi, idesc,
                       ((kb - ti.kb0) | k) != 0);
          }
          if (!ok) break;
          if (PAIR) tc_commit_pair(&empty[stage]); else tc_commit(&empty[stage]);
          if (++stage == NST) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) { if (PAIR) tc_commit_pair(&acc_full[acc]); else tc_commit(&acc_full[acc]); }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    int local = 0;
    for (int t = cta; t < num_tiles; t += n_ctas) {
      const TileInfo ti = tile_info(p, t, m_tiles, n_tiles, num_kb);
      if (ti.skip) continue;
      const int acc = local & 1;
      const uint32_t acc_phase = (local >> 1) & 1;
      ++local;
      if (!mbar_wait(&acc_full[acc], acc_phase, p.status, kTimeoutAccFull, 4)) break;
      tc_fence_after();
      const int tm = ti.tm, tn = ti.tn;
      const bool empty_k = ti.kb1 <= ti.kb0;   // nothing was accumulated: the tile is all zeros
      const long long c_off = p.mode == 2 ? (long long)ti.e * p.c_stride : 0;
      const int row = tm * TM + rank * BM + q * 32 + lane;
      const int n0 = tn * tile_n_out;
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const bool row_ok = row < p.M;

      if (swiglu) {
        __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + (long long)row * p.ldc;
        __nv_bfloat16* C2 =
            p.c2 ? reinterpret_cast<__nv_bfloat16*>(p.c2) + (long long)row * p.ldc2 : nullptr;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tmem_ld32(t_addr + c * 32, g);
          tmem_ld32(t_addr + 128 + c * 32, u);
          tmem_wait_ld();
          const int col = n0 + c * 32;
          if (row_ok && col < n_logical) {
            uint32_t o[16], pg[16], pu[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              float g0 = __uint_as_float(g[2 * j]) * p.alpha, g1 = __uint_as_float(g[2 * j + 1]) * p.alpha;
              float u0 = __uint_as_float(u[2 * j]) * p.alpha, u1 = __uint_as_float(u[2 * j + 1]) * p.alpha;
              o[j] = pack_bf16(silu_f(g0) * u0, silu_f(g1) * u1);
              pg[j] = pack_bf16(g0, g1);
              pu[j] = pack_bf16(u0, u1);
            }
            if (col + 32 <= n_logical) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                *reinterpret_cast<uint4*>(C + col + v * 8) =
                    make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
                if (C2) {
                  *reinterpret_cast<uint4*>(C2 + col + v * 8) =
                      make_uint4(pg[4 * v], pg[4 * v + 1], pg[4 * v + 2], pg[4 * v + 3]);
                  *reinterpret_cast<uint4*>(C2 + p.b_split + col + v * 8) =
                      make_uint4(pu[4 * v], pu[4 * v + 1], pu[4 * v + 2], pu[4 * v + 3]);
                }
              }
            } else {
              for (int j = 0; j < 32 && col + j < n_logical; ++j) {
                float2 ov = unpack_bf16(o[j >> 1]), gv = unpack_bf16(pg[j >> 1]), uv = unpack_bf16(pu[j >> 1]);
                C[col + j] = __float2bfloat16((j & 1) ? ov.y : ov.x);
                if (C2) {
                  C2[col + j] = __float2bfloat16((j & 1) ? gv.y : gv.x);
                  C2[p.b_split + col + j] = __float2bfloat16((j & 1) ? uv.y : uv.x);
                }
              }
            }
          }
        }
      } else if (p.epi == TPB_EPI_RS_BF16 || p.epi == TPB_EPI_AR_BF16) {
        // Epilogues that reduce into other GPUs' memory.  A thread owns one accumulator row, so its
        // 16-byte vectors lie 2 * ldc bytes from its neighbours' and every lane would send its own
        // small request over NVLink.  The warp therefore transposes 64 columns through a 4 KB
        // shared-memory slab (XOR-swizzled, conflict-free both ways): afterwards eight consecutive
        // lanes hold the eight vectors of one row and reduce 128 contiguous bytes.
        uint4* slab = epi_stage + q * 256;
        const int row_base = tm * TM + rank * BM + q * 32;
        const bool all_reduce = p.epi == TPB_EPI_AR_BF16;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld32(t_addr + (c + h) * 32, r);
            tmem_wait_ld();
            const int col = n0 + (c + h) * 32;
            const __nv_bfloat16* R = nullptr;
            if (all_reduce && p.aux != nullptr && row_ok)
              R = reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)row * p.ldaux + col;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) f[j] = empty_k ? 0.f : __uint_as_float(r[8 * v + j]) * p.alpha;
              if (R && col + 8 * v + 8 <= p.N) {
                const uint4 old = *reinterpret_cast<const uint4*>(R + 8 * v);
                const float2 a = unpack_bf16(old.x), b = unpack_bf16(old.y), cc = unpack_bf16(old.z), d = unpack_bf16(old.w);
                f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
                f[4] += cc.x; f[5] += cc.y; f[6] += d.x; f[7] += d.y;
              }
              slab[lane * 8 + ((h * 4 + v) ^ (lane & 7))] =
                  make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
            }
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = (lane >> 3) + 4 * i, vec = lane & 7;
            const uint4 o = slab[rr * 8 + (vec ^ (rr & 7))];
            const int grow = row_base + rr, gcol = n0 + c * 32 + vec * 8;
            if (grow >= p.M || gcol + 8 > p.N) continue;
            if (all_reduce) {
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + (long long)grow * p.ldc + gcol;
              asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(o.x),
                           "r"(o.y), "r"(o.z), "r"(o.w)
                           : "memory");
            } else {
              const long long flat = p.rs_c_offset + (long long)grow * p.ldc + gcol;
              const long long owner = flat / p.rs_shard_elems;
              __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.rs_dst[owner]) + (flat - owner * p.rs_shard_elems);
              if (p.rs_store)
                *reinterpret_cast<uint4*>(dst) = o;
              else
                asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(o.x),
                             "r"(o.y), "r"(o.z), "r"(o.w)
                             : "memory");
            }
          }
          __syncwarp();
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(t_addr + c * 32, r);
          tmem_wait_ld();
          if (empty_k) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = 0;
          }
          const int col = n0 + c * 32;
          if (!row_ok || col >= p.N) continue;
          const bool full_chunk = col + 32 <= p.N;
          if (p.epi == TPB_EPI_F32 || p.epi == TPB_EPI_F32_ACC) {
            float* C = reinterpret_cast<float*>(p.C) + c_off + (long long)row * p.ldc + col;
            const bool accm = p.epi == TPB_EPI_F32_ACC;
            if (full_chunk) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                float4 o = make_float4(__uint_as_float(r[4 * v]) * p.alpha, __uint_as_float(r[4 * v + 1]) * p.alpha,
                                       __uint_as_float(r[4 * v + 2]) * p.alpha, __uint_as_float(r[4 * v + 3]) * p.alpha);
                if (accm) {
                  float4 old = *reinterpret_cast<float4*>(C + 4 * v);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(C + 4 * v) = o;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float o = __uint_as_float(r[j]) * p.alpha;
                C[j] = accm ? C[j] + o : o;
              }
            }
          } else {
            __nv_bfloat16* C = reinterpret_cast<__nv_bfloat16*>(p.C) + c_off + (long long)row * p.ldc + col;
            const __nv_bfloat16* R = nullptr;
            if (p.epi == TPB_EPI_BF16_ACC) R = C;
            if (p.epi == TPB_EPI_BF16_RES)
              R = reinterpret_cast<const __nv_bfloat16*>(p.aux) + (long long)row * p.ldaux + col;
            if (full_chunk) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[8 * v + j]) * p.alpha;
                if (R) {
                  uint4 old = *reinterpret_cast<const uint4*>(R + 8 * v);
                  float2 a = unpack_bf16(old.x), b = unpack_bf16(old.y), cc = unpack_bf16(old.z), d = unpack_bf16(old.w);
                  f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
                  f[4] += cc.x; f[5] += cc.y; f[6] += d.x; f[7] += d.y;
                }
                *reinterpret_cast<uint4*>(C + 8 * v) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]),
                                                                  pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float o = __uint_as_float(r[j]) * p.alpha;
                if (R) o += __bfloat162float(R[j]);
                C[j] = __float2bfloat16(o);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
        else mbar_arrive(&acc_empty[acc]);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // neither CTA's shared memory or TMEM goes away under the other
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------
// Host side
// ----------------------------------------------------------------------------
int make_tmap_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t pitch_elems,
                 uint32_t box_inner, uint32_t box_outer, int elem_bytes);  // tma.cu
int make_tmap_3d(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                 uint64_t stride2_elems, uint32_t box0, uint32_t box1);
int sm_count();  // runtime.cu

template <bool A_MN, bool B_MN>
cudaError_t launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                        int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<A_MN, B_MN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GEMM_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  gemm_kernel<A_MN, B_MN, false><<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(ta, tb, tb2, p);
  return cudaGetLastError();
}

// Launch as clusters of two CTAs (`grid` is even).
template <bool A_MN, bool B_MN>
cudaError_t launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tb2, const GemmParams& p,
                             int grid, cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<A_MN, B_MN, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GEMM_SMEM);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = GEMM_SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, gemm_kernel<A_MN, B_MN, true>, ta, tb, tb2, p);
}



struct GemmCall {
  const void* A; const void* B; const void* B2; void* C;
  int M, N, K, E;
  long long lda, ldb, b_expert_stride, ldc;
  int a_mn, b_mn, epi;
  float alpha;
  const void* aux; long long ldaux;
  void* c2; long long ldc2;
  int max_ctas;
  int mode; const int* tile_expert; const int* k_offsets; long long c_stride;
  int row_align;                // grouped rows mode: expert segments are padded to this many rows (128 or 256)
  // fusion with collectives (0 / null when unused)
  int ag_world, ag_copiers, ag_local; const void* const* ag_src; void* ag_dst; long long ag_shard_elems, ag_b_offset;
  unsigned* ag_flags; unsigned ag_epoch;
  void* const* ag_push_dst; unsigned* const* ag_push_flags; void* ag_push_mc;
  int rs_world; void* const* rs_dst; long long rs_shard_elems, rs_c_offset;
  int rs_rank;
  int rs_store;
  long long ag_chunk_elems;     // external gather (ag_copiers == 0): elements per flag
};

static int run_gemm(const GemmCall& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return 0;
  const bool swiglu = g.epi == TPB_EPI_SWIGLU;
  auto misaligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) % 16) != 0; };
  if ((g.lda % 8) || (g.ldb % 8) || (g.b_expert_stride % 8) || misaligned(g.A) || misaligned(g.B) || misaligned(g.C) ||
      (g.B2 && misaligned(g.B2)))
    return -2;
  const bool f32out = g.epi == TPB_EPI_F32 || g.epi == TPB_EPI_F32_ACC;
  if (g.ldc % (f32out ? 4 : 8)) return -2;
  if (swiglu && ((g.N % 2) || ((g.N / 2) % 8))) return -2;
  if (g.mode == 2 && !(g.a_mn && g.b_mn)) return -2;
  if (g.mode == 1 && g.a_mn) return -2;
  const bool two_b = swiglu && g.B2 != nullptr && g.B2 != g.B;
  const int b_extent = two_b ? g.N / 2 : g.N;       // rows (K-major) or columns (MN-major) of one B tensor
  const int b_experts = g.mode == 1 ? g.E : 1;
  CUtensorMap ta, tb, tb2;
  int r;
  if (!g.a_mn) r = make_tmap_2d(&ta, g.A, g.K, g.M, g.lda, 64, 128, 2);
  else         r = make_tmap_2d(&ta, g.A, g.M, g.K, g.lda, 64, 64, 2);
  if (r) return r < 0 ? -3 : -4;
  const uint64_t estride = b_experts > 1 ? (uint64_t)g.b_expert_stride : (uint64_t)g.ldb * (g.b_mn ? g.K : b_extent);
  auto make_b = [&](CUtensorMap* m, const void* ptr) {
    return !g.b_mn ? make_tmap_3d(m, ptr, g.K, b_extent, b_experts, g.ldb, estride, 64, 128)
                   : make_tmap_3d(m, ptr, b_extent, g.K, b_experts, g.ldb, estride, 64, 64);
  };
  r = make_b(&tb, g.B);
  if (r) return r < 0 ? -3 : -5;
  if (two_b) {
    r = make_b(&tb2, g.B2);
    if (r) return r < 0 ? -3 : -5;
  } else {
    tb2 = tb;
  }

  GemmParams p;
  p.M = g.M; p.N = g.N; p.K = g.K;
  p.C = g.C; p.ldc = g.ldc;
  p.aux = g.aux; p.ldaux = g.ldaux;
  p.c2 = g.c2; p.ldc2 = g.ldc2;
  p.b_split = g.N / 2;
  p.b2_off = two_b ? 0 : g.N / 2;
  p.alpha = g.alpha;
  p.epi = g.epi;
  p.status = status_block();
  p.mode = g.mode; p.num_experts = g.E; p.tile_expert = g.tile_expert; p.k_offsets = g.k_offsets;
  p.c_stride = g.c_stride;
  p.ag_world = g.ag_world; p.ag_copiers = g.ag_world > 0 ? g.ag_copiers : 0;
  p.ag_dst = g.ag_dst; p.ag_shard_elems = g.ag_shard_elems; p.ag_chunk_elems = 16384; p.ag_b_offset = g.ag_b_offset;
  p.ag_flags = g.ag_flags; p.ag_epoch = g.ag_epoch; p.ag_local = g.ag_world > 0 ? g.ag_local : -1;
  p.rs_world = g.rs_world; p.rs_shard_elems = g.rs_shard_elems; p.rs_c_offset = g.rs_c_offset;
  p.tile_rot = 0;
  p.te_stride = 1;
  p.rs_store = g.rs_store;
  if (g.ag_world > 0 && g.ag_copiers == 0) p.ag_chunk_elems = g.ag_chunk_elems;   // external gather: the caller's flags
  p.ag_push = (g.ag_world > 0 && g.ag_push_dst != nullptr && g.ag_push_flags != nullptr) ? 1 : 0;
  p.ag_push_mc = p.ag_push ? g.ag_push_mc : nullptr;
  if (p.ag_push) p.ag_chunk_elems = 131072;   // 256 KB per flag: a CTA streams a chunk with one fence at its end
  for (int i = 0; i < 8; ++i) {
    p.ag_push_dst[i] = (p.ag_push && i < g.ag_world) ? g.ag_push_dst[i] : nullptr;
    p.ag_push_flags[i] = (p.ag_push && i < g.ag_world) ? g.ag_push_flags[i] : nullptr;
    p.ag_src[i] = (g.ag_world > 0 && g.ag_src != nullptr && i < g.ag_world) ? g.ag_src[i] : nullptr;
    p.rs_dst[i] = (g.rs_world > 0 && i < g.rs_world) ? g.rs_dst[i] : nullptr;
  }
  if (g.ag_world > 0) {
    if (g.ag_world > 8 || g.b_mn || g.mode != 0) return -2;
    if (g.ldb != g.K || (g.ag_shard_elems % 8) || p.ag_copiers < 0 || p.ag_copiers >= sm_count()) return -2;
    if (p.ag_copiers == 0 && (p.ag_chunk_elems <= 0 || p.ag_flags == nullptr || p.ag_push)) return -2;
    if (p.ag_push && (g.ag_local < 0 || g.ag_local >= g.ag_world)) return -2;
  }
  if (g.epi == TPB_EPI_AR_BF16 && ((g.N % 32) || (g.ldc % 8) || g.mode != 0 || g.ag_world > 0)) return -2;
  if (g.epi == TPB_EPI_RS_BF16) {
    if (g.rs_world < 1 || g.rs_world > 8 || (g.N % 8) || (g.ldc % 8) || (g.rs_shard_elems % 8) || (g.rs_c_offset % 8))
      return -2;
  }
  const int n_logical = swiglu ? g.N / 2 : g.N;
  const int tile_n = swiglu ? BN / 2 : BN;
  const int m_tiles = (g.M + BM - 1) / BM, n_tiles = (n_logical + tile_n - 1) / tile_n;
  p.group_m = m_tiles < 16 ? m_tiles : 16;
  long long tiles = (long long)m_tiles * n_tiles * (g.mode == 2 ? g.E : 1);
  int cap = sm_count() - p.ag_copiers;
  if (g.max_ctas > 0 && g.max_ctas < cap) cap = g.max_ctas;
  const int grid = (tiles > cap ? cap : (int)tiles) + p.ag_copiers;
  const bool rs_rotate = g.epi == TPB_EPI_RS_BF16 && g.rs_world > 1 && g.rs_rank > 0;
  if (rs_rotate)
    p.tile_rot = (int)(tiles * g.rs_rank / g.rs_world);   // every rank starts in a different owner's part of C
  cudaError_t e;
  // CTA pairs for dense GEMMs with enough 256 x 256 tiles to fill the machine (TPB_GEMM_PAIR=0
  // keeps the single-CTA kernel)
  // TPB_GEMM_PAIR: 0 = never, 2 = for every dense shape (tests), default = when the tiles fill the machine
  static const int pair_mode = []() { const char* v = getenv("TPB_GEMM_PAIR"); return v ? atoi(v) : 1; }();
  static const int max_pairs = []() {
    // clusters of two that can be resident at once (an SM without a free partner stays idle)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = GEMM_SMEM;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    cudaFuncSetAttribute(gemm_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM);
    if (cudaOccupancyMaxActiveClusters(&n, gemm_kernel<false, false, true>, &cfg) != cudaSuccess || n < 1) n = 0;
    (void)cudaGetLastError();
    return n < sm_count() / 2 ? n : sm_count() / 2;
  }();
  const long long pair_tiles = (long long)((g.M + 2 * BM - 1) / (2 * BM)) * n_tiles * (g.mode == 2 ? g.E : 1);
  // grouped modes: rows mode needs expert segments padded to whole 256-row tiles; the per-expert
  // K-range mode (weight gradients) has no such condition
  const bool pair_shape_ok = g.mode == 0 || g.mode == 2 || (g.mode == 1 && g.row_align > 0 && g.row_align % (2 * BM) == 0);
  // (the in-kernel copier CTAs of the fused all-gather and the red.add reduce-scatter were tuned on the
  // single-CTA kernel and stay there; waiting on an external gather and the store-mode scatter run on pairs)
  const bool pair_coll_ok = (g.ag_world == 0 || p.ag_copiers == 0) && (g.epi != TPB_EPI_RS_BF16 || g.rs_store);
  if (pair_mode != 0 && max_pairs > 0 && pair_shape_ok && pair_coll_ok &&
      g.max_ctas == 0 && (pair_mode == 2 || pair_tiles >= max_pairs)) {
    p.te_stride = 2;
    if (rs_rotate) p.tile_rot = (int)(pair_tiles * g.rs_rank / g.rs_world);
    const int pairs = pair_tiles > max_pairs ? max_pairs : (int)pair_tiles;
    const int m_tiles2 = (g.M + 2 * BM - 1) / (2 * BM);
    p.group_m = m_tiles2 < 8 ? m_tiles2 : 8;
    if (!g.a_mn && !g.b_mn)      e = launch_gemm_pair<false, false>(ta, tb, tb2, p, 2 * pairs, stream);
    else if (!g.a_mn && g.b_mn)  e = launch_gemm_pair<false, true>(ta, tb, tb2, p, 2 * pairs, stream);
    else if (g.a_mn && !g.b_mn)  e = launch_gemm_pair<true, false>(ta, tb, tb2, p, 2 * pairs, stream);
    else                         e = launch_gemm_pair<true, true>(ta, tb, tb2, p, 2 * pairs, stream);
    return e == cudaSuccess ? 0 : 1000 + (int)e;
  }
  if (!g.a_mn && !g.b_mn)      e = launch_gemm<false, false>(ta, tb, tb2, p, grid, stream);
  else if (!g.a_mn && g.b_mn)  e = launch_gemm<false, true>(ta, tb, tb2, p, grid, stream);
  else if (g.a_mn && !g.b_mn)  e = launch_gemm<true, false>(ta, tb, tb2, p, grid, stream);
  else                         e = launch_gemm<true, true>(ta, tb, tb2, p, grid, stream);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

}  // namespace tpb

using namespace tpb;

extern "C" int tpb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                             long long ldb, long long ldc, int a_mn, int b_mn, int epi, float alpha,
                             const void* aux, long long ldaux, void* c2, long long ldc2, int max_ctas,
                             void* stream_) {
  GemmCall g{};
  g.A = A; g.B = B; g.B2 = nullptr; g.C = C;
  g.M = M; g.N = N; g.K = K; g.E = 1;
  g.lda = lda; g.ldb = ldb; g.b_expert_stride = 0; g.ldc = ldc;
  g.a_mn = a_mn; g.b_mn = b_mn; g.epi = epi; g.alpha = alpha;
  g.aux = aux; g.ldaux = ldaux; g.c2 = c2; g.ldc2 = ldc2; g.max_ctas = max_ctas;
  g.mode = 0;
  return run_gemm(g, reinterpret_cast<cudaStream_t>(stream_));
}

extern "C" int tpb_grouped_gemm_bf16(const void* A, const void* B, const void* B2, void* C, int M, int N, int K,
                                     int E, long long lda, long long ldb, long long b_expert_stride, long long ldc,
                                     int a_mn, int b_mn, int epi, float alpha, void* c2, long long ldc2, int mode,
                                     const int* tile_expert, const int* k_offsets, long long c_stride,
                                     int row_align, void* stream_) {
  if (mode != 1 && mode != 2) return -2;
  if (mode == 1 && !tile_expert) return -2;
  if (mode == 2 && !k_offsets) return -2;
  GemmCall g{};
  g.A = A; g.B = B; g.B2 = B2; g.C = C;
  g.M = M; g.N = N; g.K = K; g.E = E;
  g.lda = lda; g.ldb = ldb; g.b_expert_stride = b_expert_stride; g.ldc = ldc;
  g.a_mn = a_mn; g.b_mn = b_mn; g.epi = epi; g.alpha = alpha;
  g.aux = nullptr; g.ldaux = 0; g.c2 = c2; g.ldc2 = ldc2; g.max_ctas = 0;
  g.mode = mode; g.tile_expert = tile_expert; g.k_offsets = k_offsets; g.c_stride = c_stride;
  g.row_align = row_align;
  return run_gemm(g, reinterpret_cast<cudaStream_t>(stream_));
}


// C = A * B^T where the flat bf16 buffer holding B is sharded over `world` GPUs: shard_ptrs[r] is
// rank r's shard (peer-mapped symmetric memory), `gathered` the local buffer that receives all
// shards (world * shard_elems elements), B starts b_offset elements into it and is a dense
// row-major [N, K] matrix.  `flags` has world * ceil(shard_elems / 16384) entries (local memory,
// zero-initialised once); pass a fresh non-zero `epoch` per call.  The whole buffer is gathered.
// local_rank >= 0: that rank's shard is already in `gathered` (it is neither copied nor waited for).
// push_gathered / push_flags (both non-null): push mode, tables of every rank's gathered buffer and
// flag array in symmetric memory (`gathered` and `flags` are this rank's entries); the copier CTAs
// then send the local shard to the peers instead of fetching theirs.
extern "C" int tpb_ag_gemm_bf16(const void* A, void* C, int M, int N, int K, long long lda, long long ldc, int epi,
                                const void* aux, long long ldaux, void* c2, long long ldc2,
                                const void* const* shard_ptrs, int world, long long shard_elems, void* gathered,
                                long long b_offset, unsigned* flags, unsigned epoch, int copiers, int local_rank,
                                void* const* push_gathered, unsigned* const* push_flags, void* push_multicast,
                                void* stream_) {
  GemmCall g{};
  g.A = A; g.B = reinterpret_cast<const __nv_bfloat16*>(gathered) + b_offset; g.B2 = nullptr; g.C = C;
  g.M = M; g.N = N; g.K = K; g.E = 1;
  g.lda = lda; g.ldb = K; g.b_expert_stride = 0; g.ldc = ldc;
  g.a_mn = 0; g.b_mn = 0; g.epi = epi; g.alpha = 1.f;
  g.aux = aux; g.ldaux = ldaux; g.c2 = c2; g.ldc2 = ldc2; g.max_ctas = 0; g.mode = 0;
  g.ag_world = world; g.ag_copiers = copiers; g.ag_src = shard_ptrs; g.ag_dst = gathered;
  g.ag_shard_elems = shard_elems; g.ag_b_offset = b_offset; g.ag_flags = flags; g.ag_epoch = epoch;
  g.ag_local = local_rank;
  g.ag_push_dst = push_gathered; g.ag_push_flags = push_flags; g.ag_push_mc = push_multicast;
  return run_gemm(g, reinterpret_cast<cudaStream_t>(stream_));
}

// C[M,N] = alpha * A * B^T reduced over ranks into the owners' bf16 shards: element (row, col) of C
// has flat index c_offset + row * ldc + col in a buffer sharded `shard_elems` per rank;
// shard_ptrs[r] is rank r's (peer-mapped) shard.  Shards must be zeroed (and all ranks past a
// barrier) before the first contributing kernel, and a barrier must follow the last one.
extern "C" int tpb_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                                long long ldc, int a_mn, int b_mn, float alpha, void* const* shard_ptrs, int world,
                                long long shard_elems, long long c_offset, int rank, void* stream_) {
  GemmCall g{};
  g.A = A; g.B = B; g.B2 = nullptr; g.C = shard_ptrs[0];
  g.M = M; g.N = N; g.K = K; g.E = 1;
  g.lda = lda; g.ldb = ldb; g.b_expert_stride = 0; g.ldc = ldc;
  g.a_mn = a_mn; g.b_mn = b_mn; g.epi = TPB_EPI_RS_BF16; g.alpha = alpha;
  g.mode = 0;
  g.rs_world = world; g.rs_dst = shard_ptrs; g.rs_shard_elems = shard_elems; g.rs_c_offset = c_offset;
  g.rs_rank = rank;
  return run_gemm(g, reinterpret_cast<cudaStream_t>(stream_));
}

// C = A * B^T (+ epilogue) where B is a dense row-major [N, K] matrix `b_offset` elements into a
// gathered buffer that somebody else (the copy engines, see fsdp_comm.cu) is still filling: the
// buffer is `world` shards of `shard_elems` elements, every `chunk_elems` elements of a shard have
// one flag (flags[owner * ceil(shard_elems / chunk_elems) + chunk], local memory) that holds the
// epoch of the newest gather that has landed there.  The TMA producer waits (bounded) until the flags
// under its B tile have reached `epoch` before it loads the tile.
extern "C" int tpb_gemm_ag_wait_bf16(const void* A, void* C, int M, int N, int K, long long lda, long long ldc,
                                     int epi, const void* aux, long long ldaux, void* c2, long long ldc2,
                                     const void* gathered, long long b_offset, int world, long long shard_elems,
                                     long long chunk_elems, unsigned* flags, unsigned epoch, void* stream_) {
  GemmCall g{};
  g.A = A; g.B = reinterpret_cast<const __nv_bfloat16*>(gathered) + b_offset; g.B2 = nullptr; g.C = C;
  g.M = M; g.N = N; g.K = K; g.E = 1;
  g.lda = lda; g.ldb = K; g.b_expert_stride = 0; g.ldc = ldc;
  g.a_mn = 0; g.b_mn = 0; g.epi = epi; g.alpha = 1.f;
  g.aux = aux; g.ldaux = ldaux; g.c2 = c2; g.ldc2 = ldc2; g.max_ctas = 0; g.mode = 0;
  g.ag_world = world; g.ag_copiers = 0; g.ag_src = nullptr; g.ag_dst = const_cast<void*>(gathered);
  g.ag_shard_elems = shard_elems; g.ag_b_offset = b_offset; g.ag_flags = flags; g.ag_epoch = epoch;
  g.ag_local = -1; g.ag_chunk_elems = chunk_elems;
  return run_gemm(g, reinterpret_cast<cudaStream_t>(stream_));
}

// tpb_gemm_rs_bf16 with plain stores: `slot_ptrs[o]` is THIS rank's staging slot inside owner o's memory
// (shard_elems elements); the tile elements that owner o's shard covers are stored there, nothing is added
// and nothing needs to be zero.  The owner reduces the slots of all sources afterwards (tpb_rs_reduce_bf16).
extern "C" int tpb_gemm_rs_store_bf16(const void* A, const void* B, int M, int N, int K, long long lda,
                                      long long ldb, long long ldc, int a_mn, int b_mn, float alpha,
                                      void* const* slot_ptrs, int world, long long shard_elems, long long c_offset,
                                      int rank, void* stream_) {
  GemmCall g{};
  g.A = A; g.B = B; g.B2 = nullptr; g.C = slot_ptrs[0];
  g.M = M; g.N = N; g.K = K; g.E = 1;
  g.lda = lda; g.ldb = ldb; g.b_expert_stride = 0; g.ldc = ldc;
  g.a_mn = a_mn; g.b_mn = b_mn; g.epi = TPB_EPI_RS_BF16; g.alpha = alpha;
  g.mode = 0;
  g.rs_world = world; g.rs_dst = slot_ptrs; g.rs_shard_elems = shard_elems; g.rs_c_offset = c_offset;
  g.rs_rank = rank; g.rs_store = 1;
  return run_gemm(g, reinterpret_cast<cudaStream_t>(stream_));
}
