// Flash-attention backward for sm_100a (tcgen05 + TMEM + TMA), GQA-native, head dim 128.
//
// Two tensor-core kernels working on 128 x 128 score tiles; neither needs atomics or a
// cross-CTA reduction.  Every MMA is 128 x 128 x 16, the smallest shape that runs at the full
// tensor rate with operands in shared memory (a 128 x 64 MMA is bound by operand fetch).
//
//  attn_bwd_dkv_kernel   one CTA per (128-key block, kv head, batch).  K and V of the block
//      stay in shared memory; dK and dV accumulate in TMEM over every 128-row query tile and
//      every query head of the GQA group that can see the block.  Transposed frame (TMEM lane
//      = key row); TMEM: dK [0,128), dV [128,256), S^T [256,384), dP^T [384,512).
//        S^T  = K Q^T  (SS)              dP^T = V dO^T  (SS)
//        P^T  = exp2(S^T*c - lse)        bf16, written over S^T      (compute phase 1)
//        dS^T = P^T o (dP^T - delta)     bf16, written over dP^T     (compute phase 2)
//        dV  += P^T dO (TS)              dK  += dS^T Q (TS; scale applied in the epilogue)
//      Tensor stream per step i:  dV(i), S^T(i+1), dK(i), dP^T(i+1): phase 1 of step i+1
//      overlaps dK(i) and dP^T(i+1), phase 2 overlaps dV(i+1) and S^T(i+2).
//
//  attn_bwd_dq_kernel    one CTA per (128-row query tile, query head, batch); TMEM lane =
//      query row; TMEM: dQ [0,128), S double buffered [128,384), dP [384,512).
//        S  = Q K^T (SS)    dP = dO V^T (SS)    dS = exp2(S*c - lse) o (dP - delta)  over dP
//        dQ += dS K (TS, B = K tile MN-major; scale applied in the epilogue)
//      Tensor stream per step j:  S(j+1), dQ(j), dP(j+1).
//
// Both kernels: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 compute.  Warps w and w+4
// share a TMEM lane quarter and split the 128 score columns of a step; each writes its bf16
// result over the first half of its OWN 64 input columns, so the two never touch each other's
// columns and the A operand of the following MMA is addressed per 16-column k-step.

#include "common.cuh"
#include "tpb.h"

namespace tpb {

int make_tmap_3d(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                 uint64_t stride2_elems, uint32_t box0, uint32_t box1);
int sm_count();

constexpr int BWD_D = 128;
constexpr int BWD_T = 128;         // score tile edge (rows and columns) in both kernels
constexpr int BWD_THREADS = 320;   // TMA warp, MMA warp, 8 compute warps
constexpr int TILE_BYTES = BWD_T * BWD_D * 2;   // one 128 x 128 bf16 operand tile: 32 KB
constexpr int KV_QSTAGES = 2;      // dK/dV kernel: Q tile ring
constexpr int KV_DOSTAGES = 2;     // dK/dV kernel: dO tile ring
constexpr int KV_MAX_TILES = 512;  // query tiles whose position range fits the shared-memory table
constexpr int DQ_KSTAGES = 3;      // dQ kernel: K tile ring (a K tile is held from S(j) to dQ(j))
constexpr int DQ_VSTAGES = 2;      // dQ kernel: V tile ring
constexpr float kLog2e = 1.4426950408889634f;

struct AttnBwdParams {
  int B, Sq, Sk, Hq, Hkv;
  float scale, scale_log2;
  float softcap_in;     // logit soft cap: scores become cap * tanh(q.k * scale / cap); this is scale / cap (0: off),
                        // and scale_log2 is then cap * log2(e)
  int causal, window;
  const int* q_pos;
  const int* q_seg;
  const int* kv_seg;
  const float* lse2;    // [B,Hq,Sq_pad] log-sum-exp in log2 units, +inf in the padding rows
  const float* delta;   // [B,Hq,Sq_pad] rowsum(dO o O), 0 in the padding rows
  int Sq_pad;           // Sq rounded up to 128
  int aux_bulk;         // q_pos / q_seg rows can be bulk-copied (16-byte aligned for every tile)
  __nv_bfloat16* dQ; long long lddq;
  __nv_bfloat16* dK; long long lddk;
  __nv_bfloat16* dV; long long lddv;
  int* status;
};

namespace dkv {
constexpr int OFF_K = 0;
constexpr int OFF_V = OFF_K + TILE_BYTES;
constexpr int OFF_Q = OFF_V + TILE_BYTES;
constexpr int OFF_DO = OFF_Q + KV_QSTAGES * TILE_BYTES;
constexpr int OFF_AUX = OFF_DO + KV_DOSTAGES * TILE_BYTES;   // per Q stage: lse2[128], delta[128], qpos[128], qseg[128]
constexpr int AUX_STAGE = 4 * BWD_T * 4;
constexpr int OFF_TILES = OFF_AUX + KV_QSTAGES * AUX_STAGE;  // tile min/max table: 2 * KV_MAX_TILES ints
constexpr int OFF_BAR = OFF_TILES + 2 * KV_MAX_TILES * 4;
constexpr int TOTAL = OFF_BAR + 256 + 1024;
constexpr int T_DK = 0, T_DV = 128, T_S = 256, T_DP = 384;
}  // namespace dkv

namespace dqk {
constexpr int OFF_Q = 0;
constexpr int OFF_DO = OFF_Q + TILE_BYTES;
constexpr int OFF_K = OFF_DO + TILE_BYTES;
constexpr int OFF_V = OFF_K + DQ_KSTAGES * TILE_BYTES;
constexpr int OFF_BAR = OFF_V + DQ_VSTAGES * TILE_BYTES;
constexpr int TOTAL = OFF_BAR + 256 + 1024;
constexpr int T_DQ = 0, T_S = 128, T_DP = 384;
}  // namespace dqk

// delta[b,h,q] = sum_d dO * O and lse2[b,h,q] = lse * log2(e), both with row pitch Sq_pad; the
// padding rows get delta = 0 and lse2 = +inf so that they produce P = 0 without a branch.
// (dO, O: [B*Sq, Hq, 128] contiguous; lse: [B,Hq,Sq])
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                      const float* __restrict__ lse, float* __restrict__ lse2,
                                      float* __restrict__ delta, int B, int Sq, int Sq_pad, int Hq) {
  // Sixteen lanes per (token, head) row of 128 values: one 16-byte load of dO and of O per lane, two rows
  // per lane in flight, four shuffle steps.  (One warp per row with 8-byte loads ran at a quarter of the
  // copy bandwidth.)
  const long long total = (long long)B * Sq * Hq;
  const int sub = threadIdx.x & 15;
  const long long stride = ((long long)gridDim.x * blockDim.x) >> 4;
  auto finish = [&](long long w, float s) {
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (sub == 0 && w < total) {
      const long long row = w / Hq;
      const int h = (int)(w % Hq);
      const long long b = row / Sq;
      const int q = (int)(row % Sq);
      delta[(b * Hq + h) * Sq_pad + q] = s;
      lse2[(b * Hq + h) * Sq_pad + q] = lse[(b * Hq + h) * Sq + q] * kLog2e;
    }
  };
  auto dot8 = [](const uint4& a, const uint4& c) {
    const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
    const float2 c0 = unpack_bf16(c.x), c1 = unpack_bf16(c.y), c2 = unpack_bf16(c.z), c3 = unpack_bf16(c.w);
    return (a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y) +
           (a2.x * c2.x + a2.y * c2.y + a3.x * c3.x + a3.y * c3.y);
  };
  // every lane of a warp runs the same number of iterations (the shuffles need the whole warp)
  const long long w_first = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 4;
  const long long warp_first = (blockIdx.x * (long long)blockDim.x + (threadIdx.x & ~31)) >> 4;
  for (long long base = warp_first, w = w_first; base < total; base += 2 * stride, w += 2 * stride) {
    const long long w2 = w + stride;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    const uint4 a = w < total ? reinterpret_cast<const uint4*>(dO + w * BWD_D)[sub] : zero;
    const uint4 c = w < total ? reinterpret_cast<const uint4*>(O + w * BWD_D)[sub] : zero;
    const uint4 a2 = w2 < total ? reinterpret_cast<const uint4*>(dO + w2 * BWD_D)[sub] : zero;
    const uint4 c2 = w2 < total ? reinterpret_cast<const uint4*>(O + w2 * BWD_D)[sub] : zero;
    finish(w, dot8(a, c));
    finish(w2, dot8(a2, c2));
  }
  const int pad = Sq_pad - Sq;
  const long long n_pad = (long long)B * Hq * pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_pad;
       i += (long long)gridDim.x * blockDim.x) {
    const long long bh = i / pad;
    const int q = Sq + (int)(i % pad);
    delta[bh * Sq_pad + q] = 0.f;
    lse2[bh * Sq_pad + q] = INFINITY;
  }
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Writes one fp32 TMEM accumulator row slice (64 columns starting at `col0`) times `mul` as bf16.
__device__ __forceinline__ void store_acc_row(uint32_t tsrc, int col0, __nv_bfloat16* dst, bool have, bool write,
                                              float mul) {
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t o[32];
    if (have) {
      tmem_ld32(tsrc + col0 + c * 32, o);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int e = 0; e < 32; ++e) o[e] = 0;
    }
    if (write) {
#pragma unroll
      for (int v = 0; v < 4; ++v)
        *reinterpret_cast<uint4*>(dst + col0 + c * 32 + v * 8) = make_uint4(
            pack_bf16(__uint_as_float(o[8 * v]) * mul, __uint_as_float(o[8 * v + 1]) * mul),
            pack_bf16(__uint_as_float(o[8 * v + 2]) * mul, __uint_as_float(o[8 * v + 3]) * mul),
            pack_bf16(__uint_as_float(o[8 * v + 4]) * mul, __uint_as_float(o[8 * v + 5]) * mul),
            pack_bf16(__uint_as_float(o[8 * v + 6]) * mul, __uint_as_float(o[8 * v + 7]) * mul));
    }
  }
}

// Elementwise product of two packed bf16 pairs (one HMUL2.BF16).
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// Operand tiles are [128 rows][128 d] in two 64-wide d blocks.  Descriptor low words (the high
// word kDescHi is common): K-major use, k-step k covers 16 d; MN-major use (N = d contiguous,
// K = rows), k-step k covers 16 rows.  The k-dependent part is a compile-time constant.
constexpr uint32_t kDescHi = smem_desc_hi(1024);
__device__ __forceinline__ uint32_t kmajor_lo(uint32_t tile) { return smem_desc_lo(tile, 16); }
__device__ __forceinline__ uint32_t mnmajor_lo(uint32_t tile) { return smem_desc_lo(tile, BWD_T * 128); }
__device__ __forceinline__ constexpr uint32_t kmajor_k(int k) { return (uint32_t)(((k >> 2) * (BWD_T * 128) + (k & 3) * 32) >> 4); }
__device__ __forceinline__ constexpr uint32_t mnmajor_k(int k) { return (uint32_t)((k * 2048) >> 4); }
// TMEM column (relative to the tile) where the bf16 A operand of k-step k lives: compute half
// k >> 2 packed its 64 results into the first 32 columns of its own 64-column range.
__device__ __forceinline__ uint32_t a_col(int k) { return (uint32_t)((k >> 2) * 64 + (k & 3) * 8); }

// ------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------
template <bool SOFTCAP>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const AttnBwdParams p) {
  using namespace dkv;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;                    // [KV_QSTAGES]
  uint64_t* q_empty = q_full + KV_QSTAGES;
  uint64_t* do_full = q_empty + KV_QSTAGES;       // [KV_DOSTAGES]
  uint64_t* do_empty = do_full + KV_DOSTAGES;
  uint64_t* s_full = do_empty + KV_DOSTAGES;      // S^T of a step is in TMEM
  uint64_t* p_full = s_full + 1;                  // count 256: P^T written
  uint64_t* dp_full = s_full + 2;
  uint64_t* ds_full = s_full + 3;                 // count 256: dS^T written
  uint64_t* acc_done = s_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
  int* tile_min = reinterpret_cast<int*>(smem + OFF_TILES);
  int* tile_max = tile_min + KV_MAX_TILES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // linear block id is key-block major so that under a causal mask the blocks with the most
  // visible query tiles (lowest key index) are scheduled first on every head
  const int kb = blockIdx.x / (p.Hkv * p.B);
  const int hkv = (blockIdx.x / p.B) % p.Hkv, b = blockIdx.x % p.B;
  const int G = p.Hq / p.Hkv;
  const int kv0 = kb * BWD_T;
  const int pos_off = p.Sk - p.Sq;
  const int n_tiles = (p.Sq + BWD_T - 1) / BWD_T;   // host guarantees <= KV_MAX_TILES

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < KV_QSTAGES; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < KV_DOSTAGES; ++i) { mbar_init(&do_full[i], 1); mbar_init(&do_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 256); mbar_init(dp_full, 1); mbar_init(ds_full, 256);
    mbar_init(acc_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // position range of every query tile (decides which tiles this key block can see)
  for (int t = threadIdx.x; t < n_tiles; t += BWD_THREADS) {
    const int r0 = t * BWD_T, r1 = min(p.Sq, r0 + BWD_T);
    int mn = 0x7fffffff, mx = -0x7fffffff;
    if (p.q_pos) {
      for (int r = r0; r < r1; ++r) {
        const int v = p.q_pos[(long long)b * p.Sq + r];
        mn = min(mn, v); mx = max(mx, v);
      }
    } else {
      mn = r0 + pos_off; mx = r1 - 1 + pos_off;
    }
    tile_min[t] = mn; tile_max[t] = mx;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto visible = [&](int t) -> bool {
    if (p.causal && tile_max[t] < kv0) return false;
    if (p.window > 0 && tile_min[t] - (kv0 + BWD_T - 1) >= p.window) return false;
    return true;
  };
  int n_vis = 0;
  for (int t = 0; t < n_tiles; ++t) n_vis += visible(t) ? 1 : 0;
  const int n_steps = n_vis * G;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (n_steps > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
        mbar_expect_tx(kv_full, 2 * TILE_BYTES);
        for (int c = 0; c < BWD_D / 64; ++c) {
          tma_load_3d(smem + OFF_K + c * (BWD_T * 128), &tmK, kv_full, c * 64, b * p.Sk + kv0, hkv);
          tma_load_3d(smem + OFF_V + c * (BWD_T * 128), &tmV, kv_full, c * 64, b * p.Sk + kv0, hkv);
        }
      }
      const bool aux_rows = p.q_pos != nullptr || p.q_seg != nullptr;
      int step = 0;
      bool ok = true;
      for (int g = 0; g < G && ok; ++g) {
        const int hq = hkv * G + g;
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (!visible(t)) continue;
          const int sq = step % KV_QSTAGES, sd = step % KV_DOSTAGES;
          const int q0 = t * BWD_T;
          int okw = 1;
          if (lane == 0)
            okw = mbar_wait(&q_empty[sq], ((step / KV_QSTAGES) & 1) ^ 1, p.status, kTimeoutStageFree, 21) ? 1 : 0;
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) { ok = false; break; }
          float* aux = reinterpret_cast<float*>(smem + OFF_AUX + sq * AUX_STAGE);
          int* auxi = reinterpret_cast<int*>(aux);
          if (aux_rows && !p.aux_bulk) {
            // rows that cannot be bulk-copied (unaligned sequence length): plain loads, made
            // visible to the consumers by the release of the arrive below
            for (int c = lane; c < BWD_T; c += 32) {
              const int r = min(q0 + c, p.Sq - 1);
              auxi[2 * BWD_T + c] = p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : 0;
              auxi[3 * BWD_T + c] = p.q_seg ? p.q_seg[(long long)b * p.Sq + r] : 0;
            }
            __syncwarp();
          }
          if (lane == 0) {
            const uint32_t rows_bytes = (uint32_t)min(BWD_T, p.Sq - q0) * 4u;
            uint32_t tx = TILE_BYTES + 2 * BWD_T * 4;
            if (aux_rows && p.aux_bulk) tx += (p.q_pos ? rows_bytes : 0u) + (p.q_seg ? rows_bytes : 0u);
            mbar_expect_tx(&q_full[sq], tx);
            for (int c = 0; c < BWD_D / 64; ++c)
              tma_load_3d(smem + OFF_Q + sq * TILE_BYTES + c * (BWD_T * 128), &tmQ, &q_full[sq], c * 64,
                          b * p.Sq + q0, hq);
            const long long li = ((long long)b * p.Hq + hq) * p.Sq_pad + q0;
            bulk_load(aux, p.lse2 + li, BWD_T * 4, &q_full[sq]);
            bulk_load(aux + BWD_T, p.delta + li, BWD_T * 4, &q_full[sq]);
            if (aux_rows && p.aux_bulk) {
              if (p.q_pos) bulk_load(auxi + 2 * BWD_T, p.q_pos + (long long)b * p.Sq + q0, rows_bytes, &q_full[sq]);
              if (p.q_seg) bulk_load(auxi + 3 * BWD_T, p.q_seg + (long long)b * p.Sq + q0, rows_bytes, &q_full[sq]);
            }
            if (mbar_wait(&do_empty[sd], ((step / KV_DOSTAGES) & 1) ^ 1, p.status, kTimeoutStageFree, 29)) {
              mbar_expect_tx(&do_full[sd], TILE_BYTES);
              for (int c = 0; c < BWD_D / 64; ++c)
                tma_load_3d(smem + OFF_DO + sd * TILE_BYTES + c * (BWD_T * 128), &tmdO, &do_full[sd], c * 64,
                            b * p.Sq + q0, hq);
            } else {
              okw = 0;
            }
          }
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) { ok = false; break; }
          ++step;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t id_s = make_idesc_bf16(BWD_T, BWD_T, false, false);    // S^T, dP^T
      constexpr uint32_t id_acc = make_idesc_bf16(BWD_T, BWD_D, false, true);   // dV, dK (A in TMEM, B MN-major)
      const uint32_t dK = kmajor_lo(smem_u32(smem + OFF_K)), dVd = kmajor_lo(smem_u32(smem + OFF_V));
      const uint32_t aQ0 = smem_u32(smem + OFF_Q), aDO0 = smem_u32(smem + OFF_DO);
      const uint32_t tS = tmem_base + T_S, tDP = tmem_base + T_DP;
      // The MMA queue is shallow, so whatever this thread does between two MMAs is tensor idle
      // time: every wait is therefore placed before the LAST MMA of the preceding group, where
      // its latency hides behind the seven MMAs still in flight.
      auto wait_q = [&](int i) { return mbar_wait(&q_full[i % KV_QSTAGES], (i / KV_QSTAGES) & 1, p.status, kTimeoutTmaFull, 23); };
      auto wait_do = [&](int i) { return mbar_wait(&do_full[i % KV_DOSTAGES], (i / KV_DOSTAGES) & 1, p.status, kTimeoutTmaFull, 24); };
      auto wait_p = [&](int i) { return mbar_wait(p_full, i & 1, p.status, kTimeoutSoftmax, 25); };
      auto wait_ds = [&](int i) { return mbar_wait(ds_full, i & 1, p.status, kTimeoutSoftmax, 26); };
      auto group = [&](auto&& mma, auto&& hook) -> bool {
#pragma unroll
        for (int k = 0; k < 7; ++k) mma(k);
        if (!hook()) return false;
        tc_fence_after();
        mma(7);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutTmaFull, 22) && wait_q(0);
      tc_fence_after();
      auto issue_s = [&](int i, auto&& hook) -> bool {      // S^T(i) = K Q(i)^T
        const uint32_t dQ = kmajor_lo(aQ0 + (i % KV_QSTAGES) * TILE_BYTES);
        if (!group([&](int k) { mma_ss_w(tS, dK + kmajor_k(k), kDescHi, dQ + kmajor_k(k), kDescHi, id_s, k != 0); }, hook))
          return false;
        tc_commit(s_full);
        return true;
      };
      auto issue_dp = [&](int i, auto&& hook) -> bool {     // dP^T(i) = V dO(i)^T
        const uint32_t dDO = kmajor_lo(aDO0 + (i % KV_DOSTAGES) * TILE_BYTES);
        if (!group([&](int k) { mma_ss_w(tDP, dVd + kmajor_k(k), kDescHi, dDO + kmajor_k(k), kDescHi, id_s, k != 0); }, hook))
          return false;
        tc_commit(dp_full);
        return true;
      };
      auto none = [] { return true; };
      if (ok) ok = issue_s(0, [&] { return wait_do(0); });
      if (ok) ok = issue_dp(0, none);
      for (int i = 0; i < n_steps && ok; ++i) {
        const uint32_t mQ = mnmajor_lo(aQ0 + (i % KV_QSTAGES) * TILE_BYTES);
        const uint32_t mDO = mnmajor_lo(aDO0 + (i % KV_DOSTAGES) * TILE_BYTES);
        const bool more = i + 1 < n_steps;
        // Waits on the compute warps stay where the data is needed: hooking them into the previous
        // group would hold back that group's commit, which the compute warps are waiting for.
        if (!wait_p(i)) break;
        tc_fence_after();
        // dV += P^T dO
        ok = group([&](int k) { mma_ts_w(tmem_base + T_DV, tS + a_col(k), mDO + mnmajor_k(k), kDescHi, id_acc, (i | k) != 0); },
                   [&] { return more ? wait_q(i + 1) : true; });
        if (!ok) break;
        tc_commit(&do_empty[i % KV_DOSTAGES]);
        if (more && !issue_s(i + 1, none)) break;
        if (!wait_ds(i)) break;
        tc_fence_after();
        // dK += dS^T Q
        ok = group([&](int k) { mma_ts_w(tmem_base + T_DK, tDP + a_col(k), mQ + mnmajor_k(k), kDescHi, id_acc, (i | k) != 0); },
                   [&] { return more ? wait_do(i + 1) : true; });
        if (!ok) break;
        tc_commit(&q_empty[i % KV_QSTAGES]);
        if (more && !issue_dp(i + 1, none)) break;
      }
      tc_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    // Warp w may touch TMEM lanes 32*(w%4)..+31, so warps w and w+4 share a lane quarter (the
    // same 32 key rows) and split the 128 query columns of a step between them.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;             // which 64 of the 128 query columns
    const int r_local = qd * 32 + lane;           // key row == TMEM lane
    const int kp = kv0 + r_local;                 // key position (keys are in natural order)
    const bool key_ok = kp < p.Sk;
    const int kseg = (p.kv_seg && key_ok) ? p.kv_seg[(long long)b * p.Sk + kp] : 0;
    const uint32_t tb = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t tS = tb + T_S + half * 64, tDP = tb + T_DP + half * 64;
    const int win = p.window > 0 ? p.window : 0x7fffffff;
    const int cmax = p.causal ? kp : -0x7fffffff;   // keep needs qp >= cmax
    bool ok = true;

    int step = 0;
    for (int g = 0; g < G && ok; ++g) {
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (!visible(t)) continue;
        const int sq = step % KV_QSTAGES;
        const float* aux = reinterpret_cast<const float*>(smem + OFF_AUX + sq * AUX_STAGE);
        const int* auxi = reinterpret_cast<const int*>(aux);
        const bool need_mask = !key_ok || (kv0 + BWD_T > p.Sk) || (p.causal && tile_min[t] < kv0 + BWD_T - 1) ||
                               (p.window > 0 && tile_max[t] - kv0 >= p.window) || p.q_seg != nullptr;
        // ---- phase 1: P^T = exp2(S^T * c - lse), kept packed for phase 2 and written over S^T
        if (!mbar_wait(s_full, step & 1, p.status, kTimeoutAccFull, 27)) { ok = false; break; }
        tc_fence_after();
        uint32_t pk_p[32];
        uint32_t pk_f[SOFTCAP ? 32 : 1];   // 1 - tanh^2 of the capped scores (the derivative of the cap)
        uint32_t sreg[64];
        tmem_ld32(tS, sreg);
        tmem_ld32(tS + 32, sreg + 32);
        tmem_wait_ld();
#pragma unroll
        for (int ch = 0; ch < 2; ++ch) {
          const uint32_t* s = sreg + ch * 32;
          const float4* lse4 = reinterpret_cast<const float4*>(aux + half * 64 + ch * 32);
          if (!need_mask) {
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              const float4 L = lse4[c4];
              float sv[4] = {__uint_as_float(s[4 * c4]), __uint_as_float(s[4 * c4 + 1]), __uint_as_float(s[4 * c4 + 2]),
                             __uint_as_float(s[4 * c4 + 3])};
              if (SOFTCAP) {
#pragma unroll
                for (int e = 0; e < 4; ++e) sv[e] = tanh_approx(sv[e] * p.softcap_in);
                pk_f[ch * 16 + 2 * c4] = pack_bf16(1.f - sv[0] * sv[0], 1.f - sv[1] * sv[1]);
                pk_f[ch * 16 + 2 * c4 + 1] = pack_bf16(1.f - sv[2] * sv[2], 1.f - sv[3] * sv[3]);
              }
              const float p0 = exp2f(fmaf(sv[0], p.scale_log2, -L.x));
              const float p1 = exp2f(fmaf(sv[1], p.scale_log2, -L.y));
              const float p2 = exp2f(fmaf(sv[2], p.scale_log2, -L.z));
              const float p3 = exp2f(fmaf(sv[3], p.scale_log2, -L.w));
              pk_p[ch * 16 + 2 * c4] = pack_bf16(p0, p1);
              pk_p[ch * 16 + 2 * c4 + 1] = pack_bf16(p2, p3);
            }
          } else {
            const int4* qp4 = reinterpret_cast<const int4*>(auxi + 2 * BWD_T + half * 64 + ch * 32);
            const int4* qs4 = reinterpret_cast<const int4*>(auxi + 3 * BWD_T + half * 64 + ch * 32);
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              const float4 L = lse4[c4];
              const int qn = t * BWD_T + pos_off + half * 64 + ch * 32 + 4 * c4;   // natural positions
              const int4 QP = p.q_pos ? qp4[c4] : make_int4(qn, qn + 1, qn + 2, qn + 3);
              const int4 QS = p.q_seg ? qs4[c4] : make_int4(0, 0, 0, 0);
              const float l[4] = {L.x, L.y, L.z, L.w};
              const int qp[4] = {QP.x, QP.y, QP.z, QP.w}, qs[4] = {QS.x, QS.y, QS.z, QS.w};
              float pv[4], fv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const bool keep = key_ok & (qp[e] >= cmax) & (qp[e] - kp < win) & (qs[e] == kseg);
                float sv = __uint_as_float(s[4 * c4 + e]);
                if (SOFTCAP) {
                  sv = tanh_approx(sv * p.softcap_in);
                  fv[e] = 1.f - sv * sv;
                }
                const float pe = exp2f(fmaf(sv, p.scale_log2, -l[e]));
                pv[e] = keep ? pe : 0.f;
              }
              if (SOFTCAP) {
                pk_f[ch * 16 + 2 * c4] = pack_bf16(fv[0], fv[1]);
                pk_f[ch * 16 + 2 * c4 + 1] = pack_bf16(fv[2], fv[3]);
              }
              pk_p[ch * 16 + 2 * c4] = pack_bf16(pv[0], pv[1]);
              pk_p[ch * 16 + 2 * c4 + 1] = pack_bf16(pv[2], pv[3]);
            }
          }
        }
        tmem_st32(tS, pk_p);
        if (SOFTCAP) {   // dV takes P^T as it is; dS^T takes P^T times the derivative of the cap
#pragma unroll
          for (int c = 0; c < 32; ++c) pk_p[c] = mul_bf16x2(pk_p[c], pk_f[c]);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(p_full);
        // ---- phase 2: dS^T = P^T o (dP^T - delta), written over dP^T
        if (!mbar_wait(dp_full, step & 1, p.status, kTimeoutAccFull, 28)) { ok = false; break; }
        tc_fence_after();
        {
          uint32_t dreg[64], pk_ds[32];
          tmem_ld32(tDP, dreg);
          tmem_ld32(tDP + 32, dreg + 32);
          tmem_wait_ld();
          const float4* dlt4 = reinterpret_cast<const float4*>(aux + BWD_T + half * 64);
#pragma unroll
          for (int c4 = 0; c4 < 16; ++c4) {
            const float4 Dl = dlt4[c4];
            pk_ds[2 * c4] = mul_bf16x2(pk_p[2 * c4], pack_bf16(__uint_as_float(dreg[4 * c4]) - Dl.x,
                                                               __uint_as_float(dreg[4 * c4 + 1]) - Dl.y));
            pk_ds[2 * c4 + 1] = mul_bf16x2(pk_p[2 * c4 + 1], pack_bf16(__uint_as_float(dreg[4 * c4 + 2]) - Dl.z,
                                                                       __uint_as_float(dreg[4 * c4 + 3]) - Dl.w));
          }
          // all 64 inputs of this warp are in registers, so its first 32 columns can be overwritten
          tmem_st32(tDP, pk_ds);
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(ds_full);
        ++step;
      }
    }
    // ---- dK / dV
    if (ok && n_steps > 0) ok = mbar_wait(acc_done, 0, p.status, kTimeoutAccFull, 28);
    tc_fence_after();
    const bool have = ok && n_steps > 0;
    store_acc_row(tb + T_DK, half * 64, p.dK + ((long long)b * p.Sk + kp) * p.lddk + (long long)hkv * BWD_D, have,
                  key_ok, p.scale);
    store_acc_row(tb + T_DV, half * 64, p.dV + ((long long)b * p.Sk + kp) * p.lddv + (long long)hkv * BWD_D, have,
                  key_ok, 1.f);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------
template <bool SOFTCAP>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const AttnBwdParams p) {
  using namespace dqk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* qdo_full = bars;
  uint64_t* k_full = bars + 1;                    // [DQ_KSTAGES]
  uint64_t* k_empty = k_full + DQ_KSTAGES;
  uint64_t* v_full = k_empty + DQ_KSTAGES;        // [DQ_VSTAGES]
  uint64_t* v_empty = v_full + DQ_VSTAGES;
  uint64_t* s_full = v_empty + DQ_VSTAGES;        // [2]
  uint64_t* dp_full = s_full + 2;
  uint64_t* ds_full = s_full + 3;                 // count 256
  uint64_t* acc_done = s_full + 4;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 5);
  int* tile_minmax = reinterpret_cast<int*>(s_full + 6);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (p.Sq + BWD_T - 1) / BWD_T;
  // heaviest (latest) query tiles first under a causal mask
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (p.Hq * p.B));
  const int hq = (blockIdx.x / p.B) % p.Hq, b = blockIdx.x % p.B;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = qt * BWD_T;
  const int pos_off = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < DQ_KSTAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < DQ_VSTAGES; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(dp_full, 1); mbar_init(ds_full, 256);
    mbar_init(acc_done, 1);
    tile_minmax[0] = 0x7fffffff;
    tile_minmax[1] = -0x7fffffff;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (threadIdx.x < BWD_T) {
    const int r = q0 + threadIdx.x;
    if (r < p.Sq) {
      const int qp = p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : r + pos_off;
      atomicMin(&tile_minmax[0], qp);
      atomicMax(&tile_minmax[1], qp);
    }
  }
  __syncthreads();
  const int qpos_min = tile_minmax[0], qpos_max = tile_minmax[1];
  const int nblk_total = (p.Sk + BWD_T - 1) / BWD_T;
  int blk_hi = p.causal ? min(nblk_total, qpos_max / BWD_T + 1) : nblk_total;
  int blk_lo = (p.window > 0) ? max(0, (qpos_min - p.window + 1) / BWD_T) : 0;
  if (qpos_max < 0) blk_hi = 0;
  const int nblk = max(0, blk_hi - blk_lo);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      mbar_expect_tx(qdo_full, 2 * TILE_BYTES);
#pragma unroll
      for (int c = 0; c < BWD_D / 64; ++c) {
        tma_load_3d(smem + OFF_Q + c * (BWD_T * 128), &tmQ, qdo_full, c * 64, b * p.Sq + q0, hq);
        tma_load_3d(smem + OFF_DO + c * (BWD_T * 128), &tmdO, qdo_full, c * 64, b * p.Sq + q0, hq);
      }
      for (int j = 0; j < nblk; ++j) {
        const int sk = j % DQ_KSTAGES, sv = j % DQ_VSTAGES;
        const int row = b * p.Sk + (blk_lo + j) * BWD_T;
        if (!mbar_wait(&k_empty[sk], ((j / DQ_KSTAGES) & 1) ^ 1, p.status, kTimeoutStageFree, 31)) break;
        mbar_expect_tx(&k_full[sk], TILE_BYTES);
#pragma unroll
        for (int c = 0; c < BWD_D / 64; ++c)
          tma_load_3d(smem + OFF_K + sk * TILE_BYTES + c * (BWD_T * 128), &tmK, &k_full[sk], c * 64, row, hkv);
        if (!mbar_wait(&v_empty[sv], ((j / DQ_VSTAGES) & 1) ^ 1, p.status, kTimeoutStageFree, 35)) break;
        mbar_expect_tx(&v_full[sv], TILE_BYTES);
#pragma unroll
        for (int c = 0; c < BWD_D / 64; ++c)
          tma_load_3d(smem + OFF_V + sv * TILE_BYTES + c * (BWD_T * 128), &tmV, &v_full[sv], c * 64, row, hkv);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t id_s = make_idesc_bf16(BWD_T, BWD_T, false, false);    // S, dP
      constexpr uint32_t id_dq = make_idesc_bf16(BWD_T, BWD_D, false, true);    // dQ (A in TMEM, B MN-major)
      const uint32_t dQ = kmajor_lo(smem_u32(smem + OFF_Q)), dDO = kmajor_lo(smem_u32(smem + OFF_DO));
      const uint32_t aK0 = smem_u32(smem + OFF_K), aV0 = smem_u32(smem + OFF_V);
      const uint32_t tDP = tmem_base + T_DP;
      // Waits sit before the last MMA of the preceding group (see the dK/dV kernel).
      auto wait_k = [&](int j) { return mbar_wait(&k_full[j % DQ_KSTAGES], (j / DQ_KSTAGES) & 1, p.status, kTimeoutTmaFull, 33); };
      auto wait_v = [&](int j) { return mbar_wait(&v_full[j % DQ_VSTAGES], (j / DQ_VSTAGES) & 1, p.status, kTimeoutTmaFull, 37); };
      auto wait_ds = [&](int j) { return mbar_wait(ds_full, j & 1, p.status, kTimeoutSoftmax, 34); };
      auto group = [&](auto&& mma, auto&& hook) -> bool {
#pragma unroll
        for (int k = 0; k < 7; ++k) mma(k);
        if (!hook()) return false;
        tc_fence_after();
        mma(7);
        return true;
      };
      bool ok = mbar_wait(qdo_full, 0, p.status, kTimeoutTmaFull, 32) && wait_k(0);
      tc_fence_after();
      auto issue_s = [&](int j, auto&& hook) -> bool {      // S(j) = Q K_j^T
        const uint32_t dK = kmajor_lo(aK0 + (j % DQ_KSTAGES) * TILE_BYTES);
        const uint32_t tS = tmem_base + T_S + (j & 1) * BWD_T;
        if (!group([&](int k) { mma_ss_w(tS, dQ + kmajor_k(k), kDescHi, dK + kmajor_k(k), kDescHi, id_s, k != 0); }, hook))
          return false;
        tc_commit(&s_full[j & 1]);
        return true;
      };
      auto issue_dp = [&](int j, auto&& hook) -> bool {     // dP(j) = dO V_j^T
        const uint32_t dV = kmajor_lo(aV0 + (j % DQ_VSTAGES) * TILE_BYTES);
        if (!group([&](int k) { mma_ss_w(tDP, dDO + kmajor_k(k), kDescHi, dV + kmajor_k(k), kDescHi, id_s, k != 0); }, hook))
          return false;
        tc_commit(&v_empty[j % DQ_VSTAGES]);
        tc_commit(dp_full);
        return true;
      };
      auto none = [] { return true; };
      if (ok) ok = issue_s(0, [&] { return wait_v(0); });
      if (ok) ok = issue_dp(0, [&] { return nblk > 1 ? wait_k(1) : true; });
      for (int j = 0; j < nblk && ok; ++j) {
        const bool more = j + 1 < nblk;
        if (more && !issue_s(j + 1, none)) break;
        if (!wait_ds(j)) break;   // not hooked into S(j+1): that would hold back its commit
        tc_fence_after();
        const uint32_t mK = mnmajor_lo(aK0 + (j % DQ_KSTAGES) * TILE_BYTES);
        // dQ += dS K   (K tile [128 keys][128 d]: N = d contiguous)
        ok = group([&](int k) { mma_ts_w(tmem_base + T_DQ, tDP + a_col(k), mK + mnmajor_k(k), kDescHi, id_dq, (j | k) != 0); },
                   [&] { return more ? wait_v(j + 1) : true; });
        if (!ok) break;
        tc_commit(&k_empty[j % DQ_KSTAGES]);
        if (more && !issue_dp(j + 1, [&] { return j + 2 < nblk ? wait_k(j + 2) : true; })) break;
      }
      tc_commit(acc_done);
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;             // which 64 of the 128 key columns
    const int r_local = qd * 32 + lane;           // query row == TMEM lane
    const int row = q0 + r_local;
    const bool row_ok = row < p.Sq;
    const long long grow = (long long)b * p.Sq + row;
    const int qpos = row_ok ? (p.q_pos ? p.q_pos[grow] : row + pos_off) : -1;
    const int qseg = (p.q_seg && row_ok) ? p.q_seg[grow] : 0;
    const long long li = ((long long)b * p.Hq + hq) * p.Sq_pad + row;   // row < Sq_pad: padded to 128
    const float lse2 = p.lse2[li];
    const float delta = p.delta[li];
    const uint32_t tb = tmem_base + ((uint32_t)(qd * 32) << 16);
    const uint32_t tDP = tb + T_DP + half * 64;
    const int* ks = p.kv_seg ? p.kv_seg + (long long)b * p.Sk : nullptr;
    const int win = p.window > 0 ? p.window : 0x7fffffff;
    const int kmax = p.causal ? min(qpos, p.Sk - 1) : p.Sk - 1;   // keep needs kp <= kmax
    bool ok = true;

    for (int j = 0; j < nblk && ok; ++j) {
      const int kv0 = (blk_lo + j) * BWD_T;
      const bool need_mask = (p.causal && kv0 + BWD_T - 1 > qpos_min) || (kv0 + BWD_T > p.Sk) ||
                             (p.window > 0 && qpos_max - kv0 >= p.window) || p.q_seg != nullptr;
      const uint32_t tS = tb + T_S + (j & 1) * BWD_T + half * 64;
      // ---- phase 1: P = exp2(S * c - lse), packed bf16 in registers
      if (!mbar_wait(&s_full[j & 1], (j >> 1) & 1, p.status, kTimeoutAccFull, 36)) { ok = false; break; }
      tc_fence_after();
      uint32_t pk_p[32];
      uint32_t sreg[64];
      tmem_ld32(tS, sreg);
      tmem_ld32(tS + 32, sreg + 32);
      tmem_wait_ld();
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        const uint32_t* s = sreg + ch * 32;
        if (!need_mask) {
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float s0 = __uint_as_float(s[c]), s1 = __uint_as_float(s[c + 1]), f0 = 1.f, f1 = 1.f;
            if (SOFTCAP) {   // P only feeds dS here, so the derivative of the cap is folded into it
              s0 = tanh_approx(s0 * p.softcap_in);
              s1 = tanh_approx(s1 * p.softcap_in);
              f0 = 1.f - s0 * s0;
              f1 = 1.f - s1 * s1;
            }
            pk_p[ch * 16 + c / 2] = pack_bf16(f0 * exp2f(fmaf(s0, p.scale_log2, -lse2)),
                                              f1 * exp2f(fmaf(s1, p.scale_log2, -lse2)));
          }
        } else {
          const int kbase = kv0 + half * 64 + ch * 32;
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float pv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kp = kbase + c + e;
              bool keep = (kp <= kmax) & (qpos - kp < win);
              if (ks) keep = keep & (__ldg(ks + min(kp, p.Sk - 1)) == qseg);
              float sv = __uint_as_float(s[c + e]), fv = 1.f;
              if (SOFTCAP) {
                sv = tanh_approx(sv * p.softcap_in);
                fv = 1.f - sv * sv;
              }
              const float pe = fv * exp2f(fmaf(sv, p.scale_log2, -lse2));
              pv[e] = keep ? pe : 0.f;
            }
            pk_p[ch * 16 + c / 2] = pack_bf16(pv[0], pv[1]);
          }
        }
      }
      // ---- phase 2: dS = P o (dP - delta), written over dP
      if (!mbar_wait(dp_full, j & 1, p.status, kTimeoutAccFull, 39)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t dreg[64], pk[32];
        tmem_ld32(tDP, dreg);
        tmem_ld32(tDP + 32, dreg + 32);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c)
          pk[c] = mul_bf16x2(pk_p[c], pack_bf16(__uint_as_float(dreg[2 * c]) - delta,
                                                __uint_as_float(dreg[2 * c + 1]) - delta));
        tmem_st32(tDP, pk);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(ds_full);
    }
    if (ok && nblk > 0) ok = mbar_wait(acc_done, 0, p.status, kTimeoutAccFull, 38);
    tc_fence_after();
    store_acc_row(tb + T_DQ, half * 64, p.dQ + grow * p.lddq + (long long)hq * BWD_D, ok && nblk > 0, row_ok,
                  p.scale);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace tpb

using namespace tpb;


// Floats of scratch `tpb_attn_bwd` needs (scaled log-sum-exp and delta rows, padded to 128).
extern "C" long long tpb_attn_bwd_scratch_floats(int B, int Sq, int Hq) {
  const long long sq_pad = (Sq + BWD_T - 1) / BWD_T * BWD_T;
  return 2LL * B * Hq * sq_pad;
}

// `softcap` > 0: the scores were capped as softcap * tanh(q.k * scale / softcap) in the forward pass.
extern "C" int tpb_attn_bwd_softcap(const void* dO, const void* q, const void* k, const void* v, const void* o,
                                    const float* lse, float* scratch, void* dq, void* dk, void* dv, int B, int Sq,
                                    int Sk, int Hq, int Hkv, int dqk, int dvd, long long ldq, long long ldk,
                                    long long ldv, long long lddo, long long lddq, long long lddk, long long lddv,
                                    float scale, int causal, int window, const int* q_pos, const int* q_seg,
                                    const int* kv_seg, float softcap, void* stream_) {
  if (dqk != 128 || dvd != 128 || Hq % Hkv) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -2;
  if (lddo != (long long)Hq * dvd) return -2;   // dO and O are contiguous [B*Sq, Hq, 128]
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if ((Sq + BWD_T - 1) / BWD_T > KV_MAX_TILES) return -6;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int sq_pad = (Sq + BWD_T - 1) / BWD_T * BWD_T;
  float* lse2 = scratch;
  float* delta = scratch + (long long)B * Hq * sq_pad;
  {
    const long long warps = (long long)B * Sq * Hq;
    long long blocks = (warps * 32 + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    attn_bwd_delta_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dO),
                                                           reinterpret_cast<const __nv_bfloat16*>(o), lse, lse2, delta,
                                                           B, Sq, sq_pad, Hq);
  }
  AttnBwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale;
  p.softcap_in = softcap > 0.f ? scale / softcap : 0.f;
  p.scale_log2 = (softcap > 0.f ? softcap : scale) * kLog2e;
  p.causal = causal; p.window = window;
  p.q_pos = q_pos; p.q_seg = q_seg; p.kv_seg = kv_seg;
  p.lse2 = lse2; p.delta = delta; p.Sq_pad = sq_pad;
  p.aux_bulk = (Sq % 4 == 0) && (reinterpret_cast<uintptr_t>(q_pos) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(q_seg) % 16 == 0);
  p.dQ = reinterpret_cast<__nv_bfloat16*>(dq); p.lddq = lddq;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.lddk = lddk;
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv); p.lddv = lddv;
  p.status = status_block();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd_dq_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dqk::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd_dkv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd_dq_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dqk::TOTAL);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  // every operand is streamed as 128-row tiles in two 64-wide d blocks
  CUtensorMap tq, tk, tv, tdo;
  if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, BWD_T)) return -3;
  if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, BWD_T)) return -4;
  if (make_tmap_3d(&tv, v, dvd, (uint64_t)B * Sk, Hkv, ldv, dvd, 64, BWD_T)) return -5;
  if (make_tmap_3d(&tdo, dO, dvd, (uint64_t)B * Sq, Hq, lddo, dvd, 64, BWD_T)) return -5;
  dim3 grid_kv(((Sk + BWD_T - 1) / BWD_T) * Hkv * B, 1, 1);
  if (softcap > 0.f) attn_bwd_dkv_kernel<true><<<grid_kv, BWD_THREADS, dkv::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  else attn_bwd_dkv_kernel<false><<<grid_kv, BWD_THREADS, dkv::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return 1000 + (int)e;
  dim3 grid_q(((Sq + BWD_T - 1) / BWD_T) * Hq * B, 1, 1);
  if (softcap > 0.f) attn_bwd_dq_kernel<true><<<grid_q, BWD_THREADS, dqk::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  else attn_bwd_dq_kernel<false><<<grid_q, BWD_THREADS, dqk::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

extern "C" int tpb_attn_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o,
                            const float* lse, float* scratch, void* dq, void* dk, void* dv, int B, int Sq,
                            int Sk, int Hq, int Hkv, int dqk, int dvd, long long ldq, long long ldk, long long ldv,
                            long long lddo, long long lddq, long long lddk, long long lddv, float scale, int causal,
                            int window, const int* q_pos, const int* q_seg, const int* kv_seg, void* stream_) {
  return tpb_attn_bwd_softcap(dO, q, k, v, o, lse, scratch, dq, dk, dv, B, Sq, Sk, Hq, Hkv, dqk, dvd, ldq, ldk, ldv, lddo,
                              lddq, lddk, lddv, scale, causal, window, q_pos, q_seg, kv_seg, 0.f, stream_);
}
