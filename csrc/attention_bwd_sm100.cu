// Flash-attention backward for sm_100a (tcgen05 + TMEM + TMA), GQA-native, head dim 128.
//
// Two tensor-core kernels, neither of which needs atomics or a cross-CTA reduction:
//
//  attn_bwd_dkv_kernel   one CTA per (128-key block, kv head, batch).  K and V of the block
//      stay in shared memory; dK and dV accumulate in TMEM over every 64-row query tile and
//      every query head of the GQA group that can see the block.  Computed in the transposed
//      frame (TMEM lane = key row):
//        S^T  = K Q^T   (SS) 128x64 fp32      dP^T = V dO^T   (SS) 128x64 fp32
//        P^T  = exp2(S^T*c - lse), dS^T = P^T o (dP^T - delta)   (registers; the softmax scale
//                                                               is applied to dK in the epilogue)
//        dV  += P^T dO  (TS, A = bf16 P^T  written over the S^T columns)
//        dK  += dS^T Q  (TS, A = bf16 dS^T written over the dP^T columns)
//      TMEM: dK [0,128), dV [128,256), two score buffers {S^T, dP^T} at [256,384), [384,512).
//
//  attn_bwd_dq_kernel    one CTA per (128-row query tile, query head, batch), the mirror
//      image of the forward kernel (TMEM lane = query row):
//        S  = Q K^T     (SS) 128x64 fp32      dP = dO V^T     (SS) 128x64 fp32
//        dS = exp2(S*c - lse) o (dP - delta)                      (scale applied to dQ at the end)
//        dQ += dS K     (TS, A = bf16 dS written over the dP columns, B = K tile MN-major)
//      TMEM: dQ [0,128), two score buffers at [128,256), [256,384).
//
// Both kernels: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9 compute.  Warps w and w+4
// share a TMEM lane quarter and split the 64 score columns of a step; each writes its bf16
// result over the first half of its OWN 32 input columns, so the two never touch each other's
// columns and the A operand of the following MMA is simply addressed per 16-column k-step.
// The score buffers are double buffered: the MMA warp issues the scores of step i+1 before it
// waits for the compute warps of step i, so tensor core and compute warps overlap.

#include <cstdlib>

#include "common.cuh"
#include "tpb.h"

namespace tpb {

int make_tmap_3d(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                 uint64_t stride2_elems, uint32_t box0, uint32_t box1);
int sm_count();

constexpr int BWD_D = 128;
constexpr int BWD_THREADS = 320;   // TMA warp, MMA warp, 8 compute warps
constexpr int KV_STAGES = 4;       // dK/dV kernel: depth of the Q/dO tile ring
constexpr int DQ_KSTAGES = 5;      // dQ kernel: depth of the K tile ring (a K tile is held for two steps)
constexpr int DQ_VSTAGES = 4;      // dQ kernel: depth of the V tile ring
constexpr float kLog2e = 1.4426950408889634f;

// dK/dV kernel tiles
constexpr int KV_BK = 128;         // keys per CTA
constexpr int KV_BQ = 64;          // query rows per step
constexpr int KV_MAX_TILES = 512;  // query tiles whose position range fits the shared-memory table
// dQ kernel tiles
constexpr int DQ_BM = 128;         // query rows per CTA
constexpr int DQ_BN = 64;          // keys per step

struct AttnBwdParams {
  int B, Sq, Sk, Hq, Hkv;
  float scale, scale_log2;
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
  long long* prof;   // optional cycle counters (see tpb_attn_bwd_set_prof), normally null
};

namespace dkv {
constexpr int K_BYTES = KV_BK * BWD_D * 2;       // 32 KB
constexpr int V_BYTES = KV_BK * BWD_D * 2;       // 32 KB
constexpr int Q_BYTES = KV_BQ * BWD_D * 2;       // 16 KB
constexpr int DO_BYTES = KV_BQ * BWD_D * 2;      // 16 KB
constexpr int OFF_K = 0;
constexpr int OFF_V = OFF_K + K_BYTES;
constexpr int OFF_Q = OFF_V + V_BYTES;
constexpr int OFF_DO = OFF_Q + KV_STAGES * Q_BYTES;
constexpr int OFF_AUX = OFF_DO + KV_STAGES * DO_BYTES;   // per stage: lse2[64], delta[64], qpos[64], qseg[64]
constexpr int AUX_STAGE = 4 * KV_BQ * 4;
constexpr int OFF_TILES = OFF_AUX + KV_STAGES * AUX_STAGE;  // tile min/max table: 2 * KV_MAX_TILES ints
constexpr int OFF_BAR = OFF_TILES + 2 * KV_MAX_TILES * 4;
constexpr int TOTAL = OFF_BAR + 256 + 1024;
// TMEM columns; score buffer i holds S^T at T_BUF + 128*i and dP^T 64 columns further
constexpr int T_DK = 0, T_DV = 128, T_BUF = 256;
}  // namespace dkv

namespace dqk {
constexpr int Q_BYTES = DQ_BM * BWD_D * 2;       // 32 KB
constexpr int DO_BYTES = DQ_BM * BWD_D * 2;      // 32 KB
constexpr int K_BYTES = DQ_BN * BWD_D * 2;       // 16 KB
constexpr int V_BYTES = DQ_BN * BWD_D * 2;       // 16 KB
constexpr int OFF_Q = 0;
constexpr int OFF_DO = OFF_Q + Q_BYTES;
constexpr int OFF_K = OFF_DO + DO_BYTES;
constexpr int OFF_V = OFF_K + DQ_KSTAGES * K_BYTES;
constexpr int OFF_BAR = OFF_V + DQ_VSTAGES * V_BYTES;
constexpr int TOTAL = OFF_BAR + 256 + 1024;
constexpr int T_DQ = 0, T_BUF = 128;
}  // namespace dqk

// delta[b,h,q] = sum_d dO * O and lse2[b,h,q] = lse * log2(e), both with row pitch Sq_pad; the
// padding rows get delta = 0 and lse2 = +inf so that they produce P = 0 without a branch.
// (dO, O: [B*Sq, Hq, 128] contiguous; lse: [B,Hq,Sq])
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                      const float* __restrict__ lse, float* __restrict__ lse2,
                                      float* __restrict__ delta, int B, int Sq, int Sq_pad, int Hq) {
  const long long total = (long long)B * Sq * Hq;
  const int lane = threadIdx.x & 31;
  for (long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; w < total;
       w += ((long long)gridDim.x * blockDim.x) >> 5) {
    const uint2 a = reinterpret_cast<const uint2*>(dO + w * BWD_D)[lane];
    const uint2 c = reinterpret_cast<const uint2*>(O + w * BWD_D)[lane];
    float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), c0 = unpack_bf16(c.x), c1 = unpack_bf16(c.y);
    float s = a0.x * c0.x + a0.y * c0.y + a1.x * c1.x + a1.y * c1.y;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
      const long long row = w / Hq;
      const int h = (int)(w % Hq);
      const long long b = row / Sq;
      const int q = (int)(row % Sq);
      delta[(b * Hq + h) * Sq_pad + q] = s;
      lse2[(b * Hq + h) * Sq_pad + q] = lse[(b * Hq + h) * Sq + q] * kLog2e;
    }
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

// ------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                    const AttnBwdParams p) {
  using namespace dkv;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;                  // [KV_STAGES]
  uint64_t* qdo_empty = qdo_full + KV_STAGES;     // [KV_STAGES]
  uint64_t* sdp_full = qdo_empty + KV_STAGES;     // [2] scores of a buffer are in TMEM
  uint64_t* pds_full = sdp_full + 2;              // [2] count 256: P^T / dS^T of a buffer are in TMEM
  uint64_t* acc_done = pds_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  int* tile_min = reinterpret_cast<int*>(smem + OFF_TILES);
  int* tile_max = tile_min + KV_MAX_TILES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // linear block id is key-block major so that under a causal mask the blocks with the most
  // visible query tiles (lowest key index) are scheduled first on every head
  const int kb = blockIdx.x / (p.Hkv * p.B);
  const int hkv = (blockIdx.x / p.B) % p.Hkv, b = blockIdx.x % p.B;
  const int G = p.Hq / p.Hkv;
  const int kv0 = kb * KV_BK;
  const int pos_off = p.Sk - p.Sq;
  const int n_tiles = (p.Sq + KV_BQ - 1) / KV_BQ;   // host guarantees <= KV_MAX_TILES

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < KV_STAGES; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&pds_full[i], 256); }
    mbar_init(acc_done, 1);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // position range of every query tile (decides which tiles this key block can see)
  for (int t = threadIdx.x; t < n_tiles; t += BWD_THREADS) {
    const int r0 = t * KV_BQ, r1 = min(p.Sq, r0 + KV_BQ);
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
    if (p.window > 0 && tile_min[t] - (kv0 + KV_BK - 1) >= p.window) return false;
    return true;
  };
  int n_vis = 0;
  for (int t = 0; t < n_tiles; ++t) n_vis += visible(t) ? 1 : 0;
  const int n_steps = n_vis * G;

  uint8_t* sK = smem + OFF_K;
  uint8_t* sV = smem + OFF_V;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (n_steps > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
        mbar_expect_tx(kv_full, K_BYTES + V_BYTES);
        for (int c = 0; c < BWD_D / 64; ++c) {
          tma_load_3d(sK + c * (KV_BK * 128), &tmK, kv_full, c * 64, b * p.Sk + kv0, hkv);
          tma_load_3d(sV + c * (KV_BK * 128), &tmV, kv_full, c * 64, b * p.Sk + kv0, hkv);
        }
      }
      int step = 0;
      bool ok = true;
      for (int g = 0; g < G && ok; ++g) {
        const int hq = hkv * G + g;
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (!visible(t)) continue;
          const int st = step % KV_STAGES;
          const uint32_t ph = (step / KV_STAGES) & 1;
          int okw = 1;
          if (lane == 0) okw = mbar_wait(&qdo_empty[st], ph ^ 1, p.status, kTimeoutStageFree, 21) ? 1 : 0;
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) { ok = false; break; }
          const int q0 = t * KV_BQ;
          float* aux = reinterpret_cast<float*>(smem + OFF_AUX + st * AUX_STAGE);
          int* auxi = reinterpret_cast<int*>(aux);
          const bool aux_rows = p.q_pos != nullptr || p.q_seg != nullptr;
          if (aux_rows && !p.aux_bulk) {
            // rows that cannot be bulk-copied (unaligned sequence length): plain loads, made
            // visible to the consumers by the release of the arrive below
            for (int c = lane; c < KV_BQ; c += 32) {
              const int r = min(q0 + c, p.Sq - 1);
              auxi[2 * KV_BQ + c] = p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : 0;
              auxi[3 * KV_BQ + c] = p.q_seg ? p.q_seg[(long long)b * p.Sq + r] : 0;
            }
            __syncwarp();
          }
          if (lane == 0) {
            const uint32_t rows_bytes = (uint32_t)min(KV_BQ, p.Sq - q0) * 4u;
            uint32_t tx = Q_BYTES + DO_BYTES + 2 * KV_BQ * 4;
            if (aux_rows && p.aux_bulk) tx += (p.q_pos ? rows_bytes : 0u) + (p.q_seg ? rows_bytes : 0u);
            mbar_expect_tx(&qdo_full[st], tx);
            for (int c = 0; c < BWD_D / 64; ++c) {
              tma_load_3d(smem + OFF_Q + st * Q_BYTES + c * (KV_BQ * 128), &tmQ, &qdo_full[st], c * 64,
                          b * p.Sq + q0, hq);
              tma_load_3d(smem + OFF_DO + st * DO_BYTES + c * (KV_BQ * 128), &tmdO, &qdo_full[st], c * 64,
                          b * p.Sq + q0, hq);
            }
            const long long li = ((long long)b * p.Hq + hq) * p.Sq_pad + q0;
            bulk_load(aux, p.lse2 + li, KV_BQ * 4, &qdo_full[st]);
            bulk_load(aux + KV_BQ, p.delta + li, KV_BQ * 4, &qdo_full[st]);
            if (aux_rows && p.aux_bulk) {
              if (p.q_pos) bulk_load(auxi + 2 * KV_BQ, p.q_pos + (long long)b * p.Sq + q0, rows_bytes, &qdo_full[st]);
              if (p.q_seg) bulk_load(auxi + 3 * KV_BQ, p.q_seg + (long long)b * p.Sq + q0, rows_bytes, &qdo_full[st]);
            }
          }
          ++step;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t id_s = make_idesc_bf16(KV_BK, KV_BQ, false, false);    // S^T, dP^T
      constexpr uint32_t id_acc = make_idesc_bf16(KV_BK, BWD_D, false, true);   // dV, dK (A in TMEM, B MN-major)
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutTmaFull, 22);
      auto issue_scores = [&](int step) -> bool {
        const int st = step % KV_STAGES;
        if (!mbar_wait(&qdo_full[st], (step / KV_STAGES) & 1, p.status, kTimeoutTmaFull, 23)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(smem + OFF_Q + st * Q_BYTES), aDO = smem_u32(smem + OFF_DO + st * DO_BYTES);
        const uint32_t tS = tmem_base + T_BUF + (step & 1) * 128;
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t ad = make_smem_desc(aK + (k >> 2) * (KV_BK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aQ + (k >> 2) * (KV_BQ * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tS, ad, bd, id_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t ad = make_smem_desc(aV + (k >> 2) * (KV_BK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aDO + (k >> 2) * (KV_BQ * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tS + 64, ad, bd, id_s, k != 0);
        }
        tc_commit(&sdp_full[step & 1]);
        return true;
      };
      const bool prof = p.prof != nullptr;
      long long m_tiles = 0, m_ds = 0, t0 = 0, t1 = 0;
      const long long m_start = prof ? clock64() : 0;
      if (ok) ok = issue_scores(0);
      for (int step = 0; step < n_steps && ok; ++step) {
        const int st = step % KV_STAGES;
        // The other buffer is free: its P^T / dS^T were consumed by MMAs issued one iteration ago.
        if (prof) t0 = clock64();
        if (step + 1 < n_steps) {
          if (!issue_scores(step + 1)) break;
        }
        if (prof) { t1 = clock64(); m_tiles += t1 - t0; }
        if (!mbar_wait(&pds_full[step & 1], (step >> 1) & 1, p.status, kTimeoutSoftmax, 24)) break;
        tc_fence_after();
        if (prof) m_ds += clock64() - t1;
        const uint32_t aQ = smem_u32(smem + OFF_Q + st * Q_BYTES), aDO = smem_u32(smem + OFF_DO + st * DO_BYTES);
        const uint32_t tP = tmem_base + T_BUF + (step & 1) * 128, tDS = tP + 64;
        // k-step k covers query columns 16k..16k+15; half k>>1 wrote them at column 32*(k>>1) + 8*(k&1)
#pragma unroll
        for (int k = 0; k < KV_BQ / 16; ++k) {   // dV += P^T dO
          const uint64_t bd = make_smem_desc(aDO + k * 2048, KV_BQ * 128, 1024);
          mma_ts(tmem_base + T_DV, tP + (k >> 1) * 32 + (k & 1) * 8, bd, id_acc, (step | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < KV_BQ / 16; ++k) {   // dK += dS^T Q
          const uint64_t bd = make_smem_desc(aQ + k * 2048, KV_BQ * 128, 1024);
          mma_ts(tmem_base + T_DK, tDS + (k >> 1) * 32 + (k & 1) * 8, bd, id_acc, (step | k) != 0);
        }
        tc_commit(&qdo_empty[st]);
      }
      tc_commit(acc_done);
      if (prof) {
        atomicAdd((unsigned long long*)p.prof + 5, (unsigned long long)m_tiles);
        atomicAdd((unsigned long long*)p.prof + 6, (unsigned long long)m_ds);
        atomicAdd((unsigned long long*)p.prof + 7, (unsigned long long)(clock64() - m_start));
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    // Warp w may touch TMEM lanes 32*(w%4)..+31, so warps w and w+4 share a lane quarter (the
    // same 32 key rows) and split the 64 query columns of a step between them.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;             // which 32 of the 64 query columns
    const int r_local = qd * 32 + lane;           // key row == TMEM lane
    const int kp = kv0 + r_local;                 // key position (keys are in natural order)
    const bool key_ok = kp < p.Sk;
    const int kseg = (p.kv_seg && key_ok) ? p.kv_seg[(long long)b * p.Sk + kp] : 0;
    const uint32_t tb = tmem_base + ((uint32_t)(qd * 32) << 16);
    bool ok = true;

    const bool prof = p.prof != nullptr && threadIdx.x == 64;
    long long c_wait = 0, c_ld = 0, c_math = 0, c_st = 0, t0 = 0, t1 = 0;
    int step = 0;
    for (int g = 0; g < G && ok; ++g) {
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (!visible(t)) continue;
        const int st = step % KV_STAGES;
        const int buf = step & 1;
        if (prof) t0 = clock64();
        if (!mbar_wait(&sdp_full[buf], (step >> 1) & 1, p.status, kTimeoutAccFull, 26)) { ok = false; break; }
        tc_fence_after();
        if (prof) { t1 = clock64(); c_wait += t1 - t0; }
        const float* aux = reinterpret_cast<const float*>(smem + OFF_AUX + st * AUX_STAGE);
        const int* auxi = reinterpret_cast<const int*>(aux);
        const bool need_mask = !key_ok || (kv0 + KV_BK > p.Sk) || (p.causal && tile_min[t] < kv0 + KV_BK - 1) ||
                               (p.window > 0 && tile_max[t] - kv0 >= p.window) || p.q_seg != nullptr;
        const uint32_t tS = tb + T_BUF + buf * 128 + half * 32, tDP = tS + 64;
        uint32_t pk_p[16], pk_ds[16];
        {
          uint32_t s[32], dp[32];
          tmem_ld32(tS, s);
          tmem_ld32(tDP, dp);
          tmem_wait_ld();
          if (prof) { t0 = clock64(); c_ld += t0 - t1; }
          const float4* lse4 = reinterpret_cast<const float4*>(aux + half * 32);
          const float4* dlt4 = reinterpret_cast<const float4*>(aux + KV_BQ + half * 32);
          if (!need_mask) {
            // branch-free hot path: one FFMA, one EX2, one FADD and one FMUL per score; the
            // softmax scale of dS is applied once to the dK rows in the epilogue
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              const float4 L = lse4[c4], Dl = dlt4[c4];
              const float l[4] = {L.x, L.y, L.z, L.w}, d[4] = {Dl.x, Dl.y, Dl.z, Dl.w};
              float pv[4], dv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                pv[e] = exp2f(fmaf(__uint_as_float(s[4 * c4 + e]), p.scale_log2, -l[e]));
                dv[e] = pv[e] * (__uint_as_float(dp[4 * c4 + e]) - d[e]);
              }
              pk_p[2 * c4] = pack_bf16(pv[0], pv[1]); pk_p[2 * c4 + 1] = pack_bf16(pv[2], pv[3]);
              pk_ds[2 * c4] = pack_bf16(dv[0], dv[1]); pk_ds[2 * c4 + 1] = pack_bf16(dv[2], dv[3]);
            }
          } else {
            const int4* qp4 = reinterpret_cast<const int4*>(auxi + 2 * KV_BQ + half * 32);
            const int4* qs4 = reinterpret_cast<const int4*>(auxi + 3 * KV_BQ + half * 32);
            const int win = p.window > 0 ? p.window : 0x7fffffff;
            const int cmax = p.causal ? kp : -0x7fffffff;   // keep needs qp >= cmax
#pragma unroll
            for (int c4 = 0; c4 < 8; ++c4) {
              const float4 L = lse4[c4], Dl = dlt4[c4];
              const int qn = t * KV_BQ + pos_off + half * 32 + 4 * c4;   // natural positions
              const int4 QP = p.q_pos ? qp4[c4] : make_int4(qn, qn + 1, qn + 2, qn + 3);
              const int4 QS = p.q_seg ? qs4[c4] : make_int4(0, 0, 0, 0);
              const float l[4] = {L.x, L.y, L.z, L.w}, d[4] = {Dl.x, Dl.y, Dl.z, Dl.w};
              const int qp[4] = {QP.x, QP.y, QP.z, QP.w}, qs[4] = {QS.x, QS.y, QS.z, QS.w};
              float pv[4], dv[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const bool keep = key_ok & (qp[e] >= cmax) & (qp[e] - kp < win) & (qs[e] == kseg);
                const float pe = exp2f(fmaf(__uint_as_float(s[4 * c4 + e]), p.scale_log2, -l[e]));
                pv[e] = keep ? pe : 0.f;
                dv[e] = pv[e] * (__uint_as_float(dp[4 * c4 + e]) - d[e]);
              }
              pk_p[2 * c4] = pack_bf16(pv[0], pv[1]); pk_p[2 * c4 + 1] = pack_bf16(pv[2], pv[3]);
              pk_ds[2 * c4] = pack_bf16(dv[0], dv[1]); pk_ds[2 * c4 + 1] = pack_bf16(dv[2], dv[3]);
            }
          }
        }
        if (prof) { t1 = clock64(); c_math += t1 - t0; }
        tmem_st16(tS, pk_p);
        tmem_st16(tDP, pk_ds);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&pds_full[buf]);
        if (prof) c_st += clock64() - t1;
        ++step;
      }
    }
    if (prof) {
      atomicAdd((unsigned long long*)p.prof + 0, (unsigned long long)c_wait);
      atomicAdd((unsigned long long*)p.prof + 1, (unsigned long long)c_ld);
      atomicAdd((unsigned long long*)p.prof + 2, (unsigned long long)c_math);
      atomicAdd((unsigned long long*)p.prof + 3, (unsigned long long)c_st);
      atomicAdd((unsigned long long*)p.prof + 4, (unsigned long long)n_steps);
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
  uint64_t* k_empty = k_full + DQ_KSTAGES;        // [DQ_KSTAGES]
  uint64_t* v_full = k_empty + DQ_KSTAGES;        // [DQ_VSTAGES]
  uint64_t* v_empty = v_full + DQ_VSTAGES;        // [DQ_VSTAGES]
  uint64_t* sdp_full = v_empty + DQ_VSTAGES;      // [2]
  uint64_t* ds_full = sdp_full + 2;               // [2] count 256
  uint64_t* acc_done = ds_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  int* tile_minmax = reinterpret_cast<int*>(acc_done + 2);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (p.Sq + DQ_BM - 1) / DQ_BM;
  // heaviest (latest) query tiles first under a causal mask
  const int qt = n_qtiles - 1 - (int)(blockIdx.x / (p.Hq * p.B));
  const int hq = (blockIdx.x / p.B) % p.Hq, b = blockIdx.x % p.B;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = qt * DQ_BM;
  const int pos_off = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int i = 0; i < DQ_KSTAGES; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < DQ_VSTAGES; ++i) { mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&ds_full[i], 256); }
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

  if (threadIdx.x < DQ_BM) {
    const int r = q0 + threadIdx.x;
    if (r < p.Sq) {
      const int qp = p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : r + pos_off;
      atomicMin(&tile_minmax[0], qp);
      atomicMax(&tile_minmax[1], qp);
    }
  }
  __syncthreads();
  const int qpos_min = tile_minmax[0], qpos_max = tile_minmax[1];
  const int nblk_total = (p.Sk + DQ_BN - 1) / DQ_BN;
  int blk_hi = p.causal ? min(nblk_total, qpos_max / DQ_BN + 1) : nblk_total;
  int blk_lo = (p.window > 0) ? max(0, (qpos_min - p.window + 1) / DQ_BN) : 0;
  if (qpos_max < 0) blk_hi = 0;
  const int nblk = max(0, blk_hi - blk_lo);

  uint8_t* sQ = smem + OFF_Q;
  uint8_t* sdO = smem + OFF_DO;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmdO);
      mbar_expect_tx(qdo_full, Q_BYTES + DO_BYTES);
#pragma unroll
      for (int c = 0; c < BWD_D / 64; ++c) {
        tma_load_3d(sQ + c * (DQ_BM * 128), &tmQ, qdo_full, c * 64, b * p.Sq + q0, hq);
        tma_load_3d(sdO + c * (DQ_BM * 128), &tmdO, qdo_full, c * 64, b * p.Sq + q0, hq);
      }
      for (int j = 0; j < nblk; ++j) {
        const int sk = j % DQ_KSTAGES, sv = j % DQ_VSTAGES;
        const int row = b * p.Sk + (blk_lo + j) * DQ_BN;
        if (!mbar_wait(&k_empty[sk], ((j / DQ_KSTAGES) & 1) ^ 1, p.status, kTimeoutStageFree, 31)) break;
        mbar_expect_tx(&k_full[sk], K_BYTES);
#pragma unroll
        for (int c = 0; c < BWD_D / 64; ++c)
          tma_load_3d(smem + OFF_K + sk * K_BYTES + c * (DQ_BN * 128), &tmK, &k_full[sk], c * 64, row, hkv);
        if (!mbar_wait(&v_empty[sv], ((j / DQ_VSTAGES) & 1) ^ 1, p.status, kTimeoutStageFree, 35)) break;
        mbar_expect_tx(&v_full[sv], V_BYTES);
#pragma unroll
        for (int c = 0; c < BWD_D / 64; ++c)
          tma_load_3d(smem + OFF_V + sv * V_BYTES + c * (DQ_BN * 128), &tmV, &v_full[sv], c * 64, row, hkv);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t id_s = make_idesc_bf16(DQ_BM, DQ_BN, false, false);    // S, dP
      constexpr uint32_t id_dq = make_idesc_bf16(DQ_BM, BWD_D, false, true);    // dQ (A in TMEM, B MN-major)
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sdO);
      bool ok = mbar_wait(qdo_full, 0, p.status, kTimeoutTmaFull, 32);
      auto issue_scores = [&](int j) -> bool {
        const int sk = j % DQ_KSTAGES, sv = j % DQ_VSTAGES;
        if (!mbar_wait(&k_full[sk], (j / DQ_KSTAGES) & 1, p.status, kTimeoutTmaFull, 33)) return false;
        if (!mbar_wait(&v_full[sv], (j / DQ_VSTAGES) & 1, p.status, kTimeoutTmaFull, 37)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(smem + OFF_K + sk * K_BYTES), aV = smem_u32(smem + OFF_V + sv * V_BYTES);
        const uint32_t tS = tmem_base + T_BUF + (j & 1) * 128;
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t ad = make_smem_desc(aQ + (k >> 2) * (DQ_BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aK + (k >> 2) * (DQ_BN * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tS, ad, bd, id_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t ad = make_smem_desc(aDO + (k >> 2) * (DQ_BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aV + (k >> 2) * (DQ_BN * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tS + 64, ad, bd, id_s, k != 0);
        }
        tc_commit(&v_empty[sv]);
        tc_commit(&sdp_full[j & 1]);
        return true;
      };
      const bool prof = p.prof != nullptr;
      long long m_tiles = 0, m_ds = 0, t0 = 0, t1 = 0;
      const long long m_start = prof ? clock64() : 0;
      if (ok) ok = issue_scores(0);
      for (int j = 0; j < nblk && ok; ++j) {
        const int sk = j % DQ_KSTAGES;
        if (prof) t0 = clock64();
        if (j + 1 < nblk) {
          if (!issue_scores(j + 1)) break;
        }
        if (prof) { t1 = clock64(); m_tiles += t1 - t0; }
        if (!mbar_wait(&ds_full[j & 1], (j >> 1) & 1, p.status, kTimeoutSoftmax, 34)) break;
        tc_fence_after();
        if (prof) m_ds += clock64() - t1;
        const uint32_t aK = smem_u32(smem + OFF_K + sk * K_BYTES);
        const uint32_t tDS = tmem_base + T_BUF + (j & 1) * 128 + 64;
#pragma unroll
        for (int k = 0; k < DQ_BN / 16; ++k) {   // dQ += dS K   (K tile [64 keys][128 d]: N = d contiguous)
          const uint64_t bd = make_smem_desc(aK + k * 2048, DQ_BN * 128, 1024);
          mma_ts(tmem_base + T_DQ, tDS + (k >> 1) * 32 + (k & 1) * 8, bd, id_dq, (j | k) != 0);
        }
        tc_commit(&k_empty[sk]);
      }
      tc_commit(acc_done);
      if (prof) {
        atomicAdd((unsigned long long*)p.prof + 21, (unsigned long long)m_tiles);
        atomicAdd((unsigned long long*)p.prof + 22, (unsigned long long)m_ds);
        atomicAdd((unsigned long long*)p.prof + 23, (unsigned long long)(clock64() - m_start));
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;             // which 32 of the 64 key columns
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
    const int* ks = p.kv_seg ? p.kv_seg + (long long)b * p.Sk : nullptr;
    bool ok = true;

    const bool prof = p.prof != nullptr && (threadIdx.x == 64 || threadIdx.x == 160);
    const int pslot = threadIdx.x == 64 ? 16 : 24;
    long long c_wait = 0, c_ld = 0, c_math = 0, c_st = 0, t0 = 0, t1 = 0;
    for (int j = 0; j < nblk && ok; ++j) {
      const int buf = j & 1;
      if (prof) t0 = clock64();
      if (!mbar_wait(&sdp_full[buf], (j >> 1) & 1, p.status, kTimeoutAccFull, 36)) { ok = false; break; }
      tc_fence_after();
      if (prof) { t1 = clock64(); c_wait += t1 - t0; }
      const int kv0 = (blk_lo + j) * DQ_BN;
      const bool need_mask = (p.causal && kv0 + DQ_BN - 1 > qpos_min) || (kv0 + DQ_BN > p.Sk) ||
                             (p.window > 0 && qpos_max - kv0 >= p.window) || p.q_seg != nullptr;
      const uint32_t tS = tb + T_BUF + buf * 128 + half * 32, tDP = tS + 64;
      uint32_t pk[16];
      {
        uint32_t s[32], dp[32];
        tmem_ld32(tS, s);
        tmem_ld32(tDP, dp);
        tmem_wait_ld();
        if (prof) { t0 = clock64(); c_ld += t0 - t1; }
        if (!need_mask) {
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const float p0 = exp2f(fmaf(__uint_as_float(s[c]), p.scale_log2, -lse2));
            const float p1 = exp2f(fmaf(__uint_as_float(s[c + 1]), p.scale_log2, -lse2));
            pk[c / 2] = pack_bf16(p0 * (__uint_as_float(dp[c]) - delta), p1 * (__uint_as_float(dp[c + 1]) - delta));
          }
        } else {
          const int win = p.window > 0 ? p.window : 0x7fffffff;
          const int kmax = p.causal ? min(qpos, p.Sk - 1) : p.Sk - 1;   // keep needs kp <= kmax
          const int kbase = kv0 + half * 32;
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float dv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kp = kbase + c + e;
              bool keep = (kp <= kmax) & (qpos - kp < win);
              if (ks) keep = keep & (__ldg(ks + min(kp, p.Sk - 1)) == qseg);
              const float pe = exp2f(fmaf(__uint_as_float(s[c + e]), p.scale_log2, -lse2));
              dv[e] = keep ? pe * (__uint_as_float(dp[c + e]) - delta) : 0.f;
            }
            pk[c / 2] = pack_bf16(dv[0], dv[1]);
          }
        }
      }
      if (prof) { t1 = clock64(); c_math += t1 - t0; }
      tmem_st16(tDP, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&ds_full[buf]);
      if (prof) c_st += clock64() - t1;
    }
    if (prof) {
      atomicAdd((unsigned long long*)p.prof + pslot, (unsigned long long)c_wait);
      atomicAdd((unsigned long long*)p.prof + pslot + 1, (unsigned long long)c_ld);
      atomicAdd((unsigned long long*)p.prof + pslot + 2, (unsigned long long)c_math);
      atomicAdd((unsigned long long*)p.prof + pslot + 3, (unsigned long long)c_st);
      if (threadIdx.x == 64) atomicAdd((unsigned long long*)p.prof + 20, (unsigned long long)nblk);
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

static long long* g_attn_bwd_prof = nullptr;

// Profiling aid: 32 device counters (cycles) the backward kernels add to when the pointer is
// non-null.  [0..7] dK/dV kernel, [16..23] dQ kernel: compute thread waiting for scores, TMEM
// loads, math, TMEM stores + arrive, steps; MMA thread issuing scores (includes waiting for the
// operand tiles), waiting for the compute warps, whole loop.
extern "C" void tpb_attn_bwd_set_prof(long long* counters) { g_attn_bwd_prof = counters; }

// Floats of scratch `tpb_attn_bwd` needs (scaled log-sum-exp and delta rows, padded to 128).
extern "C" long long tpb_attn_bwd_scratch_floats(int B, int Sq, int Hq) {
  const long long sq_pad = (Sq + DQ_BM - 1) / DQ_BM * DQ_BM;
  return 2LL * B * Hq * sq_pad;
}

extern "C" int tpb_attn_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o,
                            const float* lse, float* scratch, void* dq, void* dk, void* dv, int B, int Sq,
                            int Sk, int Hq, int Hkv, int dqk, int dvd, long long ldq, long long ldk, long long ldv,
                            long long lddo, long long lddq, long long lddk, long long lddv, float scale, int causal,
                            int window, const int* q_pos, const int* q_seg, const int* kv_seg, void* stream_) {
  if (dqk != 128 || dvd != 128 || Hq % Hkv) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -2;
  if (lddo != (long long)Hq * dvd) return -2;   // dO and O are contiguous [B*Sq, Hq, 128]
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  if ((Sq + KV_BQ - 1) / KV_BQ > KV_MAX_TILES) return -6;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int sq_pad = (Sq + DQ_BM - 1) / DQ_BM * DQ_BM;
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
  p.scale = scale; p.scale_log2 = scale * kLog2e;
  p.causal = causal; p.window = window;
  p.q_pos = q_pos; p.q_seg = q_seg; p.kv_seg = kv_seg;
  p.lse2 = lse2; p.delta = delta; p.Sq_pad = sq_pad;
  p.aux_bulk = (Sq % 4 == 0) && (reinterpret_cast<uintptr_t>(q_pos) % 16 == 0) &&
               (reinterpret_cast<uintptr_t>(q_seg) % 16 == 0);
  p.dQ = reinterpret_cast<__nv_bfloat16*>(dq); p.lddq = lddq;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.lddk = lddk;
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv); p.lddv = lddv;
  p.status = status_block();
  p.prof = g_attn_bwd_prof;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::TOTAL);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dqk::TOTAL);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  cudaError_t e;
  {
    CUtensorMap tq, tk, tv, tdo;
    if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, KV_BQ)) return -3;
    if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, KV_BK)) return -4;
    if (make_tmap_3d(&tv, v, dvd, (uint64_t)B * Sk, Hkv, ldv, dvd, 64, KV_BK)) return -5;
    if (make_tmap_3d(&tdo, dO, dvd, (uint64_t)B * Sq, Hq, lddo, dvd, 64, KV_BQ)) return -5;
    dim3 grid(((Sk + KV_BK - 1) / KV_BK) * Hkv * B, 1, 1);
    attn_bwd_dkv_kernel<<<grid, BWD_THREADS, dkv::TOTAL, stream>>>(tq, tk, tv, tdo, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) return 1000 + (int)e;
  }
  {
    CUtensorMap tq, tk, tv, tdo;
    if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, DQ_BM)) return -3;
    if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, DQ_BN)) return -4;
    if (make_tmap_3d(&tv, v, dvd, (uint64_t)B * Sk, Hkv, ldv, dvd, 64, DQ_BN)) return -5;
    if (make_tmap_3d(&tdo, dO, dvd, (uint64_t)B * Sq, Hq, lddo, dvd, 64, DQ_BM)) return -5;
    dim3 grid(((Sq + DQ_BM - 1) / DQ_BM) * Hq * B, 1, 1);
    attn_bwd_dq_kernel<<<grid, BWD_THREADS, dqk::TOTAL, stream>>>(tq, tk, tv, tdo, p);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
