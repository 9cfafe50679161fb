// Flash-attention backward for sm_100a (tcgen05 + TMEM + TMA), GQA-native, head dim 128.
//
// One CTA per (128-key block, kv head, batch).  K and V of the block stay in shared
// memory, dK and dV accumulate in TMEM over every query tile (64 rows) and every query
// head of the GQA group that can see the block, so they need no atomics; dQ tiles are
// reduced into an fp32 buffer with coalesced `red.add` and converted afterwards.
//
// Everything is computed in the transposed frame (rows = keys) so that each of the 128
// compute threads owns one key row, i.e. one TMEM lane:
//
//   S^T  = K Q^T            (SS)   128 x 64 fp32            TMEM [256,320)
//   dP^T = V dO^T           (SS)   128 x 64 fp32            TMEM [320,384)
//   P^T  = exp2(S^T*c - lse), dS^T = P^T o (dP^T - delta) * scale     (registers)
//   dV  += P^T  dO          (TS)   A = P^T  bf16 in TMEM [384,416)
//   dK  += dS^T Q           (TS)   A = dS^T bf16 in TMEM [416,448)
//   dQ^T = K^T dS^T         (SS)   B = dS^T bf16 in shared memory, result TMEM [448,512)
//   dK: TMEM [0,128), dV: TMEM [128,256)
//
// The Q and dO tiles are loaded once per step and used through two descriptors: K-major
// (for S^T, dP^T) and MN-major (for dK, dV); K likewise (K-major for S^T, MN-major for
// dQ^T).  Roles: warp 0 TMA producer (+ lse/delta/position staging), warp 1 MMA issuer,
// warps 2-5 compute.  The MMA warp issues S^T/dP^T of step i+1 before dV/dK/dQ^T of
// step i, so the tensor core works on the next scores while the compute warps are busy.

#include <cstdlib>

#include "common.cuh"
#include "tpb.h"

namespace tpb {

int make_tmap_3d(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                 uint64_t stride2_elems, uint32_t box0, uint32_t box1);
int sm_count();

constexpr int BWD_BK = 128;   // keys per CTA
constexpr int BWD_BQ = 64;    // query rows per step
constexpr int BWD_D = 128;
constexpr int BWD_THREADS = 320;   // TMA warp, MMA warp, 8 compute warps
constexpr int BWD_MAX_TILES = 512;
constexpr int BWD_STAGES = 3;  // Q/dO tile ring depth

struct AttnBwdParams {
  int B, Sq, Sk, Hq, Hkv;
  float scale, scale_log2;
  int causal, window;
  const int* q_pos;
  const int* q_seg;
  const int* kv_seg;
  const float* lse;     // [B,Hq,Sq] natural log
  const float* delta;   // [B,Hq,Sq]
  float* dq_acc;        // [B,Hq,Sq_pad,128] fp32, zero-initialised (Sq_pad = Sq rounded up to 64)
  int Sq_pad;
  int debug;            // profiling aid: 1 = skip dQ reduction, 2 = skip the exp/dS math
  __nv_bfloat16* dK; long long lddk;
  __nv_bfloat16* dV; long long lddv;
  int* status;
};

namespace bwd {
constexpr int K_BYTES = BWD_BK * BWD_D * 2;       // 32 KB
constexpr int V_BYTES = BWD_BK * BWD_D * 2;       // 32 KB
constexpr int Q_BYTES = BWD_BQ * BWD_D * 2;       // 16 KB
constexpr int DO_BYTES = BWD_BQ * BWD_D * 2;      // 16 KB
constexpr int DS_BYTES = BWD_BK * BWD_BQ * 2;     // 16 KB
constexpr int OFF_K = 0;
constexpr int OFF_V = OFF_K + K_BYTES;
constexpr int OFF_Q = OFF_V + V_BYTES;
constexpr int OFF_DO = OFF_Q + BWD_STAGES * Q_BYTES;
constexpr int OFF_DS = OFF_DO + BWD_STAGES * DO_BYTES;
constexpr int DQ_STAGE_BYTES = BWD_BQ * BWD_D * 4; // 32 KB fp32 [64 q][128 d] staging for the bulk reduce
constexpr int OFF_DQS = OFF_DS + DS_BYTES;
constexpr int OFF_AUX = OFF_DQS + DQ_STAGE_BYTES; // per stage: lse2[64], delta[64], qpos[64], qseg[64]  (1 KB)
constexpr int AUX_STAGE = 4 * BWD_BQ * 4;
constexpr int OFF_TILES = OFF_AUX + BWD_STAGES * AUX_STAGE;  // tile min/max table: 2 * BWD_MAX_TILES ints
constexpr int OFF_BAR = OFF_TILES + 2 * BWD_MAX_TILES * 4;
constexpr int TOTAL = OFF_BAR + 256 + 1024;
// TMEM columns
constexpr int T_DK = 0, T_DV = 128, T_S = 256, T_DP = 320, T_P = 384, T_DS = 416, T_DQ = 448;
}  // namespace bwd

// delta[b,h,q] = sum_d dO * O      (dO, O: [B*Sq, Hq, 128] contiguous)
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                      float* __restrict__ delta, int B, int Sq, int Hq) {
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
      delta[(b * Hq + h) * Sq + q] = s;
    }
  }
}

// dq[b, q, h, :] (bf16, row pitch lddq) = acc[b, h, q, :] (fp32, [B,Hq,Sq_pad,128])
__global__ void attn_bwd_convert_dq_kernel(const float4* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int B,
                                           int Sq, int Sq_pad, int Hq, long long lddq) {
  const long long total = (long long)B * Sq * Hq * (BWD_D / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % (BWD_D / 4));
    long long r = i / (BWD_D / 4);
    const int h = (int)(r % Hq);
    r /= Hq;
    const int q = (int)(r % Sq);
    const long long b = r / Sq;
    const float4 v = acc[((b * Hq + h) * Sq_pad + q) * (BWD_D / 4) + c];
    *reinterpret_cast<uint2*>(dq + (b * Sq + q) * lddq + h * BWD_D + c * 4) =
        make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  }
}

__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                const AttnBwdParams p) {
  using namespace bwd;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;                  // [BWD_STAGES], count 2 (TMA expect_tx arrive + aux arrive)
  uint64_t* qdo_empty = qdo_full + BWD_STAGES;    // [BWD_STAGES]
  uint64_t* sdp_full = qdo_empty + BWD_STAGES;
  uint64_t* pds_full = sdp_full + 1;   // count 256
  uint64_t* dq_full = sdp_full + 2;
  uint64_t* dq_empty = sdp_full + 3;   // count 8
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sdp_full + 4);
  int* tile_min = reinterpret_cast<int*>(smem + OFF_TILES);
  int* tile_max = tile_min + BWD_MAX_TILES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // linear block id is key-block major so that under a causal mask the blocks with the most
  // visible query tiles (lowest key index) are scheduled first on every head
  const int kb = blockIdx.x / (p.Hkv * p.B);
  const int hkv = (blockIdx.x / p.B) % p.Hkv, b = blockIdx.x % p.B;
  const int G = p.Hq / p.Hkv;
  const int kv0 = kb * BWD_BK;
  const int pos_off = p.Sk - p.Sq;
  const int n_tiles = min((p.Sq + BWD_BQ - 1) / BWD_BQ, BWD_MAX_TILES);

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) { mbar_init(&qdo_full[i], 2); mbar_init(&qdo_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 256);
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, 8);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // position range of every query tile (decides which tiles this key block can see)
  for (int t = threadIdx.x; t < n_tiles; t += BWD_THREADS) {
    const int r0 = t * BWD_BQ, r1 = min(p.Sq, r0 + BWD_BQ);
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
    if (p.window > 0 && tile_min[t] - (kv0 + BWD_BK - 1) >= p.window) return false;
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
          tma_load_3d(sK + c * (BWD_BK * 128), &tmK, kv_full, c * 64, b * p.Sk + kv0, hkv);
          tma_load_3d(sV + c * (BWD_BK * 128), &tmV, kv_full, c * 64, b * p.Sk + kv0, hkv);
        }
      }
      int step = 0;
      bool ok = true;
      for (int g = 0; g < G && ok; ++g) {
        const int hq = hkv * G + g;
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (!visible(t)) continue;
          const int st = step % BWD_STAGES;
          const uint32_t ph = (step / BWD_STAGES) & 1;
          int okw = 1;
          if (lane == 0) okw = mbar_wait(&qdo_empty[st], ph ^ 1, p.status, kTimeoutStageFree, 21) ? 1 : 0;
          okw = __shfl_sync(0xffffffffu, okw, 0);
          if (!okw) { ok = false; break; }
          const int q0 = t * BWD_BQ;
          if (lane == 0) {
            mbar_expect_tx(&qdo_full[st], Q_BYTES + DO_BYTES);
            for (int c = 0; c < BWD_D / 64; ++c) {
              tma_load_3d(smem + OFF_Q + st * Q_BYTES + c * (BWD_BQ * 128), &tmQ, &qdo_full[st], c * 64,
                          b * p.Sq + q0, hq);
              tma_load_3d(smem + OFF_DO + st * DO_BYTES + c * (BWD_BQ * 128), &tmdO, &qdo_full[st], c * 64,
                          b * p.Sq + q0, hq);
            }
          }
          float* aux = reinterpret_cast<float*>(smem + OFF_AUX + st * AUX_STAGE);
          int* auxi = reinterpret_cast<int*>(aux);
          for (int c = lane; c < BWD_BQ; c += 32) {
            const int r = q0 + c;
            const bool rok = r < p.Sq;
            const long long li = ((long long)b * p.Hq + hq) * p.Sq + r;
            aux[c] = (p.debug & 4) ? 3.f : (rok ? p.lse[li] * 1.4426950408889634f : INFINITY);
            aux[BWD_BQ + c] = (p.debug & 4) ? 0.f : (rok ? p.delta[li] : 0.f);
            auxi[2 * BWD_BQ + c] = rok ? (p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : r + pos_off) : -0x40000000;
            auxi[3 * BWD_BQ + c] = (rok && p.q_seg) ? p.q_seg[(long long)b * p.Sq + r] : 0;
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&qdo_full[st]);
          ++step;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t id_s = make_idesc_bf16(BWD_BK, BWD_BQ, false, false);   // S^T, dP^T
      constexpr uint32_t id_acc = make_idesc_bf16(BWD_BK, BWD_D, false, true);   // dV, dK (A in TMEM, B MN-major)
      constexpr uint32_t id_dq = make_idesc_bf16(BWD_D, BWD_BQ, true, true);     // dQ^T
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aDS = smem_u32(smem + OFF_DS);
      bool ok = mbar_wait(kv_full, 0, p.status, kTimeoutTmaFull, 22);
      auto issue_scores = [&](int step) -> bool {
        const int st = step % BWD_STAGES;
        if (!mbar_wait(&qdo_full[st], (step / BWD_STAGES) & 1, p.status, kTimeoutTmaFull, 23)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(smem + OFF_Q + st * Q_BYTES), aDO = smem_u32(smem + OFF_DO + st * DO_BYTES);
        if (!(p.debug & 64)) {
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t ad = make_smem_desc(aK + (k >> 2) * (BWD_BK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aQ + (k >> 2) * (BWD_BQ * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tmem_base + T_S, ad, bd, id_s, k != 0);
        }
#pragma unroll
        for (int k = 0; k < BWD_D / 16; ++k) {
          const uint64_t ad = make_smem_desc(aV + (k >> 2) * (BWD_BK * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t bd = make_smem_desc(aDO + (k >> 2) * (BWD_BQ * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tmem_base + T_DP, ad, bd, id_s, k != 0);
        }
        }
        tc_commit(sdp_full);
        return true;
      };
      if (ok) ok = issue_scores(0);
      for (int step = 0; step < n_steps && ok; ++step) {
        const int st = step % BWD_STAGES;
        if (!mbar_wait(pds_full, step & 1, p.status, kTimeoutSoftmax, 24)) break;
        tc_fence_after();
        if (step + 1 < n_steps) {
          if (!issue_scores(step + 1)) break;
        }
        const uint32_t aQ = smem_u32(smem + OFF_Q + st * Q_BYTES), aDO = smem_u32(smem + OFF_DO + st * DO_BYTES);
        if (!(p.debug & 16)) {
#pragma unroll
        for (int k = 0; k < BWD_BQ / 16; ++k) {   // dV += P^T dO
          const uint64_t bd = make_smem_desc(aDO + k * 2048, BWD_BQ * 128, 1024);
          mma_ts(tmem_base + T_DV, tmem_base + T_P + k * 8, bd, id_acc, (step | k) != 0);
        }
#pragma unroll
        for (int k = 0; k < BWD_BQ / 16; ++k) {   // dK += dS^T Q
          const uint64_t bd = make_smem_desc(aQ + k * 2048, BWD_BQ * 128, 1024);
          mma_ts(tmem_base + T_DK, tmem_base + T_DS + k * 8, bd, id_acc, (step | k) != 0);
        }
        }
        if (step > 0) {
          if (!mbar_wait(dq_empty, (step - 1) & 1, p.status, kTimeoutAccFree, 25)) break;
          tc_fence_after();
        }
        if (!(p.debug & 32))
#pragma unroll
        for (int k = 0; k < BWD_BK / 16; ++k) {   // dQ^T = K^T dS^T
          const uint64_t ad = make_smem_desc(aK + k * 2048, BWD_BK * 128, 1024);
          const uint64_t bd = make_smem_desc(aDS + k * 2048, BWD_BK * 128, 1024);
          mma_ss(tmem_base + T_DQ, ad, bd, id_dq, k != 0);
        }
        tc_commit(&qdo_empty[st]);
        tc_commit(dq_full);
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    // Eight warps: warp w may touch TMEM lanes 32*(w%4)..+31, so warps w and w+4 share a lane
    // quarter (the same 32 key rows) and split the 64 query columns of a step between them.
    // Two warps per scheduler keep the exp/FMA chains of one hidden behind the other's.
    const int qd = warp & 3;
    const int half = (warp - 2) >> 2;             // which 32 of the 64 query columns
    const int r_local = qd * 32 + lane;           // key row == TMEM lane
    const int kp = kv0 + r_local;                 // key position (keys are in natural order)
    const bool key_ok = kp < p.Sk;
    const int kseg = (p.kv_seg && key_ok) ? p.kv_seg[(long long)b * p.Sk + kp] : 0;
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const uint32_t tb = tmem_base + lane_addr;
    uint8_t* sDS = smem + OFF_DS;
    bool ok = true;

    float* sDQ = reinterpret_cast<float*>(smem + OFF_DQS);
    const bool leader = (threadIdx.x == 64);
    auto reduce_dq = [&](int hq_prev, int q0_prev) {
      // dQ^T tile in TMEM: lane = d, column = query row.  Transpose it through shared memory
      // into a contiguous fp32 [64 q][128 d] tile and add it to the global accumulator with
      // one bulk reduce (the tile is contiguous in the [B,Hq,Sq_pad,128] accumulator).
      if (p.debug & 1) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(dq_empty);
        return;
      }
      if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      asm volatile("bar.sync 1, 256;" ::: "memory");
      {
        uint32_t v[32];
        tmem_ld32(tb + T_DQ + half * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) sDQ[(half * 32 + c) * BWD_D + r_local] = __uint_as_float(v[c]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_empty);
      fence_proxy_async();
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (leader) {
        float* dst = p.dq_acc + (((long long)b * p.Hq + hq_prev) * p.Sq_pad + q0_prev) * BWD_D;
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst),
                     "r"(smem_u32(sDQ)), "r"((uint32_t)DQ_STAGE_BYTES)
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    };

    int step = 0, prev_hq = 0, prev_q0 = 0;
    for (int g = 0; g < G && ok; ++g) {
      const int hq = hkv * G + g;
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (!visible(t)) continue;
        const int st = step % BWD_STAGES;
        const int q0 = t * BWD_BQ;
        if (!mbar_wait(sdp_full, step & 1, p.status, kTimeoutAccFull, 26)) { ok = false; break; }
        tc_fence_after();
        const float* aux = reinterpret_cast<const float*>(smem + OFF_AUX + st * AUX_STAGE);
        const int* auxi = reinterpret_cast<const int*>(aux);
        const bool need_mask = !key_ok || (kv0 + BWD_BK > p.Sk) || (p.causal && tile_min[t] < kv0 + BWD_BK - 1) ||
                               (p.window > 0 && tile_max[t] - kv0 >= p.window) || p.q_seg != nullptr;
        uint32_t pk_p[16], pk_ds[16];
        {
          uint32_t s[32], dp[32];
          tmem_ld32(tb + T_S + half * 32, s);
          tmem_ld32(tb + T_DP + half * 32, dp);
          tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float pv[2], dv[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int col = half * 32 + c + e;
              float pe = (p.debug & 2) ? 0.5f : exp2f(__uint_as_float(s[c + e]) * p.scale_log2 - aux[col]);
              if (need_mask) {
                const int qp = auxi[2 * BWD_BQ + col];
                bool keep = key_ok;
                if (p.causal) keep = keep && kp <= qp;
                if (p.window > 0) keep = keep && (qp - kp < p.window);
                if (p.q_seg) keep = keep && (auxi[3 * BWD_BQ + col] == kseg);
                pe = keep ? pe : 0.f;
              }
              pv[e] = pe;
              dv[e] = pe * (__uint_as_float(dp[c + e]) - aux[BWD_BQ + col]) * p.scale;
            }
            pk_p[c / 2] = pack_bf16(pv[0], pv[1]);
            pk_ds[c / 2] = pack_bf16(dv[0], dv[1]);
          }
        }
        // the previous step's MMAs must be done reading P^T / dS^T (TMEM and shared memory)
        if (step > 0) {
          if (!mbar_wait(dq_full, (step - 1) & 1, p.status, kTimeoutAccFull, 27)) { ok = false; break; }
          tc_fence_after();
        }
        tmem_st16(tb + T_P + half * 16, pk_p);
        tmem_st16(tb + T_DS + half * 16, pk_ds);
        if (!(p.debug & 8)) {
          uint8_t* rowp = sDS + r_local * 128;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(rowp + (((half * 4 + j) ^ (r_local & 7)) << 4)) =
                make_uint4(pk_ds[4 * j], pk_ds[4 * j + 1], pk_ds[4 * j + 2], pk_ds[4 * j + 3]);
        }
        fence_proxy_async();
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(pds_full);
        if (step > 0) reduce_dq(prev_hq, prev_q0);
        prev_hq = hq; prev_q0 = q0;
        ++step;
      }
    }
    // ---- tail: last dQ^T tile, then dK / dV
    if (ok && n_steps > 0) {
      ok = mbar_wait(dq_full, (n_steps - 1) & 1, p.status, kTimeoutAccFull, 28);
      tc_fence_after();
      if (ok) reduce_dq(prev_hq, prev_q0);
    }
    if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __nv_bfloat16* dk_row = p.dK + ((long long)b * p.Sk + kp) * p.lddk + (long long)hkv * BWD_D;
    __nv_bfloat16* dv_row = p.dV + ((long long)b * p.Sk + kp) * p.lddv + (long long)hkv * BWD_D;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* dst = which == 0 ? dk_row : dv_row;
      const uint32_t tsrc = tb + (which == 0 ? T_DK : T_DV);
#pragma unroll 1
      for (int c = half * 2; c < half * 2 + 2; ++c) {
        uint32_t o[32];
        if (n_steps > 0 && ok) {
          tmem_ld32(tsrc + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0;
        }
        if (key_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v)
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = make_uint4(
                pack_bf16(__uint_as_float(o[8 * v]), __uint_as_float(o[8 * v + 1])),
                pack_bf16(__uint_as_float(o[8 * v + 2]), __uint_as_float(o[8 * v + 3])),
                pack_bf16(__uint_as_float(o[8 * v + 4]), __uint_as_float(o[8 * v + 5])),
                pack_bf16(__uint_as_float(o[8 * v + 6]), __uint_as_float(o[8 * v + 7])));
        }
      }
    }
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

extern "C" int tpb_attn_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o,
                            const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                            int Sk, int Hq, int Hkv, int dqk, int dvd, long long ldq, long long ldk, long long ldv,
                            long long lddo, long long lddq, long long lddk, long long lddv, float scale, int causal,
                            int window, const int* q_pos, const int* q_seg, const int* kv_seg, void* stream_) {
  if (dqk != 128 || dvd != 128 || Hq % Hkv) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (lddo % 8) || (lddq % 4) || (lddk % 8) || (lddv % 8)) return -2;
  if (lddo != (long long)Hq * dvd) return -2;   // dO and O are contiguous [B*Sq, Hq, 128]
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  {
    const long long warps = (long long)B * Sq * Hq;
    long long blocks = (warps * 32 + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    attn_bwd_delta_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(dO),
                                                           reinterpret_cast<const __nv_bfloat16*>(o), delta, B, Sq, Hq);
  }
  CUtensorMap tq, tk, tv, tdo;
  if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, BWD_BQ)) return -3;
  if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, BWD_BK)) return -4;
  if (make_tmap_3d(&tv, v, dvd, (uint64_t)B * Sk, Hkv, ldv, dvd, 64, BWD_BK)) return -5;
  if (make_tmap_3d(&tdo, dO, dvd, (uint64_t)B * Sq, Hq, lddo, dvd, 64, BWD_BQ)) return -5;
  AttnBwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal; p.window = window;
  p.q_pos = q_pos; p.q_seg = q_seg; p.kv_seg = kv_seg;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.Sq_pad = (Sq + BWD_BQ - 1) / BWD_BQ * BWD_BQ;
  {
    const char* dbg = getenv("TPB_ATTN_BWD_DEBUG");
    p.debug = dbg ? atoi(dbg) : 0;
  }
  p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.lddk = lddk;
  p.dV = reinterpret_cast<__nv_bfloat16*>(dv); p.lddv = lddv;
  p.status = status_block();
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bwd::TOTAL);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  dim3 grid(((Sk + BWD_BK - 1) / BWD_BK) * Hkv * B, 1, 1);
  attn_bwd_kernel<<<grid, BWD_THREADS, bwd::TOTAL, stream>>>(tq, tk, tv, tdo, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return 1000 + (int)e;
  {
    const long long total = (long long)B * Sq * Hq * (BWD_D / 4);
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    attn_bwd_convert_dq_kernel<<<(int)blocks, 256, 0, stream>>>(reinterpret_cast<const float4*>(dq_acc),
                                                                reinterpret_cast<__nv_bfloat16*>(dq), B, Sq,
                                                                (Sq + BWD_BQ - 1) / BWD_BQ * BWD_BQ, Hq, lddq);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
