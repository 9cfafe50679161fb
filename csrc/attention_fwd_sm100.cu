// Flash-attention forward for sm_100a (tcgen05 + TMEM + TMA), GQA-native.
//
// One CTA per (128-row query tile, query head, batch); two CTAs are resident per SM
// (96-112 KB shared memory, 256 TMEM columns each) so the tensor core always has the
// other CTA's MMAs to run while this one is in its softmax.
//
//   warp 0      TMA producer: Q tile once, then a 2-stage ring of 64-key K tiles and a
//               2-stage ring of 64-key V tiles (all 128-byte swizzled, non-multicast).
//   warp 1      MMA issuer: S[j%2] = Q K_j^T (SS, fp32 in TMEM), then O += P_j V_j with
//               P read straight from TMEM (TS).  S is double buffered, so Q K_{j+1}^T is
//               in flight while the softmax of block j runs.
//   warps 2..5  softmax: thread r owns query row r (TMEM lane r): tcgen05.ld of its 64
//               scores, masking, exp2 with a lazily updated running maximum (O is only
//               rescaled when the maximum moved by more than 2^8), bf16 P written back
//               over the same TMEM columns.  Final O / l and the log-sum-exp are written
//               by the same threads.
//
// Masks: causal, sliding window, segment ids (packed sequences) and explicit query
// positions (rows of a context-parallel shard in zig-zag order).  Key blocks that no
// query of the tile can see are skipped; only blocks that straddle a mask edge pay for
// per-element masking.

#include "common.cuh"
#include "tpb.h"

namespace tpb {

int make_tmap_3d(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_elems,
                 uint64_t stride2_elems, uint32_t box0, uint32_t box1);
int sm_count();

constexpr int FWD_BM = 128;     // query rows per CTA
constexpr int FWD_BN = 64;      // keys per block
constexpr int FWD_DV = 128;
constexpr int FWD_THREADS = 192;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct AttnFwdParams {
  int B, Sq, Sk, Hq, Hkv;
  float scale_log2;
  int causal, window;
  const int* q_pos;    // [B*Sq] or null
  const int* q_seg;    // [B*Sq] or null
  const int* kv_seg;   // [B*Sk] or null
  __nv_bfloat16* O;
  long long ldo;       // elements between consecutive tokens of O
  float* lse;          // [B, Hq, Sq]
  int* status;
};

template <int DQK>
struct FwdSmem {
  static constexpr int Q_BYTES = FWD_BM * DQK * 2;
  static constexpr int K_BYTES = FWD_BN * DQK * 2;
  static constexpr int V_BYTES = FWD_BN * FWD_DV * 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * K_BYTES;
  static constexpr int OFF_BAR = OFF_V + 2 * V_BYTES;
  static constexpr int TOTAL = OFF_BAR + 256 + 1024;
};

template <int DQK>
__global__ void __launch_bounds__(FWD_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using L = FwdSmem<DQK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2]
  uint64_t* p_full = bars + 11;   // [2]
  uint64_t* o_done = bars + 13;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  int* tile_minmax = reinterpret_cast<int*>(bars + 15);  // [2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qtiles = (p.Sq + FWD_BM - 1) / FWD_BM;
  const int qt = n_qtiles - 1 - (int)blockIdx.x;   // heaviest (latest) tiles first under a causal mask
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = qt * FWD_BM;
  const int pos_off = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 128);
    }
    mbar_init(o_done, 1);
    tile_minmax[0] = 0x7fffffff;
    tile_minmax[1] = -0x7fffffff;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Range of positions covered by this tile's query rows.
  if (threadIdx.x < FWD_BM) {
    const int r = q0 + threadIdx.x;
    if (r < p.Sq) {
      const int qp = p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : r + pos_off;
      atomicMin(&tile_minmax[0], qp);
      atomicMax(&tile_minmax[1], qp);
    }
  }
  __syncthreads();
  const int qpos_min = tile_minmax[0], qpos_max = tile_minmax[1];
  const int nblk_total = (p.Sk + FWD_BN - 1) / FWD_BN;
  int blk_hi = p.causal ? min(nblk_total, qpos_max / FWD_BN + 1) : nblk_total;
  int blk_lo = (p.window > 0) ? max(0, (qpos_min - p.window + 1) / FWD_BN) : 0;
  if (qpos_max < 0) blk_hi = 0;
  const int nblk = max(0, blk_hi - blk_lo);

  uint8_t* sQ = smem;
  uint8_t* sK = smem + L::OFF_K;
  uint8_t* sV = smem + L::OFF_V;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < DQK / 64; ++c)
        tma_load_3d(sQ + c * (FWD_BM * 128), &tmQ, q_full, c * 64, b * p.Sq + q0, hq);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = b * p.Sk + (blk_lo + j) * FWD_BN;
        if (!mbar_wait(&k_empty[s], ph ^ 1, p.status, kTimeoutStageFree, 11)) break;
        mbar_expect_tx(&k_full[s], L::K_BYTES);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c)
          tma_load_3d(sK + s * L::K_BYTES + c * (FWD_BN * 128), &tmK, &k_full[s], c * 64, row, hkv);
        if (!mbar_wait(&v_empty[s], ph ^ 1, p.status, kTimeoutStageFree, 12)) break;
        mbar_expect_tx(&v_full[s], L::V_BYTES);
#pragma unroll
        for (int c = 0; c < FWD_DV / 64; ++c)
          tma_load_3d(sV + s * L::V_BYTES + c * (FWD_BN * 128), &tmV, &v_full[s], c * 64, row, hkv);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(FWD_BM, FWD_BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(FWD_BM, FWD_DV, false, true);
      const uint32_t tS = tmem_base, tO = tmem_base + 128;
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutTmaFull, 13);
      tc_fence_after();
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(&k_full[s], (j >> 1) & 1, p.status, kTimeoutTmaFull, 14)) return false;
        tc_fence_after();
        const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK + s * L::K_BYTES);
#pragma unroll
        for (int k = 0; k < DQK / 16; ++k) {
          const uint64_t qd = make_smem_desc(aQ + (k >> 2) * (FWD_BM * 128) + (k & 3) * 32, 16, 1024);
          const uint64_t kd = make_smem_desc(aK + (k >> 2) * (FWD_BN * 128) + (k & 3) * 32, 16, 1024);
          mma_ss(tS + s * FWD_BN, qd, kd, idesc_qk, k != 0);
        }
        tc_commit(&k_empty[s]);
        tc_commit(&s_full[s]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nblk && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j + 1 < nblk) {
          if (!issue_qk(j + 1)) break;
        }
        if (!mbar_wait(&p_full[s], ph, p.status, kTimeoutSoftmax, 15)) break;
        if (!mbar_wait(&v_full[s], ph, p.status, kTimeoutTmaFull, 16)) break;
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + s * L::V_BYTES);
#pragma unroll
        for (int k = 0; k < FWD_BN / 16; ++k) {
          // V tile is [64 keys][128 d] in two 64-wide d blocks: MN-major B (N = d contiguous)
          const uint64_t vd = make_smem_desc(aV + k * 2048, FWD_BN * 128, 1024);
          mma_ts(tO, tS + s * FWD_BN + k * 8, vd, idesc_pv, (j | k) != 0);
        }
        tc_commit(&v_empty[s]);
        tc_commit(o_done);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int q = warp & 3;
    const int r_local = q * 32 + lane;
    const int row = q0 + r_local;
    const bool row_ok = row < p.Sq;
    const long long grow = (long long)b * p.Sq + row;
    const int qpos = row_ok ? (p.q_pos ? p.q_pos[grow] : row + pos_off) : -1;
    const int qseg = (p.q_seg && row_ok) ? p.q_seg[grow] : 0;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr, tO = tmem_base + 128 + lane_addr;

    float m_used = -INFINITY;   // maximum the exponentials are currently taken against (log2 units)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < nblk && ok; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[s], ph, p.status, kTimeoutAccFull, 17)) { ok = false; break; }
      tc_fence_after();
      uint32_t r[64];
      tmem_ld32(tS + s * FWD_BN, r);
      tmem_ld32(tS + s * FWD_BN + 32, r + 32);
      tmem_wait_ld();
      const int kv0 = (blk_lo + j) * FWD_BN;
      const bool need_mask = (p.causal && kv0 + FWD_BN - 1 > qpos_min) || (kv0 + FWD_BN > p.Sk) ||
                             (p.window > 0 && qpos_max - kv0 >= p.window) || p.q_seg != nullptr;
      float t[64];
      float m_blk = -INFINITY;
      if (need_mask) {
        const int* ks = p.kv_seg ? p.kv_seg + (long long)b * p.Sk : nullptr;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int kp = kv0 + c;
          bool keep = kp < p.Sk && row_ok;
          if (p.causal) keep = keep && kp <= qpos;
          if (p.window > 0) keep = keep && (qpos - kp < p.window);
          if (ks) keep = keep && (kp < p.Sk) && (__ldg(ks + min(kp, p.Sk - 1)) == qseg);
          t[c] = keep ? __uint_as_float(r[c]) * p.scale_log2 : -INFINITY;
          m_blk = fmaxf(m_blk, t[c]);
        }
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          t[c] = __uint_as_float(r[c]) * p.scale_log2;
          m_blk = fmaxf(m_blk, t[c]);
        }
      }
      // lazy running maximum
      float alpha = 1.f;
      bool rescale = false;
      if (m_blk > m_used + kRescaleThreshold || (m_used == -INFINITY && m_blk > -INFINITY)) {
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_blk);
        rescale = (m_used != -INFINITY);
        m_used = m_blk;
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      float sum = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const float p0 = exp2f(t[2 * c] - m_safe), p1 = exp2f(t[2 * c + 1] - m_safe);
        sum += p0 + p1;
        pk[c] = pack_bf16(p0, p1);
      }
      l = l * alpha + sum;
      if (j > 0) {
        if (!mbar_wait(o_done, (j - 1) & 1, p.status, kTimeoutAccFull, 18)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
          for (int c = 0; c < FWD_DV / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(tO + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
            tmem_st32(tO + c * 32, o);
          }
        }
      }
      tmem_st32(tS + s * FWD_BN, pk);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
    }

    // ---- epilogue: O / l, log-sum-exp
    if (ok && nblk > 0) ok = mbar_wait(o_done, (nblk - 1) & 1, p.status, kTimeoutAccFull, 19);
    tc_fence_after();
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    if (row_ok && p.lse) {
      const float lse = (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : INFINITY;
      p.lse[((long long)b * p.Hq + hq) * p.Sq + row] = lse;
    }
    __nv_bfloat16* orow = p.O + grow * p.ldo + (long long)hq * FWD_DV;
#pragma unroll 1
    for (int c = 0; c < FWD_DV / 32; ++c) {
      uint32_t o[32];
      if (nblk > 0 && ok) {
        tmem_ld32(tO + c * 32, o);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) o[e] = 0;
      }
      if (row_ok) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(o[8 * v + e]) * inv_l;
          *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) =
              make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

template <int DQK>
cudaError_t launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnFwdParams& p,
                       cudaStream_t stream) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<DQK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FwdSmem<DQK>::TOTAL);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  dim3 grid((p.Sq + FWD_BM - 1) / FWD_BM, p.Hq, p.B);
  attn_fwd_kernel<DQK><<<grid, FWD_THREADS, FwdSmem<DQK>::TOTAL, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace tpb

using namespace tpb;

// q: [B*Sq, ...] with row pitch ldq and head h at column h*dqk; k, v likewise (v heads are 128 wide).
extern "C" int tpb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                            int Hq, int Hkv, int dqk, int dv, long long ldq, long long ldk, long long ldv,
                            long long ldo, float scale, int causal, int window, const int* q_pos, const int* q_seg,
                            const int* kv_seg, void* stream_) {
  if (dv != 128 || (dqk != 128 && dqk != 192) || Hq % Hkv) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -2;
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  CUtensorMap tq, tk, tv;
  if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, FWD_BM)) return -3;
  if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, FWD_BN)) return -4;
  if (make_tmap_3d(&tv, v, dv, (uint64_t)B * Sk, Hkv, ldv, dv, 64, FWD_BN)) return -5;
  AttnFwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal; p.window = window;
  p.q_pos = q_pos; p.q_seg = q_seg; p.kv_seg = kv_seg;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.lse = lse;
  p.status = status_block();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = dqk == 128 ? launch_fwd<128>(tq, tk, tv, p, stream) : launch_fwd<192>(tq, tk, tv, p, stream);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
