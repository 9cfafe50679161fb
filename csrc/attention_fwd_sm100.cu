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

#include <cstdlib>

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
  float softcap_in;    // logit soft cap: scores become cap * tanh(q.k * scale / cap); this is scale / cap (0: off)
                       // and scale_log2 is then cap * log2(e).  Only attn_fwd_kernel applies it.
  int causal, window;
  const int* q_pos;    // [B*Sq] or null
  const int* q_seg;    // [B*Sq] or null
  const int* kv_seg;   // [B*Sk] or null
  __nv_bfloat16* O;
  long long ldo;       // elements between consecutive tokens of O
  float* lse;          // [B, Hq, Sq]
  int* status;
  // Context-parallel K/V exchange fused into the kernel (cp_world > 1): the first cp_copiers CTAs
  // push this rank's K/V rows into every rank's gathered buffers (plain 16-byte stores over NVLink,
  // natural key order, so the zig-zag permutation costs nothing) and raise one flag per 128 keys in
  // every rank's flag array; the TMA producer of an attention CTA waits (bounded) for the flag of a
  // key block before loading it from the local gathered buffer.
  int cp_world, cp_rank, cp_copiers, cp_zigzag;
  int cp_s_local;                      // keys per rank and batch row (multiple of 128; of 256 if zig-zag)
  const __nv_bfloat16* cp_k_src;       // this rank's keys  [B * cp_s_local rows], row pitch cp_ld_k
  const __nv_bfloat16* cp_v_src;
  long long cp_ld_k, cp_ld_v;
  int cp_row_elems;                    // Hkv * 128: elements per key row in the gathered buffers
  __nv_bfloat16* cp_k_dst[8];          // gathered K [B * Sk, Hkv * 128] of every rank
  __nv_bfloat16* cp_v_dst[8];
  __nv_bfloat16* cp_k_mc;              // NVSwitch multicast addresses of the gathered K / V (one store reaches
  __nv_bfloat16* cp_v_mc;              // every rank), or null: one store per rank
  unsigned* cp_flags[8];               // [B * Sk / 128] of every rank
  unsigned cp_epoch;
};

constexpr int CP_CHUNK = 128;          // keys per flag

// Build with -DTPB_ATTN_PROF to accumulate per-phase cycle counts of one softmax thread and of the
// MMA thread of every CTA (read back with tpb_attn_fwd_prof_read).  Not part of normal builds.
#ifdef TPB_ATTN_PROF
__device__ unsigned long long g_fwd_prof[16];
#define PROF_DECL_(n) unsigned prof_acc[n] = {}; unsigned prof_t = (unsigned)clock();
#define PROF_MARK_(i) { const unsigned now_ = (unsigned)clock(); prof_acc[i] += now_ - prof_t; prof_t = now_; }
#define PROF_FLUSH_(base, n, on) if (on) { for (int i_ = 0; i_ < n; ++i_) atomicAdd(&g_fwd_prof[base + i_], (unsigned long long)prof_acc[i_]); }
#else
#define PROF_DECL_(n)
#define PROF_MARK_(i)
#define PROF_FLUSH_(base, n, on)
#endif
// -DTPB_ATTN_ABLATE=<bits> removes parts of the v2 softmax to see what each costs (results are wrong):
// 1 no exponentials, 2 no row maximum / exchange barrier, 4 no score loads, 8 no P stores
#ifndef TPB_ATTN_ABLATE
#define TPB_ATTN_ABLATE 0
#endif
#ifdef TPB_ATTN_PROF
#define TPB_ATTN_PROF_LEVEL TPB_ATTN_PROF
#else
#define TPB_ATTN_PROF_LEVEL 0
#endif
// counters of the MMA thread (which has registers to spare) with -DTPB_ATTN_PROF=1 or 2, those of a
// softmax thread (they cost it registers and perturb what they measure) only with -DTPB_ATTN_PROF=2
#define PROF_I_DECL(n) PROF_DECL_(n)
#define PROF_I_MARK(i) PROF_MARK_(i)
#define PROF_I_FLUSH(base, n, on) PROF_FLUSH_(base, n, on)
#if defined(TPB_ATTN_PROF) && TPB_ATTN_PROF >= 2
#define PROF_DECL(n) PROF_DECL_(n)
#define PROF_MARK(i) PROF_MARK_(i)
#define PROF_FLUSH(base, n, on) PROF_FLUSH_(base, n, on)
#define PROF_COUNT(i) prof_acc[i] += 1;
#else
#define PROF_DECL(n)
#define PROF_MARK(i)
#define PROF_FLUSH(base, n, on)
#define PROF_COUNT(i)
#endif
// -DTPB_ATTN_PROF=3: clocks per MMA issue of tile a's issuer (slots 0-7: P V k-steps, 8-15: Q K^T k-steps)
#if defined(TPB_ATTN_PROF) && TPB_ATTN_PROF == 3
#define PROF_K_DECL unsigned kacc[16] = {}; unsigned kt = 0;
#define PROF_K_START kt = (unsigned)clock();
#define PROF_K_MARK(i) { const unsigned now_ = (unsigned)clock(); kacc[i] += now_ - kt; kt = now_; }
#define PROF_K_FLUSH(on) if (on) { for (int i_ = 0; i_ < 16; ++i_) atomicAdd(&g_fwd_prof[i_], (unsigned long long)kacc[i_]); }
#else
#define PROF_K_DECL
#define PROF_K_START
#define PROF_K_MARK(i)
#define PROF_K_FLUSH(on)
#endif
#ifdef TPB_ATTN_PROF
#define PROF_I_COUNT(i) prof_acc[i] += 1;
#else
#define PROF_I_COUNT(i)
#endif

// Natural position of local key row t (0 <= t < s_local) of rank r.
__device__ __forceinline__ int cp_natural_pos(int t, int r, int world, int s_local, int zigzag) {
  if (!zigzag) return r * s_local + t;
  const int half = s_local / 2;
  return t < half ? r * half + t : (2 * world - 1 - r) * half + (t - half);
}

// Copier CTA: chunks c, c + G, ... (128 key rows of one batch row each) of the local K and V.
__device__ void cp_pusher(const AttnFwdParams& p) {
  const int chunks_per_row = p.cp_s_local / CP_CHUNK;
  const int n_chunks = p.B * chunks_per_row;
  const int vec_per_row = p.cp_row_elems / 8;            // 16-byte vectors per key row
  const int nvec = CP_CHUNK * vec_per_row;
  for (int ch = blockIdx.x; ch < n_chunks; ch += p.cp_copiers) {
    const int b = ch / chunks_per_row, t0 = (ch % chunks_per_row) * CP_CHUNK;
    const int pos0 = cp_natural_pos(t0, p.cp_rank, p.cp_world, p.cp_s_local, p.cp_zigzag);
    const long long dst_row0 = (long long)b * p.Sk + pos0;
    for (int which = 0; which < 2; ++which) {
      const __nv_bfloat16* src = which == 0 ? p.cp_k_src : p.cp_v_src;
      const long long ld = which == 0 ? p.cp_ld_k : p.cp_ld_v;
      const long long src_row0 = (long long)b * p.cp_s_local + t0;
      for (int i = threadIdx.x; i < nvec; i += 8 * blockDim.x) {
        uint4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int k = i + u * blockDim.x;
          if (k < nvec)
            v[u] = *reinterpret_cast<const uint4*>(src + (src_row0 + k / vec_per_row) * ld + (k % vec_per_row) * 8);
        }
        __nv_bfloat16* mc = which == 0 ? p.cp_k_mc : p.cp_v_mc;
        if (mc != nullptr) {
          uint4* dst = reinterpret_cast<uint4*>(mc + dst_row0 * p.cp_row_elems);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int k = i + u * blockDim.x;
            if (k < nvec)
              asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + k),
                           "f"(__uint_as_float(v[u].x)), "f"(__uint_as_float(v[u].y)),
                           "f"(__uint_as_float(v[u].z)), "f"(__uint_as_float(v[u].w))
                           : "memory");
          }
          continue;
        }
        for (int r = 0; r < p.cp_world; ++r) {
          uint4* dst = reinterpret_cast<uint4*>((which == 0 ? p.cp_k_dst[r] : p.cp_v_dst[r]) +
                                                dst_row0 * p.cp_row_elems);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int k = i + u * blockDim.x;
            if (k < nvec) dst[k] = v[u];
          }
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const long long f = (long long)b * (p.Sk / CP_CHUNK) + pos0 / CP_CHUNK;
      for (int r = 0; r < p.cp_world; ++r)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.cp_flags[r] + f), "r"(p.cp_epoch) : "memory");
    }
  }
}

// Bounded wait for the flag of the 128-key chunk that holds key `kv0` of batch row `b`.
__device__ __forceinline__ bool cp_wait_keys(const AttnFwdParams& p, int b, int kv0) {
  const unsigned* f = p.cp_flags[p.cp_rank] + (long long)b * (p.Sk / CP_CHUNK) + kv0 / CP_CHUNK;
  long long t0 = 0;
  int spins = 0;
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (v == p.cp_epoch) break;
    if (++spins == 64) {
      spins = 0;
      if (t0 == 0) t0 = clock64();
      else if (clock64() - t0 > kSpinBudgetCycles) { report(p.status, kTimeoutPeerFlag, 51); return false; }
      __nanosleep(100);
    }
  }
  asm volatile("fence.proxy.async;" ::: "memory");   // the rows were written with generic stores
  return true;
}


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
  int bx = blockIdx.x, by = blockIdx.y, bz = blockIdx.z;
  if (p.cp_world > 1) {
    // one-dimensional grid: the copier CTAs come first so that they are scheduled first
    if ((int)blockIdx.x < p.cp_copiers) {
      cp_pusher(p);
      return;
    }
    const int id = (int)blockIdx.x - p.cp_copiers;
    bx = id % n_qtiles; by = (id / n_qtiles) % p.Hq; bz = id / (n_qtiles * p.Hq);
  }
  const int qt = n_qtiles - 1 - bx;   // heaviest (latest) tiles first under a causal mask
  const int hq = by, b = bz;
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
        if (p.cp_world > 1 && !cp_wait_keys(p, b, (blk_lo + j) * FWD_BN)) break;
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
      if (p.softcap_in != 0.f) {
#pragma unroll
        for (int c = 0; c < 64; ++c) r[c] = __float_as_uint(tanh_approx(__uint_as_float(r[c]) * p.softcap_in));
      }
      // masked scores become -inf (the scale is positive, so masking and the row maximum work on
      // the raw scores); the maximum runs as four chains of three-input max instructions
      float m_blk;
      if (need_mask) {
        const int* ks = p.kv_seg ? p.kv_seg + (long long)b * p.Sk : nullptr;
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int kp = kv0 + c;
          bool keep = kp < p.Sk && row_ok;
          if (p.causal) keep = keep && kp <= qpos;
          if (p.window > 0) keep = keep && (qpos - kp < p.window);
          if (ks) keep = keep && (kp < p.Sk) && (__ldg(ks + min(kp, p.Sk - 1)) == qseg);
          r[c] = keep ? r[c] : 0xff800000u;
        }
      }
      {
        float mx[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) mx[e] = fmaxf(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
#pragma unroll
        for (int c = 8; c < 64; c += 8)
#pragma unroll
          for (int e = 0; e < 4; ++e)
            mx[e] = fmax3(mx[e], __uint_as_float(r[c + 2 * e]), __uint_as_float(r[c + 2 * e + 1]));
        m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
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
      // P = exp2(s * c - m): the multiply-add and the row sum on packed pairs
      const f32x2 c2 = f2_pack(p.scale_log2, p.scale_log2), nm2 = f2_pack(-m_safe, -m_safe);
      f32x2 acc[2] = {0ull, 0ull};
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        float p0, p1;
        f2_unpack(f2_fma(f2_pack_bits(r[2 * c], r[2 * c + 1]), c2, nm2), p0, p1);
        p0 = ex2_approx(p0);
        p1 = ex2_approx(p1);
        acc[c & 1] = f2_add(acc[c & 1], f2_pack(p0, p1));
        pk[c] = pack_bf16(p0, p1);
      }
      float s0, s1;
      f2_unpack(f2_add(acc[0], acc[1]), s0, s1);
      const float sum = s0 + s1;
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

// ------------------------------------------------------------------------------------------
// Head dim 128: two 128-row query tiles per CTA, 128-key steps.
//
// Every MMA is 128 x 128 x 16 (full tensor rate with operands in shared memory; the 64-key steps
// of the kernel above are bound by operand fetch), each K/V tile is loaded once for 256 query
// rows, and the two tiles alternate on the tensor core: while the softmax warps of tile a work on
// step j, the tensor core runs P V and the next Q K^T of tile b.
//
//   warp 0      TMA producer: both Q tiles once, then 2-stage rings of 128-key K and V tiles.
//   warp 1      MMA issuer.  Per step j and tile x: O_x += P_x(j) V_j, then S_x(j+1) = Q_x K_{j+1}^T
//               into the columns P_x(j) has just been read from (S and P share TMEM columns).
//   warps 4-11  softmax of tile a, warps 12-19 softmax of tile b: two threads per query row (TMEM lane),
//               one for keys [0,64) and one for keys [64,128) of the step; the two exchange their partial
//               row maximum through shared memory.  Two warps per scheduler and tile hide each other's
//               TMEM, MUFU and instruction-fetch latencies; every fourth pair of exponentials runs on
//               the FMA pipe.  (Warps 2-3 idle: roles are laid out by warpgroup so that registers can
//               move between them.)
//   TMEM        S_a [0,128)  S_b [128,256)  O_a [256,384)  O_b [384,512)
// ------------------------------------------------------------------------------------------
// 2^x for x <= 0 on the FMA pipe (no MUFU): round-to-nearest split x = n + f with the 1.5 * 2^23
// trick, a degree-3 polynomial for 2^f on [-0.5, 0.5] (relative error 8e-5, far below the bf16
// rounding of the result) and an integer add of n into the exponent.  -inf gives 0.
__device__ __forceinline__ float exp2_fma(float x) {
  x = fmaxf(x, -125.f);
  const float fl = x + 12582912.f;
  const float f = x - (fl - 12582912.f);
  float pl = fmaf(0.05508868f, f, 0.24260405f);
  pl = fmaf(pl, f, 0.69327623f);
  pl = fmaf(pl, f, 0.99992895f);
  return __int_as_float(__float_as_int(pl) + (__float_as_int(fl) << 23));
}

// The same for a packed pair: six packed FMA-pipe instructions, two clamps and two integer
// multiply-adds for two results.
__device__ __forceinline__ void exp2_fma_pair(f32x2 x, float& r0, float& r1) {
  float x0, x1;
  f2_unpack(x, x0, x1);
  x = f2_pack(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const f32x2 magic = f2_pack(12582912.f, 12582912.f), neg_magic = f2_pack(-12582912.f, -12582912.f);
  const f32x2 fl = f2_add(x, magic);
  const f32x2 f = f2_sub(x, f2_add(fl, neg_magic));
  f32x2 pl = f2_fma(f2_pack(0.05508868f, 0.05508868f), f, f2_pack(0.24260405f, 0.24260405f));
  pl = f2_fma(pl, f, f2_pack(0.69327623f, 0.69327623f));
  pl = f2_fma(pl, f, f2_pack(0.99992895f, 0.99992895f));
  float p0, p1, n0, n1;
  f2_unpack(pl, p0, p1);
  f2_unpack(fl, n0, n1);
  r0 = __int_as_float(__float_as_int(p0) + (__float_as_int(n0) << 23));
  r1 = __int_as_float(__float_as_int(p1) + (__float_as_int(n1) << 23));
}

constexpr int F2_T = 128;                 // tile edge: rows per query tile, keys per step
constexpr int F2_THREADS = 640;            // warpgroup 0: TMA + MMA warps (two idle), warpgroups 1-2 / 3-4: softmax of tile a / b
// Registers move from the copy / MMA warpgroup to the softmax warpgroups, whose threads hold 64 scores
// each (spills go through the same L1 / shared-memory port the MMAs fetch their operands from and stall
// the whole pipeline).  setmaxnreg.inc can only take what the same CTA released with setmaxnreg.dec (the
// pool is the CTA's allocation at launch) and blocks for ever when that is less than it asks for, so the
// budget must balance against the count the kernel is launched with; the host checks that count.
constexpr int F2_REGS_LAUNCH = 96, F2_REGS_IO = 64, F2_REGS_SOFTMAX = 104;
static_assert(128 * (F2_REGS_LAUNCH - F2_REGS_IO) >= 512 * (F2_REGS_SOFTMAX - F2_REGS_LAUNCH),
              "the softmax warpgroups would wait for registers nobody releases");
constexpr int F2_TILE_BYTES = F2_T * 128 * 2;   // 32 KB
namespace f2 {
constexpr int OFF_Q = 0;                          // two tiles
constexpr int OFF_K = 2 * F2_TILE_BYTES;          // two stages
constexpr int OFF_V = OFF_K + 2 * F2_TILE_BYTES;
constexpr int OFF_BAR = OFF_V + 2 * F2_TILE_BYTES;
constexpr int OFF_X = OFF_BAR + 256;              // float [2 tiles][2 step parities][2 halves][128 rows]
constexpr int TOTAL = OFF_X + 2 * 2 * 2 * F2_T * 4 + 1024;
}  // namespace f2

__global__ void __launch_bounds__(F2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnFwdParams p) {
  using namespace f2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;    // [2 tiles]
  uint64_t* p_full = bars + 11;   // [2 tiles], count 256
  uint64_t* o_done = bars + 13;   // [2 tiles]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  int* tile_minmax = reinterpret_cast<int*>(bars + 16);  // [2 tiles][2]
  int* pair_fail = reinterpret_cast<int*>(bars + 18);    // [2 tiles][4 quarters][2 halves]: that softmax warp gave up waiting

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_ctiles = (p.Sq + 2 * F2_T - 1) / (2 * F2_T);
  const int ct = n_ctiles - 1 - (int)(blockIdx.x / (p.Hq * p.B));   // heaviest (latest) rows first
  const int hq = (blockIdx.x / p.B) % p.Hq, b = blockIdx.x % p.B;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = ct * 2 * F2_T;
  const int pos_off = p.Sk - p.Sq;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 256); mbar_init(&o_done[i], 1);
      for (int w = 0; w < 8; ++w) pair_fail[8 * i + w] = 0;
      tile_minmax[2 * i] = 0x7fffffff;
      tile_minmax[2 * i + 1] = -0x7fffffff;
    }
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

  // position range of each query tile
  if (threadIdx.x < 2 * F2_T) {
    const int r = q0 + threadIdx.x;
    if (r < p.Sq) {
      const int qp = p.q_pos ? p.q_pos[(long long)b * p.Sq + r] : r + pos_off;
      atomicMin(&tile_minmax[2 * (threadIdx.x / F2_T)], qp);
      atomicMax(&tile_minmax[2 * (threadIdx.x / F2_T) + 1], qp);
    }
  }
  __syncthreads();
  const int nblk_total = (p.Sk + F2_T - 1) / F2_T;
  int lo[2], hi[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int mn = tile_minmax[2 * x], mx = tile_minmax[2 * x + 1];
    hi[x] = p.causal ? min(nblk_total, mx / F2_T + 1) : nblk_total;
    lo[x] = (p.window > 0) ? max(0, (mn - p.window + 1) / F2_T) : 0;
    if (mx < 0) hi[x] = 0;
    if (hi[x] <= lo[x]) { lo[x] = 0; hi[x] = 0; }
  }
  const int any = (hi[0] > lo[0]) || (hi[1] > lo[1]);
  const int blk_lo = !any ? 0 : ((hi[0] > lo[0] && hi[1] > lo[1]) ? min(lo[0], lo[1]) : (hi[0] > lo[0] ? lo[0] : lo[1]));
  const int blk_hi = max(hi[0], hi[1]);
  const int nblk = any ? blk_hi - blk_lo : 0;
  auto active = [&](int x, int j) { const int blk = blk_lo + j; return blk >= lo[x] && blk < hi[x]; };

  // a softmax thread keeps the 128 scores of its row in registers: the copy / MMA warpgroup hands its
  // registers over (with 168 per thread for everybody the scores spilled to local memory)
  if (warp < 4) {
  setmaxnreg_dec<F2_REGS_IO>();
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && nblk > 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 2 * F2_TILE_BYTES);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_3d(smem + OFF_Q + x * F2_TILE_BYTES + c * (F2_T * 128), &tmQ, q_full, c * 64,
                      b * p.Sq + q0 + x * F2_T, hq);
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = b * p.Sk + (blk_lo + j) * F2_T;
        if (!mbar_wait(&k_empty[s], ph ^ 1, p.status, kTimeoutStageFree, 41)) break;
        mbar_expect_tx(&k_full[s], F2_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_3d(smem + OFF_K + s * F2_TILE_BYTES + c * (F2_T * 128), &tmK, &k_full[s], c * 64, row, hkv);
        if (!mbar_wait(&v_empty[s], ph ^ 1, p.status, kTimeoutStageFree, 42)) break;
        mbar_expect_tx(&v_full[s], F2_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c)
          tma_load_3d(smem + OFF_V + s * F2_TILE_BYTES + c * (F2_T * 128), &tmV, &v_full[s], c * 64, row, hkv);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // One thread issues for both tiles, alternating.  (One thread per tile was tried: left to
    // themselves the two fall into step, both tiles in their softmax at the same time; made to take
    // turns through a pair of mbarriers they were slower than this single thread, 0.655 against
    // 0.594 ms at S = 8192.)
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t id_qk = make_idesc_bf16(F2_T, F2_T, false, false);
      constexpr uint32_t id_pv = make_idesc_bf16(F2_T, FWD_DV, false, true);
      constexpr uint32_t hi_w = smem_desc_hi(1024);
      const uint32_t qlo[2] = {smem_desc_lo(smem_u32(smem + OFF_Q), 16),
                               smem_desc_lo(smem_u32(smem + OFF_Q + F2_TILE_BYTES), 16)};
      const uint32_t k0 = smem_u32(smem + OFF_K), v0 = smem_u32(smem + OFF_V);
      bool ok = mbar_wait(q_full, 0, p.status, kTimeoutTmaFull, 43);
      tc_fence_after();
      int steps[2] = {0, 0};   // steps issued per tile (barrier phases)
      PROF_K_DECL
      auto issue_s = [&](int x, int j) {   // S_x = Q_x K_j^T
        PROF_K_START
        const uint32_t klo = smem_desc_lo(k0 + (j & 1) * F2_TILE_BYTES, 16);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t kk = (uint32_t)(((k >> 2) * (F2_T * 128) + (k & 3) * 32) >> 4);
          mma_ss_w(tmem_base + x * F2_T, qlo[x] + kk, hi_w, klo + kk, hi_w, id_qk, k != 0);
          PROF_K_MARK(8 + k)
        }
        tc_commit(&s_full[x]);
      };
      auto issue_pv = [&](int x, int j, bool first) {   // O_x += P_x V_j
        PROF_K_START
        const uint32_t vlo = smem_desc_lo(v0 + (j & 1) * F2_TILE_BYTES, F2_T * 128);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          mma_ts_w(tmem_base + 256 + x * F2_T, tmem_base + x * F2_T + k * 8, vlo + (uint32_t)((k * 2048) >> 4), hi_w,
                   id_pv, (!first) | (k != 0));
          PROF_K_MARK(k)
        }
        tc_commit(&o_done[x]);
      };
      if (ok) ok = mbar_wait(&k_full[0], 0, p.status, kTimeoutTmaFull, 44);
      tc_fence_after();
      if (ok) {
        if (active(0, 0)) issue_s(0, 0);
        if (active(1, 0)) issue_s(1, 0);
        tc_commit(&k_empty[0]);
      }
      PROF_I_DECL(7)
      for (int j = 0; j < nblk && ok; ++j) {
        const int jn = j + 1;
        // the tiles this step needs were requested a step ago: these waits are off the softmax handshake
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1, p.status, kTimeoutTmaFull, 46)) { ok = false; break; }
        if (jn < nblk && !mbar_wait(&k_full[jn & 1], (jn >> 1) & 1, p.status, kTimeoutTmaFull, 47)) { ok = false; break; }
        PROF_I_MARK(5)
#pragma unroll
        for (int x = 0; x < 2; ++x) {
          if (active(x, j)) {
            PROF_I_MARK(0)
            if (!mbar_wait(&p_full[x], steps[x] & 1, p.status, kTimeoutSoftmax, 45)) { ok = false; break; }
            PROF_I_MARK(1)
            PROF_I_COUNT(2)
            tc_fence_after();
            issue_pv(x, j, steps[x] == 0);
            ++steps[x];
            PROF_I_MARK(4)
          }
          if (jn < nblk && active(x, jn)) {
            issue_s(x, jn);
            PROF_I_MARK(6)
          }
        }
        if (!ok) break;
        tc_commit(&v_empty[j & 1]);
        if (jn < nblk) tc_commit(&k_empty[jn & 1]);
        PROF_I_MARK(3)
      }
      PROF_I_FLUSH(8, 7, TPB_ATTN_PROF_LEVEL != 3)
      PROF_K_FLUSH(true)
    }
  }
  } else {
    setmaxnreg_inc<F2_REGS_SOFTMAX>();
    // ------------------------------------------------------------------ softmax + epilogue
    const int x = (warp - 4) >> 3;                // query tile of this warp
    const int h = ((warp - 4) >> 2) & 1;          // key half of the step / column half of O
    const int q = warp & 3;                       // TMEM lane quarter (four consecutive warps cover all four)
    const int r_local = q * 32 + lane;
    const int row = q0 + x * F2_T + r_local;
    const bool row_ok = row < p.Sq;
    const long long grow = (long long)b * p.Sq + row;
    const int qpos = row_ok ? (p.q_pos ? p.q_pos[grow] : row + pos_off) : -1;
    const int qseg = (p.q_seg && row_ok) ? p.q_seg[grow] : 0;
    const int qpos_min = tile_minmax[2 * x], qpos_max = tile_minmax[2 * x + 1];
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tS = tmem_base + x * F2_T + lane_addr, tO = tmem_base + 256 + x * F2_T + lane_addr;
    const int* ks = p.kv_seg ? p.kv_seg + (long long)b * p.Sk : nullptr;
    const int win = p.window > 0 ? p.window : 0x7fffffff;
    const int kmax = p.causal ? min(qpos, p.Sk - 1) : p.Sk - 1;   // keep needs kp <= kmax
    float* xch = reinterpret_cast<float*>(smem + OFF_X) + x * (4 * F2_T);   // [parity][half][row]
    // The two warps that share the rows of a TMEM lane quarter (one per key half) synchronise on a named
    // barrier of their own: 64 threads, so no warp waits for the slowest of the tile's eight.
    const int pair_bar = 1 + 4 * x + q;
    int* my_fail = pair_fail + 8 * x + 2 * q;     // [2 halves] of this pair

    float m_used = -INFINITY;   // maximum the exponentials are currently taken against (log2 units)
    float l = 0.f;              // sum over this thread's keys
    bool ok = true;
    int step = 0;
    PROF_DECL(6)
    for (int j = 0; j < nblk && ok; ++j) {
      if (!active(x, j)) continue;
      const bool waited = mbar_wait(&s_full[x], step & 1, p.status, kTimeoutAccFull, 48);
      if (__any_sync(0xffffffffu, !waited) && lane == 0) my_fail[h] = 1;
      tc_fence_after();
      PROF_MARK(0)
      const int kv0 = (blk_lo + j) * F2_T + 64 * h;
      const bool need_mask = (p.causal && kv0 + 63 > qpos_min) || (kv0 + 64 > p.Sk) ||
                             (p.window > 0 && qpos_max - kv0 >= p.window) || p.q_seg != nullptr;
      uint32_t r[64];
      if (!(TPB_ATTN_ABLATE & 4)) {
        tmem_ld32(tS + 64 * h, r);
        tmem_ld32(tS + 64 * h + 32, r + 32);
        tmem_wait_ld();
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) r[c] = __float_as_uint(-1.f - c - lane);
      }
      PROF_MARK(1)
      if (need_mask) {
        // key c of this half is kept iff lo_c < c <= hi_c (causal / window / sequence end / row padding)
        const int hi_c = row_ok ? kmax - kv0 : -1;
        const int lo_c = qpos - win - kv0;
#pragma unroll
        for (int c = 0; c < 64; ++c) r[c] = (c <= hi_c && c > lo_c) ? r[c] : 0xff800000u;   // -inf
        if (ks) {
          const int* kseg = ks + kv0;
          const int last = p.Sk - 1 - kv0;
#pragma unroll
          for (int c = 0; c < 64; ++c) r[c] = (__ldg(kseg + min(c, last)) == qseg) ? r[c] : 0xff800000u;
        }
      }
      float mx[8];   // eight independent chains of three-input max instructions
#pragma unroll
      for (int c = 0; c < 64; c += 16)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a0 = __uint_as_float(r[c + 2 * e]), a1 = __uint_as_float(r[c + 2 * e + 1]);
          mx[e] = (c == 0) ? fmaxf(a0, a1) : fmax3(mx[e], a0, a1);
        }
      float m_blk = fmax3(fmax3(mx[0], mx[1], mx[2]), fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7]));
      // the other half's maximum.  Both warps of a pair reach the barrier in every step they enter and
      // leave the loop together: a warp whose wait ran out raises its flag before the barrier, and both
      // read both flags after it.
      float* slot = xch + (step & 1) * (2 * F2_T);
      if (!(TPB_ATTN_ABLATE & 2)) {
        slot[h * F2_T + r_local] = m_blk;
        PROF_MARK(2)
        named_bar_sync(pair_bar, 64);
        if (*reinterpret_cast<volatile int*>(&my_fail[0]) | *reinterpret_cast<volatile int*>(&my_fail[1])) { ok = false; break; }
        m_blk = fmaxf(m_blk, slot[(h ^ 1) * F2_T + r_local]) * p.scale_log2;   // scale > 0: max(s) * c == max(s * c)
      } else {
        m_blk = 0.f;
      }
      PROF_MARK(3)
      // lazy running maximum (both threads of the row take the same decision)
      float alpha = 1.f;
      bool rescale = false;
      if (m_blk > m_used + kRescaleThreshold || (m_used == -INFINITY && m_blk > -INFINITY)) {
        alpha = (m_used == -INFINITY) ? 0.f : exp2f(m_used - m_blk);
        rescale = (m_used != -INFINITY);
        m_used = m_blk;
      }
      const float m_safe = (m_used == -INFINITY) ? 0.f : m_used;
      // The previous P V of this tile is complete: its commit precedes the one of this S.  Each thread
      // rescales its half of the O columns.
      if (step > 0 && __any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + 64 * h + c * 32, o);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
          tmem_st32(tO + 64 * h + c * 32, o);
        }
      }
      // P = exp2(s * c - m) as packed bf16 over score columns [32 h, 32 h + 32) (the other thread has
      // read its scores before the barrier above; masked scores are -inf and give exactly 0).  The
      // exponentials of a step cost as many MUFU cycles as its MMAs cost tensor cycles, so every
      // fourth pair is evaluated on the FMA pipe (exp2_fma_pair).
      const f32x2 c2 = f2_pack(p.scale_log2, p.scale_log2), nm2 = f2_pack(-m_safe, -m_safe);
      f32x2 acc[2] = {0ull, 0ull};
#pragma unroll
      for (int ch = 0; ch < 2; ++ch) {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          const f32x2 t = f2_fma(f2_pack_bits(r[32 * ch + 2 * c], r[32 * ch + 2 * c + 1]), c2, nm2);
          float p0, p1;
          if (TPB_ATTN_ABLATE & 1) {
            f2_unpack(t, p0, p1);
          } else if ((c & 3) == 3) {
            exp2_fma_pair(t, p0, p1);
          } else {
            f2_unpack(t, p0, p1);
            p0 = ex2_approx(p0);
            p1 = ex2_approx(p1);
          }
          acc[c & 1] = f2_add(acc[c & 1], f2_pack(p0, p1));
          pk[c] = pack_bf16(p0, p1);
        }
        if (!(TPB_ATTN_ABLATE & 8)) tmem_st16(tS + 32 * h + 16 * ch, pk);
        else if (pk[3] == 0x12345678u) l += 1.f;
      }
      float s0, s1;
      f2_unpack(f2_add(acc[0], acc[1]), s0, s1);
      l = l * alpha + (s0 + s1);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[x]);
      ++step;
      PROF_MARK(4)
      PROF_COUNT(5)
    }
    PROF_FLUSH(0, 6, warp == 4 && lane == 0)

    // ---- epilogue: O / l, log-sum-exp
    if (ok && step > 0) ok = mbar_wait(&o_done[x], (step - 1) & 1, p.status, kTimeoutAccFull, 50);
    tc_fence_after();
    // row sum = sum of the two halves (the exchange slots of parity `step` were last read two steps ago)
    float* slot = xch + (step & 1) * (2 * F2_T);
    slot[h * F2_T + r_local] = l;
    named_bar_sync(pair_bar, 64);
    l += slot[(h ^ 1) * F2_T + r_local];
    const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
    if (row_ok && p.lse && h == 0) {
      const float lse = (l > 0.f) ? (m_used + log2f(l)) * 0.6931471805599453f : INFINITY;
      p.lse[((long long)b * p.Hq + hq) * p.Sq + row] = lse;
    }
    __nv_bfloat16* orow = p.O + grow * p.ldo + (long long)hq * FWD_DV + 64 * h;
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      uint32_t o[32];
      if (step > 0 && ok) {
        tmem_ld32(tO + 64 * h + c * 32, o);
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
    tmem_dealloc(tmem_base, 512);
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
// `softcap` > 0 caps the scores as softcap * tanh(q.k * scale / softcap) before the softmax.
extern "C" int tpb_attn_fwd_softcap(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq,
                                    int Sk, int Hq, int Hkv, int dqk, int dv, long long ldq, long long ldk,
                                    long long ldv, long long ldo, float scale, int causal, int window,
                                    const int* q_pos, const int* q_seg, const int* kv_seg, float softcap,
                                    void* stream_) {
  if (dv != 128 || (dqk != 128 && dqk != 192) || Hq % Hkv) return -2;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -2;
  if (B <= 0 || Sq <= 0 || Sk <= 0) return 0;
  // TPB_ATTN_FWD_V2=1 selects the two-tile, 128-key-step kernel.  It is correct and 3-4 % ahead of the
  // 64-key kernel at B=1, S=8192, 32/8 heads (0.565-0.571 against 0.590 ms on one box), no more: with
  // its softmax threads doing nothing it still takes 0.513 ms, the time of its MMA stream and of the
  // handshakes of the single issuing thread.  Earlier forms: one thread per row with 168 registers
  // spilled the 128 scores (0.66 ms); one softmax warpgroup serving both tiles (six warps, 210
  // registers) was slower still (1.04 ms), a single warp per scheduler cannot hide the TMEM and
  // MUFU latencies.
  static const bool use_v2 = []() { const char* v = getenv("TPB_ATTN_FWD_V2"); return v && v[0] == '1'; }();
  if (dqk == 128 && use_v2 && !(softcap > 0.f)) {
    // two query tiles per CTA, 128-key steps
    CUtensorMap tq, tk, tv;
    if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, F2_T)) return -3;
    if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, F2_T)) return -4;
    if (make_tmap_3d(&tv, v, dv, (uint64_t)B * Sk, Hkv, ldv, dv, 64, F2_T)) return -5;
    AttnFwdParams p{};
    p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.causal = causal; p.window = window;
    p.q_pos = q_pos; p.q_seg = q_seg; p.kv_seg = kv_seg;
    p.O = reinterpret_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.lse = lse;
    p.status = status_block();
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(attn_fwd2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, f2::TOTAL);
      if (e != cudaSuccess) return 1000 + (int)e;
      // the register hand-over inside the kernel is balanced for exactly this launch allocation
      cudaFuncAttributes fa;
      e = cudaFuncGetAttributes(&fa, attn_fwd2_kernel);
      if (e != cudaSuccess) return 1000 + (int)e;
      if (fa.numRegs != F2_REGS_LAUNCH) return -9;
      configured = true;
    }
    const int n_ctiles = (Sq + 2 * F2_T - 1) / (2 * F2_T);
    attn_fwd2_kernel<<<n_ctiles * Hq * B, F2_THREADS, f2::TOTAL, reinterpret_cast<cudaStream_t>(stream_)>>>(tq, tk, tv, p);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : 1000 + (int)e;
  }
  CUtensorMap tq, tk, tv;
  if (make_tmap_3d(&tq, q, dqk, (uint64_t)B * Sq, Hq, ldq, dqk, 64, FWD_BM)) return -3;
  if (make_tmap_3d(&tk, k, dqk, (uint64_t)B * Sk, Hkv, ldk, dqk, 64, FWD_BN)) return -4;
  if (make_tmap_3d(&tv, v, dv, (uint64_t)B * Sk, Hkv, ldv, dv, 64, FWD_BN)) return -5;
  AttnFwdParams p{};
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.softcap_in = softcap > 0.f ? scale / softcap : 0.f;
  p.scale_log2 = (softcap > 0.f ? softcap : scale) * 1.4426950408889634f;
  p.causal = causal; p.window = window;
  p.q_pos = q_pos; p.q_seg = q_seg; p.kv_seg = kv_seg;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.lse = lse;
  p.status = status_block();
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  cudaError_t e = dqk == 128 ? launch_fwd<128>(tq, tk, tv, p, stream) : launch_fwd<192>(tq, tk, tv, p, stream);
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

extern "C" int tpb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                            int Hq, int Hkv, int dqk, int dv, long long ldq, long long ldk, long long ldv,
                            long long ldo, float scale, int causal, int window, const int* q_pos, const int* q_seg,
                            const int* kv_seg, void* stream_) {
  return tpb_attn_fwd_softcap(q, k, v, o, lse, B, Sq, Sk, Hq, Hkv, dqk, dv, ldq, ldk, ldv, ldo, scale, causal, window,
                              q_pos, q_seg, kv_seg, 0.f, stream_);
}

// Causal attention forward with the context-parallel K/V exchange fused in (head dim 128).
// q: this rank's query rows [B*Sq, ...] (row pitch ldq); k_local / v_local: this rank's
// [B*s_local] key/value rows (row pitches ld_k_local / ld_v_local, Hkv*128 elements used per row);
// k_all / v_all / flags: tables of every rank's gathered K [B*Sk, Hkv*128], gathered V and flag
// array [B*Sk/128] in symmetric memory (Sk = world * s_local); entry `rank` is this rank's own.
// k_multicast / v_multicast: multicast addresses of the same gathered buffers, or null.
// q_pos: absolute positions of the query rows.  `epoch` must differ from the previous call's, and
// all ranks must have finished reading their gathered buffers before any rank starts this call.
extern "C" int tpb_attn_fwd_cp(const void* q, const void* k_local, const void* v_local, void* const* k_all,
                               void* const* v_all, unsigned* const* flags, void* o, float* lse, int B, int Sq,
                               int s_local, int Hq, int Hkv, long long ldq, long long ld_k_local,
                               long long ld_v_local, long long ldo, float scale, const int* q_pos, int world, int rank,
                               int zigzag, int copiers, unsigned epoch, void* k_multicast, void* v_multicast,
                               void* stream_) {
  if (world < 2 || world > 8 || rank < 0 || rank >= world || Hq % Hkv) return -2;
  if ((ldq % 8) || (ld_k_local % 8) || (ld_v_local % 8) || (ldo % 8)) return -2;
  if (s_local % (zigzag ? 2 * CP_CHUNK : CP_CHUNK)) return -2;
  if (B <= 0 || Sq <= 0 || s_local <= 0) return 0;
  const int Sk = world * s_local;
  const int row_elems = Hkv * 128;
  CUtensorMap tq, tk, tv;
  if (make_tmap_3d(&tq, q, 128, (uint64_t)B * Sq, Hq, ldq, 128, 64, FWD_BM)) return -3;
  if (make_tmap_3d(&tk, k_all[rank], 128, (uint64_t)B * Sk, Hkv, row_elems, 128, 64, FWD_BN)) return -4;
  if (make_tmap_3d(&tv, v_all[rank], 128, (uint64_t)B * Sk, Hkv, row_elems, 128, 64, FWD_BN)) return -5;
  AttnFwdParams p{};
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = 1; p.window = 0;
  p.q_pos = q_pos; p.q_seg = nullptr; p.kv_seg = nullptr;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.ldo = ldo; p.lse = lse;
  p.status = status_block();
  p.cp_world = world; p.cp_rank = rank; p.cp_zigzag = zigzag; p.cp_s_local = s_local;
  const int n_chunks = B * (s_local / CP_CHUNK);
  p.cp_copiers = copiers < 1 ? 1 : (copiers > n_chunks ? n_chunks : copiers);
  p.cp_k_src = reinterpret_cast<const __nv_bfloat16*>(k_local);
  p.cp_v_src = reinterpret_cast<const __nv_bfloat16*>(v_local);
  p.cp_ld_k = ld_k_local; p.cp_ld_v = ld_v_local;
  p.cp_row_elems = row_elems;
  for (int r = 0; r < 8; ++r) {
    p.cp_k_dst[r] = r < world ? reinterpret_cast<__nv_bfloat16*>(k_all[r]) : nullptr;
    p.cp_v_dst[r] = r < world ? reinterpret_cast<__nv_bfloat16*>(v_all[r]) : nullptr;
    p.cp_flags[r] = r < world ? flags[r] : nullptr;
  }
  p.cp_epoch = epoch;
  const bool mc = k_multicast != nullptr && v_multicast != nullptr;
  p.cp_k_mc = mc ? reinterpret_cast<__nv_bfloat16*>(k_multicast) : nullptr;
  p.cp_v_mc = mc ? reinterpret_cast<__nv_bfloat16*>(v_multicast) : nullptr;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         FwdSmem<128>::TOTAL);
    if (e != cudaSuccess) return 1000 + (int)e;
    configured = true;
  }
  const int n_qtiles = (Sq + FWD_BM - 1) / FWD_BM;
  const int grid = p.cp_copiers + n_qtiles * Hq * B;
  attn_fwd_kernel<128><<<grid, FWD_THREADS, FwdSmem<128>::TOTAL, reinterpret_cast<cudaStream_t>(stream_)>>>(tq, tk, tv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

#ifdef TPB_ATTN_PROF
// Copies the 16 profiling counters to `host16` and clears them.
extern "C" int tpb_attn_fwd_prof_read(unsigned long long* host16) {
  unsigned long long zero[16] = {};
  if (cudaMemcpyFromSymbol(host16, tpb::g_fwd_prof, sizeof(zero)) != cudaSuccess) return 1;
  return cudaMemcpyToSymbol(tpb::g_fwd_prof, zero, sizeof(zero)) == cudaSuccess ? 0 : 1;
}
#endif
