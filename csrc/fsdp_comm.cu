// Building blocks of the peer-memory FSDP collectives (parallel/fsdp_comm.py).
//
// The parameter all-gather of an FSDP unit is done by the copy engines: every rank copies each peer's
// shard out of the peer's (mapped) memory into its own gathered buffer and raises one local flag per
// shard when the copy has landed; the consuming GEMMs wait on those flags inside their TMA producer
// (gemm_sm100.cu, external-gather mode), so no SM moves parameter bytes.
//
// The gradient reduce-scatter is a push into per-source staging slots followed by a reduction in a
// fixed order at the owner: the weight-gradient GEMM epilogues (and copy-engine copies for whatever
// the GEMMs did not produce) store rank r's bf16 contribution to owner o's shard into
// stage_o[r][...]; when every rank has signalled, the owner adds the slots in rank order in fp32.
// The result does not depend on arrival order and each element is rounded to bf16 once.
//
// Flags only grow (a use counter per staging slot / gather), comparisons are on the signed
// difference, and every wait is bounded: a wait that runs out reports kTimeoutPeerFlag and returns.

#include "common.cuh"
#include "tpb.h"

namespace tpb {

constexpr int kMaxPeers = 64;

struct PeerFlagTable {
  unsigned* flags[kMaxPeers];
};

__global__ void flag_set_kernel(unsigned* flag, unsigned value) {
  __threadfence();
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

// Thread t stores `value` into word `index` of peer t's flag array.  Everything this stream did
// before (kernels that stored into peer memory, copy-engine copies) is visible to a reader that
// acquires the flag.
__global__ void peer_signal_kernel(PeerFlagTable peers, int world, long long index, unsigned value) {
  const int t = threadIdx.x;
  if (t >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[t] + index), "r"(value) : "memory");
}

// Thread t waits until flags[t * stride] has reached `value`.
__global__ void flag_wait_kernel(const unsigned* flags, int n, long long stride, unsigned value, int* status,
                                 int site) {
  const int t = threadIdx.x;
  if (t >= n) return;
  const unsigned* f = flags + t * stride;
  const long long t0 = clock64();
  while (true) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if ((int)(v - value) >= 0) break;
    if (clock64() - t0 > kSpinBudgetCycles) {
      report(status, kTimeoutPeerFlag, site);
      break;
    }
    __nanosleep(200);
  }
}

// out[i] (=|+=) scale * sum over src = 0 .. world-1 (in that order) of stage[src * stride + i].
template <bool OUT_F32>
__global__ void __launch_bounds__(256)
rs_reduce_kernel(const __nv_bfloat16* __restrict__ stage, int world, long long stride, long long n,
                 void* __restrict__ out_, int accumulate, float scale) {
  const long long nvec = n / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < world; ++s) {
      const uint4 v = *reinterpret_cast<const uint4*>(stage + s * stride + i * 8);
      const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] *= scale;
    if (OUT_F32) {
      float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out_) + i * 8);
      float4 lo = make_float4(acc[0], acc[1], acc[2], acc[3]), hi = make_float4(acc[4], acc[5], acc[6], acc[7]);
      if (accumulate) {
        const float4 a = o[0], b = o[1];
        lo.x += a.x; lo.y += a.y; lo.z += a.z; lo.w += a.w;
        hi.x += b.x; hi.y += b.y; hi.z += b.z; hi.w += b.w;
      }
      o[0] = lo;
      o[1] = hi;
    } else {
      uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out_) + i * 8);
      if (accumulate) {
        const uint4 v = *o;
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
        acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
      *o = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                      pack_bf16(acc[6], acc[7]));
    }
  }
}

struct PeerShards {
  const uint4* shard[kMaxPeers];
};

// out[t, :] = row ids[t] of a [vocab, dim] table that lives, flattened, `base_vec` 16-byte vectors into
// a buffer sharded `shard_vec` vectors per rank: every vector is loaded from the shard of the rank
// that owns it (plain peer loads over NVLink; a row may straddle two owners).  Only the rows that are
// looked up cross the link, instead of the whole table.
__global__ void embedding_fwd_peer_kernel(PeerShards ps, const long long* __restrict__ ids, uint4* __restrict__ out,
                                          long long tokens, int nvec, long long vocab, long long shard_vec,
                                          long long base_vec) {
  const long long total = tokens * nvec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / nvec;
    const int c = (int)(idx % nvec);
    const long long id = ids[t];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < vocab) {
      const long long flat = base_vec + id * nvec + c;
      const long long owner = flat / shard_vec;
      v = ps.shard[owner][flat - owner * shard_vec];
    }
    out[idx] = v;
  }
}

int sm_count();  // runtime.cu

}  // namespace tpb

using namespace tpb;

static inline int launch_rc() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

// *flag = value, ordered after everything enqueued on `stream` before it (device scope).
extern "C" int tpb_flag_set(unsigned* flag, unsigned value, void* stream) {
  if (!flag) return -2;
  flag_set_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flag, value);
  return launch_rc();
}

// flag_tables[t][index] = value for every rank t of the group (this rank's own table included).
extern "C" int tpb_peer_signal(void* const* flag_tables, int world, long long index, unsigned value, void* stream) {
  if (!flag_tables || world < 1 || world > kMaxPeers || index < 0) return -2;
  PeerFlagTable peers;
  for (int i = 0; i < world; ++i) peers.flags[i] = reinterpret_cast<unsigned*>(flag_tables[i]);
  peer_signal_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(peers, world, index, value);
  return launch_rc();
}

// Returns (on the stream) when flags[0], flags[stride], ... flags[(n-1) * stride] have all reached
// `value`, or when the wait budget ran out (status code 5, site `site`).
extern "C" int tpb_flag_wait(const unsigned* flags, int n, long long stride, unsigned value, int site, void* stream) {
  if (!flags || n < 1 || n > kMaxPeers) return -2;
  flag_wait_kernel<<<1, 64, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flags, n, stride, value, status_block(),
                                                                         site);
  return launch_rc();
}

// Fixed-order reduction of `world` bf16 staging slots (`stride` elements apart) of `n` elements each
// into out (bf16 or fp32; overwritten, or added to when `accumulate`).  n % 8 == 0, 16-byte aligned.
extern "C" int tpb_rs_reduce_bf16(const void* stage, int world, long long stride, long long n, void* out,
                                  int out_is_f32, int accumulate, float scale, void* stream) {
  if (!stage || !out || world < 1 || n < 0 || (n % 8) || (stride % 8)) return -2;
  if ((reinterpret_cast<uintptr_t>(stage) % 16) || (reinterpret_cast<uintptr_t>(out) % 16)) return -2;
  if (n == 0) return 0;
  const long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (out_is_f32)
    rs_reduce_kernel<true><<<(int)blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(stage), world, stride, n,
                                                        out, accumulate, scale);
  else
    rs_reduce_kernel<false><<<(int)blocks, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(stage), world, stride, n,
                                                         out, accumulate, scale);
  return launch_rc();
}

// Embedding lookup straight out of the owners' parameter shards (see embedding_fwd_peer_kernel).
// shards[r]: rank r's shard of the flat buffer that holds the table (peer-mapped), `shard_elems`
// elements each; the table starts `table_offset` elements into the flat buffer.
extern "C" int tpb_embedding_fwd_peer(void* const* shards, int world, long long shard_elems, long long table_offset,
                                      const long long* ids, void* out, int tokens, int dim, long long vocab,
                                      void* stream) {
  if (!shards || world < 1 || world > kMaxPeers || (dim % 8) || (shard_elems % 8) || (table_offset % 8)) return -2;
  if (tokens <= 0) return 0;
  PeerShards ps;
  for (int i = 0; i < world; ++i) ps.shard[i] = reinterpret_cast<const uint4*>(shards[i]);
  const long long total = (long long)tokens * (dim / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  embedding_fwd_peer_kernel<<<(int)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      ps, ids, reinterpret_cast<uint4*>(out), tokens, dim / 8, vocab, shard_elems / 8, table_offset / 8);
  return launch_rc();
}
