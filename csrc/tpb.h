// C ABI of libtpb200.so: hand-written sm_100a kernels for the training hot path.
// All pointers are device pointers unless stated otherwise; `stream` is a
// cudaStream_t passed as void*.  Functions return 0 on success, a negative value
// for rejected arguments and 1000 + cudaError_t for launch failures.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// GEMM epilogues (tpb_gemm_bf16 `epi`).
enum {
  TPB_EPI_BF16 = 0,      // C(bf16) = alpha * acc
  TPB_EPI_F32 = 1,       // C(f32)  = alpha * acc
  TPB_EPI_F32_ACC = 2,   // C(f32) += alpha * acc
  TPB_EPI_BF16_ACC = 3,  // C(bf16) = C + alpha * acc
  TPB_EPI_BF16_RES = 4,  // C(bf16) = aux + alpha * acc   (residual add)
  TPB_EPI_SWIGLU = 5,    // B = [gate; up] rows, C[M, N/2] = silu(g) * u, optional c2[M, N] = [g | u]
  TPB_EPI_RS_BF16 = 6,   // reduce-scatter: red.add alpha * acc into the owner's bf16 shard over P2P
  TPB_EPI_AR_BF16 = 7,   // all-reduce: C is the NVSwitch multicast address of a zeroed symmetric buffer;
                         // multimem.red adds alpha * acc (+ aux, if given) into every rank's copy
};

// Status block: {code, site, block, thread}; code 0 = no kernel ever timed out.
int tpb_status(int* out4);
void tpb_status_clear(void);
int tpb_sm_count(void);
// Bounded device-side wait on a flag (failure-detection building block): *result = 1 when the flag
// reached `expected`, -1 (and status code 5) when `budget_cycles` ran out first.
int tpb_bounded_wait(const unsigned* flag, unsigned expected, long long budget_cycles, int* result, void* stream);

// C[M,N] = alpha * A[M,K] * B[N,K]^T.  a_mn / b_mn = 1 when that operand is stored
// with its M/N index contiguous ([K][M] resp. [K][N]) instead of K contiguous.
int tpb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, int a_mn, int b_mn, int epi, float alpha,
                  const void* aux, long long ldaux, void* c2, long long ldc2, int max_ctas,
                  void* stream);

// y = rmsnorm(x [+ res]) * w.  h_out (optional) receives x + res.  rstd: [rows] fp32.
int tpb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                    int rows, int dim, float eps, void* stream);
// dx = d/dx of the above (+ dres if given).  dw_f32 [dim] is accumulated with atomics.
int tpb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dres,
                    void* dx, float* dw_f32, int rows, int dim, void* stream);

// In-place rotate-half RoPE on `heads` heads of width `dim` starting at column
// `col0` of a [tokens, ld] bf16 matrix.  cos/sin: fp32 [max_pos, dim/2].
// pos: optional int32 [tokens] positions (else token % seq_len).  inverse=1 applies R^T.
int tpb_rope(void* x, long long ld, int col0, int heads, int dim, const float* cos, const float* sin,
             const int* pos, int tokens, int seq_len, int inverse, int interleaved, void* stream);

// Same with heads `head_stride` elements apart (rotating a `dim`-wide slice of wider heads).
int tpb_rope_strided(void* x, long long ld, int col0, int heads, int dim, int head_stride, const float* cos,
                     const float* sin, const int* pos, int tokens, int seq_len, int inverse, int interleaved,
                     void* stream);

// act[T,F] = silu(gu[:, :F]) * gu[:, F:]
int tpb_swiglu_fwd(const void* gu, void* act, int rows, int f, void* stream);
// dgu[T,2F] from dact[T,F] and gu
int tpb_swiglu_bwd(const void* dact, const void* gu, void* dgu, int rows, int f, void* stream);

// Row-wise softmax cross entropy on bf16 logits [rows, vocab] (row pitch ld).
// loss_sum += sum_i loss_i (fp32 atomics), logits are overwritten with
// (softmax - onehot) * *grad_scale; rows with target < 0 produce zeros.
int tpb_ce_fwd_bwd(void* logits, long long ld, const long long* targets, float* loss_sum,
                   const float* grad_scale, int rows, int vocab, void* stream);

// Fused AdamW over flat fp32 state; grads bf16 (grad_is_bf16=1) or fp32.
// clip_coef: optional device scalar multiplied into the gradient.
int tpb_adamw(float* p32, float* m, float* v, const void* grad, void* p16, long long n, float lr,
              float beta1, float beta2, float eps, float wd, float bc1, float bc2, const float* clip_coef,
              int grad_is_bf16, void* stream);
// *out += sum(g^2)   (out: fp32 device scalar)
int tpb_sumsq(const void* g, long long n, int is_bf16, float* out, void* stream);
// coef = min(1, max_norm / (sqrt(*sumsq) + 1e-6)); norm_out = sqrt(*sumsq)
int tpb_clip_coef(const float* sumsq, float max_norm, float* coef, float* norm_out, void* stream);

// out[t,:] = table[ids[t],:]
int tpb_embedding_fwd(const void* table, const long long* ids, void* out, int tokens, int dim,
                      long long vocab, long long row0, void* stream);
// dtable[ids[t]-row0,:] += dout[t,:] for rows owned by this shard
int tpb_embedding_bwd(const void* dout, const long long* ids, void* dtable, int tokens, int dim,
                      long long rows_local, long long row0, int dtable_is_f32, void* stream);

// bf16 <- fp32 with scale, and fp32 accumulate into bf16 destinations
int tpb_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, int accumulate, void* stream);

// Grouped (mixture-of-experts) GEMM, see GemmParams::mode in gemm_sm100.cu.
//  mode 1: C[rows of expert e] = A[rows of e] * B[e]^T; rows are grouped in 128-row aligned
//          segments, tile_expert[m_tile] names the expert of each 128-row tile (-1: unused).
//          B (and B2 for the "up" half of a SwiGLU epilogue) hold E matrices b_expert_stride apart.
//  mode 2: per-expert wgrad C[e] = A[:, rows of e] * B[:, rows of e]^T with both operands stored
//          row-major over the grouped rows (a_mn = b_mn = 1); k_offsets[E+1] are 64-aligned.
// row_align: rows to which expert segments are padded in mode 1 (128, or 256: CTA-pair tiles may be used).
int tpb_grouped_gemm_bf16(const void* A, const void* B, const void* B2, void* C, int M, int N, int K, int E,
                          long long lda, long long ldb, long long b_expert_stride, long long ldc, int a_mn, int b_mn,
                          int epi, float alpha, void* c2, long long ldc2, int mode, const int* tile_expert,
                          const int* k_offsets, long long c_stride, int row_align, void* stream);

// GEMM fused with the all-gather of the (flat, sharded) buffer that holds B, and GEMM fused with the
// reduce-scatter of C into the owners' shards; see the comments at the definitions in gemm_sm100.cu.
int tpb_ag_gemm_bf16(const void* A, void* C, int M, int N, int K, long long lda, long long ldc, int epi,
                     const void* aux, long long ldaux, void* c2, long long ldc2, const void* const* shard_ptrs,
                     int world, long long shard_elems, void* gathered, long long b_offset, unsigned* flags,
                     unsigned epoch, int copiers, int local_rank, void* const* push_gathered,
                     unsigned* const* push_flags, void* push_multicast, void* stream);
int tpb_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb, long long ldc,
                     int a_mn, int b_mn, float alpha, void* const* shard_ptrs, int world, long long shard_elems,
                     long long c_offset, int rank, void* stream);

// GEMM whose B operand sits in a gathered buffer that is still being filled by somebody else (copy
// engines); the TMA producer waits on per-chunk flags.  GEMM whose epilogue stores every tile into this
// rank's staging slot at the owner of that part of the flat gradient buffer.  See gemm_sm100.cu.
int tpb_gemm_ag_wait_bf16(const void* A, void* C, int M, int N, int K, long long lda, long long ldc, int epi,
                          const void* aux, long long ldaux, void* c2, long long ldc2, const void* gathered,
                          long long b_offset, int world, long long shard_elems, long long chunk_elems,
                          unsigned* flags, unsigned epoch, void* stream);
int tpb_gemm_rs_store_bf16(const void* A, const void* B, int M, int N, int K, long long lda, long long ldb,
                           long long ldc, int a_mn, int b_mn, float alpha, void* const* slot_ptrs, int world,
                           long long shard_elems, long long c_offset, int rank, void* stream);

// Flags and the fixed-order reduction of the peer-memory FSDP collectives (fsdp_comm.cu).
int tpb_flag_set(unsigned* flag, unsigned value, void* stream);
int tpb_peer_signal(void* const* flag_tables, int world, long long index, unsigned value, void* stream);
int tpb_flag_wait(const unsigned* flags, int n, long long stride, unsigned value, int site, void* stream);
int tpb_rs_reduce_bf16(const void* stage, int world, long long stride, long long n, void* out, int out_is_f32,
                       int accumulate, float scale, void* stream);

// Embedding rows read straight from the owners' (peer-mapped) shards of the flat buffer that holds the table.
int tpb_embedding_fwd_peer(void* const* shards, int world, long long shard_elems, long long table_offset,
                           const long long* ids, void* out, int tokens, int dim, long long vocab, void* stream);

// Router: one warp per token.  mode 0 softmax-top-k(-renormalise); mode 1 sigmoid + bias with
// group-limited selection.  w_out [T,K] fp32, idx_out [T,K] int32, scores_out [T,E] fp32 (optional).
int tpb_router_topk(const void* logits, int logits_is_bf16, const float* bias, float* w_out, int* idx_out,
                    float* scores_out, int tokens, int E, int K, int mode, int n_group, int topk_group, int norm_topk,
                    float scale, void* stream);
// out[r,:] = src_row[r] >= 0 ? row_scale[r] * x[src_row[r],:] : 0
int tpb_moe_gather(const void* x, const int* src_row, const float* row_scale, void* out, long long rows, int dim,
                   void* stream);
// out[t,:] = sum_k w[t,k] * rows[dest[t,k],:]
int tpb_moe_combine(const void* rows, const int* dest, const float* w, void* out, long long tokens, int K, int dim,
                    void* stream);
// dw[t,k] = <rows[dest[t,k],:], dout[t,:]>
int tpb_moe_combine_dw(const void* rows, const int* dest, const void* dout, float* dw, long long tokens, int K,
                       int dim, void* stream);

// Variable-size all-to-all of rows by plain stores into the peers' receive buffers (moe.cu).
// Stable counting sort of (token, slot) pairs by expert into 128-row padded segments (see moe.cu).
int tpb_moe_plan(const int* idx, int tokens, int K, int E, int rows, int align, int* counts, int* k_offsets,
                 int* dest, int* src_row, long long* src_pair, int* tile_expert, void* stream);
int tpb_a2a_push_rows(const void* src, int n_rows, int dim, int world, int me, const int* src_start,
                      const long long* dst_row0, void* const* dst, unsigned* const* flags, unsigned epoch,
                      unsigned* done_counter, void* stream);
int tpb_a2a_push_blocks(const void* src, int n_rows, int dim, int n_blocks, int world, int me,
                        const long long* desc_dev, void* const* dst, unsigned* const* flags, unsigned epoch,
                        unsigned* done_counter, void* stream);
int tpb_a2a_wait(const unsigned* flags, int world, unsigned epoch, void* stream);

// Flash attention (attention_fwd_sm100.cu / attention_bwd_sm100.cu); token-major [B*S, heads*dim] views.
int tpb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk, int Hq,
                 int Hkv, int dqk, int dv, long long ldq, long long ldk, long long ldv, long long ldo, float scale,
                 int causal, int window, const int* q_pos, const int* q_seg, const int* kv_seg, void* stream);
// The same with a logit soft cap: scores become softcap * tanh(q.k * scale / softcap) (softcap <= 0: none).
int tpb_attn_fwd_softcap(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Sq, int Sk,
                         int Hq, int Hkv, int dqk, int dv, long long ldq, long long ldk, long long ldv, long long ldo,
                         float scale, int causal, int window, const int* q_pos, const int* q_seg, const int* kv_seg,
                         float softcap, void* stream);
// Causal forward with the context-parallel K/V exchange fused in (see attention_fwd_sm100.cu).
int tpb_attn_fwd_cp(const void* q, const void* k_local, const void* v_local, void* const* k_all, void* const* v_all,
                    unsigned* const* flags, void* o, float* lse, int B, int Sq, int s_local, int Hq, int Hkv,
                    long long ldq, long long ld_k_local, long long ld_v_local, long long ldo, float scale,
                    const int* q_pos, int world, int rank, int zigzag, int copiers, unsigned epoch, void* k_multicast,
                    void* v_multicast, void* stream);
// `scratch` holds tpb_attn_bwd_scratch_floats(B, Sq, Hq) floats; dq/dk/dv are fully overwritten.
long long tpb_attn_bwd_scratch_floats(int B, int Sq, int Hq);
int tpb_attn_bwd(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                 float* scratch, void* dq, void* dk, void* dv, int B, int Sq, int Sk, int Hq, int Hkv,
                 int dqk, int dvd, long long ldq, long long ldk, long long ldv, long long lddo, long long lddq,
                 long long lddk, long long lddv, float scale, int causal, int window, const int* q_pos,
                 const int* q_seg, const int* kv_seg, void* stream);
int tpb_attn_bwd_softcap(const void* dO, const void* q, const void* k, const void* v, const void* o, const float* lse,
                 float* scratch, void* dq, void* dk, void* dv, int B, int Sq, int Sk, int Hq, int Hkv,
                 int dqk, int dvd, long long ldq, long long ldk, long long ldv, long long lddo, long long lddq,
                 long long lddk, long long lddv, float scale, int causal, int window, const int* q_pos,
                 const int* q_seg, const int* kv_seg, float softcap, void* stream);

// ---- symmetric-memory runtime (symm_runtime.cu): segments that every rank maps, and a bounded
// device-side barrier on their signal pads.
int tpb_symm_alloc(long long bytes, void** payload, unsigned char* handle64);
int tpb_symm_open(const unsigned char* handle64, void** payload);
int tpb_symm_release(void* payload);
int tpb_symm_copy(void* dst, const void* src, long long bytes, void* stream);
int tpb_symm_live_segments(void);
int tpb_symm_barrier(void* const* payloads, int rank, int world, unsigned epoch, void* stream);

#ifdef __cplusplus
}
#endif
