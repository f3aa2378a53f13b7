/* nxd_b200 -- C ABI of the sm_100a kernel library (libnxd_b200.so).
 *
 * Conventions: every function returns 0 on success, a cudaError_t value or -1 otherwise
 * (nxd_last_error() gives the message of the last failure on the calling thread).  Pointers
 * are device pointers unless stated otherwise; `stream` is a cudaStream_t; bf16 tensors are
 * row-major with the stated shape.  No entry point allocates device memory: scratch buffers
 * are passed by the caller (their sizes come from the *_num_* helpers).
 * The "reference" citations name the file:line of the upstream NeuronxDistributed code whose
 * behaviour the kernel provides on B200.
 */
#ifndef NXD_B200_H
#define NXD_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- runtime ---------------------------------------------------------------------------- */
const char* nxd_last_error(void);
int nxd_version(void);
int nxd_device_sm_count(void);
/* Kernel launches made by this library in the calling process so far (bench.py's "gpu_launches"). */
unsigned long long nxd_kernel_launches(void);
/* Overwrite `bytes` of `buf` (> L2 size) so the next timed iteration starts with a cold L2. */
int nxd_l2_flush(void* buf, size_t bytes, void* stream);

/* ---- GEMM: D[M,N] (+)= A_op[M,K] * B_op[N,K]^T on tcgen05/TMEM/TMA -------------------------
 * reference: parallel_layers/layers.py:325 (fwd), :348 (dgrad), :409 (wgrad) -- torch.matmul.
 * layout 0 "nt": a = [M,K], b = [N,K];  1 "nn": a = [M,K], b = [K,N];  2 "tn": a = [K,M], b = [K,N].
 * lda/ldb/ldd: row pitch in elements of the tensors as stored.  out_mode 0 bf16, 1 fp32,
 * 2 fp32 accumulate (d += result).  block_n 0 = auto, else 128 or 256. */
int nxd_gemm_bf16(int layout, const void* a, const void* b, void* d, int M, int N, int K, long long lda,
                  long long ldb, long long ldd, int out_mode, int block_n, void* stream);

/* ---- RMSNorm (reference: examples/training/llama/modeling_llama_nxd.py:142-149;
 *      examples/inference/modules/custom_calls.py:5-16) ---------------------------------------- */
int nxd_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* residual_out,
                    float* rstd, int rows, int H, float eps, void* stream);
int nxd_rmsnorm_bwd_num_partials(int rows);
/* scratch: nxd_rmsnorm_bwd_num_partials(rows) * H floats */
int nxd_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, const void* dresidual,
                    void* dx, void* dw_bf16, float* dw_f32, int accumulate, float* scratch, int rows, int H,
                    void* stream);

/* No counterpart in the reference.  Same computation as nxd_rmsnorm_bwd for callers that cannot supply (or allocate)
 * a scratch buffer: the dW partial sums go to a 4 MiB __device__ array inside the library.  H <= 8192 (see
 * nxd_rmsnorm_bwd_static_max_h), larger H returns an error.  No allocation happens in the call; the first call on a
 * device looks up the array's address, so issue it before any stream capture.  Calls share the array: do not let two
 * of them overlap on the GPU. */
int nxd_rmsnorm_bwd_static_max_h(void);
int nxd_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, const float* rstd, const void* dresidual,
                           void* dx, void* dw_bf16, float* dw_f32, int accumulate, int rows, int H, void* stream);

/* ---- SwiGLU / RoPE (reference: modeling_llama_nxd.py:197-208, :398-399;
 *      examples/inference/modules/attention/utils.py:27-41) ------------------------------------- */
int nxd_swiglu_fwd(const void* gate_up, void* out, long long rows, int I, void* stream);
int nxd_swiglu_bwd(const void* gate_up, const void* dy, void* dgate_up, long long rows, int I, void* stream);
int nxd_rope_inplace(void* x, const float* cos_t, const float* sin_t, const int* positions, long long T,
                     int heads_total, int n_rot_heads, int D, int pos_div, int pos_mod, int inverse,
                     void* stream);

/* ---- vocab-parallel cross entropy (reference: parallel_layers/loss_functions.py:11-130) ------- */
int nxd_ce_stats(const void* logits, const long long* target, float* stats, long long T, int V, int vocab_start,
                 void* stream);
int nxd_ce_bwd(const void* logits, const long long* target, const float* lse, const float* grad_out,
               void* grad_logits, long long T, int V, int vocab_start, float smoothing, int vocab_global,
               void* stream);

/* ---- optimizer / grad-norm (reference: optimizer/zero_redundancy_optimizer.py:29-156,
 *      utils/adamw_fp32_optim_params.py:88-153, parallel_layers/grads.py:33-240) ----------------- */
int nxd_sumsq_num_partials(void);
int nxd_sumsq(const void* x, long long n, int dtype, float* scratch, float* out, int accumulate, void* stream);
int nxd_clip_coef(const float* total_sumsq, float max_norm, float* coef, float* norm_out, void* stream);
int nxd_adamw_step(float* master, float* exp_avg, float* exp_avg_sq, const void* grad, int grad_dtype,
                   void* param_out, long long n, float lr, float beta1, float beta2, float eps,
                   float weight_decay, int step, float grad_scale, const float* clip_coef, void* stream);
int nxd_scale_inplace(void* x, long long n, int dtype, float scale, const float* dev_scale, void* stream);

/* ---- sampling (reference: utils/sampling.py:27-77) -------------------------------------------- */
int nxd_argmax(const void* logits, int dtype, int B, int V, long long row_stride, long long* out, void* stream);
int nxd_topk_sample(const void* logits, int dtype, int B, int V, long long row_stride, int top_k, float top_p,
                    float temperature, const float* uniform, long long* out, void* stream);

/* ---- decode attention + KV cache (reference: examples/inference/modules/attention/
 *      attention_base.py:141-170; modules/model_base.py:388-422) -------------------------------- */
int nxd_decode_attn_num_splits(int B, int n_kv, int max_len);
/* scratch: B * n_q * n_splits * (D + 2) floats */
int nxd_decode_attn(const void* q, const void* cache_k, const void* cache_v, const int* lengths,
                    const int* block_table, long long stride_b, long long stride_h, int page_size,
                    int max_pages, void* out, float* scratch, int B, int n_q, int n_kv, int D, int n_splits,
                    float scale, void* stream);
/* Same with a cache-line table: seq_ids[b] = cache line (contiguous cache) or block-table row (paged cache) of batch
 * row b (continuous batching reads the lines in place instead of gathering them first). */
int nxd_decode_attn_lines(const void* q, const void* cache_k, const void* cache_v, const int* lengths,
                          const int* block_table, const int* seq_ids, long long stride_b, long long stride_h,
                          int page_size, int max_pages, void* out, float* scratch, int B, int n_q, int n_kv, int D,
                          int n_splits, float scale, void* stream);
int nxd_kv_cache_update(const void* new_k, const void* new_v, void* cache_k, void* cache_v, const int* positions,
                        const int* seq_ids, const int* block_table, long long stride_b, long long stride_h,
                        int page_size, int max_pages, int B, int n_kv, int T_new, int D, void* stream);

/* ---- embedding (reference: parallel_layers/layers.py:215-238) ---------------------------------- */
int nxd_embedding_fwd(const long long* ids, const void* weight, void* out, long long T, int H, int vocab_start,
                      int vocab_local, int B, int S, int seq_first_out, void* stream);
int nxd_embedding_bwd(const long long* ids, const void* dy, float* dw, long long T, int H, int vocab_start,
                      int vocab_local, int B, int S, int seq_first_in, void* stream);

/* ---- flash attention (reference: kernels/flash_attn.py nki_flash_attn_func; attention_base.py prefill) ----------
 * bf16 tensors addressed as (batch, head, row) element strides with unit stride on the head dimension:
 * strides = {q_b,q_h,q_s, k_b,k_h,k_s, v_b,v_h,v_s, o_b,o_h,o_s} (forward, 12 entries) followed in the backward
 * by the same triple for dout, dq, dk, dv (24 entries).  lse: [B, Hq, Sq] floats (natural log).  GQA: Hq % Hkv == 0.
 * *_tc = tcgen05 / TMEM / TMA kernels (forward D = 64 or 128; backward D = 128), the others are the portable
 * mma.sync kernels (D = 64 or 128). */
int nxd_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const long long* strides,
                       int B, int Hq, int Hkv, int Sq, int Sk, int D, float scale, int causal, void* stream);
/* delta: [B, Hq, Sq] floats of scratch */
int nxd_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                       const float* lse, float* delta, void* dq, void* dk, void* dv, const long long* strides, int B,
                       int Hq, int Hkv, int Sq, int Sk, int D, float scale, int causal, void* stream);
int nxd_flash_attn_fwd_tc(const void* q, const void* k, const void* v, void* o, float* lse,
                          const long long* strides, int B, int Hq, int Hkv, int Sq, int Sk, int D, float scale,
                          int causal, void* stream);
/* scratch: lse_pad, delta_pad = B * Hq * roundup(Sq, 64) floats each; dq_accum = B * Hq * D * roundup(Sq, 64) floats (d-major), ZEROED
 * by the caller before the call (dQ is accumulated with TMA reduce-add).  dkv_accum: NULL, or 2 * B * Hkv * Sk * D
 * ZEROED floats: then nxd_flash_attn_bwd_tc_num_splits() CTAs share each K/V block and reduce-add their partial
 * dK / dV (few heads per GPU under tensor parallelism would otherwise leave most SMs idle). */
int nxd_flash_attn_bwd_tc_num_splits(int B, int Hq, int Hkv, int Sq, int Sk);
int nxd_flash_attn_bwd_tc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                          const float* lse, float* lse_pad, float* delta_pad, float* dq_accum, float* dkv_accum,
                          void* dq, void* dk, void* dv, const long long* strides, int B, int Hq, int Hkv, int Sq,
                          int Sk, int D, float scale, int causal, void* stream);

/* ---- symmetric (peer-mapped) memory over CUDA IPC + fused compute/collective kernels ---------------------------
 * No counterpart in the reference (its collectives are XLA ops).  One process per GPU: every rank allocates a
 * region, exchanges the 64-byte handles out of band (torch.distributed), opens the peers' handles and passes the
 * resulting pointer tables to the kernels.  A signal pad (uint32 flags, zero-initialised) is one more such region. */
int nxd_symm_handle_bytes(void);
int nxd_symm_alloc(size_t bytes, void** ptr, unsigned char* handle_out);   /* cudaMalloc + memset 0 + export */
int nxd_symm_open(const unsigned char* handle, void** ptr);                /* map a peer's region */
int nxd_symm_close(void* ptr);
int nxd_symm_free(void* ptr);
/* all ranks rendezvous on the device: flag `slot` of every pad, `epoch` strictly increasing per slot */
int nxd_symm_barrier(void* const* sig_peers, void* sig_local, int world, int rank, int slot, unsigned epoch,
                     void* stream);
/* Y[tp*R, N] = all_gather_r(X_r[R, K]) * op(W)  (reference: layers.py:312-325 all_gather then matmul).
 * layout 0: W is [N, K] (nt); 1: W is [K, N] (nn).  xt_ptrs: tp pointers to every rank's gathered buffer
 * [tp*R, K] (symmetric memory; on return the local one holds the gathered input), sig_ptrs: tp signal pads,
 * slot_chunks: first of tp * R/256 flags, epoch: call counter of this (buffer, flags) pair starting at 1,
 * comm_ctas: even number of CTAs that drive the copy engine, block_n: 0 = auto, trace: NULL or 16 x u64. */
int nxd_ag_gemm_bf16(int layout, const void* x_local, const void* w, void* y, int R, int N, int K, long long ldw,
                     long long ldy, void* const* xt_ptrs, void* const* sig_ptrs, int tp, int rank, int slot_chunks,
                     unsigned epoch, int comm_ctas, int block_n, void* trace, void* stream);
/* EXPERIMENTAL (compiled, not yet run on hardware): same, but the copy CTAs store the local shard ONCE to the NVLS
 * multicast address of the gathered buffer (multimem.st) instead of once per peer. */
int nxd_ag_gemm_bf16_nvls(int layout, const void* x_local, const void* w, void* y, int R, int N, int K, long long ldw,
                          long long ldy, void* const* xt_ptrs, void* const* sig_ptrs, int tp, int rank, int slot_chunks,
                          unsigned epoch, int comm_ctas, int block_n, void* mc_total, void* stream);
/* out[R, N] = reduce_scatter_r(X[tp*R, K] * op(W))  (reference: layers.py:452-461 matmul then reduce_scatter).
 * stage_ptrs: tp pointers to every rank's staging region [tp][R][N] bf16 (double-buffered by the caller through
 * epoch parity), slot_cnt: first of tp * R/256 flags. */
int nxd_gemm_rs_bf16(int layout, const void* x, const void* w, void* out, int R, int N, int K, long long ldx,
                     long long ldw, long long ldo, void* const* stage_ptrs, void* const* sig_ptrs, int tp, int rank,
                     int slot_cnt, unsigned epoch, int block_n, void* trace, void* stream);
/* Expert parallelism (reference: modules/moe/experts.py:121-152, enter / exit_expert_parallel_region all-to-all around
 * the expert matmuls).  Dispatch: x_local is [ep][E_loc, C, K] (slab d = tokens routed to the experts of rank d); every
 * rank receives X_total = [ep(source)][E_loc, C, K] in its symmetric buffer and y[(s, e, c), :] = X_total[s, e, c, :] * W_e.
 * Combine: x is [ep(source)][E_loc, C, K]; result tiles are stored straight into the token owner's output
 * [E, C, N] (out_ptrs: every rank's symmetric output buffer of this call), nothing is reduced.
 * W: stacked expert weights, layout 0 = [E_loc * N, K], 1 = [E_loc * K, N].  R = E_loc * C, C % 256 == 0. */
int nxd_a2a_gemm_bf16(int layout, const void* x_local, const void* w, void* y, int R, int C, int N, int K,
                      long long ldw, long long ldy, void* const* xt_ptrs, void* const* sig_ptrs, int ep, int rank,
                      int slot_chunks, unsigned epoch, int comm_ctas, int block_n, void* trace, void* stream);
int nxd_gemm_a2a_bf16(int layout, const void* x, const void* w, int R, int C, int N, int K, long long ldx,
                      long long ldw, void* const* out_ptrs, void* const* sig_ptrs, int ep, int rank, int slot_cnt,
                      unsigned epoch, int block_n, void* trace, void* stream);
/* ZeRO-1 step over peer memory (reference: the ZeRO-1 optimizer configured in trainer/trainer.py:244-269: reduce-scatter
 * of the gradient bucket, inner optimizer on the shard, all-gather of the parameters).  grad_ptrs / param_ptrs: dp
 * pointers to every rank's flat gradient / parameter buffer (symmetric memory).  reduce_shard: out[0..n) (fp32) = sum
 * over ranks of grad_r[lo..lo+n) in rank order (grad_dtype 0 = fp32, 1 = bf16).  adamw_allgather: AdamW on the shard,
 * the bf16 result is stored into param_r[lo..lo+n) of EVERY rank.  lo, n in elements, multiples of 8.  The caller
 * brackets the pair with nxd_symm_barrier. */
int nxd_zero1_reduce_shard(void* const* grad_ptrs, int grad_dtype, long long lo, long long n, float* out, int dp, int rank,
                           void* stream);
/* The same reduction with the local part of the gradient norm folded in: sum_sharded[0] += sum of out[i]^2
 * for i < split_at, sum_replicated[0] += the rest; partials = 2 * nxd_zero1_reduce_blocks(n, dtype) floats of scratch. */
int nxd_zero1_reduce_blocks(long long n, int grad_dtype);
int nxd_zero1_reduce_shard_sumsq(void* const* grad_ptrs, int grad_dtype, long long lo, long long n, float* out, int dp,
                                 int rank, long long split_at, float* partials, float* sum_sharded, float* sum_replicated,
                                 void* stream);
int nxd_zero1_adamw_allgather(float* master, float* exp_avg, float* exp_avg_sq, const float* grad,
                              void* const* param_ptrs, long long lo, long long n, float lr, float beta1, float beta2,
                              float eps, float weight_decay, int step, float grad_scale, const float* clip_coef, int dp,
                              int rank, void* stream);
/* Token-generation path (reference: RowParallelLinear matmul + all-reduce, layers.py:452-468 / mappings.py:176-190):
 * out[B, N] (+ residual) = sum over ranks of x[B, K] * w[N, K]^T in ONE launch, B <= 16; the fp32 partial blocks are
 * pushed into every peer's staging slot and added in rank order (bit-identical on all ranks).  stage_ptrs: tp regions
 * of 2 * tp * slot_elems floats; slot: first of nxd_oneshot_num_flags() flags; state: 2 zeroed uint32 of local device
 * memory per staging region (call counter, kept on the device so that CUDA-graph replays stay correct).
 * tp == 1 is a plain weight-streaming skinny GEMM (no symmetric memory needed). */
int nxd_oneshot_num_flags(void);
int nxd_skinny_gemm_ar_bf16(const void* x, const void* w, const void* residual, void* out, int B, int N, int K,
                            long long ldx, long long ldw, long long ldo, void* const* stage_ptrs,
                            void* const* sig_ptrs, size_t slot_elems, int tp, int rank, int slot, void* state,
                            void* stream);
/* Weight-streaming tcgen05 GEMM for 1..128 activation rows (batched token generation): out[B, N] = x[B, K] @ w[N, K]^T
 * (+ residual[B, N]); the weight rows are the UMMA M dimension, the padded row count (16/32/64/128) the UMMA N dimension;
 * split-K over a thread-block cluster with a distributed-shared-memory reduction.  K, ldx, ldw % 8 == 0;
 * splits: 0 = choose, else 1 / 2 / 4 / 8. */
int nxd_gemm_smallm_bf16(const void* x, const void* w, const void* residual, void* out, int B, int N, int K,
                         long long ldx, long long ldw, long long ldo, long long ldr, int splits, void* stream);
/* The same kernel with the decoder layer's element-wise neighbours in its epilogue (batched counterparts of
 * nxd_decode_qkv_rope_cache / nxd_decode_gate_up_swiglu, without the norm: x is the normalised activation).
 * qkv: B <= 128, D in {64, 128}; gate_up: B <= 64, I % 8 == 0 (a CTA streams gate slab t and up slab t). */
int nxd_smallm_qkv_rope_cache(const void* x, long long ldx, const void* w, long long ldw, const float* cos_t,
                              const float* sin_t, const int* positions, void* q_out, void* cache_k, void* cache_v,
                              const int* seq_ids, const int* block_table, long long stride_b, long long stride_h,
                              int page_size, int max_pages, int B, int K, int n_q, int n_kv, int D, int splits,
                              void* stream);
int nxd_smallm_gate_up_swiglu(const void* x, long long ldx, const void* w, long long ldw, void* out, long long ldo, int B,
                              int K, int I, int splits, void* stream);
/* Weight-only int8 skinny GEMM (reference: quantization_layers.py:444-478 dequantise + matmul): out[B, N] (+ residual) =
 * (x[B, K] bf16 * w[N, K]^T int8) * scale, fp32 accumulation; scale_n == 1 (per tensor) or N (per output channel).
 * B <= 8, K % 16 == 0, ldw (bytes) % 16 == 0.  Streams half the bytes of the bf16 skinny GEMM. */
int nxd_skinny_gemm_i8(const void* x, const void* w, const void* scale, int scale_n, const void* residual, void* out,
                       int B, int N, int K, long long ldx, long long ldw, long long ldo, void* stream);
/* out[n] = sum over ranks of in[n] (bf16, n % 8 == 0, n <= slot_elems): one-shot all-reduce for small messages */
int nxd_allreduce_oneshot(const void* in, void* out, long long n, void* const* stage_ptrs, void* const* sig_ptrs,
                          size_t slot_elems, int tp, int rank, int slot, void* state, void* stream);
/* Sequence-parallel embedding forward without the reduce-scatter of a mostly-zero tensor (reference: layers.py:215-238
 * + mappings.py reduce_scatter): the rank that owns a token's vocab row writes it into the output shard
 * [S/tp, B, H] of the rank that owns the sequence position (symmetric memory), then the ranks exchange flags.
 * ids: all B*S ids, identical on every rank; done: one zeroed uint32 of local device memory. */
int nxd_embedding_fwd_sp_push(const long long* ids, const void* weight, void* const* out_ptrs, void* const* sig_ptrs,
                              void* done, long long T, int H, int vocab_start, int vocab_local, int B, int S, int tp,
                              int rank, int slot, unsigned epoch, void* stream);
/* tooling: NVLink push-bandwidth probe (tools/bench_p2p.py) */
int nxd_p2p_push_probe(int mode, const void* src, const void* const* dst_ptrs, int n_dst, size_t bytes, int ctas,
                       int chunk, int bufs, int read_lag, int sig_mode, int sig_every, size_t flag_off, void* stream);

/* ---- MoE: grouped expert GEMM and token permutation (reference: modules/moe/moe_parallel_layers.py:78,94,108 einsum
 *      over e; modules/moe/expert_mlps.py:183-265 gather by token_assignments / weighted scatter-combine) -------------
 * E problems of one shape in one launch; stride_* = elements between consecutive problems; M needs no alignment. */
int nxd_gemm_grouped_bf16(int layout, const void* a, const void* b, void* d, int E, int M, int N, int K, long long lda,
                          long long ldb, long long ldd, long long stride_a, long long stride_b, long long stride_d,
                          int out_mode, void* stream);
/* out[r] = slot_token[r] >= 0 ? scale[r] * x[slot_token[r]] : 0   (scale NULL = 1) */
int nxd_moe_gather(const void* x, const int* slot_token, const float* scale, void* out, long long slots, int H,
                   void* stream);
/* out[t] = sum_j w[t, j] * y[slot_of[t, j]]   (pairs with w == 0 are skipped) */
int nxd_moe_combine(const void* y, const int* slot_of, const float* w, void* out, long long T, int k, int H, void* stream);
/* dw[t, j] = kept[t, j] ? <dout[t], y[slot_of[t, j]]> : 0 */
int nxd_moe_combine_dw(const void* y, const void* dout, const int* slot_of, const unsigned char* kept, float* dw,
                       long long T, int k, int H, void* stream);

/* Attention dropout (reference: nki_flash_attn_func(q, k, v, dropout_p, ..., seed), kernels/flash_attn.py:122-127,151-160).
 * Same arguments as the calls above plus dropout_p in [0, 1) and a seed; the keep mask is a hash of
 * (seed, batch, head, query, key), so the backward call regenerates it from the same two values. */
int nxd_flash_attn_fwd_tc_dropout(const void* q, const void* k, const void* v, void* o, float* lse,
                                  const long long* strides, int B, int Hq, int Hkv, int Sq, int Sk, int D, float scale,
                                  int causal, float dropout_p, unsigned long long seed, void* stream);
int nxd_flash_attn_bwd_tc_dropout(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                  const float* lse, float* lse_pad, float* delta_pad, float* dq_accum, float* dkv_accum,
                                  void* dq, void* dk, void* dv, const long long* strides, int B, int Hq, int Hkv, int Sq,
                                  int Sk, int D, float scale, int causal, float dropout_p, unsigned long long seed,
                                  void* stream);

/* ---- token-generation projections with fused neighbours (reference: the token-generation graph,
 *      examples/inference/modules/model_base.py:459-518, attention_base.py:172-200) ----------------------------------
 * q, k, v = W_qkv rmsnorm(x); RoPE(q, k) at positions[b]; q -> q_out [B, n_q, D]; k, v -> the KV cache row
 * (contiguous [lines, n_kv, S, D] with strides in elements, or paged with block_table [lines, max_pages]).
 * norm_w NULL = no norm.  B <= 8, D in {64, 128}. */
int nxd_decode_qkv_rope_cache(const void* x, long long ldx, const void* norm_w, float eps, const void* w, long long ldw,
                              const float* cos_t, const float* sin_t, const int* positions, void* q_out, void* cache_k,
                              void* cache_v, const int* seq_ids, const int* block_table, long long stride_b,
                              long long stride_h, int page_size, int max_pages, int B, int K, int n_q, int n_kv, int D,
                              void* stream);
/* out[B, I] = silu(W_gate rmsnorm(x)) * (W_up rmsnorm(x)); w = [2 I, K] with the gate rows first.  B <= 8. */
int nxd_decode_gate_up_swiglu(const void* x, long long ldx, const void* norm_w, float eps, const void* w, long long ldw,
                              void* out, long long ldo, int B, int K, int I, void* stream);

/* ---- windowed attention over the KV cache, post-norm residual, sparse MoE (no counterpart in the reference) -----------
 * dtype arguments: 0 = bf16, 1 = fp32.  Cache: contiguous [lines, G, S, D] (block_table NULL) or paged
 * [pages, G, page_size, D] with block_table [lines, table_cols]; strides in elements.
 * visible(i, j) = j <= i and (window <= 0 or i - j < window or j < keep_first);
 * score(i, j) = scale * <q_i, k_j> - slopes[h] * (i - j)  (slopes NULL: no bias). */
int nxd_qk_norm_cache_write(int dtype, const void* qkv, long long ld, void* q_out, void* cache_k, void* cache_v,
                            long long k_stride_line, long long k_stride_head, long long v_stride_line,
                            long long v_stride_head, const int* block_table, int page_size, int table_cols,
                            const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G, int D,
                            int Dv, int has_kv, int normalize, float eps, int max_pos, int writeback, void* stream);
/* impl: 0 = choose, 1 = generic kernel, 2 = mma.sync kernel (error when it does not apply) */
int nxd_window_attn_prefill(int dtype, const void* q, const void* cache_k, const void* cache_v, long long k_stride_line,
                            long long k_stride_head, long long v_stride_line, long long v_stride_head,
                            const int* block_table, int page_size, int table_cols, void* out, const int* q_start,
                            const int* n_new, const int* seq_ids, const float* slopes, int B, int Tn, int H, int G, int D,
                            int Dv, float scale, int window, int keep_first, int impl, void* stream);
int nxd_window_attn_decode(int dtype, const void* q, const void* cache_k, const void* cache_v, long long k_stride_line,
                           long long k_stride_head, long long v_stride_line, long long v_stride_head,
                           const int* block_table, int page_size, int table_cols, void* out, const int* positions,
                           const int* seq_ids, const float* slopes, int B, int H, int G, int D, int Dv, float scale,
                           int window, int keep_first, int impl, void* stream);
/* The same kernels with a chunk mask (chunk > 0: floor(i / chunk) == floor(j / chunk) as well), a per-head sink logit in
 * the softmax denominator (sinks [H] fp32 or NULL) and explicit cache-row pitches (k_row, v_row, in elements: v_row ==
 * k_row when the values are columns of the key rows).  nxd_qk_prep_cache_write adds norm weights (fp32 [D] or NULL),
 * pairwise rotation from cos / sin tables [positions, rope_dims / 2] (pairs (2i, 2i + 1), or with rope_halves
 * (i, i + rope_dims / 2)), value_from_key (cached value = raw key) and whole_norm (the norm's statistic over all query /
 * all key heads of a row at once, weights of H * D / G * D values; row_stat [B * Tn, 2] fp32 scratch for the statistics,
 * or NULL). */
int nxd_qk_prep_cache_write(int dtype, const void* qkv, long long ld, void* q_out, void* cache_k, void* cache_v,
                            long long k_stride_line, long long k_stride_head, long long v_stride_line,
                            long long v_stride_head, const int* block_table, int page_size, int table_cols,
                            const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G, int D,
                            int Dv, int has_kv, int normalize, float eps, int max_pos, int writeback,
                            const float* q_weight, const float* k_weight, const float* rope_cos, const float* rope_sin,
                            int rope_dims, int value_from_key, int value_heads, int rope_halves, int whole_norm,
                            float* row_stat, void* stream);
/* value_heads (0 = as many as key heads): head g of the value cache serves the key heads g, g + value_heads, ...
 * (several attention maps over the same values); the projection row then holds value_heads value heads. */
int nxd_masked_attn_prefill(int dtype, const void* q, const void* cache_k, const void* cache_v, long long k_stride_line,
                            long long k_stride_head, long long k_row, long long v_stride_line, long long v_stride_head,
                            long long v_row, const int* block_table, int page_size, int table_cols, void* out,
                            const int* q_start, const int* n_new, const int* seq_ids, const float* slopes,
                            const float* sinks, int B, int Tn, int H, int G, int D, int Dv, float scale, int window,
                            int keep_first, int chunk, int impl, int value_heads, void* stream);
int nxd_masked_attn_decode(int dtype, const void* q, const void* cache_k, const void* cache_v, long long k_stride_line,
                           long long k_stride_head, long long k_row, long long v_stride_line, long long v_stride_head,
                           long long v_row, const int* block_table, int page_size, int table_cols, void* out,
                           const int* positions, const int* seq_ids, const float* slopes, const float* sinks, int B, int H,
                           int G, int D, int Dv, float scale, int window, int keep_first, int chunk, int impl,
                           int value_heads, void* stream);
/* differential attention: maps [N, 2 * H, Dv] (first H heads = map 1, last H = map 2) -> out [N, H * Dv] =
 * rms_head(a1 - lambda * a2) * (1 - diff), lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff (vectors fp32 [D]) */
int nxd_diff_attn_combine(int dtype, const void* maps, void* out, const float* lq1, const float* lk1, const float* lq2,
                          const float* lk2, long long N, int H, int Dv, int D, float diff, float eps, void* stream);
/* latent attention: un-rotated query columns -> q_nope, rotated query columns -> q_rot, cache row [norm(c) * w | k_rot] */
int nxd_latent_prep(int dtype, const void* proj, long long ld, int q_off, int kv_off, void* q_nope, long long nope_head,
                    void* q_rot, long long rot_head, void* cache, long long stride_line, long long row_pitch,
                    const int* block_table, int page_size, int table_cols, const float* c_weight, const float* rope_cos,
                    const float* rope_sin, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H,
                    int dim, int rot, int rank, float eps, int max_pos, void* stream);
/* bf16 token generation over latent rows (values = the first Dv columns of the D-column rows); partial: fp32 scratch
 * [B, H, nsplit, Dv + 2]; returns 2 when no kernel is compiled for (D, Dv) */
int nxd_latent_decode(const void* q, const void* cache, long long stride_line, long long row_pitch, const int* block_table,
                      int page_size, int table_cols, void* out, float* partial, const int* positions, const int* seq_ids,
                      const float* sinks, int B, int H, int D, int Dv, float scale, int nsplit, void* stream);
int nxd_mlstm_chunk_states(float* u, const float* ftot, const float* mloc, const float* s0, const float* m0, float* s_out,
                           float* m_start, float* m_out, long long BH, int NC, long long E, void* stream);
/* recurrent matrix memory: fp32 gates (soft cap, log-sigmoid forget gate), scan over a step on the line's fp32 state,
 * gated / normalised head output, squared ReLU */
int nxd_mlstm_gates(int dtype, const void* h, const void* w, const float* bias, float* gi, float* gf, long long N, int W,
                    int H, float cap, void* stream);
int nxd_mlstm_scan(int dtype, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* gi,
                   const float* gf, float* state_s, float* state_n, float* state_m, float* next_n, float* next_m,
                   float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int D,
                   int Dv, float qscale, void* stream);
int nxd_head_norm_gate(int o_dtype, int dtype, const void* o, const void* gate, long long ld_g, int g_off,
                       const float* weight, void* out, long long N, int H, int Dv, int normalize, float eps,
                       int gate_act /* 0 sigmoid, 1 silu */, void* stream);
int nxd_relu_squared(int dtype, const void* x, void* y, long long n, void* stream);
/* x (fp32, in place) += norm(y) * w_post (y may be NULL); h (may be NULL) = cast(norm(x) * w_next); center: 1 = layer
 * norm without bias, 0 = RMS norm */
int nxd_norm_chain(int y_dtype, int h_dtype, const void* y, const float* w_post, float* x, const float* w_next, void* h,
                   long long rows, int W, float eps, int center, void* stream);
/* tcgen05 flash attention with window / kept first keys / distance bias; tensors and strides as nxd_flash_attn_fwd_tc */
int nxd_flash_attn_fwd_tc_window(const void* q, const void* k, const void* v, void* o, const long long* strides, int B,
                                 int Hq, int Hkv, int Sq, int Sk, int D, float scale, int window, int keep_first,
                                 const float* slopes, void* stream);
/* n = y / sqrt(mean(y^2) + eps) * (offset + w);  x (fp32, may be NULL) += n in place;  h (may be NULL) = cast(x or n) */
int nxd_post_norm_residual(int y_dtype, int w_dtype, int h_dtype, const void* y, const void* w, float* x, void* h,
                           long long rows, int W, float eps, float offset, void* stream);
/* parallel sublayers with layer scale and sigmoid-gated residual on an fp32 stream, then the next norm (one weight):
 * x += ls1 * sigmoid(gate[off1 + c] + gb1) * y1 + ls2 * sigmoid(gate[off2 + c] + gb2) * (y2 + y2_bias);
 * h = cast(x / sqrt(mean(x^2) + eps) * w_next[0]).  NULL y1: no update; NULL y2 / gate / w_next: that part is skipped */
int nxd_gated_residual_norm(float* x, const void* y1, int y1_dtype, const void* y2, int y2_dtype, const float* y2_bias,
                            const void* gate, int gate_dtype, long long ld_g, int off1, int off2, const float* gb1,
                            const float* gb2, const float* ls1, const float* ls2, const float* w_next, void* h,
                            int h_dtype, long long rows, int W, float eps, void* stream);
/* gated delta rule (csrc/delta_rule.cu): short convolution + silu + unit norm, convolution state, recurrence */
int nxd_delta_prep(int dtype, const void* proj, long long ld, int off_q, int off_k, int off_v, const float* conv_w,
                   const float* conv_state, float* qn, float* kn, float* vn, const int* q_start, const int* n_new,
                   const int* seq_ids, int B, int Tn, int H, int G, int D, int Dv, int taps, float qscale, float unit_eps,
                   void* stream);
int nxd_delta_conv_state(int dtype, const void* proj, long long ld, int off_q, int off_k, int off_v, float* conv_state,
                         const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G, int D,
                         int Dv, int taps, void* stream);
int nxd_delta_scan(const float* qn, const float* kn, const float* vn, float* apre, long long ld_a, int a_off,
                   float* bpre, long long ld_b, int b_off, const float* a_log, const float* dt_bias, float* S,
                   float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn, int H, int G, int D,
                   int Dv, int per_channel, void* stream);
/* gate and up columns of a wider row (+ fp32 biases or NULL) -> gated activation as in nxd_clamped_glu, out [rows, F];
 * act_kind 1: the gate goes through the tanh form of gelu instead of g * sigmoid(alpha g) */
int nxd_glu_bias(int dtype, const void* src, long long ld, int gate_off, int up_off, const float* gate_bias,
                 const float* up_bias, void* out, long long rows, int F, float limit, float alpha, float up_shift,
                 int act_kind, void* stream);
/* router: s = softmax(wr h + zbias); the `top` largest (s + corr) are chosen, weight = s * out_scale; sgate =
 * sigmoid(<wsg, h>).  mode 1: the `top` largest logits are chosen, weight = softmax over the chosen logits; mode 2:
 * s = sigmoid of every logit instead of the softmax */
int nxd_moe_router(int dtype, const void* h, const float* wr, const float* corr, const float* wsg, int* idx, float* wts,
                   float* sgate, long long N, int W, int R, int top, float out_scale, const float* zbias, int mode,
                   void* stream);
/* expert weights [E, in, out]; an index outside [0, E) is an identity expert; in_scale [P] fp32 or NULL multiplies the
 * pair's input row */
int nxd_moe_gate_up_act(int dtype, const void* h, const void* wgu, const int* idx, void* act, long long P,
                        int pairs_per_token, int W, int F, int E, float limit, float alpha, float up_shift,
                        const float* in_scale, void* stream);
int nxd_moe_down_combine(int dtype, const void* act, const void* wd, const int* idx, const float* wts, const void* h,
                         const void* act_s, const void* wds, const float* sgate, float* y, long long N, int top, int W,
                         int F, int Fs, int E, void* stream);
int nxd_clamped_glu(int dtype, const void* gate_up, void* out, long long M, int F, float limit, float alpha,
                    float up_shift, void* stream);
int nxd_moe_gather_combine(int dtype, const void* ys, const int* slot, const int* idx, const float* wts, const void* h,
                           const void* shared_out, const float* sgate, float* y, long long N, int top, int W, int E,
                           void* stream);

/* Retention (csrc/retention.cu): S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t on the fp32 state [lines, H, D, Dv] of
 * cache line seq_ids[b] (or b; zero state where q_start[b] == 0).  proj [B * Tn, ld] holds q / k / v head-major at the
 * column offsets (dtype 0 bf16, 1 fp32); q and k turn on their first rot dimensions by cos / sin tables [max_pos, rot / 2]
 * (NULL: no rotation; halves: pairs (i, i + rot / 2), else (2i, 2i + 1)), k is multiplied by kscale afterwards.
 * out [B * Tn, H, Dv] fp32; tokens t >= n_new[b] are padding.  The chunk-wise form (chunks of 64 tokens) needs fp32
 * scratch U [B, H, ceil(Tn / 64), D, Dv] and qrot [B * Tn, H, D]. */
int nxd_retention_scan(int dtype, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* decay,
                       float* state, float* out, const int* q_start, const int* n_new, const int* seq_ids, int B, int Tn,
                       int H, int D, int Dv, float kscale, const float* rope_cos, const float* rope_sin, int rot,
                       int halves, int max_pos, void* stream);
int nxd_retention_chunkwise(int dtype, const void* proj, long long ld, int q_off, int k_off, int v_off, const float* decay,
                            float* state, float* out, float* U, float* qrot, const int* q_start, const int* n_new,
                            const int* seq_ids, int B, int Tn, int H, int D, int Dv, float kscale, const float* rope_cos,
                            const float* rope_sin, int rot, int halves, int max_pos, void* stream);
/* Hyper-connections (csrc/hyper_connection.cu): X [N, S, W] fp32 streams.  ya != NULL: x_t <- sum_s mix[s][t] x_s +
 * outw[t] * y with y = ya, or (yb != NULL) 0.5 * (rmsnorm(ya) * wa + rmsnorm(yb) * wb).  inw != NULL: h [N, W] = RMS norm
 * (weight wn) of sum_s inw[s] x_s, of the streams as the write left them.  y_dtype / h_dtype: 0 bf16, 1 fp32. */
int nxd_hc_step(int y_dtype, int h_dtype, float* X, const void* ya, const void* yb, const float* wa, const float* wb,
                const float* mix, const float* outw, const float* inw, const float* wn, void* h, long long N, int S, int W,
                float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NXD_B200_H */
