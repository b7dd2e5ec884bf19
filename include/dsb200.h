/* dsb200.h -- C ABI of libdsb200.so (CUDA, sm_100a only) and libdsb200_host.so (CPU).
 *
 * Every function returns 0 on success; on failure dsb200_last_error() describes what went wrong (thread-local).
 * Pointers are device pointers unless stated otherwise; `stream` is a cudaStream_t.  dtype codes: 0 = bf16,
 * 1 = fp16, 2 = fp32.  Reference citations name the file of delock/DeepSpeedSYCLSupport whose role the entry takes.
 */
#ifndef DSB200_H_
#define DSB200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* dsb200_stream_t;

const char* dsb200_last_error(void);
int dsb200_version(void);

/* ---- tcgen05 GEMM (reference: csrc/transformer/cublas_wrappers.cu:62,153; inference/v2/kernels/core_ops/blas_kernels/blas.h:35-138)
 * C[M,N] (=|+=) A*B, bf16 inputs, fp32 accumulate.  a_mn_major=0: A is [M][K]; 1: A stored [K][M].  b_mn_major=0: B is
 * [N][K]; 1: B stored [K][N].  out_mode 0 bf16 store, 1 fp32 store, 2 fp32 accumulate, 3 bf16 accumulate.
 * max_ctas caps the persistent grid (0 = all SMs). */
int dsb200_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn_major,
                     int b_mn_major, int out_mode, int max_ctas, dsb200_stream_t stream);

/* ---- fused optimizers on flat fp32 shards (reference: csrc/adam/multi_tensor_adam.cu, csrc/lion/multi_tensor_lion.cu,
 * csrc/lamb/fused_lamb_cuda_kernel.cu, csrc/common/custom_cuda_kernel.cu).  grad_type 0 fp32 / 1 bf16 / 2 fp16;
 * lp = optional 16-bit parameter copy written in the same pass (lp_type 0 none / 1 bf16 / 2 fp16);
 * inv_scale, skip: optional DEVICE scalars (gradient multiplier; non-zero skip leaves all buffers untouched). */
int dsb200_fused_adam_flat(float* p, float* m, float* v, const void* g, int grad_type, void* lp, int lp_type, long long n,
                           float lr, float beta1, float beta2, float eps, float weight_decay, int adamw_mode,
                           int bias_correction, int step, const float* inv_scale, const int* skip, dsb200_stream_t stream);
int dsb200_fused_lion_flat(float* p, float* m, const void* g, int grad_type, void* lp, int lp_type, long long n, float lr,
                           float beta1, float beta2, float weight_decay, const float* inv_scale, const int* skip,
                           dsb200_stream_t stream);
int dsb200_fused_adagrad_flat(float* p, float* h, const void* g, int grad_type, void* lp, int lp_type, long long n, float lr,
                              float eps, float weight_decay, const float* inv_scale, const int* skip, dsb200_stream_t stream);
int dsb200_fused_lamb_scratch_floats(long long n);
int dsb200_fused_lamb_flat(float* p, float* m, float* v, const void* g, int grad_type, void* lp, int lp_type, float* u,
                           float* scratch, long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                           int bias_correction, int step, float max_coeff, float min_coeff, const float* inv_scale,
                           const int* skip, float* coeff_out, dsb200_stream_t stream);
/* list-of-tensors Adam: p/m/v/g/n are HOST arrays (of device pointers / element counts) */
int dsb200_multi_tensor_adam(int ntensors, void** p, void** m, void** v, const void** g, const long long* n, int grad_type,
                             float lr, float beta1, float beta2, float eps, float weight_decay, int adamw_mode,
                             int bias_correction, int step, const float* inv_scale, const int* skip, dsb200_stream_t stream);

/* ---- RMSNorm / LayerNorm (reference: inference/v2/kernels/core_ops/cuda_rms_norm/rms_norm.cu, cuda_layer_norm/layer_norm.cu,
 * csrc/transformer/normalize_kernels.cu).  residual/res_out/beta/mean/rstd/dx_add/dbeta may be NULL. */
int dsb200_norm_fwd(const void* x, const void* residual, const void* gamma, const void* beta, void* y, void* res_out,
                    float* mean, float* rstd, int rows, int hidden, float eps, int layer_norm, int dtype, dsb200_stream_t stream);
long long dsb200_norm_bwd_scratch_floats(int rows, int hidden, int layer_norm);
int dsb200_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* dx_add,
                    void* dx, void* dgamma, void* dbeta, float* scratch, int rows, int hidden, int layer_norm, int dtype,
                    int dparam_f32, int accumulate, dsb200_stream_t stream);

/* RMSNorm backward that allocates nothing.  It has no counterpart in the reference.  For callers that cannot get device
 * memory when they run (a server whose KV-cache pool already owns all free HBM; a latency-critical loop that must avoid
 * the device-wide stall of cudaMalloc/cudaFree): the dgamma partials live in a fixed 4.6 MiB device array inside the
 * library (148 CTAs x hidden <= 8192 floats) that every GPU loading the library holds until exit.  hidden > 8192 is
 * rejected.  The first call on a device looks up the array's address -- make it before any stream capture.  All calls
 * share the array (it keeps the previous call's contents; nothing needs zeroing), so calls overlapping on the GPU race. */
int dsb200_rms_norm_bwd_noalloc(const void* dy, const void* x, const void* gamma, const float* rstd, const void* dx_add,
                                void* dx, void* dgamma, int rows, int hidden, int dtype, int dparam_f32, int accumulate,
                                dsb200_stream_t stream);

/* ---- element-wise transformer ops (reference: csrc/transformer/inference/csrc/apply_rotary_pos_emb.cu,
 * inference/v2/kernels/core_ops/gated_activations, core_ops/bias_activations, csrc/transformer/softmax_kernels.cu) */
int dsb200_rope_inplace(void* x, const int* positions, const float* inv_freq, long long tokens, int row_stride, int head0,
                        int nheads, int head_dim, int seq_len, int backward, int dtype, dsb200_stream_t stream);
int dsb200_gated_act_fwd(const void* in, const void* bias, void* out, long long rows, int F, int act, int interleaved, int dtype,
                         dsb200_stream_t stream);
int dsb200_gated_act_bwd(const void* in, const void* dout, void* din, long long rows, int F, int act, int interleaved, int dtype,
                         dsb200_stream_t stream);
int dsb200_bias_act(const void* in, const void* bias, void* out, long long rows, int cols, int act, int dtype,
                    dsb200_stream_t stream);
int dsb200_cross_entropy_fwd(const void* logits, const long long* labels, float* loss, float* lse, long long rows, int V,
                             long long ld, long long ignore_index, int dtype, dsb200_stream_t stream);
int dsb200_cross_entropy_bwd(void* logits, const long long* labels, const float* lse, const float* gscale, long long rows, int V,
                             long long ld, long long ignore_index, int dtype, dsb200_stream_t stream);
int dsb200_add(const void* a, const void* b, void* out, long long n, int dtype, dsb200_stream_t stream);

/* ---- host library (libdsb200_host.so; reference: csrc/adam/cpu_adam_impl.cpp, csrc/adagrad/cpu_adagrad.cpp,
 * csrc/lion/cpu_lion_impl.cpp).  All pointers are HOST pointers. */
int dsbh_simd_width(void);
int dsbh_adam_step(float* p, float* m, float* v, const void* g, int grad_type, void* lp, int lp_type, int64_t n, float lr,
                   float beta1, float beta2, float eps, float weight_decay, int adamw_mode, int bias_correction, int step,
                   float grad_scale);
int dsbh_adagrad_step(float* p, float* h, const void* g, int grad_type, void* lp, int lp_type, int64_t n, float lr, float eps,
                      float weight_decay, float grad_scale);
int dsbh_lion_step(float* p, float* m, const void* g, int grad_type, void* lp, int lp_type, int64_t n, float lr, float beta1,
                   float beta2, float weight_decay, float grad_scale);
int dsbh_cast_f32_lp(const float* src, void* dst, int lp_type, int64_t n);
double dsbh_sumsq(const void* g, int grad_type, int64_t n);

/* ==== generated by tools/gen_header.py from csrc/ -- do not edit below this line ==== */

/* ---- csrc/attn/evoformer.cu */
/* dtype: 0 bf16, 1 fp16.  q, k, v, o: [B][N][L][H][D] contiguous, D <= 64; bias1 [B][N][L] or NULL; bias2 [B][H][L][L] or NULL (same dtype);
 * lse: [B][N][H][L] fp32 (written). */
int dsb200_evoformer_attn_fwd(const void* q, const void* k, const void* v, const void* bias1, const void* bias2, void* o,
                              float* lse, int B, int N, int L, int H, int D, float scale, int dtype,
                              dsb200_stream_t stream);
/* Gradients: dq, dk, dv as q; dbias1 [B][N][L] / dbias2 [B][H][L][L] fp32, ZERO-INITIALISED by the caller (NULL = not wanted);
 * delta: [B][N][H][L] fp32 scratch. */
int dsb200_evoformer_attn_bwd(const void* q, const void* k, const void* v, const void* bias1, const void* bias2,
                              const void* o, const void* d_o, const float* lse, void* dq, void* dk, void* dv, float* delta,
                              float* dbias1, float* dbias2, int B, int N, int L, int H, int D, float scale, int dtype,
                              dsb200_stream_t stream);

/* ---- csrc/attn/flash_bwd.cu */
/* Gradient of dsb200_flash_attn_fwd.  dout/out: [B*S, hq*D] bf16; qkv, dqkv: packed [B*S, (hq+2*hkv)*D] bf16;
 * lse: [B, hq, S] from the forward.  Scratch supplied by the caller: dq_acc [B*S, hq*D] fp32 ZERO-INITIALISED,
 * delta [B, hq, S] fp32. */
int dsb200_flash_attn_bwd(const void* dout, const void* qkv, const void* out, const float* lse, void* dqkv, float* dq_acc,
                          float* delta, int B, int S, int hq, int hkv, int head_dim, int causal, float scale,
                          dsb200_stream_t stream);

/* ---- csrc/attn/flash_fwd.cu */
/* debug hook: device buffer (>= 8192 int64) receiving clock64 stamps of one CTA of the next forward launches; nullptr = off */
int dsb200_flash_fwd_trace(long long* buf);
/* out[B*S, hq*D] = softmax(Q K^T * scale [+ causal mask]) V with Q,K,V read from packed qkv [B*S, (hq+2*hkv)*D] (bf16).
 * lse: optional [B, hq, S] fp32 (natural-log sum-exp of the scaled scores) for the backward pass. */
int dsb200_flash_attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int hq, int hkv, int head_dim, int causal,
                          float scale, dsb200_stream_t stream);

/* ---- csrc/attn/paged_flash.cu */
/* Bytes of scratch dsb200_paged_flash_attention needs: atom list + count, plus the split-KV partials when n_splits > 1. */
long long dsb200_paged_flash_scratch_bytes(int n_tokens, int hq, int head_dim, int max_atoms, int n_splits);
/* out[t][hq*D] = attention of ragged token t over keys [0, tok_pos[t]] of its sequence, KV read from the blocked cache
 * [num_blocks][2][block_size][hkv][D] (bf16) through the block table.  max_atoms >= number of atoms of the batch
 * (<= n_tokens; ceil(n_tokens / (128/group)) + number of sequences is enough).  n_splits >= 1 splits the KV range of every atom.
 * alibi_slopes: optional [hq] fp32 (device): score += slope[head] * key position; NULL = none.
 * window > 0: local attention, a token sees its last `window` keys (itself included); 0 = the whole history. */
int dsb200_paged_flash_attention(const void* qkv, const void* kv_cache, void* out, const int* tok_seq, const int* tok_pos,
                                 const int* block_table, int n_tokens, int hq, int hkv, int head_dim, int block_size,
                                 int max_blocks_per_seq, int num_blocks, float scale, int max_atoms, int n_splits,
                                 void* scratch, const float* alibi_slopes, int window, dsb200_stream_t stream);
/* Same contract as dsb200_paged_flash_attention for batches of small atoms (decode steps): atoms hold at most 16 / group tokens,
 * keys take the M dimension of the MMAs (see paged_decode_kernel).  head_dim 128, q:kv head ratio dividing 16.
 * max_atoms >= ceil(n_tokens / (16/group)) + number of sequences (<= n_tokens). */
int dsb200_paged_flash_decode(const void* qkv, const void* kv_cache, void* out, const int* tok_seq, const int* tok_pos,
                              const int* block_table, int n_tokens, int hq, int hkv, int head_dim, int block_size,
                              int max_blocks_per_seq, int num_blocks, float scale, int max_atoms, int n_splits,
                              void* scratch, const float* alibi_slopes, int window, dsb200_stream_t stream);
/* Attention over a paged cache of latents: every one of the query heads of a token attends to the SAME cached rows, which serve as
 * keys and as values (one plane per block: cache [num_blocks][block_size][rank], bf16).  q holds q_heads <= heads query heads of
 * `rank` values per token at element strides q_head_stride / q_tok_stride (multiples of 8; token-major [T][heads][rank] or
 * head-major [heads][T][rank]); the kernel works on `heads` heads (a divisor of 128), the ones past q_heads read as zero.
 * out is [n_tokens][heads][rank] bf16; rank 64 or 128.  decode != 0 selects the small-atom kernel (rank 128, heads dividing 16).
 * Scratch and atoms as for dsb200_paged_flash_attention with hq = heads.
 * sink_logit (null, or `heads` floats): exp(sink_logit[h]) joins head h's softmax denominator, an entry without key and value. */
int dsb200_paged_flash_latent_sink(const void* q, int q_heads, long long q_head_stride, long long q_tok_stride,
                                   const void* cache, void* out, const int* tok_seq, const int* tok_pos,
                                   const int* block_table, int n_tokens, int heads, int rank, int block_size,
                                   int max_blocks_per_seq, int num_blocks, float scale, const float* sink_logit,
                                   int max_atoms, int n_splits, void* scratch, int decode, dsb200_stream_t stream);
int dsb200_paged_flash_latent(const void* q, int q_heads, long long q_head_stride, long long q_tok_stride,
                              const void* cache, void* out, const int* tok_seq, const int* tok_pos, const int* block_table,
                              int n_tokens, int heads, int rank, int block_size, int max_blocks_per_seq, int num_blocks,
                              float scale, int max_atoms, int n_splits, void* scratch, int decode, dsb200_stream_t stream);
/* Sliding-window attention that keeps the first keys visible, on the tensor-core kernels: a query at position p sees the keys j <= p with
 * p - j < window or j < keep_first.  q [n_tokens][hq][head_dim] bf16 at q_tok_stride elements per token (a multiple of 8), kv_cache
 * [num_blocks][2][block_size][hkv][head_dim] bf16; out rows at out_ld elements per token (a multiple of 8), multiplied by out_scale before
 * rounding.  Only the pages of the kept keys and of the window are visited.  decode != 0 selects the small-atom kernel (head_dim 128, q:kv
 * head ratio dividing 16).  Scratch and atoms as for dsb200_paged_flash_attention. */
int dsb200_paged_flash_window(const void* q, long long q_tok_stride, const void* kv_cache, void* out, long long out_ld,
                              const int* tok_seq, const int* tok_pos, const int* block_table, int n_tokens, int hq,
                              int hkv, int head_dim, int block_size, int max_blocks_per_seq, int num_blocks, float scale,
                              float out_scale, int window, int keep_first, int max_atoms, int n_splits, void* scratch,
                              int decode, dsb200_stream_t stream);
/* Causal attention with soft-capped scores and a sink in the softmax, on the tensor-core kernels: weights exp(s_j) / (sink + sum_j exp(s_j)),
 * s_j = scale q . k_j, capped as softcap tanh(s_j / softcap) when softcap > 0 (two more MUFU operations per score).  q [n_tokens][hq][head_dim]
 * bf16 at q_tok_stride elements per token (a multiple of 8), kv_cache [num_blocks][2][block_size][hkv][head_dim] bf16; out rows at out_ld
 * elements per token (a multiple of 8).  decode != 0 selects the small-atom kernel (head_dim 128, q:kv head ratios dividing 16).
 * sink_logit (hq floats): learned sinks, exp(sink_logit[h]) joins head h's denominator; r1, r2 (hq floats each): the score of key j for the
 * query at position i loses r1[h] ln(1 + r2[h] (i - j)); part > 0: a query sees only the keys of its own part of `part` positions.  Each may
 * be absent (null / 0). */
int dsb200_paged_flash_sink_ex(const void* q, long long q_tok_stride, const void* kv_cache, void* out, long long out_ld,
                               const int* tok_seq, const int* tok_pos, const int* block_table, int n_tokens, int hq,
                               int hkv, int head_dim, int block_size, int max_blocks_per_seq, int num_blocks, float scale,
                               float softcap, float sink, const float* sink_logit, const float* r1, const float* r2,
                               int part, int max_atoms, int n_splits, void* scratch, int decode, dsb200_stream_t stream);
int dsb200_paged_flash_sink(const void* q, long long q_tok_stride, const void* kv_cache, void* out, long long out_ld,
                            const int* tok_seq, const int* tok_pos, const int* block_table, int n_tokens, int hq, int hkv,
                            int head_dim, int block_size, int max_blocks_per_seq, int num_blocks, float scale,
                            float softcap, float sink, int max_atoms, int n_splits, void* scratch, int decode,
                            dsb200_stream_t stream);

/* ---- csrc/comm/symm.cu */
/* ---- allocation / mapping (host pointers unless noted) */
int dsb200_symm_alloc(long long bytes, void** ptr, unsigned char* handle64);
int dsb200_symm_open(const unsigned char* handle64, void** ptr);
int dsb200_symm_close(void* ptr);
int dsb200_symm_free(void* ptr);
/* peer_ptrs: HOST array of `world` device pointers (this process's mappings of every rank's buffer, own included) */
int dsb200_symm_barrier(void* const* peer_ptrs, long long flag_off, int rank, int world, unsigned int epoch,
                        dsb200_stream_t stream);
/* flag_off: a pad of `world` uint32 used ONLY by device-epoch barriers (zero-initialised); epoch_ctr: local device uint32 */
int dsb200_symm_barrier_dev(void* const* peer_ptrs, long long flag_off, int rank, int world, unsigned int* epoch_ctr,
                            dsb200_stream_t stream);
int dsb200_p2p_allgather(void* const* peer_ptrs, long long src_off, void* dst, long long bytes_per_rank, int rank,
                         int world, int max_ctas, dsb200_stream_t stream);
/* dst[p * bytes_per_chunk ...] = chunk `rank` of peer p's buffer at src_off (equal-split all_to_all_single); dst is local memory. */
int dsb200_p2p_alltoall(void* const* peer_ptrs, long long src_off, void* dst, long long bytes_per_chunk, int rank,
                        int world, int max_ctas, dsb200_stream_t stream);
/* src dtype / dst dtype: 0 bf16, 2 fp32.  n = elements per rank (multiple of 8).  sumsq: optional device float (+= sum g^2). */
int dsb200_p2p_reduce_scatter(void* const* peer_ptrs, long long src_off, int src_dtype, void* dst, int dst_dtype,
                              long long n, int rank, int world, float scale, int accumulate, float* sumsq, int max_ctas,
                              dsb200_stream_t stream);
/* Range form: Adam on elements [elem_lo, elem_lo + n) of this rank's slice (slice length n_per_rank) of the W*n_per_rank
 * bf16 gradient buffer at src_off.  p/m/v/lp/g_out point at element elem_lo of the local shard.  mc_base != NULL: the sum
 * comes from the NVSwitch (multimem.ld_reduce); NULL: pulled from the peers.  g_out / sumsq optional (may be NULL). */
int dsb200_p2p_rs_adam_range(void* const* peer_ptrs, void* mc_base, long long src_off, long long n_per_rank,
                             long long elem_lo, long long n, float* p, float* m, float* v, void* lp, void* g_out,
                             float* sumsq, int rank, int world, float scale, float lr, float beta1, float beta2, float eps,
                             float weight_decay, int adamw_mode, int bias_correction, int step, int max_ctas,
                             dsb200_stream_t stream);
int dsb200_p2p_rs_adam(void* const* peer_ptrs, long long src_off, float* p, float* m, float* v, void* lp, long long n,
                       int rank, int world, float scale, float lr, float beta1, float beta2, float eps, float weight_decay,
                       int adamw_mode, int bias_correction, int step, int max_ctas, dsb200_stream_t stream);
int dsb200_p2p_allreduce_bf16(void* const* peer_ptrs, long long src_off, void* dst, long long n, int rank, int world,
                              int max_ctas, dsb200_stream_t stream);
/* All-gather on the copy engines: one peer -> local cudaMemcpyAsync per rank (NVLink DMA, zero SMs), staggered so that at any
 * moment the ranks read from different peers.  dst is local memory; the peers' shards sit at src_off of their symmetric buffers. */
int dsb200_p2p_allgather_ce(void* const* peer_ptrs, long long src_off, void* dst, long long bytes_per_rank, int rank,
                            int world, dsb200_stream_t stream);
/* ---- NVLS entry points.  `mc_base` = multicast mapping of the symmetric buffer (every rank bound), DEVICE pointer.
 * src dtype / dst dtype: 0 bf16, 2 fp32.  n = elements per rank (multiple of 8). */
int dsb200_nvls_reduce_scatter(void* mc_base, long long src_off, int src_dtype, void* dst, int dst_dtype, long long n,
                               int rank, int world, float scale, int accumulate, float* sumsq, int max_ctas,
                               dsb200_stream_t stream);
/* In-place bf16 all-reduce of n elements at `off` (n % (8*world) == 0).  The caller brackets it with dsb200_symm_barrier. */
int dsb200_nvls_allreduce_bf16(void* mc_base, long long off, long long n, int rank, int world, int max_ctas,
                               dsb200_stream_t stream);
int dsb200_nvls_allgather(void* mc_base, long long dst_off, const void* src, long long bytes, int rank, int max_ctas,
                          dsb200_stream_t stream);
/* qgZ consumer: q_off / s_off = byte offsets of the fp8 payload (W*n bytes) and the fp32 block scales (W*n/128 floats) in
 * every rank's symmetric buffer; n = elements per rank (multiple of 128); dst dtype 0 bf16 / 2 fp32. */
int dsb200_p2p_fp8_reduce_scatter(void* const* peer_ptrs, long long q_off, long long s_off, void* dst, int dst_dtype,
                                  long long n, int rank, int world, float scale, int accumulate, float* sumsq,
                                  int max_ctas, dsb200_stream_t stream);
/* ---- MoE expert-parallel dispatch / combine over peer memory.  buf_off: byte offset of the [W][n_local][capacity][M] bf16
 * receive buffer inside every rank's symmetric buffer; token_expert / token_slot: [S][K] int32 (expert < 0 = dropped token). */
int dsb200_moe_dispatch_push(void* const* peer_ptrs, long long buf_off, const void* x, const int* token_expert,
                             const int* token_slot, const float* row_scale, int S, int K, int M, int rank, int world,
                             int n_local, int capacity, dsb200_stream_t stream);
/* out [S][M] bf16 (may be NULL when only dot_out is wanted); weights [S][K] fp32 or NULL; dot_with [S][M] bf16 + dot_out [S][K]
 * fp32 (zero-initialised by the caller) optional. */
int dsb200_moe_combine_pull(void* const* peer_ptrs, long long buf_off, void* out, const int* token_expert,
                            const int* token_slot, const float* weights, const void* dot_with, float* dot_out, int S,
                            int K, int M, int rank, int world, int n_local, int capacity, dsb200_stream_t stream);
/* Ulysses head <-> sequence exchange over peer memory.  `local`: [B * S_local][src_ld] bf16 (source layout); the dest-layout buffer
 * [B * S_local * world][dst_ld] lives at buf_off of every rank's symmetric buffer.  segs: n_seg x {src_col, dst_col, heads,
 * heads_per_rank} (ints, host).  push = 1: local -> owners' buffers; push = 0: owners' buffers -> local. */
int dsb200_ulysses_heads_exchange(void* const* peer_ptrs, long long buf_off, void* local, int B, int S_local, int rank,
                                  int world, int D, int src_ld, int dst_ld, const int* segs, int n_seg, int push,
                                  int max_ctas, dsb200_stream_t stream);

/* ---- csrc/elementwise/elementwise.cu */
/* out[0] += sum(x[i]^2) over n elements (dtype 0 bf16 / 1 fp16 / 2 fp32).  x must be 16-byte aligned. */
int dsb200_sumsq(const void* x, long long n, int dtype, float* out, dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_ag.cu */
/* C[M,N] (bf16) = A[M,K] * W^T with W[N,K] gathered from peers INSIDE the kernel.
 *   b_local     : [N,K] bf16 destination of the gather (kept for backward); also the GEMM's B operand
 *   peer_shards : HOST array of `world` device pointers -- each rank's shard region of the unit (this process's mappings)
 *   w_off       : flat element offset of W[0][0] inside the unit; shard_numel: elements per rank shard
 *   flags       : device scratch, >= ceil(N/256) + 1 ints (zeroed by this call): per n-block arrival counters + one work-claim counter */
int dsb200_gemm_ag_bf16(const void* A, void* b_local, void* C, int M, int N, int K, int lda, int ldc,
                        void* const* peer_shards, long long w_off, long long shard_numel, int* flags, int world,
                        dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_ar.cu */
int dsb200_gemm_ar_bf16(const void* A, const void* B, void* const* peer_ptrs, long long part_off, long long flag_off,
                        unsigned int epoch, void* out, const void* residual, int M, int N, int K, int lda, int ldb,
                        int ldo, int ldr, int rank, int world, int max_ctas, dsb200_stream_t stream);
/* GEMM -> reduce-scatter over rows (sequence-parallel tensor parallelism): same kernel, but this rank reduces and writes only rows
 * [row_lo, row_hi) of the sum -- out and residual are [row_hi - row_lo][N].  Every rank still publishes its whole partial (the
 * owners of the other rows need it); the row ranges of the ranks must cover [0, M) and every rank must own at least one row. */
int dsb200_gemm_rs_bf16(const void* A, const void* B, void* const* peer_ptrs, long long part_off, long long flag_off,
                        unsigned int epoch, void* out, const void* residual, int M, int N, int K, int lda, int ldb,
                        int ldo, int ldr, int rank, int world, int row_lo, int row_hi, int max_ctas,
                        dsb200_stream_t stream);
/* Graph-capturable forms: the epoch lives in device memory (`epoch_ctr`, one uint32 of LOCAL memory per rank, all ranks start it at
 * the same value); every call bumps it with a one-thread kernel in front of the GEMM, and the GEMM picks the partial area
 * part_off0 / part_off1 by the bumped value's parity.  A captured call therefore replays correctly any number of times.
 * row_lo = 0, row_hi = M: all-reduce; a sub-range: reduce-scatter over rows. */
int dsb200_gemm_ar_bf16_dev(const void* A, const void* B, void* const* peer_ptrs, long long part_off0, long long part_off1,
                            long long flag_off, unsigned int* epoch_ctr, void* out, const void* residual, int M, int N,
                            int K, int lda, int ldb, int ldo, int ldr, int rank, int world, int row_lo, int row_hi,
                            int max_ctas, dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_fp8.cu */
/* C[M,N] (bf16) = diag(sa) * (A * B^T) * diag(sb) with A [M][K], B [N][K] in e4m3 (one byte per element, K contiguous).
 * sa [M] / sb [N] fp32 scales, either may be null (= 1).  lda / ldb in elements (= bytes), multiples of 16; ldc multiple of 8. */
int dsb200_gemm_fp8(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N, int K, int lda,
                    int ldb, int ldc, int max_ctas, dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_fp8_block.cu */
/* C[M,N] (bf16) = sum over 128-wide K blocks of sa[m][kb] * sb[n][kb] * (A_kb * B_kb^T); A [M][K], B [N][K] e4m3 (K contiguous,
 * K % 128 == 0), sa [M][K/128], sb [N][K/128] fp32 (the layout dsb200_fp8_block_quantize writes for row-major operands). */
int dsb200_gemm_fp8_block(const void* A, const void* B, void* C, const float* sa, const float* sb, int M, int N, int K,
                          int lda, int ldb, int ldc, int max_ctas, dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_grouped.cu */
/* C[r, :] = A[r, :] * W[expert(r)]^T for rows sorted by expert; `cum` (device, int64[E]) holds inclusive cumulative row counts.
 * Rows at or beyond cum[E-1] are left untouched.  N must be a multiple of 8; A, W, C 16-byte aligned with 16-byte row strides. */
int dsb200_moe_gemm_bf16(const void* A, const void* W, void* C, const long long* cum, int R, int N, int K, int E, int lda,
                         int ldw, int ldc, dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_mxfp8.cu */
/* Bytes of the packed scale tensor for a [rows][K] operand (rows padded to a multiple of 256 so either operand role works). */
long long dsb200_mxfp8_sf_bytes(int rows, int K);
/* x [rows][K] (row stride ldx elements; dtype 0 bf16, 1 fp16, 2 fp32; K % 128 == 0) -> q [rows][K] e4m3 + sf (dsb200_mxfp8_sf_bytes,
 * ZERO-INITIALISED by the caller: rows beyond `rows` keep scale byte 0). */
int dsb200_mxfp8_quantize(const void* x, void* q, void* sf, int rows, int K, long long ldx, int dtype,
                          dsb200_stream_t stream);
/* C[M,N] (bf16) = dequant(A) * dequant(B)^T with MXFP8 operands (payload + packed UE8M0 scales from dsb200_mxfp8_quantize). */
int dsb200_gemm_mxfp8(const void* A, const void* B, void* C, const void* sfa, const void* sfb, int M, int N, int K,
                      int lda, int ldb, int ldc, int max_ctas, dsb200_stream_t stream);

/* ---- csrc/gemm/gemm_skinny.cu */
/* out[M][N] (bf16, row stride ldo) = x[M][K] w[N][K]^T, bf16 operands, M <= 128.  splits >= 1 cuts K; with splits > 1 the caller
 * passes a workspace of splits * M * N floats and N must be a multiple of 4.  K, ldx, ldw multiples of 8 (16-byte rows for TMA). */
int dsb200_gemm_skinny_bf16(const void* x, const void* w, void* out, void* workspace, int M, int N, int K, int ldx,
                            int ldw, int ldo, int splits, dsb200_stream_t stream);
/* out[M][N] (bf16) = x[M][K] (bf16) * dequant(wq)[N][K]^T, M <= 128.  bits = 8: wq int8 [N][K]; bits = 4: wq uint8 [N][K/2] (low nibble
 * first, value = nibble - 8).  scales fp32 [N][K / group], group a multiple of 64 dividing K; K a multiple of 64.
 * splits > 1 needs a workspace of splits * M * N floats and N, ldo multiples of 4. */
int dsb200_gemm_skinny_mixed(const void* x, const void* wq, const void* scales, void* out, void* workspace, int M, int N,
                             int K, int ldx, int ldo, int bits, int group, int splits, dsb200_stream_t stream);

/* ---- csrc/host/aio.cpp */
void* dsbh_aio_create(int64_t block_size, int queue_depth, int single_submit, int overlap_events, int num_threads);
void dsbh_aio_destroy(void* hp);
int64_t dsbh_aio_block_size(void* hp);
int dsbh_aio_queue_depth(void* hp);
int dsbh_aio_thread_count(void* hp);
/* Returns bytes waited for (>= 0) or -1 if any chunk failed since the last wait. */
int64_t dsbh_aio_wait(void* hp);
int dsbh_aio_pread(void* hp, void* buffer, int64_t nbytes, const char* path, int async, int64_t file_offset);
int dsbh_aio_pwrite(void* hp, const void* buffer, int64_t nbytes, const char* path, int async, int64_t file_offset);

/* ---- csrc/host/ragged_host.cpp */
void* dsbh_allocator_create(int num_blocks);
void dsbh_allocator_destroy(void* h);
int dsbh_allocator_free_blocks(void* h);
/* returns 0 on success, -1 when fewer than n blocks are free (nothing is allocated then) */
int dsbh_allocator_allocate(void* h, int n, int32_t* out);
/* returns 0 on success, -1 on an invalid / double free (allocator unchanged) */
int dsbh_allocator_free(void* h, const int32_t* blocks, int n);
/* seq_meta: per sequence (start token in batch, n new tokens, tokens already in the KV cache). Returns the atom count. */
int dsbh_build_atoms(const int32_t* seq_start, const int32_t* seq_ntok, const int32_t* seq_seen, int n_seqs, int q_block,
                     int kv_block, int32_t* atoms_out, int max_atoms);
/* Pack the per-token metadata of a ragged batch: tok_seq[t], tok_pos[t], last_tok[s]. */
int dsbh_pack_batch(const int32_t* seq_ntok, const int32_t* seq_seen, int n_seqs, int32_t* tok_seq, int32_t* tok_pos,
                    int32_t* last_tok);

/* ---- csrc/host/shm_comm.cpp */
/* Creates (rank 0) or attaches to the segment `/name`.  Returns an opaque handle or nullptr. */
void* dsbh_shm_open(const char* name, int rank, int world, long long chunk_bytes, double timeout_s);
/* In-place sum over all ranks of `numel` elements at `data`.  Returns 0, 1 (bad argument) or 2 (peer timeout). */
int dsbh_shm_allreduce(void* handle, void* data, long long numel, int dtype, double timeout_s);
int dsbh_shm_barrier(void* handle, double timeout_s);
void dsbh_shm_close(void* handle);

/* ---- csrc/host/sparse_lut.cpp */
/* Returns the number of non-zero blocks.  With out_h == nullptr only counts (and fills row_ptr if given). */
long long dsbh_sparse_lut(const int64_t* layout, int H, int M, int N, int64_t* out_h, int64_t* out_r, int64_t* out_c,
                          int64_t* row_ptr);

/* ---- csrc/quant/onebit.cu */
/* x[n] fp32 (read only), err[n] fp32 (error feedback, updated), packed[n/8], scale_io[2] fp32 device scratch:
 * on return scale_io[0] = ||x+err||_2 / sqrt(n).  n must be a multiple of 8; x/err 16-byte aligned. */
int dsb200_onebit_compress(void* x, void* err, void* packed, void* scale_io, long long n, dsb200_stream_t stream);
int dsb200_onebit_decompress(const void* packed, const void* scales, void* out, int rows, long long chunk_bytes, int mode,
                             dsb200_stream_t stream);

/* ---- csrc/quant/quantizer.cu */
/* x: n elements (n % 128 == 0) -> q: n bytes (e4m3), scales: n/128 floats */
int dsb200_fp8_block_quantize(const void* x, void* q, float* scales, long long n, int dtype, dsb200_stream_t stream);
int dsb200_fp8_block_dequantize(const void* q, const float* scales, void* out, long long n, int dtype,
                                dsb200_stream_t stream);
/* q: parts * n bytes, scales: parts * n/128 ; out: n elements = scale_out * sum over parts */
int dsb200_fp8_block_dequant_reduce(const void* q, const float* scales, void* out, long long n, int parts, float scale_out,
                                    int dtype, dsb200_stream_t stream);
/* groups * group_size elements; params: groups*2 floats (scale, offset); bits 8 or 4; q bytes = n * bits / 8 */
int dsb200_int_quantize(const void* x, void* q, float* params, long long groups, int group_size, int bits, int symmetric,
                        int dtype, dsb200_stream_t stream);
int dsb200_int_dequantize(const void* q, const float* params, void* out, long long groups, int group_size, int bits,
                          int symmetric, int dtype, dsb200_stream_t stream);
int dsb200_fake_quantize(void* x, long long groups, int group_size, int bits, int symmetric, int stochastic,
                         long long seed, int dtype, dsb200_stream_t stream);
/* q[rows][cols] (e4m3) and scales[rows] (fp32) with x ~= q * scale per row; x: [rows][cols] with row stride ldx (elements).
 * dtype: 0 bf16, 1 fp16, 2 fp32.  cols must be a multiple of 8. */
int dsb200_fp8_rowwise_quantize(const void* x, void* q, float* scales, int rows, int cols, long long ldx, int dtype,
                                dsb200_stream_t stream);

/* ---- csrc/ragged/latent_ops.cu */
/* out[t, :] = table[ids[t], :] + sinusoid(tok_pos[t]): entry 2i = sin(p f_i), entry 2i + 1 = cos(p f_i); `freq` holds the
 * ceil(dim / 2) frequencies as doubles on the device, or is null for no position vector (tok_pos is then unused).
 * table_dtype: 0 = bf16, 1 = fp32.  out is fp32.  The table row is multiplied by `scale` (in fp32) before the position vector is added. */
int dsb200_embed_sinusoid(const long long* ids, const void* table, int table_dtype, const int* tok_pos, const double* freq,
                          float* out, int n_tokens, int dim, float scale, dsb200_stream_t stream);
/* Per row of the fp32 residual x [n_rows, dim] (row rows[r] when `rows` is given): if y: x += y_mult * rms_norm(y) * (wb + ob); if w:
 * out = rms_norm(x) * (w + o); if plain_out (and no w): out = x.  y and out are bf16 (dtype 0) or fp32 (dtype 1); the weights are fp32.
 * out32 (optional, fp32 [n_rows, dim]) receives the normed values before their rounding to out's dtype (a router that decides in fp32
 * reads these). */
int dsb200_sandwich_norm(float* x, const void* y, int y_dtype, const float* wb, float ob, float y_mult, const float* w,
                         float o, void* out, int out_dtype, float* out32, const int* rows, int n_rows, int dim, float eps,
                         int plain_out, dsb200_stream_t stream);
/* Output row r works on row src = rows[r] (src = r without `rows`) of the fp32 residual x and of the branches: x[src] + y0[src] + y1[src] +
 * y2[src] (each branch optional; y0 and y1 in dtype y_dtype, y2 fp32) -- written back to x only without `rows` -- then, if w: out[r] = that
 * row split into `groups` equal consecutive parts, each over its own root mean square (eps inside the root), times w.  out bf16
 * (out_dtype 0) or fp32 (1); out32 (optional) the same values before rounding. */
int dsb200_stream_group_norm(float* x, const void* y0, const void* y1, int y_dtype, const float* y2, const float* w,
                             void* out, int out_dtype, float* out32, const int* rows, int n_rows, int dim, int groups,
                             float eps, dsb200_stream_t stream);
/* lat [n_tokens, ld] holds (query latent [nq] | key/value latent [nkv]) of every token.  cq [n_tokens, nq] = plain-weight RMS norm
 * of the first part; the RMS-normed second part is written to the token's row of cache [blocks, block_size, cache_ld] (cache_ld >= nkv:
 * rows may be padded to a width the tensor-core attention takes; the padding is never written). */
int dsb200_latent_norm_append(const void* lat, int ld, const float* wq, const float* wkv, void* cq, void* cache,
                              const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride,
                              int block_size, int cache_ld, int n_tokens, int nq, int nkv, float eps, int dtype,
                              dsb200_stream_t stream);
/* floats of scratch `dsb200_latent_attention` needs for n_splits > 1 */
long long dsb200_latent_attention_scratch_floats(int n_tokens, int H, int R, int n_splits);
/* out[t, h, :] = sum_j softmax_j(scale * q[t, h, :] . c_j) c_j over the cached latents c_0 .. c_pos(t) of the token's sequence.
 * q: bf16 / fp32 (q_dtype 0 / 1) with element strides per token and head; cache [blocks, block_size, R] bf16 / fp32 (cache_dtype);
 * out fp32 with element strides per token and head.  R <= 1024. */
int dsb200_latent_attention(const void* q, int q_dtype, long long q_tok_stride, long long q_head_stride, const void* cache,
                            int cache_dtype, float* out, long long o_tok_stride, long long o_head_stride, float* scratch,
                            const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride, int block_size,
                            int n_tokens, int H, int R, float scale, int n_splits, dsb200_stream_t stream);
/* a[r, c] *= sigmoid(g[r, c]) over [rows, cols] with row strides (elements).  dtype 0 = bf16, 1 = fp32. */
int dsb200_sigmoid_gate_mul(void* a, long long a_ld, const void* g, long long g_ld, long long rows, int cols, int dtype,
                            dsb200_stream_t stream);
/* out [n_tokens, H * dv] = heads of a [H, n_tokens, dv] (contiguous) laid side by side per token, times sigmoid(g) with g [n_tokens, H * dv]
 * at row stride g_ld (elements); g may be null (plain transposition).  dtype 0 = bf16, 1 = fp32. */
int dsb200_gate_heads(const void* a, const void* g, long long g_ld, void* out, int n_tokens, int H, int dv, int dtype,
                      dsb200_stream_t stream);
/* gu [rows, 2 F] = (gate | up) -> out [rows, F] = g' * sigmoid(alpha g') * (clamp(u, -limit, limit) + shift), g' = min(g, limit) */
int dsb200_clamped_swish_gate(const void* gu, void* out, long long rows, int F, float alpha, float limit, float shift,
                              int dtype, dsb200_stream_t stream);
/* out[r, c] = g' * sigmoid(alpha g') * (clamp(u, -limit, limit) + shift) with g' = min(gu[r, gate_col0 + c], limit), u = gu[r, up_col0 + c], c < F:
 * gate and up are column ranges of one fused projection gu [rows, ld]; out [rows, out_ld] may be a column range of a wider buffer. */
int dsb200_clamped_swish_gate_cols(const void* gu, long long ld, int gate_col0, int up_col0, void* out, long long out_ld,
                                   long long rows, int F, float alpha, float limit, float shift, int dtype,
                                   dsb200_stream_t stream);
/* x[r, c] = cap * tanh(x[r, c] / cap) over fp32 [rows, cols] with row stride ld */
int dsb200_softcap(float* x, long long ld, long long rows, int cols, float cap, dsb200_stream_t stream);
/* Router: scores = softmax over the E logits of a token, or (sigmoid_scores) the sigmoid of every logit on its own; selection score =
 * score + correction[e] (correction may be null); experts are split
 * into `groups` contiguous groups of equal size, of which the `keep` with the largest maximal selection score stay selectable; the top_k
 * selectable experts by selection score are assigned; their weights are the uncorrected scores (divided by their sum when
 * `normalize`).  Outputs as dsb200_top_k_gating; expert_counts must be zeroed by the caller. */
int dsb200_grouped_topk_gating(const float* logits, const float* correction, int* expert_counts, float* scores,
                               int* assignments, int* offsets, int n_tokens, int n_experts, int top_k, int groups,
                               int keep, int normalize, int sigmoid_scores, dsb200_stream_t stream);
/* Rows of x [n_tokens, dim] copied into expert-sorted order (any dim; dtype 0 = bf16, 1 = fp32); also writes the inclusive
 * per-expert row cumsum and every (token, k)'s row.  row_scale (optional, fp32 [n_tokens, top_k]): copy k of token t is multiplied by
 * row_scale[t, k] (routers whose weight applies to the expert's input). */
int dsb200_moe_scatter_rows(const void* x, const int* expert_counts, const int* assignments, const int* offsets,
                            long long* expert_cumsum, void* moe_in, int* mapped_slots, int n_tokens, int n_experts,
                            int dim, int top_k, int dtype, const float* row_scale, dsb200_stream_t stream);
/* out[t, :] (fp32) = sum_k scores[t, k] * moe_out[mapped_slots[t, k], :]; scores may be null (plain sum).  With `assignments` (the chosen
 * expert of every (token, k)): experts n_real and above are identity experts whose output is the token's row of identity_src (fp32
 * [n_tokens, dim]) instead of a row of moe_out. */
int dsb200_moe_gather_rows(const void* moe_out, const float* scores, const int* mapped_slots, float* out, int n_tokens,
                           int dim, int top_k, int dtype, const int* assignments, int n_real, const float* identity_src,
                           dsb200_stream_t stream);
/* Grouped expert GEMM on CUDA cores: out[r, :] = w[expert(r)] x[r, :] for the R rows sorted by expert; x [R, K], w [E, N, K],
 * out [R, N], all bf16 (dtype 0) or all fp32 (dtype 1), contiguous; fp32 accumulation.  expert_cumsum [E] int64 on the device. */
int dsb200_moe_gemm_rows(const void* x, const void* w, void* out, const long long* expert_cumsum, int R, int N, int K,
                         int E, int dtype, dsb200_stream_t stream);
/* x [rows, dim] fp32, in place: x <- s / sqrt(mean(s^2) + eps) * w with s = alpha x + y + y32 + bias; y [rows, dim] in y_dtype (0 = bf16,
 * 1 = fp32), y32 [rows, dim] fp32, bias [dim] fp32 -- each may be null.  out (null, or [rows, dim] in out_dtype): the new x, rounded. */
int dsb200_post_sum_norm(float* x, const void* y, int y_dtype, const float* y32, const float* bias, const float* w,
                         void* out, int out_dtype, long long rows, int dim, float alpha, float eps,
                         dsb200_stream_t stream);
/* out [rows, F] = xIELU(u [rows, ld]): z > 0: coef[0] z^2 + z / 2; z <= 0: coef[1] (exp(z) - 1 - z) + z / 2; coef: two floats on the device. */
int dsb200_xielu(const void* u, long long ld, void* out, long long rows, int F, const float* coef, int dtype,
                 dsb200_stream_t stream);
/* out[t, h dv + c] = a[h, t, c] * sigmoid(g[t, h]): a [H, n_tokens, dv] contiguous, g [n_tokens, g_ld] with one number per head. */
int dsb200_gate_heads_scalar(const void* a, const void* g, long long g_ld, void* out, long long out_ld, int n_tokens,
                             int H, int dv, int dtype, dsb200_stream_t stream);

/* ---- csrc/ragged/ragged_ops.cu */
int dsb200_kv_rotary_append(void* qkv, void* kv_cache, const int* tok_seq, const int* tok_pos, const int* block_table,
                            const float* inv_freq, int n_tokens, int hq, int hkv, int head_dim, int block_size,
                            int max_blocks_per_seq, int rot_dim, dsb200_stream_t stream);
int dsb200_paged_attention(const void* qkv, const void* kv_cache, void* out, const int* tok_seq, const int* tok_pos,
                           const int* block_table, int n_tokens, int hq, int hkv, int head_dim, int block_size,
                           int max_blocks_per_seq, float scale, dsb200_stream_t stream);
int dsb200_ragged_embed(const long long* ids, const void* wte, const void* wpe, const int* tok_pos, void* out,
                        int n_tokens, int dim, int pos_offset, dsb200_stream_t stream);
int dsb200_logits_gather(const void* hidden, const int* last_tok, void* out, int n_seqs, int dim, dsb200_stream_t stream);
/* expert_counts must be zeroed by the caller.  K <= 8, E <= 2048. */
int dsb200_top_k_gating(const float* logits, int* expert_counts, float* scores, int* assignments, int* offsets,
                        int n_tokens, int n_experts, int top_k, int normalize, dsb200_stream_t stream);
int dsb200_moe_scatter(const void* x, const int* expert_counts, const int* assignments, const int* offsets,
                       long long* expert_cumsum, void* moe_in, int* mapped_slots, int n_tokens, int n_experts, int dim,
                       int top_k, dsb200_stream_t stream);
int dsb200_moe_gather(const void* moe_out, const float* scores, const int* mapped_slots, void* out, int n_tokens, int dim,
                      int top_k, dsb200_stream_t stream);

/* ---- csrc/ragged/recurrent_ops.cu */
/* Floats of state_S per (slot, head) for a d x dv recurrent state (the layout is the scan kernels' own). */
long long dsb200_scan_state_floats(int d, int dv);
/* proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds, per token, the projections a windowed attention mixer convolves: queries [H d] at
 * column q_col0 and keys [G d] at k_col0.  Per token: short convolution (weights fp32 [channels, taps], last column = current token,
 * earlier rows from the batch or from `state` [slots, taps - 1, (H + G) d]) -> the convolved keys go to plane 1 of the token's cache row
 * (they are the values); RMS norm over the whole q / whole k projection with plain weights norm_q / norm_k; rotation of pairs (2i, 2i + 1)
 * of the first rot_dims entries of every head by pos * freq[i] (freq: doubles on the device); q to q_out [T, q_ld], k to cache plane 0.
 * cache [blocks, 2, block_size, G, d].  Call dsb200_conv_state_update afterwards. */
int dsb200_window_qk_prepare(const void* proj, long long ld, int q_col0, int k_col0, const float* conv_q,
                             const float* conv_k, const float* norm_q, const float* norm_k, const void* state,
                             const int* seq_desc, const int* tok_seq, const int* tok_pos, const int* block_table,
                             int bt_stride, int block_size, void* cache, void* q_out, long long q_ld, const double* freq,
                             int n_tokens, int H, int G, int d, int taps, int rot_dims, float eps, int dtype,
                             dsb200_stream_t stream);
/* Columns st_col0 .. st_col0 + C of state [slots, taps - 1, st_ld] <- the last taps - 1 projected rows (columns col0 .. col0 + C of proj
 * [T, ld]) of every sequence of the batch, older rows shifting up when the step brought fewer than taps - 1 tokens.  Run after the
 * kernels that read the state. */
int dsb200_conv_state_update(const void* proj, long long ld, int col0, void* state, int st_ld, int st_col0,
                             const int* seq_desc, int n_seqs, int C, int taps, int dtype, dsb200_stream_t stream);
/* out[t, h d + c] = out_scale * sum_j softmax_j(scale q_h . k_j) v_j[c] over the keys j <= pos(t) of the token's sequence with
 * pos - j < window or j < keep_first.  q [T, q_ld] (H heads of d), cache [blocks, 2, block_size, G, d] (plane 0 keys, 1 values), query head
 * h reads key/value head h / (H / G); out [T, out_ld].  CUDA cores, fp32 scores and accumulation, any sizes; dtype 0 = bf16, 1 = fp32. */
int dsb200_window_attention(const void* q, long long q_ld, const void* cache, const int* tok_seq, const int* tok_pos,
                            const int* block_table, int bt_stride, int block_size, void* out, long long out_ld,
                            int n_tokens, int H, int G, int d, int window, int keep_first, float scale, float out_scale,
                            int dtype, dsb200_stream_t stream);
/* Matrix memory with exponential gating, per sequence and head, over the new tokens in order:
 *   i = cap tanh((gates[t, h] + bias_i[h]) / cap),  f = logsigmoid(cap tanh((gates[t, H + h] + bias_f[h]) / cap)),
 *   m' = max(f + m, i);  S <- exp(f + m - m') S + exp(i - m') k v^T;  n likewise with k;  out = S^T q / (max(|n . q|, exp(-m')) + 1e-6)
 * with q = proj[q_col0 ..] * d^-1/2, k, v from proj [T, ld] (dtype 0 = bf16, 1 = fp32); gates fp32 [T, 2 H]; out fp32 [T, H dv].
 * state_S [slots, H, dsb200_scan_state_floats(d, dv)], state_n [slots, H, d], state_m [slots, H], all fp32; a sequence at position 0 starts
 * from zeros (m = 0). */
int dsb200_matrix_memory_scan(const void* proj, long long ld, int q_col0, int k_col0, int v_col0, const float* gates,
                              const float* bias_i, const float* bias_f, float cap, const int* seq_desc, float* state_S,
                              float* state_n, float* state_m, float* out, int n_seqs, int H, int d, int dv, int dtype,
                              dsb200_stream_t stream);
/* Inputs of the delta-rule scan from the fused projection proj [T, ld] (dtype 0 = bf16, 1 = fp32): q [G d] at q_col0, k [G d] at k_col0, v
 * [H dv] at v_col0, each through its short convolution (weights fp32 [channels, taps]; earlier rows from the batch or from `state`
 * [slots, taps - 1, 2 G d + H dv]) and silu; q and k then scaled to unit length per head (x / sqrt(sum x^2 + 1e-6)), q also by d^-1/2.
 * qn, kn fp32 [T, G d]; vo fp32 [T, H dv].  In place: a_pre fp32 [T, H d] <- exp(-exp(A_log[h]) softplus(a_pre + dt_bias)) (the decays) and
 * beta_pre fp32 [T, H] <- sigmoid(beta_pre).  Call dsb200_conv_state_update afterwards. */
int dsb200_delta_prepare(const void* proj, long long ld, int q_col0, int k_col0, int v_col0, const float* conv_q,
                         const float* conv_k, const float* conv_v, const void* state, const int* seq_desc,
                         const int* tok_seq, float* qn, float* kn, float* vo, float* a_pre, float* beta_pre,
                         const float* A_log, const float* dt_bias, int n_tokens, int G, int H, int d, int dv, int taps,
                         int dtype, dsb200_stream_t stream);
/* Gated delta rule with one decay per head and key channel, per sequence and head over the new tokens in order:
 *   S <- diag(decay[t, h, :]) S;  u = beta[t, h] (v - S^T k);  S <- S + k u^T;  out = S^T q
 * qn, kn fp32 [T, G d] (head h reads q / k head h / (H / G)), v fp32 [T, H dv], beta fp32 [T, H], decay fp32 [T, H d] (as dsb200_delta_prepare
 * leaves them); out fp32 [T, H dv]; state_S [slots, H, dsb200_scan_state_floats(d, dv)] fp32; a sequence at position 0 starts from zeros. */
int dsb200_delta_rule_scan(const float* qn, const float* kn, const float* v, const float* beta, const float* decay,
                           const int* seq_desc, float* state_S, float* out, int n_seqs, int H, int G, int d, int dv,
                           dsb200_stream_t stream);
/* Linear attention with the forget gate tied to the write strength, per sequence and head over the new tokens in order:
 *   q = silu(proj[q_col0 ..]),  f = lower + (1 - lower) sigmoid(proj[f_col0 ..] + f_bias),  S <- diag(f) S + (1 - f) v^T,  out = S^T q
 * proj [T, ld] (dtype 0 = bf16, 1 = fp32) with H heads of d (queries, gates) and dv (values); f_bias, lower fp32 [H d]; out fp32 [T, H dv];
 * state_S [slots, H, dsb200_scan_state_floats(d, dv)] fp32; a sequence at position 0 starts from zeros. */
int dsb200_tied_gate_scan(const void* proj, long long ld, int q_col0, int f_col0, int v_col0, const float* f_bias,
                          const float* lower, const int* seq_desc, float* state_S, float* out, int n_seqs, int H, int d,
                          int dv, int dtype, dsb200_stream_t stream);
/* out[t, h dv + c] = o[t, h, c] / sqrt(mean_c o[t, h, :]^2 + eps) * w[h * w_stride + c] * sigmoid(gate[t, h dv + c]) * mult.  o fp32
 * [T, H dv]; w fp32 (w_stride = dv: one weight row per head, 0: one row shared by the heads); gate [T, gate_ld] and out [T, out_ld] in the
 * activation dtype (0 = bf16, 1 = fp32).  gate may be null: mixers without an output gate. */
int dsb200_head_norm_gate(const float* o, const float* w, int w_stride, const void* gate, long long gate_ld, void* out,
                          long long out_ld, int n_tokens, int H, int dv, float eps, float mult, int dtype,
                          dsb200_stream_t stream);
long long dsb200_mingru_scratch_floats(int n_tokens, int n_seqs, int W);
/* Minimal gated recurrence over every sequence's new tokens.  proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds the gate, candidate and output-gate
 * pre-activations at columns z_col0 / x_col0 / g_col0 (W each); zb, xb fp32 [W]; state fp32 [slots, W]; out [T, out_ld] in proj's dtype.
 * seq_desc [n_seqs, 4] = (first row, new tokens, tokens seen before, slot); tok_seq [T].  scratch: dsb200_mingru_scratch_floats floats, used
 * when `pieces` != 0 (portions cut into pieces that are walked side by side); else one thread per (sequence, channel) walks its tokens. */
int dsb200_mingru_scan(const void* proj, long long ld, int z_col0, int x_col0, int g_col0, const float* zb,
                       const float* xb, const int* tok_seq, const int* seq_desc, float* state, void* out, long long out_ld,
                       int n_tokens, int n_seqs, int W, int pieces, float* scratch, int dtype, dsb200_stream_t stream);

/* ---- csrc/ragged/sink_attention_ops.cu */
/* proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds per token the query heads [H d] at q_col0, the key heads [G d] at k_col0 and the value heads
 * [G dv] at v_col0.  Query / key heads: RMS norm over d with the weights wq / wk [d] (shared by the heads; null = no norm), then rotation
 * of the first rot_dims entries (pairs (i, i + rot_dims / 2)) by pos * freq[i] (freq: rot_dims / 2 doubles on the device) with cosine and
 * sine multiplied by `mag`.  Value heads: divided by their root mean square over dv when norm_v.  Queries -> q_out [T, q_ld]; keys ->
 * k_cache, values -> v_cache at the token's (block, slot) (see the file header for the plane addressing).  q_row / k_row / v_row: elements
 * between consecutive heads of a query row / a cached key row / a cached value row (>= d, d, dv); what lies past a head's own entries is
 * written as zeros, so that heads padded to a common width of 64 / 128 can be served by the tensor-core attention kernels. */
int dsb200_head_norm_rotary_append(const void* proj, long long ld, int q_col0, int k_col0, int v_col0, const float* wq,
                                   const float* wk, const double* freq, float mag, const int* tok_seq, const int* tok_pos,
                                   const int* block_table, int bt_stride, int block_size, void* k_cache,
                                   long long k_block_stride, void* v_cache, long long v_block_stride, void* q_out,
                                   long long q_ld, int n_tokens, int H, int G, int d, int dv, int rot_dims, float eps,
                                   int norm_v, int q_row, int k_row, int v_row, int dtype, dsb200_stream_t stream);
/* out[t, h dv + c] = sum_j p_j v_j[c] over the keys j <= pos(t) of the token's sequence, p_j = exp(s_j) / (sink + sum_j exp(s_j)),
 * s_j = scale q_h . k_j, soft-capped as cap tanh(s_j / cap) when cap > 0.  q [T, q_ld] (H heads of d); query head h reads key/value head
 * h / (H / G); out [T, out_ld] (H heads of dv).  CUDA cores, fp32 scores and accumulation, any sizes; dtype 0 = bf16, 1 = fp32. */
int dsb200_sink_attention(const void* q, long long q_ld, const void* k_cache, long long k_block_stride,
                          const void* v_cache, long long v_block_stride, const int* tok_seq, const int* tok_pos,
                          const int* block_table, int bt_stride, int block_size, void* out, long long out_ld, int n_tokens,
                          int H, int G, int d, int dv, float scale, float cap, float sink, int dtype,
                          dsb200_stream_t stream);
/* `sink_attention` with learned sinks, a distance term, a mask by parts and free strides:
 *   sink_logit [H] (or null): exp(sink_logit[h]) joins head h's denominator;   r1, r2 [H] (or both null): s_j -= r1[h] ln(1 + r2[h] (pos - j));
 *   part > 0: only the keys of the query's own part of `part` positions (counted from position 0 of the sequence) are visible;
 *   q[t * q_ld + h * q_head_stride + c], out[t * out_ld + h * out_head_stride + c]; a cached key / value head starts every k_row / v_row
 *   elements of its token's row (one plane may serve as keys and as values: pass it twice, with d and dv entries read from a head's start). */
int dsb200_sink_attention_ex(const void* q, long long q_ld, long long q_head_stride, const void* k_cache,
                             long long k_block_stride, int k_row, const void* v_cache, long long v_block_stride, int v_row,
                             const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride, int block_size,
                             void* out, long long out_ld, long long out_head_stride, int n_tokens, int H, int G, int d,
                             int dv, float scale, float cap, float sink, const float* sink_logit, const float* r1,
                             const float* r2, int part, int dtype, dsb200_stream_t stream);
/* Low-rank attention with one rotated key part shared by the heads.  proj [T, ld] (dtype 0 = bf16, 1 = fp32) holds per token the H query heads
 * (d plain entries, then dr entries to rotate) from q_col0 and the low-rank row (R entries, then dr entries to rotate) from kv_col0.  The
 * query heads' rotated parts are rotated IN PLACE (first rot_dims of the dr entries; entry i pairs with entry i + rot_dims / 2; angle =
 * pos * freq[i], freq: rot_dims / 2 doubles on the device); the first R entries of the low-rank row are RMS-normed with wkv [R] and, with the
 * rotated last dr entries behind them, written to the token's row of cache [blocks, block_size, row_w] (zeros from R + dr on). */
int dsb200_latent_rotary_append(void* proj, long long ld, int q_col0, int kv_col0, const float* wkv, const double* freq,
                                const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride,
                                int block_size, void* cache, int row_w, int n_tokens, int H, int d, int dr, int R,
                                int rot_dims, float eps, int dtype, dsb200_stream_t stream);
/* Attention inputs behind a short causal convolution.  proj [T, ld] holds from col0 on the query heads [H d], the key heads [G d] and the value
 * heads [G dv] of every token; bias (fp32, that many entries, or null) is added to every row before the convolution with conv_w (fp32
 * [taps, channels]: y_t = sum_j w[j, :] u_(t - taps + 1 + j), zeros before the sequence's start).  state [slots, taps - 1, channels]: the last
 * rows of the sequence's earlier steps, WITHOUT the bias (update it afterwards with dsb200_conv_state_update).  Query / key heads: RMS norm over
 * d with wq / wk [d] shared by the heads -> q_out [T, q_ld] (head h at h * q_row) / the key plane.  Value heads: v_own (null, or [T, G dv])
 * receives the convolved values; with v_other ([T, G dv]) and mix (one float on the device) the cached value is (1 - mix) v + mix v_other.
 * Heads are padded with zeros to q_row / k_row / v_row entries. */
int dsb200_conv_head_norm_append(const void* proj, long long ld, int col0, const float* bias, const float* conv_w,
                                 const float* wq, const float* wk, const void* state, const int* seq_desc,
                                 const int* tok_seq, const int* tok_pos, const int* block_table, int bt_stride,
                                 int block_size, void* k_cache, long long k_block_stride, void* v_cache,
                                 long long v_block_stride, void* q_out, long long q_ld, const void* v_other,
                                 const float* mix, void* v_own, int n_tokens, int H, int G, int d, int dv, int taps,
                                 float eps, int q_row, int k_row, int v_row, int dtype, dsb200_stream_t stream);

/* ---- csrc/random_ltd/token_ops.cu */
/* idx: int32 [rows, reserved] of unique positions in [0, seq); sorted ascending in place, row by row. */
int dsb200_token_sort(void* idx, int rows, int reserved, int seq, dsb200_stream_t stream);
/* part[B,R,row] (batch_first) or part[R,B,row]  <-  all[B,S,row] / all[S,B,row] at idx[B,R] */
int dsb200_token_gather(const void* all, void* part, const void* idx, int B, int S, int R, long long row_bytes,
                        int batch_first, dsb200_stream_t stream);
int dsb200_token_scatter(void* all, const void* part, const void* idx, int B, int S, int R, long long row_bytes,
                         int batch_first, dsb200_stream_t stream);

/* ---- csrc/spatial/bias_add.cu */
/* dtype: 0 = fp32, 1 = fp16, 2 = bf16.  other / other_bias may be null.  channels * sizeof(T) must be a multiple of 16. */
int dsb200_nhwc_bias_add(const void* act, const void* bias, const void* other, const void* other_bias, void* out,
                         long long total, int channels, int dtype, dsb200_stream_t stream);

/* ==== end of generated section ==== */

#ifdef __cplusplus
}
#endif
#endif /* DSB200_H_ */
