// C entry points of the sm_100a kernels. Pointers are device pointers; every launcher enqueues on
// `stream` and returns 0 or an error code (cudaError_t value, or a negative code for bad arguments).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// GEMM epilogue flags
#define GEMM_FLAG_BIAS 1          // + bias[n]
#define GEMM_FLAG_GELU 2          // tanh-GeLU after bias
#define GEMM_FLAG_SAVE_PREACT 4   // also write (acc + bias) to aux_out (needed by the GeLU backward)
#define GEMM_FLAG_DGELU 8         // multiply by gelu'(aux[m,n])
#define GEMM_FLAG_RESIDUAL 16     // + aux[m,n] (aux has the output dtype)
#define GEMM_FLAG_OUT_FP32 32     // D is fp32 (default: same 16-bit type as the inputs)
#define GEMM_FLAG_ACCUMULATE 64   // D += result
#define GEMM_FLAG_FP16 128        // inputs are fp16 (default bf16)
#define GEMM_FLAG_CE_STATS 256    // LM head + cross-entropy, forward: no D; per (row, 128-column block) the epilogue emits
                                  // (max, sum exp(x - max), logit of the row's label if it lies in the block)
#define GEMM_FLAG_CE_GRAD 512     // LM head + cross-entropy, backward: D = (exp(x - lse[row]) - [col == label]) * scale[row]
#define GEMM_CE_BLOCK 128         // columns per statistics record

#define OSLO_DT_BF16 0
#define OSLO_DT_FP16 1
#define OSLO_DT_FP32 2

#ifdef __cplusplus
extern "C" {
#endif

int oslo_gemm_16bit(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd,
                    int a_mn_major, int b_mn_major, const void* bias, const void* aux, int ld_aux, void* aux_out,
                    int ld_aux_out, int flags, float alpha, int* err_word, int num_sms, cudaStream_t stream);

// LM-head product with the cross-entropy pieces in its epilogue (x = A B^T + bias, never written as logits):
//   mode 0 (GEMM_FLAG_CE_STATS): stats [ceil(N / 128), M, 3] fp32 records (max, sum exp, label logit or 0)
//   mode 1 (GEMM_FLAG_CE_GRAD):  D [M, N] (input dtype) = (softmax - onehot) * scale, from lse / scale fp32 [M]
// labels int64 [M] are global vocabulary ids; this rank's columns are ids vocab_start .. vocab_start + N - 1
int oslo_gemm_ce_16bit(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int b_mn_major,
                       const void* bias, const long long* labels, long long vocab_start, int mode, float* stats,
                       const float* lse, const float* scale, void* D, int ldd, int fp16, int* err_word, int num_sms,
                       cudaStream_t stream);
// (max, sum exp, label logit) per row from the per-block records of mode 0
int oslo_ce_reduce_stats(const float* stats, float* rowmax, float* sumexp, float* target, int rows, int blocks,
                         cudaStream_t stream);

// few-row GEMM for decode steps (M <= 128): k range cut into `split_k` slices, slice s writes its fp32 partial sums
// to plane s of D [split_k, M, N]; oslo_gemm_split_k_for suggests the slice count (1 = use oslo_gemm_16bit)
int oslo_gemm_split_k_for(int M, int N, int K, int num_sms);
int oslo_gemm_splitk_16bit(const void* A, const void* B, float* D, int M, int N, int K, int lda, int ldb, int ldd,
                           int a_mn_major, int b_mn_major, int fp16, int split_k, int* err_word, int num_sms,
                           cudaStream_t stream);
// out = T(act(sum over planes of ws + bias)) for the [split_k, rows, cols] fp32 result of the split-K GEMM;
// tanh-GeLU on columns >= gelu_from (-1 = none)
int oslo_splitk_finalize(const float* ws, const void* bias, void* out, long long rows, int cols, int split_k,
                         int gelu_from, int dtype, cudaStream_t stream);

// LayerNorm over the last dim of [rows, cols]; mean/rstd are fp32 [rows]
int oslo_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows,
                       int cols, float eps, int dtype, cudaStream_t stream);
// dw/db partial sums: [parts, cols] fp32 workspaces, reduced by a second kernel into dw/db (input dtype)
int oslo_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx,
                       float* dw_part, float* db_part, void* dw, void* db, int rows, int cols, int parts, int dtype,
                       cudaStream_t stream);

int oslo_bias_gelu_fwd(const void* x, const void* bias, void* y, long long rows, int cols, int dtype,
                       cudaStream_t stream);
int oslo_bias_gelu_bwd(const void* dy, const void* x, const void* bias, void* dx, long long rows, int cols, int dtype,
                       cudaStream_t stream);
// y = dropout(x + bias) + residual; the keep-mask is a counter hash of (seed, element index), so backward
// regenerates it instead of storing it. mode 0 = forward, 1 = backward (x is dy; bias/residual ignored)
int oslo_bias_dropout_residual(const void* x, const void* bias, const void* residual, void* y, long long rows,
                               int cols, float p, unsigned long long seed, int mode, int dtype, cudaStream_t stream);
// column sums of [rows, cols] into fp32 [cols] (bias gradients); part is a [parts, cols] workspace
int oslo_colsum(const void* x, float* part, float* out, int rows, int cols, int parts, int dtype,
                cudaStream_t stream);

// GPT-J rotary on [B, S, heads, D] (contiguous), pairs (2i, 2i+1) of the first rotary_dim dims; positions
// int64 [B, S]; inverse = 1 applies the transpose rotation (backward)
int oslo_rotary(const void* x, void* y, const long long* positions, int B, int S, int H, int D, int rotary_dim,
                float base, int inverse, int dtype, cudaStream_t stream);

// same rotation applied in place; touches only the first rotary_dim dims of each head (rotary_dim % 8 == 0, D % 8 == 0)
int oslo_rotary_inplace(void* x, const long long* positions, int B, int S, int H, int D, int rotary_dim, float base,
                        int inverse, int dtype, cudaStream_t stream);

// softmax on materialised scores
int oslo_causal_softmax_fwd(const void* x, void* y, int batches, int sq, int sk, float scale, int dtype,
                            cudaStream_t stream);
int oslo_masked_softmax_fwd(const void* x, const uint8_t* mask, void* y, int b, int h, int sq, int sk,
                            int mask_b, float scale, int dtype, cudaStream_t stream);
int oslo_softmax_bwd(const void* y, const void* dy, void* dx, long long rows, int cols, float scale, int dtype,
                     cudaStream_t stream);

// cross-entropy pieces over logits [rows, cols] (16-bit or fp32), labels int64 shifted by vocab_start
int oslo_ce_stats(const void* logits, const long long* labels, float* rowmax, float* sumexp, float* target,
                  int rows, int cols, int ld, long long vocab_start, int dtype, cudaStream_t stream);
int oslo_ce_grad(void* logits, const long long* labels, const float* lse, const float* scale, int rows, int cols,
                 int ld, long long vocab_start, int dtype, cudaStream_t stream);

// AdamW on flat buffers: fp32 master p, 16-bit or fp32 grads, optional 16-bit copy of the new params
int oslo_adam(float* p, const void* g, float* m, float* v, void* p_lp, long long n, float lr, float beta1,
              float beta2, float eps, float wd, float bc1, float bc2, float grad_scale, const float* inv_scale_dev,
              int g_dtype, int lp_dtype, cudaStream_t stream);
// sum of squares of a flat buffer into out[0] (atomic add; zero it first)
int oslo_sumsq(const void* x, float* out, long long n, int dtype, cudaStream_t stream);

// n-gram repeat blocking: lprobs[row, tok] = -inf for tokens that would complete a seen n-gram
int oslo_ngram_ban(const long long* tokens, float* lprobs, int rows, int len, int vocab, int n, int* err_word,
                   cudaStream_t stream);

// flash attention. q/k/v/o: element strides for (batch, head, seq); last dim contiguous
int oslo_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const uint8_t* kpm, int B,
                   int H, int Sq, int Sk, int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                   long long k_sh, long long k_ss, long long v_sb, long long v_sh, long long v_ss, long long o_sb,
                   long long o_sh, long long o_ss, float scale, int causal, int window, int dtype,
                   cudaStream_t stream);
// same contract as oslo_flash_fwd, on the tcgen05 tensor cores with TMEM accumulators (attention_sm100.cu)
int oslo_flash_fwd_sm100(const void* q, const void* k, const void* v, void* o, float* lse, const uint8_t* kpm, int B,
                         int H, int Sq, int Sk, int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                         long long k_sh, long long k_ss, long long v_sb, long long v_sh, long long v_ss, long long o_sb,
                         long long o_sh, long long o_ss, float scale, int causal, int window, int dtype, int* err_word,
                         cudaStream_t stream);
int oslo_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                   float* delta, float* dq_acc, void* dq, void* dk, void* dv, const uint8_t* kpm, int B, int H,
                   int Sq, int Sk, int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb,
                   long long k_sh, long long k_ss, long long v_sb, long long v_sh, long long v_ss, long long o_sb,
                   long long o_sh, long long o_ss, long long do_sb, long long do_sh, long long do_ss, float scale,
                   int causal, int window, int dtype, cudaStream_t stream);
// same contract on the tcgen05 tensor cores (attention_bwd_sm100.cu); dq / dk / dv use the strides of q / k / v
int oslo_flash_bwd_sm100(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                         float* delta, void* dq, void* dk, void* dv, const uint8_t* kpm, int B, int H, int Sq, int Sk,
                         int D, long long q_sb, long long q_sh, long long q_ss, long long k_sb, long long k_sh,
                         long long k_ss, long long v_sb, long long v_sh, long long v_ss, long long o_sb, long long o_sh,
                         long long o_ss, long long do_sb, long long do_sh, long long do_ss, float scale, int causal,
                         int window, int dtype, int* err_word, cudaStream_t stream);
// single-query attention over a static cache [B, H, T, D]; lengths int32 [B]
int oslo_decode_attn(const void* q, const void* kc, const void* vc, void* o, const int* lengths, float* ws, int B,
                     int H, int T, int D, int splits, float scale, int window, int dtype, int* err_word,
                     cudaStream_t stream);

// GEMM fused with a tensor-parallel collective (fused_comm_gemm.cu); mode 1 = all-reduce (result left in the
// symmetric staging matrix), 2 = reduce-scatter into out, 3 = all-gather of A then GEMM into out
// aux / ld_aux: with GEMM_FLAG_RESIDUAL in the reduce modes, another per-rank partial sum [M, N] added before the reduction
int oslo_gemm_comm_16bit(const void* A, const void* B, int M, int N, int K, int lda, int ldb, int a_mn_major,
                         int b_mn_major, const void* bias, const void* aux, int ld_aux, void* aux_out, int ld_aux_out,
                         int flags, float alpha,
                         void* const* peer_bufs_dev, void* own_buf, void* mc_base, long long data_off,
                         long long flag_off, long long flag_bytes, int rank, int world, unsigned epoch,
                         unsigned done_base, int mode, int use_multimem, void* out, int ld_out, int wide_tiles,
                         unsigned long long* trace, int* err_word, int num_sms, cudaStream_t stream);

// symmetric-memory collectives (comm.cu)
int oslo_allreduce_symm(void* const* peer_ptrs_dev, void* mc_ptr, uint32_t* const* signal_ptrs_dev, void* out,
                        long long n, int rank, int world, int dtype, int use_multimem, int* err_word,
                        cudaStream_t stream);

// data-parallel reduce-scatter / all-gather of one bucket [lo, hi) (16-bit elements) of a symmetric flat buffer whose
// rank r owns [r * shard, (r + 1) * shard); in place (comm.cu)
int oslo_dp_reduce_scatter(void* const* peer_ptrs_dev, void* mc_ptr, uint32_t* const* signal_ptrs_dev, long long lo,
                           long long hi, long long shard, int rank, int world, int dtype, int use_multimem,
                           int* err_word, cudaStream_t stream);
int oslo_dp_all_gather(void* const* peer_ptrs_dev, void* mc_ptr, uint32_t* const* signal_ptrs_dev, long long lo,
                       long long hi, long long shard, int rank, int world, int use_multimem, int* err_word,
                       cudaStream_t stream);

// vocabulary-parallel cross-entropy: combine every rank's per-row (max, sum exp, label logit) over the group in one
// kernel through a symmetric staging buffer of 2 x 3 x cap floats (comm.cu)
int oslo_ce_combine(const float* mx, const float* se, const float* tg, float* out_mx, float* out_se, float* out_tg,
                    void* const* peer_ptrs_dev, uint32_t* const* signal_ptrs_dev, uint32_t* counters, int n, int cap,
                    int rank, int world, int* err_word, cudaStream_t stream);

// decode-step kernels (decode_sm100.cu). gemv_rows: out[m, n] = act([x1 | x2][m, :] . W[n, :] + bias[n]) for M <= 4
// rows, W [N, K1 + K2] K-major, tanh-GeLU on columns >= gelu_from (-1 = none); x2 may be null.
// `res` [M, N] (row stride ldr) is added after the activation; bias and res may be null.
int oslo_gemv_rows(const void* x1, int ld1, int K1, const void* x2, int ld2, int K2, const void* W, int ldw,
                   const void* bias, const void* res, int ldr, void* out, int ldo, int M, int N, int gelu_from,
                   int dtype, int num_sms, cudaStream_t stream);
// rotary on the new token's q and k, q -> q_out [B, H, D], k / v -> cache [B, H, Tmax, D] at write_index[0];
// the rotary position of row b is lengths[b]
int oslo_rotary_append(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
                       void* q_out, void* kc, void* vc, const int* lengths, const long long* write_index, int B, int H,
                       int D, int Tmax, int rotary_dim, float base, int dtype, int* err_word, cudaStream_t stream);

// vocab-parallel embedding lookup + its collective in one kernel (comm.cu): the owner of a token's row stores it into
// every rank's staging half of the symmetric buffer, one cross-rank barrier, copy-out
int oslo_vocab_embed(const long long* ids, const void* weight, void* out, void* const* peer_ptrs_dev, void* mc_ptr,
                     uint32_t* const* signal_ptrs_dev, uint32_t* counters, long long tokens, int H, long long lo,
                     long long hi, long long half_bytes, int rank, int world, int dtype, int use_multimem, int* err_word,
                     int num_sms, cudaStream_t stream);

// bounded wait on a local flag with a caller-chosen limit (<= 1 s); for tests of the give-up path (comm.cu)
int oslo_wait_probe(const uint32_t* flag, uint32_t target, unsigned long long limit_ns, int* err_word,
                    unsigned long long* waited_ns, cudaStream_t stream);

// one-kernel all-reduce for small tensors (comm.cu): in -> staging half in symmetric memory -> sum over ranks -> out
int oslo_allreduce_oneshot(const void* in, void* out, void* const* peer_ptrs_dev, void* mc_ptr,
                           uint32_t* const* signal_ptrs_dev, uint32_t* counters, long long n, long long stage_off,
                           long long half_bytes, int rank, int world, int dtype, int use_multimem, int* err_word,
                           cudaStream_t stream);

#ifdef __cplusplus
}
#endif
