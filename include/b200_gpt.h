/*
 * C ABI of libb200gpt: the GPT-2 forward hot path as hand-written sm_100a kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the given
 * CUDA stream (a cudaStream_t passed as void*; NULL = the legacy default stream)
 * and returns immediately with an int status (B200_OK or a B200_ERR_* code); none
 * of them synchronises, allocates or frees device memory, and none keeps a pointer
 * after it returns.  All tensors are row-major.  "dtype" arguments are b200_dtype
 * codes.  Citations name the operator of the reference project (gpt-triton) that an
 * entry point stands in for, by file:line within that project.
 */
#ifndef B200_GPT_H_
#define B200_GPT_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { B200_F32 = 0, B200_F16 = 1, B200_BF16 = 2 } b200_dtype;

enum {
  B200_OK = 0,
  B200_ERR_BAD_ARGUMENT = 1, /* a size, dtype code or NULL pointer the op cannot take */
  B200_ERR_ALIGNMENT = 2,    /* a pointer or leading dimension breaks a stated alignment rule */
  B200_ERR_CUDA = 3,         /* a CUDA runtime/driver call failed; see b200_last_cuda_error() */
  B200_ERR_UNSUPPORTED = 4,  /* valid for the reference operator but not built here (e.g. dropout > 0) */
  B200_ERR_WORKSPACE = 5,    /* workspace NULL or smaller than the *_workspace_bytes() figure */
  B200_ERR_DEVICE_WAIT = 6   /* a kernel gave up on a bounded on-chip wait; results are invalid */
};

/* Human-readable name of a status code (static storage). */
const char* b200_status_string(int status);
/* cudaGetErrorString of the last failing CUDA call made by this library on this thread. */
const char* b200_last_cuda_error(void);
/* ABI version of this header (6); bumped when a signature changes or an entry point is added. */
int b200_abi_version(void);
/* Number of kernels this library has launched in this process so far (all entry points). */
uint64_t b200_launch_count(void);

/*
 * out[t,:] = wte[ids[t],:] + wpe[t % L,:]   for t in [0, B*L)
 * Stands in for fused_embeddings (kernels.py:76-101; kernel kernels.py:37-72).
 * ids: int64 [B*L]; wte [V,H]; wpe [P,H]; out [B*L,H]; all of `dtype`.  Requires L <= P.
 * An id outside [0,V) writes a zero row and, if bad_id_flag (device int*) is not NULL,
 * stores 1 there (the reference reads out of bounds instead).
 */
int b200_embedding(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t B, int64_t L, int64_t V,
                   int64_t P, int64_t H, int dtype, int* bad_id_flag, void* stream);

/*
 * Row LayerNorm with fp32 statistics: out = (x - mean) * rsqrt(var + eps) * w + b.
 * Stands in for fused_layer_norm (kernels.py:149-164; kernel kernels.py:104-145).
 * x [M,H], w [H], b [H] of in_dtype; out [M,H] of out_dtype.  The reference always has
 * out_dtype == in_dtype; the (in, out) pairs built here are F32->F32, F16->F16, BF16->BF16
 * and F32->F16 / F32->BF16 (a 16-bit output from fp32 input gives the bits the following
 * GEMM would have produced by rounding its operand).  Any other pair of valid dtype codes
 * returns B200_ERR_UNSUPPORTED.
 */
int b200_layernorm(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t H, float eps,
                   int in_dtype, int out_dtype, void* stream);

/*
 * LayerNorm folded into the GEMM that follows it (the fusion the reference's author leaves as a TODO at
 * kernels.py:132-133): for a row x with statistics (mean, rstd), LayerNorm weight g and bias beta,
 *   LN(x) . w + bias = rstd * ( x . (g*w)  -  mean * colsum(g*w)  +  (1/rstd) * (beta . w + bias) ),
 * so a GEMM can take the RAW rows x and the normalised activations never exist in memory.  The two rank-one
 * terms are added by the tensor cores themselves: every row carries a 64-element "row extension"
 * [-mean, 1/rstd as high/low 16-bit parts, 0 ...] and every output column a "weight extension"
 * [colsum, beta.w + bias as high/low parts, 0 ...]; the consuming GEMM runs one extra 64-wide k-block over the
 * two, and its epilogue only multiplies by rstd.  B200_LN_EXT_COLS is the width of both extensions; they are of
 * the model's 16-bit dtype.  The entry points below produce and consume these pieces.
 */
#define B200_LN_EXT_COLS 64

/*
 * b200_embedding that also returns the LayerNorm statistics of every row it stores:
 * ln_stats_out (fp32 pairs, [B*L][2], 8-byte aligned) receives (mean, 1 / sqrt(variance + eps)) over the H
 * stored (rounded) values of the row, variance biased, both in fp32: exactly the two numbers
 * fused_layer_norm derives per row (kernels.py:116-130 of the reference).  ln_ext_out (optional; 16-bit dtype
 * only; [B*L][B200_LN_EXT_COLS] of `dtype`, 16-byte aligned) receives the rows' extensions.
 */
int b200_embedding_ln_stats(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t B, int64_t L, int64_t V,
                            int64_t P, int64_t H, int dtype, int* bad_id_flag, float eps, float* ln_stats_out, void* ln_ext_out, void* stream);

/*
 * LayerNorm statistics (and optionally row extensions) of the rows of an existing x [M,H] of `dtype`:
 * the statistics half of fused_layer_norm (kernels.py:116-130) without the normalised output.  Entry into a
 * chain of b200_gemm_ln calls for rows that no kernel of this library made.
 */
int b200_row_ln_stats(const void* x, float* ln_stats_out, void* ln_ext_out, int64_t M, int64_t H, float eps, int dtype, void* stream);

/*
 * Weight-side half of the fold, done once per weight version.  From w [K,N] row-major (the state-dict layout
 * of c_attn / c_fc), gamma and beta [K] (LayerNorm weight and bias) and bias [N] or NULL, all of the 16-bit
 * `dtype`, this writes
 *   packed [N, ld_packed] K-major (ld_packed >= K, a multiple of 8; tail columns zero) = round(gamma[k]*w[k,n]),
 *   colsum [N] fp32 = sum over k of the rounded packed values,   bias_out [N] fp32 = bias + beta . w,
 *   w_ext [N, B200_LN_EXT_COLS] of `dtype` (16-byte aligned) = the weight extensions made of those two.
 * B200_ERR_UNSUPPORTED for B200_F32 (the fp32 path keeps LayerNorm apart).
 */
int b200_fold_layernorm(const void* w, const void* gamma, const void* beta, const void* bias, void* packed, float* colsum, float* bias_out,
                        void* w_ext, int64_t K, int64_t N, int64_t ld_packed, int dtype, void* stream);

/*
 * b200_gemm with a LayerNorm on one side of it; io_dtype == op_dtype, 16-bit; 16-byte aligned out/residual
 * with pitches that are multiples of 8 elements (else B200_ERR_UNSUPPORTED).  Exactly one role per call:
 *
 * Consumer (ln_stats != NULL, ln_stats_out == NULL): A holds the RAW rows x [M,K], ln_stats[row] their
 * (mean, rstd), ln_ext [M, B200_LN_EXT_COLS] their extensions, B the `packed` weights and w_ext the weight
 * extensions of b200_fold_layernorm; stores [gelu](LN(x) . w + bias) + residual.  `bias` must be NULL (it is
 * inside w_ext).  Replaces fused_layer_norm + fused_ffn (gpt.py:40-43, 94-101) without the normalised
 * tensor; differs from that pair by roundings only (the normalised row is not rounded to 16 bits before the
 * product).
 *
 * Producer (ln_stats_out != NULL, ln_stats == NULL, add_gelu == 0): plain b200_gemm that also leaves
 * ln_stats_out[row] = (mean, 1 / sqrt(variance + eps)) over the N columns of every row it stores (taken from
 * the fp32 values before they are rounded) and ln_ext_out [M, B200_LN_EXT_COLS], ready for a following
 * consumer call.  The epilogue writes per-128-column partial sums to `workspace`
 * (b200_gemm_ln_workspace_bytes(M, N) bytes, 16-byte aligned) and a small second kernel merges them.
 */
size_t b200_gemm_ln_workspace_bytes(int64_t M, int64_t N);
int b200_gemm_ln(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype, int add_gelu, const float* ln_stats,
                 const void* ln_ext, const void* w_ext, float* ln_stats_out, void* ln_ext_out, float eps, void* workspace, size_t workspace_bytes,
                 int* status_word, void* stream);

/*
 * Operand packing for b200_gemm: dst[r, c] = cast(src[r, c]) (transpose == 0) or
 * dst[c, r] = cast(src[r, c]) (transpose != 0); columns of dst between the logical
 * width and ld_dst are zero-filled.  src [rows, cols] with leading dimension ld_src.
 * No counterpart in the reference, whose kernel casts operands on the fly
 * (kernels.py:229, 234); packing once is how the same rounding is obtained here.
 * dst_dtype must be 16-bit; f32->f16, f16->f16 and bf16->bf16 are supported.
 */
int b200_pack_operand(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst,
                      int transpose, int src_dtype, int dst_dtype, void* stream);

/*
 * out[M,N] = [gelu_new](A[M,K] . B[N,K]^T + bias[N]) + residual[M,N]
 * on the tcgen05 tensor cores, fp32 accumulation in tensor memory, epilogue order
 * bias -> GELU -> residual -> cast.  The compute core behind fused_ffn
 * (kernels.py:261-315; kernel kernels.py:169-257), with both operands K-major.
 * A [M,K] (lda) and B [N,K] (ldb) are 16-bit of op_dtype (F16 or BF16); bias,
 * residual (ld_res) and out (ld_out) are of io_dtype; bias and residual may be NULL.
 * Alignment: A and B 16-byte aligned, lda and ldb multiples of 8 elements.
 * status_word: optional device int*, set non-zero if a kernel abandons a bounded wait.
 */
int b200_gemm(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
              int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
              int add_gelu, int* status_word, void* stream);

/*
 * b200_gemm that additionally returns, per output row, the column of the row's maximum:
 * argmax_out[row] (int64, device) = argmax over the stored (rounded) out[row, 0..N), the lowest
 * column on ties.  Meant for the tied lm_head (gpt.py:159-161, 172-179 of the reference): greedy
 * next-token ids come out of the GEMM's epilogue instead of a second pass over the [tokens, vocab]
 * logits.  If lse_out (float, device, [M]) is not NULL it also receives the row log-sum-exp
 * log(sum_j exp(out[row, j])) over the stored values, so that a token's cross-entropy is
 * lse_out[row] - out[row, target] without reading the row again.  The epilogue writes per-128-column
 * partial results to `workspace` (b200_gemm_argmax_workspace_bytes(M, N) bytes, 16-byte aligned), a
 * small second kernel reduces them.
 */
size_t b200_gemm_argmax_workspace_bytes(int64_t M, int64_t N);
int b200_gemm_argmax(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                     int add_gelu, int64_t* argmax_out, float* lse_out, void* workspace, size_t workspace_bytes, int* status_word,
                     void* stream);

/*
 * Row statistics of the product without the product: for logits[M,N] = A[M,K] . B[N,K]^T (+ bias[N]) rounded to
 * round_dtype (F16 or BF16) exactly as b200_gemm would store them, returns per row argmax_out (int64, lowest column
 * on ties), lse_out (float, log-sum-exp over the rounded values; may be NULL, which saves one exponential per
 * logit) and, if `targets` (int64 [M], device) is not NULL,
 * target_logit_out[row] = logits[row, targets[row]] (float; rows whose target lies outside [0, N) are left
 * untouched).  Nothing of size M x N touches memory: the tied lm_head (gpt.py:159-161, 172-179 of the reference)
 * for greedy next-token ids or per-token cross-entropy (lse - target logit) without the [tokens, vocab] tensor.
 * bias is of round_dtype or NULL.  Workspace: b200_gemm_argmax_workspace_bytes(M, N) bytes, 16-byte aligned.
 */
int b200_gemm_rowstats(const void* a, const void* b, const void* bias, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                       int op_dtype, int round_dtype, const int64_t* targets, int64_t* argmax_out, float* lse_out,
                       float* target_logit_out, void* workspace, size_t workspace_bytes, int* status_word, void* stream);

/*
 * z = [gelu_new](x @ w + bias) + residual with the reference operator's own layouts:
 * stands in for fused_ffn (kernels.py:261-315).  x [M,K], w [K,N] (w_is_nk == 0, the
 * HF Conv1D layout) or [N,K] (w_is_nk != 0, e.g. the tied wte for lm_head,
 * gpt.py:159-161), bias [N], residual [M,N], out [M,N] with leading dimension ld_out,
 * all of `dtype`.  Operands are rounded to fp16 (bf16 stays bf16, which gives the same
 * products) exactly once.  workspace: scratch of at least b200_ffn_workspace_bytes()
 * bytes, 256-byte aligned, used for packed operands when x or w cannot be fed to the
 * tensor cores in place (fp32 storage, [K,N] weights, K not a multiple of 8,
 * unaligned pointers); may be NULL when that figure is 0.
 */
size_t b200_ffn_workspace_bytes(int64_t M, int64_t N, int64_t K, int w_is_nk, int dtype);
int b200_ffn(const void* x, const void* w, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
             int64_t K, int64_t ld_out, int w_is_nk, int add_gelu, int dtype, void* workspace, size_t workspace_bytes,
             int* status_word, void* stream);

/*
 * b200_ffn for callers that cannot allocate device memory (no counterpart in the reference, whose
 * operators allocate freely through torch).  Examples: a serving runtime that has given all free HBM
 * to its own pool, or an enqueue-style plugin callback where cudaMalloc and the device-wide
 * synchronisation it implies are not allowed.  Same arguments and results as b200_ffn minus the
 * workspace: the packed operands go to an array of B200_FFN_STATIC_SCRATCH_BYTES that is part of the
 * library image on every GPU that loads it (held until the process exits).  The call makes no
 * cudaMalloc/cudaFree or other allocating call.
 *  - Limit: what this call has to pack (an operand is packed unless it is 16-bit, 16-byte aligned, has
 *    K % 8 == 0 and, for w, the [N, K] layout; 2 * rows * roundup8(K) bytes each, rounded up to 256) must
 *    fit B200_FFN_STATIC_SCRATCH_BYTES, else the call returns B200_ERR_WORKSPACE and launches nothing.
 *    A call that packs nothing (e.g. the tied lm_head in fp16) is never refused for size.
 *  - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and keeps it; make that first call outside any stream capture.  The address
 *    belongs to the device's primary context: do not call again on a device after cudaDeviceReset.
 *  - Every call on a device shares the one array, which keeps the previous call's contents (nothing
 *    needs clearing: each call overwrites what it reads).  Two calls that may overlap on the GPU
 *    (different streams) race on it; serialise them.
 */
#define B200_FFN_STATIC_SCRATCH_BYTES (32u << 20)
int b200_ffn_static_scratch(const void* x, const void* w, const void* bias, const void* residual, void* out, int64_t M,
                            int64_t N, int64_t K, int64_t ld_out, int w_is_nk, int add_gelu, int dtype, int* status_word,
                            void* stream);

/*
 * Causal attention with online softmax over 64-key blocks, fp16 operands, fp32
 * statistics: stands in for flash_attention_v1 (kernels.py:478-525; kernel
 * kernels.py:375-474).  q, k, v, out are addressed as base + b*s[0] + h*s[1] + l*s[2] + d
 * with element strides s = {batch, head, row}; the innermost (head_dim) stride is 1.
 * Contiguous [B,NH,L,D] tensors use {NH*L*D, L*D, D}; views into a fused [B*L, 3*NH*D]
 * qkv buffer use {L*3*NH*D, D, 3*NH*D}, which is how the split/transposes of
 * matmul_and_split_qkv (kernels.py:348-367) and the merge of gpt.py:51 cost nothing.
 * D in {16, 32, 64, 128, 256}; scale is normally 1/sqrt(D).
 * status_word: optional device int*, set non-zero if the tensor-core kernel abandons a bounded wait.
 */
int b200_attention(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L, int64_t D,
                   const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                   const int64_t o_strides[3], float scale, int in_dtype, int out_dtype, int* status_word, void* stream);

/*
 * Token-by-token generation: key/value cache, one-query attention, sampling.  None of these has a counterpart in
 * the reference, which lists "KV cache + sampling" among the things it never built (README.md:55); the attention
 * arithmetic follows its flash_attention_v1 (kernels.py:417-474), so that a cached step gives what re-running
 * the whole sequence through b200_attention would, to rounding.
 *
 * Whatever changes from one generated token to the next is read from DEVICE memory, so the launches of a
 * decode step can be recorded once in a CUDA graph and replayed: `pos_dev` is a device int32 pair, 4-byte aligned,
 * pos_dev[0] = number of tokens whose keys/values are in the cache (= position of the token being decoded),
 * pos_dev[1] = length of the prompt.  The cache of one layer is [B, cache_len, 2H] of the model's dtype, keys in
 * columns [0, H), values in [H, 2H) (H = NH * D), 16-byte aligned.
 */

/*
 * b200_embedding (with the optional LayerNorm outputs of b200_embedding_ln_stats: pass NULL for both, or
 * ln_stats_out alone, or both) whose first position is *pos0_dev instead of 0:
 * out[t,:] = wte[ids[t],:] + wpe[*pos0_dev + t % L,:].  A position outside [0, P) is treated like a bad id
 * (zero row, *bad_id_flag = 1).
 */
int b200_embedding_at(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t B, int64_t L, int64_t V, int64_t P, int64_t H,
                      int dtype, int* bad_id_flag, float eps, float* ln_stats_out, void* ln_ext_out, const int32_t* pos0_dev, void* stream);

/*
 * After the prompt's forward: cache[b, l, 0:2H] = qkv[b, l, H:3H] for l < L, from the fused c_attn output
 * qkv [B, L, 3H] (q | k | v).  Needs L <= cache_len, H * element size a multiple of 16, 16-byte aligned pointers.
 */
int b200_kv_cache_fill(const void* qkv, void* cache, int64_t B, int64_t L, int64_t H, int64_t cache_len, int dtype, void* stream);

/*
 * One decode step of causal attention for every (batch, head): with pos = pos_dev[0], stores the new token's
 * key and value (qkv_new [B, 3H] = q | k | v of that token) into cache[b, pos, :] and writes
 * out[b, head*D : (head+1)*D] = softmax(q . K[0..pos]^T * scale) . V[0..pos]   (out [B, H]).
 * D in {32, 64, 128}, else B200_ERR_UNSUPPORTED.  If pos is outside [0, cache_len) nothing is read or written and
 * *status_word (device int*, may be NULL) receives the code 41.
 */
int b200_attention_decode(const void* qkv_new, void* cache, void* out, int64_t B, int64_t NH, int64_t D, int64_t cache_len, float scale, int dtype,
                          const int32_t* pos_dev, int* status_word, void* stream);

/*
 * tokens[b, column] = next_ids[b] with column = pos_dev[0] - pos_dev[1] + (advance ? 1 : 0); then, if advance,
 * pos_dev[0] += 1.  advance = 0 stores the token predicted by the prompt's forward (column 0), advance = 1 the
 * one predicted by a decode step.  tokens [B, n_cols] int64 with row pitch ld_tokens; a column outside
 * [0, n_cols) writes nothing and leaves the code 42 in *status_word.  feedback (int64 [B], may be NULL) receives
 * the same ids: the fixed buffer the next decode step's b200_embedding_at reads, so a replayed step feeds itself.
 */
int b200_decode_append(const int64_t* next_ids, int64_t* tokens, int64_t ld_tokens, int64_t n_cols, int64_t B, int32_t* pos_dev, int advance,
                       int64_t* feedback, int* status_word, void* stream);

/*
 * ids_out[b] = a draw from softmax(logits[b, :] / temperature) restricted to the top_k largest logits of the row
 * (top_k = 0: all V columns; logits tied with the top_k-th largest all stay in).  logits [B, V] of `dtype`, row
 * pitch ld; temperature > 0.  The draw is the Gumbel-max form, argmax_j(logit_j / temperature - log(-log(u_j))),
 * lowest j on ties, with u_j in (0, 1) a counter-based function of (seed, *step_dev, b, j) (step_dev: device
 * int32*, NULL = 0), so that a (seed, step) pair always gives the same ids.  Greedy decoding needs no call: the
 * lm_head GEMM returns the row argmax (b200_gemm_argmax / b200_gemm_rowstats).
 */
int b200_sample_logits(const void* logits, int64_t ld, int64_t B, int64_t V, int dtype, float temperature, int top_k, uint64_t seed,
                       const int32_t* step_dev, int64_t* ids_out, void* stream);

/*
 * Self-test of the bounded waits every tensor-core kernel of this library uses (no reference counterpart): launches
 * one warp that waits, with the library's own wait routine, on a shared-memory barrier that nothing ever completes.
 * After limit_cycles SM clock cycles (1 <= limit_cycles <= 4e9) the wait gives up, the kernel writes
 * B200_ERR_DEVICE_WAIT to *status_word (device int*, must be zero beforehand) and returns normally; the context
 * stays usable.  Shows on a healthy GPU that a lost signal ends in a status code and not in a hang.
 */
int b200_selftest_bounded_wait(int* status_word, int64_t limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_GPT_H_ */
