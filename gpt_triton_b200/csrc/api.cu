// extern "C" surface of libb200gpt (declared in include/b200_gpt.h): argument checks and
// composition of the kernels; no kernel code lives here.
#include "common.cuh"

#include <stdint.h>

namespace {
thread_local cudaError_t g_last_cuda = cudaSuccess;
int note(int st) {
  if (st == B200_ERR_CUDA) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) g_last_cuda = e;
  }
  return st;
}
bool valid_dtype(int dt) { return dt == B200_F32 || dt == B200_F16 || dt == B200_BF16; }
size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }
bool direct_operand_ok(int dtype, int64_t K) { return dtype != B200_F32 && K % 8 == 0; }
constexpr int64_t kMaxExtent = 0x7fffffffLL - 256;  // largest M, N or K the GEMM kernel indexes
}  // namespace

extern "C" {

const char* b200_status_string(int status) {
  switch (status) {
    case B200_OK: return "ok";
    case B200_ERR_BAD_ARGUMENT: return "bad argument";
    case B200_ERR_ALIGNMENT: return "alignment rule violated";
    case B200_ERR_CUDA: return "CUDA call failed";
    case B200_ERR_UNSUPPORTED: return "not supported";
    case B200_ERR_WORKSPACE: return "workspace missing or too small";
    case B200_ERR_DEVICE_WAIT: return "a kernel abandoned a bounded wait";
  }
  return "unknown status";
}

const char* b200_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda); }

int b200_abi_version(void) { return 6; }

uint64_t b200_launch_count(void) { return b200::launches_so_far(); }

int b200_embedding(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t B, int64_t L, int64_t V,
                   int64_t P, int64_t H, int dtype, int* bad_id_flag, void* stream) {
  if (B < 0 || L < 0 || V < 1 || P < 1 || H < 0 || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (L > P) return B200_ERR_BAD_ARGUMENT;
  if (B * L == 0 || H == 0) return B200_OK;
  if (!ids || !wte || !wpe || !out) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_embedding(ids, wte, wpe, out, B * L, L, V, P, H, dtype, bad_id_flag, nullptr, nullptr, 0.f, nullptr, (cudaStream_t)stream));
}

int b200_embedding_ln_stats(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t B, int64_t L, int64_t V,
                            int64_t P, int64_t H, int dtype, int* bad_id_flag, float eps, float* ln_stats_out, void* ln_ext_out, void* stream) {
  if (B < 0 || L < 0 || V < 1 || P < 1 || H < 0 || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (L > P) return B200_ERR_BAD_ARGUMENT;
  if (B * L == 0 || H == 0) return B200_OK;
  if (!ids || !wte || !wpe || !out || !ln_stats_out || (reinterpret_cast<uintptr_t>(ln_stats_out) & 7) || (reinterpret_cast<uintptr_t>(ln_ext_out) & 15))
    return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_embedding(ids, wte, wpe, out, B * L, L, V, P, H, dtype, bad_id_flag, ln_stats_out, ln_ext_out, eps, nullptr, (cudaStream_t)stream));
}

// ------------------------------------------------------------------ token-by-token generation
int b200_embedding_at(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t B, int64_t L, int64_t V, int64_t P, int64_t H,
                      int dtype, int* bad_id_flag, float eps, float* ln_stats_out, void* ln_ext_out, const int32_t* pos0_dev, void* stream) {
  if (B < 0 || L < 0 || V < 1 || P < 1 || H < 0 || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (L > P) return B200_ERR_BAD_ARGUMENT;
  if (B * L == 0 || H == 0) return B200_OK;
  if (!ids || !wte || !wpe || !out || !pos0_dev || (reinterpret_cast<uintptr_t>(pos0_dev) & 3) || (ln_ext_out && !ln_stats_out) ||
      (reinterpret_cast<uintptr_t>(ln_stats_out) & 7) || (reinterpret_cast<uintptr_t>(ln_ext_out) & 15))
    return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_embedding(ids, wte, wpe, out, B * L, L, V, P, H, dtype, bad_id_flag, ln_stats_out, ln_ext_out, eps, pos0_dev, (cudaStream_t)stream));
}

int b200_kv_cache_fill(const void* qkv, void* cache, int64_t B, int64_t L, int64_t H, int64_t cache_len, int dtype, void* stream) {
  if (B < 0 || L < 0 || H < 0 || cache_len < L || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (B == 0 || L == 0 || H == 0) return B200_OK;
  if (!qkv || !cache) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_kv_cache_fill(qkv, cache, B, L, H, cache_len, dtype, (cudaStream_t)stream));
}

int b200_attention_decode(const void* qkv_new, void* cache, void* out, int64_t B, int64_t NH, int64_t D, int64_t cache_len, float scale, int dtype,
                          const int32_t* pos_dev, int* status_word, void* stream) {
  if (B < 0 || NH < 0 || D < 1 || cache_len < 1 || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (D != 32 && D != 64 && D != 128) return B200_ERR_UNSUPPORTED;
  if (B == 0 || NH == 0) return B200_OK;
  if (!qkv_new || !cache || !out || !pos_dev || (reinterpret_cast<uintptr_t>(pos_dev) & 3)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_attention_decode(qkv_new, cache, out, B, NH, D, cache_len, scale, dtype, pos_dev, status_word, (cudaStream_t)stream));
}

int b200_decode_append(const int64_t* next_ids, int64_t* tokens, int64_t ld_tokens, int64_t n_cols, int64_t B, int32_t* pos_dev, int advance,
                       int64_t* feedback, int* status_word, void* stream) {
  if (B < 0 || n_cols < 1 || ld_tokens < n_cols) return B200_ERR_BAD_ARGUMENT;
  if (!next_ids || !tokens || !pos_dev || (reinterpret_cast<uintptr_t>(pos_dev) & 3)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_decode_append(next_ids, tokens, ld_tokens, n_cols, B, pos_dev, advance, feedback, status_word, (cudaStream_t)stream));
}

int b200_sample_logits(const void* logits, int64_t ld, int64_t B, int64_t V, int dtype, float temperature, int top_k, uint64_t seed,
                       const int32_t* step_dev, int64_t* ids_out, void* stream) {
  if (B < 0 || V < 1 || ld < V || !valid_dtype(dtype) || !(temperature > 0.f) || top_k < 0) return B200_ERR_BAD_ARGUMENT;
  if (B == 0) return B200_OK;
  if (!logits || !ids_out || (reinterpret_cast<uintptr_t>(step_dev) & 3)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_sample_rows(logits, ld, B, V, dtype, temperature, top_k, seed, step_dev, ids_out, (cudaStream_t)stream));
}

int b200_row_ln_stats(const void* x, float* ln_stats_out, void* ln_ext_out, int64_t M, int64_t H, float eps, int dtype, void* stream) {
  if (M < 0 || H < 0 || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (M == 0 || H == 0) return B200_OK;
  if (!x || !ln_stats_out || (reinterpret_cast<uintptr_t>(ln_stats_out) & 7) || (reinterpret_cast<uintptr_t>(ln_ext_out) & 15)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_row_ln_stats(x, ln_stats_out, ln_ext_out, M, H, eps, dtype, (cudaStream_t)stream));
}

int b200_fold_layernorm(const void* w, const void* gamma, const void* beta, const void* bias, void* packed, float* colsum, float* bias_out,
                        void* w_ext, int64_t K, int64_t N, int64_t ld_packed, int dtype, void* stream) {
  if (K < 0 || N < 0 || !valid_dtype(dtype)) return B200_ERR_BAD_ARGUMENT;
  if (dtype == B200_F32) return B200_ERR_UNSUPPORTED;
  if (K == 0 || N == 0) return B200_OK;
  if (!w || !gamma || !beta || !packed || !colsum || !bias_out || !w_ext || ld_packed < K || (reinterpret_cast<uintptr_t>(w_ext) & 15))
    return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_fold_layernorm(w, gamma, beta, bias, packed, colsum, bias_out, w_ext, K, N, ld_packed, dtype, (cudaStream_t)stream));
}

size_t b200_gemm_ln_workspace_bytes(int64_t M, int64_t N) { return b200::gemm_ln_workspace_bytes(M, N); }

int b200_gemm_ln(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                 int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype, int add_gelu, const float* ln_stats,
                 const void* ln_ext, const void* w_ext, float* ln_stats_out, void* ln_ext_out, float eps, void* workspace, size_t workspace_bytes,
                 int* status_word, void* stream) {
  if (!valid_dtype(io_dtype)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_gemm_ln(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, io_dtype, add_gelu, ln_stats, ln_ext,
                                   w_ext, ln_stats_out, ln_ext_out, eps, workspace, workspace_bytes, status_word, (cudaStream_t)stream));
}

int b200_layernorm(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t H, float eps,
                   int in_dtype, int out_dtype, void* stream) {
  if (M < 0 || H < 0 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype)) return B200_ERR_BAD_ARGUMENT;
  if (M == 0 || H == 0) return B200_OK;
  if (!x || !w || !b || !out) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_layernorm(x, w, b, out, M, H, eps, in_dtype, out_dtype, (cudaStream_t)stream));
}

int b200_pack_operand(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst,
                      int transpose, int src_dtype, int dst_dtype, void* stream) {
  if (rows < 0 || cols < 0 || !valid_dtype(src_dtype) || dst_dtype == B200_F32 || !valid_dtype(dst_dtype)) return B200_ERR_BAD_ARGUMENT;
  if (rows == 0 || cols == 0) return B200_OK;
  if (!src || !dst || ld_src < cols || ld_dst < (transpose ? rows : cols)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_pack(src, dst, rows, cols, ld_src, ld_dst, transpose, src_dtype, dst_dtype, (cudaStream_t)stream));
}

int b200_gemm(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
              int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
              int add_gelu, int* status_word, void* stream) {
  if (!valid_dtype(io_dtype)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_gemm(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, io_dtype, add_gelu,
                                status_word, (cudaStream_t)stream));
}

size_t b200_gemm_argmax_workspace_bytes(int64_t M, int64_t N) { return b200::gemm_argmax_workspace_bytes(M, N); }

int b200_gemm_argmax(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                     int add_gelu, int64_t* argmax_out, float* lse_out, void* workspace, size_t workspace_bytes, int* status_word,
                     void* stream) {
  if (!valid_dtype(io_dtype) || !argmax_out) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_gemm_argmax(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, io_dtype, add_gelu,
                                       argmax_out, lse_out, workspace, workspace_bytes, status_word, (cudaStream_t)stream));
}

int b200_gemm_rowstats(const void* a, const void* b, const void* bias, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                       int op_dtype, int round_dtype, const int64_t* targets, int64_t* argmax_out, float* lse_out,
                       float* target_logit_out, void* workspace, size_t workspace_bytes, int* status_word, void* stream) {
  if (!valid_dtype(round_dtype)) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_gemm_rowstats(a, b, bias, M, N, K, lda, ldb, op_dtype, round_dtype, targets, argmax_out, lse_out,
                                         target_logit_out, workspace, workspace_bytes, status_word, (cudaStream_t)stream));
}

size_t b200_ffn_workspace_bytes(int64_t M, int64_t N, int64_t K, int w_is_nk, int dtype) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent) return SIZE_MAX;  // b200_ffn rejects such a problem; no figure can be met
  const size_t kp = (size_t)((K + 7) / 8 * 8);
  size_t bytes = 0;
  if (!direct_operand_ok(dtype, K)) bytes += round256((size_t)M * kp * 2);
  if (!(w_is_nk && direct_operand_ok(dtype, K))) bytes += round256((size_t)N * kp * 2);
  return bytes;
}

int b200_ffn(const void* x, const void* w, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
             int64_t K, int64_t ld_out, int w_is_nk, int add_gelu, int dtype, void* workspace, size_t workspace_bytes,
             int* status_word, void* stream) {
  if (!valid_dtype(dtype) || M < 0 || N < 0 || K < 0) return B200_ERR_BAD_ARGUMENT;
  if (M == 0 || N == 0) return B200_OK;
  if (K == 0 || !x || !w || !out || ld_out < N) return B200_ERR_BAD_ARGUMENT;
  if (M > kMaxExtent || N > kMaxExtent || K > kMaxExtent) return B200_ERR_BAD_ARGUMENT;  // before any size arithmetic or packing launch
  cudaStream_t s = (cudaStream_t)stream;
  const int op_dtype = dtype == B200_BF16 ? B200_BF16 : B200_F16;
  const int64_t kp = (K + 7) / 8 * 8;
  const bool x_direct = direct_operand_ok(dtype, K) && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  const bool w_direct = w_is_nk && direct_operand_ok(dtype, K) && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
  size_t need = 0;
  if (!x_direct) need += round256((size_t)M * kp * 2);
  if (!w_direct) need += round256((size_t)N * kp * 2);
  if (need > 0 && (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))) return B200_ERR_WORKSPACE;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  const void* a = x;
  const void* b = w;
  int64_t lda = K, ldb = K;
  if (!x_direct) {
    int st = note(b200::launch_pack(x, ws, M, K, K, kp, 0, dtype, op_dtype, s));
    if (st != B200_OK) return st;
    a = ws;
    lda = kp;
    ws += round256((size_t)M * kp * 2);
  }
  if (!w_direct) {
    int st = w_is_nk ? note(b200::launch_pack(w, ws, N, K, K, kp, 0, dtype, op_dtype, s))
                     : note(b200::launch_pack(w, ws, K, N, N, kp, 1, dtype, op_dtype, s));
    if (st != B200_OK) return st;
    b = ws;
    ldb = kp;
  }
  return note(b200::launch_gemm(a, b, bias, residual, out, M, N, K, lda, ldb, N, ld_out, op_dtype, dtype, add_gelu, status_word, s));
}

int b200_attention(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L, int64_t D,
                   const int64_t q_strides[3], const int64_t k_strides[3], const int64_t v_strides[3],
                   const int64_t o_strides[3], float scale, int in_dtype, int out_dtype, int* status_word, void* stream) {
  if (B < 0 || NH < 0 || L < 0 || !valid_dtype(in_dtype) || !valid_dtype(out_dtype)) return B200_ERR_BAD_ARGUMENT;
  if (D != 16 && D != 32 && D != 64 && D != 128 && D != 256) return B200_ERR_BAD_ARGUMENT;
  if (B == 0 || NH == 0 || L == 0) return B200_OK;
  if (!q || !k || !v || !out || !q_strides || !k_strides || !v_strides || !o_strides) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_attention(q, k, v, out, B, NH, L, D, q_strides, k_strides, v_strides, o_strides, scale, in_dtype,
                                     out_dtype, status_word, (cudaStream_t)stream));
}

int b200_selftest_bounded_wait(int* status_word, int64_t limit_cycles, void* stream) {
  if (!status_word || limit_cycles < 1 || limit_cycles > 4000000000LL) return B200_ERR_BAD_ARGUMENT;
  return note(b200::launch_bounded_wait_selftest(status_word, limit_cycles, (cudaStream_t)stream));
}

}  // extern "C"
