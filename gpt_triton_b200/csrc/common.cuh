// Shared definitions for the sm_100a kernels of the GPT-2 forward path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_gpt.h"

namespace b200 {

// ------------------------------------------------------------------ dtype helpers
template <typename T>
struct DType;
template <>
struct DType<float> {
  static constexpr int code = B200_F32;
};
template <>
struct DType<__half> {
  static constexpr int code = B200_F16;
};
template <>
struct DType<__nv_bfloat16> {
  static constexpr int code = B200_BF16;
};

__host__ __device__ inline int dtype_size(int dt) { return dt == B200_F32 ? 4 : 2; }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ __half from_float<__half>(float v) {
  return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// 8 consecutive elements <-> 8 floats.  The vector forms need 16-byte alignment.
template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&f)[8]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  float4 b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(h[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x, f[2 * i + 1] = t.y;
  }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float (&f)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&f)[8]) {
  uint4 u;
  __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ LayerNorm folded into a GEMM: the extension k-block
// A GEMM that consumes raw rows x with their LayerNorm folded in (rstd * (x W' - mean * colsum(W')) + bias') lets the
// tensor cores add the two rank-one terms: one extra 64-wide k-block whose A side ("row extension", one per row of
// x) and B side ("weight extension", one per output column) are laid out so that their dot product is
//     -mean * colsum + (1 / rstd) * bias',
// each factor split into a high and a low 16-bit part (v = hi + lo to twice the type's precision) and the four cross
// products spelled out:
//     row extension    [-mean_hi, -mean_lo, -mean_hi, -mean_lo,  sd_hi, sd_lo, sd_hi, sd_lo, 0 ...]     sd = 1 / rstd
//     weight extension [  cs_hi,    cs_hi,    cs_lo,    cs_lo,   b_hi,  b_hi,  b_lo,  b_lo,  0 ...]
constexpr int kLnExtCols = 64;

template <typename T>
__device__ __forceinline__ void split_hi_lo(float v, T& hi, T& lo) {
  hi = from_float<T>(v);
  lo = from_float<T>(v - to_float(hi));
}
template <typename T>
__device__ __forceinline__ uint32_t pack_pair(T a, T b) {
  return (uint32_t)(*reinterpret_cast<const uint16_t*>(&a)) | ((uint32_t)(*reinterpret_cast<const uint16_t*>(&b)) << 16);
}
// First 8 elements (16 bytes) of a row extension; the other 56 elements are zero.
template <typename T>
__device__ __forceinline__ uint4 ln_ext_head(float mean, float sd) {
  T mh, ml, sh, sl;
  split_hi_lo<T>(-mean, mh, ml);
  split_hi_lo<T>(sd, sh, sl);
  return make_uint4(pack_pair(mh, ml), pack_pair(mh, ml), pack_pair(sh, sl), pack_pair(sh, sl));
}
// First 8 elements of a weight extension.
template <typename T>
__device__ __forceinline__ uint4 ln_ext_weight_head(float colsum, float bias) {
  T ch, cl, bh, bl;
  split_hi_lo<T>(colsum, ch, cl);
  split_hi_lo<T>(bias, bh, bl);
  return make_uint4(pack_pair(ch, ch), pack_pair(cl, cl), pack_pair(bh, bh), pack_pair(bl, bl));
}

// tanh-form GELU with tanh(y) = 2*sigmoid(2y) - 1, the formulation the reference
// kernel evaluates (kernels.py:15-26 of the reference project).
__device__ __forceinline__ float gelu_new(float x) {
  const float a = 0.7978845608028654f;  // sqrt(2/pi)
  float b = x + 0.044715f * x * x * x;
  float y = a * b;
  float s = 1.0f / (1.0f + __expf(-2.0f * y));
  float t = 2.0f * s - 1.0f;
  return 0.5f * x * (1.0f + t);
}

// ------------------------------------------------------------------ programmatic dependent launch
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in the
// stream is still running.  pdl_wait() blocks until the predecessor grid has completed and its memory is visible, so
// what a kernel does before it (barrier set-up, tensor-memory allocation) overlaps the predecessor's tail;
// pdl_launch_dependents() lets the successor's CTAs be scheduled as soon as SM resources free up.  Both are no-ops in a
// kernel launched without the attribute.  Every CTA of every kernel that is launched with the attribute calls
// pdl_wait() before its first access to global memory, on every path, so that "my predecessor has completed" stays
// transitive along the stream (kernels launched without it are serialised by the stream as usual).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ------------------------------------------------------------------ launch helpers
inline int status_from_cuda(cudaError_t e) { return e == cudaSuccess ? B200_OK : B200_ERR_CUDA; }

// Whether kernels are launched with the programmatic-stream-serialization attribute: only when the environment
// variable B200GPT_PDL=1 (read once) asks for it.  Off by default because it measured slower: in a replayed CUDA graph
// the kernels of the forward already follow each other within 0.3 us, and letting the next kernel's CTAs take their
// SMs early cost 2 % at 512 x 300 tokens and 3 % at 64 x 300.
bool pdl_enabled();

// cudaLaunchConfig_t with room for the two attributes this library uses: cluster size and programmatic serialization.
struct LaunchSetup {
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attrs[2];
  LaunchSetup(dim3 grid, dim3 block, size_t smem_bytes, cudaStream_t stream, int cluster_x = 1, bool allow_pdl = true) {
    cfg = cudaLaunchConfig_t{};
    cfg.gridDim = grid, cfg.blockDim = block, cfg.dynamicSmemBytes = smem_bytes, cfg.stream = stream;
    unsigned n = 0;
    if (cluster_x > 1) {
      attrs[n].id = cudaLaunchAttributeClusterDimension;
      attrs[n].val.clusterDim.x = (unsigned)cluster_x, attrs[n].val.clusterDim.y = 1, attrs[n].val.clusterDim.z = 1;
      ++n;
    }
    if (allow_pdl && pdl_enabled()) {
      attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attrs[n].val.programmaticStreamSerializationAllowed = 1;
      ++n;
    }
    cfg.attrs = attrs, cfg.numAttrs = n;
  }
};

int sm_count();  // cached multiprocessor count of the current device
// Index of the current device for per-device caches (kernel attributes, occupancy figures); -1 if it cannot be had.
constexpr int kMaxDevices = 64;
int device_slot();
void note_launches(int n);  // adds to the library-wide count of kernels launched
uint64_t launches_so_far();

// ------------------------------------------------------------------ internal launchers
// ln_stats (optional, fp32 pairs [T]): (mean, 1 / sqrt(variance + eps)) of every stored row; ln_ext (with it): the
// rows' extensions [T, kLnExtCols] in the storage type (16-bit types only)
// pos0_dev (optional, device int32): position of each sequence's first token (token-by-token generation); NULL = 0
int launch_embedding(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t T, int64_t L, int64_t V,
                     int64_t P, int64_t H, int dtype, int* bad_id_flag, float* ln_stats, void* ln_ext, float eps, const int* pos0_dev,
                     cudaStream_t stream);
// Token-by-token generation (decode.cu).  pos_dev: device int32 pair {tokens in the cache, prompt length}.
int launch_kv_cache_fill(const void* qkv, void* cache, int64_t B, int64_t L, int64_t H, int64_t cache_len, int dtype, cudaStream_t stream);
int launch_attention_decode(const void* qkv_new, void* cache, void* out, int64_t B, int64_t NH, int64_t D, int64_t cache_len, float scale, int dtype,
                            const int* pos_dev, int* status_word, cudaStream_t stream);
int launch_decode_append(const int64_t* next_ids, int64_t* tokens, int64_t ld_tokens, int64_t n_cols, int64_t B, int* pos_dev, int advance,
                         int64_t* feedback, int* status_word, cudaStream_t stream);
int launch_sample_rows(const void* logits, int64_t ld, int64_t B, int64_t V, int dtype, float temperature, int top_k, uint64_t seed,
                       const int* step_dev, int64_t* ids_out, cudaStream_t stream);
int launch_row_ln_stats(const void* x, float* ln_stats, void* ln_ext, int64_t M, int64_t H, float eps, int dtype, cudaStream_t stream);
int launch_fold_layernorm(const void* w, const void* gamma, const void* beta, const void* bias, void* packed, float* colsum, float* bias_out,
                          void* w_ext, int64_t K, int64_t N, int64_t ld_dst, int dtype, cudaStream_t stream);
size_t gemm_ln_workspace_bytes(int64_t M, int64_t N);
int launch_gemm_ln(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                   int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype, int add_gelu, const float* ln_stats,
                   const void* a_ext, const void* b_ext, float* stats_out, void* ext_out, float eps, void* workspace, size_t workspace_bytes,
                   int* status_word, cudaStream_t stream);
int launch_layernorm(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t H, float eps,
                     int in_dtype, int out_dtype, cudaStream_t stream);
int launch_pack(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst, int transpose,
                int src_dtype, int dst_dtype, cudaStream_t stream);
int launch_gemm(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                int add_gelu, int* status_word, cudaStream_t stream);
// launch_gemm that also writes argmax_out[row] = column of the row's maximum over the (rounded) output, lowest column
// on ties, and, if lse_out is not NULL, lse_out[row] = log(sum_j exp(out[row, j])).  workspace:
// gemm_argmax_workspace_bytes(M, N) bytes, 16-byte aligned.  argmax_out == NULL: plain GEMM.
size_t gemm_argmax_workspace_bytes(int64_t M, int64_t N);
int launch_gemm_argmax(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                       int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                       int add_gelu, int64_t* argmax_out, float* lse_out, void* workspace, size_t workspace_bytes, int* status_word,
                       cudaStream_t stream);
int launch_gemm_rowstats(const void* a, const void* b, const void* bias, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int op_dtype, int round_dtype, const int64_t* targets, int64_t* argmax_out, float* lse_out, float* target_out,
                         void* workspace, size_t workspace_bytes, int* status_word, cudaStream_t stream);
int launch_attention(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L,
                     int64_t D, const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                     const int64_t* o_strides, float scale, int in_dtype, int out_dtype, int* status_word, cudaStream_t stream);

// One warp waiting (bounded) on a barrier that nothing completes: reports B200_ERR_DEVICE_WAIT through status_word.
int launch_bounded_wait_selftest(int* status_word, int64_t limit_cycles, cudaStream_t stream);
// tcgen05/TMA attention (head size 64, fp16); B200_ERR_UNSUPPORTED means "use the generic kernel".
int launch_attention_sm100(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L, int64_t D,
                           const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides, const int64_t* o_strides,
                           float scale, int in_dtype, int out_dtype, int* status_word, cudaStream_t stream);

}  // namespace b200
