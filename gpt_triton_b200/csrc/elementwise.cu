// HBM-bound kernels of the forward path: embedding gather, LayerNorm, operand packing.
// All three move each byte once: 128-bit loads/stores, one warp per row, statistics by
// warp shuffles, grid sized in multiples of the SM count.
#include <stdlib.h>

#include <atomic>

#include "common.cuh"

namespace b200 {

bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("B200GPT_PDL");
    return v && v[0] == '1';
  }();
  return on;
}

static std::atomic<uint64_t> g_launches{0};
void note_launches(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }
uint64_t launches_so_far() { return g_launches.load(std::memory_order_relaxed); }

int device_slot() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

static std::atomic<int> g_sm_count[kMaxDevices];
int sm_count() {
  const int slot = device_slot();
  if (slot < 0) return 148;
  int n = g_sm_count[slot].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, slot) != cudaSuccess || n <= 0) n = 148;
    g_sm_count[slot].store(n, std::memory_order_relaxed);
  }
  return n;
}

constexpr int kWarpsPerBlock = 8;

// ------------------------------------------------------------------ embedding
// One warp per token row.  VEC: rows are moved as 8-element vectors (needs H % 8 == 0 and
// 16-byte aligned tables); otherwise element by element.
// `stats` (optional): per row, the LayerNorm statistics (mean, 1 / sqrt(variance + eps)) of the stored row, and `ext`
// (optional, 16-bit T): the row's extension (common.cuh), the two things a GEMM with a folded LayerNorm takes for the
// rows of its input.
template <typename T, bool VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
embedding_kernel(const int64_t* __restrict__ ids, const T* __restrict__ wte, const T* __restrict__ wpe,
                 T* __restrict__ out, int64_t T_rows, int64_t L, int64_t V, int64_t H, int* bad_id_flag, float2* __restrict__ stats, T* __restrict__ ext,
                 float eps, const int* __restrict__ pos0_dev, int64_t P) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  pdl_launch_dependents();
  pdl_wait();
  // position of a sequence's first token: 0, or (token-by-token generation) read from device memory
  const int64_t pos0 = pos0_dev ? pos0_dev[0] : 0;
  for (int64_t t = warp0; t < T_rows; t += stride) {
    const int64_t id = ids[t];
    const int64_t pos = pos0 + t % L;
    const bool ok = id >= 0 && id < V && pos >= 0 && pos < P;  // (pos < P always holds when pos0 is 0: the host checked L <= P)
    if (!ok && lane == 0 && bad_id_flag) *bad_id_flag = 1;
    const T* e = wte + (ok ? id : 0) * H;
    const T* p = wpe + (ok ? pos : 0) * H;
    T* o = out + t * H;
    // sums of (value - shift) and its square over the values as stored; the shift (the row's first value) keeps the
    // centred sum of squares free of cancellation
    float shift = 0.f, s1 = 0.f, s2 = 0.f;
    if (stats) shift = ok ? to_float(from_float<T>(to_float(e[0]) + to_float(p[0]))) : 0.f;
    if (VEC) {
      for (int64_t c = (int64_t)lane * 8; c < H; c += 256) {
        float a[8], b[8];
        load8(e + c, a);
        load8(p + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = ok ? a[i] + b[i] : 0.f;
        store8(o + c, a);
        if (stats) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float d = to_float(from_float<T>(a[i])) - shift;
            s1 += d, s2 = fmaf(d, d, s2);
          }
        }
      }
    } else {
      for (int64_t c = lane; c < H; c += 32) {
        const T v = ok ? from_float<T>(to_float(e[c]) + to_float(p[c])) : from_float<T>(0.f);
        o[c] = v;
        const float d = to_float(v) - shift;
        s1 += d, s2 = fmaf(d, d, s2);
      }
    }
    if (stats) {
      s1 = warp_sum(s1), s2 = warp_sum(s2);
      const float m2 = fmaxf(s2 - s1 * s1 / (float)H, 0.f);
      const float mean = shift + s1 / (float)H, sd = sqrtf(m2 / (float)H + eps);
      if (lane == 0) stats[t] = make_float2(mean, 1.0f / sd);
      if constexpr (sizeof(T) == 2) {
        if (ext && lane < kLnExtCols * 2 / 16)
          reinterpret_cast<uint4*>(ext + t * kLnExtCols)[lane] = lane == 0 ? ln_ext_head<T>(mean, sd) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
  }
}

// (mean, rstd) of the rows of an existing [M, H] matrix: the entry into a chain of LayerNorm-folded GEMMs for rows that
// no kernel of this library produced.
template <typename T>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
row_ln_stats_kernel(const T* __restrict__ x, int64_t M, int64_t H, float eps, float2* __restrict__ stats, T* __restrict__ ext) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  const bool vec = (H % 8 == 0) && aligned16(x);
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t row = warp0; row < M; row += stride) {
    const T* xr = x + row * H;
    const float shift = to_float(xr[0]);
    float s1 = 0.f, s2 = 0.f;
    if (vec) {
      for (int64_t c = (int64_t)lane * 8; c < H; c += 256) {
        float a[8];
        load8(xr + c, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = a[i] - shift;
          s1 += d, s2 = fmaf(d, d, s2);
        }
      }
    } else {
      for (int64_t c = lane; c < H; c += 32) {
        const float d = to_float(xr[c]) - shift;
        s1 += d, s2 = fmaf(d, d, s2);
      }
    }
    s1 = warp_sum(s1), s2 = warp_sum(s2);
    const float m2 = fmaxf(s2 - s1 * s1 / (float)H, 0.f);
    const float mean = shift + s1 / (float)H, sd = sqrtf(m2 / (float)H + eps);
    if (lane == 0) stats[row] = make_float2(mean, 1.0f / sd);
    if constexpr (sizeof(T) == 2) {
      if (ext && lane < kLnExtCols * 2 / 16)
        reinterpret_cast<uint4*>(ext + row * kLnExtCols)[lane] = lane == 0 ? ln_ext_head<T>(mean, sd) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

static unsigned row_grid(int64_t rows) {
  int64_t blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (unsigned)blocks;
}

template <typename T>
static int embedding_typed(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t T_rows, int64_t L,
                           int64_t V, int64_t H, int* flag, float2* stats, void* ext, float eps, const int* pos0_dev, int64_t P, cudaStream_t stream) {
  const bool vec = (H % 8 == 0) && ((reinterpret_cast<uintptr_t>(wte) | reinterpret_cast<uintptr_t>(wpe) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  LaunchSetup ls(dim3(row_grid(T_rows)), dim3(kWarpsPerBlock * 32), 0, stream);
  const cudaError_t e = vec ? cudaLaunchKernelEx(&ls.cfg, embedding_kernel<T, true>, ids, (const T*)wte, (const T*)wpe, (T*)out, T_rows, L, V, H, flag, stats, (T*)ext, eps, pos0_dev, P)
                            : cudaLaunchKernelEx(&ls.cfg, embedding_kernel<T, false>, ids, (const T*)wte, (const T*)wpe, (T*)out, T_rows, L, V, H, flag, stats, (T*)ext, eps, pos0_dev, P);
  note_launches(1);
  return status_from_cuda(e);
}

int launch_embedding(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t T_rows, int64_t L,
                     int64_t V, int64_t P, int64_t H, int dtype, int* bad_id_flag, float* ln_stats, void* ln_ext, float eps, const int* pos0_dev,
                     cudaStream_t stream) {
  if (T_rows == 0 || H == 0) return B200_OK;
  if (ln_ext && (dtype == B200_F32 || !ln_stats)) return B200_ERR_UNSUPPORTED;
  float2* st = reinterpret_cast<float2*>(ln_stats);
  switch (dtype) {
    case B200_F32: return embedding_typed<float>(ids, wte, wpe, out, T_rows, L, V, H, bad_id_flag, st, nullptr, eps, pos0_dev, P, stream);
    case B200_F16: return embedding_typed<__half>(ids, wte, wpe, out, T_rows, L, V, H, bad_id_flag, st, ln_ext, eps, pos0_dev, P, stream);
    case B200_BF16: return embedding_typed<__nv_bfloat16>(ids, wte, wpe, out, T_rows, L, V, H, bad_id_flag, st, ln_ext, eps, pos0_dev, P, stream);
  }
  return B200_ERR_BAD_ARGUMENT;
}

int launch_row_ln_stats(const void* x, float* ln_stats, void* ln_ext, int64_t M, int64_t H, float eps, int dtype, cudaStream_t stream) {
  if (M == 0 || H == 0) return B200_OK;
  if (ln_ext && dtype == B200_F32) return B200_ERR_UNSUPPORTED;
  LaunchSetup ls(dim3(row_grid(M)), dim3(kWarpsPerBlock * 32), 0, stream);
  float2* st = reinterpret_cast<float2*>(ln_stats);
  cudaError_t e;
  switch (dtype) {
    case B200_F32: e = cudaLaunchKernelEx(&ls.cfg, row_ln_stats_kernel<float>, (const float*)x, M, H, eps, st, (float*)nullptr); break;
    case B200_F16: e = cudaLaunchKernelEx(&ls.cfg, row_ln_stats_kernel<__half>, (const __half*)x, M, H, eps, st, (__half*)ln_ext); break;
    case B200_BF16: e = cudaLaunchKernelEx(&ls.cfg, row_ln_stats_kernel<__nv_bfloat16>, (const __nv_bfloat16*)x, M, H, eps, st, (__nv_bfloat16*)ln_ext); break;
    default: return B200_ERR_BAD_ARGUMENT;
  }
  note_launches(1);
  return status_from_cuda(e);
}

// ------------------------------------------------------------------ LayerNorm
// Register-resident row: each lane holds NV vectors of 8 elements (row read from HBM once,
// written once).  Statistics in fp32: mean, then the centred sum of squares (two passes over
// registers, not over memory).
template <typename TI, typename TO, int NV>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layernorm_vec_kernel(const TI* __restrict__ x, const TI* __restrict__ w, const TI* __restrict__ b, TO* __restrict__ out,
                     int64_t M, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  const float inv_h = 1.0f / (float)H;
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t row = warp0; row < M; row += stride) {
    const TI* xr = x + row * (int64_t)H;
    float v[NV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
        load8(xr + c, v[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) s += v[i][j];
      }
    }
    const float mean = warp_sum(s) * inv_h;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          v[i][j] -= mean;
          q += v[i][j] * v[i][j];
        }
      }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(q) * inv_h + eps);
    TO* orow = out + row * (int64_t)H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = (i * 32 + lane) * 8;
      if (c < H) {
        float g[8], be[8];
        load8(w + c, g);
        load8(b + c, be);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[i][j] = (v[i][j] * rstd) * g[j] + be[j];
        store8(orow + c, v[i]);
      }
    }
  }
}

// Any H, any alignment: three passes over the row (it stays in L1 after the first).
template <typename TI, typename TO>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
layernorm_generic_kernel(const TI* __restrict__ x, const TI* __restrict__ w, const TI* __restrict__ b,
                         TO* __restrict__ out, int64_t M, int64_t H, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  const float inv_h = 1.0f / (float)H;
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t row = warp0; row < M; row += stride) {
    const TI* xr = x + row * H;
    float s = 0.f;
    for (int64_t c = lane; c < H; c += 32) s += to_float(xr[c]);
    const float mean = warp_sum(s) * inv_h;
    float q = 0.f;
    for (int64_t c = lane; c < H; c += 32) {
      const float d = to_float(xr[c]) - mean;
      q += d * d;
    }
    const float rstd = 1.0f / sqrtf(warp_sum(q) * inv_h + eps);
    TO* orow = out + row * H;
    for (int64_t c = lane; c < H; c += 32)
      orow[c] = from_float<TO>(((to_float(xr[c]) - mean) * rstd) * to_float(w[c]) + to_float(b[c]));
  }
}

template <typename TI, typename TO>
static int layernorm_typed(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t H, float eps,
                           cudaStream_t stream) {
  LaunchSetup ls(dim3(row_grid(M)), dim3(kWarpsPerBlock * 32), 0, stream);
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out);
  const bool vec = (H % 8 == 0) && (al & 15) == 0 && H <= 4096;
  const TI *xp = (const TI*)x, *wp = (const TI*)w, *bp = (const TI*)b;
  TO* op = (TO*)out;
  if (vec) {
    const int nv = (int)((H + 255) / 256);
#define B200_LN_CASE(NV)                                                                                                  \
  if (nv <= NV) {                                                                                                         \
    const cudaError_t e = cudaLaunchKernelEx(&ls.cfg, layernorm_vec_kernel<TI, TO, NV>, xp, wp, bp, op, M, (int)H, eps);  \
    note_launches(1);                                                                                                     \
    return status_from_cuda(e);                                                                                           \
  }
    B200_LN_CASE(1) B200_LN_CASE(2) B200_LN_CASE(3) B200_LN_CASE(4) B200_LN_CASE(7) B200_LN_CASE(8) B200_LN_CASE(16)
#undef B200_LN_CASE
  }
  const cudaError_t e = cudaLaunchKernelEx(&ls.cfg, layernorm_generic_kernel<TI, TO>, xp, wp, bp, op, M, H, eps);
  note_launches(1);
  return status_from_cuda(e);
}

int launch_layernorm(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t H, float eps,
                     int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || H == 0) return B200_OK;
  if (in_dtype == B200_F32 && out_dtype == B200_F32) return layernorm_typed<float, float>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_F32 && out_dtype == B200_F16) return layernorm_typed<float, __half>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_F16 && out_dtype == B200_F16) return layernorm_typed<__half, __half>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_F32 && out_dtype == B200_BF16) return layernorm_typed<float, __nv_bfloat16>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_BF16 && out_dtype == B200_BF16) return layernorm_typed<__nv_bfloat16, __nv_bfloat16>(x, w, b, out, M, H, eps, stream);
  return B200_ERR_UNSUPPORTED;  // valid dtype codes, but a pair that is not built (16-bit input with a different output type)
}

// ------------------------------------------------------------------ operand packing
// 32x32 tiles through shared memory; handles cast, optional transpose and zero padding of
// the destination's tail columns [width, ld_dst).
template <typename TS, typename TD, bool TRANSPOSE>
__global__ void __launch_bounds__(256)
pack_kernel(const TS* __restrict__ src, TD* __restrict__ dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  // destination is [drows, dcols_padded]
  const int64_t drows = TRANSPOSE ? cols : rows;
  const int64_t dwidth = TRANSPOSE ? rows : cols;
  const int64_t c0 = (int64_t)blockIdx.x * 32;  // destination column tile
  const int64_t r0 = (int64_t)blockIdx.y * 32;  // destination row tile
  if (TRANSPOSE) {
    // read src rows = destination columns, src cols = destination rows
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t sr = c0 + ty + i * 8, sc = r0 + tx;
      tile[ty + i * 8][tx] = (sr < rows && sc < cols) ? to_float(src[sr * ld_src + sc]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t dr = r0 + ty + i * 8, dc = c0 + tx;
      if (dr < drows && dc < ld_dst) dst[dr * ld_dst + dc] = from_float<TD>(dc < dwidth ? tile[tx][ty + i * 8] : 0.f);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t r = r0 + ty + i * 8, c = c0 + tx;
      if (r < drows && c < ld_dst) dst[r * ld_dst + c] = from_float<TD>(c < dwidth ? to_float(src[r * ld_src + c]) : 0.f);
    }
  }
}

template <typename TS, typename TD>
static int pack_typed(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst, int transpose,
                      cudaStream_t stream) {
  const int64_t drows = transpose ? cols : rows;
  dim3 grid((unsigned)((ld_dst + 31) / 32), (unsigned)((drows + 31) / 32));
  if (grid.y > 65535) {
    // very tall destinations: fold the row tiles into several launches
    const int64_t rows_per = 65535LL * 32;
    for (int64_t r = 0; r < drows; r += rows_per) {
      const int64_t n = (drows - r < rows_per) ? drows - r : rows_per;
      int st = transpose ? pack_typed<TS, TD>((const TS*)src + r, (TD*)dst + r * ld_dst, rows, n, ld_src, ld_dst, 1, stream)
                         : pack_typed<TS, TD>((const TS*)src + r * ld_src, (TD*)dst + r * ld_dst, n, cols, ld_src, ld_dst, 0, stream);
      if (st != B200_OK) return st;
    }
    return B200_OK;
  }
  if (transpose)
    pack_kernel<TS, TD, true><<<grid, 256, 0, stream>>>((const TS*)src, (TD*)dst, rows, cols, ld_src, ld_dst);
  else
    pack_kernel<TS, TD, false><<<grid, 256, 0, stream>>>((const TS*)src, (TD*)dst, rows, cols, ld_src, ld_dst);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

int launch_pack(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst, int transpose,
                int src_dtype, int dst_dtype, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return B200_OK;
  if (src_dtype == B200_F32 && dst_dtype == B200_F16) return pack_typed<float, __half>(src, dst, rows, cols, ld_src, ld_dst, transpose, stream);
  if (src_dtype == B200_F16 && dst_dtype == B200_F16) return pack_typed<__half, __half>(src, dst, rows, cols, ld_src, ld_dst, transpose, stream);
  if (src_dtype == B200_BF16 && dst_dtype == B200_BF16) return pack_typed<__nv_bfloat16, __nv_bfloat16>(src, dst, rows, cols, ld_src, ld_dst, transpose, stream);
  return B200_ERR_BAD_ARGUMENT;
}

// ------------------------------------------------------------------ LayerNorm folded into the next GEMM's weights
// LN(x) W + b = rstd * (x (g*W) - mean * colsum(g*W)) + (beta W + b) for a row x with LayerNorm weight g and bias
// beta: the weight-side quantities, computed once per weight version.
//   w [K, N] row-major (the state-dict layout), gamma/beta [K], bias [N] or NULL, all 16-bit T
//   packed [N, ld_dst] K-major = round_T(gamma[k] * w[k, n]), columns [K, ld_dst) zero
//   colsum[n] = sum_k packed[n, k] (over the rounded values the tensor cores will see), fp32
//   bias_out[n] = bias[n] + sum_k beta[k] * w[k, n], fp32
//   w_ext [N, kLnExtCols] = the weight extension built from those two (common.cuh)
// One block per 32 output columns; 32x32 tiles through shared memory for the transpose.
template <typename T>
__global__ void __launch_bounds__(256)
fold_layernorm_kernel(const T* __restrict__ w, const T* __restrict__ gamma, const T* __restrict__ beta, const T* __restrict__ bias,
                      T* __restrict__ packed, float* __restrict__ colsum, float* __restrict__ bias_out, T* __restrict__ w_ext, int64_t K, int64_t N,
                      int64_t ld_dst) {
  __shared__ float tile[32][33];
  __shared__ float red_c[8][32], red_b[8][32];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int64_t n0 = (int64_t)blockIdx.x * 32;
  float c_acc = 0.f, b_acc = 0.f;
  for (int64_t k0 = 0; k0 < ld_dst; k0 += 32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t k = k0 + ty + i * 8, n = n0 + tx;
      float pv = 0.f;
      if (k < K && n < N) {
        const float wv = to_float(w[k * N + n]);
        pv = to_float(from_float<T>(to_float(gamma[k]) * wv));
        c_acc += pv;
        b_acc = fmaf(to_float(beta[k]), wv, b_acc);
      }
      tile[ty + i * 8][tx] = pv;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int64_t n = n0 + ty + i * 8, k = k0 + tx;
      if (n < N && k < ld_dst) packed[n * ld_dst + k] = from_float<T>(tile[tx][ty + i * 8]);
    }
    __syncthreads();
  }
  red_c[ty][tx] = c_acc, red_b[ty][tx] = b_acc;
  __syncthreads();
  if (ty == 0 && n0 + tx < N) {
    float c = 0.f, b = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) c += red_c[i][tx], b += red_b[i][tx];
    b += bias ? to_float(bias[n0 + tx]) : 0.f;
    colsum[n0 + tx] = c;
    bias_out[n0 + tx] = b;
    uint4* dst = reinterpret_cast<uint4*>(w_ext + (n0 + tx) * kLnExtCols);
    dst[0] = ln_ext_weight_head<T>(c, b);
#pragma unroll
    for (int i = 1; i < kLnExtCols * 2 / 16; ++i) dst[i] = make_uint4(0u, 0u, 0u, 0u);
  }
}

int launch_fold_layernorm(const void* w, const void* gamma, const void* beta, const void* bias, void* packed, float* colsum, float* bias_out,
                          void* w_ext, int64_t K, int64_t N, int64_t ld_dst, int dtype, cudaStream_t stream) {
  if (K == 0 || N == 0) return B200_OK;
  const unsigned grid = (unsigned)((N + 31) / 32);
  if (dtype == B200_F16)
    fold_layernorm_kernel<__half><<<grid, 256, 0, stream>>>((const __half*)w, (const __half*)gamma, (const __half*)beta, (const __half*)bias,
                                                            (__half*)packed, colsum, bias_out, (__half*)w_ext, K, N, ld_dst);
  else if (dtype == B200_BF16)
    fold_layernorm_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16*)w, (const __nv_bfloat16*)gamma, (const __nv_bfloat16*)beta,
                                                                   (const __nv_bfloat16*)bias, (__nv_bfloat16*)packed, colsum, bias_out, (__nv_bfloat16*)w_ext, K, N,
                                                                   ld_dst);
  else
    return B200_ERR_UNSUPPORTED;
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

}  // namespace b200
