// HBM-bound kernels of the forward path: embedding gather, LayerNorm, operand packing.
// All three move each byte once: 128-bit loads/stores, one warp per row, statistics by
// warp shuffles, grid sized in multiples of the SM count.
#include <atomic>

#include "common.cuh"

namespace b200 {

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
template <typename T, bool VEC>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
embedding_kernel(const int64_t* __restrict__ ids, const T* __restrict__ wte, const T* __restrict__ wpe,
                 T* __restrict__ out, int64_t T_rows, int64_t L, int64_t V, int64_t H, int* bad_id_flag) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * kWarpsPerBlock;
  for (int64_t t = warp0; t < T_rows; t += stride) {
    const int64_t id = ids[t];
    const bool ok = id >= 0 && id < V;
    if (!ok && lane == 0 && bad_id_flag) *bad_id_flag = 1;
    const T* e = wte + (ok ? id : 0) * H;
    const T* p = wpe + (t % L) * H;
    T* o = out + t * H;
    if (VEC) {
      for (int64_t c = (int64_t)lane * 8; c < H; c += 256) {
        float a[8], b[8];
        load8(e + c, a);
        load8(p + c, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] = ok ? a[i] + b[i] : 0.f;
        store8(o + c, a);
      }
    } else {
      for (int64_t c = lane; c < H; c += 32) o[c] = ok ? from_float<T>(to_float(e[c]) + to_float(p[c])) : from_float<T>(0.f);
    }
  }
}

template <typename T>
static int embedding_typed(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t T_rows, int64_t L,
                           int64_t V, int64_t H, int* flag, cudaStream_t stream) {
  const bool vec = (H % 8 == 0) && ((reinterpret_cast<uintptr_t>(wte) | reinterpret_cast<uintptr_t>(wpe) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  int64_t blocks = (T_rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (vec)
    embedding_kernel<T, true><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, stream>>>(ids, (const T*)wte, (const T*)wpe, (T*)out, T_rows, L, V, H, flag);
  else
    embedding_kernel<T, false><<<(unsigned)blocks, kWarpsPerBlock * 32, 0, stream>>>(ids, (const T*)wte, (const T*)wpe, (T*)out, T_rows, L, V, H, flag);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

int launch_embedding(const int64_t* ids, const void* wte, const void* wpe, void* out, int64_t T_rows, int64_t L,
                     int64_t V, int64_t P, int64_t H, int dtype, int* bad_id_flag, cudaStream_t stream) {
  (void)P;
  if (T_rows == 0 || H == 0) return B200_OK;
  switch (dtype) {
    case B200_F32: return embedding_typed<float>(ids, wte, wpe, out, T_rows, L, V, H, bad_id_flag, stream);
    case B200_F16: return embedding_typed<__half>(ids, wte, wpe, out, T_rows, L, V, H, bad_id_flag, stream);
    case B200_BF16: return embedding_typed<__nv_bfloat16>(ids, wte, wpe, out, T_rows, L, V, H, bad_id_flag, stream);
  }
  return B200_ERR_BAD_ARGUMENT;
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
  int64_t blocks = (M + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  const unsigned g = (unsigned)blocks, t = kWarpsPerBlock * 32;
  const uintptr_t al = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(out);
  const bool vec = (H % 8 == 0) && (al & 15) == 0 && H <= 4096;
  const TI *xp = (const TI*)x, *wp = (const TI*)w, *bp = (const TI*)b;
  TO* op = (TO*)out;
  if (vec) {
    const int nv = (int)((H + 255) / 256);
#define B200_LN_CASE(NV)                                                                            \
  if (nv <= NV) {                                                                                   \
    layernorm_vec_kernel<TI, TO, NV><<<g, t, 0, stream>>>(xp, wp, bp, op, M, (int)H, eps);          \
    note_launches(1);                                                                               \
    return status_from_cuda(cudaGetLastError());                                                    \
  }
    B200_LN_CASE(1) B200_LN_CASE(2) B200_LN_CASE(3) B200_LN_CASE(4) B200_LN_CASE(7) B200_LN_CASE(8) B200_LN_CASE(16)
#undef B200_LN_CASE
  }
  layernorm_generic_kernel<TI, TO><<<g, t, 0, stream>>>(xp, wp, bp, op, M, H, eps);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

int launch_layernorm(const void* x, const void* w, const void* b, void* out, int64_t M, int64_t H, float eps,
                     int in_dtype, int out_dtype, cudaStream_t stream) {
  if (M == 0 || H == 0) return B200_OK;
  if (in_dtype == B200_F32 && out_dtype == B200_F32) return layernorm_typed<float, float>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_F32 && out_dtype == B200_F16) return layernorm_typed<float, __half>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_F16 && out_dtype == B200_F16) return layernorm_typed<__half, __half>(x, w, b, out, M, H, eps, stream);
  if (in_dtype == B200_BF16 && out_dtype == B200_BF16) return layernorm_typed<__nv_bfloat16, __nv_bfloat16>(x, w, b, out, M, H, eps, stream);
  return B200_ERR_BAD_ARGUMENT;
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

}  // namespace b200
