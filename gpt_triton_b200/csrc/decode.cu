// Token-by-token generation on top of the forward path: key/value cache, one-query attention, sampling.
// The reference project lists "KV cache + sampling" among the things it never built (README.md:55), so nothing
// here has a counterpart there; the arithmetic follows the reference's flash_attention_v1 (kernels.py:417-474:
// 64-key blocks, fp16 dot operands, fp32 running maximum and denominator, P rounded to fp16 relative to the
// running maximum of its block), so that a cached step gives what re-running the whole sequence would.
//
// Everything that changes from one generated token to the next is read from DEVICE memory (the int32 pair
// `pos` = {tokens in the cache, prompt length}), so that the kernels of a decode step can be recorded once in a
// CUDA graph and replayed for every step.  All of these kernels are HBM-bound gathers and streams:
//   kv_cache_fill_kernel      cache[b, l, 0:2H] = qkv[b, l, H:3H] after the prompt's forward   (2 x B L 2H bytes)
//   attention_decode_kernel   appends the new token's k, v and attends its q over the cache    (B (pos+1) 2H elements read)
//   sample_rows_kernel        top-k filter + Gumbel-max draw over a row of logits              (passes over B V logits, mostly L2)
//   decode_append_kernel      tokens[b, column] = next id (also into the buffer the next step embeds); pos += 1
#include "common.cuh"

namespace b200 {
namespace {

// codes left in the status word (site numbers above those of the tensor-core kernels)
constexpr int kSiteCachePosition = 41;  // the cache has no room for the position being written
constexpr int kSiteTokenColumn = 42;    // the token buffer has no column for the id being appended

// ------------------------------------------------------------------ prompt -> cache
// One warp per (batch, position) row: 2H elements as 16-byte vectors.
__global__ void __launch_bounds__(256)
kv_cache_fill_kernel(const uint4* __restrict__ qkv, uint4* __restrict__ cache, int64_t rows, int64_t L, int64_t cache_len, int vec_per_h) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * 8;
  for (int64_t t = warp0; t < rows; t += stride) {
    const int64_t b = t / L, l = t % L;
    const uint4* src = qkv + (t * 3 + 1) * vec_per_h;
    uint4* dst = cache + (b * cache_len + l) * 2 * vec_per_h;
    for (int c = lane; c < 2 * vec_per_h; c += 32) dst[c] = src[c];
  }
}

// ------------------------------------------------------------------ one-query attention over the cache
// The value a dot product sees: fp32 storage is rounded to fp16 first (kernels.py:229, 234 of the reference cast every
// dot operand to fp16); 16-bit storage is used as it is.
template <typename T>
__device__ __forceinline__ float dot_operand(float v) {
  return v;
}
template <>
__device__ __forceinline__ float dot_operand<float>(float v) {
  return __half2float(__float2half_rn(v));
}
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// N consecutive elements moved as one access (N * sizeof(T) is 2, 4, 8 or 16 bytes; the address is aligned to it)
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// qkv_new [B, 3H] holds the new token's q | k | v; cache [B, cache_len, 2H] holds k | v of the earlier positions.
// The pos + 1 keys are walked in the reference's blocks of 64 (kernels.py:509).  A PAIR of lanes owns a key: lane
// 2i takes the first D/2 elements of the key and value rows of keys i, i + 16, i + 32, i + 48 of the block, lane
// 2i + 1 the second D/2, read as 16-byte vectors, so one warp-wide load covers whole 32-byte sectors of 16 rows;
// the two halves of a dot product meet in one shuffle.  All loads of a block are independent of each other, so many
// are in flight per lane.  The softmax reference point of a block is the running maximum over the blocks up
// to and including it, exactly as in the reference's loop (kernels.py:440-468): P = exp(s - that maximum) is
// rounded to fp16 before it multiplies V, the denominator sums the unrounded P.  Every lane keeps a private D/2-wide
// piece of the output row in registers (the rescale factor of a block is the same for all lanes); at the end the
// 16 pieces of each half are added by a halving exchange (D/2 -> D/32 values per lane in four shuffle rounds) that
// leaves lane l with output columns (l & 1) * D/2 + (l >> 1) * D/32 + [0, D/32).
// SPLIT = 1: one warp per (batch, head), four per block, no block-level synchronisation.  SPLIT = 4 (few sequences:
// not enough warps to fill the GPU): the four warps of a block share one (batch, head) and take the 64-key blocks
// 4g .. 4g + 3 of a group g side by side; the block maxima of a group go through shared memory (one block-level
// barrier per group), so that warp w still uses the running maximum over blocks 0 .. 4g + w; the warps' partial
// rows are merged through shared memory at the end.
template <typename T, int D, int SPLIT>
__global__ void __launch_bounds__(128)  // (76 registers at D = 64, six blocks per SM; capping at 64 registers for eight measured 16 % slower)
attention_decode_kernel(const T* __restrict__ qkv_new, T* __restrict__ cache, T* __restrict__ out, int64_t BH, int NH, int64_t cache_len,
                        float scale_log2e, const int* __restrict__ pos_dev, int* status_word) {
  __shared__ __align__(16) float q_s[4][D + 4];  // the second half of q sits 4 floats further on: the two lanes of a pair read different banks
  __shared__ float part_o[4][D];
  __shared__ float part_ml[4][2];
  __shared__ float group_max[2][4];
  constexpr int DPL = D / 32;  // output columns per lane
  constexpr int DH = D / 2;    // elements of a row per lane of a pair
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int side = lane & 1, kl = lane >> 1;  // which half of the rows; which of the 16 key slots
  const int64_t w = SPLIT == 1 ? (int64_t)blockIdx.x * 4 + warp : (int64_t)blockIdx.x;
  const int part = SPLIT == 1 ? 0 : warp;
  const int pos = pos_dev[0];
  if (pos < 0 || pos >= cache_len) {
    if (threadIdx.x == 0 && status_word) atomicCAS(status_word, 0, kSiteCachePosition);
    return;
  }
  if (w >= BH) return;  // (SPLIT = 4: the whole block leaves together)
  const int64_t b = w / NH;
  const int h = (int)(w % NH);
  const int64_t H = (int64_t)NH * D, pitch = 2 * H;
  const T* qn = qkv_new + b * 3 * H + (int64_t)h * D;
  const T* kn = qn + H;
  const T* vn = kn + H;
  T* kc = cache + b * cache_len * pitch + (int64_t)h * D;
  T* vc = kc + H;
  for (int i = lane; i < D; i += 32) {
    q_s[warp][i + (i >= D / 2 ? 4 : 0)] = dot_operand<T>(to_float(qn[i]));
    if (part == 0) {
      kc[(int64_t)pos * pitch + i] = kn[i];
      vc[(int64_t)pos * pitch + i] = vn[i];
    }
  }
  __syncwarp();
  // (the new token's own key and value are read from qkv_new below, not back from the cache)
  const int n_keys = pos + 1;
  const int n_groups = (n_keys + 64 * SPLIT - 1) / (64 * SPLIT);
  float m_run = -INFINITY;  // reference maximum of this warp's latest block
  float m_all = -INFINITY;  // running maximum over all blocks of the groups done so far
  float l_lane = 0.f;
  float o[DH];
#pragma unroll
  for (int d = 0; d < DH; ++d) o[d] = 0.f;
  const float* q_mine = q_s[warp] + side * (DH + 4);
  for (int g = 0; g < n_groups; ++g) {
    const int k0 = (g * SPLIT + part) * 64;
    float s[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int key = k0 + j * 16 + kl;
      float a = 0.f;
      if (key < n_keys) {
        const T* kr = (key == pos ? kn : kc + (int64_t)key * pitch) + side * DH;
#pragma unroll
        for (int c = 0; c < DH; c += 8) {
          float f[8];
          load8(kr + c, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) a = fmaf(q_mine[c + i], dot_operand<T>(f[i]), a);
        }
      }
      a += __shfl_xor_sync(0xffffffffu, a, 1);                      // the other half of the dot product
      s[j] = key < n_keys ? a * scale_log2e : -INFINITY;            // score in log2 units
    }
    const float bm = warp_max(fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3])));
    float m_new = fmaxf(m_all, bm);
    if (SPLIT > 1) {
      if (lane == 0) group_max[g & 1][warp] = bm;
      __syncthreads();
#pragma unroll
      for (int p2 = 0; p2 < SPLIT; ++p2) {
        const float other = group_max[g & 1][p2];
        if (p2 < part) m_new = fmaxf(m_new, other);
        m_all = fmaxf(m_all, other);
      }
    } else {
      m_all = m_new;
    }
    if (bm == -INFINITY) continue;  // no key of this block exists (warp-uniform; SPLIT = 4 only)
    const float mult = ex2_ftz(m_run - m_new);  // 0 for the warp's first block
    m_run = m_new;
    float ph[4], psum = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float pj = ex2_ftz(s[j] - m_new);  // 0 for keys beyond the last
      psum += pj;
      ph[j] = __half2float(__float2half_rn(pj));
    }
    l_lane = fmaf(l_lane, mult, side == 0 ? psum : 0.f);  // (both lanes of a pair hold the same scores: count them once)
#pragma unroll
    for (int d = 0; d < DH; ++d) o[d] *= mult;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int key = k0 + j * 16 + kl;
      if (key < n_keys) {
        const T* vr = (key == pos ? vn : vc + (int64_t)key * pitch) + side * DH;
#pragma unroll
        for (int c = 0; c < DH; c += 8) {
          float f[8];
          load8(vr + c, f);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[c + i] = fmaf(ph[j], dot_operand<T>(f[i]), o[c + i]);
        }
      }
    }
  }
  // add up the lanes' pieces and denominators (all relative to the same maximum m_run)
  float l_warp = warp_sum(l_lane);
#pragma unroll
  for (int n = DH / 2, off = 16; off > 1; n >>= 1, off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const float mine = upper ? o[i + n] : o[i];
      const float theirs = upper ? o[i] : o[i + n];
      o[i] = mine + __shfl_xor_sync(0xffffffffu, theirs, off);
    }
  }
  const int col0 = side * DH + kl * DPL;  // first of this lane's DPL output columns
  // o[0 .. DPL) now holds output columns col0 + j of this warp's blocks
  if (SPLIT > 1) {
#pragma unroll
    for (int j = 0; j < DPL; ++j) part_o[warp][col0 + j] = o[j];
    if (lane == 0) part_ml[warp][0] = m_run, part_ml[warp][1] = l_warp;
    __syncthreads();
    if (warp != 0) return;
    l_warp = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) o[j] = 0.f;
#pragma unroll
    for (int p2 = 0; p2 < SPLIT; ++p2) {
      const float mp = part_ml[p2][0];
      const float f = mp == -INFINITY ? 0.f : ex2_ftz(mp - m_all);  // (m_all is the maximum over every block by now)
      l_warp = fmaf(part_ml[p2][1], f, l_warp);
#pragma unroll
      for (int j = 0; j < DPL; ++j) o[j] = fmaf(part_o[p2][col0 + j], f, o[j]);
    }
  }
  const float inv = 1.0f / l_warp;
  Vec<T, DPL> res;
#pragma unroll
  for (int d = 0; d < DPL; ++d) res.v[d] = from_float<T>(o[d] * inv);
  *reinterpret_cast<Vec<T, DPL>*>(out + b * H + (int64_t)h * D + col0) = res;
}

template <typename T, int D>
int attention_decode_sized(const void* qkv_new, void* cache, void* out, int64_t BH, int64_t NH, int64_t cache_len, float sl, const int* pos_dev,
                           int* status_word, cudaStream_t stream) {
  // one warp per (batch, head) fills the GPU from about 16 warps per SM on; below that, four warps share one
  if (BH >= (int64_t)sm_count() * 16)
    attention_decode_kernel<T, D, 1><<<(unsigned)((BH + 3) / 4), 128, 0, stream>>>((const T*)qkv_new, (T*)cache, (T*)out, BH, (int)NH, cache_len, sl,
                                                                                    pos_dev, status_word);
  else
    attention_decode_kernel<T, D, 4><<<(unsigned)BH, 128, 0, stream>>>((const T*)qkv_new, (T*)cache, (T*)out, BH, (int)NH, cache_len, sl, pos_dev,
                                                                       status_word);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

template <typename T>
int attention_decode_typed(const void* qkv_new, void* cache, void* out, int64_t B, int64_t NH, int64_t D, int64_t cache_len, float scale,
                           const int* pos_dev, int* status_word, cudaStream_t stream) {
  const float sl = scale * 1.4426950408889634f;
  if (D == 32) return attention_decode_sized<T, 32>(qkv_new, cache, out, B * NH, NH, cache_len, sl, pos_dev, status_word, stream);
  if (D == 64) return attention_decode_sized<T, 64>(qkv_new, cache, out, B * NH, NH, cache_len, sl, pos_dev, status_word, stream);
  if (D == 128) return attention_decode_sized<T, 128>(qkv_new, cache, out, B * NH, NH, cache_len, sl, pos_dev, status_word, stream);
  return B200_ERR_UNSUPPORTED;
}

// ------------------------------------------------------------------ append + advance
// One block: every thread reads the position before thread 0 moves it.
__global__ void __launch_bounds__(256)
decode_append_kernel(const int64_t* __restrict__ next_ids, int64_t* __restrict__ tokens, int64_t ld_tokens, int64_t n_cols, int64_t B, int* pos_dev,
                     int advance, int64_t* __restrict__ feedback, int* status_word) {
  const int64_t col = (int64_t)pos_dev[0] - pos_dev[1] + (advance ? 1 : 0);
  __syncthreads();
  if (col < 0 || col >= n_cols) {
    if (threadIdx.x == 0 && status_word) atomicCAS(status_word, 0, kSiteTokenColumn);
    return;
  }
  for (int64_t b = threadIdx.x; b < B; b += blockDim.x) {
    const int64_t id = next_ids[b];
    tokens[b * ld_tokens + col] = id;
    if (feedback) feedback[b] = id;  // what the next decode step embeds
  }
  if (advance && threadIdx.x == 0) pos_dev[0] += 1;
}

// ------------------------------------------------------------------ sampling
// Counter-based uniform numbers: the 64-bit finaliser of SplitMix64 (Steele, Lea, Flood 2014) applied to
// seed + golden ratio * (step + 1) and then, xored with (row, column), once more; 23 random bits -> u = (n + 1/2) / 2^23 in (0, 1), exact in fp32.
__host__ __device__ inline uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t stream_key, uint32_t row, uint32_t col) {
  const uint64_t x = mix64(stream_key ^ (((uint64_t)row << 32) | col));
  return ((float)(uint32_t)(x >> 41) + 0.5f) * (1.0f / 8388608.0f);
}
// Unsigned key with the order of the floats (larger float <-> larger key).
__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int kSampleThreads = 512;

// One block per row.  top_k > 0: four 8-bit radix passes find the key of the top_k-th largest logit; every logit at
// or above it stays in (ties at the threshold all stay, as with the usual `logits < kth_value -> -inf` filter).
// Then Gumbel-max: id = argmax_j (logit_j / temperature - log(-log(u_j))), lowest j on ties, which draws from
// softmax(logits / temperature) over the kept columns.
template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const T* __restrict__ logits, int64_t ld, int V, float inv_temperature, int top_k, uint64_t seed, const int* __restrict__ step_dev,
                   int64_t* __restrict__ ids_out) {
  __shared__ int hist[256];
  __shared__ int sel_bin, sel_want;
  __shared__ float red_val[kSampleThreads / 32];
  __shared__ int red_idx[kSampleThreads / 32];
  const int row = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + (int64_t)row * ld;
  uint32_t thr_key = 0;
  if (top_k > 0 && top_k < V) {
    uint32_t prefix = 0, mask = 0;
    int want = top_k;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (int i = tid; i < V; i += kSampleThreads) {
        const uint32_t key = order_key(to_float(x[i]));
        if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, bin = 255;
        for (; bin > 0; --bin) {
          if (cum + hist[bin] >= want) break;
          cum += hist[bin];
        }
        sel_bin = bin, sel_want = want - cum;
      }
      __syncthreads();
      prefix |= (uint32_t)sel_bin << shift;
      mask |= 255u << shift;
      want = sel_want;
      __syncthreads();
    }
    thr_key = prefix;
  }
  const uint64_t stream_key = mix64(seed + 0x9E3779B97F4A7C15ull * ((uint64_t)(uint32_t)(step_dev ? step_dev[0] : 0) + 1));
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < V; i += kSampleThreads) {
    const float f = to_float(x[i]);
    if (!(f == f) || order_key(f) < thr_key) continue;  // NaN or filtered out
    const float g = -logf(-logf(uniform01(stream_key, (uint32_t)row, (uint32_t)i)));
    const float sc = fmaf(f, inv_temperature, g);
    if (sc > best) best = sc, best_i = i;  // ascending i within a thread: the first maximum stays
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
  }
  if ((tid & 31) == 0) red_val[tid >> 5] = best, red_idx[tid >> 5] = best_i;
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < kSampleThreads / 32; ++w)
      if (red_val[w] > best || (red_val[w] == best && red_idx[w] < best_i)) best = red_val[w], best_i = red_idx[w];
    ids_out[row] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

}  // namespace

int launch_kv_cache_fill(const void* qkv, void* cache, int64_t B, int64_t L, int64_t H, int64_t cache_len, int dtype, cudaStream_t stream) {
  if (B == 0 || L == 0 || H == 0) return B200_OK;
  const int64_t row_bytes = H * dtype_size(dtype);
  if (row_bytes % 16 || ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(cache)) & 15)) return B200_ERR_ALIGNMENT;
  if (L > cache_len || row_bytes / 16 > 0x3fffffff) return B200_ERR_BAD_ARGUMENT;
  const int64_t rows = B * L;
  int64_t blocks = (rows + 7) / 8;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  kv_cache_fill_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const uint4*)qkv, (uint4*)cache, rows, L, cache_len, (int)(row_bytes / 16));
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

int launch_attention_decode(const void* qkv_new, void* cache, void* out, int64_t B, int64_t NH, int64_t D, int64_t cache_len, float scale, int dtype,
                            const int* pos_dev, int* status_word, cudaStream_t stream) {
  if (B == 0 || NH == 0) return B200_OK;
  // half key rows are read as 16-byte vectors
  if (((reinterpret_cast<uintptr_t>(qkv_new) | reinterpret_cast<uintptr_t>(cache)) & 15) || (D / 2 * dtype_size(dtype)) % 16) return B200_ERR_ALIGNMENT;
  if (B * NH > 0x7fffffffLL * 4 || NH > 0x7fffffff) return B200_ERR_BAD_ARGUMENT;
  switch (dtype) {
    case B200_F32: return attention_decode_typed<float>(qkv_new, cache, out, B, NH, D, cache_len, scale, pos_dev, status_word, stream);
    case B200_F16: return attention_decode_typed<__half>(qkv_new, cache, out, B, NH, D, cache_len, scale, pos_dev, status_word, stream);
    case B200_BF16: return attention_decode_typed<__nv_bfloat16>(qkv_new, cache, out, B, NH, D, cache_len, scale, pos_dev, status_word, stream);
  }
  return B200_ERR_BAD_ARGUMENT;
}

int launch_decode_append(const int64_t* next_ids, int64_t* tokens, int64_t ld_tokens, int64_t n_cols, int64_t B, int* pos_dev, int advance,
                         int64_t* feedback, int* status_word, cudaStream_t stream) {
  decode_append_kernel<<<1, 256, 0, stream>>>(next_ids, tokens, ld_tokens, n_cols, B, pos_dev, advance, feedback, status_word);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

int launch_sample_rows(const void* logits, int64_t ld, int64_t B, int64_t V, int dtype, float temperature, int top_k, uint64_t seed,
                       const int* step_dev, int64_t* ids_out, cudaStream_t stream) {
  if (B == 0) return B200_OK;
  if (V <= 0 || V > 0x7fffffff || B > 0x7fffffff || !(temperature > 0.f) || top_k < 0) return B200_ERR_BAD_ARGUMENT;
  const float inv_t = 1.0f / temperature;
  switch (dtype) {
    case B200_F32: sample_rows_kernel<float><<<(unsigned)B, kSampleThreads, 0, stream>>>((const float*)logits, ld, (int)V, inv_t, top_k, seed, step_dev, ids_out); break;
    case B200_F16: sample_rows_kernel<__half><<<(unsigned)B, kSampleThreads, 0, stream>>>((const __half*)logits, ld, (int)V, inv_t, top_k, seed, step_dev, ids_out); break;
    case B200_BF16:
      sample_rows_kernel<__nv_bfloat16><<<(unsigned)B, kSampleThreads, 0, stream>>>((const __nv_bfloat16*)logits, ld, (int)V, inv_t, top_k, seed, step_dev, ids_out);
      break;
    default: return B200_ERR_BAD_ARGUMENT;
  }
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

}  // namespace b200
