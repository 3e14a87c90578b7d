// out[M,N] = [gelu](A[M,K] . B[N,K]^T + bias) + residual  on the 5th-generation tensor cores.
//
// Persistent, warp-specialised kernel, one CTA per SM.  Two variants of one template:
//   CTAS = 1   a CTA computes a 128x256 tile alone (small problems)
//   CTAS = 2   a cluster of two CTAs computes a 256x256 tile with tcgen05.mma.cta_group::2: each CTA stages
//              its own 128 rows of A and its own 128-row half of the B tile, the even CTA issues the MMAs for
//              both, each CTA drains its own 128 accumulator rows.  Halving the B bytes per CTA is what lets
//              shared memory feed the tensor cores at full rate, and it buys a 5-deep instead of 3-deep ring.
// Roles per CTA:
//   warp 0      TMA producer: 128x64 tile of A and (256/CTAS)x64 tile of B per stage, 128-byte swizzle,
//               completion by mbarrier transaction bytes; every CTA issues its own loads
//   warp 1      allocates the 512 tensor-memory columns and issues tcgen05.mma (one thread);
//               tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-9   epilogue: tcgen05.ld the 128x256 fp32 accumulator (one row per thread, each warp
//               128 of the 256 columns), bias -> GELU -> residual -> cast.  For 16-bit data each warp
//               owns two 32-row x 64-column staging boxes in shared memory (128-byte swizzle): the
//               residual tile is TMA-loaded into them before the accumulator is awaited, results
//               overwrite it in place and leave as TMA tile stores, which also clip the ragged M and N
//               edges.  fp32 or unaligned outputs are stored from registers (residual prefetched into
//               registers).  The bias goes to shared memory ahead of the accumulator as well.
// Two 128x256 accumulators (2 x 256 columns) let the epilogue of tile i overlap the main
// loop of tile i+1.  Every wait on an mbarrier is bounded; a wait that gives up raises a
// CTA-wide abort flag, reports through status_word and the kernel drains and exits.
//
// Optional row statistics (template parameter STATS) for the tied lm_head: 1 = row argmax next to the stored
// product, 2 = argmax and log-sum-exp, 3 = argmax, optional log-sum-exp and the value at a per-row target column
// with nothing stored.  On a power-capped part every epilogue instruction per output element shows up in the
// clock of the main loop, so the epilogue is kept lean: packed fp32x2 adds/multiplies, no add without a bias,
// the row maximum by packed 16-bit max instructions over the rounded values; which column it sits in is looked up
// once per tile in the staging boxes when nothing is stored, and left to the small second kernel that reduces the
// per-slice partials when the product is stored (it re-reads the 32 stored values of the one chunk that wins the row).
#include <string.h>

#include <atomic>

#include "sm100_primitives.cuh"

namespace b200 {
namespace gemm {

using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + NUM_EPI_WARPS);
constexpr int EPI_COLS = BN / (NUM_EPI_WARPS / 4);  // columns per epilogue warp
constexpr int EPI_CHUNKS = EPI_COLS / 32;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_ROWS = 2048;  // rows per raster group (keeps a group's A rows and B columns L2-resident)
constexpr int CTRL_BYTES = 256;   // mbarriers, tensor-memory base, abort flag
constexpr int BIAS_BYTES = 2 * BN * 4;  // bias of the current and the next tile, as fp32
constexpr int EPI_BOX_COLS = 64;        // TMA store box: 64 columns (128 bytes of 16-bit data) x 32 rows
constexpr int EPI_BOX_BYTES = 32 * EPI_BOX_COLS * 2;        // 4 KB
constexpr int EPI_WARP_STAGE_BYTES = (EPI_COLS / EPI_BOX_COLS) * EPI_BOX_BYTES;  // one box per 64 of the warp's 128 columns: 8 KB
constexpr int EPI_STAGE_BYTES = NUM_EPI_WARPS * EPI_WARP_STAGE_BYTES;
static_assert(kLnExtCols == BK, "the LayerNorm extension is exactly one k-block");

template <int CTAS>
struct Cfg {
  static constexpr int STAGES = CTAS == 1 ? 3 : 5;
  static constexpr int TILE_M = BM * CTAS;  // rows per tile of the CTA group
  static constexpr int B_ROWS = BN / CTAS;  // rows of the B tile this CTA stages
  static constexpr int A_STAGE_BYTES = BM * BK * 2;
  static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_STAGE_BYTES + CTRL_BYTES + BIAS_BYTES;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  static constexpr int GROUP_M = GROUP_ROWS / TILE_M;
};

// Shared-memory matrix descriptor, K-major operand, 128-byte swizzle: rows are 128 bytes, an
// 8-row group is 1024 bytes (stride byte offset), leading byte offset unused for swizzled
// K-major layouts (set to 1), descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor for kind::f16: D fp32, A/B fp16 (0) or bf16 (1), both K-major, M = 128 (one CTA) or
// 256 (CTA pair), N = 256.
__host__ __device__ constexpr uint32_t make_idesc(int ab_format, int mma_m) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(mma_m >> 4) << 24);
}

struct TileCoord {
  int m, n;
};
// Raster: the column tiles are cut into panels of panel_n tiles (the host sizes a panel so that its part of B stays
// in L2: with a vocabulary-sized N the whole of B does not, and would be fetched from HBM again for every row
// group); inside a panel, groups of GROUP_M row tiles (GROUP_ROWS rows); inside a group the row tile varies
// fastest, so the CTAs that run at the same time share a few B column tiles and GROUP_M A row tiles in L2.
template <int GROUP_M>
__device__ __forceinline__ TileCoord tile_coord(int64_t t, int m_tiles, int n_tiles, int panel_n) {
  const int64_t per_panel = (int64_t)m_tiles * panel_n;
  const int panel = (int)(t / per_panel);
  const int64_t rem = t - (int64_t)panel * per_panel;
  const int n_first = panel * panel_n;
  const int pn = min(panel_n, n_tiles - n_first);
  const int64_t per_group = (int64_t)GROUP_M * pn;
  const int group = (int)(rem / per_group);
  const int within = (int)(rem - (int64_t)group * per_group);
  const int m_first = group * GROUP_M;
  const int gm = min(GROUP_M, m_tiles - m_first);
  TileCoord c;
  c.m = m_first + within % gm;
  c.n = n_first + within / gm;
  return c;
}

struct ArgmaxPartials {
  float* val;
  int* idx;
  float* sum;  // optional: per-slice sum of exp(value - slice maximum), for the row log-sum-exp
  int64_t ld;
};

// Running (maximum, its column, sum of exp(value - maximum)) of one thread's part of an output row.
struct RowStats {
  float best_val;
  int best_idx;
  float sumexp;
  int pending_col0;  // >= 0: best_val was found in the staged 32-column chunk starting here; its column is looked up once per tile
};

template <typename OutT>
struct EpilogueArgs {
  const OutT* bias;
  const OutT* residual;
  OutT* out;
  int64_t ld_res, ld_out;
  int tma_store;  // 16-bit output whose base and pitch allow a tensor map: results leave through TMA stores
  // Optional row-argmax partials: for every row, the maximum of each 128-column slice of the (rounded) output
  // and its column, stored slice-major: amax_val[slice * amax_ld + row].  NULL = not requested.
  float* amax_val;
  int* amax_idx;
  float* amax_sum;  // optional, same layout: sum over the slice of exp(value - slice maximum)
  int64_t amax_ld;
  // Statistics-only launches: optional per-row target column and where that row's (rounded) value at it goes.
  const int64_t* targets;
  float* target_val;
  // Output is written once and not read back soon, and B is large: store it with evict-first priority so that it
  // does not push B out of L2 (the tied lm_head: 77 MB of B against gigabytes of logits).
  int stream_out;
  // LN == 1, a LayerNorm folded into this GEMM: A holds the raw rows x, B the weights already multiplied by the
  // LayerNorm weight, and one extra 64-wide k-block comes from the two "extension" matrices (see launch_gemm_ln): its
  // products add  -mean_row * colsum[col] + (1 / rstd_row) * ln_bias[col]  to the accumulator, so that all the
  // epilogue has left to do is  out = rstd_row * acc  (then GELU / residual as usual).  No bias vector is read.
  const float2* ln_stats;  // per row of A: (mean, rstd)
  // LN == 2, the producer side: per row and per EPI_COLS-column slice of the output, the (mean, centred sum of
  // squares) of the values this epilogue stores, slice-major: stats_out[slice * stats_out_ld + row].  A small second
  // kernel merges a row's slices into its (mean, rstd).
  float2* stats_out;
  int64_t stats_out_ld;
};

// Shifted sums of one thread's part of an output row (LN == 2): sum and sum of squares of (value - shift), the shift
// being the first value seen, so that the centred sum of squares comes out without cancellation.
struct SliceMoments {
  float shift, s1, s2, n;
};

// x * sigmoid(2y), y = sqrt(2/pi) (x + 0.044715 x^3): algebraically the reference's
// 0.5 x (1 + tanh(y)) with tanh(y) = 2 sigmoid(2y) - 1 (kernels.py:15-26 of the reference),
// evaluated with one ex2 and one reciprocal on the special-function unit.
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float gelu_fast(float x) {
  const float c0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;  // -2 sqrt(2/pi) log2(e)
  const float c1 = c0 * 0.044715f;
  const float z = x * fmaf(x * x, c1, c0);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

// The same function with a single special-function operation: 0.5 x (1 + tanh(y)) on the hardware tanh.
// Its 2^-11 relative error in tanh is at most half a 16-bit ulp of the result, so it is used only when the
// output is rounded to fp16/bf16; fp32 outputs take gelu_fast.
// Two values at once: the multiplies and fused multiply-adds are packed fp32x2 instructions (rounded as the
// scalar forms).
__device__ __forceinline__ float2 gelu_tanh_approx2(float2 x) {
  const float c0 = 0.7978845608028654f, c1 = 0.7978845608028654f * 0.044715f;
  const float2 y = __fmul2_rn(x, __ffma2_rn(__fmul2_rn(x, x), make_float2(c1, c1), make_float2(c0, c0)));
  float2 t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(y.x));
  asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(y.y));
  const float2 h = __fmul2_rn(x, make_float2(0.5f, 0.5f));
  return __ffma2_rn(h, t, h);
}

__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// Tile store shared -> global through a tensor map; rows/columns outside the tensor are clipped.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src), "r"(c0), "r"(c1)
               : "memory");
}
// The same store with an L2 eviction-priority hint (a policy word from createpolicy).
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, uint32_t src, int c0, int c1, uint64_t policy) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group.L2::cache_hint [%0, {%2, %3}], [%1], %4;" ::"l"(map), "r"(src),
               "r"(c0), "r"(c1), "l"(policy)
               : "memory");
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all of this thread's earlier bulk stores have finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... all but the most recent one
__device__ __forceinline__ void tma_store_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t (&v)[4]) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <typename OutT>
__device__ __forceinline__ float2 unpack2(uint32_t u);
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}

// Element-wise maximum of two packed 16-bit pairs (a NaN loses against a number).
template <typename OutT>
__device__ __forceinline__ uint32_t max2(uint32_t a, uint32_t b);
template <>
__device__ __forceinline__ uint32_t max2<__half>(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
template <>
__device__ __forceinline__ uint32_t max2<__nv_bfloat16>(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// Lowest column of this thread's staged 32-column chunk (64 bytes of its row in a 128-byte-swizzled staging box,
// 16-byte slots [4*half, 4*half+4)) whose value equals `best`; 0 if there is none.
template <typename OutT>
__device__ __forceinline__ int find_staged_column(uint32_t box, int half, int lane, float best) {
  const uint32_t rowaddr = box + (uint32_t)lane * 128u;
  const uint32_t sw = (uint32_t)(lane & 7);
  int idx = 0;
#pragma unroll
  for (int g = 3; g >= 0; --g) {
    uint32_t q[4];
    ld_shared_v4(rowaddr + ((((uint32_t)(half * 4 + g)) ^ sw) << 4), q);
#pragma unroll
    for (int j = 3; j >= 0; --j) {
      const float2 r = unpack2<OutT>(q[j]);
      if (r.y == best) idx = g * 8 + 2 * j + 1;
      if (r.x == best) idx = g * 8 + 2 * j;
    }
  }
  return idx;
}

// How a thread may store its 32-column pieces of an output row.
enum StoreMode { STORE_SCALAR = 0, STORE_16B = 1, STORE_32B = 2 };

// Residual of one thread's row for its warp's EPI_COLS columns, fetched ahead of the accumulator.
// Only used on the wide path with a 16-bit output type: EPI_COLS halves = EPI_COLS/8 uint4.
struct ResidualRegs {
  uint4 v[EPI_COLS / 8];
};

// One thread, one row, 32 consecutive columns starting at col0: acc (+bias) -> GELU -> (+residual) -> out.
// `bias_s` points at this chunk's 32 fp32 bias values in shared memory (zeros when there is no bias).
// With `stage` != 0 (TMA-store path, 16-bit output) the 64 result bytes go to this thread's row of the warp's
// staging tile at 16-byte slots [4*half, 4*half+4) (128-byte swizzle); otherwise they are stored to global memory.
template <typename OutT, bool GELU, int STATS, int LN>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&acc)[32], const float* bias_s, const EpilogueArgs<OutT>& e,
                                               const uint4* res_regs, int64_t row, int col0, int64_t N, int mode, uint32_t stage,
                                               int half, int lane, bool row_ok, bool res_staged, RowStats& st, float ln_r, SliceMoments& mom) {
  // Two columns per instruction where the hardware has packed fp32 forms (add, mul, fma: same roundings as the
  // scalar ones); no bias, no add.
  float f[32];
  if constexpr (LN == 1) {
    // folded LayerNorm: the extension k-block already put -mean * colsum + ln_bias / rstd into the accumulator
    const float2 r2 = make_float2(ln_r, ln_r);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const float2 v2 = __fmul2_rn(make_float2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1])), r2);
      f[j] = v2.x, f[j + 1] = v2.y;
    }
  } else if (e.bias) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 b = *reinterpret_cast<const float4*>(bias_s + j);
      const float2 lo = __fadd2_rn(make_float2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1])), make_float2(b.x, b.y));
      const float2 hi = __fadd2_rn(make_float2(__uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3])), make_float2(b.z, b.w));
      f[j] = lo.x, f[j + 1] = lo.y, f[j + 2] = hi.x, f[j + 3] = hi.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(acc[j]);
  }
  if (GELU) {
    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
      for (int j = 0; j < 32; j += 2) {
        const float2 g = gelu_tanh_approx2(make_float2(f[j], f[j + 1]));
        f[j] = g.x, f[j + 1] = g.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = gelu_fast(f[j]);
    }
  }
  const bool full = col0 + 32 <= N;
  if constexpr (sizeof(OutT) == 2) {
    if (stage != 0 || (mode != STORE_SCALAR && full)) {
      if (res_staged) {
        // residual tile already sits in this thread's slots of the staging box (zero outside the matrix)
        const uint32_t rowaddr = stage + (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint32_t rw[4];
          ld_shared_v4(rowaddr + ((((uint32_t)(half * 4 + g)) ^ sw) << 4), rw);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 r = unpack2<OutT>(rw[j]);
            f[g * 8 + 2 * j] += r.x;
            f[g * 8 + 2 * j + 1] += r.y;
          }
        }
      } else if (res_regs) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const uint32_t* rw = reinterpret_cast<const uint32_t*>(&res_regs[g]);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 r = unpack2<OutT>(rw[j]);
            f[g * 8 + 2 * j] += r.x;
            f[g * 8 + 2 * j + 1] += r.y;
          }
        }
      } else if (e.residual && row_ok) {
        // ragged last column chunk on the staged path: element-wise, inside the matrix only
        const OutT* rrow = e.residual + row * e.ld_res + col0;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < N) f[j] += to_float(rrow[j]);
      }
      if constexpr (LN == 2) {
        // moments of this row's slice, over the fp32 values about to be rounded and stored
        if (mom.n == 0.f) mom.shift = f[0];
        const float2 sh = make_float2(-mom.shift, -mom.shift);
        if (full) {
          float2 a1 = make_float2(0.f, 0.f), a2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 d = __fadd2_rn(make_float2(f[j], f[j + 1]), sh);
            a1 = __fadd2_rn(a1, d);
            a2 = __ffma2_rn(d, d, a2);
          }
          mom.s1 += a1.x + a1.y, mom.s2 += a2.x + a2.y, mom.n += 32.f;
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (col0 + j < N) {
              const float d = f[j] - mom.shift;
              mom.s1 += d, mom.s2 = fmaf(d, d, mom.s2), mom.n += 1.f;
            }
          }
        }
      }
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] = pack2<OutT>(f[2 * j], f[2 * j + 1]);
      if constexpr (STATS) {
        // compare what is stored (the rounded values); strict '>' keeps the lowest column among equal maxima
        const float m_old = st.best_val;
        if (stage != 0 && full) {
          // chunk maximum with packed 16-bit max instructions; which column it sits in is looked up later, once per
          // tile, in the staging tile (find_staged_column), and only for the chunk that won
          uint32_t m = w[0];
#pragma unroll
          for (int j = 1; j < 16; ++j) m = max2<OutT>(m, w[j]);
          const float2 mm = unpack2<OutT>(m);
          const float cm = fmaxf(mm.x, mm.y);
          if (cm > st.best_val) st.best_val = cm, st.pending_col0 = col0;
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 r = unpack2<OutT>(w[j]);
            if (col0 + 2 * j < N && r.x > st.best_val) st.best_val = r.x, st.best_idx = col0 + 2 * j, st.pending_col0 = -1;
            if (col0 + 2 * j + 1 < N && r.y > st.best_val) st.best_val = r.y, st.best_idx = col0 + 2 * j + 1, st.pending_col0 = -1;
          }
        }
        if (STATS == 2 && st.best_val > -INFINITY) {
          // online log-sum-exp: rescale what was summed against the old maximum, add this chunk
          const float kLog2e = 1.4426950408889634f;
          const float m2 = st.best_val * kLog2e;
          float acc_sum = st.sumexp * ex2_approx(m_old * kLog2e - m2);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 r = unpack2<OutT>(w[j]);
            if (col0 + 2 * j < N) acc_sum += ex2_approx(fmaf(r.x, kLog2e, -m2));
            if (col0 + 2 * j + 1 < N) acc_sum += ex2_approx(fmaf(r.y, kLog2e, -m2));
          }
          st.sumexp = acc_sum;
        }
      }
      if (stage != 0) {
        const uint32_t rowaddr = stage + (uint32_t)lane * 128u;
        const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
        for (int g = 0; g < 4; ++g) st_shared_v4(rowaddr + ((((uint32_t)(half * 4 + g)) ^ sw) << 4), w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
      } else {
        OutT* orow = e.out + row * e.ld_out + col0;
        if (mode == STORE_32B) {
          st_global_v8(orow, reinterpret_cast<const uint32_t(&)[8]>(w[0]));
          st_global_v8(orow + 16, reinterpret_cast<const uint32_t(&)[8]>(w[8]));
        } else {
#pragma unroll
          for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(orow + g * 8) = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
        }
      }
      return;
    }
  } else {
    if (mode != STORE_SCALAR && full) {
      float* orow = reinterpret_cast<float*>(e.out) + row * e.ld_out + col0;
      if (e.residual) {
        const float* rrow = reinterpret_cast<const float*>(e.residual) + row * e.ld_res + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 r = *reinterpret_cast<const float4*>(rrow + j);
          f[j] += r.x, f[j + 1] += r.y, f[j + 2] += r.z, f[j + 3] += r.w;
        }
      }
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(orow + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
      if constexpr (STATS) {
        const float m_old = st.best_val;
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (f[j] > st.best_val) st.best_val = f[j], st.best_idx = col0 + j, st.pending_col0 = -1;
        if (STATS == 2 && st.best_val > -INFINITY) {
          const float kLog2e = 1.4426950408889634f;
          const float m2 = st.best_val * kLog2e;
          float acc_sum = st.sumexp * ex2_approx(m_old * kLog2e - m2);
#pragma unroll
          for (int j = 0; j < 32; ++j) acc_sum += ex2_approx(fmaf(f[j], kLog2e, -m2));
          st.sumexp = acc_sum;
        }
      }
      return;
    }
  }
  // element-wise tail: ragged columns, unaligned output
  OutT* orow = e.out + row * e.ld_out + col0;
  const OutT* rrow = e.residual ? e.residual + row * e.ld_res + col0 : nullptr;
  const float m_old = st.best_val;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (col0 + j < N) {
      float v = f[j];
      if (rrow) v += to_float(rrow[j]);
      if constexpr (LN == 2) {  // (reached by the narrow-tile kernel's ragged last chunk only)
        if (mom.n == 0.f) mom.shift = v;
        const float d = v - mom.shift;
        mom.s1 += d, mom.s2 = fmaf(d, d, mom.s2), mom.n += 1.f;
      }
      const OutT o = from_float<OutT>(v);
      orow[j] = o;
      f[j] = to_float(o);
      if (STATS && f[j] > st.best_val) st.best_val = f[j], st.best_idx = col0 + j, st.pending_col0 = -1;
    }
  }
  if (STATS == 2 && st.best_val > -INFINITY) {
    const float kLog2e = 1.4426950408889634f;
    const float m2 = st.best_val * kLog2e;
    float acc_sum = st.sumexp * ex2_approx(m_old * kLog2e - m2);
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < N) acc_sum += ex2_approx(fmaf(f[j], kLog2e, -m2));
    st.sumexp = acc_sum;
  }
}

// Statistics-only epilogue (nothing goes to global memory): the 32 values a thread would have written, rounded to
// the output type as the storing epilogue rounds them, update the row's running maximum / column and, if wanted,
// its sum of exponentials; the value at column `tgt` (if it falls into this chunk) is picked out.
template <typename OutT>
__device__ __forceinline__ void stats_only_chunk(const uint32_t (&acc)[32], const float* bias_s, bool has_bias, bool want_lse, int col0, int64_t N,
                                                 int tgt, uint32_t box, int half, int lane, RowStats& st, float& picked) {
  static_assert(sizeof(OutT) == 2, "row statistics without the product are built for 16-bit rounding");
  float f[32];
  if (has_bias) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      const float4 b = *reinterpret_cast<const float4*>(bias_s + j);
      const float2 lo = __fadd2_rn(make_float2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1])), make_float2(b.x, b.y));
      const float2 hi = __fadd2_rn(make_float2(__uint_as_float(acc[j + 2]), __uint_as_float(acc[j + 3])), make_float2(b.z, b.w));
      f[j] = lo.x, f[j + 1] = lo.y, f[j + 2] = hi.x, f[j + 3] = hi.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(acc[j]);
  }
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) w[j] = pack2<OutT>(f[2 * j], f[2 * j + 1]);
  const float m_old = st.best_val;
  const bool full = col0 + 32 <= N;
  if (full) {
    // chunk maximum with packed 16-bit max instructions; the chunk is parked in the warp's staging tile so that the
    // column of the tile's maximum can be looked up once per tile (find_staged_column)
    const uint32_t rowaddr = box + (uint32_t)lane * 128u;
    const uint32_t sw = (uint32_t)(lane & 7);
#pragma unroll
    for (int g = 0; g < 4; ++g) st_shared_v4(rowaddr + ((((uint32_t)(half * 4 + g)) ^ sw) << 4), w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
    uint32_t m = w[0];
#pragma unroll
    for (int j = 1; j < 16; ++j) m = max2<OutT>(m, w[j]);
    const float2 mm = unpack2<OutT>(m);
    const float cm = fmaxf(mm.x, mm.y);
    if (cm > st.best_val) st.best_val = cm, st.pending_col0 = col0;
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 r = unpack2<OutT>(w[j]);
      if (col0 + 2 * j < N && r.x > st.best_val) st.best_val = r.x, st.best_idx = col0 + 2 * j, st.pending_col0 = -1;  // strict '>': lowest column wins ties
      if (col0 + 2 * j + 1 < N && r.y > st.best_val) st.best_val = r.y, st.best_idx = col0 + 2 * j + 1, st.pending_col0 = -1;
    }
  }
  if (want_lse && st.best_val > -INFINITY) {
    const float kLog2e = 1.4426950408889634f;
    const float m2 = st.best_val * kLog2e;
    float acc_sum = st.sumexp * ex2_approx(m_old * kLog2e - m2);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 r = unpack2<OutT>(w[j]);
      if (full || col0 + 2 * j < N) acc_sum += ex2_approx(fmaf(r.x, kLog2e, -m2));
      if (full || col0 + 2 * j + 1 < N) acc_sum += ex2_approx(fmaf(r.y, kLog2e, -m2));
    }
    st.sumexp = acc_sum;
  }
  if (tgt >= col0 && tgt < col0 + 32) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float2 r = unpack2<OutT>(w[j]);
      if (col0 + 2 * j == tgt) picked = r.x;
      if (col0 + 2 * j + 1 == tgt) picked = r.y;
    }
  }
}

// LN: 0 = plain; 1 = a LayerNorm of A's rows is folded into the epilogue (EpilogueArgs::ln_*); 2 = the epilogue also
// emits per-slice row moments of what it stores (EpilogueArgs::stats_out), which a following LN == 1 GEMM consumes.
template <typename OutT, bool GELU, int CTAS, int STATS, int LN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_out, const __grid_constant__ CUtensorMap map_res,
               const __grid_constant__ CUtensorMap map_a_ext, const __grid_constant__ CUtensorMap map_b_ext, EpilogueArgs<OutT> epi,
               int64_t M, int64_t N, int64_t K, uint32_t idesc, int panel_n, int* status_word) {
  using C = Cfg<CTAS>;
  constexpr int STAGES = C::STAGES;
  // 128-byte-swizzled tiles need 1024-byte aligned bases (the dynamic shared memory base is the same in both
  // CTAs of a pair, so the two CTAs use identical offsets, which cta_group::2 descriptors rely on).
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);
  if (base & 1023u) {  // never expected; refuse to run rather than compute on misplaced tiles (uniform over the grid)
    pdl_wait();
    if (threadIdx.x == 0 && status_word) atomicCAS(status_word, 0, 99);
    return;
  }
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + STAGES * C::A_STAGE_BYTES;
  const uint32_t smem_epi = base + STAGES * C::STAGE_BYTES;  // [NUM_EPI_WARPS][32 rows][128 bytes]
  uint8_t* ctrl = smem + STAGES * C::STAGE_BYTES + EPI_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);  // full[S], empty[S], acc_full[2], acc_empty[2], bias_ready[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_acc_full = bar_empty + 8 * STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  const uint32_t bar_bias = bar_acc_empty + 16;
  const uint32_t bar_res = bar_bias + 16;  // [NUM_EPI_WARPS]: residual boxes of a warp have landed
  constexpr int NUM_BARS = 2 * STAGES + 6 + NUM_EPI_WARPS;
  static_assert(8 * NUM_BARS + 16 <= CTRL_BYTES, "control block too small");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 8 * NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * NUM_BARS + 8);
  float* bias_smem = reinterpret_cast<float*>(ctrl + CTRL_BYTES);  // [2][BN]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = CTAS == 2 ? cluster_ctarank() : 0u;  // 0 = leader (issues the MMAs)
  const int64_t group_id = CTAS == 2 ? (int64_t)(blockIdx.x >> 1) : (int64_t)blockIdx.x;
  const int64_t num_groups = CTAS == 2 ? (int64_t)(gridDim.x >> 1) : (int64_t)gridDim.x;

  const int m_tiles = (int)((M + C::TILE_M - 1) / C::TILE_M);
  const int n_tiles = (int)((N + BN - 1) / BN);
  const int64_t num_tiles = (int64_t)m_tiles * n_tiles;
  const int num_kb_ab = (int)((K + BK - 1) / BK);
  const int num_kb = num_kb_ab + (LN == 1 ? 1 : 0);  // a folded LayerNorm appends the extension k-block

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_acc_full + 8 * a, 1);
      mbar_init(bar_acc_empty + 8 * a, NUM_EPI_WARPS * CTAS);  // the leader's barrier collects both CTAs' epilogue warps
      mbar_init(bar_bias + 8 * a, NUM_EPI_WARPS);
    }
    for (int w = 0; w < NUM_EPI_WARPS; ++w) mbar_init(bar_res + 8 * w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    if constexpr (CTAS == 2) {
      tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // both CTAs' barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only this CTA's own shared and tensor memory and may overlap the previous kernel of the
  // stream; from here on global memory is read and written.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      // completion bytes of both CTAs' loads are posted on the leader's full barrier
      const uint32_t full_base = CTAS == 2 ? mapa_shared(bar_full, 0) : bar_full;
      for (int64_t t = group_id; t < num_tiles && alive; t += num_groups) {
        const TileCoord tc = tile_coord<C::GROUP_M>(t, m_tiles, n_tiles, panel_n);
        const int row_a = tc.m * C::TILE_M + (int)cta_rank * BM;
        const int row_b = tc.n * BN + (int)cta_rank * C::B_ROWS;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status_word, 1)) {
            alive = false;
            break;
          }
          // (LN == 1: the last k-block is the 64-wide extension pair, at column 0 of its own two matrices)
          const bool ext = LN == 1 && kb == num_kb_ab;
          const CUtensorMap* ma = ext ? &map_a_ext : &map_a;
          const CUtensorMap* mb = ext ? &map_b_ext : &map_b;
          const int kcol = ext ? 0 : kb * BK;
          if constexpr (CTAS == 2) {
            if (cta_rank == 0) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * C::STAGE_BYTES);
            tma_load_2d_pair(smem_a + stage * C::A_STAGE_BYTES, ma, full_base + 8 * stage, kcol, row_a);
            tma_load_2d_pair(smem_b + stage * C::B_STAGE_BYTES, mb, full_base + 8 * stage, kcol, row_b);
          } else {
            mbar_arrive_expect_tx(bar_full + 8 * stage, C::STAGE_BYTES);
            tma_load_2d(smem_a + stage * C::A_STAGE_BYTES, ma, bar_full + 8 * stage, kcol, row_a);
            tma_load_2d(smem_b + stage * C::B_STAGE_BYTES, mb, bar_full + 8 * stage, kcol, row_b);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (the leader CTA's only, for a pair)
    if (lane == 0 && cta_rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      for (int64_t t = group_id; t < num_tiles && alive; t += num_groups) {
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, status_word, 2)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, status_word, 3)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_a + stage * C::A_STAGE_BYTES);
          const uint64_t db = make_smem_desc(smem_b + stage * C::B_STAGE_BYTES);
          // (LN == 1: only the first 8 columns of the extension k-block are non-zero: one 16-wide MMA covers it)
          const int k_steps = (LN == 1 && kb == num_kb_ab) ? 1 : BK / UMMA_K;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (k >= k_steps) break;
            // advance 16 elements (32 bytes) along K inside the swizzle row: +2 in 16-byte units
            if constexpr (CTAS == 2)
              umma_f16_pair(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (uint32_t)((kb | k) != 0));
            else
              umma_f16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (uint32_t)((kb | k) != 0));
          }
          if constexpr (CTAS == 2) umma_commit_pair(bar_empty + 8 * stage); else umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        if constexpr (CTAS == 2) umma_commit_pair(bar_acc_full + 8 * acc); else umma_commit(bar_acc_full + 8 * acc);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;             // a warp may only touch tensor-memory lanes [32*(warp%4), +32)
    const int col_half = (warp - 2) >> 2;     // which EPI_COLS-wide column range of the tile this warp owns
    const int epi_tid = (int)threadIdx.x - 64;  // 0 .. 32*NUM_EPI_WARPS-1
    int acc = 0;
    uint32_t acc_phase = 0;
    constexpr int esz = (int)sizeof(OutT);
    const uintptr_t out_al = reinterpret_cast<uintptr_t>(epi.out) | (uintptr_t)(epi.ld_out * esz);
    const uintptr_t res_al = epi.residual ? (reinterpret_cast<uintptr_t>(epi.residual) | (uintptr_t)(epi.ld_res * esz)) : 0;
    int mode = STORE_SCALAR;
    if (((out_al | res_al) & 15) == 0) mode = (esz == 2 && (out_al & 31) == 0) ? STORE_32B : STORE_16B;
    const uint32_t acc_empty_base = CTAS == 2 ? mapa_shared(bar_acc_empty, 0) : bar_acc_empty;
    const bool use_tma = STATS != 3 && esz == 2 && epi.tma_store != 0;
    const bool res_tma = use_tma && epi.residual != nullptr;  // (the host only sets tma_store when the residual can be mapped too)
    const uint32_t stage_addr = use_tma ? smem_epi + (uint32_t)(warp - 2) * EPI_WARP_STAGE_BYTES : 0u;
    const uint32_t stats_stage = smem_epi + (uint32_t)(warp - 2) * EPI_WARP_STAGE_BYTES;  // statistics-only launches park chunks here
    const uint32_t my_res_bar = bar_res + 8 * (uint32_t)(warp - 2);
    uint32_t res_phase = 0;
    const uint64_t out_policy = l2_policy_evict_first();
    for (int64_t t = group_id; t < num_tiles; t += num_groups) {
      const TileCoord tc = tile_coord<C::GROUP_M>(t, m_tiles, n_tiles, panel_n);
      const int64_t row = (int64_t)tc.m * C::TILE_M + (int64_t)cta_rank * BM + quarter * 32 + lane;
      const int col_base = tc.n * BN + col_half * EPI_COLS;
      const int row_warp = (int)(tc.m * C::TILE_M + (int)cta_rank * BM + quarter * 32);  // first row of this warp's 32
      const bool row_ok = row < M;
      // Prefetch what does not depend on the accumulator: bias -> shared memory, residual -> staging boxes (TMA)
      // or registers.
      if (res_tma) {
        // both staging boxes are about to be overwritten by the residual: the previous tile's TMA stores must be done reading them
        if (lane == 0) {
          tma_store_wait_read();
          {
            mbar_arrive_expect_tx(my_res_bar, EPI_WARP_STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < EPI_COLS / EPI_BOX_COLS; ++b)
              tma_load_2d(stage_addr + b * EPI_BOX_BYTES, &map_res, my_res_bar, col_base + b * EPI_BOX_COLS, row_warp);
          }
        }
        __syncwarp();
      }
      float* bias_s = bias_smem + acc * BN;
      for (int i = epi_tid; i < BN; i += 32 * NUM_EPI_WARPS) {
        const int c = tc.n * BN + i;
        if constexpr (LN != 1) bias_s[i] = (epi.bias && c < N) ? to_float(epi.bias[c]) : 0.f;
      }
      // folded LayerNorm: this row's rstd
      float ln_r = 1.f;
      if constexpr (LN == 1) {
        if (row_ok) ln_r = __ldg(epi.ln_stats + row).y;
      }
      SliceMoments mom{0.f, 0.f, 0.f, 0.f};
      ResidualRegs res;
      const bool res_in_regs = !use_tma && esz == 2 && epi.residual && mode != STORE_SCALAR && row_ok;
      if (res_in_regs) {
        const OutT* rrow = epi.residual + row * epi.ld_res + col_base;
#pragma unroll
        for (int i = 0; i < EPI_COLS / 8; ++i) {
          if (col_base + (i / 4) * 32 + 32 <= N) res.v[i] = *reinterpret_cast<const uint4*>(rrow + i * 8);
        }
      }
      // bias visible to all epilogue warps (an mbarrier, not bar.sync: its wait is bounded like every other)
      if constexpr (LN != 1) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_bias + 8 * acc);
        if (!mbar_wait(bar_bias + 8 * acc, acc_phase, abort_flag, status_word, 5)) break;
      }
      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, status_word, 4)) break;
      if (res_tma) {
        if (!mbar_wait(my_res_bar, res_phase, abort_flag, status_word, 6)) break;
        res_phase ^= 1u;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + col_half * EPI_COLS);
      RowStats stats{-INFINITY, 0, 0.f, -1};
      float picked = 0.f;
      int tgt = -1;
      if constexpr (STATS == 3) {
        if (epi.targets && row_ok) {
          const int64_t t64 = epi.targets[row];
          tgt = (t64 >= col_base && t64 < col_base + EPI_COLS) ? (int)t64 : -1;
        }
      }
#pragma unroll(STATS == 2 ? 1 : EPI_CHUNKS)  // argmax + log-sum-exp + store: rolled, or the unrolled body spills
      for (int c = 0; c < EPI_CHUNKS; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (c == EPI_CHUNKS - 1) {
          // accumulator fully read: hand it back to the MMA warp before doing the last chunk's math
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if constexpr (CTAS == 2) mbar_arrive_cluster(acc_empty_base + 8 * acc); else mbar_arrive(bar_acc_empty + 8 * acc);
          }
        }
        const int col0 = col_base + c * 32;
        if constexpr (STATS == 3) {
          if constexpr (sizeof(OutT) == 2) {
            if (row_ok && col0 < N)
              stats_only_chunk<OutT>(v, bias_s + col_half * EPI_COLS + c * 32, epi.bias != nullptr, epi.amax_sum != nullptr, col0, N, tgt,
                                     stats_stage + (uint32_t)(c >> 1) * EPI_BOX_BYTES, c & 1, lane, stats, picked);
          }
        } else if (use_tma) {
          const uint32_t box = stage_addr + (uint32_t)(c >> 1) * EPI_BOX_BYTES;
          if (!res_tma && (c & 1) == 0) {
            // about to overwrite this box: its store of the previous tile is the second most recent bulk group
            if (lane == 0) tma_store_wait_read_but_one();
            __syncwarp();
          }
          if (col0 < N)
            epilogue_chunk<OutT, GELU, STATS, LN>(v, bias_s + col_half * EPI_COLS + c * 32, epi, nullptr, row, col0, N, mode, box, c & 1, lane, row_ok,
                                                  res_tma, stats, ln_r, mom);
          if ((c & 1) == 1) {
            fence_proxy_async_smem();
            __syncwarp();
            const int box_col = col_base + (c >> 1) * EPI_BOX_COLS;
            if (lane == 0) {
              if (box_col < N && row_warp < M) {
                if (epi.stream_out) tma_store_2d_hint(&map_out, box, box_col, row_warp, out_policy);
                else tma_store_2d(&map_out, box, box_col, row_warp);
              }
              tma_store_commit();  // always one bulk group per box and tile (possibly empty): the waits above count groups
            }
          }
        } else if (row_ok && col0 < N) {
          epilogue_chunk<OutT, GELU, STATS, LN>(v, bias_s + col_half * EPI_COLS + c * 32, epi, (res_in_regs && col0 + 32 <= N) ? &res.v[c * 4] : nullptr, row, col0, N,
                                                mode, 0u, 0, lane, row_ok, false, stats, ln_r, mom);
        }
      }
      if constexpr (STATS != 0 && sizeof(OutT) == 2) {
        if (stats.pending_col0 >= 0) {
          if constexpr (STATS == 3) {
            // nothing is stored: look the column up now; the winning chunk still sits in this warp's staging boxes
            // (nothing overwrites them before the next tile)
            const int c = (stats.pending_col0 - col_base) >> 5;
            stats.best_idx = stats.pending_col0 + find_staged_column<OutT>(stats_stage + (uint32_t)(c >> 1) * EPI_BOX_BYTES, c & 1, lane, stats.best_val);
          } else {
            // the product is stored: only the 32-column chunk of the maximum is recorded here (as -(first column + 1));
            // the reducing kernel reads those 32 stored values of the one chunk that wins the whole row
            stats.best_idx = -(stats.pending_col0 + 1);
          }
        }
      }
      if constexpr (LN == 2) {
        if (row_ok && mom.n > 0.f) {
          // (mean, centred sum of squares) of this row's slice
          const float inv = 1.0f / mom.n;
          const int64_t slice = (int64_t)tc.n * (BN / EPI_COLS) + col_half;
          epi.stats_out[slice * epi.stats_out_ld + row] = make_float2(fmaf(mom.s1, inv, mom.shift), fmaxf(mom.s2 - mom.s1 * mom.s1 * inv, 0.f));
        }
      }
      if (STATS && row_ok) {
        const int64_t slice = (int64_t)tc.n * (BN / EPI_COLS) + col_half;
        epi.amax_val[slice * epi.amax_ld + row] = stats.best_val;
        epi.amax_idx[slice * epi.amax_ld + row] = stats.best_idx;
        if (STATS == 2 || (STATS == 3 && epi.amax_sum)) epi.amax_sum[slice * epi.amax_ld + row] = stats.sumexp;
        if (STATS == 3 && tgt >= 0 && tgt < N) epi.target_val[row] = picked;
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (use_tma && lane == 0) tma_store_wait_read();  // staging memory must outlive the last bulk store's read
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    // Give copies and MMAs already in flight time to land before shared and tensor memory go away.
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (CTAS == 2) cluster_sync_all();  // the peer may still be signalling this CTA's barriers or reading its tiles
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CTAS == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ------------------------------------------------------------------ narrow-tile variant for few rows
// With M <= kNarrowMaxRows (one generated token per sequence; tiny configurations) the 256 x 256 tiles of the kernel
// above leave most of the GPU idle: a 512 x 768 x 3072 product is 6 tiles, each a serial loop of 48 k-blocks.  This
// kernel computes ONE 128 x 64 tile per CTA (grid = column tiles x row tiles, no persistence, one accumulator), so
// the same product becomes 48 CTAs: the same TMA ring, tcgen05.mma (M = 128, N = 64, cta_group::1) and fused
// epilogue arithmetic (epilogue_chunk, direct 16-byte stores), k-blocks in the same order, hence the same bits.
// 16-bit output, no row statistics of the argmax kind; LN = 1 / 2 as above, the moments of LN = 2 per 64-column slice.
// Warp 0: TMA producer; warp 1: tensor-memory owner and MMA issuer; warps 2-5: epilogue (one row per thread).
constexpr int NARROW_BN = 64;
constexpr int NARROW_STAGES = 6;
constexpr int NARROW_A_BYTES = BM * BK * 2;         // 16 KB
constexpr int NARROW_B_BYTES = NARROW_BN * BK * 2;  // 8 KB
constexpr int NARROW_STAGE_BYTES = NARROW_A_BYTES + NARROW_B_BYTES;
constexpr int NARROW_THREADS = 192;
constexpr int NARROW_CTRL_BYTES = 256;
constexpr int NARROW_SMEM_BYTES = NARROW_STAGES * NARROW_STAGE_BYTES + 1024 + NARROW_CTRL_BYTES + NARROW_BN * 4;
constexpr int kNarrowMaxRows = 512;

template <typename OutT, bool GELU, int LN>
__global__ void __launch_bounds__(NARROW_THREADS, 1)
gemm_narrow_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_a_ext, const __grid_constant__ CUtensorMap map_b_ext, EpilogueArgs<OutT> epi,
                   int64_t M, int64_t N, int64_t K, uint32_t idesc, int* status_word) {
  static_assert(sizeof(OutT) == 2, "the narrow-tile kernel stores 16-bit outputs");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;  // 128-byte-swizzled tiles need 1024-byte aligned bases
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + NARROW_STAGES * NARROW_A_BYTES;
  uint8_t* ctrl = smem + NARROW_STAGES * NARROW_STAGE_BYTES;
  const uint32_t bars = smem_u32(ctrl);
  const uint32_t bar_full = bars, bar_empty = bars + 8 * NARROW_STAGES, bar_acc = bars + 16 * NARROW_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 16 * NARROW_STAGES + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 16 * NARROW_STAGES + 16);
  static_assert(16 * NARROW_STAGES + 24 <= NARROW_CTRL_BYTES, "control block too small");
  float* bias_s = reinterpret_cast<float*>(ctrl + NARROW_CTRL_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * NARROW_BN, m0 = blockIdx.y * BM;
  const int num_kb_ab = (int)((K + BK - 1) / BK);
  const int num_kb = num_kb_ab + (LN == 1 ? 1 : 0);
  if (threadIdx.x == 0) {
    for (int i = 0; i < NARROW_STAGES; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, 1);
    }
    mbar_init(bar_acc, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), NARROW_BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_slot;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status_word, 31)) break;
        const bool ext = LN == 1 && kb == num_kb_ab;
        mbar_arrive_expect_tx(bar_full + 8 * stage, NARROW_STAGE_BYTES);
        tma_load_2d(smem_a + stage * NARROW_A_BYTES, ext ? &map_a_ext : &map_a, bar_full + 8 * stage, ext ? 0 : kb * BK, m0);
        tma_load_2d(smem_b + stage * NARROW_B_BYTES, ext ? &map_b_ext : &map_b, bar_full + 8 * stage, ext ? 0 : kb * BK, n0);
        if (++stage == NARROW_STAGES) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, status_word, 32)) {
          alive = false;
          break;
        }
        tc_fence_after();
        const uint64_t da = make_smem_desc(smem_a + stage * NARROW_A_BYTES);
        const uint64_t db = make_smem_desc(smem_b + stage * NARROW_B_BYTES);
        const int k_steps = (LN == 1 && kb == num_kb_ab) ? 1 : BK / UMMA_K;  // (the extension block: 8 non-zero columns)
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {
          if (k >= k_steps) break;
          umma_f16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (uint32_t)((kb | k) != 0));
        }
        umma_commit(bar_empty + 8 * stage);
        if (++stage == NARROW_STAGES) stage = 0, phase ^= 1u;
      }
      if (alive) umma_commit(bar_acc);
    }
  } else {
    // epilogue: warp w reads tensor-memory lanes [32 * (w % 4), + 32) = rows of the tile
    const int quarter = warp & 3;
    const int64_t row = (int64_t)m0 + quarter * 32 + lane;
    const bool row_ok = row < M;
    const int epi_tid = threadIdx.x - 64;
    if (epi_tid < NARROW_BN) {
      const int c = n0 + epi_tid;
      bias_s[epi_tid] = (LN != 1 && epi.bias && c < N) ? to_float(epi.bias[c]) : 0.f;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
    float ln_r = 1.f;
    if constexpr (LN == 1) {
      if (row_ok) ln_r = __ldg(epi.ln_stats + row).y;
    }
    const uintptr_t out_al = reinterpret_cast<uintptr_t>(epi.out) | (uintptr_t)(epi.ld_out * 2);
    const uintptr_t res_al = epi.residual ? (reinterpret_cast<uintptr_t>(epi.residual) | (uintptr_t)(epi.ld_res * 2)) : 0;
    const int mode = ((out_al | res_al) & 15) == 0 ? STORE_16B : STORE_SCALAR;
    // residual of this thread's row, fetched while the main loop runs
    uint4 res[NARROW_BN / 8];
    const bool res_in_regs = epi.residual && mode != STORE_SCALAR && row_ok;
    if (res_in_regs) {
      const OutT* rrow = epi.residual + row * epi.ld_res + n0;
#pragma unroll
      for (int i = 0; i < NARROW_BN / 8; ++i)
        if (n0 + (i / 4) * 32 + 32 <= N) res[i] = *reinterpret_cast<const uint4*>(rrow + i * 8);
    }
    if (mbar_wait(bar_acc, 0, abort_flag, status_word, 33)) {
      tc_fence_after();
      RowStats unused{-INFINITY, 0, 0.f, -1};
      SliceMoments mom{0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < NARROW_BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= N) break;  // (warp-uniform)
        uint32_t v[32];
        tmem_ld_32x32(tmem_d + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (row_ok)
          epilogue_chunk<OutT, GELU, 0, LN>(v, bias_s + c * 32, epi, (res_in_regs && col0 + 32 <= N) ? &res[c * 4] : nullptr, row, col0, N, mode, 0u,
                                            c & 1, lane, row_ok, false, unused, ln_r, mom);
      }
      if constexpr (LN == 2) {
        if (row_ok && mom.n > 0.f) {
          const float inv = 1.0f / mom.n;
          epi.stats_out[(int64_t)blockIdx.x * epi.stats_out_ld + row] = make_float2(fmaf(mom.s1, inv, mom.shift), fmaxf(mom.s2 - mom.s1 * mom.s1 * inv, 0.f));
        }
      }
    }
  }

  // ------------------------------------------------------------ teardown
  __syncwarp();
  if (*abort_flag) {
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_d, NARROW_BN);
  }
}

// ------------------------------------------------------------------ host side
// 2-D map over a row-major [rows, cols] 16-bit matrix with leading dimension ld; box = 64 columns x box_rows.
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows, int op_dtype) {
  const uint64_t dims[2] = {(uint64_t)cols, (uint64_t)rows}, strides[1] = {(uint64_t)ld * 2};
  const uint32_t box[2] = {(uint32_t)BK, (uint32_t)box_rows};
  return encode_tensor_map(map, ptr, 2, dims, strides, box, op_dtype, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

// Largest number of 2-CTA clusters of this kernel that can be resident at once (cached per instantiation).
template <typename OutT, bool GELU, int STATS, int LN>
static int max_pairs() {
  static std::atomic<int> cache[kMaxDevices];  // per device; stored as value + 1 so that 0 means "not asked yet"
  const int slot = device_slot();
  if (slot < 0) return 0;
  const int seen = cache[slot].load(std::memory_order_acquire);
  if (seen > 0) return seen - 1;
  if (cudaFuncSetAttribute(gemm_tn_kernel<OutT, GELU, 2, STATS, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<2>::SMEM_BYTES) != cudaSuccess) {
    cudaGetLastError();
    cache[slot].store(1, std::memory_order_release);
    return 0;
  }
  LaunchSetup ls(dim3((unsigned)sm_count() / 2 * 2), dim3(NUM_THREADS), Cfg<2>::SMEM_BYTES, nullptr, 2, false);
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, gemm_tn_kernel<OutT, GELU, 2, STATS, LN>, &ls.cfg) != cudaSuccess || n < 1) {
    cudaGetLastError();
    n = 0;
  }
  cache[slot].store(n + 1, std::memory_order_release);
  return n;
}

// Map over a 16-bit [M, N] matrix (pitch ld) for tile stores/loads of 64 columns x 32 rows (output, residual).
static int make_out_map(CUtensorMap* map, void* ptr, int64_t M, int64_t N, int64_t ld_out, int io_dtype) {
  const uint64_t dims[2] = {(uint64_t)N, (uint64_t)M}, strides[1] = {(uint64_t)ld_out * 2};
  const uint32_t box[2] = {(uint32_t)EPI_BOX_COLS, 32};
  return encode_tensor_map(map, ptr, 2, dims, strides, box, io_dtype, CU_TENSOR_MAP_L2_PROMOTION_NONE);
}

template <typename OutT, bool GELU, int CTAS, int STATS, int LN>
static int launch_variant(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mo, const CUtensorMap& mr, const CUtensorMap& mae,
                          const CUtensorMap& mbe, const EpilogueArgs<OutT>& epi, int64_t M, int64_t N, int64_t K, int op_dtype, int64_t groups,
                          int* status_word, cudaStream_t stream) {
  using C = Cfg<CTAS>;
  static std::atomic<bool> attr_set[kMaxDevices];  // kernel attributes are per device
  const int slot = device_slot();
  if (slot < 0) return B200_ERR_CUDA;
  if (!attr_set[slot].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(gemm_tn_kernel<OutT, GELU, CTAS, STATS, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return B200_ERR_CUDA;
    attr_set[slot].store(true, std::memory_order_release);
  }
  const uint32_t idesc = make_idesc(op_dtype == B200_BF16 ? 1 : 0, BM * CTAS);
  LaunchSetup ls(dim3((unsigned)(groups * CTAS)), dim3(NUM_THREADS), C::SMEM_BYTES, stream, CTAS);
  // column panel: about 16 MB of B (panel_n * 256 rows of K 16-bit elements), at least 8 tiles
  int panel_n = (int)(16e6 / ((double)BN * (double)K * 2.0));
  if (panel_n < 8) panel_n = 8;
  cudaError_t e = cudaLaunchKernelEx(&ls.cfg, gemm_tn_kernel<OutT, GELU, CTAS, STATS, LN>, ma, mb, mo, mr, mae, mbe, epi, M, N, K, idesc, panel_n, status_word);
  note_launches(1);
  return status_from_cuda(e);
}

// What a LayerNorm-aware launch adds to the plain arguments (see EpilogueArgs).
struct LnArgs {
  const float2* stats = nullptr;  // consumer: (mean, rstd) of A's rows
  const void* a_ext = nullptr;    // consumer: [M, kLnExtCols] row extension (write_ln_ext), 16-bit of the operand type
  const void* b_ext = nullptr;    // consumer: [N, kLnExtCols] weight extension (fold_layernorm_kernel)
  float2* stats_out = nullptr;  // producer: per-slice row moments of the output
  int64_t stats_out_ld = 0;
};


// kind::f16 instruction descriptor of the narrow-tile kernel: M = 128, N = 64.
static constexpr uint32_t make_idesc_narrow(int ab_format) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)(NARROW_BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

template <typename OutT, bool GELU, int LN>
static int launch_narrow(const void* a, const void* b, const EpilogueArgs<OutT>& epi, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int op_dtype, const LnArgs& ln, int* status_word, cudaStream_t stream) {
  if constexpr (sizeof(OutT) != 2) {
    return B200_ERR_UNSUPPORTED;
  } else {
    static std::atomic<bool> attr_set[kMaxDevices];
    const int slot = device_slot();
    if (slot < 0) return B200_ERR_CUDA;
    if (!attr_set[slot].load(std::memory_order_acquire)) {
      if (cudaFuncSetAttribute(gemm_narrow_kernel<OutT, GELU, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, NARROW_SMEM_BYTES) != cudaSuccess)
        return B200_ERR_CUDA;
      attr_set[slot].store(true, std::memory_order_release);
    }
    CUtensorMap ma, mb, mae, mbe;
    memset(&mae, 0, sizeof(mae));
    memset(&mbe, 0, sizeof(mbe));
    int st = make_map(&ma, a, M, K, lda, BM, op_dtype);
    if (st == B200_OK) st = make_map(&mb, b, N, K, ldb, NARROW_BN, op_dtype);
    if (st == B200_OK && LN == 1) st = make_map(&mae, ln.a_ext, M, kLnExtCols, kLnExtCols, BM, op_dtype);
    if (st == B200_OK && LN == 1) st = make_map(&mbe, ln.b_ext, N, kLnExtCols, kLnExtCols, NARROW_BN, op_dtype);
    if (st != B200_OK) return st;
    LaunchSetup ls(dim3((unsigned)((N + NARROW_BN - 1) / NARROW_BN), (unsigned)((M + BM - 1) / BM)), dim3(NARROW_THREADS), NARROW_SMEM_BYTES, stream);
    const cudaError_t e = cudaLaunchKernelEx(&ls.cfg, gemm_narrow_kernel<OutT, GELU, LN>, ma, mb, mae, mbe, epi, M, N, K,
                                             make_idesc_narrow(op_dtype == B200_BF16 ? 1 : 0), status_word);
    note_launches(1);
    return status_from_cuda(e);
  }
}

// Whether a product goes to the narrow-tile kernel: few rows, 16-bit output, vector-aligned output and residual.
template <typename OutT, int STATS>
static bool takes_narrow_tiles(int64_t M, const void* out, int64_t ld_out, const void* residual, int64_t ld_res) {
  return STATS == 0 && sizeof(OutT) == 2 && M <= kNarrowMaxRows && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ld_out % 8 == 0 &&
         (!residual || ((reinterpret_cast<uintptr_t>(residual) & 15) == 0 && ld_res % 8 == 0));
}

template <typename OutT, bool GELU, int STATS, int LN = 0>
static int launch_typed(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N, int64_t K,
                        int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, const ArgmaxPartials& am, int* status_word,
                        cudaStream_t stream, const int64_t* targets = nullptr, float* target_val = nullptr, const LnArgs& ln = LnArgs()) {
  EpilogueArgs<OutT> epi{(const OutT*)bias, (const OutT*)residual, (OutT*)out, ld_res, ld_out, 0, am.val, am.idx, am.sum, am.ld, targets, target_val, 0,
                         ln.stats, ln.stats_out, ln.stats_out_ld};
  if constexpr (STATS == 0) {
    if (takes_narrow_tiles<OutT, STATS>(M, out, ld_out, residual, ld_res)) return launch_narrow<OutT, GELU, LN>(a, b, epi, M, N, K, lda, ldb, op_dtype, ln, status_word, stream);
  }
  CUtensorMap mo, mr;
  memset(&mo, 0, sizeof(mo));
  memset(&mr, 0, sizeof(mr));
  // TMA epilogue: 16-bit output (and residual, if any) with 16-byte aligned base and pitch
  if (STATS != 3 && sizeof(OutT) == 2 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && ld_out % 8 == 0 &&
      (!residual || ((reinterpret_cast<uintptr_t>(residual) & 15) == 0 && ld_res % 8 == 0)) &&
      make_out_map(&mo, out, M, N, ld_out, DType<OutT>::code) == B200_OK &&
      (!residual || make_out_map(&mr, const_cast<void*>(residual), M, N, ld_res, DType<OutT>::code) == B200_OK))
    epi.tma_store = 1;
  if (LN != 0 && !epi.tma_store) return B200_ERR_UNSUPPORTED;  // the LayerNorm-aware epilogues exist on the staged 16-bit path only
  epi.stream_out = epi.tma_store && (double)N * (double)K * 2.0 >= 32e6 && (double)M * (double)N * sizeof(OutT) >= 512e6;
  const int64_t n_tiles = (N + BN - 1) / BN;
  const int pairs = M > BM ? max_pairs<OutT, GELU, STATS, LN>() : 0;
  CUtensorMap ma, mb, mae, mbe;
  memset(&mae, 0, sizeof(mae));
  memset(&mbe, 0, sizeof(mbe));
  int st = make_map(&ma, a, M, K, lda, BM, op_dtype);
  if (st != B200_OK) return st;
  if (LN == 1) {
    st = make_map(&mae, ln.a_ext, M, kLnExtCols, kLnExtCols, BM, op_dtype);
    if (st != B200_OK) return st;
  }
  if (pairs > 0) {
    st = make_map(&mb, b, N, K, ldb, Cfg<2>::B_ROWS, op_dtype);
    if (st == B200_OK && LN == 1) st = make_map(&mbe, ln.b_ext, N, kLnExtCols, kLnExtCols, Cfg<2>::B_ROWS, op_dtype);
    if (st != B200_OK) return st;
    const int64_t tiles = ((M + Cfg<2>::TILE_M - 1) / Cfg<2>::TILE_M) * n_tiles;
    return launch_variant<OutT, GELU, 2, STATS, LN>(ma, mb, mo, mr, mae, mbe, epi, M, N, K, op_dtype, tiles < pairs ? tiles : pairs, status_word, stream);
  }
  st = make_map(&mb, b, N, K, ldb, Cfg<1>::B_ROWS, op_dtype);
  if (st == B200_OK && LN == 1) st = make_map(&mbe, ln.b_ext, N, kLnExtCols, kLnExtCols, Cfg<1>::B_ROWS, op_dtype);
  if (st != B200_OK) return st;
  const int64_t tiles = ((M + BM - 1) / BM) * n_tiles;
  const int64_t sms = sm_count();
  return launch_variant<OutT, GELU, 1, STATS, LN>(ma, mb, mo, mr, mae, mbe, epi, M, N, K, op_dtype, tiles < sms ? tiles : sms, status_word, stream);
}

}  // namespace gemm

// Row argmax (and optionally the row log-sum-exp) from the per-slice partials the GEMM epilogue wrote.  A block
// covers 32 rows with 8 threads per row: thread (x, y) walks slices y, y + 8, ... of row x (32 consecutive rows of
// one slice are one 128-byte line), then the 8 partial results of a row are merged through shared memory.  Strict
// '>' within a thread and the lower column on equal values across threads keep the lowest column among equal maxima.
// A partial's column is either exact (>= 0) or -(c0 + 1): "somewhere in the 32 stored columns starting at c0"; for the
// row's winner that chunk of the stored product is read back and its first column equal to the maximum taken.
constexpr int kReduceRows = 32, kReduceSplit = 8;
__device__ __forceinline__ int partial_column(int enc) { return enc < 0 ? -enc - 1 : enc; }
__global__ void __launch_bounds__(kReduceRows * kReduceSplit)
argmax_reduce_kernel(const float* __restrict__ val, const int* __restrict__ idx, const float* __restrict__ sum, int64_t ld, int slices,
                     int64_t M, int64_t* __restrict__ out, float* __restrict__ lse_out, const void* __restrict__ product, int64_t ld_product,
                     int product_is_bf16, int64_t N) {
  __shared__ float s_val[kReduceSplit][kReduceRows];
  __shared__ int s_idx[kReduceSplit][kReduceRows];
  __shared__ float s_sum[kReduceSplit][kReduceRows];
  const int x = threadIdx.x & (kReduceRows - 1), y = threadIdx.x / kReduceRows;
  const int64_t row = (int64_t)blockIdx.x * kReduceRows + x;
  pdl_launch_dependents();
  pdl_wait();
  float best = -INFINITY, total = 0.f;
  int where = 0x7fffffff;
  if (row < M) {
    for (int s = y; s < slices; s += kReduceSplit) {
      const float v = val[(int64_t)s * ld + row];
      if (v > best) {
        if (sum) total *= __expf(best - v);  // re-base what was summed so far (0 * exp(-inf) = 0 the first time)
        best = v, where = idx[(int64_t)s * ld + row];
      }
      if (sum && v > -INFINITY) total += sum[(int64_t)s * ld + row] * __expf(v - best);
    }
  }
  s_val[y][x] = best, s_idx[y][x] = where, s_sum[y][x] = total;
  __syncthreads();
  if (y == 0 && row < M) {
#pragma unroll
    for (int k = 1; k < kReduceSplit; ++k) {
      const float v = s_val[k][x];
      const int w = s_idx[k][x];
      const float t = s_sum[k][x];
      if (v > best || (v == best && w != 0x7fffffff && (where == 0x7fffffff || partial_column(w) < partial_column(where)))) {
        total = total * (best > -INFINITY ? __expf(best - v) : 0.f) + t;
        best = v, where = w;
      } else if (v > -INFINITY) {
        total += t * __expf(v - best);
      }
    }
    if (where == 0x7fffffff) {
      where = 0;
    } else if (where < 0) {
      const int c0 = -where - 1;
      where = c0;
      if (product) {
        for (int i = 0; i < 32 && c0 + i < N; ++i) {
          const float pv = product_is_bf16 ? to_float(static_cast<const __nv_bfloat16*>(product)[row * ld_product + c0 + i])
                                           : to_float(static_cast<const __half*>(product)[row * ld_product + c0 + i]);
          if (pv == best) {
            where = c0 + i;
            break;
          }
        }
      }
    }
    out[row] = where;
    if (lse_out) lse_out[row] = best + logf(total);
  }
}

static int launch_argmax_reduce(const float* val, const int* idx, const float* sum, int64_t ld, int slices, int64_t M, int64_t* out, float* lse_out,
                                const void* product, int64_t ld_product, int product_dtype, int64_t N, cudaStream_t stream) {
  LaunchSetup ls(dim3((unsigned)((M + kReduceRows - 1) / kReduceRows)), dim3(kReduceRows * kReduceSplit), 0, stream);
  const int is_bf16 = product_dtype == B200_BF16;
  if (product_dtype == B200_F32) product = nullptr;  // fp32 products never defer the column
  const cudaError_t e = cudaLaunchKernelEx(&ls.cfg, argmax_reduce_kernel, val, idx, sum, ld, slices, M, out, lse_out, product, ld_product, is_bf16, N);
  note_launches(1);
  return status_from_cuda(e);
}

// Merges the per-slice (mean, centred sum of squares) pairs a LN == 2 epilogue wrote into one (mean, rstd) per row:
// mean = sum_s n_s mean_s / n,  M2 = sum_s M2_s + sum_s n_s (mean_s - mean)^2  (every term non-negative: no
// cancellation),  rstd = 1 / sqrt(M2 / n + eps); also writes the row's extension for a consuming GEMM.  One thread per
// row; the slices of 32 consecutive rows are consecutive in memory.
template <typename T>
__global__ void __launch_bounds__(256)
ln_stats_from_moments_kernel(const float2* __restrict__ moments, int64_t ld, int slices, int slice_cols, int cols, float eps, int64_t M,
                             float2* __restrict__ stats, T* __restrict__ ext) {
  const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const bool active = row < M;  // (no early return: the whole warp takes part in the shuffles below)
  const int64_t rrow = active ? row : M - 1;
  float wsum = 0.f;
  for (int s = 0; s < slices; ++s) wsum = fmaf((float)min(slice_cols, cols - s * slice_cols), moments[(int64_t)s * ld + rrow].x, wsum);
  const float mean = wsum / (float)cols;
  float m2 = 0.f;
  for (int s = 0; s < slices; ++s) {
    const float2 part = moments[(int64_t)s * ld + rrow];
    const float d = part.x - mean;
    m2 += fmaf((float)min(slice_cols, cols - s * slice_cols) * d, d, part.y);
  }
  const float sd = sqrtf(m2 / (float)cols + eps);
  if (active) stats[row] = make_float2(mean, 1.0f / sd);
  if (ext) {
    // The extensions of a warp's 32 consecutive rows are 4 KB of consecutive memory (16 meaningful bytes and 112
    // zero bytes per row): written as 8 fully coalesced 512-byte warp stores, the heads fetched by shuffle.
    const uint4 head = ln_ext_head<T>(mean, sd);
    const int lane = threadIdx.x & 31;
    const int64_t warp_row0 = row - lane;
    uint4* dst = reinterpret_cast<uint4*>(ext + warp_row0 * kLnExtCols);
    constexpr int kChunksPerRow = kLnExtCols * 2 / 16;  // 8
#pragma unroll
    for (int i = 0; i < kChunksPerRow; ++i) {
      const int chunk = i * 32 + lane;          // 16-byte chunk of the warp's 4 KB
      const int src = chunk / kChunksPerRow;    // the row (lane) it belongs to
      uint4 v;
      v.x = __shfl_sync(0xffffffffu, head.x, src);
      v.y = __shfl_sync(0xffffffffu, head.y, src);
      v.z = __shfl_sync(0xffffffffu, head.z, src);
      v.w = __shfl_sync(0xffffffffu, head.w, src);
      if (chunk % kChunksPerRow != 0) v = make_uint4(0u, 0u, 0u, 0u);
      if (warp_row0 + src < M) dst[chunk] = v;
    }
  }
}

size_t gemm_ln_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  const int64_t slices = (N + gemm::NARROW_BN - 1) / gemm::NARROW_BN;  // (the narrow-tile kernel's slices; the wide kernel uses every other one)
  return (size_t)(slices * ((M + 63) / 64 * 64)) * 8;
}

// GEMM with a LayerNorm on either side of it (16-bit data, staged epilogue only):
//  * consumer (ln_stats != NULL): A holds raw rows x whose LayerNorm is folded into this GEMM: ln_stats[row] =
//    (mean, rstd) of x's rows and a_ext [M, kLnExtCols] their extension (both written by one of the statistics
//    producers), B holds the weights already multiplied by the LayerNorm weight and b_ext [N, kLnExtCols] their
//    extension (both written by fold_layernorm_kernel); `bias` is not used (it is inside b_ext);
//  * producer (stats_out != NULL): plain GEMM that also leaves stats_out[row] = (mean, rstd over N columns, with eps)
//    and ext_out [M, kLnExtCols] of the rows it stores, for a following consumer; `workspace`
//    (gemm_ln_workspace_bytes) holds the per-slice moments.
int launch_gemm_ln(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                   int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype, int add_gelu, const float* ln_stats,
                   const void* a_ext, const void* b_ext, float* stats_out, void* ext_out, float eps, void* workspace, size_t workspace_bytes,
                   int* status_word, cudaStream_t stream) {
  using namespace gemm;
  if (M == 0 || N == 0) return B200_OK;
  if (K < 1 || M < 0 || N < 0) return B200_ERR_BAD_ARGUMENT;
  if (op_dtype != B200_F16 && op_dtype != B200_BF16) return B200_ERR_BAD_ARGUMENT;
  if (io_dtype != B200_F16 && io_dtype != B200_BF16) return B200_ERR_UNSUPPORTED;
  if (!a || !b || !out) return B200_ERR_BAD_ARGUMENT;
  if ((ln_stats != nullptr) == (stats_out != nullptr)) return B200_ERR_BAD_ARGUMENT;  // exactly one of the two roles per launch
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || lda % 8 || ldb % 8 || lda < K || ldb < K)
    return B200_ERR_ALIGNMENT;
  if (ld_out < N || (residual && ld_res < N)) return B200_ERR_BAD_ARGUMENT;
  if (M > 0x7fffffffLL - 256 || N > 0x7fffffffLL - 256 || K > 0x7fffffffLL - 64) return B200_ERR_BAD_ARGUMENT;
  LnArgs ln;
  if (op_dtype != io_dtype) return B200_ERR_UNSUPPORTED;  // the extensions are written in the storage type and fed to the tensor cores as they are
  if (ln_stats) {
    if (!a_ext || !b_ext || (reinterpret_cast<uintptr_t>(ln_stats) & 7) || (reinterpret_cast<uintptr_t>(a_ext) & 15) ||
        (reinterpret_cast<uintptr_t>(b_ext) & 15))
      return B200_ERR_BAD_ARGUMENT;
    ln.stats = reinterpret_cast<const float2*>(ln_stats), ln.a_ext = a_ext, ln.b_ext = b_ext;
  } else {
    if (add_gelu || !ext_out || (reinterpret_cast<uintptr_t>(stats_out) & 7) || (reinterpret_cast<uintptr_t>(ext_out) & 15)) return B200_ERR_BAD_ARGUMENT;
    if (!workspace || workspace_bytes < gemm_ln_workspace_bytes(M, N) || (reinterpret_cast<uintptr_t>(workspace) & 15)) return B200_ERR_WORKSPACE;
    ln.stats_out = reinterpret_cast<float2*>(workspace), ln.stats_out_ld = (M + 63) / 64 * 64;
  }
  const ArgmaxPartials none{nullptr, nullptr, nullptr, 0};
  int st;
#define B200_GEMM_LN_DISPATCH(T)                                                                                                                 \
  st = ln_stats ? (add_gelu ? launch_typed<T, true, 0, 1>(a, b, nullptr, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, none, status_word, \
                                                          stream, nullptr, nullptr, ln)                                                          \
                            : launch_typed<T, false, 0, 1>(a, b, nullptr, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, none, status_word, \
                                                           stream, nullptr, nullptr, ln))                                                        \
                : launch_typed<T, false, 0, 2>(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, none, status_word, stream, \
                                               nullptr, nullptr, ln)
  if (io_dtype == B200_F16) B200_GEMM_LN_DISPATCH(__half);
  else B200_GEMM_LN_DISPATCH(__nv_bfloat16);
#undef B200_GEMM_LN_DISPATCH
  if (st != B200_OK || !stats_out) return st;
  // width of the column slices whose moments the GEMM left: the wide kernel's epilogue warps cover EPI_COLS columns, a
  // narrow tile NARROW_BN
  const bool narrow = io_dtype == B200_F16 ? takes_narrow_tiles<__half, 0>(M, out, ld_out, residual, ld_res)
                                           : takes_narrow_tiles<__nv_bfloat16, 0>(M, out, ld_out, residual, ld_res);
  const int slice_cols = narrow ? NARROW_BN : EPI_COLS;
  const int slices = (int)((N + slice_cols - 1) / slice_cols);
  LaunchSetup ls(dim3((unsigned)((M + 255) / 256)), dim3(256), 0, stream);
  const cudaError_t e =
      io_dtype == B200_F16
          ? cudaLaunchKernelEx(&ls.cfg, ln_stats_from_moments_kernel<__half>, (const float2*)ln.stats_out, ln.stats_out_ld, slices, slice_cols,
                               (int)N, eps, M, reinterpret_cast<float2*>(stats_out), static_cast<__half*>(ext_out))
          : cudaLaunchKernelEx(&ls.cfg, ln_stats_from_moments_kernel<__nv_bfloat16>, (const float2*)ln.stats_out, ln.stats_out_ld, slices,
                               slice_cols, (int)N, eps, M, reinterpret_cast<float2*>(stats_out), static_cast<__nv_bfloat16*>(ext_out));
  note_launches(1);
  return status_from_cuda(e);
}

int launch_gemm(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                int add_gelu, int* status_word, cudaStream_t stream) {
  return launch_gemm_argmax(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, io_dtype, add_gelu, nullptr, nullptr,
                            nullptr, 0, status_word, stream);
}

size_t gemm_argmax_workspace_bytes(int64_t M, int64_t N) {
  if (M <= 0 || N <= 0) return 0;
  const int64_t slices = (N + gemm::BN - 1) / gemm::BN * (gemm::BN / gemm::EPI_COLS);
  const int64_t ld = (M + 63) / 64 * 64;
  return (size_t)(slices * ld) * 12;  // maximum, column, sum of exponentials
}

int launch_gemm_argmax(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                       int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                       int add_gelu, int64_t* argmax_out, float* lse_out, void* workspace, size_t workspace_bytes, int* status_word,
                       cudaStream_t stream) {
  using namespace gemm;
  ArgmaxPartials am{nullptr, nullptr, nullptr, 0};
  if (argmax_out) {
    const size_t need = gemm_argmax_workspace_bytes(M, N);
    if (need > 0 && (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))) return B200_ERR_WORKSPACE;
    am.ld = (M + 63) / 64 * 64;
    const int64_t slices = (N + BN - 1) / BN * (BN / EPI_COLS);
    am.val = static_cast<float*>(workspace);
    am.idx = reinterpret_cast<int*>(am.val + slices * am.ld);
    if (lse_out) am.sum = am.val + 2 * slices * am.ld;
  }
  if (M == 0 || N == 0) return B200_OK;
  if (K < 1 || M < 0 || N < 0) return B200_ERR_BAD_ARGUMENT;
  if (op_dtype != B200_F16 && op_dtype != B200_BF16) return B200_ERR_BAD_ARGUMENT;
  if (!a || !b || !out) return B200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || lda % 8 || ldb % 8 || lda < K || ldb < K)
    return B200_ERR_ALIGNMENT;
  if (ld_out < N || (residual && ld_res < N)) return B200_ERR_BAD_ARGUMENT;
  if (M > 0x7fffffffLL - 256 || N > 0x7fffffffLL - 256 || K > 0x7fffffffLL - 64) return B200_ERR_BAD_ARGUMENT;
  if (argmax_out && add_gelu) return B200_ERR_UNSUPPORTED;  // row statistics are built for the plain and residual epilogues only
  int st = B200_ERR_BAD_ARGUMENT;
#define B200_GEMM_DISPATCH(T)                                                                                                              \
  st = (argmax_out && lse_out) ? launch_typed<T, false, 2>(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, am, status_word, stream) \
       : argmax_out ? launch_typed<T, false, 1>(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, am, status_word, stream)  \
       : add_gelu ? launch_typed<T, true, 0>(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, am, status_word, stream)  \
                  : launch_typed<T, false, 0>(a, b, bias, residual, out, M, N, K, lda, ldb, ld_res, ld_out, op_dtype, am, status_word, stream)
  switch (io_dtype) {
    case B200_F32: B200_GEMM_DISPATCH(float); break;
    case B200_F16: B200_GEMM_DISPATCH(__half); break;
    case B200_BF16: B200_GEMM_DISPATCH(__nv_bfloat16); break;
  }
#undef B200_GEMM_DISPATCH
  if (st != B200_OK || !argmax_out) return st;
  const int64_t slices = (N + BN - 1) / BN * (BN / EPI_COLS);
  return launch_argmax_reduce(am.val, am.idx, am.sum, am.ld, (int)slices, M, argmax_out, lse_out, out, ld_out, io_dtype, N, stream);
}

// Row statistics of A B^T (+ bias) without storing the product: argmax, log-sum-exp and, optionally, the value at a
// per-row target column, all taken from the values as they would be rounded to `round_dtype` (fp16 or bf16).
int launch_gemm_rowstats(const void* a, const void* b, const void* bias, int64_t M, int64_t N, int64_t K, int64_t lda, int64_t ldb,
                         int op_dtype, int round_dtype, const int64_t* targets, int64_t* argmax_out, float* lse_out, float* target_out,
                         void* workspace, size_t workspace_bytes, int* status_word, cudaStream_t stream) {
  using namespace gemm;
  if (!argmax_out || (targets != nullptr) != (target_out != nullptr)) return B200_ERR_BAD_ARGUMENT;
  if (K < 1 || M < 0 || N < 0) return B200_ERR_BAD_ARGUMENT;
  if (M == 0 || N == 0) return B200_OK;
  if (op_dtype != B200_F16 && op_dtype != B200_BF16) return B200_ERR_BAD_ARGUMENT;
  if (round_dtype != B200_F16 && round_dtype != B200_BF16) return B200_ERR_UNSUPPORTED;
  if (!a || !b) return B200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || lda % 8 || ldb % 8 || lda < K || ldb < K)
    return B200_ERR_ALIGNMENT;
  if (M > 0x7fffffffLL - 256 || N > 0x7fffffffLL - 256 || K > 0x7fffffffLL - 64) return B200_ERR_BAD_ARGUMENT;
  const size_t need = gemm_argmax_workspace_bytes(M, N);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15)) return B200_ERR_WORKSPACE;
  ArgmaxPartials am;
  am.ld = (M + 63) / 64 * 64;
  const int64_t slices = (N + BN - 1) / BN * (BN / EPI_COLS);
  am.val = static_cast<float*>(workspace);
  am.idx = reinterpret_cast<int*>(am.val + slices * am.ld);
  am.sum = lse_out ? am.val + 2 * slices * am.ld : nullptr;
  int st;
  if (round_dtype == B200_F16)
    st = launch_typed<__half, false, 3>(a, b, bias, nullptr, nullptr, M, N, K, lda, ldb, 0, N, op_dtype, am, status_word, stream, targets, target_out);
  else
    st = launch_typed<__nv_bfloat16, false, 3>(a, b, bias, nullptr, nullptr, M, N, K, lda, ldb, 0, N, op_dtype, am, status_word, stream, targets, target_out);
  if (st != B200_OK) return st;
  return launch_argmax_reduce(am.val, am.idx, am.sum, am.ld, (int)slices, M, argmax_out, lse_out, nullptr, 0, round_dtype, N, stream);
}

}  // namespace b200
