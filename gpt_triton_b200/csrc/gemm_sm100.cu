// out[M,N] = [gelu](A[M,K] . B[N,K]^T + bias) + residual  on the 5th-generation tensor cores.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 128x64 tile of A and 256x64 tile of B per stage, 128-byte swizzle,
//               completion by mbarrier transaction bytes (no multicast anywhere)
//   warp 1      allocates the 512 tensor-memory columns and issues tcgen05.mma (one thread);
//               tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-9   epilogue: tcgen05.ld the 128x256 fp32 accumulator (one row per thread, each warp
//               128 of the 256 columns), bias -> GELU -> residual -> cast -> global store.  The
//               residual rows are fetched into registers and the bias into shared memory before
//               the accumulator is awaited, so their latency hides behind the main loop.
// Two 128x256 accumulators (2 x 256 columns) let the epilogue of tile i overlap the main
// loop of tile i+1.  Every wait on an mbarrier is bounded; a wait that gives up raises a
// CTA-wide abort flag, reports through status_word and the kernel drains and exits.
#include "sm100_primitives.cuh"

namespace b200 {
namespace gemm {

using namespace sm100;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_EPI_WARPS = 8;
constexpr int NUM_THREADS = 32 * (2 + NUM_EPI_WARPS);
constexpr int EPI_COLS = BN / (NUM_EPI_WARPS / 4);  // columns per epilogue warp
constexpr int EPI_CHUNKS = EPI_COLS / 32;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;  // row tiles per raster group (keeps a group's A rows and B columns L2-resident)
constexpr int CTRL_BYTES = 256;  // mbarriers, tensor-memory base, abort flag
constexpr int BIAS_BYTES = 2 * BN * 4;  // bias of the current and the next tile, as fp32
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + CTRL_BYTES + BIAS_BYTES;

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
// Instruction descriptor for kind::f16: D fp32, A/B fp16 (0) or bf16 (1), both K-major, M=128, N=256.
__host__ __device__ constexpr uint32_t make_idesc(int ab_format) {
  return (1u << 4) | ((uint32_t)ab_format << 7) | ((uint32_t)ab_format << 10) | ((uint32_t)(BN >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}

struct TileCoord {
  int m, n;
};
// Raster: groups of GROUP_M row tiles; inside a group the row tile varies fastest, so the CTAs
// that run at the same time share a few B column tiles and GROUP_M A row tiles in L2.
__device__ __forceinline__ TileCoord tile_coord(int64_t t, int m_tiles, int n_tiles) {
  const int64_t per_group = (int64_t)GROUP_M * n_tiles;
  const int group = (int)(t / per_group);
  const int within = (int)(t - (int64_t)group * per_group);
  const int m_first = group * GROUP_M;
  const int gm = min(GROUP_M, m_tiles - m_first);
  TileCoord c;
  c.m = m_first + within % gm;
  c.n = within / gm;
  return c;
}

template <typename OutT>
struct EpilogueArgs {
  const OutT* bias;
  const OutT* residual;
  OutT* out;
  int64_t ld_res, ld_out;
};

// x * sigmoid(2y), y = sqrt(2/pi) (x + 0.044715 x^3): algebraically the reference's
// 0.5 x (1 + tanh(y)) with tanh(y) = 2 sigmoid(2y) - 1 (kernels.py:15-26 of the reference),
// evaluated with one ex2 and one reciprocal on the special-function unit.
__device__ __forceinline__ float gelu_fast(float x) {
  const float c0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;  // -2 sqrt(2/pi) log2(e)
  const float c1 = c0 * 0.044715f;
  const float z = x * fmaf(x * x, c1, c0);
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(z));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
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

// How a thread may store its 32-column pieces of an output row.
enum StoreMode { STORE_SCALAR = 0, STORE_16B = 1, STORE_32B = 2 };

// Residual of one thread's row for its warp's EPI_COLS columns, fetched ahead of the accumulator.
// Only used on the wide path with a 16-bit output type: EPI_COLS halves = EPI_COLS/8 uint4.
struct ResidualRegs {
  uint4 v[EPI_COLS / 8];
};

// One thread, one row, 32 consecutive columns starting at col0: acc (+bias) -> GELU -> (+residual) -> store.
// `bias_s` points at this chunk's 32 fp32 bias values in shared memory (zeros when there is no bias).
template <typename OutT, bool GELU>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&acc)[32], const float* bias_s, const EpilogueArgs<OutT>& e,
                                               const uint4* res_regs, int64_t row, int col0, int64_t N, int mode) {
  float f[32];
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    const float4 b = *reinterpret_cast<const float4*>(bias_s + j);
    f[j] = __uint_as_float(acc[j]) + b.x;
    f[j + 1] = __uint_as_float(acc[j + 1]) + b.y;
    f[j + 2] = __uint_as_float(acc[j + 2]) + b.z;
    f[j + 3] = __uint_as_float(acc[j + 3]) + b.w;
  }
  if (GELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = gelu_fast(f[j]);
  }
  OutT* orow = e.out + row * e.ld_out + col0;
  const bool full = col0 + 32 <= N;
  if (mode != STORE_SCALAR && full) {
    if constexpr (sizeof(OutT) == 2) {
      if (res_regs) {
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
      }
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) w[j] = pack2<OutT>(f[2 * j], f[2 * j + 1]);
      if (mode == STORE_32B) {
        st_global_v8(orow, reinterpret_cast<const uint32_t(&)[8]>(w[0]));
        st_global_v8(orow + 16, reinterpret_cast<const uint32_t(&)[8]>(w[8]));
      } else {
#pragma unroll
        for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(orow + g * 8) = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
      }
    } else {
      if (e.residual) {
        const float* rrow = reinterpret_cast<const float*>(e.residual) + row * e.ld_res + col0;
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 r = *reinterpret_cast<const float4*>(rrow + j);
          f[j] += r.x, f[j + 1] += r.y, f[j + 2] += r.z, f[j + 3] += r.w;
        }
      }
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(reinterpret_cast<float*>(orow) + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    }
  } else {
    const OutT* rrow = e.residual ? e.residual + row * e.ld_res + col0 : nullptr;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col0 + j < N) {
        float v = f[j];
        if (rrow) v += to_float(rrow[j]);
        orow[j] = from_float<OutT>(v);
      }
    }
  }
}

template <typename OutT, bool GELU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, EpilogueArgs<OutT> epi,
               int64_t M, int64_t N, int64_t K, uint32_t idesc, int* status_word) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte aligned bases.
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_a = base;
  const uint32_t smem_b = base + STAGES * A_STAGE_BYTES;
  uint8_t* ctrl = smem + STAGES * STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);  // full[S], empty[S], acc_full[2], acc_empty[2], bias_ready[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_acc_full = bar_empty + 8 * STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  const uint32_t bar_bias = bar_acc_empty + 16;
  static_assert(8 * (2 * STAGES + 6) + 16 <= CTRL_BYTES, "control block too small");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 8 * (2 * STAGES + 6));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * (2 * STAGES + 6) + 8);
  float* bias_smem = reinterpret_cast<float*>(ctrl + CTRL_BYTES);  // [2][BN]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int m_tiles = (int)((M + BM - 1) / BM);
  const int n_tiles = (int)((N + BN - 1) / BN);
  const int64_t num_tiles = (int64_t)m_tiles * n_tiles;
  const int num_kb = (int)((K + BK - 1) / BK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_acc_full + 8 * a, 1);
      mbar_init(bar_acc_empty + 8 * a, NUM_EPI_WARPS);
      mbar_init(bar_bias + 8 * a, NUM_EPI_WARPS);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool alive = true;
      for (int64_t t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, m_tiles, n_tiles);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, status_word, 1)) {
            alive = false;
            break;
          }
          mbar_arrive_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
          tma_load_2d(smem_a + stage * A_STAGE_BYTES, &map_a, bar_full + 8 * stage, kb * BK, tc.m * BM);
          tma_load_2d(smem_b + stage * B_STAGE_BYTES, &map_b, bar_full + 8 * stage, kb * BK, tc.n * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool alive = true;
      for (int64_t t = blockIdx.x; t < num_tiles && alive; t += gridDim.x) {
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, abort_flag, status_word, 2)) break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, status_word, 3)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = make_smem_desc(smem_a + stage * A_STAGE_BYTES);
          const uint64_t db = make_smem_desc(smem_b + stage * B_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance 16 elements (32 bytes) along K inside the swizzle row: +2 in 16-byte units
            umma_f16(tmem_d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (uint32_t)((kb | k) != 0));
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!alive) break;
        umma_commit(bar_acc_full + 8 * acc);
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
    for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const TileCoord tc = tile_coord(t, m_tiles, n_tiles);
      const int64_t row = (int64_t)tc.m * BM + quarter * 32 + lane;
      const int col_base = tc.n * BN + col_half * EPI_COLS;
      const bool row_ok = row < M;
      // Prefetch what does not depend on the accumulator: bias -> shared memory, residual -> registers.
      float* bias_s = bias_smem + acc * BN;
      for (int i = epi_tid; i < BN; i += 32 * NUM_EPI_WARPS) {
        const int c = tc.n * BN + i;
        bias_s[i] = (epi.bias && c < N) ? to_float(epi.bias[c]) : 0.f;
      }
      ResidualRegs res;
      const bool res_in_regs = esz == 2 && epi.residual && mode != STORE_SCALAR && row_ok;
      if (res_in_regs) {
        const OutT* rrow = epi.residual + row * epi.ld_res + col_base;
#pragma unroll
        for (int i = 0; i < EPI_COLS / 8; ++i) {
          if (col_base + (i / 4) * 32 + 32 <= N) res.v[i] = *reinterpret_cast<const uint4*>(rrow + i * 8);
        }
      }
      // bias visible to all epilogue warps (an mbarrier, not bar.sync: its wait is bounded like every other)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_bias + 8 * acc);
      if (!mbar_wait(bar_bias + 8 * acc, acc_phase, abort_flag, status_word, 5)) break;
      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, status_word, 4)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN + col_half * EPI_COLS);
#pragma unroll
      for (int c = 0; c < EPI_CHUNKS; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (c == EPI_CHUNKS - 1) {
          // accumulator fully read: hand it back to the MMA warp before doing the last chunk's math
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
        }
        const int col0 = col_base + c * 32;
        if (row_ok && col0 < N)
          epilogue_chunk<OutT, GELU>(v, bias_s + col_half * EPI_COLS + c * 32, epi, res_in_regs ? &res.v[c * 4] : nullptr, row, col0, N, mode);
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
// 2-D map over a row-major [rows, cols] 16-bit matrix with leading dimension ld; box = 64 columns x box_rows.
static int make_map(CUtensorMap* map, const void* ptr, int64_t rows, int64_t cols, int64_t ld, int box_rows, int op_dtype) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return B200_ERR_CUDA;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, op_dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200_OK : B200_ERR_CUDA;
}

template <typename OutT, bool GELU>
static int launch_typed(const CUtensorMap& ma, const CUtensorMap& mb, const void* bias, const void* residual, void* out,
                        int64_t M, int64_t N, int64_t K, int64_t ld_res, int64_t ld_out, int op_dtype, int* status_word,
                        cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tn_kernel<OutT, GELU>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return B200_ERR_CUDA;
    attr_set = true;
  }
  EpilogueArgs<OutT> epi{(const OutT*)bias, (const OutT*)residual, (OutT*)out, ld_res, ld_out};
  const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int64_t grid = sm_count();
  if (grid > tiles) grid = tiles;
  gemm_tn_kernel<OutT, GELU><<<(unsigned)grid, NUM_THREADS, SMEM_BYTES, stream>>>(ma, mb, epi, M, N, K, make_idesc(op_dtype == B200_BF16 ? 1 : 0),
                                                                                 status_word);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

}  // namespace gemm

int launch_gemm(const void* a, const void* b, const void* bias, const void* residual, void* out, int64_t M, int64_t N,
                int64_t K, int64_t lda, int64_t ldb, int64_t ld_res, int64_t ld_out, int op_dtype, int io_dtype,
                int add_gelu, int* status_word, cudaStream_t stream) {
  using namespace gemm;
  if (M == 0 || N == 0) return B200_OK;
  if (K < 1 || M < 0 || N < 0) return B200_ERR_BAD_ARGUMENT;
  if (op_dtype != B200_F16 && op_dtype != B200_BF16) return B200_ERR_BAD_ARGUMENT;
  if (!a || !b || !out) return B200_ERR_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15) || lda % 8 || ldb % 8 || lda < K || ldb < K)
    return B200_ERR_ALIGNMENT;
  if (ld_out < N || (residual && ld_res < N)) return B200_ERR_BAD_ARGUMENT;
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return B200_ERR_BAD_ARGUMENT;
  CUtensorMap ma, mb;
  int st = make_map(&ma, a, M, K, lda, BM, op_dtype);
  if (st != B200_OK) return st;
  st = make_map(&mb, b, N, K, ldb, BN, op_dtype);
  if (st != B200_OK) return st;
#define B200_GEMM_DISPATCH(T)                                                                                               \
  return add_gelu ? launch_typed<T, true>(ma, mb, bias, residual, out, M, N, K, ld_res, ld_out, op_dtype, status_word, stream) \
                  : launch_typed<T, false>(ma, mb, bias, residual, out, M, N, K, ld_res, ld_out, op_dtype, status_word, stream)
  switch (io_dtype) {
    case B200_F32: B200_GEMM_DISPATCH(float);
    case B200_F16: B200_GEMM_DISPATCH(__half);
    case B200_BF16: B200_GEMM_DISPATCH(__nv_bfloat16);
  }
#undef B200_GEMM_DISPATCH
  return B200_ERR_BAD_ARGUMENT;
}

}  // namespace b200
