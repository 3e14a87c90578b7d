// out[M,N] = [gelu](A[M,K] . B[N,K]^T + bias) + residual  on the 5th-generation tensor cores.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer: 128x64 tile of A and 256x64 tile of B per stage, 128-byte swizzle,
//               completion by mbarrier transaction bytes (no multicast anywhere)
//   warp 1      allocates the 512 tensor-memory columns and issues tcgen05.mma (one thread);
//               tcgen05.commit releases smem stages and publishes finished accumulators
//   warps 2-5   epilogue: tcgen05.ld the 128x256 fp32 accumulator (one row per thread),
//               bias -> GELU -> residual -> cast -> global store
// Two 128x256 accumulators (2 x 256 columns) let the epilogue of tile i overlap the main
// loop of tile i+1.  Every wait on an mbarrier is bounded; a wait that gives up raises a
// CTA-wide abort flag, reports through status_word and the kernel drains and exits.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace b200 {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 x 2 bytes = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int B_STAGE_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int NUM_EPI_WARPS = 4;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;  // row tiles per raster group (keeps a group's A rows and B columns L2-resident)
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about one second

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (this wait or another one timed out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status_word, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
      *abort_flag = 1;
      if (status_word) atomicCAS(status_word, 0, where);
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]^T, 128 x 256 x 16, issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// mbarrier arrives once all tcgen05.mma issued so far by this thread have completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

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

// Epilogue for one thread's 32 consecutive columns of one row.
template <typename OutT, bool GELU>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&acc)[32], const EpilogueArgs<OutT>& e, int64_t row, int col0,
                                               int64_t M, int64_t N, bool vec_ok) {
  if (row >= M || col0 >= N) return;
  const bool full = col0 + 32 <= N;
  OutT* orow = e.out + row * e.ld_out + col0;
  const OutT* rrow = e.residual ? e.residual + row * e.ld_res + col0 : nullptr;
  const OutT* brow = e.bias ? e.bias + col0 : nullptr;
  if (full && vec_ok) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(acc[g * 8 + j]);
      if (brow) {
        float b[8];
        load8(brow + g * 8, b);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += b[j];
      }
      if (GELU) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = gelu_new(f[j]);
      }
      if (rrow) {
        float r[8];
        load8(rrow + g * 8, r);
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] += r[j];
      }
      store8(orow + g * 8, f);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      if (col0 + j < N) {
        float f = __uint_as_float(acc[j]);
        if (brow) f += to_float(brow[j]);
        if (GELU) f = gelu_new(f);
        if (rrow) f += to_float(rrow[j]);
        orow[j] = from_float<OutT>(f);
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
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);  // full[S], empty[S], acc_full[2], acc_empty[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_acc_full = bar_empty + 8 * STAGES;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 8 * (2 * STAGES + 4));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 8 * (2 * STAGES + 4) + 8);

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
    const int quarter = warp & 3;  // a warp may only touch tensor-memory lanes [32*(warp%4), +32)
    int acc = 0;
    uint32_t acc_phase = 0;
    const int esz = (int)sizeof(OutT);
    const bool vec_ok = aligned16(epi.out) && (epi.ld_out * esz) % 16 == 0 &&
                        (!epi.residual || (aligned16(epi.residual) && (epi.ld_res * esz) % 16 == 0)) &&
                        (!epi.bias || aligned16(epi.bias));
    for (int64_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const TileCoord tc = tile_coord(t, m_tiles, n_tiles);
      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, abort_flag, status_word, 4)) break;
      tc_fence_after();
      const int64_t row = (int64_t)tc.m * BM + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(taddr + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        epilogue_chunk<OutT, GELU>(v, epi, row, tc.n * BN + c * 32, M, N, vec_ok);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_acc_empty + 8 * acc);
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

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
