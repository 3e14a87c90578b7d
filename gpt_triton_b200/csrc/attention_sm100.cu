// Causal flash attention on the 5th-generation tensor cores, head size 64, fp16 or bf16 storage.
// bf16 Q and K feed S = Q K^T as they are (exact products).  P is fp16 for both storage types, as in the
// reference, and both operands of one MMA must have the same format, so a bf16 V tile is converted to
// fp16 in place (exact in fp16's normal range) by the softmax warps before P V.
//
// Work item = up to 128 query rows of one (batch, head); a ragged sequence length puts its short tile first
// (see decode_item).  Persistent CTAs (two per SM) walk the items, longest first.  Per CTA:
//   warp 0      TMA producer: the 128x64 Q tile (double-buffered) and, per 64-key block, the K and V tiles
//               (3-stage ring), all 128-byte swizzled, straight out of the strided q/k/v views (4-D tensor
//               maps: head_dim, row, head, batch); every CTA issues its own loads
//   warp 1      tcgen05.mma issuer: S = Q K^T (128x64, fp32, tensor memory, double-buffered, issued one
//               block ahead) and O (+)= P V, which accumulates in tensor memory over the key blocks of an item
//   warps 2-9   softmax: TWO threads per query row (warps w and w + 4 own the same 32 rows; each takes 32 of the
//               block's 64 keys and 32 of the 64 output columns).  A thread loads its 32 scores from tensor memory
//               ONCE and keeps them in registers for both the block maximum and the exponentials (S is handed
//               back to the tensor cores as soon as the load has landed); the two halves of a row exchange their
//               block maxima through shared memory; running maximum/denominator in fp32; P = exp(s - max)
//               rounded to fp16 goes into shared memory in the swizzled K-major operand layout and, when the
//               running maximum of any row of the warp moved, the warp rescales its 32 rows x 32 columns of O in
//               tensor memory (load, multiply, store) before P V of the block is issued:
//               o = o * exp(m_old - m_new) + P V.
// The output row never lives in registers across blocks, and a softmax thread makes two round trips to tensor
// memory per block (scores; output rescale).  The work of a row is serial in its thread (exponentials at one warp
// instruction per 8 cycles on the special-function unit, dependent arithmetic, barrier hand-offs); two threads per
// row halve that chain and double the warps the SM can interleave.
// The softmax runs over 64-key blocks with P rounded relative to the running maximum of each
// block, which is the arithmetic of the reference's flash_attention_v1 kernel (kernels.py:417-474
// of the reference); blocks above the diagonal are skipped.  Every mbarrier wait is bounded.
#include <atomic>

#include "sm100_primitives.cuh"

namespace b200 {
namespace attn100 {

using namespace sm100;

constexpr int D = 64;
constexpr int BLOCK_M = 128;
constexpr int BLOCK_N = 64;
constexpr int KV_STAGES = 3;
constexpr int Q_BYTES = BLOCK_M * D * 2;        // 16 KB
constexpr int KV_TILE_BYTES = BLOCK_N * D * 2;  // 8 KB each for K and V
constexpr int KV_STAGE_BYTES = 2 * KV_TILE_BYTES;
constexpr int P_BYTES = BLOCK_M * BLOCK_N * 2;  // 16 KB
constexpr int NUM_SOFTMAX_WARPS = 8;  // two threads per query row: warps w and w + 4 share a 32-row quarter, 32 keys each
constexpr int NUM_THREADS = 32 * (2 + NUM_SOFTMAX_WARPS);
constexpr int CTAS_PER_SM = 2;
constexpr int TMEM_COLS = 256;  // S[2] (64 columns each) + O (64 columns); allocations are powers of two
constexpr int CTRL_BYTES = 256;
constexpr int XCHG_BYTES = 3 * 2 * BLOCK_M * 4;  // [slot][half][row]: block maximum / row sum of each half of a row, for its partner thread
constexpr int SMEM_BYTES = 2 * Q_BYTES + KV_STAGES * KV_STAGE_BYTES + P_BYTES + 1024 + CTRL_BYTES + XCHG_BYTES;

struct Params {
  void* out;
  int64_t so_b, so_h, so_l;
  int B, NH, L;
  float scale_log2e;  // softmax scale times log2(e)
  int out_vec32;      // output rows may be written with 32-byte stores
  int q_head_inner, k_head_inner, v_head_inner;  // tensor map dimension order is {D, head, row, batch} instead of {D, row, head, batch}
  int* status_word;
};

// K-major operand, 128-byte swizzle (rows of 128 bytes, 8-row groups of 1024 bytes).
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// MN-major operand, 128-byte swizzle: 64 contiguous MN elements per 128-byte row, 8 K-rows per 1024-byte
// group; groups along K are `stride byte offset` apart, 64-wide MN chunks `leading byte offset` apart
// (one chunk only here).  This is how a [keys, head_dim] V tile serves as the B operand of P V.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: fp32 accumulator, M = 128, N = 64.
__host__ __device__ constexpr uint32_t idesc(int a_fmt, int b_fmt, int b_mn_major) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(BLOCK_N >> 3) << 17) |
         ((uint32_t)(BLOCK_M >> 4) << 24);
}

struct Item {
  int b, h, q0, q_end, nblk;
};
// Query rows [0, L) are cut into n_qt = ceil(L / 128) tiles of at most 128 rows whose ENDS are as early as they can be:
// tile i ends at min(L, round_up(L - 128 * (n_qt - 1 - i), 64)) and starts where tile i - 1 ends.  A tile costs one
// 64-key block per 64 rows up to its end, so a ragged L puts its short tile first, where the causal rows are
// shortest (L = 300: rows [0,64) [64,192) [192,300) = 1 + 3 + 5 key blocks, where [0,128) [128,256) [256,300) would
// take 2 + 4 + 5); starts stay multiples of 64, so only the last two key blocks of a tile need per-element masks.
// A tile always loads 128 rows of Q; rows at or beyond its end are computed and dropped.
// Items ordered by decreasing row-tile index (the longest causal rows first), then (batch, head).
__device__ __forceinline__ int tile_end(int i, int n_qt, int L) {
  const int e = (L - BLOCK_M * (n_qt - 1 - i) + BLOCK_N - 1) / BLOCK_N * BLOCK_N;
  return min(L, e);
}
__device__ __forceinline__ Item decode_item(int64_t idx, int bh_total, int n_qt, int NH, int L) {
  const int qt = n_qt - 1 - (int)(idx / bh_total);
  const int bh = (int)(idx % bh_total);
  Item it;
  it.b = bh / NH;
  it.h = bh % NH;
  it.q0 = qt == 0 ? 0 : tile_end(qt - 1, n_qt, L);
  it.q_end = tile_end(qt, n_qt, L);
  it.nblk = (it.q_end - 1) / BLOCK_N + 1;
  return it;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t (&v)[4]) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
template <typename T>
__device__ __forceinline__ uint32_t pack_out(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack_out<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack_out<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]),
        "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <typename T>
__global__ void __launch_bounds__(NUM_THREADS, CTAS_PER_SM)
attention_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, Params p, uint32_t idesc_s, uint32_t idesc_pv) {
  constexpr bool IS_FP16 = DType<T>::code == B200_F16;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t smem_q = base;                                  // [2][128][64]
  const uint32_t smem_kv = smem_q + 2 * Q_BYTES;                 // [KV_STAGES]{K[64][64], V[64][64]}
  const uint32_t smem_p = smem_kv + KV_STAGES * KV_STAGE_BYTES;  // [128][64] fp16
  uint8_t* ctrl = smem + 2 * Q_BYTES + KV_STAGES * KV_STAGE_BYTES + P_BYTES;
  const uint32_t bars = smem_u32(ctrl);
  const uint32_t bar_q_full = bars;                             // [2] Q tile of an item has landed
  const uint32_t bar_q_empty = bars + 16;                       // [2] every S of the item has been computed: the buffer may be overwritten
  const uint32_t bar_kv_full = bars + 32;                       // [KV_STAGES]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * KV_STAGES;    // [KV_STAGES]
  const uint32_t bar_s_full = bar_kv_empty + 8 * KV_STAGES;     // [2] S of a block is in tensor memory
  const uint32_t bar_s_empty = bar_s_full + 16;                 // [2] the four softmax warps hold its scores in registers
  const uint32_t bar_p_full = bar_s_empty + 16;                 // P of a block is in shared memory and O has been rescaled
  const uint32_t bar_pv_done = bar_p_full + 8;                  // P V of a block has been accumulated: P is free, O is current
  const uint32_t bar_pair = bar_pv_done + 8;                    // [4] the two warps that share a 32-row quarter have published their halves
  constexpr int BAR_BYTES = 32 + 16 * KV_STAGES + 32 + 16 + 32;
  static_assert(BAR_BYTES + 16 <= CTRL_BYTES, "control block too small");
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + BAR_BYTES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + BAR_BYTES + 8);
  float* xchg = reinterpret_cast<float*>(ctrl + CTRL_BYTES);  // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.L + BLOCK_M - 1) / BLOCK_M;
  const int bh_total = p.B * p.NH;
  const int64_t n_items = (int64_t)n_qt * bh_total;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + 8 * i, 1);
      mbar_init(bar_q_empty + 8 * i, 1);
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_s_empty + 8 * i, NUM_SOFTMAX_WARPS);
    }
    for (int i = 0; i < KV_STAGES; ++i) {
      mbar_init(bar_kv_full + 8 * i, 1);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    mbar_init(bar_p_full, NUM_SOFTMAX_WARPS);
    mbar_init(bar_pv_done, 1);
    for (int i = 0; i < 4; ++i) mbar_init(bar_pair + 8 * i, 2);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // set-up done (own shared and tensor memory only); global memory from here on
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t tmem_s = tmem_base;                // S[buf]: columns [64 * buf, 64 * buf + 64)
  const uint32_t tmem_o = tmem_base + 2 * BLOCK_N;  // O: columns [128, 192)

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t qi = 0, ki = 0;
      bool alive = true;
      for (int64_t idx = blockIdx.x; idx < n_items && alive; idx += gridDim.x) {
        const Item it = decode_item(idx, bh_total, n_qt, p.NH, p.L);
        const uint32_t qb = qi & 1;
        if (!mbar_wait(bar_q_empty + 8 * qb, ((qi >> 1) & 1) ^ 1u, abort_flag, p.status_word, 11)) break;
        mbar_arrive_expect_tx(bar_q_full + 8 * qb, Q_BYTES);
        tma_load_4d(smem_q + qb * Q_BYTES, &map_q, bar_q_full + 8 * qb, 0, p.q_head_inner ? it.h : it.q0, p.q_head_inner ? it.q0 : it.h, it.b);
        ++qi;
        for (int j = 0; j < it.nblk; ++j) {
          const uint32_t st = ki % KV_STAGES;
          if (!mbar_wait(bar_kv_empty + 8 * st, ((ki / KV_STAGES) & 1) ^ 1u, abort_flag, p.status_word, 12)) {
            alive = false;
            break;
          }
          mbar_arrive_expect_tx(bar_kv_full + 8 * st, KV_STAGE_BYTES);
          tma_load_4d(smem_kv + st * KV_STAGE_BYTES, &map_k, bar_kv_full + 8 * st, 0, p.k_head_inner ? it.h : j * BLOCK_N, p.k_head_inner ? j * BLOCK_N : it.h, it.b);
          tma_load_4d(smem_kv + st * KV_STAGE_BYTES + KV_TILE_BYTES, &map_v, bar_kv_full + 8 * st, 0, p.v_head_inner ? it.h : j * BLOCK_N, p.v_head_inner ? j * BLOCK_N : it.h, it.b);
          ++ki;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      uint32_t qi = 0, ks = 0, kp = 0, si = 0, pi = 0;
      bool alive = true;
      // S_next = Q . K^T into S[si & 1]: needs the block's K/V stage and that buffer's previous scores to be in registers
      auto issue_s = [&](uint32_t qb) -> bool {
        const uint32_t st = ks % KV_STAGES;
        if (!mbar_wait(bar_kv_full + 8 * st, (ks / KV_STAGES) & 1, abort_flag, p.status_word, 13)) return false;
        const uint32_t sb = si & 1;
        if (!mbar_wait(bar_s_empty + 8 * sb, ((si >> 1) & 1) ^ 1u, abort_flag, p.status_word, 14)) return false;
        tc_fence_after();
        const uint64_t da = desc_kmajor(smem_q + qb * Q_BYTES);
        const uint64_t db = desc_kmajor(smem_kv + st * KV_STAGE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) umma_f16(tmem_s + sb * BLOCK_N, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc_s, (uint32_t)(k != 0));
        umma_commit(bar_s_full + 8 * sb);
        ++si;
        ++ks;
        return true;
      };
      for (int64_t idx = blockIdx.x; idx < n_items && alive; idx += gridDim.x) {
        const Item it = decode_item(idx, bh_total, n_qt, p.NH, p.L);
        const uint32_t qb = qi & 1;
        if (!mbar_wait(bar_q_full + 8 * qb, (qi >> 1) & 1, abort_flag, p.status_word, 15)) break;
        if (!issue_s(qb)) break;
        for (int j = 0; j < it.nblk; ++j) {
          if (j + 1 < it.nblk) {
            if (!issue_s(qb)) {
              alive = false;
              break;
            }
          } else {
            umma_commit(bar_q_empty + 8 * qb);  // every S of this item is issued: Q is free once they finish
          }
          // O (+)= P_j . V_j : P written, O rescaled (and, for bf16 storage, V converted) by the softmax warps
          const uint32_t st = kp % KV_STAGES;
          if (!mbar_wait(bar_p_full, pi & 1, abort_flag, p.status_word, 16)) {
            alive = false;
            break;
          }
          tc_fence_after();
          const uint64_t da = desc_kmajor(smem_p);
          const uint64_t db = desc_mnmajor(smem_kv + st * KV_STAGE_BYTES + KV_TILE_BYTES);
#pragma unroll
          for (int k = 0; k < BLOCK_N / 16; ++k) {
            // A: +16 keys = +32 bytes inside the swizzled row; B: +16 keys = two 8-key groups = +2048 bytes
            umma_f16(tmem_o, da + (uint64_t)(2 * k), db + (uint64_t)(128 * k), idesc_pv, (uint32_t)((j | k) != 0));
          }
          umma_commit(bar_pv_done);
          umma_commit(bar_kv_empty + 8 * st);
          ++pi;
          ++kp;
        }
        ++qi;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warps: two threads per query row
    const int quarter = warp & 3;               // tensor-memory lanes [32 * quarter, +32) are this warp's rows
    const int half = (warp - 2) >> 2;           // which 32 of a block's 64 keys / of the 64 output columns
    const int r_in_tile = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t p_row = smem_p + (uint32_t)r_in_tile * 128u;
    const uint32_t sw = (uint32_t)(r_in_tile & 7);
    const uint32_t o_addr = tmem_o + lane_addr + (uint32_t)(half * 32);
    // Exchange between the two threads of a row: slot layout [3][2][128] floats.  Block exchanges alternate between
    // slots 0 and 1 (a thread can only be one exchange ahead of its partner), the end-of-item exchange uses slot 2.
    float* my_x = xchg + half * BLOCK_M + r_in_tile;
    const float* partner_x = xchg + (half ^ 1) * BLOCK_M + r_in_tile;
    const uint32_t my_pair_bar = bar_pair + 8 * (uint32_t)quarter;
    uint32_t xphase = 0;
    // publish `val` for the partner, wait (bounded) for the partner's, return it; false when the CTA is aborting
    auto exchange = [&](int slot, float val, float& other) -> bool {
      my_x[slot * 2 * BLOCK_M] = val;
      __syncwarp();
      if (lane == 0) mbar_arrive(my_pair_bar);
      if (!mbar_wait(my_pair_bar, xphase, abort_flag, p.status_word, 22)) return false;
      xphase ^= 1u;
      other = partner_x[slot * 2 * BLOCK_M];
      return true;
    };
    uint32_t it_count = 0;  // 64-key blocks processed so far by this CTA
    bool alive = true;
    for (int64_t idx = blockIdx.x; idx < n_items && alive; idx += gridDim.x) {
      const Item it = decode_item(idx, bh_total, n_qt, p.NH, p.L);
      const int row = it.q0 + r_in_tile;
      const int warp_row0 = it.q0 + quarter * 32;       // first query row of this warp
      const bool warp_live = warp_row0 < it.q_end;      // a warp whose 32 rows all lie beyond the tile's end only keeps the handshakes going
      float m_run = -INFINITY, l_run = 0.f;             // l_run: this thread's half of the row's denominator
      for (int j = 0; j < it.nblk; ++j, ++it_count) {
        const uint32_t sb = it_count & 1;
        if (!mbar_wait(bar_s_full + 8 * sb, (it_count >> 1) & 1, abort_flag, p.status_word, 18)) {
          alive = false;
          break;
        }
        tc_fence_after();
        const int k0 = j * BLOCK_N + half * 32;  // first key of this thread's 32
        // keys above this warp's last row are masked for the whole warp
        const bool live = warp_live && k0 <= warp_row0 + 31;
        uint32_t v[32];
        if (live) {
          tmem_ld_32x32(tmem_s + lane_addr + sb * BLOCK_N + (uint32_t)(half * 32), v);
          tmem_ld_wait();
        }
        // S[sb] is in registers: the Q K^T after next may overwrite it
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_s_empty + 8 * sb);
        // maximum of the raw scores (the scale is positive, so it commutes with max).  Per-element masking only if the
        // diagonal crosses these 32 keys for some row of this warp; masked scores become -inf here, so that the
        // exponentials below need no second test.
        float bm = -INFINITY;
        if (live) {
          if (k0 + 31 > warp_row0) {
            const int lim = row - k0;  // keys i <= lim are visible to this row
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (i > lim) v[i] = 0xff800000u;
              bm = fmaxf(bm, __uint_as_float(v[i]));
            }
          } else {
            float b1 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              bm = fmax3(bm, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
              b1 = fmax3(b1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
            }
            bm = fmaxf(bm, b1);
          }
        }
        // the row's block maximum is the larger of its two halves
        float partner_bm;
        if (!exchange((int)(it_count & 1), bm, partner_bm)) {
          alive = false;
          break;
        }
        bm = fmaxf(bm, partner_bm);
        const float m_new = fmaxf(m_run, bm * p.scale_log2e);  // running maximum, in log2 units
        const float mult = ex2f(m_run - m_new);
        m_run = m_new;
        // the previous block's P V must be complete: it read the P tile that is about to be overwritten, and it
        // produced the O that is about to be rescaled (the first block of an item finds both free: the previous
        // item's last P V was awaited before its output was stored)
        if (j > 0 && !mbar_wait(bar_pv_done, (it_count - 1) & 1, abort_flag, p.status_word, 19)) {
          alive = false;
          break;
        }
        tc_fence_after();
        // p = exp(s - max) from the registers, partial row sum in fp32, P rounded to fp16 into the swizzled operand tile
        // (a masked score is -inf: 2^-inf = 0; a row with nothing visible yet has max = -inf and is never stored)
        float psum0 = 0.f, psum1 = 0.f;
        if (live) {
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float p0 = ex2f(fmaf(__uint_as_float(v[i]), p.scale_log2e, -m_new));
            const float p1 = ex2f(fmaf(__uint_as_float(v[i + 1]), p.scale_log2e, -m_new));
            psum0 += p0;
            psum1 += p1;
            __half2 h = __floats2half2_rn(p0, p1);
            w[i / 2] = *reinterpret_cast<uint32_t*>(&h);
          }
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint32_t chunk = (uint32_t)(half * 4 + g);
            st_shared_v4(p_row + ((chunk ^ sw) << 4), w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
          }
        } else if (warp_live) {
          // masked for every row of the warp: P = 0 (rows beyond L may keep whatever is there: nothing reads their output)
#pragma unroll
          for (int g = 0; g < 4; ++g) st_shared_v4(p_row + ((((uint32_t)(half * 4 + g)) ^ sw) << 4), 0u, 0u, 0u, 0u);
        }
        if constexpr (sizeof(T) == 2 && !IS_FP16) {
          // bf16 storage: V_j -> fp16 in place, 32 bytes per softmax thread (the swizzle is address-agnostic)
          const uint32_t vaddr = smem_kv + (it_count % KV_STAGES) * KV_STAGE_BYTES + KV_TILE_BYTES + (uint32_t)(threadIdx.x - 64) * 32u;
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            uint32_t w4[4];
            ld_shared_v4(vaddr + g * 16, w4);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f2 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w4[i]));
              const __half2 h2 = __floats2half2_rn(f2.x, f2.y);
              w4[i] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            st_shared_v4(vaddr + g * 16, w4[0], w4[1], w4[2], w4[3]);
          }
        }
        // o = o * exp(m_old - m_new) in tensor memory, for this warp's 32 rows x 32 columns, unless no row's maximum moved
        if (j > 0 && warp_live && __any_sync(0xffffffffu, mult != 1.0f)) {
          uint32_t a[32];
          tmem_ld_32x32(o_addr, a);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * mult);
          tmem_st_32x32(o_addr, a);
          tmem_st_wait();
        }
        // P (and, for bf16, the converted V) is complete, O is rescaled: P V of this block may be issued
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_p_full);
        l_run = l_run * mult + (psum0 + psum1);
      }
      if (!alive) break;
      // the row's denominator is the sum of its two halves (the same rescale factors went into both)
      float partner_l;
      if (!exchange(2, l_run, partner_l)) break;
      const float l_row = l_run + partner_l;
      // the last block's P V, then normalise and store this thread's 32 output columns of the row
      if (!mbar_wait(bar_pv_done, (it_count - 1) & 1, abort_flag, p.status_word, 21)) break;
      tc_fence_after();
      if (warp_live) {  // (warp-uniform: the tensor-memory load below is a warp-wide instruction)
        const float inv = 1.0f / l_row;
        T* dst = reinterpret_cast<T*>(p.out) + (int64_t)it.b * p.so_b + (int64_t)it.h * p.so_h + (int64_t)row * p.so_l + half * 32;
        uint32_t a[32];
        tmem_ld_32x32(o_addr, a);
        tmem_ld_wait();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = pack_out<T>(__uint_as_float(a[2 * i]) * inv, __uint_as_float(a[2 * i + 1]) * inv);
        if (row < it.q_end) {
          if (p.out_vec32) {
            st_global_v8(dst, &w[0]);
            st_global_v8(dst + 16, &w[8]);
          } else {
#pragma unroll
            for (int g = 0; g < 4; ++g) *reinterpret_cast<uint4*>(dst + g * 8) = make_uint4(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3]);
          }
        }
      }
      // (this warp's reads of O are ordered before its next arrival on bar_p_full, which is what lets the next
      // item's first P V overwrite O)
      tc_fence_before();
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
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// 4-D map over a strided (batch, head, row) view with contiguous head_dim.  The two middle dimensions are
// ordered by ascending stride ({D, row, head, batch} for contiguous [B, NH, L, D] tensors, {D, head, row, batch}
// for views into a fused [B, L, 3*NH*D] projection); *head_inner tells the kernel which order was used.
static int make_map(CUtensorMap* map, const void* ptr, int64_t B, int64_t NH, int64_t L, const int64_t* s, int box_rows, int dtype,
                    int* head_inner) {
  *head_inner = s[1] < s[2];
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)L, (uint64_t)NH, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)s[2] * 2, (uint64_t)s[1] * 2, (uint64_t)s[0] * 2};
  uint32_t box[4] = {(uint32_t)D, (uint32_t)box_rows, 1, 1};
  if (*head_inner) {
    dims[1] = (uint64_t)NH, dims[2] = (uint64_t)L;
    strides[0] = (uint64_t)s[1] * 2, strides[1] = (uint64_t)s[2] * 2;
    box[1] = 1, box[2] = (uint32_t)box_rows;
  }
  return encode_tensor_map(map, ptr, 4, dims, strides, box, dtype, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
}

static bool view_ok(const void* ptr, const int64_t* s, int64_t B, int64_t NH) {
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return false;
  // TMA wants 16-byte multiples for every stride; a stride of a size-1 dimension is never used but must still encode
  for (int i = 0; i < 3; ++i)
    if (s[i] % 8 != 0 || s[i] <= 0 || (uint64_t)s[i] * 2 >= (1ull << 40)) return false;
  (void)B;
  (void)NH;
  return true;
}

}  // namespace attn100

// Returns B200_ERR_UNSUPPORTED when the problem does not fit this kernel (the caller then takes the generic one).
int launch_attention_sm100(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L, int64_t Dh,
                           const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, float scale, int in_dtype,
                           int out_dtype, int* status_word, cudaStream_t stream) {
  using namespace attn100;
  if (Dh != D || in_dtype != out_dtype || (in_dtype != B200_F16 && in_dtype != B200_BF16)) return B200_ERR_UNSUPPORTED;
  if (!view_ok(q, qs, B, NH) || !view_ok(k, ks, B, NH) || !view_ok(v, vs, B, NH) || !view_ok(out, os, B, NH)) return B200_ERR_UNSUPPORTED;
  if (B * NH > 0x7fffffffLL || L > 0x7fffff00LL || B > 0x7fffffffLL) return B200_ERR_UNSUPPORTED;
  CUtensorMap mq, mk, mv;
  Params p;
  int st = make_map(&mq, q, B, NH, L, qs, BLOCK_M, in_dtype, &p.q_head_inner);
  if (st == B200_OK) st = make_map(&mk, k, B, NH, L, ks, BLOCK_N, in_dtype, &p.k_head_inner);
  if (st == B200_OK) st = make_map(&mv, v, B, NH, L, vs, BLOCK_N, in_dtype, &p.v_head_inner);
  if (st != B200_OK) return B200_ERR_UNSUPPORTED;  // e.g. strides the tensor map cannot express
  static std::atomic<bool> attr_set[kMaxDevices];  // kernel attributes are per device
  const int slot = device_slot();
  if (slot < 0) return B200_ERR_CUDA;
  if (!attr_set[slot].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attention_sm100_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(attention_sm100_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return B200_ERR_CUDA;
    attr_set[slot].store(true, std::memory_order_release);
  }
  p.out = out;
  p.so_b = os[0], p.so_h = os[1], p.so_l = os[2];
  p.B = (int)B, p.NH = (int)NH, p.L = (int)L;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.out_vec32 = (reinterpret_cast<uintptr_t>(out) & 31) == 0 && os[0] % 16 == 0 && os[1] % 16 == 0 && os[2] % 16 == 0;
  p.status_word = status_word;
  const int64_t n_items = ((L + BLOCK_M - 1) / BLOCK_M) * B * NH;
  int64_t grid = (int64_t)sm_count() * CTAS_PER_SM;
  if (grid > n_items) grid = n_items;
  // S = Q K^T in the storage format; P V always fp16 x fp16 (see the top of this file)
  LaunchSetup ls(dim3((unsigned)grid), dim3(NUM_THREADS), SMEM_BYTES, stream);
  const cudaError_t e = in_dtype == B200_BF16
                            ? cudaLaunchKernelEx(&ls.cfg, attention_sm100_kernel<__nv_bfloat16>, mq, mk, mv, p, idesc(1, 1, 0), idesc(0, 0, 1))
                            : cudaLaunchKernelEx(&ls.cfg, attention_sm100_kernel<__half>, mq, mk, mv, p, idesc(0, 0, 0), idesc(0, 0, 1));
  note_launches(1);
  return status_from_cuda(e);
}

}  // namespace b200
