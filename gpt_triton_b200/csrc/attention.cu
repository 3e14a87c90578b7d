// Causal attention with online softmax over 64-key blocks (fp16 operands, fp32 statistics): the
// generic kernel (any storage type, head size 16..256, any alignment) on mma.sync tensor-core
// instructions.  fp16 tensors with head size 64 are routed to the tcgen05/TMA kernel instead.
//
// One CTA = 64 query rows of one (batch, head); 4 warps x 16 rows.  Q, K, V are read through
// (batch, head, row) element strides, so the fused [tokens, 3*hidden] output of the c_attn
// projection is consumed in place and the result is written straight into [batch, seq, hidden].
// Inputs of any storage type are rounded to fp16 when staged in shared memory, P is rounded to
// fp16 relative to the running maximum of each 64-key block and the running maximum and
// denominator are fp32 -- the arithmetic of the reference's flash_attention_v1 kernel.  Key
// blocks that the causal mask removes entirely are skipped (they contribute exact zeros).
#include <atomic>

#include "common.cuh"

namespace b200 {
namespace attn {

constexpr int BLOCK = 64;  // query rows per CTA == keys per block
constexpr int NUM_WARPS = 4;
constexpr int PAD = 8;  // halves of padding per shared-memory row (keeps ldmatrix conflict-free)

struct Strides {
  int64_t b, h, l;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// exp for the softmax: correctly-rounded-ish expf when the storage type is fp32 (the 1e-4 parity
// path: a fast exp flips too many fp16 roundings of P), the ex2-based intrinsic otherwise.
template <typename TIn>
__device__ __forceinline__ float softmax_exp(float x) {
  if constexpr (sizeof(TIn) == 4) {
    return expf(x);
  } else {
    return __expf(x);
  }
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Stage rows [row0, row0+64) x D of one (batch, head) slice into shared memory as fp16; rows >= L are zero.
template <int D, typename TIn>
__device__ __forceinline__ void stage_tile(__half* dst, const TIn* src, int64_t row_stride, int row0, int L, bool vec) {
  constexpr int LDS = D + PAD;
  constexpr int VPR = D / 8;  // 8-element vectors per row
  for (int i = threadIdx.x; i < BLOCK * VPR; i += NUM_WARPS * 32) {
    const int r = i / VPR, c = (i % VPR) * 8;
    float f[8];
    if (row0 + r < L) {
      const TIn* p = src + (int64_t)(row0 + r) * row_stride + c;
      if (vec) {
        load8(p, f);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = to_float(p[j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
    store8(dst + r * LDS + c, f);
  }
}

template <int D, typename TIn, typename TOut>
__global__ void __launch_bounds__(NUM_WARPS * 32)
attention_kernel(const TIn* __restrict__ q, const TIn* __restrict__ k, const TIn* __restrict__ v, TOut* __restrict__ out,
                 int NH, int L, Strides sq, Strides sk, Strides sv, Strides so, float scale, int vec_in, int vec_out) {
  constexpr int LDS = D + PAD;
  constexpr bool Q_IN_REGS = D <= 64;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __half* sQ = reinterpret_cast<__half*>(smem_raw);
  __half* sK = sQ + BLOCK * LDS;
  __half* sV = sK + BLOCK * LDS;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;
  const int n_qblocks = (L + BLOCK - 1) / BLOCK;
  const int qb = n_qblocks - 1 - (int)blockIdx.x;  // longest rows first
  const int bh = blockIdx.y;
  const int b = bh / NH, h = bh % NH;
  const TIn* qp = q + (int64_t)b * sq.b + (int64_t)h * sq.h;
  const TIn* kp = k + (int64_t)b * sk.b + (int64_t)h * sk.h;
  const TIn* vp = v + (int64_t)b * sv.b + (int64_t)h * sv.h;
  const int q0 = qb * BLOCK;

  stage_tile<D, TIn>(sQ, qp, sq.l, q0, L, vec_in);
  __syncthreads();

  const uint32_t sQ_u = (uint32_t)__cvta_generic_to_shared(sQ);
  const uint32_t sK_u = (uint32_t)__cvta_generic_to_shared(sK);
  const uint32_t sV_u = (uint32_t)__cvta_generic_to_shared(sV);
  // per-lane ldmatrix offsets (bytes)
  const uint32_t q_off = (uint32_t)(((warp * 16 + (lane & 15)) * LDS + (lane >> 4) * 8) * 2);
  const uint32_t k_off = (uint32_t)((((lane & 7) + ((lane >> 4) << 3)) * LDS + ((lane >> 3) & 1) * 8) * 2);
  const uint32_t v_off = (uint32_t)((((lane & 7) + ((lane >> 3) & 1) * 8) * LDS + (lane >> 4) * 8) * 2);

  uint32_t qf[Q_IN_REGS ? D / 16 : 1][4];
  if constexpr (Q_IN_REGS) {
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], sQ_u + q_off + ks * 32);
  }

  float o[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int row_g[2] = {q0 + warp * 16 + g, q0 + warp * 16 + g + 8};

  for (int kb = 0; kb <= qb; ++kb) {
    const int k0 = kb * BLOCK;
    __syncthreads();  // previous block's K/V fully consumed
    stage_tile<D, TIn>(sK, kp, sk.l, k0, L, vec_in);
    stage_tile<D, TIn>(sV, vp, sv.l, k0, L, vec_in);
    __syncthreads();

    // S = Q K^T  (16 rows x 64 keys per warp)
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a[4];
      if constexpr (Q_IN_REGS) {
        a[0] = qf[ks][0], a[1] = qf[ks][1], a[2] = qf[ks][2], a[3] = qf[ks][3];
      } else {
        ldmatrix_x4(a, sQ_u + q_off + ks * 32);
      }
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t bfr[4];
        ldmatrix_x4(bfr, sK_u + k_off + (uint32_t)((np * 16 * LDS + ks * 16) * 2));
        mma_16816(s[2 * np], a, bfr[0], bfr[1]);
        mma_16816(s[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }

    // scale, causal mask, block maximum
    float bm[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + nt * 8 + t4 * 2 + (e & 1);
        const int r = e >> 1;
        float x = s[nt][e] * scale;
        x = (row_g[r] >= key) ? x : -INFINITY;
        s[nt][e] = x;
        bm[r] = fmaxf(bm[r], x);
      }
    }
    float mult[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 1));
      bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 2));
      const float m_new = fmaxf(m_run[r], bm[r]);
      mult[r] = softmax_exp<TIn>(m_run[r] - m_new);
      m_run[r] = m_new;
    }
    float psum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const float p = softmax_exp<TIn>(s[nt][e] - m_run[r]);
        s[nt][e] = p;
        psum[r] += p;
      }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 1);
      psum[r] += __shfl_xor_sync(0xffffffffu, psum[r], 2);
      l_run[r] = l_run[r] * mult[r] + psum[r];
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o[i][0] *= mult[0], o[i][1] *= mult[0];
      o[i][2] *= mult[1], o[i][3] *= mult[1];
    }

    // O += P V   (P rounded to fp16)
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_half2(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_half2(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_half2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_half2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        uint32_t bfr[4];
        ldmatrix_x4_trans(bfr, sV_u + v_off + (uint32_t)((kk * 16 * LDS + dp * 16) * 2));
        mma_16816(o[2 * dp], a, bfr[0], bfr[1]);
        mma_16816(o[2 * dp + 1], a, bfr[2], bfr[3]);
      }
    }
  }

  // normalise, stage the 64 x D tile in shared memory, then store rows with wide accesses
  __syncthreads();
  constexpr int LDO = D + (sizeof(TOut) == 4 ? 4 : 8);
  TOut* sO = reinterpret_cast<TOut*>(smem_raw);
  const float inv_l[2] = {1.0f / l_run[0], 1.0f / l_run[1]};
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      TOut* p = sO + (warp * 16 + g + r * 8) * LDO + i * 8 + t4 * 2;
      p[0] = from_float<TOut>(o[i][2 * r] * inv_l[r]);
      p[1] = from_float<TOut>(o[i][2 * r + 1] * inv_l[r]);
    }
  }
  __syncthreads();
  TOut* op = out + (int64_t)b * so.b + (int64_t)h * so.h;
  constexpr int VPR = D / 8;
  for (int i = threadIdx.x; i < BLOCK * VPR; i += NUM_WARPS * 32) {
    const int r = i / VPR, c = (i % VPR) * 8;
    if (q0 + r < L) {
      TOut* dst = op + (int64_t)(q0 + r) * so.l + c;
      const TOut* src = sO + r * LDO + c;
      if (vec_out) {
        if (sizeof(TOut) == 4) {
          *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
          *reinterpret_cast<float4*>(dst + 4) = *reinterpret_cast<const float4*>(src + 4);
        } else {
          *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) dst[j] = src[j];
      }
    }
  }
}

template <int D>
constexpr size_t smem_bytes() {
  size_t in = (size_t)3 * BLOCK * (D + PAD) * 2;
  size_t o = (size_t)BLOCK * (D + 4) * 4;
  return in > o ? in : o;
}

template <int D, typename TIn, typename TOut>
static int launch_typed(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L,
                        Strides sq, Strides sk, Strides sv, Strides so, float scale, cudaStream_t stream) {
  constexpr size_t smem = smem_bytes<D>();
  static std::atomic<bool> attr_set[kMaxDevices];  // kernel attributes are per device
  const int slot = device_slot();
  if (slot < 0) return B200_ERR_CUDA;
  if (smem > 48 * 1024 && !attr_set[slot].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(attention_kernel<D, TIn, TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return B200_ERR_CUDA;
    attr_set[slot].store(true, std::memory_order_release);
  }
  auto ok_in = [](const void* p, const Strides& s) {
    const int64_t m = sizeof(TIn) == 4 ? 4 : 8;
    return (reinterpret_cast<uintptr_t>(p) & 15) == 0 && s.b % m == 0 && s.h % m == 0 && s.l % m == 0;
  };
  const int vec_in = ok_in(q, sq) && ok_in(k, sk) && ok_in(v, sv);
  const int64_t mo = sizeof(TOut) == 4 ? 4 : 8;
  const int vec_out = (reinterpret_cast<uintptr_t>(out) & 15) == 0 && so.b % mo == 0 && so.h % mo == 0 && so.l % mo == 0;
  const int64_t n_qblocks = (L + BLOCK - 1) / BLOCK;
  const int64_t bh = B * NH;
  if (bh > 65535) {
    // fold very large batch*head counts into several launches of whole batches
    const int64_t b_per = 65535 / NH;
    if (b_per < 1) return B200_ERR_BAD_ARGUMENT;
    for (int64_t b0 = 0; b0 < B; b0 += b_per) {
      const int64_t nb = (B - b0 < b_per) ? B - b0 : b_per;
      int st = launch_typed<D, TIn, TOut>((const TIn*)q + b0 * sq.b, (const TIn*)k + b0 * sk.b, (const TIn*)v + b0 * sv.b,
                                          (TOut*)out + b0 * so.b, nb, NH, L, sq, sk, sv, so, scale, stream);
      if (st != B200_OK) return st;
    }
    return B200_OK;
  }
  dim3 grid((unsigned)n_qblocks, (unsigned)bh);
  attention_kernel<D, TIn, TOut><<<grid, NUM_WARPS * 32, smem, stream>>>((const TIn*)q, (const TIn*)k, (const TIn*)v, (TOut*)out, (int)NH,
                                                                        (int)L, sq, sk, sv, so, scale, vec_in, vec_out);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

template <typename TIn, typename TOut>
static int dispatch_d(int64_t D, const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L,
                      Strides sq, Strides sk, Strides sv, Strides so, float scale, cudaStream_t stream) {
  switch (D) {
    case 16: return launch_typed<16, TIn, TOut>(q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
    case 32: return launch_typed<32, TIn, TOut>(q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
    case 64: return launch_typed<64, TIn, TOut>(q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
    case 128: return launch_typed<128, TIn, TOut>(q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
    case 256: return launch_typed<256, TIn, TOut>(q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
  }
  return B200_ERR_BAD_ARGUMENT;
}

}  // namespace attn

int launch_attention(const void* q, const void* k, const void* v, void* out, int64_t B, int64_t NH, int64_t L,
                     int64_t D, const int64_t* qs, const int64_t* ks, const int64_t* vs, const int64_t* os, float scale,
                     int in_dtype, int out_dtype, int* status_word, cudaStream_t stream) {
  using namespace attn;
  if (B == 0 || NH == 0 || L == 0) return B200_OK;
  if (L > 0x7fffffffLL - BLOCK) return B200_ERR_BAD_ARGUMENT;
  {
    // tensor-core path for the shapes it covers; everything else takes the generic kernel below
    const int st = launch_attention_sm100(q, k, v, out, B, NH, L, D, qs, ks, vs, os, scale, in_dtype, out_dtype, status_word, stream);
    if (st != B200_ERR_UNSUPPORTED) return st;
  }
  Strides sq{qs[0], qs[1], qs[2]}, sk{ks[0], ks[1], ks[2]}, sv{vs[0], vs[1], vs[2]}, so{os[0], os[1], os[2]};
  if (in_dtype == B200_F32 && out_dtype == B200_F32) return dispatch_d<float, float>(D, q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
  if (in_dtype == B200_F32 && out_dtype == B200_F16) return dispatch_d<float, __half>(D, q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
  if (in_dtype == B200_F16 && out_dtype == B200_F16) return dispatch_d<__half, __half>(D, q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
  if (in_dtype == B200_BF16 && out_dtype == B200_BF16) return dispatch_d<__nv_bfloat16, __nv_bfloat16>(D, q, k, v, out, B, NH, L, sq, sk, sv, so, scale, stream);
  return B200_ERR_BAD_ARGUMENT;
}

}  // namespace b200
