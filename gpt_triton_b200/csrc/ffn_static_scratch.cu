// b200_ffn_static_scratch: the fused_ffn operator for callers that may not allocate device memory.
//
// b200_ffn needs scratch for its packed operands whenever x or w cannot be fed to the tensor cores in
// place (fp32 storage, [K, N] weights, K not a multiple of 8) and expects the caller to bring it.  Some
// callers cannot: a serving runtime that has already handed every free byte of HBM to its own pool, or an
// enqueue-style plugin callback in which cudaMalloc (and its implicit device-wide synchronisation) is off
// limits.  For them the scratch lives in the library image itself, in the file-scope array below: every
// GPU that loads the library carries B200_FFN_STATIC_SCRATCH_BYTES of it until the process exits, and no
// allocation call of any kind is made here.
#include <mutex>

#include "common.cuh"

namespace {

static __device__ __align__(256) unsigned char g_ffn_scratch[B200_FFN_STATIC_SCRATCH_BYTES];

// In host code `g_ffn_scratch` is only a handle for the runtime, not a device address; the address that
// kernels may use is obtained once per device, with that device current, from cudaGetSymbolAddress.  The
// cached address belongs to the device's primary context as it was at that first call: after a
// cudaDeviceReset in this process it is stale, and the entry point must not be called again on that device.
constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {};

int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_ffn_scratch);
    if (e != cudaSuccess || !p) return B200_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return B200_OK;
}

size_t round256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

extern "C" int b200_ffn_static_scratch(const void* x, const void* w, const void* bias, const void* residual, void* out, int64_t M,
                                       int64_t N, int64_t K, int64_t ld_out, int w_is_nk, int add_gelu, int dtype, int* status_word,
                                       void* stream) {
  if (M < 0 || N < 0 || K < 0) return B200_ERR_BAD_ARGUMENT;
  if (M == 0 || N == 0) return B200_OK;
  if (M > 0x7fffffffLL - 256 || N > 0x7fffffffLL - 256 || K > 0x7fffffffLL - 256) return B200_ERR_BAD_ARGUMENT;
  // What this very call needs, decided the way b200_ffn decides it: an operand is packed into scratch unless it can be
  // fed to the tensor cores in place (16-bit storage, K a multiple of 8, 16-byte aligned, and for w the [N, K] layout).
  // Refuse, before anything is launched, a problem whose packed operands do not fit the built-in array.
  const bool in_place_ok = dtype != B200_F32 && K % 8 == 0;
  const size_t kp = (size_t)((K + 7) / 8 * 8);
  size_t need = 0;
  if (!(in_place_ok && (reinterpret_cast<uintptr_t>(x) & 15) == 0)) need += round256((size_t)M * kp * 2);
  if (!(w_is_nk && in_place_ok && (reinterpret_cast<uintptr_t>(w) & 15) == 0)) need += round256((size_t)N * kp * 2);
  if (need > (size_t)B200_FFN_STATIC_SCRATCH_BYTES) return B200_ERR_WORKSPACE;
  void* scratch = nullptr;
  const int st = scratch_for_current_device(&scratch);
  if (st != B200_OK) return st;
  // Same kernels as b200_ffn, with the device address of the static array as their workspace.  The packing
  // kernels write every byte they later read (padding columns included), so nothing has to be cleared even
  // though the array still holds the previous call's operands.
  return b200_ffn(x, w, bias, residual, out, M, N, K, ld_out, w_is_nk, add_gelu, dtype, scratch, (size_t)B200_FFN_STATIC_SCRATCH_BYTES,
                  status_word, stream);
}
