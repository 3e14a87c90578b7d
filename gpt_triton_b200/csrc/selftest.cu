// Self-test of the bounded mbarrier wait: one warp waits, with the routine every tensor-core kernel of this
// library uses, on a barrier whose phase nothing ever completes.  The wait gives up after the given number of
// clock cycles, the status word receives B200_ERR_DEVICE_WAIT and the kernel returns normally.
#include "sm100_primitives.cuh"

namespace b200 {

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int* status_word, long long limit_cycles) {
  __shared__ __align__(8) uint64_t barrier;
  __shared__ int abort_word;
  const uint32_t bar = sm100::smem_u32(&barrier);
  if (threadIdx.x == 0) {
    sm100::mbar_init(bar, 1);  // one arrival expected; none will come
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  // every lane waits, as the epilogue and softmax warps of the real kernels do; `where` is the status code to report
  const bool completed = sm100::mbar_wait(bar, 0, &abort_word, status_word, B200_ERR_DEVICE_WAIT, limit_cycles);
  if (completed && threadIdx.x == 0) atomicCAS(status_word, 0, -1);  // cannot happen: would mean the barrier completed by itself
}

int launch_bounded_wait_selftest(int* status_word, int64_t limit_cycles, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status_word, (long long)limit_cycles);
  note_launches(1);
  return status_from_cuda(cudaGetLastError());
}

}  // namespace b200
