// Bounded-wait probe: the primitive every cross-GPU wait in this library is built on, exposed on
// its own so that its time-out path can be exercised without a failing peer.  One warp spins on a
// device-visible counter with ld.acquire.sys until it reaches `target` or `limit_ns` elapse; the
// outcome (0 = reached, 5 = gave up) goes to `status` and, on a time-out, to the library error word.
// The kernel always returns by itself, the context stays usable.
#include "../kernels/common.cuh"

namespace {
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t target, unsigned long long limit_ns, int* status, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x != 0) return;
  const uint64_t t0 = kh_globaltimer();
  int st = 5;
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - target) >= 0) { st = 0; break; }
    if ((it & 15) == 15) {
      if (kh_globaltimer() - t0 > limit_ns) break;
      __nanosleep(256);
    }
  }
  *status = st;
  if (st) atomicCAS(err, 0, 5);
}
}  // namespace

extern "C" int kh_wait_probe(const void* flag, unsigned target, unsigned limit_ms, void* status, void* stream) {
  if (limit_ms > 2000) { kh_set_error("wait_probe: limit above 2000 ms"); return -1; }
  KH_LAUNCH(wait_probe_kernel, 1, 32, 0, (cudaStream_t)stream, (const uint32_t*)flag, target, (unsigned long long)limit_ms * 1000000ull,
                                                       (int*)status, kh_error_word_dev());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { kh_set_error("wait_probe: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}
