// Pipeline-stage mailboxes over NVLink peer memory (sm_100a).
//
// The reference moves the activations and their gradients between pipeline stages with blocking
// ncclSend / ncclRecv pairs on the compute stream (src/parallel/comms.cu:58-74, src/pp_train.c:24-53):
// a send does not return before the matching receive has been posted, which ties the two stages'
// schedules together.  Here the sender PUSHES a message into a slot of the receiver's memory and
// raises the slot's counter; nothing on the sender waits for the receiver.  The receiver runs a
// one-thread kernel in stream order in front of the first consumer that waits (bounded) until the
// slot's counter has reached the expected value.
//
//   kh_p2p_put   copy `bytes` from local `src` to the peer's slot with 16-byte stores from all
//                SMs, then (last CTA, after a system-scope fence) store-release the sequence number
//                into the peer's slot counter.  The sequence number is a device word that the
//                kernel itself advances, so the launch arguments never change: the call can be part
//                of a recorded launch plan or a CUDA graph.
//   kh_p2p_wait  spin with ld.acquire.sys on the local slot counter until it reaches the next
//                expected value (also a device word advanced by the kernel).  Gives up after
//                `limit_ms`, writes code 7 to the library error word and returns; the context
//                stays usable.
//
// A slot may be rewritten only after its previous content has been consumed.  The pipeline engine
// guarantees that by construction: message i of step n+1 is produced after the producer has
// received, in step n, a message that the consumer sent after consuming message i of step n.
#include "../kernels/common.cuh"

namespace {

constexpr int PUT_THREADS = 256;
constexpr int PUT_UNROLL = 4;

__global__ void __launch_bounds__(PUT_THREADS)
p2p_put_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16, uint32_t* peer_flag, uint32_t* local) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t stride = (size_t)gridDim.x * PUT_THREADS;
  size_t i = (size_t)blockIdx.x * PUT_THREADS + threadIdx.x;
  for (; i + (PUT_UNROLL - 1) * stride < n16; i += PUT_UNROLL * stride) {
    uint4 v[PUT_UNROLL];
#pragma unroll
    for (int u = 0; u < PUT_UNROLL; u++) v[u] = __ldcs(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < PUT_UNROLL; u++) dst[i + u * stride] = v[u];
  }
  for (; i < n16; i += stride) dst[i] = __ldcs(src + i);
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    // local[0]: messages sent through this slot so far; local[1]: CTAs of this launch that are done
    if (atomicAdd(local + 1, 1u) == gridDim.x - 1) {
      local[1] = 0;
      const uint32_t seq = local[0] + 1u;
      local[0] = seq;
      __threadfence_system();
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_flag), "r"(seq) : "memory");
    }
  }
}

__global__ void p2p_wait_kernel(const uint32_t* flag, uint32_t* expected, unsigned long long limit_ns, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x != 0) return;
  const uint32_t want = *expected + 1u;
  const uint64_t t0 = kh_globaltimer();
  for (uint32_t it = 0;; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if ((int32_t)(v - want) >= 0) { *expected = want; return; }
    if ((it & 15) == 15) {
      if (kh_globaltimer() - t0 > limit_ns) break;
      __nanosleep(128);
    }
  }
  atomicCAS(err, 0, 7);
}

int g_sms = 0;

}  // namespace

// src: local, dst: the slot in the peer's memory as mapped into this process, peer_flag: the slot's
// counter in the peer's memory, local: two zero-initialised device words owned by this (slot, direction).
extern "C" int kh_p2p_put(const void* src, void* dst, long long bytes, void* peer_flag, void* local, void* stream) {
  if (bytes <= 0 || (bytes & 15) || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15)) {
    kh_set_error("p2p_put: %lld bytes / pointers must be multiples of 16", bytes);
    return -1;
  }
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  const size_t n16 = (size_t)bytes / 16;
  size_t want = (n16 + PUT_THREADS * PUT_UNROLL - 1) / (PUT_THREADS * PUT_UNROLL);
  const int grid = (int)(want < (size_t)g_sms ? (want ? want : 1) : (size_t)g_sms);
  KH_LAUNCH(p2p_put_kernel, grid, PUT_THREADS, 0, (cudaStream_t)stream, (const uint4*)src, (uint4*)dst, n16, (uint32_t*)peer_flag,
                                                                  (uint32_t*)local);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { kh_set_error("p2p_put: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

// flag: this rank's slot counter (written by the peer), expected: one zero-initialised local device word.
extern "C" int kh_p2p_wait(const void* flag, void* expected, unsigned limit_ms, void* stream) {
  if (limit_ms == 0 || limit_ms > 60000) { kh_set_error("p2p_wait: limit %u ms outside (0, 60000]", limit_ms); return -1; }
  KH_LAUNCH(p2p_wait_kernel, 1, 32, 0, (cudaStream_t)stream, (const uint32_t*)flag, (uint32_t*)expected,
                                                       (unsigned long long)limit_ms * 1000000ull, kh_error_word_dev());
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { kh_set_error("p2p_wait: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}
