// ZeRO-1 optimizer step as ONE kernel over NVLink peer memory (sm_100a):
//
//   gradient reduce-scatter (average)  +  fp32 AdamW on this rank's slice of the flat arena
//   +  bf16 parameter all-gather (push)  +  gradient clear
//
// replaces ncclReduceScatter(fp32, avg) -> adamw_k -> ncclAllGather(fp32) of the reference
// (src/core/adamw.c:48-58, src/parallel/comms.cu:101-107).  The fp32 gradient arena and the bf16
// compute copy of every data-parallel rank live in symmetric (peer-mapped) memory:
//
//   phase 0  every rank announces "my gradients are final" (stream order guarantees it) and
//            waits, bounded, for the same announcement of every peer;
//   phase 1  for each element of its slice a rank PULLS the peers' fp32 gradients with plain
//            loads, sums them in rank order, scales by 1/dp, updates master / moments, and
//            PUSHES the bf16 value into the compute copy of every rank (8-byte stores, a warp
//            covers 256 contiguous bytes);
//   phase 2  every CTA announces completion to every rank (its own included) and waits until all
//            CTAs of all ranks have done so: everybody, the other CTAs of this launch too, has
//            finished reading this rank's gradients and writing this rank's compute copy;
//   phase 3  the local gradient arena is cleared for the next accumulation.
//
// Only 2 bytes per parameter travel in the gather direction (the reference gathers 4), and the
// fp32 master outside a rank's slice is not kept current between checkpoints.  Summation order
// is fixed, so all ranks hold identical bf16 weights and runs are reproducible.  All waits are
// bounded (error word code 5).
#include "../kernels/common.cuh"

#define KH_LAUNCH_CHECK(name)                                                     \
  do {                                                                            \
    cudaError_t e_ = cudaGetLastError();                                          \
    if (e_ != cudaSuccess) { kh_set_error(name ": %s", cudaGetErrorString(e_)); return -1; } \
  } while (0)

namespace {
constexpr int MAX_DP = 8;

struct ZeroParams {
  int dp, rank;
  long shard;                  // elements per rank (multiple of 4)
  long n_total;                // dp * shard
  float* g[MAX_DP];            // gradient arenas (own entry local)
  bf16* wb[MAX_DP];            // compute copies (may be null entries when the model computes in fp32)
  uint32_t* ctr[MAX_DP];       // per rank: [0..dp) ready counters, [dp..2dp) done counters
  float* w; float* m; float* v;   // local master (full arena), local moment shards
  float lr, b1, b2, eps, wd, bc1, bc2, inv_dp;
  uint32_t epoch;
  uint64_t wait_ns;            // limit of the waits on the other ranks
  int* err;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, int* err, uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
    if ((it & 63) == 63) {
      if (*(volatile int*)err) return false;
      const uint64_t now = kh_globaltimer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) { atomicCAS(err, 0, 5); return false; }
      __nanosleep(128);
    }
  }
}

__global__ void __launch_bounds__(256)
zero1_step_kernel(const ZeroParams p) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  // ---- phase 0
  if (tid == 0) {
    if (blockIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < p.dp; r++)
        if (r != p.rank) red_release_sys_add(p.ctr[r] + p.rank, 1);
    }
    int ok = 1;
    for (int r = 0; r < p.dp && ok; r++)
      if (r != p.rank) ok = wait_counter(p.ctr[p.rank] + r, p.epoch, p.err, p.wait_ns) ? 1 : 0;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  // ---- phase 1
  const long lo = (long)p.rank * p.shard;
  const long nvec = p.shard / 4;
  for (long i = (long)blockIdx.x * blockDim.x + tid; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long e = lo + i * 4;
    float4 gs = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
    for (int r = 0; r < p.dp; r++) {
      const float4 gr = __ldcg(reinterpret_cast<const float4*>(p.g[r] + e));
      gs.x += gr.x; gs.y += gr.y; gs.z += gr.z; gs.w += gr.w;
    }
    float4 ww = *reinterpret_cast<float4*>(p.w + e);
    float4 mm = *reinterpret_cast<float4*>(p.m + i * 4), vv = *reinterpret_cast<float4*>(p.v + i * 4);
    float* ga = &gs.x; float* wa = &ww.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const float gk = ga[k] * p.inv_dp;
      ma[k] = p.b1 * ma[k] + (1.f - p.b1) * gk;
      va[k] = p.b2 * va[k] + (1.f - p.b2) * gk * gk;
      const float mh = ma[k] / p.bc1, vh = va[k] / p.bc2;
      wa[k] = wa[k] * (1.f - p.lr * p.wd) - p.lr * mh / (sqrtf(vh) + p.eps);
    }
    *reinterpret_cast<float4*>(p.w + e) = ww;
    *reinterpret_cast<float4*>(p.m + i * 4) = mm;
    *reinterpret_cast<float4*>(p.v + i * 4) = vv;
    const uint2 packed = make_uint2(pack_bf16(wa[0], wa[1]), pack_bf16(wa[2], wa[3]));
    for (int r = 0; r < p.dp; r++)
      if (p.wb[r]) *reinterpret_cast<uint2*>(p.wb[r] + e) = packed;
  }
  // ---- phase 2
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    // the local counter is part of the barrier: phase 3 of one CTA overwrites gradients that a
    // slower CTA of the same launch may still have to read in phase 1
    for (int r = 0; r < p.dp; r++) red_release_sys_add(p.ctr[r] + p.dp + p.rank, 1);
    int ok = 1;
    for (int r = 0; r < p.dp && ok; r++)
      ok = wait_counter(p.ctr[p.rank] + p.dp + r, p.epoch * gridDim.x, p.err, p.wait_ns) ? 1 : 0;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  // ---- phase 3
  const long nv_all = p.n_total / 4;
  float4* gz = reinterpret_cast<float4*>(p.g[p.rank]);
  for (long i = (long)blockIdx.x * blockDim.x + tid; i < nv_all; i += (long)gridDim.x * blockDim.x)
    gz[i] = make_float4(0.f, 0.f, 0.f, 0.f);
}
}  // namespace

// One fused ZeRO-1 step.  g_ptrs / wb_ptrs / ctr_ptrs: dp entries, index r = rank r's buffer as
// mapped in this process; ctr holds 2*dp zero-initialised uint32 per rank.  `epoch` is the 1-based
// call count (identical on all ranks); `grid` must be the same on all ranks.  Returns 0 or -1.
extern "C" int kh_zero1_step(const unsigned long long* g_ptrs, const unsigned long long* wb_ptrs,
                             const unsigned long long* ctr_ptrs, void* w, void* m, void* v, long shard, int dp,
                             int rank, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             unsigned epoch, int grid, void* stream) {
  if (dp < 2 || dp > MAX_DP || rank < 0 || rank >= dp) { kh_set_error("zero1: bad dp/rank %d/%d", rank, dp); return -1; }
  if (shard % 4) { kh_set_error("zero1: shard length must be a multiple of 4"); return -1; }
  if (grid < 1 || grid > 1184) { kh_set_error("zero1: grid %d out of range", grid); return -1; }
  ZeroParams p = {};
  p.dp = dp; p.rank = rank; p.shard = shard; p.n_total = shard * dp;
  for (int r = 0; r < dp; r++) {
    p.g[r] = (float*)g_ptrs[r];
    p.wb[r] = wb_ptrs ? (bf16*)wb_ptrs[r] : nullptr;
    p.ctr[r] = (uint32_t*)ctr_ptrs[r];
  }
  p.w = (float*)w; p.m = (float*)m; p.v = (float*)v;
  p.lr = lr; p.b1 = b1; p.b2 = b2; p.eps = eps; p.wd = wd; p.bc1 = bc1; p.bc2 = bc2; p.inv_dp = 1.f / dp;
  p.epoch = epoch;
  p.wait_ns = kh_peer_wait_limit_ns();
  p.err = kh_error_word_dev();
  // The exit barrier spans the grid, so every CTA has to be resident at the same time: a cooperative
  // launch either places the whole grid or fails, also when other streams occupy part of the GPU.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t le = cudaLaunchKernelEx(&cfg, zero1_step_kernel, p);
  if (le != cudaSuccess) { kh_set_error("zero1_step: launch of %d CTAs failed: %s", grid, cudaGetErrorString(le)); return -1; }
  KH_LAUNCH_CHECK("zero1_step");
  return 0;
}

// Largest grid kh_zero1_step can place on the current device (all CTAs resident at once).
extern "C" int kh_zero1_max_grid() {
  int dev = 0, sms = 0, per_sm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, zero1_step_kernel, 256, 0) != cudaSuccess) return 0;
  return sms * per_sm;
}
