// Vocabulary-parallel softmax: exchange and combination of the per-rank row statistics in one kernel.
//
// Each TP rank owns a slice of the vocabulary and has computed, per row, (max, sum exp(x - max),
// target logit or -inf) over its slice (xent_stats_k).  This kernel
//   1. stores the rank's triples into every peer's symmetric buffer (plain st.global to peer memory),
//   2. releases one arrival counter per (source rank, 256-row block) on every peer,
//   3. waits (bounded) until the peers' triples of its own row block have arrived,
//   4. writes gmax = max_r m_r, gsum = sum_r s_r * exp(m_r - gmax) and the row loss
//      log(gsum) + gmax - target logit (0 for ignored rows).
// It stands where the reference, whose head is replicated on every TP rank, has nothing
// (src/core/gpt.c:16); the collective-based evaluation of the same step is GPT._vp_combine.
//
// Flow control as in the fused GEMMs: the buffer has two parities selected by the call number, which
// lives in a device word that the last CTA advances; counters only grow (one per call).  A rank cannot
// be two calls ahead of a peer, because finishing a call needs that peer's triples of the same call.
// Every wait is bounded: on expiry the library error word receives code 5 and the CTA returns without
// writing results.
#include "../kernels/common.cuh"

namespace {
constexpr int MAX_TP = 8, ROWS = 256;

struct VpParams {
  const float* stats;          // local [R, 3]
  float* all[MAX_TP];          // all[r]: rank r's buffer [2 parities][tp sources][R][3]
  uint32_t* flags[MAX_TP];     // flags[r]: rank r's counters [tp sources][blocks]
  uint32_t* epoch;             // local: [0] calls completed, [1] CTAs finished
  const int* tgt;
  float *gmax, *gsum, *rowloss;
  int R, tp, rank;
  uint64_t wait_ns;
  int* err;
};

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(ROWS) vp_combine_k(const VpParams p) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1u;
  const size_t slab = (size_t)p.tp * p.R * 3;
  float* mine = p.all[p.rank] + (size_t)(call & 1u) * slab;
  const int nblk = (int)gridDim.x;
  const int r = (int)blockIdx.x * ROWS + (int)threadIdx.x;
  float m = -INFINITY, s = 0.f, x = -INFINITY;
  if (r < p.R) {
    m = p.stats[3 * r]; s = p.stats[3 * r + 1]; x = p.stats[3 * r + 2];
    for (int pr = 0; pr < p.tp; pr++) {
      if (pr == p.rank) continue;
      float* dst = p.all[pr] + (size_t)(call & 1u) * slab + ((size_t)p.rank * p.R + r) * 3;
      dst[0] = m; dst[1] = s; dst[2] = x;
    }
  }
  __threadfence_system();
  __syncthreads();
  if ((int)threadIdx.x < p.tp && (int)threadIdx.x != p.rank) {
    const int pr = (int)threadIdx.x;
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.flags[pr] + (size_t)p.rank * nblk + blockIdx.x), "r"(1u) : "memory");
    // the same thread waits for that peer's triples of this row block
    const uint32_t* f = p.flags[p.rank] + (size_t)pr * nblk + blockIdx.x;
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
      if ((int32_t)(ld_acquire_sys_u32(f) - call) >= 0) break;
      if ((it & 63) == 63) {
        const uint64_t now = kh_globaltimer();
        if (t0 == 0) t0 = now;
        else if (now - t0 > p.wait_ns) { s_bad = 1; atomicCAS(p.err, 0, 5); break; }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  if (!s_bad && r < p.R) {
    float gm = m, xt = x;
    float ms[MAX_TP], ss[MAX_TP];
#pragma unroll
    for (int src = 0; src < MAX_TP; src++) {
      if (src >= p.tp) break;
      if (src == p.rank) { ms[src] = m; ss[src] = s; continue; }
      const float* q = mine + ((size_t)src * p.R + r) * 3;
      ms[src] = __ldcg(q); ss[src] = __ldcg(q + 1);
      xt = fmaxf(xt, __ldcg(q + 2));
      gm = fmaxf(gm, ms[src]);
    }
    float gs = 0.f;                      // summed in rank order: identical bits on every rank
#pragma unroll
    for (int src = 0; src < MAX_TP; src++) {
      if (src >= p.tp) break;
      gs += ms[src] == -INFINITY ? 0.f : ss[src] * expf(ms[src] - gm);
    }
    p.gmax[r] = gm;
    p.gsum[r] = gs;
    p.rowloss[r] = p.tgt[r] >= 0 ? logf(gs) + gm - xt : 0.f;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.epoch + 1, 1u) == gridDim.x - 1) {
      p.epoch[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.epoch) = call;
    }
  }
}
}  // namespace

// `all_ptrs[r]`, `flag_ptrs[r]`: rank r's symmetric buffers as mapped into this process (own entry =
// local).  all: 2 * tp * R * 3 floats; flags: tp * ceil(R / 256) zero-initialised counters;
// `epoch_ptr`: two zero-initialised local words.  Returns 0 or -1.
extern "C" int kh_vp_combine(const void* stats, const unsigned long long* all_ptrs, const unsigned long long* flag_ptrs,
                             unsigned long long epoch_ptr, const void* tgt, void* gmax, void* gsum, void* rowloss,
                             int R, int tp, int rank, void* stream) {
  if (tp < 2 || tp > MAX_TP || rank < 0 || rank >= tp || R < 1 || !epoch_ptr) {
    kh_set_error("vp_combine: bad arguments (R=%d tp=%d rank=%d)", R, tp, rank);
    return -1;
  }
  VpParams p = {};
  p.stats = (const float*)stats;
  for (int r = 0; r < tp; r++) { p.all[r] = (float*)all_ptrs[r]; p.flags[r] = (uint32_t*)flag_ptrs[r]; }
  p.epoch = (uint32_t*)epoch_ptr;
  p.tgt = (const int*)tgt;
  p.gmax = (float*)gmax; p.gsum = (float*)gsum; p.rowloss = (float*)rowloss;
  p.R = R; p.tp = tp; p.rank = rank;
  p.wait_ns = kh_peer_wait_limit_ns();
  p.err = kh_error_word_dev();
  const int grid = (R + ROWS - 1) / ROWS;
  if (grid > 148) { kh_set_error("vp_combine: %d rows need more CTAs than can be resident together", R); return -1; }
  KH_LAUNCH(vp_combine_k, grid, ROWS, 0, (cudaStream_t)stream, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { kh_set_error("vp_combine: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}
