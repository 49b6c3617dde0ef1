// bf16 GEMM family on the 5th-generation tensor cores (sm_100a).
//
//   C[M,N] (+)= op(A) * op(B)          fp32 accumulation in TMEM
//
// A is either K-major ([M,K] row-major) or M-major ([K,M] row-major); B is either K-major
// ([N,K] row-major, i.e. an nn.Linear weight) or N-major ([K,N] row-major).  That covers
// the three products of a linear layer without any transposed copies:
//   forward        Y  = X  * W^T      A K-major,  B K-major     (reference mm_nt_bf16o, kernels.cu:34-39)
//   input grad     dX = dY * W        A K-major,  B N-major     (reference mm_nn_bf16o, kernels.cu:55-60)
//   weight grad    dW = dY^T * X      A M-major,  B N-major     (reference mm_tn_bf16[_acc], kernels.cu:41-53)
//
// Structure: persistent CTAs (one per SM), 6 warps.  Warp 0 streams operand tiles with TMA
// into a ring of 128-byte-swizzled shared-memory stages; one lane of warp 1 issues
// tcgen05.mma (128 x BN x 16 per instruction) into one of two TMEM accumulator buffers and
// commits stage-release / accumulator-ready mbarriers; warps 2-5 drain the other
// accumulator with tcgen05.ld and run the fused epilogue, so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Fused epilogues replace the reference's separate elementwise kernels
// (add_bias_k kernels.cu:174, bias_gelu_k :292, bias_residual_k :274, gelu_bwd_k :431,
// add_k :262) and the beta=1 weight-gradient accumulation.
//
// Bias gradients: with `colsum` set (weight-gradient products, A = dY in M-major form) four more
// warps add up the columns of the A tiles while they sit in shared memory and the CTAs that own
// the first column of output tiles add the sums into colsum[M] -- the reference's separate
// colsum_k pass over dY (kernels.cu:511-524) disappears.  A stage is handed back to the TMA
// producer only after both the MMAs and these warps are done with it.
//
// Every mbarrier wait is bounded: on expiry the CTA stores a code in the library error word,
// all roles unwind, TMEM is released and the kernel returns.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>
#include <unordered_map>

#include "common.cuh"

__device__ int g_kh_error_word = 0;
int* kh_error_word_dev() {
  static int* ptr[64] = {nullptr};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return nullptr;
  if (!ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_kh_error_word) == cudaSuccess) ptr[dev] = (int*)p;
  }
  return ptr[dev];
}

// ------------------------------------------------------------------------------- host util
static unsigned long long g_peer_wait_ns = 0;
unsigned long long kh_peer_wait_limit_ns() {
  if (g_peer_wait_ns == 0) {
    unsigned long long ms = 30000;
    if (const char* e = getenv("KHARON_PEER_WAIT_MS")) {
      const long v = atol(e);
      if (v > 0) ms = (unsigned long long)v;
    }
    g_peer_wait_ns = ms * 1000000ull;
  }
  return g_peer_wait_ns;
}
// Limit of every in-kernel wait on another rank, in milliseconds; returns the previous value.
extern "C" long kh_set_peer_wait_limit_ms(long ms) {
  const long old = (long)(kh_peer_wait_limit_ns() / 1000000ull);
  if (ms > 0) g_peer_wait_ns = (unsigned long long)ms * 1000000ull;
  return old;
}
static int g_pdl = -1;
int kh_pdl_enabled() {
  if (g_pdl < 0) {
    const char* e = getenv("KHARON_PDL");
    g_pdl = (e && e[0] == '0') ? 0 : 1;
  }
  return g_pdl;
}
// Programmatic dependent launch for all kernels of the library on/off; returns the previous setting.
extern "C" int kh_set_pdl(int on) {
  const int old = kh_pdl_enabled();
  g_pdl = on ? 1 : 0;
  return old;
}
static thread_local std::string g_host_err;
void kh_set_error(const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_host_err = buf;
}
extern "C" const char* kh_cuda_last_error() { return g_host_err.c_str(); }
extern "C" int kh_cuda_error_word(int reset) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_kh_error_word, sizeof(int)) != cudaSuccess) return -1;
  if (reset && v != 0) {
    int z = 0;
    cudaMemcpyToSymbol(g_kh_error_word, &z, sizeof(int));
  }
  return v;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

struct TmapKey {
  uint64_t base, rows, cols, ld;
  uint32_t br, bc;
  bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
    h ^= (k.rows + 0x632BE59BD9B4E019ull) + (h << 6) + (h >> 2);
    h ^= (k.cols * 31 + k.ld) + (h << 6) + (h >> 2);
    h ^= ((uint64_t)k.br << 32 | k.bc) + (h << 6) + (h >> 2);
    return (size_t)h;
  }
};
static size_t g_tmap_limit = 1u << 16;
// Test hook: number of cached descriptors after which the index is dropped (returns the old limit).
extern "C" long kh_tmap_cache_limit(long n) {
  const long old = (long)g_tmap_limit;
  if (n > 0) g_tmap_limit = (size_t)n;
  return old;
}

// Returns a descriptor that stays valid for the life of the process: callers hold the pointer
// across further look-ups (a launch fetches the A, B and output maps one after the other).
const CUtensorMap* kh_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                                   uint32_t box_rows, uint32_t box_cols) {
  static std::unordered_map<TmapKey, CUtensorMap*, TmapHash> cache;
  static std::mutex mu;
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = (uint64_t)base; key.rows = rows; key.cols = cols; key.ld = ld; key.br = box_rows; key.bc = box_cols;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  EncodeTiledFn fn = encode_fn();
  if (!fn) { kh_set_error("cuTensorMapEncodeTiled is not available from the driver"); return nullptr; }
  if (((uint64_t)base & 15) || ((ld * 2) & 15)) {
    kh_set_error("TMA operand needs a 16-byte aligned base and row pitch (base %p, ld %llu elements)", base,
                 (unsigned long long)ld);
    return nullptr;
  }
  CUtensorMap* m = new CUtensorMap;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult rc = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    delete m;
    kh_set_error("cuTensorMapEncodeTiled failed with %d (rows %llu cols %llu ld %llu box %ux%u)", (int)rc,
                 (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows, box_cols);
    return nullptr;
  }
  if (cache.size() >= g_tmap_limit) {
    // Buffers come from long-lived arenas, so this only bounds pathological churn.  The index is
    // dropped but the descriptors themselves are deliberately NOT freed (128 bytes each): pointers
    // handed out earlier, possibly a moment ago to the caller that triggered this insertion, must
    // not dangle.
    cache.clear();
  }
  cache[key] = m;
  return m;
}

const CUtensorMap* kh_tmap_3d_bf16(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t ld1, uint64_t ld2,
                                   uint32_t box_d1, uint32_t box_d0) {
  struct Key3 {
    uint64_t v[6];
    uint32_t b[2];
    bool operator==(const Key3& o) const { return memcmp(this, &o, sizeof(Key3)) == 0; }
  };
  struct Hash3 {
    size_t operator()(const Key3& k) const {
      uint64_t h = 0x9E3779B97F4A7C15ull;
      for (int i = 0; i < 6; i++) h ^= (k.v[i] + 0x632BE59BD9B4E019ull) + (h << 6) + (h >> 2);
      h ^= ((uint64_t)k.b[0] << 32 | k.b[1]) + (h << 6) + (h >> 2);
      return (size_t)h;
    }
  };
  static std::unordered_map<Key3, CUtensorMap*, Hash3> cache;
  static std::mutex mu;
  Key3 key;
  memset(&key, 0, sizeof(key));
  key.v[0] = (uint64_t)base; key.v[1] = d0; key.v[2] = d1; key.v[3] = d2; key.v[4] = ld1; key.v[5] = ld2;
  key.b[0] = box_d1; key.b[1] = box_d0;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  EncodeTiledFn fn = encode_fn();
  if (!fn) { kh_set_error("cuTensorMapEncodeTiled is not available from the driver"); return nullptr; }
  if (((uint64_t)base & 15) || ((ld1 * 2) & 15) || ((ld2 * 2) & 15)) {
    kh_set_error("TMA operand needs a 16-byte aligned base and pitches (base %p, pitches %llu / %llu elements)", base,
                 (unsigned long long)ld1, (unsigned long long)ld2);
    return nullptr;
  }
  CUtensorMap* m = new CUtensorMap;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1 * 2, ld2 * 2};
  cuuint32_t box[3] = {box_d0, box_d1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) {
    delete m;
    kh_set_error("cuTensorMapEncodeTiled (3-D) failed with %d", (int)rc);
    return nullptr;
  }
  if (cache.size() >= g_tmap_limit) cache.clear();      // descriptors stay allocated, see kh_tmap_2d_bf16
  cache[key] = m;
  return m;
}

// ------------------------------------------------------------------------------- kernel
enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2, EPI_BIAS_RESID = 3, EPI_DGELU = 4, EPI_RESID = 5 };

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;          // operand majors (0 = K-major, 1 = M/N-major)
  void* C; int ldc;        // output, bf16 or fp32
  int out_fp32, accumulate;
  int epi;
  const bf16* bias;        // [N]
  bf16* aux; int ldaux;    // EPI_BIAS_GELU: pre-activation out; EPI_BIAS_RESID/EPI_RESID: residual in; EPI_DGELU: pre-activation in
  float alpha;             // scales the accumulator before the epilogue
  float* colsum;           // [M] fp32 or null: colsum[m] (+)= sum_k op(A)[m, k]  (needs a_mn; launch with CSUM_THREADS)
  int* err;                // library error word
};

constexpr int BM = 128, BK = 64, UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int CSUM_THREADS = 320;          // + four column-sum warps

// PAIR: two CTAs of a cluster form one 256 x BN tile (tcgen05 cta_group::2).  Each CTA stages its
// own 128 rows of A and its own half of B, so a pair moves and re-reads 2/3 of the shared-memory
// bytes of two independent 128 x BN tiles.
template <int BN, bool PAIR = false> struct GemmCfg {
  static constexpr int BN_CTA = PAIR ? BN / 2 : BN;          // B rows (or columns) staged by one CTA
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN_CTA * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = PAIR ? 6 : ((BN == 256) ? 4 : (BN == 128 ? 6 : 8));
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

template <int BN, bool PAIR>
__global__ void __launch_bounds__(CSUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b, const GemmParams p) {
  using Cfg = GemmCfg<BN, PAIR>;
  constexpr int TM = PAIR ? 2 * BM : BM;                       // rows of one scheduled tile
  const uint32_t crank = PAIR ? cluster_ctarank() : 0u;        // 0 = leader (issues the MMAs)
  const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + Cfg::STAGES * Cfg::STAGE_BYTES);
  // bars: full[STAGES], empty[STAGES], tfull[2], tempty[2], free[STAGES], then tmem base word + abort flag
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * Cfg::STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * Cfg::STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_free = bar_tempty + 16;         // column-sum warps are done with the stage
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * Cfg::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const bool csum = p.colsum != nullptr;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + TM - 1) / TM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; s++) {
      mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); mbar_init(bar_free + 8 * s, 4);
    }
    // accumulator-free barrier: one arrival per epilogue warp of every CTA that reads the accumulator
    for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, PAIR ? 8 : 4); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    if (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS); tmem_relinquish(); }
  }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&tma_a); tma_prefetch_desc(&tma_b); }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                        // operands and outputs belong to earlier kernels of the stream up to here
  pdl_launch_dependents();

  // tile id -> (tm, tn): bands of 8 M-tiles, N fastest inside a band keeps both panels in L2
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int GROUP = 8;
    int band = t / (GROUP * tiles_n);
    int first = band * GROUP;
    int gsz = min(GROUP, tiles_m - first);
    int r = t - band * GROUP * tiles_n;
    tm = first + r % gsz;
    tn = r / gsz;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = worker; ok && t < num_tiles; t += n_workers) {
        int tm, tn;
        tile_coord(t, tm, tn);
        const int m0 = tm * TM + (int)crank * BM;               // first A row of this CTA
        const int n0 = tn * BN + (int)crank * Cfg::BN_CTA;      // first B row/column of this CTA
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, 2, p.err)) { ok = false; break; }
          if (csum && !mbar_wait(bar_free + 8 * s, ph ^ 1, abort_flag, 2, p.err)) { ok = false; break; }
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
          if (!PAIR) {
            mbar_expect_tx(bar_full + 8 * s, Cfg::STAGE_BYTES);
            if (!p.a_mn) tma_load_2d(sa, &tma_a, bar_full + 8 * s, kb * BK, m0);
            else
              for (int j = 0; j < BM / 64; j++) tma_load_2d(sa + j * (BK * 128), &tma_a, bar_full + 8 * s, m0 + j * 64, kb * BK);
            if (!p.b_mn) tma_load_2d(sb, &tma_b, bar_full + 8 * s, kb * BK, n0);
            else
              for (int j = 0; j < BN / 64; j++) tma_load_2d(sb + j * (BK * 128), &tma_b, bar_full + 8 * s, n0 + j * 64, kb * BK);
          } else {
            // both CTAs credit the leader's barrier; the leader expects the bytes of the whole pair
            const uint32_t lbar = mapa_shared(bar_full + 8 * s, 0);
            if (crank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * Cfg::STAGE_BYTES);
            if (!p.a_mn) tma_load_2d_pair(sa, &tma_a, lbar, kb * BK, m0);
            else
              for (int j = 0; j < BM / 64; j++) tma_load_2d_pair(sa + j * (BK * 128), &tma_a, lbar, m0 + j * 64, kb * BK);
            if (!p.b_mn) tma_load_2d_pair(sb, &tma_b, lbar, kb * BK, n0);
            else
              for (int j = 0; j < Cfg::BN_CTA / 64; j++) tma_load_2d_pair(sb + j * (BK * 128), &tma_b, lbar, n0 + j * 64, kb * BK);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && crank == 0) {
      const uint32_t idesc = umma_idesc_bf16(TM, BN, p.a_mn, p.b_mn);
      // K-major: LBO unused (encoded 16 B), SBO 1024; MN-major: LBO = one 64-wide slab (BK rows x 128 B), SBO 1024
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, b_lbo = p.b_mn ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      const uint32_t b_kstep = p.b_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      int it = 0, tcount = 0;
      bool ok = true;
      for (int t = worker; ok && t < num_tiles; t += n_workers, tcount++) {
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, aph ^ 1, abort_flag, 4, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (it / Cfg::STAGES) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, 1, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
          uint64_t adesc = umma_desc_sw128(sa, a_lbo, 1024);
          uint64_t bdesc = umma_desc_sw128(sb, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++) {
            if (PAIR) umma_f16_ss_pair(d_tmem, adesc + (uint64_t)(k * a_kstep), bdesc + (uint64_t)(k * b_kstep), idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16_ss(d_tmem, adesc + (uint64_t)(k * a_kstep), bdesc + (uint64_t)(k * b_kstep), idesc,
                             (kb > 0 || k > 0) ? 1u : 0u);
          }
          // stage reusable (in both CTAs of a pair) once these MMAs retire
          if (PAIR) umma_commit_pair(bar_empty + 8 * s, 3); else umma_commit(bar_empty + 8 * s);
        }
        if (ok) { if (PAIR) umma_commit_pair(bar_tfull + 8 * acc, 3); else umma_commit(bar_tfull + 8 * acc); }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ column sums of A (bias gradient)
    // Present only in launches with CSUM_THREADS.  A stage is read after the MMAs that consume it
    // have retired (its "empty" barrier, which also reaches the second CTA of a pair) and before the
    // producer may refill it (the "free" barrier).  Warp cw owns columns [32 cw, 32 cw + 32) of the
    // 128-column A tile: four 16-byte chunks of one 64-column slab.  Lane = 8 p + 4 h + c4 reads
    // chunk c4 of rows 8 i + p + 4 h (i = 0..7): the two rows of a quarter-warp differ in bit 2, so
    // the 128-byte swizzle puts them in different bank halves.  The warp needs no other warp's
    // data, so there is no barrier between the four.
    const int cw = warp - 6;
    const int c4 = lane & 3, rsel = ((lane >> 3) & 3) + 4 * ((lane >> 2) & 1);
    const uint32_t slab_off = (uint32_t)(cw >> 1) * (BK * 128);
    const int chunk = (cw & 1) * 4 + c4;
    int it = 0;
    bool ok = true;
    for (int t = worker; ok && t < num_tiles; t += n_workers) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const bool mine = (tn == 0);
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; j++) acc[j] = 0.f;
      for (int kb = 0; kb < num_kb; kb++, it++) {
        const int s = it % Cfg::STAGES;
        const uint32_t ph = (it / Cfg::STAGES) & 1;
        if (!mbar_wait(bar_empty + 8 * s, ph, abort_flag, 2, p.err)) { ok = false; break; }
        if (mine) {
          const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES + slab_off;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int r = 8 * i + rsel;
            uint4 v;
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(sa + (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4)));
            float2 f0 = unpack_bf16(v.x), f1 = unpack_bf16(v.y), f2 = unpack_bf16(v.z), f3 = unpack_bf16(v.w);
            acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
            acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_free + 8 * s);
      }
      if (ok && mine) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
          acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 4);
          acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 8);
          acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], 16);
        }
        if (lane < 4) {
          const int m0 = tm * TM + (int)crank * BM + cw * 32 + c4 * 8;
#pragma unroll
          for (int j = 0; j < 8; j++)
            if (m0 + j < p.M) p.colsum[m0 + j] = p.accumulate ? p.colsum[m0 + j] + acc[j] : acc[j];
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int q = warp & 3;                    // TMEM lane quadrant this warp may access
    int tcount = 0;
    bool ok = true;
    for (int t = worker; ok && t < num_tiles; t += n_workers, tcount++) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      const int row = tm * TM + (int)crank * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const bool use_bias = (p.epi == EPI_BIAS || p.epi == EPI_BIAS_GELU || p.epi == EPI_BIAS_RESID);
      const bool use_aux = (p.epi == EPI_BIAS_RESID || p.epi == EPI_RESID || p.epi == EPI_DGELU);
      // Operands of the epilogue are fetched one 32-column chunk ahead (the first chunk before the
      // accumulator is even complete), so their DRAM latency is not paid once per chunk.
      uint4 nb[4], nx[4];
      auto fetch = [&](int c0) {
        const int col = tn * BN + c0;
        if (c0 >= BN || col + 32 > p.N) return;
        if (use_bias) {
          const uint4* bp = reinterpret_cast<const uint4*>(p.bias + col);
#pragma unroll
          for (int j = 0; j < 4; j++) nb[j] = __ldg(bp + j);
        }
        if (use_aux && row_ok) {
          const uint4* ap = reinterpret_cast<const uint4*>(p.aux + (size_t)row * p.ldaux + col);
#pragma unroll
          for (int j = 0; j < 4; j++) nx[j] = ap[j];
        }
      };
      if (use_aux && row_ok) {
        const char* ap = reinterpret_cast<const char*>(p.aux + (size_t)row * p.ldaux + tn * BN);
        const int nbytes = min(BN, p.N - tn * BN) * 2;
        for (int b = 128; b < nbytes; b += 128) prefetch_l2(ap + b);
      }
      fetch(0);
      if (!mbar_wait(bar_tfull + 8 * acc, aph, abort_flag, 3, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col = tn * BN + c0;
        if (col >= p.N) break;                 // uniform across the warp
        uint32_t r[32];
        tmem_ld32(taddr + c0, r);
        uint4 cb[4], cx[4];
#pragma unroll
        for (int j = 0; j < 4; j++) { cb[j] = nb[j]; cx[j] = nx[j]; }
        fetch(c0 + 32);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]) * p.alpha;
        const bool full = (col + 32 <= p.N);
        if (use_bias) {
          if (full) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
              uint4 b = cb[j];
              float2 f0 = unpack_bf16(b.x), f1 = unpack_bf16(b.y), f2 = unpack_bf16(b.z), f3 = unpack_bf16(b.w);
              v[8 * j + 0] += f0.x; v[8 * j + 1] += f0.y; v[8 * j + 2] += f1.x; v[8 * j + 3] += f1.y;
              v[8 * j + 4] += f2.x; v[8 * j + 5] += f2.y; v[8 * j + 6] += f3.x; v[8 * j + 7] += f3.y;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i++) if (col + i < p.N) v[i] += __bfloat162float(p.bias[col + i]);
          }
        }
        if (row_ok) {
          if (p.epi == EPI_BIAS_GELU) {
            bf16* ap = p.aux + (size_t)row * p.ldaux + col;
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                uint4 o;
                o.x = pack_bf16(v[8 * j], v[8 * j + 1]); o.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
                o.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]); o.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
                reinterpret_cast<uint4*>(ap)[j] = o;
              }
            } else {
              for (int i = 0; i < 32; i++) if (col + i < p.N) ap[i] = __float2bfloat16(v[i]);
            }
            // the stored pre-activation is bf16; apply GELU to the rounded value so that the
            // backward pass (which only sees the bf16 copy) differentiates the same function
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = gelu_tanh(__bfloat162float(__float2bfloat16(v[i])));
          } else if (use_aux) {
            const bf16* ap = p.aux + (size_t)row * p.ldaux + col;
            float x[32];
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                uint4 b = cx[j];
                float2 f0 = unpack_bf16(b.x), f1 = unpack_bf16(b.y), f2 = unpack_bf16(b.z), f3 = unpack_bf16(b.w);
                x[8 * j + 0] = f0.x; x[8 * j + 1] = f0.y; x[8 * j + 2] = f1.x; x[8 * j + 3] = f1.y;
                x[8 * j + 4] = f2.x; x[8 * j + 5] = f2.y; x[8 * j + 6] = f3.x; x[8 * j + 7] = f3.y;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++) x[i] = (col + i < p.N) ? __bfloat162float(ap[i]) : 0.f;
            }
            if (p.epi == EPI_DGELU) {
#pragma unroll
              for (int i = 0; i < 32; i++) v[i] *= gelu_tanh_grad(x[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; i++) v[i] += x[i];
            }
          }
          if (p.out_fp32) {
            float* cp = reinterpret_cast<float*>(p.C) + (size_t)row * p.ldc + col;
            if (full) {
              if (p.accumulate) {
#pragma unroll
                for (int j = 0; j < 8; j++) red_add_v4_f32(cp + 4 * j, v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 8; j++)
                  reinterpret_cast<float4*>(cp)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
              }
            } else {
              for (int i = 0; i < 32; i++)
                if (col + i < p.N) cp[i] = p.accumulate ? cp[i] + v[i] : v[i];
            }
          } else {
            bf16* cp = reinterpret_cast<bf16*>(p.C) + (size_t)row * p.ldc + col;
            if (full) {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                uint4 o;
                o.x = pack_bf16(v[8 * j], v[8 * j + 1]); o.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
                o.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]); o.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
                reinterpret_cast<uint4*>(cp)[j] = o;
              }
            } else {
              for (int i = 0; i < 32; i++) if (col + i < p.N) cp[i] = __float2bfloat16(v[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(mapa_shared(bar_tempty + 8 * acc, 0));   // the leader issues the MMAs
        else mbar_arrive(bar_tempty + 8 * acc);
      }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();      // no CTA leaves while its peer may still signal its barriers
  if (warp == 1) {
    tc_fence_after();
    if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS); else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------- launcher
static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

// 256-row tiles on CTA pairs.  Returns the number of clusters that can be resident (0: unsupported).
static int g_pair_clusters = -1;
static int launch_gemm_pair(const CUtensorMap* ta, const CUtensorMap* tb, const GemmParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = GemmCfg<256, true>;
  auto kern = gemm_kernel<256, true>;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.blockDim = dim3(p.colsum ? CSUM_THREADS : GEMM_THREADS); cfg.dynamicSmemBytes = Cfg::SMEM; cfg.stream = st; cfg.attrs = attr;
  cfg.numAttrs = kh_pdl_enabled() ? 2 : 1;
  if (g_pair_clusters < 0) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) { kh_set_error("gemm: cannot opt in to %d bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e)); return -1; }
    cfg.gridDim = dim3(2 * (num_sms() / 2));
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); kh_set_error("gemm: CTA-pair launch is not available: %s", cudaGetErrorString(e)); g_pair_clusters = 0; return -1; }
    g_pair_clusters = n;
  }
  if (g_pair_clusters == 0) { kh_set_error("gemm: CTA-pair launch is not available"); return -1; }
  const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * ((p.N + 255) / 256);
  int clusters = tiles < g_pair_clusters ? tiles : g_pair_clusters;
  if (max_ctas > 0 && 2 * clusters > max_ctas) clusters = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  cfg.gridDim = dim3(2 * clusters);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, *ta, *tb, p);
  if (e != cudaSuccess) { kh_set_error("gemm pair launch failed: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}
extern "C" int kh_gemm_pair_clusters() { return g_pair_clusters; }

template <int BN>
static int launch_gemm(const CUtensorMap* ta, const CUtensorMap* tb, const GemmParams& p, int max_ctas, cudaStream_t st) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_kernel<BN, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM);
    if (e != cudaSuccess) { kh_set_error("gemm: cannot opt in to %d bytes of shared memory: %s", Cfg::SMEM, cudaGetErrorString(e)); return -1; }
    attr_set = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  int grid = tiles < num_sms() ? tiles : num_sms();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  cudaError_t e = KH_LAUNCH((gemm_kernel<BN, false>), grid, p.colsum ? CSUM_THREADS : GEMM_THREADS, Cfg::SMEM, st, *ta, *tb, p);
  if (e != cudaSuccess) { kh_set_error("gemm launch failed: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}

// C[M,N] = alpha * op(A) op(B) with a fused epilogue.  lda/ldb/ldc/ldaux are row pitches in
// elements of the row-major buffers described at the top of this file.  block_n = 0 lets the
// launcher pick the tile width; max_ctas > 0 caps the grid (used to leave SMs to a
// concurrently running communication kernel).  Returns 0 or -1 (see kh_cuda_last_error).
//
// kh_gemm_bf16_colsum: same product with `colsum` [M] fp32 receiving colsum[m] (+)= sum_k op(A)[m, k]
// (`+=` when `accumulate`), computed from the A tiles in shared memory by four extra warps.  A must
// be in M-major form (a_mn), i.e. the call is a weight-gradient product dW = dY^T X and `colsum`
// is the bias gradient.
extern "C" int kh_gemm_bf16_colsum(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc,
                                   int M, int N, int K, int out_fp32, int accumulate, int epi, const void* bias, void* aux,
                                   int ldaux, float alpha, int block_n, int max_ctas, void* colsum, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) { kh_set_error("gemm: empty problem %dx%dx%d", M, N, K); return -1; }
  if (colsum && !a_mn) { kh_set_error("gemm: column sums need the A operand in M-major form"); return -1; }
  if (accumulate && !out_fp32) { kh_set_error("gemm: accumulate needs an fp32 output"); return -1; }
  if ((ldc % (out_fp32 ? 4 : 8)) != 0 || ((uintptr_t)C & 15)) { kh_set_error("gemm: output pitch/base not 16-byte aligned (ldc %d)", ldc); return -1; }
  if ((epi == EPI_BIAS || epi == EPI_BIAS_GELU || epi == EPI_BIAS_RESID) && (!bias || ((uintptr_t)bias & 15))) { kh_set_error("gemm: bias missing or misaligned"); return -1; }
  if ((epi == EPI_BIAS_GELU || epi == EPI_BIAS_RESID || epi == EPI_DGELU || epi == EPI_RESID) && (!aux || (ldaux % 8) || ((uintptr_t)aux & 15))) { kh_set_error("gemm: aux operand missing or misaligned"); return -1; }
  int bn = block_n;
  if (bn == 0) {
    // waves x relative tile time; narrower tiles reuse the A panel less and run at lower efficiency
    const int tm = (M + BM - 1) / BM, sms = num_sms();
    auto waves = [&](int w) { return (tm * ((N + w - 1) / w) + sms - 1) / sms; };
    const float c256 = waves(256) * 1.0f, c128 = waves(128) * 0.7f, c64 = waves(64) * 0.5f;
    bn = 256;
    float best = c256;
    if (c128 < best) { best = c128; bn = 128; }
    if (c64 < best) { best = c64; bn = 64; }
    if (N <= 64) bn = 64;
    else if (N <= 128 && bn == 256) bn = 128;
    // 256 x 256 tiles on CTA pairs: a wave of pairs takes about 0.93 of a wave of single tiles
    // (measured 6-19 % faster on large shapes), so prefer it unless wave quantisation eats the gain
    if (bn == 256 && M >= 512 && g_pair_clusters != 0) {
      const int clusters = g_pair_clusters > 0 ? g_pair_clusters : sms / 2;
      const int tiles2 = ((M + 255) / 256) * ((N + 255) / 256);
      const float cpair = (float)((tiles2 + clusters - 1) / clusters) * 0.93f;
      if (cpair <= best) bn = 512;
    }
  }
  const bool pair = (bn == 512);      // 256 x 256 tiles on CTA pairs (cta_group::2)
  if (pair) bn = 256;
  if (bn != 64 && bn != 128 && bn != 256) { kh_set_error("gemm: block_n must be 64, 128, 256 or 512 (CTA pairs)"); return -1; }
  const CUtensorMap* ta = a_mn ? kh_tmap_2d_bf16(A, K, M, lda, BK, 64) : kh_tmap_2d_bf16(A, M, K, lda, BM, BK);
  if (!ta) return -1;
  const CUtensorMap* tb = b_mn ? kh_tmap_2d_bf16(B, K, N, ldb, BK, 64) : kh_tmap_2d_bf16(B, N, K, ldb, pair ? 128 : bn, BK);
  if (!tb) return -1;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.C = C; p.ldc = ldc; p.out_fp32 = out_fp32;
  p.accumulate = accumulate; p.epi = epi; p.bias = (const bf16*)bias; p.aux = (bf16*)aux; p.ldaux = ldaux; p.alpha = alpha;
  p.colsum = (float*)colsum;
  p.err = kh_error_word_dev();
  cudaStream_t st = (cudaStream_t)stream;
  if (pair) return launch_gemm_pair(ta, tb, p, max_ctas, st);
  if (bn == 256) return launch_gemm<256>(ta, tb, p, max_ctas, st);
  if (bn == 128) return launch_gemm<128>(ta, tb, p, max_ctas, st);
  return launch_gemm<64>(ta, tb, p, max_ctas, st);
}

extern "C" int kh_gemm_bf16(const void* A, int lda, int a_mn, const void* B, int ldb, int b_mn, void* C, int ldc,
                            int M, int N, int K, int out_fp32, int accumulate, int epi, const void* bias, void* aux,
                            int ldaux, float alpha, int block_n, int max_ctas, void* stream) {
  return kh_gemm_bf16_colsum(A, lda, a_mn, B, ldb, b_mn, C, ldc, M, N, K, out_fp32, accumulate, epi, bias, aux, ldaux,
                             alpha, block_n, max_ctas, nullptr, stream);
}
