// Weight-streaming GEMM for decode steps (M <= 64 rows): out[M,N] = x[M,K] * W[N,K]^T + epilogue.
//
// A decode step multiplies a handful of token rows with every weight matrix, so the product is
// bound by reading W once, not by FLOPs, and a 128-row output tile would leave most CTAs idle.
// This kernel swaps the operand roles (the weights are the 128-row "A" operand of tcgen05.mma, the
// token rows are the narrow "B" operand, the accumulator in TMEM is out^T [128 weights x M]) and
// splits K across CTAs so that every SM streams a slice of W:
//
//   grid = (ceil(N/128) n-tiles) x (split-K slices), one tile per CTA, at most 4 k-blocks of 64
//   per CTA, all of whose TMA loads are issued up front (no ring to recycle);
//   split > 1: every CTA writes its fp32 partial to scratch; the CTA that arrives last at its
//   n-tile (integer ticket) adds the slices in index order and runs the epilogue -- the result is
//   independent of arrival order, so decoding is reproducible.
//
// Epilogues as in the big GEMM: bias, bias+GELU (pre-activation kept), bias+residual.
// Optional LayerNorm prologue (up to 16 rows): instead of loading x tiles with TMA, the CTA computes
// each row's mean / rstd over the full K, normalises its own K slice in registers and writes it
// into the B-operand tiles in the 128-byte-swizzled layout the MMA descriptor expects, so a decode
// layer needs no separate LayerNorm launch and the normalised rows never touch global memory.
// The reference used the same cuBLAS call for M = 1..32 as for training (src/core/infer.c:152-180).
// Waits are bounded (error word code 1/3).
#include "common.cuh"

#define KH_LAUNCH_CHECK(name)                                                     \
  do {                                                                            \
    cudaError_t e_ = cudaGetLastError();                                          \
    if (e_ != cudaSuccess) { kh_set_error(name ": %s", cudaGetErrorString(e_)); return -1; } \
  } while (0)

namespace {
constexpr int TN = 128, BK = 64, UMMA_K = 16, MAX_KB = 4;      // <= 4 k-blocks per CTA: two to three CTAs fit on an SM
constexpr int COUNTER_SLOTS = 1024;
enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2, EPI_BIAS_RESID = 3 };

struct SkinnyParams {
  int M, N, K;
  int kb_per_cta, num_kb;
  bf16* out; int ldo;
  int epi;
  const bf16* bias;
  bf16* aux; int ldaux;
  const bf16* x; int ldx;            // raw activation rows (LayerNorm prologue only)
  const bf16* ln_w; const bf16* ln_b;  // non-null: y = LayerNorm(x) * ln_w + ln_b feeds the product
  int w_static;         // the weights are not written by the kernel launched just before this one: stream them before it ends
  int* counters;        // [n_tiles], zero between launches
  float* partials;      // [split][MP][N]
  int* err;
};

template <int MP>   // padded row count = MMA N (16, 32 or 64)
__global__ void __launch_bounds__(128, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   const SkinnyParams p) {
  constexpr int W_BYTES = TN * BK * 2, X_BYTES = MP * BK * 2, STAGE = W_BYTES + X_BYTES;
  constexpr int TMEM_COLS = MP < 32 ? 32 : MP;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* al = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(al + MAX_KB * STAGE);
  const uint32_t bar_full = smem_u32(bars), bar_done = bar_full + 8 * MAX_KB;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + MAX_KB + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_last = reinterpret_cast<int*>(tmem_slot + 2);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int nt = blockIdx.x, ks = blockIdx.y, split = gridDim.y;
  const int kb0 = ks * p.kb_per_cta, kb1 = min(p.num_kb, kb0 + p.kb_per_cta);
  const int nkb = kb1 - kb0;

  if (tid == 0) {
    for (int s = 0; s < MAX_KB; s++) mbar_init(bar_full + 8 * s, 1);
    mbar_init(bar_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_w);
    tma_prefetch_desc(&map_x);
  }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  bool ok = true;
  const bool fuse_ln = (MP == 16) && p.ln_w != nullptr;
  // Programmatic dependent launch: this CTA may be resident while the previous kernel of the stream is
  // still running.  Weights that the previous kernel cannot have written (decode steps: the engine says
  // so) are requested right away, so the weight stream of this product overlaps the tail of the previous
  // one; everything an earlier kernel produces (the token rows) is touched after the wait.
  if (tid == 0) {
    for (int i = 0; i < nkb; i++) {
      mbar_expect_tx(bar_full + 8 * i, fuse_ln ? W_BYTES : STAGE);
      if (p.w_static) tma_load_2d(base + i * STAGE, &map_w, bar_full + 8 * i, (kb0 + i) * BK, nt * TN);
    }
  }
  pdl_wait();
  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < nkb; i++) {
      const uint32_t sw = base + i * STAGE, sx = sw + W_BYTES;
      if (!p.w_static) tma_load_2d(sw, &map_w, bar_full + 8 * i, (kb0 + i) * BK, nt * TN);
      if (!fuse_ln) tma_load_2d(sx, &map_x, bar_full + 8 * i, (kb0 + i) * BK, 0);
    }
  }
  if (fuse_ln) {
    // 8 threads per row: statistics over the whole row (two passes, fp32), then this CTA's K slice
    const int r = tid >> 3, sub = tid & 7;
    const bool live = r < p.M;
    const bf16* xr = p.x + (size_t)r * p.ldx;
    const int nchunk = p.K >> 3;                     // 16-byte chunks per row (K % 8 == 0)
    float sum = 0.f;
    if (live)
      for (int c = sub; c < nchunk; c += 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + c * 8);
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), e = unpack_bf16(u.w);
        sum += (a.x + a.y) + (b.x + b.y) + (cc.x + cc.y) + (e.x + e.y);
      }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1); sum += __shfl_xor_sync(0xffffffffu, sum, 2); sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    const float mean = sum / (float)p.K;
    float sq = 0.f;
    if (live)
      for (int c = sub; c < nchunk; c += 8) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + c * 8);
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), e = unpack_bf16(u.w);
        float d0 = a.x - mean, d1 = a.y - mean, d2 = b.x - mean, d3 = b.y - mean, d4 = cc.x - mean, d5 = cc.y - mean,
              d6 = e.x - mean, d7 = e.y - mean;
        sq += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3 + d4 * d4 + d5 * d5 + d6 * d6 + d7 * d7;
      }
    sq += __shfl_xor_sync(0xffffffffu, sq, 1); sq += __shfl_xor_sync(0xffffffffu, sq, 2); sq += __shfl_xor_sync(0xffffffffu, sq, 4);
    const float rstd = rsqrtf(sq / (float)p.K + 1e-5f);
    for (int i = 0; i < nkb; i++) {
      const int col = (kb0 + i) * BK + sub * 8;
      uint4 o = make_uint4(0, 0, 0, 0);
      if (live && col < p.K) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + col);
        const uint4 gw = __ldg(reinterpret_cast<const uint4*>(p.ln_w + col)), gb = __ldg(reinterpret_cast<const uint4*>(p.ln_b + col));
        const uint32_t* ui = &u.x; const uint32_t* wi = &gw.x; const uint32_t* bi = &gb.x; uint32_t* oi = &o.x;
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const float2 xv = unpack_bf16(ui[k]), wv = unpack_bf16(wi[k]), bv = unpack_bf16(bi[k]);
          oi[k] = pack_bf16((xv.x - mean) * rstd * wv.x + bv.x, (xv.y - mean) * rstd * wv.y + bv.y);
        }
      }
      const uint32_t sx = base + i * STAGE + W_BYTES;
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(sx + r * 128 + ((sub ^ (r & 7)) << 4)), "r"(o.x), "r"(o.y),
                   "r"(o.z), "r"(o.w) : "memory");
    }
    fence_proxy_async_smem();        // generic-proxy writes -> visible to the tensor core's async proxy
  }
  __syncthreads();
  if (tid == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(TN, MP, 0, 0);
    for (int i = 0; i < nkb && ok; i++) {
      if (!mbar_wait(bar_full + 8 * i, 0, abort_flag, 1, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t sw = base + i * STAGE, sx = sw + W_BYTES;
      const uint64_t adesc = umma_desc_sw128(sw, 16, 1024), bdesc = umma_desc_sw128(sx, 16, 1024);
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; k++)
        umma_f16_ss(tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (i > 0 || k > 0) ? 1u : 0u);
    }
    if (ok) umma_commit(bar_done);
  }
  if (nkb > 0 && !mbar_wait(bar_done, 0, abort_flag, 3, p.err)) ok = false;
  tc_fence_after();

  const int n = nt * TN + tid;                 // this thread's output column (weight row)
  float v[MP];
  if (ok && nkb > 0) {
#pragma unroll
    for (int c = 0; c < MP; c += 16) {
      uint32_t r[16];
      tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; i++) v[c + i] = __uint_as_float(r[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < MP; i++) v[i] = 0.f;
  }
  tc_fence_before();

  bool finish = ok;
  if (ok && split > 1) {
    if (n < p.N) {
#pragma unroll
      for (int m = 0; m < MP; m++)
        if (m < p.M) p.partials[((size_t)ks * MP + m) * p.N + n] = v[m];
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) *s_last = (atomicAdd(p.counters + nt, 1) == split - 1);
    __syncthreads();
    finish = *s_last != 0;
    if (finish) {
      __threadfence();
      if (n < p.N) {
#pragma unroll
        for (int m = 0; m < MP; m++) v[m] = 0.f;
        for (int k = 0; k < split; k++) {          // slices in index order; the MP loads of a slice are independent
#pragma unroll
          for (int m = 0; m < MP; m++)
            if (m < p.M) v[m] += __ldcg(p.partials + ((size_t)k * MP + m) * p.N + n);
        }
      }
      if (tid == 0) p.counters[nt] = 0;
    }
  }
  if (finish && n < p.N) {
    const float b = (p.epi != EPI_NONE) ? __bfloat162float(p.bias[n]) : 0.f;
#pragma unroll
    for (int m = 0; m < MP; m++) {
      if (m >= p.M) break;
      float x = v[m] + b;
      if (p.epi == EPI_BIAS_GELU) {
        const bf16 pre = __float2bfloat16(x);
        p.aux[(size_t)m * p.ldaux + n] = pre;
        x = gelu_tanh(__bfloat162float(pre));
      } else if (p.epi == EPI_BIAS_RESID) {
        x += __bfloat162float(p.aux[(size_t)m * p.ldaux + n]);
      }
      p.out[(size_t)m * p.ldo + n] = __float2bfloat16(x);
    }
  }
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

int g_sms = 0;
int num_sms() {
  if (!g_sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_sms <= 0) g_sms = 148;
  }
  return g_sms;
}
int pad_rows(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : 64); }
int pick_split(int N, int K) {
  const int n_tiles = (N + TN - 1) / TN, num_kb = (K + BK - 1) / BK;
  // every CTA issues all of its loads at once (up to 8 x 16 KB in flight), so one CTA per SM already
  // saturates HBM; more slices only lengthen the reduction
  int split = (num_sms() + n_tiles - 1) / n_tiles;
  if (split > 8) split = 8;
  const int min_split = (num_kb + MAX_KB - 1) / MAX_KB;
  if (split < min_split) split = min_split;
  if (split > num_kb) split = num_kb;
  const int per = (num_kb + split - 1) / split;
  return (num_kb + per - 1) / per;                            // no empty slices
}

template <int MP>
int launch(const CUtensorMap* mw, const CUtensorMap* mx, const SkinnyParams& p, int n_tiles, int split, cudaStream_t st) {
  constexpr int SMEM = MAX_KB * (TN * BK * 2 + MP * BK * 2) + 1024 + 128;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) { kh_set_error("gemm_skinny: shared memory opt-in failed: %s", cudaGetErrorString(e)); return -1; }
    attr = true;
  }
  dim3 grid(n_tiles, split);
  KH_LAUNCH((gemm_skinny_kernel<MP>), grid, 128, SMEM, st, *mw, *mx, p);
  KH_LAUNCH_CHECK("gemm_skinny");
  return 0;
}
}  // namespace

// fp32 elements of scratch needed for an [M,K] x [N,K]^T product (counter slots included, zeroed once)
extern "C" long kh_gemm_skinny_scratch_elems(int M, int N, int K) {
  return COUNTER_SLOTS + (long)pick_split(N, K) * pad_rows(M) * N;
}
// `weights_static` != 0: W is not written by the kernel that precedes this launch on the stream (true for
// every product of a decode step); the kernel then starts streaming W before that kernel has finished.
extern "C" int kh_gemm_skinny2(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K,
                               int epi, const void* bias, void* aux, int ldaux, void* scratch, const void* ln_w,
                               const void* ln_b, int weights_static, void* stream) {
  if (M < 1 || M > 64) { kh_set_error("gemm_skinny: M=%d outside [1, 64]", M); return -1; }
  if ((ln_w != nullptr) != (ln_b != nullptr)) { kh_set_error("gemm_skinny: LayerNorm needs both weight and bias"); return -1; }
  if (ln_w && (M > 16 || (K % 8) || (ldx % 8) || ((uintptr_t)x & 15))) {
    kh_set_error("gemm_skinny: fused LayerNorm needs M <= 16, K %% 8 == 0 and 16-byte aligned rows (M=%d K=%d)", M, K);
    return -1;
  }
  const int n_tiles = (N + TN - 1) / TN;
  if (n_tiles > COUNTER_SLOTS) { kh_set_error("gemm_skinny: N=%d exceeds %d column tiles", N, COUNTER_SLOTS * TN); return -1; }
  if (epi != EPI_NONE && !bias) { kh_set_error("gemm_skinny: bias missing"); return -1; }
  if ((epi == EPI_BIAS_GELU || epi == EPI_BIAS_RESID) && !aux) { kh_set_error("gemm_skinny: aux operand missing"); return -1; }
  const int MP = pad_rows(M);
  const CUtensorMap* mw = kh_tmap_2d_bf16(W, N, K, ldw, TN, BK);
  const CUtensorMap* mx = kh_tmap_2d_bf16(x, M, K, ldx, MP, BK);
  if (!mw || !mx) return -1;
  SkinnyParams p = {};
  p.M = M; p.N = N; p.K = K;
  p.num_kb = (K + BK - 1) / BK;
  const int split = pick_split(N, K);
  p.kb_per_cta = (p.num_kb + split - 1) / split;
  p.out = (bf16*)out; p.ldo = ldo; p.epi = epi; p.bias = (const bf16*)bias; p.aux = (bf16*)aux; p.ldaux = ldaux;
  p.x = (const bf16*)x; p.ldx = ldx; p.ln_w = (const bf16*)ln_w; p.ln_b = (const bf16*)ln_b;
  p.w_static = weights_static;
  p.counters = (int*)scratch; p.partials = (float*)scratch + COUNTER_SLOTS;
  p.err = kh_error_word_dev();
  cudaStream_t st = (cudaStream_t)stream;
  if (MP == 16) return launch<16>(mw, mx, p, n_tiles, split, st);
  if (MP == 32) return launch<32>(mw, mx, p, n_tiles, split, st);
  return launch<64>(mw, mx, p, n_tiles, split, st);
}

extern "C" int kh_gemm_skinny(const void* x, int ldx, const void* W, int ldw, void* out, int ldo, int M, int N, int K,
                              int epi, const void* bias, void* aux, int ldaux, void* scratch, const void* ln_w,
                              const void* ln_b, void* stream) {
  return kh_gemm_skinny2(x, ldx, W, ldw, out, ldo, M, N, K, epi, bias, aux, ldaux, scratch, ln_w, ln_b, 0, stream);
}
