// All transformer layers (and the vocabulary head) of one decode step in ONE persistent kernel (sm_100a).
//
// A decode step of G <= 32 sequences is latency-bound: its per-layer chain LayerNorm -> qkv -> paged
// attention -> proj -> LayerNorm -> fc/GELU -> fcproj moves a few megabytes of weights, and as five
// launches per layer (src/core/infer.c:204-262 issues more than twenty) every link of the chain pays
// a launch, a pipeline prologue and a split-K hand-off.  Here one cooperative grid (one CTA per SM)
// walks the chain for all layers; the links are grid barriers in L2 and the activations between
// them (a few KB per row) stay in L2.
//
//   phase A  xs = LN1(x)            qkv  = xs Wqkv^T + b                        (N = 3d, K = d)
//   phase B  per (sequence, head): append k, v to the paged cache, att = softmax(q K^T) V
//   phase C  xs = att               xmid = xs Wproj^T + b + x                   (N = d,  K = d)
//   phase D  xs = LN2(xmid)         act  = gelu(bf16(xs Wfc^T + b))             (N = 4d, K = d)
//   phase E  xs = act               x    = xs Wfcproj^T + b + xmid              (N = d,  K = 4d)
//   head     xs = LNf(x[rows])      logits = xs Whead^T                         (N = V,  K = d)
//
// Linear phases.  A work unit is 8 output columns; S = K / 512 warps (1, 2, 4 or 8) share a unit, each
// streaming its 512-wide K slice of the 8 weight rows straight from global memory into registers
// (sixteen 16-byte loads per lane in flight -- weights are read exactly once, so they bypass shared
// memory), and a CTA works on 8 / S units at a time.  The activation rows come into shared memory
// either by plain loads past L1 (a handful of rows: one trip to L2, LayerNorm on the row held in
// registers) or with one bulk copy per row (all in flight together, completion on an mbarrier, then
// LayerNorm in place); rows are padded by 64 bytes so that fragment loads are conflict-free.  The products run on the tensor cores as mma.sync m16n8k16 (G <= 32 rows are one or
// two m16 tiles: tcgen05's 128-row tiles, TMEM round trip and shared-memory operand staging are what
// this kernel exists to avoid; the large-M GEMMs of training and prefill use them).  The K order inside
// a 32-wide block is permuted identically for both operands so that every lane fetches 16 contiguous
// bytes of its weight row.  Partial sums of the S warps meet in shared memory; thread (g, n) adds them
// in warp order and applies the epilogue, whose bias and residual operands were fetched before the
// products.  Weights do not depend on the previous phase, so the first unit's weight loads of the
// NEXT phase are issued before the grid barrier and land while it is being crossed.
//
// Grid barrier: one monotonic arrival counter in global memory (a barrier is one atomic and one polled
// load).  Every wait is bounded: status code 9 (grid barrier) or 10 (row copies) in the library error
// word, and all CTAs leave through an abort word.
// Numerics follow the five-kernel path: bf16 activations between phases, fp32 accumulation, LayerNorm
// statistics in two passes, GELU applied to the bf16-rounded pre-activation.
#include "common.cuh"

namespace {

constexpr int THREADS = 256, WARPS = 8;
constexpr int KW = 512;                       // K slice of one warp in one sub-step
constexpr int NLD = KW / 32;                  // 16-byte weight loads per lane and sub-step
constexpr int PAD = 32;                       // bf16 elements of padding per activation row (64 bytes)
constexpr int XS_BYTES = 136 * 1024;          // activation rows in shared memory
constexpr int RED_FLOATS = WARPS * 32 * 8;    // partial tiles of the 8 warps (32 rows x 8 columns each)
constexpr int MAXQ = 8;                       // epilogue outputs per thread and turn: 8 units x 32 rows x 8 columns / 256 threads

struct LayerW {               // bf16 pointers of one layer (device array, one entry per layer)
  const bf16 *ln1_w, *ln1_b, *qkv_w, *qkv_b, *proj_w, *proj_b, *ln2_w, *ln2_b, *fc_w, *fc_b, *fcproj_w, *fcproj_b;
};

struct DecodeParams {
  int G, d, H, hd, L, bs, max_lb, max_ctx;
  const LayerW* layers;
  bf16 *x, *xmid, *qkv, *att, *act;       // [G, d], [G, d], [G, 3d], [G, d], [G, 4d]
  bf16 *kc, *vc;                          // [L, blocks, bs, H, hd]
  size_t layer_elems;
  const int *pos, *slot, *btab;
  // optional head: logits[g, :V] = LNf(x[rows[g]]) Whead^T
  const bf16 *head_w, *lnf_w, *lnf_b;
  bf16* logits;
  int ld_logits, V, n_rows;
  const int* rows;
  uint32_t* bar;                          // [0] arrivals (never reset), [1] arrivals before the current launch, [2] abort, [3] CTAs that left
  float scale;
  uint64_t wait_ns;
  int* err;
};

struct Shared {               // small control block behind the data regions
  uint64_t mbar;              // completion of the row copies
  int flag;                   // result of the last grid barrier
  int abort_flag;
  uint32_t copies;            // row-copy batches issued so far (mbarrier phase)
};

enum { EPI_BIAS = 0, EPI_RESID = 1, EPI_GELU = 2, EPI_PLAIN = 3 };

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ldg_stream(const void* p) {      // read-once weights: do not keep them in L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void bulk_row(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Activations are written by other CTAs earlier in the same launch: read them past L1.
__device__ __forceinline__ float ld_bf16_cg(const bf16* p) {
  const unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
  return __uint_as_float((uint32_t)u << 16);
}

// Grid-wide barrier number `k` (1, 2, ... within the launch).  bar[0] counts arrivals and is never reset:
// this launch's arrivals start at `base` (bar[1], which the last CTA to leave a launch advances by that
// launch's barriers x CTAs), so a barrier is one atomic and one polled load.
// Returns false when the wait ran out or another CTA has given up.
__device__ __forceinline__ bool grid_barrier(const DecodeParams& p, uint32_t base, int k, Shared* sh) {
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = sh->abort_flag ? 0 : 1;
    // arrive: a release reduction (no value comes back, so nothing waits for the atomic's round trip); it orders
    // the CTA's earlier writes, which the barrier above made visible to this thread, before the increment
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p.bar), "r"(1u) : "memory");
    const uint32_t target = base + (uint32_t)k * gridDim.x;
    uint64_t t0 = 0;
    for (uint32_t it = 0; ok && (int32_t)(ld_acquire_gpu(p.bar) - target) < 0; ++it) {
      if ((it & 255) == 255) {
        if (ld_acquire_gpu(p.bar + 2)) { ok = 0; break; }
        const uint64_t now = kh_globaltimer();
        if (t0 == 0) t0 = now;
        else if (now - t0 > p.wait_ns) { atomicCAS(p.err, 0, 9); ok = 0; break; }
      }
    }
    if (!ok) st_release_gpu(p.bar + 2, 1u);
    sh->flag = ok;
  }
  __syncthreads();
  return sh->flag != 0;
}

struct Lin {
  const bf16* W;        // [N, K] row-major
  const bf16* bias;     // [N] or null
  int N, K;
  const bf16* src;      // activation rows [*, K] (before LayerNorm, if any)
  const int* rows;      // row g of the product is src row rows[g] (null: g)
  const bf16 *ln_w, *ln_b;
  int epi;
  const bf16* resid;    // EPI_RESID: [G, N]
  bf16* out;            // [G, ldo]
  int ldo;
};

// ------------------------------------------------------------------------------------------------
// Activation staging: rows [row0, row0 + rows) of the product's input, columns [k0, k0 + kc), into
// xs[row][kc + PAD], LayerNorm'ed when the phase has `ln_w` (whole rows: k0 = 0, kc = K).
// Two routes.  Few bytes (a handful of rows): plain 16-byte loads past L1, for LayerNorm a warp per row
// with the row held in registers -- one trip to L2.  Many bytes: one bulk copy per row, all in flight
// together (completion on an mbarrier), then LayerNorm in place -- the copy engine's latency is about
// twice a load's, but it does not grow with the number of rows.
// Uniform over the CTA; false when the copies did not arrive.
__device__ __forceinline__ bool stage_rows(bf16* xs, Shared* sh, const DecodeParams& p, const Lin& L, int G, int row0, int rows,
                                           int k0, int kc) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pitch = kc + PAD;
  const int live = min(rows, G - row0);
  const int nch = kc / 8;                     // 16-byte pieces per row
  if (live <= 0) return true;
  auto src_row = [&](int r) { return L.src + (size_t)(L.rows ? L.rows[row0 + r] : row0 + r) * L.K + k0; };
  const bool direct = L.ln_w ? (live <= WARPS && nch <= 128) : (live * nch <= 4 * THREADS);
  if (direct && !L.ln_w) {
    const int total = live * nch;
    uint4 t[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < total) t[i] = __ldcg(reinterpret_cast<const uint4*>(src_row(idx / nch)) + idx % nch);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int idx = threadIdx.x + i * THREADS;
      if (idx < total) reinterpret_cast<uint4*>(xs + (size_t)(idx / nch) * pitch)[idx % nch] = t[i];
    }
    __syncthreads();
    return true;
  }
  if (direct) {               // LayerNorm, at most one row per warp, row in registers (four pieces per lane)
    if (warp < live) {
      const uint4* xr = reinterpret_cast<const uint4*>(src_row(warp));
      uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)warp * pitch);
      const uint4 z = make_uint4(0, 0, 0, 0);
      const uint4 u0 = lane < nch ? __ldcg(xr + lane) : z, u1 = lane + 32 < nch ? __ldcg(xr + lane + 32) : z;
      const uint4 u2 = lane + 64 < nch ? __ldcg(xr + lane + 64) : z, u3 = lane + 96 < nch ? __ldcg(xr + lane + 96) : z;
      auto sum8 = [](uint4 v) {
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
        return (a.x + a.y) + (b.x + b.y) + (cc.x + cc.y) + (e.x + e.y);
      };
      const float mean = warp_sum(((sum8(u0) + sum8(u1)) + sum8(u2)) + sum8(u3)) / (float)kc;
      auto dev8 = [&](uint4 v) {
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
        const float d0 = a.x - mean, d1 = a.y - mean, d2 = b.x - mean, d3 = b.y - mean, d4 = cc.x - mean, d5 = cc.y - mean,
                    d6 = e.x - mean, d7 = e.y - mean;
        return d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3 + d4 * d4 + d5 * d5 + d6 * d6 + d7 * d7;
      };
      float sq = 0.f;
      if (lane < nch) sq += dev8(u0);
      if (lane + 32 < nch) sq += dev8(u1);
      if (lane + 64 < nch) sq += dev8(u2);
      if (lane + 96 < nch) sq += dev8(u3);
      const float rstd = rsqrtf(warp_sum(sq) / (float)kc + 1e-5f);
      auto n2 = [&](uint32_t x2, uint32_t w2, uint32_t b2) {
        const float2 xv = unpack_bf16(x2), wv = unpack_bf16(w2), bv = unpack_bf16(b2);
        return pack_bf16((xv.x - mean) * rstd * wv.x + bv.x, (xv.y - mean) * rstd * wv.y + bv.y);
      };
      auto norm8 = [&](uint4 v, int c) {
        const uint4 gw = __ldg(reinterpret_cast<const uint4*>(L.ln_w) + c), gb = __ldg(reinterpret_cast<const uint4*>(L.ln_b) + c);
        return make_uint4(n2(v.x, gw.x, gb.x), n2(v.y, gw.y, gb.y), n2(v.z, gw.z, gb.z), n2(v.w, gw.w, gb.w));
      };
      if (lane < nch) dst[lane] = norm8(u0, lane);
      if (lane + 32 < nch) dst[lane + 32] = norm8(u1, lane + 32);
      if (lane + 64 < nch) dst[lane + 64] = norm8(u2, lane + 64);
      if (lane + 96 < nch) dst[lane + 96] = norm8(u3, lane + 96);
    }
    __syncthreads();
    return true;
  }
  // ---- bulk route
  const uint32_t bar = smem_u32(&sh->mbar);
  if (threadIdx.x == 0) {
    asm volatile("fence.proxy.async;" ::: "memory");     // earlier generic accesses (barrier acquire, reads of xs) before the copies
    mbar_expect_tx(bar, (uint32_t)live * (uint32_t)kc * 2u);
    for (int r = 0; r < live; r++) bulk_row(smem_u32(xs + (size_t)r * pitch), src_row(r), (uint32_t)kc * 2u, bar);
  }
  const uint32_t parity = sh->copies & 1u;
  const bool ok = mbar_wait(bar, parity, &sh->abort_flag, 10, p.err);
  __syncthreads();
  if (threadIdx.x == 0) sh->copies++;
  if (!ok) return false;
  if (L.ln_w) {
    for (int r = warp; r < live; r += WARPS) {
      uint4* row = reinterpret_cast<uint4*>(xs + (size_t)r * pitch);
      float sum = 0.f;
      for (int c = lane; c < nch; c += 32) {
        const uint4 v = row[c];
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
        sum += (a.x + a.y) + (b.x + b.y) + (cc.x + cc.y) + (e.x + e.y);
      }
      sum = warp_sum(sum);
      const float mean = sum / (float)kc;
      float sq = 0.f;
      for (int c = lane; c < nch; c += 32) {
        const uint4 v = row[c];
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
        const float d0 = a.x - mean, d1 = a.y - mean, d2 = b.x - mean, d3 = b.y - mean, d4 = cc.x - mean, d5 = cc.y - mean,
                    d6 = e.x - mean, d7 = e.y - mean;
        sq += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3 + d4 * d4 + d5 * d5 + d6 * d6 + d7 * d7;
      }
      sq = warp_sum(sq);
      const float rstd = rsqrtf(sq / (float)kc + 1e-5f);
      for (int c = lane; c < nch; c += 32) {
        const uint4 v = row[c];
        const uint4 gw = __ldg(reinterpret_cast<const uint4*>(L.ln_w) + c), gb = __ldg(reinterpret_cast<const uint4*>(L.ln_b) + c);
        auto n2 = [&](uint32_t x2, uint32_t w2, uint32_t b2) {
          const float2 xv = unpack_bf16(x2), wv = unpack_bf16(w2), bv = unpack_bf16(b2);
          return pack_bf16((xv.x - mean) * rstd * wv.x + bv.x, (xv.y - mean) * rstd * wv.y + bv.y);
        };
        row[c] = make_uint4(n2(v.x, gw.x, gb.x), n2(v.y, gw.y, gb.y), n2(v.z, gw.z, gb.z), n2(v.w, gw.w, gb.w));
      }
    }
  }
  __syncthreads();
  return true;
}

__device__ __forceinline__ int lin_S(int K) { return min(WARPS, K / KW); }

// this lane's sixteen 16-byte pieces of weight rows [8u, 8u + 8), K slice [k0, k0 + KW)
__device__ __forceinline__ void load_w(uint4 (&w)[NLD], const Lin& L, int u, int k0) {
  const int lane = threadIdx.x & 31;
  const int n = u * 8 + (lane >> 2);
  if (u >= 0 && n < L.N) {
    const bf16* p = L.W + (size_t)n * L.K + k0 + (lane & 3) * 8;
#pragma unroll
    for (int j = 0; j < NLD; j++) w[j] = ldg_stream(p + j * 32);
  } else {
#pragma unroll
    for (int j = 0; j < NLD; j++) w[j] = make_uint4(0, 0, 0, 0);
  }
}

// first work unit of this warp in a linear phase (-1: none) and its first K slice
__device__ __forceinline__ int first_unit(const Lin& L) {
  const int S = lin_S(L.K), U = WARPS / S, warp = threadIdx.x >> 5;
  const int u = (int)blockIdx.x * U + warp / S;
  return u * 8 < L.N ? u : -1;
}
__device__ __forceinline__ int first_k0(const Lin& L) {
  const int S = lin_S(L.K), warp = threadIdx.x >> 5;
  return (warp % S) * KW;
}

// One linear phase over G rows.  `w` holds the weights of (first unit, sub-step 0) when `have_w`.
// Uniform over the CTA; false when a row copy did not arrive.
__device__ __forceinline__ bool linear_phase(const DecodeParams& p, const Lin& L, int G, bf16* xs, float* red, Shared* sh,
                                             uint4 (&w)[NLD], bool have_w) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int S = lin_S(L.K), U = WARPS / S;
  const int nsub = L.K / (S * KW);
  const int GP = G > 16 ? 32 : 16;
  // rows and K range resident in shared memory at a time
  int RP = GP, kc = L.K;
  if ((size_t)RP * (kc + PAD) * 2 > XS_BYTES) RP = 16;
  const bool whole_k = (size_t)RP * (kc + PAD) * 2 <= XS_BYTES;
  if (!whole_k) kc = S * KW;                 // one sub-step's K range at a time (never needed together with LayerNorm)
  const int npass = GP / RP;
  const int pitch = kc + PAD;
  const int n_units = (L.N + 7) / 8;
  const int rounds = (n_units + (int)gridDim.x * U - 1) / ((int)gridDim.x * U);
  const int ul = warp / S, ks = warp % S;
  int staged_pass = -1, staged_sub = -1;
  int flip = 0;
  for (int r = 0; r < rounds; r++) {
    const int unit0 = (r * (int)gridDim.x + (int)blockIdx.x) * U;
    const int u = unit0 + ul;
    const bool live = u < n_units;
    for (int pass = 0; pass < npass; pass++) {
      const int rows_live = min(RP, G - pass * RP);          // rows of this pass that exist
      const int n_out = U * max(rows_live, 0) * 8;           // outputs of this CTA and turn: (unit, row, column)
      // epilogue operands of this thread's outputs: fetched now, used after the products
      float e_bias[MAXQ], e_res[MAXQ];
#pragma unroll
      for (int q = 0; q < MAXQ; q++) {
        e_bias[q] = 0.f; e_res[q] = 0.f;
        const int o = tid + q * THREADS;
        if (o < n_out) {
          const int n8 = o & 7, row = (o >> 3) % rows_live, uu = o / (rows_live * 8);
          const int g = pass * RP + row, col = (unit0 + uu) * 8 + n8;
          if (col < L.N) {
            if (L.bias) e_bias[q] = __bfloat162float(L.bias[col]);
            if (L.epi == EPI_RESID) e_res[q] = ld_bf16_cg(L.resid + (size_t)g * L.N + col);
          }
        }
      }
      float acc[2][4];
#pragma unroll
      for (int m = 0; m < 2; m++)
#pragma unroll
        for (int i = 0; i < 4; i++) acc[m][i] = 0.f;
      for (int sub = 0; sub < nsub; sub++) {
        const int k0 = (sub * S + ks) * KW;
        const bool keep = have_w && r == 0 && sub == 0 && (pass == 0 || nsub == 1);
        if (!keep && !(nsub == 1 && pass > 0)) load_w(w, L, live ? u : -1, k0);
        const int want_sub = whole_k ? 0 : sub;
        if (staged_pass != pass || staged_sub != want_sub) {
          __syncthreads();                    // everybody is done with the rows staged before
          if (!stage_rows(xs, sh, p, L, G, pass * RP, RP, whole_k ? 0 : sub * S * KW, kc)) return false;
          staged_pass = pass; staged_sub = want_sub;
        }
        if (live) {
          const int kx = (whole_k ? k0 : ks * KW) + (lane & 3) * 8;       // column inside xs of this lane's first piece
          const bf16* xa = xs + (size_t)(lane >> 2) * pitch + kx;
#pragma unroll
          for (int j = 0; j < NLD; j++) {
#pragma unroll
            for (int m = 0; m < 2; m++) {
              if (m * 16 >= RP) break;
              const uint4 a = *reinterpret_cast<const uint4*>(xa + (size_t)(m * 16) * pitch + j * 32);
              const uint4 b = *reinterpret_cast<const uint4*>(xa + (size_t)(m * 16 + 8) * pitch + j * 32);
              mma_bf16(acc[m], a.x, b.x, a.y, b.y, w[j].x, w[j].y);
              mma_bf16(acc[m], a.z, b.z, a.w, b.w, w[j].z, w[j].w);
            }
          }
        }
      }
      // partial tiles -> shared memory; thread (unit, row, column) adds the S slices in order
      float* rb = red + flip * RED_FLOATS;
      flip ^= 1;
#pragma unroll
      for (int m = 0; m < 2; m++) {
        if (m * 16 >= RP) break;
        float* t = rb + ((size_t)warp * 32 + m * 16 + (lane >> 2)) * 8 + (lane & 3) * 2;
        t[0] = acc[m][0]; t[1] = acc[m][1];
        t[64] = acc[m][2]; t[65] = acc[m][3];          // row + 8
      }
      __syncthreads();
#pragma unroll
      for (int q = 0; q < MAXQ; q++) {
        const int o = tid + q * THREADS;
        if (o >= n_out) break;
        const int n8 = o & 7, row = (o >> 3) % rows_live, uu = o / (rows_live * 8);
        const int g = pass * RP + row, col = (unit0 + uu) * 8 + n8;
        if (col >= L.N) continue;
        float v = 0.f;
        for (int s = 0; s < S; s++) v += rb[((size_t)(uu * S + s) * 32 + row) * 8 + n8];
        v += e_bias[q];
        if (L.epi == EPI_RESID) v += e_res[q];
        else if (L.epi == EPI_GELU) v = gelu_tanh(__bfloat162float(__float2bfloat16(v)));
        L.out[(size_t)g * L.ldo + col] = __float2bfloat16(v);
      }
    }
    have_w = false;
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
// Phase B: one (sequence, head) item per CTA and turn.  Appends the new k, v (from qkv) to the paged
// cache, then attends over positions 0..pos (the structure of paged_attn_k with 256 threads).
template <int HD>
__device__ void attention_phase(const DecodeParams& p, int layer, float* sm) {
  constexpr int TPR = HD / 8;                 // threads per value row
  constexpr int GROUPS = THREADS / TPR;       // value rows in flight
  float* s_q = sm;                            // HD
  float* s_red = sm + HD;                     // GROUPS * HD partial outputs
  float* s_w = s_red + GROUPS * HD;           // 8 per-warp reduction slots (+ result)
  float* s_p = s_w + 16;                      // max_ctx scores / probabilities
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int d = p.H * HD;
  bf16* kc = p.kc + (size_t)layer * p.layer_elems;
  bf16* vc = p.vc + (size_t)layer * p.layer_elems;
  for (int item = blockIdx.x; item < p.G * p.H; item += gridDim.x) {
    const int t = item / p.H, h = item % p.H;
    const int pos_t = p.pos[t], slot_t = p.slot[t];
    if (pos_t < 0 || pos_t >= p.max_ctx || pos_t / p.bs >= p.max_lb || slot_t < 0) {     // uniform over the CTA
      if (tid == 0) atomicCAS(p.err, 0, 8);
      continue;
    }
    const int ctx = pos_t + 1;
    const int* bt = p.btab + (size_t)slot_t * p.max_lb;
    const bf16* qrow = p.qkv + (size_t)t * 3 * d;
    for (int e = tid; e < HD; e += THREADS) s_q[e] = ld_bf16_cg(qrow + h * HD + e) * p.scale;
    if (tid < 2 * TPR) {
      const int which = tid / TPR, c = (tid % TPR) * 8;
      const size_t dst = ((size_t)bt[pos_t / p.bs] * p.bs + (pos_t % p.bs)) * d + h * HD + c;
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(qrow + (which + 1) * d + h * HD + c));
      *reinterpret_cast<uint4*>((which ? vc : kc) + dst) = v;
    }
    __syncthreads();
    float lmax = -INFINITY;
    for (int j = tid; j < ctx; j += THREADS) {
      const bf16* kp = kc + ((size_t)bt[j / p.bs] * p.bs + (j % p.bs)) * d + h * HD;
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        const uint4 v = *reinterpret_cast<const uint4*>(kp + c);
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
        acc += a.x * s_q[c] + a.y * s_q[c + 1] + b.x * s_q[c + 2] + b.y * s_q[c + 3] + cc.x * s_q[c + 4] +
               cc.y * s_q[c + 5] + e.x * s_q[c + 6] + e.y * s_q[c + 7];
      }
      s_p[j] = acc;
      lmax = fmaxf(lmax, acc);
    }
    lmax = warp_max(lmax);
    if (lane == 0) s_w[warp] = lmax;
    __syncthreads();
    float gmax = s_w[0];
#pragma unroll
    for (int i = 1; i < WARPS; i++) gmax = fmaxf(gmax, s_w[i]);
    __syncthreads();
    float lsum = 0.f;
    for (int j = tid; j < ctx; j += THREADS) {
      const float e = __expf(s_p[j] - gmax);
      s_p[j] = e;
      lsum += e;
    }
    lsum = warp_sum(lsum);
    if (lane == 0) s_w[warp] = lsum;
    __syncthreads();
    float tot = 0.f;
#pragma unroll
    for (int i = 0; i < WARPS; i++) tot += s_w[i];
    const float inv = 1.f / tot;
    const int c8 = (tid % TPR) * 8, grp = tid / TPR;
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] = 0.f;
    for (int j = grp; j < ctx; j += GROUPS) {
      const uint4 v = *reinterpret_cast<const uint4*>(vc + ((size_t)bt[j / p.bs] * p.bs + (j % p.bs)) * d + h * HD + c8);
      const float pj = s_p[j];
      const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
      acc[0] += pj * a.x; acc[1] += pj * a.y; acc[2] += pj * b.x; acc[3] += pj * b.y;
      acc[4] += pj * cc.x; acc[5] += pj * cc.y; acc[6] += pj * e.x; acc[7] += pj * e.y;
    }
#pragma unroll
    for (int k = 0; k < 8; k++) s_red[grp * HD + c8 + k] = acc[k];
    __syncthreads();
    if (tid < HD) {
      float o = 0.f;
      for (int g = 0; g < GROUPS; g++) o += s_red[g * HD + tid];
      p.att[(size_t)t * d + h * HD + tid] = __float2bfloat16(o * inv);
    }
    __syncthreads();               // shared memory is reused by the CTA's next item
  }
}

__device__ void decode_body(const DecodeParams& p, uint8_t* smem, Shared* sh, uint32_t base) {
  bf16* xs = reinterpret_cast<bf16*>(smem);
  float* red = reinterpret_cast<float*>(smem + XS_BYTES);
  const int d = p.d;
  uint4 w[NLD];
  auto lin = [&](const bf16* W, const bf16* b, int N, int K, const bf16* src, const bf16* lw, const bf16* lb, int epi,
                 const bf16* resid, bf16* out) {
    Lin L;
    L.W = W; L.bias = b; L.N = N; L.K = K; L.src = src; L.rows = nullptr; L.ln_w = lw; L.ln_b = lb; L.epi = epi;
    L.resid = resid; L.out = out; L.ldo = N;
    return L;
  };
  Lin head = lin(p.head_w, nullptr, p.V, d, p.x, p.lnf_w, p.lnf_b, EPI_PLAIN, nullptr, p.logits);
  head.rows = p.rows; head.ldo = p.ld_logits;
  {
    const LayerW& lw = p.layers[0];
    const Lin a = lin(lw.qkv_w, lw.qkv_b, 3 * d, d, p.x, lw.ln1_w, lw.ln1_b, EPI_BIAS, nullptr, p.qkv);
    load_w(w, a, first_unit(a), first_k0(a));
  }
  int k = 0;
  for (int l = 0; l < p.L; l++) {
    const LayerW lw = p.layers[l];
    const Lin a = lin(lw.qkv_w, lw.qkv_b, 3 * d, d, p.x, lw.ln1_w, lw.ln1_b, EPI_BIAS, nullptr, p.qkv);
    const Lin c = lin(lw.proj_w, lw.proj_b, d, d, p.att, nullptr, nullptr, EPI_RESID, p.x, p.xmid);
    const Lin f = lin(lw.fc_w, lw.fc_b, 4 * d, d, p.xmid, lw.ln2_w, lw.ln2_b, EPI_GELU, nullptr, p.act);
    const Lin e = lin(lw.fcproj_w, lw.fcproj_b, d, 4 * d, p.act, nullptr, nullptr, EPI_RESID, p.xmid, p.x);
    if (!linear_phase(p, a, p.G, xs, red, sh, w, true)) return;
    if (!grid_barrier(p, base, ++k, sh)) return;
    if (p.hd == 128) attention_phase<128>(p, l, reinterpret_cast<float*>(smem));
    else attention_phase<64>(p, l, reinterpret_cast<float*>(smem));
    load_w(w, c, first_unit(c), first_k0(c));           // lands while the barrier is crossed
    if (!grid_barrier(p, base, ++k, sh)) return;
    if (!linear_phase(p, c, p.G, xs, red, sh, w, true)) return;
    load_w(w, f, first_unit(f), first_k0(f));
    if (!grid_barrier(p, base, ++k, sh)) return;
    if (!linear_phase(p, f, p.G, xs, red, sh, w, true)) return;
    load_w(w, e, first_unit(e), first_k0(e));
    if (!grid_barrier(p, base, ++k, sh)) return;
    if (!linear_phase(p, e, p.G, xs, red, sh, w, true)) return;
    if (l + 1 < p.L) {
      const LayerW& nw = p.layers[l + 1];
      const Lin na = lin(nw.qkv_w, nw.qkv_b, 3 * d, d, p.x, nw.ln1_w, nw.ln1_b, EPI_BIAS, nullptr, p.qkv);
      load_w(w, na, first_unit(na), first_k0(na));
      if (!grid_barrier(p, base, ++k, sh)) return;
    } else if (p.head_w) {
      load_w(w, head, first_unit(head), first_k0(head));
      if (!grid_barrier(p, base, ++k, sh)) return;
      if (!linear_phase(p, head, p.n_rows, xs, red, sh, w, true)) return;
    }
  }
}

constexpr int SMEM_BYTES = XS_BYTES + 2 * RED_FLOATS * 4 + 64;

__global__ void __launch_bounds__(THREADS, 1) decode_layers_k(const DecodeParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  Shared* sh = reinterpret_cast<Shared*>(smem + XS_BYTES + 2 * RED_FLOATS * 4);
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sh->mbar), 1);
    mbar_fence_init();
    sh->flag = 1; sh->abort_flag = 0; sh->copies = 0;
  }
  __syncthreads();
  // arrivals before this launch: constant while it runs (only its last CTA to leave advances the word)
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(p.bar + 1);
  decode_body(p, smem, sh, base);
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.bar + 3, 1u) == gridDim.x - 1) {
      p.bar[3] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.bar + 1) = base + (uint32_t)(5 * p.L - 1 + (p.head_w ? 1 : 0)) * gridDim.x;
    }
  }
}

int g_grid = 0;

}  // namespace

// The decode batch sizes and model shapes the persistent decode kernel accepts.
extern "C" int kh_decode_layers_ok(int G, int d, int H, int hd, int max_ctx) {
  if (G < 1 || G > 32 || d % KW || d > 4096 || H * hd != d || (hd != 64 && hd != 128)) return 0;
  if ((size_t)(hd + (THREADS / (hd / 8)) * hd + 16 + max_ctx) * 4 > (size_t)XS_BYTES) return 0;
  for (int K = d; K <= 4 * d; K *= 4) {         // K / 512 warps share a unit: 1, 2, 4, 8, or whole sub-steps of 8
    const int q = K / KW;
    if (!(q == 1 || q == 2 || q == 4 || q % WARPS == 0)) return 0;
  }
  return 1;
}

// x [G, d] holds the embedded tokens on entry and the last layer's output on return.  `layers`: device
// array of L records of twelve bf16 pointers (ln1_w, ln1_b, qkv_w, qkv_b, proj_w, proj_b, ln2_w, ln2_b,
// fc_w, fc_b, fcproj_w, fcproj_b).  With `head_w` ([V, d]) the kernel also writes
// logits[i, :V] = LNf(x[rows[i]]) head_w^T for i < n_rows (row pitch ld_logits).  `bar`: four
// zero-initialised words in device memory that nothing else in flight uses.  Returns 0 or -1.
extern "C" int kh_decode_layers(void* x, void* xmid, void* qkv, void* att, void* act, const void* layers, int L, int G,
                                int d, int H, int hd, void* kc, void* vc, long layer_elems, const void* pos,
                                const void* slot, const void* btab, int max_lb, int bs, int max_ctx, float scale,
                                const void* head_w, const void* lnf_w, const void* lnf_b, void* logits, int ld_logits, int V,
                                const void* rows, int n_rows, void* bar, void* stream) {
  if (!kh_decode_layers_ok(G, d, H, hd, max_ctx)) { kh_set_error("decode_layers: unsupported shape G=%d d=%d H=%d hd=%d", G, d, H, hd); return -1; }
  if (head_w && (!lnf_w || !lnf_b || !logits || !rows || n_rows < 1 || n_rows > 32 || V < 1 || ld_logits < V)) {
    kh_set_error("decode_layers: incomplete head arguments");
    return -1;
  }
  if (!g_grid) {
    cudaError_t e = cudaFuncSetAttribute(decode_layers_k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) { kh_set_error("decode_layers: shared memory opt-in failed: %s", cudaGetErrorString(e)); return -1; }
    int dev = 0, sms = 0, per = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per, decode_layers_k, THREADS, SMEM_BYTES);
    if (e != cudaSuccess || per < 1 || sms < 1) { kh_set_error("decode_layers: the kernel does not fit on an SM"); return -1; }
    g_grid = sms;                 // one CTA per SM: all of them resident, as the grid barrier requires
  }
  DecodeParams p = {};
  p.G = G; p.d = d; p.H = H; p.hd = hd; p.L = L; p.bs = bs; p.max_lb = max_lb; p.max_ctx = max_ctx;
  p.layers = (const LayerW*)layers;
  p.x = (bf16*)x; p.xmid = (bf16*)xmid; p.qkv = (bf16*)qkv; p.att = (bf16*)att; p.act = (bf16*)act;
  p.kc = (bf16*)kc; p.vc = (bf16*)vc; p.layer_elems = (size_t)layer_elems;
  p.pos = (const int*)pos; p.slot = (const int*)slot; p.btab = (const int*)btab;
  p.head_w = (const bf16*)head_w; p.lnf_w = (const bf16*)lnf_w; p.lnf_b = (const bf16*)lnf_b;
  p.logits = (bf16*)logits; p.ld_logits = ld_logits; p.V = V; p.rows = (const int*)rows; p.n_rows = n_rows;
  p.bar = (uint32_t*)bar; p.scale = scale;
  p.wait_ns = KH_WAIT_LIMIT_NS;
  p.err = kh_error_word_dev();
  // cooperative launch: the driver guarantees that all CTAs are resident together (or refuses the launch)
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g_grid); cfg.blockDim = dim3(THREADS); cfg.dynamicSmemBytes = SMEM_BYTES; cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeCooperative;
  at[0].val.cooperative = 1;
  cfg.attrs = at; cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, decode_layers_k, p);
  if (e != cudaSuccess) { kh_set_error("decode_layers launch failed: %s", cudaGetErrorString(e)); return -1; }
  return 0;
}
