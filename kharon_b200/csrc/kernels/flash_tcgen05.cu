// Causal FlashAttention forward and backward on tcgen05 tensor cores (sm_100a).
//
// Operates directly on the fused projection buffer qkv [B*T, 3*H*hd] (q | k | v, head-major
// inside each third) and writes merged-head outputs [B*T, H*hd], so the reference's head
// split / merge / unmerge / combine kernels (src/core/kernels.cu:189-228, 468-509) have no
// counterpart here: the strides are folded into the TMA tensor maps.  Replaces
// src/kernels/flash.cu:26-199 (warp-per-row SIMT) and its per-call cudaMalloc (:201-229).
//
// Tiles are [rows x hd] bf16, stored in shared memory as hd/64 slabs of rows x 128 bytes with
// the 128-byte swizzle, exactly as TMA writes them.  The same slab is used as a K-major
// operand (contraction over hd) or as an MN-major operand (contraction over rows) just by
// changing the UMMA descriptor -- e.g. V for O = P V, dO for dV = P^T dO, Q for dK = dS^T Q.
//
// All three kernels are persistent and warp-specialised: a TMA warp streams operand tiles through
// mbarrier-guarded rings, one lane of an MMA warp issues every tcgen05.mma, and the remaining warps
// own the rows of the CTA's tile (softmax in the forward pass, P / dS in the backward pass).  S, dP
// and the accumulators (O; dK and dV; dQ) live in TMEM; finished tiles are staged in shared memory
// and written with TMA stores.  Details stand in front of each kernel.
// backward  delta = rowsum(dO * O); a dK/dV kernel per key tile and a dQ kernel per query tile.
//           No atomics: every output element is produced by exactly one CTA in a fixed order, so
//           gradients are reproducible bit for bit.
//
// All mbarrier waits are bounded (error word code 6); after a timeout the CTA skips its
// stores, releases TMEM and returns.
#include "common.cuh"

#define KH_LAUNCH_CHECK(name)                                                     \
  do {                                                                            \
    cudaError_t e_ = cudaGetLastError();                                          \
    if (e_ != cudaSuccess) { kh_set_error(name ": %s", cudaGetErrorString(e_)); return -1; } \
  } while (0)

namespace {

constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
  int B, T, H;
  int ld;            // row pitch of qkv / dqkv in elements
  float scale;       // 1/sqrt(hd)
  bf16* out;         // fwd: O [B*T, H*hd];          bwd: unused
  float* lse;        // [B, H, T] natural-log LSE of the scaled scores
  const bf16* o;     // bwd (delta): forward output
  const bf16* dout;  // bwd: dO [B*T, H*hd]
  float* delta;      // [B, H, T]
  bf16* dqkv;        // bwd output
  int* err;
};

// [rows x hd] tile: hd/64 slabs of rows x 128 B
template <int HD>
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* m, uint32_t bar, int col0, int row0, int rows) {
#pragma unroll
  for (int s = 0; s < HD / 64; s++) tma_load_2d(dst + s * rows * 128, m, bar, col0 + s * 64, row0);
}
// UMMA descriptors.  Contraction over the tile's columns (K-major): k-step kk of 16 columns starts
// (kk >> 2) slabs + (kk & 3) * 32 bytes into the tile.  Contraction over the tile's rows (MN-major):
// k-step kk of 16 rows starts kk * 2048 bytes in, slabs are `rows * 128` bytes apart (LBO).
// The MMA warp's single lane issues every product of a CTA, so its instruction count per tcgen05.mma
// bounds the rate: descriptors are built once per tile (dk0 / dmn0) and advanced by compile-time
// constants per k-step (one 64-bit add each).
__device__ __forceinline__ uint64_t dk0(uint32_t base) { return umma_desc_sw128(base, 16, 1024); }
__device__ __forceinline__ uint64_t dmn0(uint32_t base, int rows) { return umma_desc_sw128(base, rows * 128, 1024); }
#define DK(d0, rows, kk) ((d0) + (uint64_t)((((kk) >> 2) * (rows) * 128 + ((kk) & 3) * 32) >> 4))
#define DMN(d0, kk) ((d0) + (uint64_t)(((kk) * 2048) >> 4))
// address of the 16-byte chunk (row, chunk c of 8 bf16) in a K-major tile with `rows` rows
__device__ __forceinline__ uint32_t chunk_addr(uint32_t base, int rows, int row, int c) {
  return base + (c >> 3) * rows * 128 + row * 128 + (((c & 7) ^ (row & 7)) << 4);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ================================================================================ forward, warp-specialised
// Persistent CTAs of six warps, two CTAs per SM.  A work item is (batch, head, 128 consecutive
// queries), one thread of warps 0-3 per query row.  Warp 4 streams the Q tile and a two-stage ring of
// (K, V) tiles of 64 keys with TMA; one lane of warp 5 issues every tcgen05.mma.  Per key tile j:
//
//   S(j) = Q K_j^T  -> TMEM (two S buffers)        MMA warp, as soon as K_j has landed
//   softmax warps:     read S(j), online softmax, P(j) -> shared memory (bf16)
//   O   += P(j) V_j   accumulated in TMEM           MMA warp, when P(j) is ready
//
// S(j+1) is already in TMEM when the softmax of tile j ends, and the second CTA of the SM keeps the
// tensor cores and the exponential unit busy while this one waits, loads or stores.  O stays in TMEM
// for the whole item; when a row's running maximum grows by more than 2^8 the row is rescaled in
// place (tcgen05.ld / st), otherwise the older maximum stays the reference of the exponentials,
// which keeps the result exact (the normaliser uses the same reference) and makes rescaling rare
// after the first tiles.  Items are handed out longest first (most key tiles).
template <int HD>
struct FwdWs {
  static constexpr int BQ = 128, BKV = 64, NS = 2;
  static constexpr int Q_BYTES = BQ * HD * 2, KV_BYTES = BKV * HD * 2, P_BYTES = BQ * BKV * 2;
  static constexpr int DATA = Q_BYTES + NS * 2 * KV_BYTES + P_BYTES;
  static constexpr int SMEM = DATA + 256;      // the tiles start at the (1024-byte aligned) base of dynamic shared memory
  static constexpr int THREADS = 192, TMEM_COLS = 256;     // S: 2 x 64 columns, O: HD columns from 128
};

template <int HD>
__global__ void __launch_bounds__(192, 2)
flash_fwd_ws_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                    const __grid_constant__ CUtensorMap map_o, const AttnParams p, int n_items, int n_qt) {
  using C = FwdWs<HD>;
  constexpr int BQ = C::BQ, BKV = C::BKV, NS = C::NS;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sQ = base, sKV = sQ + C::Q_BYTES, sP = sKV + NS * 2 * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + C::DATA);
  const uint32_t b0 = smem_u32(bars);
  // K and V stages are released separately: a K stage as soon as S(j) has retired, a V stage after PV(j)
  const uint32_t bar_qfull = b0, bar_qfree = b0 + 8, bar_kfull = b0 + 16, bar_kfree = bar_kfull + 8 * NS,
                 bar_vfull = bar_kfree + 8 * NS, bar_vfree = bar_vfull + 8 * NS,
                 bar_sfull = bar_vfree + 8 * NS, bar_pready = bar_sfull + 16, bar_odone = bar_pready + 8,
                 bar_ofree = bar_odone + 8, bar_epi = bar_ofree + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 + 4 * NS + 2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(bar_qfull, 1); mbar_init(bar_qfree, 1);
    for (int s = 0; s < NS; s++) {
      mbar_init(bar_kfull + 8 * s, 1); mbar_init(bar_kfree + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1); mbar_init(bar_vfree + 8 * s, 1);
    }
    mbar_init(bar_sfull, 1); mbar_init(bar_sfull + 8, 1);
    mbar_init(bar_pready, 4); mbar_init(bar_odone, 1); mbar_init(bar_ofree, 4); mbar_init(bar_epi, 128);
    *abort_flag = (base & 1023u) ? 6 : 0;       // swizzled tiles need the 1024-byte alignment
    if (base & 1023u) atomicCAS(p.err, 0, 6);
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kv);
    tma_prefetch_desc(&map_o);
  }
  if (warp == 5) { tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();

  const int d = p.H * HD, BH = p.B * p.H;
  // item w -> (query tile, batch, head); the tiles that see the most keys come first
  auto decode = [&](int w, int& b, int& h, int& q0, int& n) {
    const int qt = n_qt - 1 - w / BH, bh = w % BH;
    b = bh / p.H; h = bh % p.H; q0 = qt * BQ;
    n = (min(q0 + BQ, p.T) + BKV - 1) / BKV;
  };
  const bool live = *abort_flag == 0;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && live) {
      int ic = 0, kvc = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x, ic++) {
        int b, h, q0, n;
        decode(w, b, h, q0, n);
        if (!mbar_wait(bar_qfree, (ic & 1) ^ 1, abort_flag, 6, p.err)) break;
        mbar_expect_tx(bar_qfull, C::Q_BYTES);
        load_tile<HD>(sQ, &map_q, bar_qfull, h * HD, b * p.T + q0, BQ);
        for (int j = 0; j < n; j++, kvc++) {
          const int s = kvc % NS;
          const uint32_t par = ((kvc / NS) & 1) ^ 1;
          const uint32_t sk = sKV + s * 2 * C::KV_BYTES, sv = sk + C::KV_BYTES;
          if (!mbar_wait(bar_kfree + 8 * s, par, abort_flag, 6, p.err)) { ok = false; break; }
          mbar_expect_tx(bar_kfull + 8 * s, C::KV_BYTES);
          load_tile<HD>(sk, &map_kv, bar_kfull + 8 * s, d + h * HD, b * p.T + j * BKV, BKV);
          if (!mbar_wait(bar_vfree + 8 * s, par, abort_flag, 6, p.err)) { ok = false; break; }
          mbar_expect_tx(bar_vfull + 8 * s, C::KV_BYTES);
          load_tile<HD>(sv, &map_kv, bar_vfull + 8 * s, 2 * d + h * HD, b * p.T + j * BKV, BKV);
        }
      }
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && live) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BKV, 0, 0);
      constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
      int ic = 0, pc = 0, kvc = 0;
      bool ok = true;
      const uint64_t dQ0 = dk0(sQ), dP0 = dk0(sP);
      for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x, ic++) {
        int b, h, q0, n;
        decode(w, b, h, q0, n);
        if (!mbar_wait(bar_qfull, ic & 1, abort_flag, 6, p.err)) break;
        const int kv_base = kvc;
        for (int j = 0; j <= n && ok; j++) {
          if (j < n) {
            const int s = kvc % NS;
            if (!mbar_wait(bar_kfull + 8 * s, (kvc / NS) & 1, abort_flag, 6, p.err)) { ok = false; break; }
            kvc++;
            tc_fence_after();
            const uint32_t sk = sKV + s * 2 * C::KV_BYTES;
            const uint32_t tS = tmem + (j & 1) * 64;
            const uint64_t dK0 = dk0(sk);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, DK(dQ0, BQ, kk), DK(dK0, BKV, kk), idesc_s, kk > 0);
            umma_commit(bar_sfull + 8 * (j & 1));
            umma_commit(bar_kfree + 8 * s);
            if (j == n - 1) umma_commit(bar_qfree);         // last use of this item's Q
          }
          if (j >= 1) {
            const int jj = j - 1;
            const int s = (kv_base + jj) % NS;
            const uint32_t sv = sKV + s * 2 * C::KV_BYTES + C::KV_BYTES;
            if (!mbar_wait(bar_vfull + 8 * s, ((kv_base + jj) / NS) & 1, abort_flag, 6, p.err)) { ok = false; break; }
            // the previous item's O has been read out
            if (jj == 0 && !mbar_wait(bar_ofree, (ic & 1) ^ 1, abort_flag, 6, p.err)) { ok = false; break; }
            if (!mbar_wait(bar_pready, pc & 1, abort_flag, 6, p.err)) { ok = false; break; }
            pc++;
            tc_fence_after();
            const uint64_t dV0 = dmn0(sv, BKV);
#pragma unroll
            for (int kk = 0; kk < BKV / 16; kk++)
              umma_f16_ss(tmem + 128, DK(dP0, BQ, kk), DMN(dV0, kk), idesc_o, (jj > 0 || kk > 0));
            umma_commit(bar_odone);
            umma_commit(bar_vfree + 8 * s);
          }
        }
      }
    }
  } else if (live) {
    // ------------------------------------------------------------------ softmax warps
    const int row = tid;
    const uint32_t lane_off = (uint32_t)(warp * 32) << 16;
    const uint32_t tO = tmem + 128 + lane_off;
    const float sl2 = p.scale * LOG2E;
    int sfc[2] = {0, 0}, odc = 0, epc = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x) {
      int b, h, q0, n;
      decode(w, b, h, q0, n);
      const int qpos = q0 + row;
      float m_ref = -INFINITY, l_run = 0.f;     // reference maximum (scaled to log2 units) and normaliser
      for (int j = 0; j < n; j++) {
        const int buf = j & 1;
        if (!mbar_wait(bar_sfull + 8 * buf, sfc[buf] & 1, abort_flag, 6, p.err)) { ok = false; break; }
        sfc[buf]++;
        tc_fence_after();
        uint32_t r[64];
        const uint32_t tS = tmem + buf * 64 + lane_off;
        tmem_ld32(tS, r);
        tmem_ld32(tS + 32, r + 32);
        tmem_ld_wait();
        const int k0 = j * BKV;
        if (k0 + BKV - 1 > q0) {               // tile touches the diagonal: mask keys after the query
#pragma unroll
          for (int i = 0; i < 64; i++)
            if (k0 + i > qpos) r[i] = 0xff800000u;
        }
        // maximum of the raw scores over four independent chains (the scale is positive)
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          mx[0] = fmaxf(mx[0], __uint_as_float(r[i])); mx[1] = fmaxf(mx[1], __uint_as_float(r[i + 1]));
          mx[2] = fmaxf(mx[2], __uint_as_float(r[i + 2])); mx[3] = fmaxf(mx[3], __uint_as_float(r[i + 3]));
        }
        const float mt = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sl2;
        bool waited = false;
        if (j == 0) {
          m_ref = mt;
        } else {
          const bool grow = mt > m_ref + 8.f;
          if (__any_sync(0xffffffffu, grow)) {
            // rescale O in place: PV(j-1) must have retired, PV(j) is issued only after P(j) below
            if (!mbar_wait(bar_odone, odc & 1, abort_flag, 6, p.err)) { ok = false; break; }
            odc++;
            waited = true;
            tc_fence_after();
            const float alpha = grow ? exp2f(m_ref - mt) : 1.f;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
              uint32_t o[32];
              tmem_ld32(tO + c, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + c, o);
            }
            tmem_st_wait();
            l_run *= alpha;
            if (grow) m_ref = mt;
          }
        }
        float rs[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[32];
        const float nm = -m_ref;
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          const float p0 = exp2f(fmaf(__uint_as_float(r[i]), sl2, nm)), p1 = exp2f(fmaf(__uint_as_float(r[i + 1]), sl2, nm));
          const float p2 = exp2f(fmaf(__uint_as_float(r[i + 2]), sl2, nm)), p3 = exp2f(fmaf(__uint_as_float(r[i + 3]), sl2, nm));
          rs[0] += p0; rs[1] += p1; rs[2] += p2; rs[3] += p3;
          pk[i >> 1] = pack_bf16(p0, p1);
          pk[(i >> 1) + 1] = pack_bf16(p2, p3);
        }
        l_run += (rs[0] + rs[1]) + (rs[2] + rs[3]);
        if (j >= 1 && !waited) {      // PV(j-1) no longer reads the P buffer
          if (!mbar_wait(bar_odone, odc & 1, abort_flag, 6, p.err)) { ok = false; break; }
          odc++;
        }
#pragma unroll
        for (int c = 0; c < 8; c++)
          st_shared_v4(chunk_addr(sP, BQ, row, c), pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_pready);
      }
      if (!ok) break;
      if (!mbar_wait(bar_odone, odc & 1, abort_flag, 6, p.err)) { ok = false; break; }
      odc++;
      tc_fence_after();
      // O tile -> bf16 -> the P buffer (free now) in the swizzled tile layout, 64 columns at a time -> one
      // TMA store per slab; rows past the end of the sequence are clipped by the tensor map
      const float inv = 1.f / l_run;
#pragma unroll 1
      for (int hf = 0; hf < HD / 64; hf++) {
#pragma unroll
        for (int c = 0; c < 64; c += 32) {
          uint32_t o[32];
          tmem_ld32(tO + hf * 64 + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; q++)
            st_shared_v4(chunk_addr(sP, BQ, row, (c >> 3) + q),
                         pack_bf16(__uint_as_float(o[8 * q]) * inv, __uint_as_float(o[8 * q + 1]) * inv),
                         pack_bf16(__uint_as_float(o[8 * q + 2]) * inv, __uint_as_float(o[8 * q + 3]) * inv),
                         pack_bf16(__uint_as_float(o[8 * q + 4]) * inv, __uint_as_float(o[8 * q + 5]) * inv),
                         pack_bf16(__uint_as_float(o[8 * q + 6]) * inv, __uint_as_float(o[8 * q + 7]) * inv));
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_epi);
        if (!mbar_wait(bar_epi, epc & 1, abort_flag, 6, p.err)) { ok = false; break; }
        epc++;
        if (tid == 0) {
          tma_store_3d(&map_o, sP, h * HD + hf * 64, q0, b);
          bulk_commit();
          bulk_wait_read_all();           // the buffer may be overwritten (next slab, next item's P)
        }
        mbar_arrive(bar_epi);
        if (!mbar_wait(bar_epi, epc & 1, abort_flag, 6, p.err)) { ok = false; break; }
        epc++;
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_ofree);
      if (qpos < p.T && p.lse) p.lse[((size_t)b * p.H + h) * p.T + qpos] = (m_ref + log2f(l_run)) / LOG2E;
    }
    if (tid == 0) bulk_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

// ================================================================================ delta
// delta[b,h,t] = sum_e dO[b,t,h,e] * O[b,t,h,e].  One warp per row of O / dO: the lanes read the row in
// 16-byte pieces (512 contiguous bytes per step), a head is HD / 8 adjacent lanes, summed with shuffles.
template <int HD>
__global__ void flash_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, float* __restrict__ delta,
                                   int B, int T, int H) {
  pdl_wait();
  pdl_launch_dependents();
  const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= (long)B * T) return;
  constexpr int LPH = HD / 8;                      // lanes per head
  const int d = H * HD;
  const uint4* a = reinterpret_cast<const uint4*>(o + row * d);
  const uint4* g = reinterpret_cast<const uint4*>(dout + row * d);
  const int b = (int)(row / T), t = (int)(row % T);
  for (int c0 = 0; c0 < d / 8; c0 += 32) {
    const int c = c0 + lane;
    float s = 0.f;
    if (c < d / 8) {
      const uint4 x = __ldg(a + c), y = __ldg(g + c);
      const float2 x0 = unpack_bf16(x.x), x1 = unpack_bf16(x.y), x2 = unpack_bf16(x.z), x3 = unpack_bf16(x.w);
      const float2 y0 = unpack_bf16(y.x), y1 = unpack_bf16(y.y), y2 = unpack_bf16(y.z), y3 = unpack_bf16(y.w);
      s = (x0.x * y0.x + x0.y * y0.y) + (x1.x * y1.x + x1.y * y1.y) + (x2.x * y2.x + x2.y * y2.y) + (x3.x * y3.x + x3.y * y3.y);
    }
#pragma unroll
    for (int off = LPH / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (c < d / 8 && (lane % LPH) == 0) delta[((size_t)b * H + c / LPH) * T + t] = s;
  }
}

// ================================================================================ backward, warp-specialised
// Both backward kernels are persistent (one CTA per SM) with ten warps: eight compute warps (two
// threads per row of the CTA's 128-row tile, each taking 32 of a sub-tile's 64 columns), a TMA warp
// and an MMA warp.  The other sequence dimension is walked in sub-tiles of 64 through a four-stage
// TMA ring, so S and dP take 64 TMEM columns each and fit twice: the MMA warp issues S(t+1),
// dP(t+1) while the compute warps turn S(t), dP(t) into P(t), dS(t), and issues the accumulating
// products of sub-tile t as soon as those are in shared memory.  Gradients stay in TMEM for the
// whole item.  Work items are handed out longest first.
template <int HD>
struct BwdWs {
  static constexpr int BT = 128, BS = 64, NS = 4;
  static constexpr int TILE = BT * HD * 2, SUB = BS * HD * 2, PS_BYTES = BT * BS * 2;
  static constexpr int THREADS = 320, TMEM_COLS = 512;
  // dK/dV: K, V tiles; ring of (Q, dO) sub-tiles; P^T and dS^T; lse / delta of two sub-tiles
  static constexpr int DATA_KV = 2 * TILE + NS * 2 * SUB + 2 * PS_BYTES + 2 * 128 * 4;
  static constexpr int SMEM_KV = DATA_KV + 256;
  // dQ: Q, dO tiles; ring of (K, V) sub-tiles; dS, with 16 KB behind it so that the pair stages the dQ tile
  static constexpr int DATA_Q = 2 * TILE + NS * 2 * SUB + 2 * PS_BYTES;
  static constexpr int SMEM_Q = DATA_Q + 256;
};

// ---- dK, dV: item = (batch, head, 128 keys); sub-tiles of 64 queries from the diagonal to the end
template <int HD>
__global__ void __launch_bounds__(320, 1)
flash_dkv_ws_kernel(const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_q,
                    const __grid_constant__ CUtensorMap map_do, const __grid_constant__ CUtensorMap map_dqkv, const AttnParams p,
                    int n_items, int n_kt) {
  using C = BwdWs<HD>;
  constexpr int BT = C::BT, BS = C::BS, NS = C::NS;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sK = base, sV = sK + C::TILE, sQD = sV + C::TILE, sP = sQD + NS * 2 * C::SUB, sDS = sP + C::PS_BYTES;
  float* s_stat = reinterpret_cast<float*>(smem_raw + 2 * C::TILE + NS * 2 * C::SUB + 2 * C::PS_BYTES);   // [2][128]: lse | delta
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + C::DATA_KV);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_kvfull = b0, bar_kvfree = b0 + 8, bar_qfull = b0 + 16, bar_qfree = bar_qfull + 8 * NS,
                 bar_sfull = bar_qfree + 8 * NS, bar_ready = bar_sfull + 16, bar_gdone = bar_ready + 8,
                 bar_accfree = bar_gdone + 8, bar_stat = bar_accfree + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 + 2 * NS + 2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(bar_kvfull, 1); mbar_init(bar_kvfree, 1);
    for (int s = 0; s < NS; s++) { mbar_init(bar_qfull + 8 * s, 1); mbar_init(bar_qfree + 8 * s, 1); }
    mbar_init(bar_sfull, 1); mbar_init(bar_sfull + 8, 1);
    mbar_init(bar_ready, 8); mbar_init(bar_gdone, 1); mbar_init(bar_accfree, 8); mbar_init(bar_stat, 256);
    *abort_flag = (base & 1023u) ? 6 : 0;
    if (base & 1023u) atomicCAS(p.err, 0, 6);
    mbar_fence_init();
    tma_prefetch_desc(&map_kv); tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_dqkv);
  }
  if (warp == 9) { tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();
  const int d = p.H * HD, BH = p.B * p.H;
  // key tile 0 sees every query: longest items first
  auto decode = [&](int w, int& b, int& h, int& k0, int& n) {
    const int jt = w / BH, bh = w % BH;
    b = bh / p.H; h = bh % p.H; k0 = jt * BT;
    n = (p.T - k0 + BS - 1) / BS;
  };
  const bool live = *abort_flag == 0;

  if (warp == 8) {
    if (lane == 0 && live) {
      int ic = 0, qc = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x, ic++) {
        int b, h, k0, n;
        decode(w, b, h, k0, n);
        if (!mbar_wait(bar_kvfree, (ic & 1) ^ 1, abort_flag, 6, p.err)) break;
        mbar_expect_tx(bar_kvfull, 2 * C::TILE);
        load_tile<HD>(sK, &map_kv, bar_kvfull, d + h * HD, b * p.T + k0, BT);
        load_tile<HD>(sV, &map_kv, bar_kvfull, 2 * d + h * HD, b * p.T + k0, BT);
        for (int t = 0; t < n; t++, qc++) {
          const int s = qc % NS;
          if (!mbar_wait(bar_qfree + 8 * s, ((qc / NS) & 1) ^ 1, abort_flag, 6, p.err)) { ok = false; break; }
          const uint32_t sq = sQD + s * 2 * C::SUB, sdo = sq + C::SUB;
          mbar_expect_tx(bar_qfull + 8 * s, 2 * C::SUB);
          load_tile<HD>(sq, &map_q, bar_qfull + 8 * s, h * HD, b * p.T + k0 + t * BS, BS);
          load_tile<HD>(sdo, &map_do, bar_qfull + 8 * s, h * HD, b * p.T + k0 + t * BS, BS);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0 && live) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BS, 0, 0);
      constexpr uint32_t idesc_g = umma_idesc_bf16(128, HD, 0, 1);
      int ic = 0, qc = 0, rc = 0;
      bool ok = true;
      const uint64_t dK0 = dk0(sK), dV0 = dk0(sV), dP0 = dk0(sP), dDS0 = dk0(sDS);
      for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x, ic++) {
        int b, h, k0, n;
        decode(w, b, h, k0, n);
        if (!mbar_wait(bar_kvfull, ic & 1, abort_flag, 6, p.err)) break;
        const int q_base = qc;
        for (int t = 0; t <= n && ok; t++) {
          if (t < n) {
            const int s = qc % NS;
            if (!mbar_wait(bar_qfull + 8 * s, (qc / NS) & 1, abort_flag, 6, p.err)) { ok = false; break; }
            qc++;
            tc_fence_after();
            const uint32_t sq = sQD + s * 2 * C::SUB, sdo = sq + C::SUB;
            const uint32_t tS = tmem + (t & 1) * 64, tDP = tmem + 128 + (t & 1) * 64;
            const uint64_t dq0 = dk0(sq), ddo0 = dk0(sdo);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
              umma_f16_ss(tS, DK(dK0, BT, kk), DK(dq0, BS, kk), idesc_s, kk > 0);
              umma_f16_ss(tDP, DK(dV0, BT, kk), DK(ddo0, BS, kk), idesc_s, kk > 0);
            }
            umma_commit(bar_sfull + 8 * (t & 1));
            if (t == n - 1) umma_commit(bar_kvfree);        // K and V are only read by these products
          }
          if (t >= 1) {
            const int tt = t - 1, s = (q_base + tt) % NS;
            const uint32_t sq = sQD + s * 2 * C::SUB, sdo = sq + C::SUB;
            if (tt == 0 && !mbar_wait(bar_accfree, (ic & 1) ^ 1, abort_flag, 6, p.err)) { ok = false; break; }
            if (!mbar_wait(bar_ready, rc & 1, abort_flag, 6, p.err)) { ok = false; break; }
            rc++;
            tc_fence_after();
            const uint64_t mdo0 = dmn0(sdo, BS), mq0 = dmn0(sq, BS);
#pragma unroll
            for (int kk = 0; kk < BS / 16; kk++) {
              umma_f16_ss(tmem + 256, DK(dP0, BT, kk), DMN(mdo0, kk), idesc_g, (tt > 0 || kk > 0));
              umma_f16_ss(tmem + 256 + HD, DK(dDS0, BT, kk), DMN(mq0, kk), idesc_g, (tt > 0 || kk > 0));
            }
            umma_commit(bar_gdone);
            umma_commit(bar_qfree + 8 * s);
          }
        }
      }
    }
  } else if (live) {
    const int row = tid & 127, half = tid >> 7;          // this thread: key row `row`, columns [32 half, 32 half + 32) of a sub-tile
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    int sfc[2] = {0, 0}, uses = 0, obs = 0, stc = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x) {
      int b, h, k0, n;
      decode(w, b, h, k0, n);
      const int kpos = k0 + row;
      const size_t stat0 = ((size_t)b * p.H + h) * p.T;
      // threads 0-63 fetch the lse of query tid of sub-tile t, threads 64-127 its delta.  The value is only
      // touched (scaled, stored) at the end of the iteration, so the load is in flight during the sub-tile.
      const float stat_mul = tid < 64 ? LOG2E : 1.f;
      auto fetch_stat = [&](int t) -> float {
        const int qp = k0 + t * BS + (tid & 63);
        if (tid >= 128 || t >= n || qp >= p.T) return tid < 64 ? INFINITY : 0.f;
        return __ldg((tid < 64 ? p.lse : p.delta) + stat0 + qp);
      };
      if (tid < 128) s_stat[tid] = fetch_stat(0) * stat_mul;
      mbar_arrive(bar_stat);
      if (!mbar_wait(bar_stat, stc & 1, abort_flag, 6, p.err)) break;
      stc++;
      for (int t = 0; t < n; t++) {
        const int buf = t & 1;
        const float next_stat = fetch_stat(t + 1);
        const float* st = s_stat + buf * 128;
        if (!mbar_wait(bar_sfull + 8 * buf, sfc[buf] & 1, abort_flag, 6, p.err)) { ok = false; break; }
        sfc[buf]++;
        tc_fence_after();
        const int q0s = k0 + t * BS;
        const bool diag = k0 + BT - 1 > q0s;
        const int c = half * 32;
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem + buf * 64 + lane_off + c, rs);
        tmem_ld32(tmem + 128 + buf * 64 + lane_off + c, rd);
        tmem_ld_wait();
        uint32_t pp[16], ds[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int u = 0; u < 2; u++) {
            const int qi = c + e + u;
            float pr = exp2f(fmaf(__uint_as_float(rs[e + u]), sl2, -st[qi]));
            if (diag && kpos > q0s + qi) pr = 0.f;
            pv[u] = pr;
            dv[u] = pr * (__uint_as_float(rd[e + u]) - st[64 + qi]) * p.scale;
          }
          pp[e >> 1] = pack_bf16(pv[0], pv[1]);
          ds[e >> 1] = pack_bf16(dv[0], dv[1]);
        }
        // the products that read P^T / dS^T of the previous sub-tile have retired
        while (obs < uses) {
          if (!mbar_wait(bar_gdone, obs & 1, abort_flag, 6, p.err)) { ok = false; break; }
          obs++;
        }
        if (!ok) break;
#pragma unroll
        for (int g = 0; g < 4; g++) {
          st_shared_v4(chunk_addr(sP, BT, row, (c >> 3) + g), pp[4 * g], pp[4 * g + 1], pp[4 * g + 2], pp[4 * g + 3]);
          st_shared_v4(chunk_addr(sDS, BT, row, (c >> 3) + g), ds[4 * g], ds[4 * g + 1], ds[4 * g + 2], ds[4 * g + 3]);
        }
        uses++;
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ready);
        if (tid < 128) s_stat[(buf ^ 1) * 128 + tid] = next_stat * stat_mul;
        mbar_arrive(bar_stat);
        if (!mbar_wait(bar_stat, stc & 1, abort_flag, 6, p.err)) { ok = false; break; }
        stc++;
      }
      if (!ok) break;
      while (obs < uses) {      // the last accumulating products have retired
        if (!mbar_wait(bar_gdone, obs & 1, abort_flag, 6, p.err)) { ok = false; break; }
        obs++;
      }
      if (!ok) break;
      tc_fence_after();
      // dV, then dK: TMEM -> bf16 -> the P^T / dS^T buffers (free now, 2 x 16 KB = one 128 x 128 tile in the
      // swizzled layout) -> one TMA store per 64-column slab; rows past the end of the sequence are clipped
#pragma unroll 1
      for (int which = 0; which < 2; which++) {
        const uint32_t tacc = tmem + 256 + which * HD + lane_off;
#pragma unroll 1
        for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
          uint32_t r1[32];
          tmem_ld32(tacc + c, r1);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 4; g++)
            st_shared_v4(chunk_addr(sP, BT, row, (c >> 3) + g),
                         pack_bf16(__uint_as_float(r1[8 * g]), __uint_as_float(r1[8 * g + 1])),
                         pack_bf16(__uint_as_float(r1[8 * g + 2]), __uint_as_float(r1[8 * g + 3])),
                         pack_bf16(__uint_as_float(r1[8 * g + 4]), __uint_as_float(r1[8 * g + 5])),
                         pack_bf16(__uint_as_float(r1[8 * g + 6]), __uint_as_float(r1[8 * g + 7])));
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_stat);
        if (!mbar_wait(bar_stat, stc & 1, abort_flag, 6, p.err)) { ok = false; break; }
        stc++;
        if (tid == 0) {
          const int col0 = (which == 0 ? 2 * d : d) + h * HD;
#pragma unroll
          for (int sl = 0; sl < HD / 64; sl++) tma_store_3d(&map_dqkv, sP + sl * C::PS_BYTES, col0 + sl * 64, k0, b);
          bulk_commit();
          bulk_wait_read_all();
        }
        mbar_arrive(bar_stat);
        if (!mbar_wait(bar_stat, stc & 1, abort_flag, 6, p.err)) { ok = false; break; }
        stc++;
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_accfree);
    }
    if (tid == 0) bulk_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

// ---- dQ: item = (batch, head, 128 queries); sub-tiles of 64 keys up to the diagonal
template <int HD>
__global__ void __launch_bounds__(320, 1)
flash_dq_ws_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_kv, const __grid_constant__ CUtensorMap map_dqkv, const AttnParams p,
                   int n_items, int n_qt) {
  using C = BwdWs<HD>;
  constexpr int BT = C::BT, BS = C::BS, NS = C::NS;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t sQ = base, sDO = sQ + C::TILE, sKV = sDO + C::TILE, sDS = sKV + NS * 2 * C::SUB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + C::DATA_Q);
  const uint32_t b0 = smem_u32(bars);
  const uint32_t bar_qfull = b0, bar_qfree = b0 + 8, bar_kvfull = b0 + 16, bar_kvfree = bar_kvfull + 8 * NS,
                 bar_sfull = bar_kvfree + 8 * NS, bar_ready = bar_sfull + 16, bar_gdone = bar_ready + 8, bar_accfree = bar_gdone + 8,
                 bar_epi = bar_accfree + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 + 2 * NS + 2 + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    mbar_init(bar_qfull, 1); mbar_init(bar_qfree, 1);
    for (int s = 0; s < NS; s++) { mbar_init(bar_kvfull + 8 * s, 1); mbar_init(bar_kvfree + 8 * s, 1); }
    mbar_init(bar_sfull, 1); mbar_init(bar_sfull + 8, 1);
    mbar_init(bar_ready, 8); mbar_init(bar_gdone, 1); mbar_init(bar_accfree, 8); mbar_init(bar_epi, 256);
    *abort_flag = (base & 1023u) ? 6 : 0;
    if (base & 1023u) atomicCAS(p.err, 0, 6);
    mbar_fence_init();
    tma_prefetch_desc(&map_kv); tma_prefetch_desc(&map_q); tma_prefetch_desc(&map_do); tma_prefetch_desc(&map_dqkv);
  }
  if (warp == 9) { tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();
  const int d = p.H * HD, BH = p.B * p.H;
  // the last query tile sees the most keys: longest items first
  auto decode = [&](int w, int& b, int& h, int& q0, int& n) {
    const int qt = n_qt - 1 - w / BH, bh = w % BH;
    b = bh / p.H; h = bh % p.H; q0 = qt * BT;
    n = (min(q0 + BT, p.T) + BS - 1) / BS;
  };
  const bool live = *abort_flag == 0;

  if (warp == 8) {
    if (lane == 0 && live) {
      int ic = 0, kvc = 0;
      bool ok = true;
      for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x, ic++) {
        int b, h, q0, n;
        decode(w, b, h, q0, n);
        if (!mbar_wait(bar_qfree, (ic & 1) ^ 1, abort_flag, 6, p.err)) break;
        mbar_expect_tx(bar_qfull, 2 * C::TILE);
        load_tile<HD>(sQ, &map_q, bar_qfull, h * HD, b * p.T + q0, BT);
        load_tile<HD>(sDO, &map_do, bar_qfull, h * HD, b * p.T + q0, BT);
        for (int j = 0; j < n; j++, kvc++) {
          const int s = kvc % NS;
          if (!mbar_wait(bar_kvfree + 8 * s, ((kvc / NS) & 1) ^ 1, abort_flag, 6, p.err)) { ok = false; break; }
          const uint32_t sk = sKV + s * 2 * C::SUB, sv = sk + C::SUB;
          mbar_expect_tx(bar_kvfull + 8 * s, 2 * C::SUB);
          load_tile<HD>(sk, &map_kv, bar_kvfull + 8 * s, d + h * HD, b * p.T + j * BS, BS);
          load_tile<HD>(sv, &map_kv, bar_kvfull + 8 * s, 2 * d + h * HD, b * p.T + j * BS, BS);
        }
      }
    }
  } else if (warp == 9) {
    if (lane == 0 && live) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(128, BS, 0, 0);
      constexpr uint32_t idesc_g = umma_idesc_bf16(128, HD, 0, 1);
      int ic = 0, kvc = 0, rc = 0;
      bool ok = true;
      const uint64_t dQ0 = dk0(sQ), dDO0 = dk0(sDO), dDS0 = dk0(sDS);
      for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x, ic++) {
        int b, h, q0, n;
        decode(w, b, h, q0, n);
        if (!mbar_wait(bar_qfull, ic & 1, abort_flag, 6, p.err)) break;
        const int kv_base = kvc;
        for (int j = 0; j <= n && ok; j++) {
          if (j < n) {
            const int s = kvc % NS;
            if (!mbar_wait(bar_kvfull + 8 * s, (kvc / NS) & 1, abort_flag, 6, p.err)) { ok = false; break; }
            kvc++;
            tc_fence_after();
            const uint32_t sk = sKV + s * 2 * C::SUB, sv = sk + C::SUB;
            const uint32_t tS = tmem + (j & 1) * 64, tDP = tmem + 128 + (j & 1) * 64;
            const uint64_t dk_0 = dk0(sk), dv_0 = dk0(sv);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) {
              umma_f16_ss(tS, DK(dQ0, BT, kk), DK(dk_0, BS, kk), idesc_s, kk > 0);
              umma_f16_ss(tDP, DK(dDO0, BT, kk), DK(dv_0, BS, kk), idesc_s, kk > 0);
            }
            umma_commit(bar_sfull + 8 * (j & 1));
            if (j == n - 1) umma_commit(bar_qfree);         // Q and dO are only read by these products
          }
          if (j >= 1) {
            const int jj = j - 1, s = (kv_base + jj) % NS;
            const uint32_t sk = sKV + s * 2 * C::SUB;
            if (jj == 0 && !mbar_wait(bar_accfree, (ic & 1) ^ 1, abort_flag, 6, p.err)) { ok = false; break; }
            if (!mbar_wait(bar_ready, rc & 1, abort_flag, 6, p.err)) { ok = false; break; }
            rc++;
            tc_fence_after();
            const uint64_t mk0 = dmn0(sk, BS);
#pragma unroll
            for (int kk = 0; kk < BS / 16; kk++)
              umma_f16_ss(tmem + 256, DK(dDS0, BT, kk), DMN(mk0, kk), idesc_g, (jj > 0 || kk > 0));
            umma_commit(bar_gdone);
            umma_commit(bar_kvfree + 8 * s);
          }
        }
      }
    }
  } else if (live) {
    const int row = tid & 127, half = tid >> 7;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    const float sl2 = p.scale * LOG2E;
    int sfc[2] = {0, 0}, uses = 0, obs = 0, epc = 0;
    bool ok = true;
    for (int w = blockIdx.x; ok && w < n_items; w += gridDim.x) {
      int b, h, q0, n;
      decode(w, b, h, q0, n);
      const int qpos = q0 + row;
      const bool qvalid = qpos < p.T;
      const size_t sidx = ((size_t)b * p.H + h) * p.T + qpos;
      const float my_lse = qvalid ? p.lse[sidx] * LOG2E : INFINITY;
      const float my_delta = qvalid ? p.delta[sidx] : 0.f;
      for (int j = 0; j < n; j++) {
        const int buf = j & 1;
        if (!mbar_wait(bar_sfull + 8 * buf, sfc[buf] & 1, abort_flag, 6, p.err)) { ok = false; break; }
        sfc[buf]++;
        tc_fence_after();
        const int k0 = j * BS;
        const bool diag = k0 + BS - 1 > q0;
        const int c = half * 32;
        uint32_t rs[32], rd[32];
        tmem_ld32(tmem + buf * 64 + lane_off + c, rs);
        tmem_ld32(tmem + 128 + buf * 64 + lane_off + c, rd);
        tmem_ld_wait();
        uint32_t ds[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float dv[2];
#pragma unroll
          for (int u = 0; u < 2; u++) {
            float pr = exp2f(fmaf(__uint_as_float(rs[e + u]), sl2, -my_lse));
            if (diag && k0 + c + e + u > qpos) pr = 0.f;
            dv[u] = pr * (__uint_as_float(rd[e + u]) - my_delta) * p.scale;
          }
          ds[e >> 1] = pack_bf16(dv[0], dv[1]);
        }
        while (obs < uses) {
          if (!mbar_wait(bar_gdone, obs & 1, abort_flag, 6, p.err)) { ok = false; break; }
          obs++;
        }
        if (!ok) break;
#pragma unroll
        for (int g = 0; g < 4; g++)
          st_shared_v4(chunk_addr(sDS, BT, row, (c >> 3) + g), ds[4 * g], ds[4 * g + 1], ds[4 * g + 2], ds[4 * g + 3]);
        uses++;
        fence_proxy_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_ready);
      }
      if (!ok) break;
      while (obs < uses) {
        if (!mbar_wait(bar_gdone, obs & 1, abort_flag, 6, p.err)) { ok = false; break; }
        obs++;
      }
      if (!ok) break;
      tc_fence_after();
      // dQ: TMEM -> bf16 -> staging tile (the dS buffer and the 16 KB behind it) -> one TMA store per slab
#pragma unroll 1
      for (int c = half * (HD / 2); c < (half + 1) * (HD / 2); c += 32) {
        uint32_t r1[32];
        tmem_ld32(tmem + 256 + lane_off + c, r1);
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < 4; g++)
          st_shared_v4(chunk_addr(sDS, BT, row, (c >> 3) + g),
                       pack_bf16(__uint_as_float(r1[8 * g]), __uint_as_float(r1[8 * g + 1])),
                       pack_bf16(__uint_as_float(r1[8 * g + 2]), __uint_as_float(r1[8 * g + 3])),
                       pack_bf16(__uint_as_float(r1[8 * g + 4]), __uint_as_float(r1[8 * g + 5])),
                       pack_bf16(__uint_as_float(r1[8 * g + 6]), __uint_as_float(r1[8 * g + 7])));
      }
      fence_proxy_async_smem();
      mbar_arrive(bar_epi);
      if (!mbar_wait(bar_epi, epc & 1, abort_flag, 6, p.err)) { ok = false; break; }
      epc++;
      if (tid == 0) {
#pragma unroll
        for (int sl = 0; sl < HD / 64; sl++) tma_store_3d(&map_dqkv, sDS + sl * C::PS_BYTES, h * HD + sl * 64, q0, b);
        bulk_commit();
        bulk_wait_read_all();
      }
      mbar_arrive(bar_epi);
      if (!mbar_wait(bar_epi, epc & 1, abort_flag, 6, p.err)) { ok = false; break; }
      epc++;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_accfree);
    }
    if (tid == 0) bulk_wait_all();
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, C::TMEM_COLS); }
}

template <typename K>
int set_smem(K kernel, int bytes, const char* name) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) { kh_set_error("%s: cannot opt in to %d bytes of shared memory: %s", name, bytes, cudaGetErrorString(e)); return -1; }
  return 0;
}

static int num_sms_attn() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

template <int HD>
int launch_fwd(const void* qkv, const AttnParams& p, cudaStream_t st) {
  using C = FwdWs<HD>;
  const size_t rows = (size_t)p.B * p.T;
  const CUtensorMap* mq = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, C::BQ, 64);
  const CUtensorMap* mkv = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, C::BKV, 64);
  const CUtensorMap* mo = kh_tmap_3d_bf16(p.out, (uint64_t)p.H * HD, p.T, p.B, (uint64_t)p.H * HD, (uint64_t)p.T * p.H * HD, 128, 64);
  if (!mq || !mkv || !mo) return -1;
  static bool once = false;
  if (!once) { if (set_smem(flash_fwd_ws_kernel<HD>, C::SMEM, "flash_fwd")) return -1; once = true; }
  const int n_qt = (p.T + 127) / 128;
  const int n_items = p.B * p.H * n_qt;
  const int ctas = 2 * num_sms_attn();                  // two CTAs per SM
  KH_LAUNCH((flash_fwd_ws_kernel<HD>), n_items < ctas ? n_items : ctas, C::THREADS, C::SMEM, st, *mq, *mkv, *mo, p, n_items, n_qt);
  KH_LAUNCH_CHECK("flash_fwd");
  return 0;
}

template <int HD>
int launch_bwd(const void* qkv, const AttnParams& p, cudaStream_t st) {
  using C = BwdWs<HD>;
  const size_t rows = (size_t)p.B * p.T;
  const CUtensorMap* mq = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, 128, 64);
  const CUtensorMap* md = kh_tmap_2d_bf16(p.dout, rows, p.H * HD, p.H * HD, 128, 64);
  const CUtensorMap* mq64 = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, 64, 64);
  const CUtensorMap* md64 = kh_tmap_2d_bf16(p.dout, rows, p.H * HD, p.H * HD, 64, 64);
  const CUtensorMap* mg = kh_tmap_3d_bf16(p.dqkv, (uint64_t)3 * p.H * HD, p.T, p.B, (uint64_t)p.ld, (uint64_t)p.T * p.ld, 128, 64);
  if (!mq || !md || !mq64 || !md64 || !mg) return -1;
  KH_LAUNCH((flash_delta_kernel<HD>), (unsigned)((rows * 32 + 255) / 256), 256, 0, st, p.o, p.dout, p.delta, p.B, p.T, p.H);
  static bool once = false;
  if (!once) {
    if (set_smem(flash_dkv_ws_kernel<HD>, C::SMEM_KV, "flash_dkv") || set_smem(flash_dq_ws_kernel<HD>, C::SMEM_Q, "flash_dq")) return -1;
    once = true;
  }
  const int n_t = (p.T + 127) / 128;
  const int n_items = p.B * p.H * n_t;
  const int sms = num_sms_attn();
  const int grid = n_items < sms ? n_items : sms;
  KH_LAUNCH((flash_dkv_ws_kernel<HD>), grid, C::THREADS, C::SMEM_KV, st, *mq, *mq64, *md64, *mg, p, n_items, n_t);
  KH_LAUNCH((flash_dq_ws_kernel<HD>), grid, C::THREADS, C::SMEM_Q, st, *mq, *md, *mq64, *mg, p, n_items, n_t);
  KH_LAUNCH_CHECK("flash_bwd");
  return 0;
}

}  // namespace

extern "C" int kh_flash_fwd(const void* qkv, void* out, void* lse, int B, int T, int H, int hd, int ld, float scale,
                            void* stream) {
  if (hd != 64 && hd != 128) { kh_set_error("flash: head dim %d is not supported (64 or 128)", hd); return -1; }
  AttnParams p = {};
  p.B = B; p.T = T; p.H = H; p.ld = ld; p.scale = scale; p.out = (bf16*)out; p.lse = (float*)lse;
  p.err = kh_error_word_dev();
  return hd == 64 ? launch_fwd<64>(qkv, p, (cudaStream_t)stream) : launch_fwd<128>(qkv, p, (cudaStream_t)stream);
}

extern "C" int kh_flash_bwd(const void* qkv, const void* out, const void* dout, const void* lse, void* dqkv,
                            void* delta, int B, int T, int H, int hd, int ld, float scale, void* stream) {
  if (hd != 64 && hd != 128) { kh_set_error("flash: head dim %d is not supported (64 or 128)", hd); return -1; }
  AttnParams p = {};
  p.B = B; p.T = T; p.H = H; p.ld = ld; p.scale = scale; p.lse = (float*)lse; p.o = (const bf16*)out;
  p.dout = (const bf16*)dout; p.delta = (float*)delta; p.dqkv = (bf16*)dqkv;
  p.err = kh_error_word_dev();
  return hd == 64 ? launch_bwd<64>(qkv, p, (cudaStream_t)stream) : launch_bwd<128>(qkv, p, (cudaStream_t)stream);
}
