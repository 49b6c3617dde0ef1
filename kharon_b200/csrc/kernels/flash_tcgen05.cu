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
// forward   CTA = (128 queries, head, batch); S = Q K^T into TMEM, one thread per query row
//           does the online softmax straight out of TMEM, P goes to shared memory as bf16 and
//           P V lands in a second TMEM region that is folded into register accumulators.
//           Two CTAs share an SM, so one CTA's softmax overlaps the other's MMAs.
// backward  delta = rowsum(dO * O); a dK/dV kernel per key tile (S^T, dP^T, dV += P^T dO,
//           dK += dS^T Q accumulated in TMEM) and a dQ kernel per query tile (S, dP,
//           dQ += dS K).  No atomics: every output element is produced by exactly one CTA
//           in a fixed order, so gradients are reproducible bit for bit.
//
// All mbarrier waits are bounded (error word code 6); after a timeout the CTA skips its
// stores, releases TMEM and returns.
#include <stdlib.h>

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
// descriptor for contraction over the tile's columns (K-major), k-step kk of 16 columns
__device__ __forceinline__ uint64_t desc_k(uint32_t base, int rows, int kk) {
  return umma_desc_sw128(base + (kk >> 2) * rows * 128 + (kk & 3) * 32, 16, 1024);
}
// descriptor for contraction over the tile's rows (MN-major), k-step kk of 16 rows
__device__ __forceinline__ uint64_t desc_mn(uint32_t base, int rows, int kk) {
  return umma_desc_sw128(base + kk * 2048, rows * 128, 1024);
}
// address of the 16-byte chunk (row, chunk c of 8 bf16) in a K-major tile with `rows` rows
__device__ __forceinline__ uint32_t chunk_addr(uint32_t base, int rows, int row, int c) {
  return base + (c >> 3) * rows * 128 + row * 128 + (((c & 7) ^ (row & 7)) << 4);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// ================================================================================ forward
template <int HD, int BKV>
__global__ void __launch_bounds__(128, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const AttnParams p) {
  constexpr int BQ = 128;
  constexpr int Q_BYTES = BQ * HD * 2, KV_BYTES = BKV * HD * 2, P_BYTES = BQ * BKV * 2;
  constexpr int TMEM_COLS = 256;          // S: BKV columns at 0, PV: HD columns at 128
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sK = sQ + Q_BYTES, sV = sK + KV_BYTES, sP = sV + KV_BYTES;
  uint8_t* al = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(al + Q_BYTES + 2 * KV_BYTES + P_BYTES);
  const uint32_t bar_q = smem_u32(bars), bar_k = bar_q + 8, bar_v = bar_q + 16, bar_s = bar_q + 24, bar_o = bar_q + 32;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int d = p.H * HD;
  const int q0 = qt * BQ;                              // first query position of the tile
  const int row0 = b * p.T + q0;                       // its row in qkv
  const int n_kv = min((q0 + BQ + BKV - 1) / BKV, (p.T + BKV - 1) / BKV);

  if (tid == 0) {
    for (int i = 0; i < 5; i++) mbar_init(bar_q + 8 * i, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_kv);
  }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tS = tmem, tO = tmem + 128;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  if (tid == 0) {
    mbar_expect_tx(bar_q, Q_BYTES);
    load_tile<HD>(sQ, &map_q, bar_q, h * HD, row0, BQ);
    mbar_expect_tx(bar_k, KV_BYTES);
    load_tile<HD>(sK, &map_kv, bar_k, d + h * HD, b * p.T, BKV);
    mbar_expect_tx(bar_v, KV_BYTES);
    load_tile<HD>(sV, &map_kv, bar_v, 2 * d + h * HD, b * p.T, BKV);
  }
  constexpr uint32_t idesc_s = umma_idesc_bf16(128, BKV, 0, 0);
  constexpr uint32_t idesc_o = umma_idesc_bf16(128, HD, 0, 1);
  const float sl2 = p.scale * LOG2E;

  float o_acc[HD];
#pragma unroll
  for (int i = 0; i < HD; i++) o_acc[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int qpos = q0 + tid;
  bool ok = true;

  for (int j = 0; j < n_kv; j++) {
    const uint32_t ph = j & 1;
    if (tid == 0) {
      if (j == 0) ok = mbar_wait(bar_q, 0, abort_flag, 6, p.err);
      ok = ok && mbar_wait(bar_k, ph, abort_flag, 6, p.err);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, desc_k(sQ, BQ, kk), desc_k(sK, BKV, kk), idesc_s, kk > 0);
        umma_commit(bar_s);
      }
    }
    if (!mbar_wait(bar_s, ph, abort_flag, 6, p.err)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 1 < n_kv) {     // K tile is free again
      mbar_expect_tx(bar_k, KV_BYTES);
      load_tile<HD>(sK, &map_kv, bar_k, d + h * HD, b * p.T + (j + 1) * BKV, BKV);
    }
    // ---- online softmax on this thread's query row
    const int k0 = j * BKV;
    const bool need_mask = k0 + BKV - 1 > q0;
    float m_new = m_run;
#pragma unroll 1
    for (int c = 0; c < BKV; c += 32) {
      uint32_t r[32];
      tmem_ld32(tS + lane_off + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i++) {
        float s = __uint_as_float(r[i]) * sl2;
        if (need_mask && k0 + c + i > qpos) s = -INFINITY;
        m_new = fmaxf(m_new, s);
      }
    }
    const float alpha = exp2f(m_run - m_new);
    float rowsum = 0.f;
#pragma unroll 1
    for (int c = 0; c < BKV; c += 32) {
      uint32_t r[32];
      tmem_ld32(tS + lane_off + c, r);
      tmem_ld_wait();
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float s0 = __uint_as_float(r[i]) * sl2, s1 = __uint_as_float(r[i + 1]) * sl2;
        if (need_mask && k0 + c + i > qpos) s0 = -INFINITY;
        if (need_mask && k0 + c + i + 1 > qpos) s1 = -INFINITY;
        float p0 = exp2f(s0 - m_new), p1 = exp2f(s1 - m_new);
        rowsum += p0 + p1;
        pk[i >> 1] = pack_bf16(p0, p1);
      }
#pragma unroll
      for (int g = 0; g < 4; g++)
        st_shared_v4(chunk_addr(sP, BQ, tid, (c >> 3) + g), pk[4 * g], pk[4 * g + 1], pk[4 * g + 2], pk[4 * g + 3]);
    }
    l_run = l_run * alpha + rowsum;
    m_run = m_new;
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      ok = mbar_wait(bar_v, ph, abort_flag, 6, p.err);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; kk++) umma_f16_ss(tO, desc_k(sP, BQ, kk), desc_mn(sV, BKV, kk), idesc_o, kk > 0);
        umma_commit(bar_o);
      }
    }
    if (!mbar_wait(bar_o, ph, abort_flag, 6, p.err)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 1 < n_kv) {     // V and P are free again
      mbar_expect_tx(bar_v, KV_BYTES);
      load_tile<HD>(sV, &map_kv, bar_v, 2 * d + h * HD, b * p.T + (j + 1) * BKV, BKV);
    }
#pragma unroll
    for (int c = 0; c < HD; c += 32) {
      uint32_t r[32];
      tmem_ld32(tO + lane_off + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; i++) o_acc[c + i] = o_acc[c + i] * alpha + __uint_as_float(r[i]);
    }
    tc_fence_before();
  }

  if (ok && !*abort_flag && qpos < p.T) {
    const float inv = 1.f / l_run;
    bf16* op = p.out + (size_t)(row0 + tid) * d + h * HD;
#pragma unroll
    for (int c = 0; c < HD; c += 8) {
      uint4 o;
      o.x = pack_bf16(o_acc[c] * inv, o_acc[c + 1] * inv); o.y = pack_bf16(o_acc[c + 2] * inv, o_acc[c + 3] * inv);
      o.z = pack_bf16(o_acc[c + 4] * inv, o_acc[c + 5] * inv); o.w = pack_bf16(o_acc[c + 6] * inv, o_acc[c + 7] * inv);
      *reinterpret_cast<uint4*>(op + c) = o;
    }
    if (p.lse) p.lse[((size_t)b * p.H + h) * p.T + qpos] = (m_run + log2f(l_run)) / LOG2E;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
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
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, desc_k(sQ, BQ, kk), desc_k(sk, BKV, kk), idesc_s, kk > 0);
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
#pragma unroll
            for (int kk = 0; kk < BKV / 16; kk++)
              umma_f16_ss(tmem + 128, desc_k(sP, BQ, kk), desc_mn(sv, BKV, kk), idesc_o, (jj > 0 || kk > 0));
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
// delta[b,h,t] = sum_e dO[b,t,h,e] * O[b,t,h,e]; one warp per (row, head)
__global__ void flash_delta_kernel(const bf16* __restrict__ o, const bf16* __restrict__ dout, float* __restrict__ delta,
                                   int B, int T, int H, int hd) {
  pdl_wait();
  pdl_launch_dependents();
  const long w = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= (long)B * T * H) return;
  const long row = w / H;
  const int h = (int)(w % H);
  const bf16* a = o + row * H * hd + (long)h * hd;
  const bf16* g = dout + row * H * hd + (long)h * hd;
  float s = 0.f;
  for (int e = lane * 2; e < hd; e += 64) {
    float2 x = unpack_bf16(*reinterpret_cast<const uint32_t*>(a + e)), y = unpack_bf16(*reinterpret_cast<const uint32_t*>(g + e));
    s += x.x * y.x + x.y * y.y;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    const int b = (int)(row / T), t = (int)(row % T);
    delta[((size_t)b * H + h) * T + t] = s;
  }
}

// ================================================================================ dK / dV
// CTA = (128 keys, head, batch); loops over the query tiles i >= j.  One thread per key row.
template <int HD>
__global__ void __launch_bounds__(128, 1)
flash_dkv_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const AttnParams p) {
  constexpr int BT = 128;
  constexpr int TILE = BT * HD * 2, PT_BYTES = BT * BT * 2;
  constexpr int TMEM_COLS = 512;      // S^T 0..127, dP^T 128..255, dV 256.., dK 256+HD..
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sK = base, sV = sK + TILE, sQ = sV + TILE, sDO = sQ + TILE, sP = sDO + TILE, sDS = sP + PT_BYTES;
  uint8_t* al = smem_raw + (base - smem_u32(smem_raw));
  float* s_lse = reinterpret_cast<float*>(al + 4 * TILE + 2 * PT_BYTES);
  float* s_delta = s_lse + BT;
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_delta + BT);
  const uint32_t bar_kv = smem_u32(bars), bar_q = bar_kv + 8, bar_s = bar_kv + 16, bar_g = bar_kv + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int jt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int d = p.H * HD;
  const int k0 = jt * BT;
  const int n_qt = (p.T + BT - 1) / BT;

  if (tid == 0) {
    for (int i = 0; i < 4; i++) mbar_init(bar_kv + 8 * i, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_qkv);
    tma_prefetch_desc(&map_do);
  }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tS = tmem, tDP = tmem + 128, tDV = tmem + 256, tDK = tmem + 256 + HD;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  if (tid == 0) {
    mbar_expect_tx(bar_kv, 2 * TILE);
    load_tile<HD>(sK, &map_qkv, bar_kv, d + h * HD, b * p.T + k0, BT);
    load_tile<HD>(sV, &map_qkv, bar_kv, 2 * d + h * HD, b * p.T + k0, BT);
    mbar_expect_tx(bar_q, 2 * TILE);
    load_tile<HD>(sQ, &map_qkv, bar_q, h * HD, b * p.T + jt * BT, BT);
    load_tile<HD>(sDO, &map_do, bar_q, h * HD, b * p.T + jt * BT, BT);
  }
  constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_g = umma_idesc_bf16(128, HD, 0, 1);
  const float sl2 = p.scale * LOG2E;
  const int kpos = k0 + tid;
  bool ok = true;
  int it = 0;
  for (int i = jt; i < n_qt; i++, it++) {
    const uint32_t ph = it & 1;
    const int q0 = i * BT;
    // per-query statistics of this tile
    {
      const int qp = q0 + tid;
      const size_t idx = ((size_t)b * p.H + h) * p.T + qp;
      s_lse[tid] = qp < p.T ? p.lse[idx] * LOG2E : INFINITY;
      s_delta[tid] = qp < p.T ? p.delta[idx] : 0.f;
    }
    if (tid == 0) {
      if (it == 0) ok = mbar_wait(bar_kv, 0, abort_flag, 6, p.err);
      ok = ok && mbar_wait(bar_q, ph, abort_flag, 6, p.err);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, desc_k(sK, BT, kk), desc_k(sQ, BT, kk), idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tDP, desc_k(sV, BT, kk), desc_k(sDO, BT, kk), idesc_s, kk > 0);
        umma_commit(bar_s);
      }
    }
    __syncthreads();   // s_lse / s_delta visible
    if (!mbar_wait(bar_s, ph, abort_flag, 6, p.err)) { ok = false; break; }
    tc_fence_after();
    const bool diag = (i == jt);
#pragma unroll 1
    for (int c = 0; c < BT; c += 32) {
      uint32_t rs[32], rd[32];
      tmem_ld32(tS + lane_off + c, rs);
      tmem_ld32(tDP + lane_off + c, rd);
      tmem_ld_wait();
      uint32_t pp[16], ds[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float pv[2], dv[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int qi = c + e + u;
          float pr = exp2f(__uint_as_float(rs[e + u]) * sl2 - s_lse[qi]);
          if (diag && kpos > q0 + qi) pr = 0.f;
          pv[u] = pr;
          dv[u] = pr * (__uint_as_float(rd[e + u]) - s_delta[qi]) * p.scale;
        }
        pp[e >> 1] = pack_bf16(pv[0], pv[1]);
        ds[e >> 1] = pack_bf16(dv[0], dv[1]);
      }
#pragma unroll
      for (int g = 0; g < 4; g++) {
        st_shared_v4(chunk_addr(sP, BT, tid, (c >> 3) + g), pp[4 * g], pp[4 * g + 1], pp[4 * g + 2], pp[4 * g + 3]);
        st_shared_v4(chunk_addr(sDS, BT, tid, (c >> 3) + g), ds[4 * g], ds[4 * g + 1], ds[4 * g + 2], ds[4 * g + 3]);
      }
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < BT / 16; kk++) umma_f16_ss(tDV, desc_k(sP, BT, kk), desc_mn(sDO, BT, kk), idesc_g, (it > 0 || kk > 0));
#pragma unroll
      for (int kk = 0; kk < BT / 16; kk++) umma_f16_ss(tDK, desc_k(sDS, BT, kk), desc_mn(sQ, BT, kk), idesc_g, (it > 0 || kk > 0));
      umma_commit(bar_g);
    }
    if (!mbar_wait(bar_g, ph, abort_flag, 6, p.err)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && i + 1 < n_qt) {
      mbar_expect_tx(bar_q, 2 * TILE);
      load_tile<HD>(sQ, &map_qkv, bar_q, h * HD, b * p.T + (i + 1) * BT, BT);
      load_tile<HD>(sDO, &map_do, bar_q, h * HD, b * p.T + (i + 1) * BT, BT);
    }
    __syncthreads();   // s_lse / s_delta may be overwritten by the next iteration
  }

  if (ok && !*abort_flag) {
    const bool store = kpos < p.T;
    bf16* dk = p.dqkv + (size_t)(b * p.T + kpos) * p.ld + d + h * HD;
    bf16* dv = p.dqkv + (size_t)(b * p.T + kpos) * p.ld + 2 * d + h * HD;
#pragma unroll 1
    for (int c = 0; c < HD; c += 32) {
      uint32_t r1[32], r2[32];
      tmem_ld32(tDV + lane_off + c, r1);
      tmem_ld32(tDK + lane_off + c, r2);
      tmem_ld_wait();
      if (store) {
#pragma unroll
        for (int g = 0; g < 4; g++) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r1[8 * g]), __uint_as_float(r1[8 * g + 1]));
          o.y = pack_bf16(__uint_as_float(r1[8 * g + 2]), __uint_as_float(r1[8 * g + 3]));
          o.z = pack_bf16(__uint_as_float(r1[8 * g + 4]), __uint_as_float(r1[8 * g + 5]));
          o.w = pack_bf16(__uint_as_float(r1[8 * g + 6]), __uint_as_float(r1[8 * g + 7]));
          *reinterpret_cast<uint4*>(dv + c + 8 * g) = o;
          o.x = pack_bf16(__uint_as_float(r2[8 * g]), __uint_as_float(r2[8 * g + 1]));
          o.y = pack_bf16(__uint_as_float(r2[8 * g + 2]), __uint_as_float(r2[8 * g + 3]));
          o.z = pack_bf16(__uint_as_float(r2[8 * g + 4]), __uint_as_float(r2[8 * g + 5]));
          o.w = pack_bf16(__uint_as_float(r2[8 * g + 6]), __uint_as_float(r2[8 * g + 7]));
          *reinterpret_cast<uint4*>(dk + c + 8 * g) = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ================================================================================ dQ
// CTA = (128 queries, head, batch); loops over the key tiles j <= i.  One thread per query row.
template <int HD>
__global__ void __launch_bounds__(128, 1)
flash_dq_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do, const AttnParams p) {
  constexpr int BT = 128;
  constexpr int TILE = BT * HD * 2, PT_BYTES = BT * BT * 2;
  constexpr int TMEM_COLS = 512;      // S 0..127, dP 128..255, dQ 256..
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t sQ = base, sDO = sQ + TILE, sK = sDO + TILE, sV = sK + TILE, sDS = sV + TILE;
  uint8_t* al = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(al + 4 * TILE + PT_BYTES);
  const uint32_t bar_q = smem_u32(bars), bar_kv = bar_q + 8, bar_s = bar_q + 16, bar_g = bar_q + 24;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int d = p.H * HD;
  const int q0 = qt * BT;

  if (tid == 0) {
    for (int i = 0; i < 4; i++) mbar_init(bar_q + 8 * i, 1);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&map_qkv);
    tma_prefetch_desc(&map_do);
  }
  if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tS = tmem, tDP = tmem + 128, tDQ = tmem + 256;
  const uint32_t lane_off = (uint32_t)(warp * 32) << 16;

  if (tid == 0) {
    mbar_expect_tx(bar_q, 2 * TILE);
    load_tile<HD>(sQ, &map_qkv, bar_q, h * HD, b * p.T + q0, BT);
    load_tile<HD>(sDO, &map_do, bar_q, h * HD, b * p.T + q0, BT);
    mbar_expect_tx(bar_kv, 2 * TILE);
    load_tile<HD>(sK, &map_qkv, bar_kv, d + h * HD, b * p.T, BT);
    load_tile<HD>(sV, &map_qkv, bar_kv, 2 * d + h * HD, b * p.T, BT);
  }
  constexpr uint32_t idesc_s = umma_idesc_bf16(128, 128, 0, 0);
  constexpr uint32_t idesc_g = umma_idesc_bf16(128, HD, 0, 1);
  const float sl2 = p.scale * LOG2E;
  const int qpos = q0 + tid;
  const bool qvalid = qpos < p.T;
  const size_t sidx = ((size_t)b * p.H + h) * p.T + qpos;
  const float my_lse = qvalid ? p.lse[sidx] * LOG2E : INFINITY;
  const float my_delta = qvalid ? p.delta[sidx] : 0.f;
  bool ok = true;
  const int n_kv = qt + 1;
  for (int j = 0; j < n_kv; j++) {
    const uint32_t ph = j & 1;
    if (tid == 0) {
      if (j == 0) ok = mbar_wait(bar_q, 0, abort_flag, 6, p.err);
      ok = ok && mbar_wait(bar_kv, ph, abort_flag, 6, p.err);
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, desc_k(sQ, BT, kk), desc_k(sK, BT, kk), idesc_s, kk > 0);
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tDP, desc_k(sDO, BT, kk), desc_k(sV, BT, kk), idesc_s, kk > 0);
        umma_commit(bar_s);
      }
    }
    if (!mbar_wait(bar_s, ph, abort_flag, 6, p.err)) { ok = false; break; }
    tc_fence_after();
    const bool diag = (j == qt);
    const int k0 = j * BT;
#pragma unroll 1
    for (int c = 0; c < BT; c += 32) {
      uint32_t rs[32], rd[32];
      tmem_ld32(tS + lane_off + c, rs);
      tmem_ld32(tDP + lane_off + c, rd);
      tmem_ld_wait();
      uint32_t ds[16];
#pragma unroll
      for (int e = 0; e < 32; e += 2) {
        float dv[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
          float pr = exp2f(__uint_as_float(rs[e + u]) * sl2 - my_lse);
          if (diag && k0 + c + e + u > qpos) pr = 0.f;
          dv[u] = pr * (__uint_as_float(rd[e + u]) - my_delta) * p.scale;
        }
        ds[e >> 1] = pack_bf16(dv[0], dv[1]);
      }
#pragma unroll
      for (int g = 0; g < 4; g++)
        st_shared_v4(chunk_addr(sDS, BT, tid, (c >> 3) + g), ds[4 * g], ds[4 * g + 1], ds[4 * g + 2], ds[4 * g + 3]);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < BT / 16; kk++) umma_f16_ss(tDQ, desc_k(sDS, BT, kk), desc_mn(sK, BT, kk), idesc_g, (j > 0 || kk > 0));
      umma_commit(bar_g);
    }
    if (!mbar_wait(bar_g, ph, abort_flag, 6, p.err)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && j + 1 < n_kv) {
      mbar_expect_tx(bar_kv, 2 * TILE);
      load_tile<HD>(sK, &map_qkv, bar_kv, d + h * HD, b * p.T + (j + 1) * BT, BT);
      load_tile<HD>(sV, &map_qkv, bar_kv, 2 * d + h * HD, b * p.T + (j + 1) * BT, BT);
    }
  }
  if (ok && !*abort_flag) {
    bf16* dq = p.dqkv + (size_t)(b * p.T + qpos) * p.ld + h * HD;
#pragma unroll 1
    for (int c = 0; c < HD; c += 32) {
      uint32_t r1[32];
      tmem_ld32(tDQ + lane_off + c, r1);
      tmem_ld_wait();
      if (qvalid) {
#pragma unroll
        for (int g = 0; g < 4; g++) {
          uint4 o;
          o.x = pack_bf16(__uint_as_float(r1[8 * g]), __uint_as_float(r1[8 * g + 1]));
          o.y = pack_bf16(__uint_as_float(r1[8 * g + 2]), __uint_as_float(r1[8 * g + 3]));
          o.z = pack_bf16(__uint_as_float(r1[8 * g + 4]), __uint_as_float(r1[8 * g + 5]));
          o.w = pack_bf16(__uint_as_float(r1[8 * g + 6]), __uint_as_float(r1[8 * g + 7]));
          *reinterpret_cast<uint4*>(dq + c + 8 * g) = o;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
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
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, desc_k(sK, BT, kk), desc_k(sq, BS, kk), idesc_s, kk > 0);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tDP, desc_k(sV, BT, kk), desc_k(sdo, BS, kk), idesc_s, kk > 0);
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
#pragma unroll
            for (int kk = 0; kk < BS / 16; kk++)
              umma_f16_ss(tmem + 256, desc_k(sP, BT, kk), desc_mn(sdo, BS, kk), idesc_g, (tt > 0 || kk > 0));
#pragma unroll
            for (int kk = 0; kk < BS / 16; kk++)
              umma_f16_ss(tmem + 256 + HD, desc_k(sDS, BT, kk), desc_mn(sq, BS, kk), idesc_g, (tt > 0 || kk > 0));
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
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tS, desc_k(sQ, BT, kk), desc_k(sk, BS, kk), idesc_s, kk > 0);
#pragma unroll
            for (int kk = 0; kk < HD / 16; kk++) umma_f16_ss(tDP, desc_k(sDO, BT, kk), desc_k(sv, BS, kk), idesc_s, kk > 0);
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
#pragma unroll
            for (int kk = 0; kk < BS / 16; kk++)
              umma_f16_ss(tmem + 256, desc_k(sDS, BT, kk), desc_mn(sk, BS, kk), idesc_g, (jj > 0 || kk > 0));
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

template <int HD, int BKV>
int launch_fwd(const void* qkv, const AttnParams& p, cudaStream_t st) {
  const size_t rows = (size_t)p.B * p.T;
  const CUtensorMap* mq = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, 128, 64);
  const CUtensorMap* mkv = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, BKV, 64);
  if (!mq || !mkv) return -1;
  static const bool serial = [] { const char* e = getenv("KHARON_FLASH_SERIAL"); return e && e[0] == '1'; }();
  if (!serial) {
    using C = FwdWs<HD>;
    mkv = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, C::BKV, 64);
    if (!mkv) return -1;
    static bool once_ws = false;
    if (!once_ws) { if (set_smem(flash_fwd_ws_kernel<HD>, C::SMEM, "flash_fwd")) return -1; once_ws = true; }
    const int n_qt = (p.T + 127) / 128;
    const int n_items = p.B * p.H * n_qt;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const int ctas = 2 * sms;                  // two CTAs per SM
    const CUtensorMap* mo = kh_tmap_3d_bf16(p.out, (uint64_t)p.H * HD, p.T, p.B, (uint64_t)p.H * HD, (uint64_t)p.T * p.H * HD, 128, 64);
    if (!mo) return -1;
    KH_LAUNCH((flash_fwd_ws_kernel<HD>), n_items < ctas ? n_items : ctas, C::THREADS, C::SMEM, st, *mq, *mkv, *mo, p, n_items, n_qt);
    KH_LAUNCH_CHECK("flash_fwd");
    return 0;
  }
  constexpr int SMEM = 128 * HD * 2 + 2 * BKV * HD * 2 + 128 * BKV * 2 + 1024 + 64;
  static bool once = false;
  if (!once) { if (set_smem(flash_fwd_kernel<HD, BKV>, SMEM, "flash_fwd")) return -1; once = true; }
  dim3 grid((p.T + 127) / 128, p.H, p.B);
  KH_LAUNCH((flash_fwd_kernel<HD, BKV>), grid, 128, SMEM, st, *mq, *mkv, p);
  KH_LAUNCH_CHECK("flash_fwd");
  return 0;
}

template <int HD>
int launch_bwd(const void* qkv, const AttnParams& p, cudaStream_t st) {
  const size_t rows = (size_t)p.B * p.T;
  const CUtensorMap* mq = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, 128, 64);
  const CUtensorMap* md = kh_tmap_2d_bf16(p.dout, rows, p.H * HD, p.H * HD, 128, 64);
  if (!mq || !md) return -1;
  const long nw = (long)rows * p.H;
  KH_LAUNCH(flash_delta_kernel, (unsigned)((nw * 32 + 255) / 256), 256, 0, st, p.o, p.dout, p.delta, p.B, p.T, p.H, HD);
  static const bool serial = [] { const char* e = getenv("KHARON_FLASH_SERIAL"); return e && e[0] == '1'; }();
  if (!serial) {
    using C = BwdWs<HD>;
    const CUtensorMap* mq64 = kh_tmap_2d_bf16(qkv, rows, 3 * p.H * HD, p.ld, 64, 64);
    const CUtensorMap* md64 = kh_tmap_2d_bf16(p.dout, rows, p.H * HD, p.H * HD, 64, 64);
    if (!mq64 || !md64) return -1;
    static bool once_ws = false;
    if (!once_ws) {
      if (set_smem(flash_dkv_ws_kernel<HD>, C::SMEM_KV, "flash_dkv") || set_smem(flash_dq_ws_kernel<HD>, C::SMEM_Q, "flash_dq")) return -1;
      once_ws = true;
    }
    const int n_t = (p.T + 127) / 128;
    const int n_items = p.B * p.H * n_t;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const int grid = n_items < sms ? n_items : sms;
    const CUtensorMap* mg = kh_tmap_3d_bf16(p.dqkv, (uint64_t)3 * p.H * HD, p.T, p.B, (uint64_t)p.ld, (uint64_t)p.T * p.ld, 128, 64);
    if (!mg) return -1;
    KH_LAUNCH((flash_dkv_ws_kernel<HD>), grid, C::THREADS, C::SMEM_KV, st, *mq, *mq64, *md64, *mg, p, n_items, n_t);
    KH_LAUNCH((flash_dq_ws_kernel<HD>), grid, C::THREADS, C::SMEM_Q, st, *mq, *md, *mq64, *mg, p, n_items, n_t);
    KH_LAUNCH_CHECK("flash_bwd");
    return 0;
  }
  constexpr int SMEM_KV = 4 * 128 * HD * 2 + 2 * 128 * 128 * 2 + 1024 + 1024 + 64;
  constexpr int SMEM_Q = 4 * 128 * HD * 2 + 128 * 128 * 2 + 1024 + 64;
  static bool once = false;
  if (!once) {
    if (set_smem(flash_dkv_kernel<HD>, SMEM_KV, "flash_dkv") || set_smem(flash_dq_kernel<HD>, SMEM_Q, "flash_dq")) return -1;
    once = true;
  }
  dim3 grid((p.T + 127) / 128, p.H, p.B);
  KH_LAUNCH((flash_dkv_kernel<HD>), grid, 128, SMEM_KV, st, *mq, *md, p);
  KH_LAUNCH((flash_dq_kernel<HD>), grid, 128, SMEM_Q, st, *mq, *md, p);
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
  return hd == 64 ? launch_fwd<64, 128>(qkv, p, (cudaStream_t)stream) : launch_fwd<128, 64>(qkv, p, (cudaStream_t)stream);
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
