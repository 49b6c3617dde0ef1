// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
//   gemm_comm, mode AR : out[M,N]      = sum_r A_r * op(B_r)   on every rank      (GEMM -> all-reduce)
//   gemm_comm, mode RS : out[M/tp,N]   = rows [rank*M/tp, ...) of that sum         (GEMM -> reduce-scatter)
//   optional gather    : A is the row-wise concatenation of per-rank shards that live in
//                        peer memory (all-gather -> GEMM).  A few CTAs of the same launch act as
//                        copiers: they pull the peers' shards over NVLink once, 32 KB at a time
//                        with non-multicast bulk copies (peer -> shared memory -> local gather
//                        buffer), and publish every 128-row block through a counter; the GEMM CTAs
//                        start on the local rows and read remote rows from the local copy.
//
// These replace the reference's cuBLAS GEMM followed by a blocking bf16 ncclAllReduce on the
// same stream (src/core/gpt.c:686-687, 692-693, 745-746, 760-761; src/parallel/comms.cu:97-99).
//
// One kernel, persistent CTAs, ten warps:
//   warp 0      TMA producer (operand tiles -> 128-byte-swizzled shared-memory ring)
//   warp 1      tcgen05.mma issuer, two TMEM accumulator buffers
//   warps 2-5   epilogue: TMEM -> bf16 partial tile in 16 KB shared-memory chunks (128 rows x 64
//               columns), each stored with TMA tensor stores to the local output (if this rank
//               reduces the tile) and into the staging slot of every rank that reduces it; then
//               fence + one red.release.sys on that rank's arrival counter for (source rank, tile).
//               (Measured alternatives that lost: 128-column tiles so that a CTA has two tiles to
//               overlap -- the narrower MMA runs at about half rate; staging laid out chunk by
//               chunk so that a push is one linear 16 KB bulk store -- 20 % slower than the
//               tensor store of the same bytes.)
//   warps 6-9   reducer: for each finished tile, wait (bounded) until every peer's partial has
//               arrived, add the partials in rank order in fp32, add bias / residual, store.
//               Runs concurrently with the main loop of the following tiles, so the NVLink
//               traffic hides behind the tensor-core work.
//
// Determinism: partials are rounded to bf16 once, summed in fp32 in rank order 0..tp-1 on every
// rank -> all ranks hold bit-identical results, run to run.
// Flow control: arrival counters only grow (4 per call and tile); staging is double-buffered
// by call parity, which is sufficient because a rank cannot be two calls ahead of a peer it
// needs partials from.  The call number lives in device memory (a word per buffer set that the
// last CTA of a launch advances), so a launch takes the same arguments every time and can be
// replayed from a CUDA graph or a recorded launch plan.  Every wait is bounded; on expiry the error word gets code 5 and all
// roles of the CTA unwind.  No TMA load here uses cluster multicast; peer memory is only
// touched by st.global / red (push) and, in gather mode, by non-multicast TMA loads.
#include "../kernels/common.cuh"

#define KH_LAUNCH_CHECK(name)                                                     \
  do {                                                                            \
    cudaError_t e_ = cudaGetLastError();                                          \
    if (e_ != cudaSuccess) { kh_set_error(name ": %s", cudaGetErrorString(e_)); return -1; } \
  } while (0)

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int THREADS = 320;
constexpr int EPI_CHUNK_BYTES = BM * 64 * 2;                 // 128 rows x 64 columns bf16, one swizzle-128B box
constexpr int SMEM = STAGES * STAGE_BYTES + 2 * EPI_CHUNK_BYTES + 1024 + 256;
constexpr int MAX_TP = 8;
enum { MODE_AR = 0, MODE_RS = 1, MODE_LOCAL = 2 };   // LOCAL: no reduction (all-gather -> GEMM only)
enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_BIAS_GELU = 2, EPI_DGELU = 4 };

struct CommParams {
  int M, N, K;
  int a_mn, b_mn;
  int mode, tp, rank;
  int gather;                  // A rows come from per-rank shards (tensor maps tma_a[r])
  bf16* out; int ldo;          // AR: [M, N]; RS: [M/tp, N]
  const bf16* bias;            // [N] or null, added by the reducer (all-gather form: by the epilogue)
  const bf16* resid; int ldr;  // residual rows aligned with `out`, or null
  int epi;                     // all-gather form only: EPI_NONE / EPI_BIAS / EPI_BIAS_GELU / EPI_DGELU
  bf16* aux; int ldaux;        // EPI_BIAS_GELU: pre-activation out [M, N]; EPI_DGELU: pre-activation in
  bf16* stage[MAX_TP];         // stage[r]: rank r's staging base for parity 0 (tp slots of M*N); parity 1 follows
  size_t slot_elems;           // tp * M * N
  uint32_t* epoch;             // local: [0] calls completed on this buffer set, [1] CTAs finished; null: host counts
  uint32_t* flags[MAX_TP];     // flags[r]: rank r's arrival counters [tp][num_tiles]
  uint32_t* ready[MAX_TP];     // gather mode: ready[r]: rank r's "shard published" counters [tp]
  const bf16* shard[MAX_TP];   // gather mode: rank r's row shard [M/tp, K], contiguous, as mapped here
  bf16* gbuf;                  // gather mode: local [M, K] buffer that receives the remote rows
  uint32_t* blk_ready;         // gather mode: per 128-row block, calls for which the block has been delivered
  int n_copy;                  // gather mode: CTAs at the end of the grid that copy instead of multiplying
  uint32_t call_no;            // 1-based call number when the host counts
  uint32_t ready_target;
  uint64_t wait_ns;            // limit of every wait in this kernel (all of them can be stalled by a peer)
  int* err;
};

// out: the local output; st[r]: slot `rank` of rank r's staging (where this rank's partial goes)
struct Maps { CUtensorMap a[MAX_TP]; CUtensorMap b; CUtensorMap out; CUtensorMap st[2][MAX_TP]; CUtensorMap g; };

constexpr int COPY_CHUNK = 32 * 1024, COPY_SLOTS = 4;
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}


__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(m), "r"(src), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// bounded spin until *p has reached `target` (counters only grow; compare with wrap-around)
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, volatile int* abort_flag, int* err,
                                             uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
    if ((it & 63) == 63) {
      if (*abort_flag) return false;
      const uint64_t now = kh_globaltimer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        *abort_flag = 5;
        atomicCAS(err, 0, 5);
        return false;
      }
      __nanosleep(64);
    }
  }
}
__device__ __forceinline__ bool wait_smem_count(volatile int* p, int target, volatile int* abort_flag, int* err,
                                                uint64_t limit_ns) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (*p >= target) return true;
    if ((it & 255) == 255) {
      if (*abort_flag) return false;
      const uint64_t now = kh_globaltimer();
      if (t0 == 0) t0 = now;
      else if (now - t0 > limit_ns) {
        *abort_flag = 5;
        atomicCAS(err, 0, 5);
        return false;
      }
    }
    __nanosleep(32);
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_comm_kernel(const __grid_constant__ Maps maps, const CommParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_al = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t smem_epi = smem_base + STAGES * STAGE_BYTES;          // two 16 KB store staging chunks
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_al + STAGES * STAGE_BYTES + 2 * EPI_CHUNK_BYTES);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_pub = reinterpret_cast<volatile int*>(tmem_slot + 2);   // epilogue warps that finished a tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int rows_per_rank = max(1, p.M / p.tp);     // only meaningful in the row-sharded modes

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int a = 0; a < 2; a++) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 4); }
    *abort_flag = 0;
    *s_pub = 0;
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();
  pdl_launch_dependents();
  // this launch's call number: every CTA reads it before any CTA can have finished, and only the
  // CTA that finishes last advances it
  const uint32_t call = p.epoch ? *reinterpret_cast<volatile uint32_t*>(p.epoch) + 1u : p.call_no;
  const uint32_t target = 4u * call;           // counter value that means "this call's partial has arrived"
  const int par = (int)(call & 1u);
  const bf16* my_stage = p.stage[p.rank] + (size_t)par * p.slot_elems;
  // gather mode: the first n_copy CTAs of the grid (scheduled first) pull the peers' shards, the others multiply
  const int n_copy = p.gather ? p.n_copy : 0;
  const int n_workers = (int)gridDim.x - n_copy;
  const int worker = (int)blockIdx.x - n_copy;
  const bool copier = worker < 0;

  // Tiles are visited M-band by M-band starting with this rank's own rows, so that in gather mode
  // local shards are consumed while the peers' shards are still being published.
  auto tile_coord = [&](int t, int& tm, int& tn) {
    const int GROUP = 8;
    int band = t / (GROUP * tiles_n);
    int first = band * GROUP;
    int gsz = min(GROUP, tiles_m - first);
    int r = t - band * GROUP * tiles_n;
    int tm0 = first + r % gsz;
    tn = r / gsz;
    const int shift = p.gather ? (p.rank * (rows_per_rank / BM)) : 0;
    tm = (tm0 + shift) % tiles_m;
  };
  // which rank reduces tile row-block tm (RS mode); AR: everyone
  auto owner_of = [&](int tm) { return (tm * BM) / rows_per_rank; };

  if (warp == 0) {
    if (lane == 0) {
      // gather mode: tell every peer that this rank's shard is final (stream order guarantees it)
      if (p.gather && worker == 0) {
        __threadfence_system();
        for (int r = 0; r < p.tp; r++)
          if (r != p.rank) red_release_sys_add(p.ready[r] + p.rank, 1);
      }
      int it = 0;
      bool ok = true;
      if (copier) {
        // ---- copier CTA: peers' shards -> local gather buffer.  Remote 128-row blocks are dealt
        // round-robin to the copiers in the order the multiplying CTAs reach them; a copier moves
        // its block in 32 KB pieces with up to four bulk loads in flight, then publishes the block
        const int cid = (int)blockIdx.x;
        for (int r = 0; r < p.tp && ok; r++)
          if (r != p.rank && !wait_counter(p.ready[p.rank] + r, p.ready_target, abort_flag, p.err, p.wait_ns)) ok = false;
        asm volatile("fence.proxy.async;" ::: "memory");     // the acquire above orders generic accesses; bulk copies are async-proxy
        const size_t blk_bytes = (size_t)BM * p.K * 2;
        const int pieces = (int)((blk_bytes + COPY_CHUNK - 1) / COPY_CHUNK);
        const int shift = p.rank * (rows_per_rank / BM);
        uint32_t uses[COPY_SLOTS] = {0, 0, 0, 0};
        int remote_no = 0;
        for (int i = 0; i < tiles_m && ok; i++) {
          const int tm = (i + shift) % tiles_m;
          const int src = owner_of(tm);
          if (src == p.rank) continue;
          if ((remote_no++) % p.n_copy != cid) continue;
          const char* sbase = reinterpret_cast<const char*>(p.shard[src]) + (size_t)(tm * BM - src * rows_per_rank) * p.K * 2;
          char* dbase = reinterpret_cast<char*>(p.gbuf) + (size_t)tm * blk_bytes;
          for (int q0 = 0; q0 < pieces && ok; q0 += COPY_SLOTS) {
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");     // slots no longer read by earlier stores
            int nb = 0;
            for (int j = 0; j < COPY_SLOTS; j++, nb++) {
              const int q = q0 + j;
              if (q >= pieces) break;
              const size_t off = (size_t)q * COPY_CHUNK;
              const uint32_t bytes = (uint32_t)min((size_t)COPY_CHUNK, blk_bytes - off);
              mbar_expect_tx(bar_full + 8 * j, bytes);
              bulk_load_1d(smem_base + j * COPY_CHUNK, sbase + off, bytes, bar_full + 8 * j);
            }
            for (int j = 0; j < nb; j++) {
              if (!mbar_wait(bar_full + 8 * j, uses[j] & 1, abort_flag, 6, p.err, p.wait_ns)) { ok = false; break; }
              uses[j]++;
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              const size_t off = (size_t)(q0 + j) * COPY_CHUNK;
              const uint32_t bytes = (uint32_t)min((size_t)COPY_CHUNK, blk_bytes - off);
              bulk_store_1d(dbase + off, smem_base + j * COPY_CHUNK, bytes);
            }
            tma_store_commit();
          }
          // block tm is complete in local memory: publish it
          tma_store_wait_all();
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          atomicAdd(p.blk_ready + tm, 1u);
        }
        tma_store_wait_all();
      }
      int ready_tm = -1;
      for (int t = worker; !copier && ok && t < num_tiles; t += n_workers) {
        int tm, tn;
        tile_coord(t, tm, tn);
        const CUtensorMap* amap = &maps.a[0];
        int row_in_src = tm * BM;
        if (p.gather) {
          const int src = owner_of(tm);
          if (src == p.rank) {
            amap = &maps.a[p.rank];
            row_in_src = tm * BM - src * rows_per_rank;
          } else {
            amap = &maps.g;
            if (ready_tm != tm) {      // the block's copier has delivered it (one increment per call)
              if (!wait_counter(p.blk_ready + tm, call, abort_flag, p.err, p.wait_ns)) { ok = false; break; }
              asm volatile("fence.proxy.async;" ::: "memory");
              ready_tm = tm;
            }
          }
        }
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1, abort_flag, 2, p.err, p.wait_ns)) { ok = false; break; }
          const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
          mbar_expect_tx(bar_full + 8 * s, STAGE_BYTES);
          if (!p.a_mn) tma_load_2d(sa, amap, bar_full + 8 * s, kb * BK, row_in_src);
          else
            for (int j = 0; j < BM / 64; j++) tma_load_2d(sa + j * (BK * 128), amap, bar_full + 8 * s, row_in_src + j * 64, kb * BK);
          if (!p.b_mn) tma_load_2d(sb, &maps.b, bar_full + 8 * s, kb * BK, tn * BN);
          else
            for (int j = 0; j < BN / 64; j++) tma_load_2d(sb + j * (BK * 128), &maps.b, bar_full + 8 * s, tn * BN + j * 64, kb * BK);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(BM, BN, p.a_mn, p.b_mn);
      const uint32_t a_lbo = p.a_mn ? BK * 128 : 16, b_lbo = p.b_mn ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      const uint32_t b_kstep = p.b_mn ? (UMMA_K * 128) >> 4 : (UMMA_K * 2) >> 4;
      int it = 0, tcount = 0;
      bool ok = true;
      for (int t = worker; !copier && ok && t < num_tiles; t += n_workers, tcount++) {
        const int acc = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(bar_tempty + 8 * acc, aph ^ 1, abort_flag, 4, p.err, p.wait_ns)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, 1, p.err, p.wait_ns)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * STAGE_BYTES, sb = sa + A_BYTES;
          const uint64_t adesc = umma_desc_sw128(sa, a_lbo, 1024), bdesc = umma_desc_sw128(sb, b_lbo, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; k++)
            umma_f16_ss(d_tmem, adesc + (uint64_t)(k * a_kstep), bdesc + (uint64_t)(k * b_kstep), idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(bar_empty + 8 * s);
        }
        if (ok) umma_commit(bar_tfull + 8 * acc);
      }
    }
  } else if (warp < 6) {
    // ---------------------------------------------------------------- epilogue: publish partial tiles
    const int q = warp & 3;
    int tcount = 0;
    bool ok = true;
    // Arrival of tile t is signalled once its bulk stores have completed; that is checked one
    // tile later (after the next tile's first store group is queued), so the epilogue never idles
    // on the NVLink round trip.
    int pend_t = -1, pend_owner = -1;
    int chunk_all = 0;               // staging chunks alternate over the whole launch (a ragged last tile may have an odd count)
    auto signal_tile = [&](int tt, int town) {
      asm volatile("fence.proxy.async;" ::: "memory");    // bulk (async-proxy) writes -> ordinary loads
      __threadfence_system();
      for (int pr = 0; pr < p.tp && p.mode != MODE_LOCAL; pr++) {
        if (pr == p.rank || (town >= 0 && pr != town)) continue;
        red_release_sys_add(p.flags[pr] + (size_t)p.rank * num_tiles + tt, 4);
      }
      atomicAdd(const_cast<int*>(s_pub), 4);
    };
    for (int t = worker; !copier && ok && t < num_tiles; t += n_workers, tcount++) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const int acc = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      if (!mbar_wait(bar_tfull + 8 * acc, aph, abort_flag, 3, p.err, p.wait_ns)) { ok = false; break; }
      tc_fence_after();
      const int owner = p.mode == MODE_RS ? owner_of(tm) : -1;
      const bool mine = owner < 0 || owner == p.rank;
      const int out_row0 = p.mode == MODE_RS ? tm * BM - p.rank * rows_per_rank : tm * BM;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      const int r_in = q * 32 + lane;                       // row inside the tile
      const int row = tm * BM + r_in;
      const bool row_ok = row < p.M;
      const bool local = p.mode == MODE_LOCAL;
      const bool issuer = (warp == 2 && lane == 0);
      int chunk_no = 0;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 64, chunk_no++) {
        const int col = tn * BN + c0;
        if (col >= p.N) break;
        const uint32_t sbuf = smem_epi + ((chunk_all++) & 1) * EPI_CHUNK_BYTES;
        // the bulk store that last read this staging chunk must be done with it
        if (issuer) tma_store_wait_read1();
        epi_bar_sync();
#pragma unroll
        for (int h = 0; h < 2; h++) {
          uint32_t r[32];
          tmem_ld32(taddr + c0 + 32 * h, r);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
          if (local && p.epi != EPI_NONE) {
            const int cb = col + 32 * h;
            const bool full = cb + 32 <= p.N;
            if (p.epi == EPI_BIAS || p.epi == EPI_BIAS_GELU) {
#pragma unroll
              for (int j = 0; j < 4; j++) {
                if (cb + 8 * j >= p.N) break;
                const uint4 b4 = __ldg(reinterpret_cast<const uint4*>(p.bias + cb + 8 * j));
                const float2 f0 = unpack_bf16(b4.x), f1 = unpack_bf16(b4.y), f2 = unpack_bf16(b4.z), f3 = unpack_bf16(b4.w);
                v[8 * j] += f0.x; v[8 * j + 1] += f0.y; v[8 * j + 2] += f1.x; v[8 * j + 3] += f1.y;
                v[8 * j + 4] += f2.x; v[8 * j + 5] += f2.y; v[8 * j + 6] += f3.x; v[8 * j + 7] += f3.y;
              }
            }
            if (p.epi == EPI_BIAS_GELU) {
              // the stored pre-activation is bf16; GELU is applied to the rounded value (as in the plain GEMM)
              if (row_ok) {
                bf16* ap = p.aux + (size_t)row * p.ldaux + cb;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  if (!full && cb + 8 * j >= p.N) break;
                  uint4 o;
                  o.x = pack_bf16(v[8 * j], v[8 * j + 1]); o.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
                  o.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]); o.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
                  reinterpret_cast<uint4*>(ap)[j] = o;
                }
              }
#pragma unroll
              for (int i = 0; i < 32; i++) v[i] = gelu_tanh(__bfloat162float(__float2bfloat16(v[i])));
            } else if (p.epi == EPI_DGELU) {
              if (row_ok) {
                const bf16* ap = p.aux + (size_t)row * p.ldaux + cb;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  if (!full && cb + 8 * j >= p.N) break;
                  const uint4 x4 = reinterpret_cast<const uint4*>(ap)[j];
                  const float2 f0 = unpack_bf16(x4.x), f1 = unpack_bf16(x4.y), f2 = unpack_bf16(x4.z), f3 = unpack_bf16(x4.w);
                  v[8 * j] *= gelu_tanh_grad(f0.x); v[8 * j + 1] *= gelu_tanh_grad(f0.y);
                  v[8 * j + 2] *= gelu_tanh_grad(f1.x); v[8 * j + 3] *= gelu_tanh_grad(f1.y);
                  v[8 * j + 4] *= gelu_tanh_grad(f2.x); v[8 * j + 5] *= gelu_tanh_grad(f2.y);
                  v[8 * j + 6] *= gelu_tanh_grad(f3.x); v[8 * j + 7] *= gelu_tanh_grad(f3.y);
                }
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 4; j++) {
            uint4 o;
            o.x = pack_bf16(v[8 * j], v[8 * j + 1]); o.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
            o.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]); o.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
            const int chunk16 = h * 4 + j;
            st_shared_v4(sbuf + r_in * 128 + ((chunk16 ^ (r_in & 7)) << 4), o);
          }
        }
        if (c0 + 64 >= BN || col + 64 >= p.N) {            // accumulator fully read: hand it back early
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * acc);
        }
        fence_proxy_async_smem();
        epi_bar_sync();
        if (issuer) {
          if (mine) tma_store_2d(&maps.out, sbuf, col, out_row0);
          for (int pr = 0; pr < p.tp && p.mode != MODE_LOCAL; pr++) {
            if (pr == p.rank || (owner >= 0 && pr != owner)) continue;
            tma_store_2d(&maps.st[par][pr], sbuf, col, tm * BM);
          }
          tma_store_commit();
          if (chunk_no == 0 && pend_t >= 0) {
            asm volatile("cp.async.bulk.wait_group 1;" ::: "memory");   // everything but the group just queued
            signal_tile(pend_t, pend_owner);
            pend_t = -1;
          }
        }
      }
      pend_t = t; pend_owner = owner;
    }
    if (warp == 2 && lane == 0 && pend_t >= 0) {
      tma_store_wait_all();
      signal_tile(pend_t, pend_owner);
    }
  } else {
    // ---------------------------------------------------------------- reducer warps
    const int rw = warp - 6;
    int tcount = 0;
    bool ok = true;
    for (int t = worker; !copier && ok && p.mode != MODE_LOCAL && t < num_tiles; t += n_workers, tcount++) {
      int tm, tn;
      tile_coord(t, tm, tn);
      const int owner = p.mode == MODE_RS ? owner_of(tm) : -1;
      int good = 1;
      if (lane == 0) {
        good = wait_smem_count(s_pub, 4 * (tcount + 1), abort_flag, p.err, p.wait_ns) ? 1 : 0;
        if (good && (owner < 0 || owner == p.rank)) {
          for (int pr = 0; pr < p.tp && good; pr++) {
            if (pr == p.rank) continue;
            good = wait_counter(p.flags[p.rank] + (size_t)pr * num_tiles + t, target, abort_flag, p.err, p.wait_ns) ? 1 : 0;
          }
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) { ok = false; break; }
      if (owner >= 0 && owner != p.rank) continue;      // another rank reduces this tile
      __threadfence();
      const int col = tn * BN + lane * 8;
      if (col >= p.N) continue;
      float bias8[8];
#pragma unroll
      for (int k = 0; k < 8; k++) bias8[k] = 0.f;
      if (p.bias) {
        uint4 b = __ldg(reinterpret_cast<const uint4*>(p.bias + col));
        float2 f0 = unpack_bf16(b.x), f1 = unpack_bf16(b.y), f2 = unpack_bf16(b.z), f3 = unpack_bf16(b.w);
        bias8[0] = f0.x; bias8[1] = f0.y; bias8[2] = f1.x; bias8[3] = f1.y; bias8[4] = f2.x; bias8[5] = f2.y; bias8[6] = f3.x; bias8[7] = f3.y;
      }
      const int row_end = min(p.M, (tm + 1) * BM);
      // 8 rows per pass so that each lane keeps 8 x (tp + 1) independent 16-byte loads in flight
      constexpr int RB = 8;
      for (int row0 = tm * BM + rw * RB; row0 < row_end; row0 += 4 * RB) {
        float a8[RB][8];
#pragma unroll
        for (int i = 0; i < RB; i++)
#pragma unroll
          for (int k = 0; k < 8; k++) a8[i][k] = bias8[k];
        for (int r = 0; r < p.tp; r++) {
          uint4 v[RB];
#pragma unroll
          for (int i = 0; i < RB; i++) {
            const int row = row0 + i;
            const int out_row = p.mode == MODE_RS ? row - p.rank * rows_per_rank : row;
            const uint4* src = (r == p.rank)
                                   ? reinterpret_cast<const uint4*>(p.out + (size_t)out_row * p.ldo + col)
                                   : reinterpret_cast<const uint4*>(my_stage + ((size_t)r * p.M + row) * p.N + col);
            v[i] = row < row_end ? __ldcg(src) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int i = 0; i < RB; i++) {
            float2 f0 = unpack_bf16(v[i].x), f1 = unpack_bf16(v[i].y), f2 = unpack_bf16(v[i].z), f3 = unpack_bf16(v[i].w);
            a8[i][0] += f0.x; a8[i][1] += f0.y; a8[i][2] += f1.x; a8[i][3] += f1.y;
            a8[i][4] += f2.x; a8[i][5] += f2.y; a8[i][6] += f3.x; a8[i][7] += f3.y;
          }
        }
        if (p.resid) {
          uint4 v[RB];
#pragma unroll
          for (int i = 0; i < RB; i++) {
            const int row = row0 + i;
            const int out_row = p.mode == MODE_RS ? row - p.rank * rows_per_rank : row;
            v[i] = row < row_end ? *reinterpret_cast<const uint4*>(p.resid + (size_t)out_row * p.ldr + col) : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
          for (int i = 0; i < RB; i++) {
            float2 f0 = unpack_bf16(v[i].x), f1 = unpack_bf16(v[i].y), f2 = unpack_bf16(v[i].z), f3 = unpack_bf16(v[i].w);
            a8[i][0] += f0.x; a8[i][1] += f0.y; a8[i][2] += f1.x; a8[i][3] += f1.y;
            a8[i][4] += f2.x; a8[i][5] += f2.y; a8[i][6] += f3.x; a8[i][7] += f3.y;
          }
        }
#pragma unroll
        for (int i = 0; i < RB; i++) {
          const int row = row0 + i;
          if (row >= row_end) break;
          const int out_row = p.mode == MODE_RS ? row - p.rank * rows_per_rank : row;
          uint4 o;
          o.x = pack_bf16(a8[i][0], a8[i][1]); o.y = pack_bf16(a8[i][2], a8[i][3]);
          o.z = pack_bf16(a8[i][4], a8[i][5]); o.w = pack_bf16(a8[i][6], a8[i][7]);
          *reinterpret_cast<uint4*>(p.out + (size_t)out_row * p.ldo + col) = o;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
  if (p.epoch && threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.epoch + 1, 1u) == gridDim.x - 1) {
      p.epoch[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(p.epoch) = call;
    }
  }
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

}  // namespace

// Fused tensor-parallel GEMM.  `a_ptrs`: one pointer (local A) or, when gather != 0, tp pointers
// to the per-rank row shards [M/tp, K] (or [K, M/tp] when a_mn) mapped into this process.
// `stage_ptrs`, `flag_ptrs`, `ready_ptrs`: tp entries each, index r = rank r's buffer as seen from
// this process (own entry = local buffer).  Staging holds tp slots of M*N bf16; flags hold
// tp * ceil(M/128) * ceil(N/256) counters; ready holds tp counters.  Staging is two parities of
// tp * M * N bf16 each; `stage_ptrs` are the parity-0 bases.  The call count of the buffer set
// (identical on all ranks) is either kept by the kernel in the two zero-initialised words at
// `epoch_ptr` (local device memory) or, when that is 0, passed as the 1-based `call_no`.
// `epi` / `aux` / `ldaux`: epilogue of the all-gather form (mode 2): 0 none, 1 + bias, 2 + bias then GELU
// with the pre-activation stored to aux, 4 times GELU'(aux).
// Returns 0 or -1.
extern "C" int kh_gemm_comm(const unsigned long long* a_ptrs, int lda, int a_mn, const void* B, int ldb, int b_mn,
                            void* out, int ldo, int M, int N, int K, int mode, int gather, int tp, int rank,
                            const unsigned long long* stage_ptrs, const unsigned long long* flag_ptrs,
                            const unsigned long long* ready_ptrs, unsigned call_no, unsigned gather_no,
                            unsigned long long epoch_ptr, void* gather_buf, void* blk_ready, const void* bias, const void* resid, int ldr,
                            int epi, void* aux, int ldaux, int max_ctas, void* stream) {
  if (tp < 2 || tp > MAX_TP || rank < 0 || rank >= tp) { kh_set_error("gemm_comm: bad tp/rank %d/%d", rank, tp); return -1; }
  if ((mode == MODE_RS || gather) && M % (tp * BM)) { kh_set_error("gemm_comm: M=%d must be a multiple of tp*128 for row-sharded modes", M); return -1; }
  if (M < 1) { kh_set_error("gemm_comm: empty problem"); return -1; }
  if (epi != EPI_NONE && mode != MODE_LOCAL) { kh_set_error("gemm_comm: epilogues other than bias + residual belong to the all-gather form"); return -1; }
  if (epi != EPI_NONE && epi != EPI_BIAS && epi != EPI_BIAS_GELU && epi != EPI_DGELU) { kh_set_error("gemm_comm: unknown epilogue %d", epi); return -1; }
  if ((epi == EPI_BIAS || epi == EPI_BIAS_GELU) && (!bias || ((uintptr_t)bias & 15))) { kh_set_error("gemm_comm: bias missing or misaligned"); return -1; }
  if ((epi == EPI_BIAS_GELU || epi == EPI_DGELU) && (!aux || (ldaux % 8) || ((uintptr_t)aux & 15))) { kh_set_error("gemm_comm: aux operand missing or misaligned"); return -1; }
  if (gather && mode != MODE_LOCAL) {
    // the gather form rotates the tile order by rank, so tile index t names different tiles on different
    // ranks and the per-tile arrival counters of a reduction would not line up
    kh_set_error("gemm_comm: the all-gather form has no reduction (mode must be 2)");
    return -1;
  }
  // the all-gather form without an epilogue writes its output only through clipped TMA stores: any N
  const bool ragged_ok = mode == MODE_LOCAL && epi == EPI_NONE;
  if ((N % 8 && !ragged_ok) || ldo % 8 || ((uintptr_t)out & 15)) { kh_set_error("gemm_comm: N and the output pitch must be multiples of 8"); return -1; }
  if (gather && (a_mn || lda != K || !gather_buf || !blk_ready || !epoch_ptr)) {
    kh_set_error("gemm_comm: gather mode needs row-major contiguous shards (lda == K), a gather buffer, block counters and an epoch word");
    return -1;
  }
  Maps maps;
  const int rows_a = gather ? M / tp : M;
  {   // the local operand: the whole A, or in gather mode this rank's own shard
    const int r = gather ? rank : 0;
    const void* A = (const void*)a_ptrs[r];
    const CUtensorMap* ta = a_mn ? kh_tmap_2d_bf16(A, K, rows_a, lda, BK, 64) : kh_tmap_2d_bf16(A, rows_a, K, lda, BM, BK);
    if (!ta) return -1;
    maps.a[r] = *ta;
  }
  if (gather) {
    const CUtensorMap* tg = kh_tmap_2d_bf16(gather_buf, M, K, K, BM, BK);
    if (!tg) return -1;
    maps.g = *tg;
  }
  const CUtensorMap* tb = b_mn ? kh_tmap_2d_bf16(B, K, N, ldb, BK, 64) : kh_tmap_2d_bf16(B, N, K, ldb, BN, BK);
  if (!tb) return -1;
  maps.b = *tb;
  const int out_rows = mode == MODE_RS ? M / tp : M;
  const CUtensorMap* to = kh_tmap_2d_bf16(out, out_rows, N, ldo, BM, 64);
  if (!to) return -1;
  maps.out = *to;
  const size_t slot_elems = (size_t)tp * M * N;
  for (int par = 0; par < 2; par++)
    for (int r = 0; r < tp; r++) {
      if (r == rank || mode == MODE_LOCAL) continue;
      const CUtensorMap* ts = kh_tmap_2d_bf16((const bf16*)stage_ptrs[r] + par * slot_elems + (size_t)rank * M * N, M, N, N, BM, 64);
      if (!ts) return -1;
      maps.st[par][r] = *ts;
    }
  CommParams p = {};
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.mode = mode; p.tp = tp; p.rank = rank; p.gather = gather;
  p.out = (bf16*)out; p.ldo = ldo; p.bias = (const bf16*)bias; p.resid = (const bf16*)resid; p.ldr = ldr;
  p.epi = epi; p.aux = (bf16*)aux; p.ldaux = ldaux;
  for (int r = 0; r < tp; r++) {
    p.stage[r] = (bf16*)stage_ptrs[r];
    p.flags[r] = (uint32_t*)flag_ptrs[r];
    p.ready[r] = ready_ptrs ? (uint32_t*)ready_ptrs[r] : nullptr;
  }
  int n_copy = 0;
  if (gather) {
    for (int r = 0; r < tp; r++) p.shard[r] = (const bf16*)a_ptrs[r];
    p.gbuf = (bf16*)gather_buf;
    p.blk_ready = (uint32_t*)blk_ready;
    n_copy = 12;
  }
  p.n_copy = n_copy;
  p.call_no = call_no;
  p.slot_elems = slot_elems;
  p.epoch = (uint32_t*)epoch_ptr;
  p.ready_target = gather_no;
  p.wait_ns = kh_peer_wait_limit_ns();
  p.err = kh_error_word_dev();
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemm_comm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) { kh_set_error("gemm_comm: shared memory opt-in failed: %s", cudaGetErrorString(e)); return -1; }
    attr = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int grid = tiles < num_sms() - n_copy ? tiles : num_sms() - n_copy;
  if (max_ctas > 0 && grid > max_ctas - n_copy) grid = max_ctas - n_copy;
  if (grid < 1) grid = 1;
  grid += n_copy;
  KH_LAUNCH(gemm_comm_kernel, grid, THREADS, SMEM, (cudaStream_t)stream, maps, p);
  KH_LAUNCH_CHECK("gemm_comm");
  return 0;
}
