// Memory-bound kernels around the GEMMs: embedding forward/backward, deterministic column
// sums (bias gradients), LayerNorm forward/backward, fused softmax-cross-entropy, fused AdamW
// with bf16 weight emission, and small utilities.  All reductions run in a fixed order (no
// floating-point atomics) so that a resumed run reproduces the original bit for bit.
//
// Reference counterparts (src/core/kernels.cu): embed_k :125, layernorm_fwd_k :145,
// ce_fwd_k/ce_bwd_k :310-353, grpo_dlogits_k :358, gather_prob_k :372, layernorm_bwd_* :380-414,
// colsum_k :511, embed_bwd_* :526-563, adamw_k :566, f2b_k :583; model_sync_bf16 gpt.c:377.
#include <atomic>

#include "common.cuh"

static inline int cdiv(long a, long b) { return (int)((a + b - 1) / b); }
#define KH_LAUNCH_CHECK(name)                                                     \
  do {                                                                            \
    cudaError_t e_ = cudaGetLastError();                                          \
    if (e_ != cudaSuccess) { kh_set_error(name ": %s", cudaGetErrorString(e_)); return -1; } \
  } while (0)

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

// ------------------------------------------------------------------------------ embedding
// out[r, :] = wte[tok[r], :] + wpe[pos[r], :]   (pos == nullptr: position r % T)
__global__ void embed_fwd_k(const int* __restrict__ tok, const int* __restrict__ pos, const bf16* __restrict__ wte,
                            const bf16* __restrict__ wpe, bf16* __restrict__ out, int rows, int d, int T, int V, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  int t = tok[r];
  int ps = pos ? pos[r] : r % T;
  // index guard (the reference indexes wte / wpe unchecked, src/kernels/paged.cu:28): an id or position
  // outside the tables is recorded in the status word (code 8) and clamped, never dereferenced
  if ((t < 0 || t >= V || ps < 0 || ps >= T) && threadIdx.x == 0) atomicCAS(err, 0, 8);
  t = min(max(t, 0), V - 1);
  ps = min(max(ps, 0), T - 1);
  const uint4* a = reinterpret_cast<const uint4*>(wte + (size_t)t * d);
  const uint4* b = reinterpret_cast<const uint4*>(wpe + (size_t)ps * d);
  uint4* o = reinterpret_cast<uint4*>(out + (size_t)r * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) {
    uint4 x = __ldg(a + i), y = __ldg(b + i), z;
    float2 x0 = unpack_bf16(x.x), y0 = unpack_bf16(y.x); z.x = pack_bf16(x0.x + y0.x, x0.y + y0.y);
    float2 x1 = unpack_bf16(x.y), y1 = unpack_bf16(y.y); z.y = pack_bf16(x1.x + y1.x, x1.y + y1.y);
    float2 x2 = unpack_bf16(x.z), y2 = unpack_bf16(y.z); z.z = pack_bf16(x2.x + y2.x, x2.y + y2.y);
    float2 x3 = unpack_bf16(x.w), y3 = unpack_bf16(y.w); z.w = pack_bf16(x3.x + y3.x, x3.y + y3.y);
    o[i] = z;
  }
}
extern "C" int kh_embed_fwd(const void* tok, const void* pos, const void* wte, const void* wpe, void* out, int rows,
                            int d, int T, int V, void* stream) {
  if (d % 8) { kh_set_error("embed: d must be a multiple of 8"); return -1; }
  KH_LAUNCH(embed_fwd_k, rows, 128, 0, (cudaStream_t)stream, (const int*)tok, (const int*)pos, (const bf16*)wte,
                                                      (const bf16*)wpe, (bf16*)out, rows, d, T, V, kh_error_word_dev());
  KH_LAUNCH_CHECK("embed_fwd");
  return 0;
}

// dwte[tok[r], :] += dx[r, :], deterministic and O(R d): integer atomics (order-independent
// results) find, per token id, its first row and its multiplicity; the first row owns the
// update and, only when the id occurs more than once, folds in the later rows in row order.
// `table` is int scratch of 2*V entries.
__global__ void embed_bwd_index_k(const int* __restrict__ tok, int* __restrict__ first, int* __restrict__ cnt,
                                  int rows, int V) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= rows) return;
  const int t = tok[r];
  if (t < 0 || t >= V) return;
  atomicMin(first + t, r);
  atomicAdd(cnt + t, 1);
}
__global__ void embed_bwd_wte_k(const int* __restrict__ tok, const bf16* __restrict__ dx, float* __restrict__ dwte,
                                const int* __restrict__ first, const int* __restrict__ cnt, int rows, int d, int V) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ int s_list[64];
  __shared__ int s_n;
  const int r = blockIdx.x;
  const int t = tok[r];
  if (t < 0 || t >= V || first[t] != r) return;
  const int dup = cnt[t];
  int n_list = 0;
  if (dup > 1) {
    // warp 0 collects the later rows with the same id, in row order (ballot + prefix popcount)
    if (threadIdx.x < 32) {
      int n = 0;
      for (int base = r + 1; base < rows && n < dup - 1; base += 32) {
        const int i = base + threadIdx.x;
        const bool hit = i < rows && tok[i] == t;
        const unsigned mask = __ballot_sync(0xffffffffu, hit);
        if (hit) {
          const int at = n + __popc(mask & ((1u << threadIdx.x) - 1));
          if (at < 64) s_list[at] = i;
        }
        n += __popc(mask);
      }
      if (threadIdx.x == 0) s_n = n;
    }
    __syncthreads();
    n_list = s_n;
  }
  for (int e = threadIdx.x * 2; e < d; e += blockDim.x * 2) {
    float2 acc = unpack_bf16(*reinterpret_cast<const uint32_t*>(dx + (size_t)r * d + e));
    if (n_list <= 64) {
      for (int k = 0; k < n_list; k++) {
        float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(dx + (size_t)s_list[k] * d + e));
        acc.x += v.x; acc.y += v.y;
      }
    } else {   // very frequent id: plain ordered scan
      for (int i = r + 1; i < rows; i++)
        if (tok[i] == t) {
          float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(dx + (size_t)i * d + e));
          acc.x += v.x; acc.y += v.y;
        }
    }
    float2* o = reinterpret_cast<float2*>(dwte + (size_t)t * d + e);
    float2 old = *o;
    old.x += acc.x; old.y += acc.y;
    *o = old;
  }
}
// dwpe[t, :] += sum_b dx[b*T + t, :]
__global__ void embed_bwd_wpe_k(const bf16* __restrict__ dx, float* __restrict__ dwpe, int B, int T, int d) {
  pdl_wait();
  pdl_launch_dependents();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)T * d) return;
  float acc = 0.f;
  for (int b = 0; b < B; b++) acc += __bfloat162float(dx[(size_t)b * T * d + i]);
  dwpe[i] += acc;
}
extern "C" int kh_embed_bwd(const void* tok, const void* dx, void* dwte, void* dwpe, void* table, int B, int T, int d,
                            int V, void* stream) {
  const int rows = B * T;
  cudaStream_t st = (cudaStream_t)stream;
  if (d % 2) { kh_set_error("embed_bwd: d must be even"); return -1; }
  if (dwte) {
    int* first = (int*)table;
    int* cnt = first + V;
    cudaMemsetAsync(first, 0x7f, (size_t)V * sizeof(int), st);
    cudaMemsetAsync(cnt, 0, (size_t)V * sizeof(int), st);
    KH_LAUNCH(embed_bwd_index_k, cdiv(rows, 256), 256, 0, st, (const int*)tok, first, cnt, rows, V);
    KH_LAUNCH(embed_bwd_wte_k, rows, 128, 0, st, (const int*)tok, (const bf16*)dx, (float*)dwte, first, cnt, rows, d, V);
  }
  if (dwpe) KH_LAUNCH(embed_bwd_wpe_k, cdiv((long)T * d, 256), 256, 0, st, (const bf16*)dx, (float*)dwpe, B, T, d);
  KH_LAUNCH_CHECK("embed_bwd");
  return 0;
}

// ------------------------------------------------------------------------------ column sum
// out[j] (+)= sum_r x[r, j], deterministic.  CTA (column block of 64, row split s) sums its rows
// with 16-byte loads (8 threads span the 64 columns, 32 row lanes) and writes one partial row
// to `scratch`; the CTA that finishes last for a column block (ticket counter) adds the splits
// in index order, so the result does not depend on which CTA that is.
// scratch layout: [KH_COUNTER_SLOTS ints, zero between launches][splits x N floats].
#define KH_COUNTER_SLOTS 1024
__global__ void colsum_k(const bf16* __restrict__ x, int ld, float* __restrict__ out, int* __restrict__ counters,
                         float* __restrict__ scratch, int rows, int N, int rows_per_split, int accumulate) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float part[32][65];
  __shared__ int s_last;
  const int cg = threadIdx.x & 7, rg = threadIdx.x >> 3;
  const int col = blockIdx.x * 64 + cg * 8;
  const int r0 = blockIdx.y * rows_per_split, r1 = min(rows, r0 + rows_per_split);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; k++) acc[k] = 0.f;
  if (col + 8 <= N) {
    auto add = [&](const uint4& v) {
      float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += e.x; acc[7] += e.y;
    };
    int r = r0 + rg;
    // four rows per trip: four independent 16-byte loads in flight per thread, added in row order
    for (; r + 96 < r1; r += 128) {
      const bf16* p0 = x + (size_t)r * ld + col;
      const uint4 v0 = *reinterpret_cast<const uint4*>(p0);
      const uint4 v1 = *reinterpret_cast<const uint4*>(p0 + (size_t)32 * ld);
      const uint4 v2 = *reinterpret_cast<const uint4*>(p0 + (size_t)64 * ld);
      const uint4 v3 = *reinterpret_cast<const uint4*>(p0 + (size_t)96 * ld);
      add(v0); add(v1); add(v2); add(v3);
    }
    for (; r < r1; r += 32) add(*reinterpret_cast<const uint4*>(x + (size_t)r * ld + col));
  } else {
    for (int r = r0 + rg; r < r1; r += 32)
      for (int k = 0; k < 8; k++) if (col + k < N) acc[k] += __bfloat162float(x[(size_t)r * ld + col + k]);
  }
#pragma unroll
  for (int k = 0; k < 8; k++) part[rg][cg * 8 + k] = acc[k];
  __syncthreads();
  const int c = blockIdx.x * 64 + threadIdx.x;
  if (threadIdx.x < 64 && c < N) {
    float sacc = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) sacc += part[k][threadIdx.x];
    scratch[(size_t)blockIdx.y * N + c] = sacc;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(counters + blockIdx.x, 1) == (int)gridDim.y - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 64 && c < N) {
    float sacc = accumulate ? out[c] : 0.f;
    for (int k = 0; k < (int)gridDim.y; k++) sacc += __ldcg(scratch + (size_t)k * N + c);
    out[c] = sacc;
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0;
}
extern "C" int kh_colsum_splits(int rows, int N) {
  const int cb = (N + 63) / 64;
  int splits = (592 + cb - 1) / cb;
  const int max_by_rows = (rows + 63) / 64;
  if (splits > max_by_rows) splits = max_by_rows;
  return splits < 1 ? 1 : splits;
}
// fp32 elements of scratch kh_colsum needs (counter slots included); must start zeroed
extern "C" long kh_colsum_scratch_elems(int rows, int N) { return KH_COUNTER_SLOTS + (long)kh_colsum_splits(rows, N) * N; }
extern "C" int kh_colsum(const void* x, int ld, void* out, void* scratch, int rows, int N, int accumulate, void* stream) {
  if (ld % 8 || ((uintptr_t)x & 15)) { kh_set_error("colsum: input pitch/base must be 16-byte aligned"); return -1; }
  if ((N + 63) / 64 > KH_COUNTER_SLOTS) { kh_set_error("colsum: N=%d exceeds %d column blocks", N, KH_COUNTER_SLOTS); return -1; }
  const int splits = kh_colsum_splits(rows, N);
  const int rps = (rows + splits - 1) / splits;
  dim3 grid(cdiv(N, 64), splits);
  KH_LAUNCH(colsum_k, grid, 256, 0, (cudaStream_t)stream, (const bf16*)x, ld, (float*)out, (int*)scratch,
                                                    (float*)scratch + KH_COUNTER_SLOTS, rows, N, rps, accumulate);
  KH_LAUNCH_CHECK("colsum");
  return 0;
}

// ---- column sum for callers that cannot allocate -------------------------------------------
// Scratch of kh_colsum_noalloc: lives in the library image, one copy per GPU that loads the
// library, held until the process exits.  Layout as for kh_colsum: ticket counters, then partial rows.
#define KH_NOALLOC_PARTIAL_FLOATS 65536
static __device__ __align__(256) float g_colsum_static_scratch[KH_COUNTER_SLOTS + KH_NOALLOC_PARTIAL_FLOATS];

// See kharon_cuda.h for the contract.  In host code the array's name is only a handle for the
// runtime, not a device address, so the address is looked up once per device with
// cudaGetSymbolAddress (with that device current) and cached.
extern "C" int kh_colsum_noalloc(const void* x, int ld, void* out, int rows, int N, int accumulate, void* stream) {
  static std::atomic<float*> dev_ptr[64];     // zero-initialised; threads may race to fill an entry with the same value
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { kh_set_error("colsum_noalloc: no current device"); return -1; }
  if (rows <= 0 || N <= 0) { kh_set_error("colsum_noalloc: empty problem %d x %d", rows, N); return -1; }
  if (ld % 8 || ((uintptr_t)x & 15)) { kh_set_error("colsum_noalloc: input pitch/base must be 16-byte aligned"); return -1; }
  const int splits = kh_colsum_splits(rows, N);
  if ((N + 63) / 64 > KH_COUNTER_SLOTS || (long)splits * N > KH_NOALLOC_PARTIAL_FLOATS) {
    kh_set_error("colsum_noalloc: %d x %d needs %ld partial floats, the built-in scratch holds %d (use kh_colsum with caller scratch)",
                 rows, N, (long)splits * N, KH_NOALLOC_PARTIAL_FLOATS);
    return -1;
  }
  if (!dev_ptr[dev].load(std::memory_order_acquire)) {   // first call on this device: resolve the array's device address
    float* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_colsum_static_scratch);
    if (e != cudaSuccess || !ptr) { kh_set_error("colsum_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e)); return -1; }
    dev_ptr[dev].store(ptr, std::memory_order_release);
  }
  float* scratch = dev_ptr[dev].load(std::memory_order_acquire);
  cudaStream_t st = (cudaStream_t)stream;
  // the array keeps whatever the previous call left; the ticket counters must start at zero
  cudaError_t e = cudaMemsetAsync(scratch, 0, KH_COUNTER_SLOTS * sizeof(int), st);
  if (e != cudaSuccess) { kh_set_error("colsum_noalloc: clearing the counters failed: %s", cudaGetErrorString(e)); return -1; }
  const int rps = (rows + splits - 1) / splits;
  dim3 grid(cdiv(N, 64), splits);
  KH_LAUNCH(colsum_k, grid, 256, 0, st, (const bf16*)x, ld, (float*)out, (int*)scratch, scratch + KH_COUNTER_SLOTS, rows, N, rps,
                                 accumulate);
  KH_LAUNCH_CHECK("colsum_noalloc");
  return 0;
}

// ------------------------------------------------------------------------------ LayerNorm
// One warp per row; statistics in fp32 with a two-pass variance (eps 1e-5, biased variance).
__global__ void layernorm_fwd_k(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                                bf16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows,
                                int d) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)row * d);
  const int nv = d / 8;
  float s = 0.f;
  for (int i = lane; i < nv; i += 32) {
    uint4 v = xp[i];
    float2 a = unpack_bf16(v.x), bb = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
    s += (a.x + a.y) + (bb.x + bb.y) + (c.x + c.y) + (e.x + e.y);
  }
  const float mu = warp_sum(s) / d;
  float q = 0.f;
  for (int i = lane; i < nv; i += 32) {
    uint4 v = xp[i];
    float2 a = unpack_bf16(v.x), bb = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
    float t;
    t = a.x - mu; q += t * t; t = a.y - mu; q += t * t; t = bb.x - mu; q += t * t; t = bb.y - mu; q += t * t;
    t = c.x - mu; q += t * t; t = c.y - mu; q += t * t; t = e.x - mu; q += t * t; t = e.y - mu; q += t * t;
  }
  const float rs = rsqrtf(warp_sum(q) / d + 1e-5f);
  if (lane == 0) { if (mean) mean[row] = mu; if (rstd) rstd[row] = rs; }
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  const uint4* bp = reinterpret_cast<const uint4*>(b);
  uint4* yp = reinterpret_cast<uint4*>(y + (size_t)row * d);
  for (int i = lane; i < nv; i += 32) {
    uint4 v = xp[i], wv = __ldg(wp + i), bv = __ldg(bp + i), o;
    const uint32_t* vi = &v.x; const uint32_t* wi = &wv.x; const uint32_t* bi = &bv.x; uint32_t* oi = &o.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 xv = unpack_bf16(vi[k]), ww = unpack_bf16(wi[k]), bb = unpack_bf16(bi[k]);
      oi[k] = pack_bf16((xv.x - mu) * rs * ww.x + bb.x, (xv.y - mu) * rs * ww.y + bb.y);
    }
    yp[i] = o;
  }
}
// Same arithmetic for d = NPL * 256: the warp reads its row once (NPL independent 16-byte loads per
// lane, all in flight together) and keeps it in registers for the three sweeps.
template <int NPL>
__global__ void __launch_bounds__(256)
layernorm_fwd_reg_k(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                    bf16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int d = NPL * 256;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)row * d);
  uint4 v[NPL];
#pragma unroll
  for (int j = 0; j < NPL; j++) v[j] = xp[lane + 32 * j];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < NPL; j++) {
    float2 a = unpack_bf16(v[j].x), bb = unpack_bf16(v[j].y), c = unpack_bf16(v[j].z), e = unpack_bf16(v[j].w);
    s += (a.x + a.y) + (bb.x + bb.y) + (c.x + c.y) + (e.x + e.y);
  }
  const float mu = warp_sum(s) / d;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < NPL; j++) {
    float2 a = unpack_bf16(v[j].x), bb = unpack_bf16(v[j].y), c = unpack_bf16(v[j].z), e = unpack_bf16(v[j].w);
    float t;
    t = a.x - mu; q += t * t; t = a.y - mu; q += t * t; t = bb.x - mu; q += t * t; t = bb.y - mu; q += t * t;
    t = c.x - mu; q += t * t; t = c.y - mu; q += t * t; t = e.x - mu; q += t * t; t = e.y - mu; q += t * t;
  }
  const float rs = rsqrtf(warp_sum(q) / d + 1e-5f);
  if (lane == 0) { if (mean) mean[row] = mu; if (rstd) rstd[row] = rs; }
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  const uint4* bp = reinterpret_cast<const uint4*>(b);
  uint4* yp = reinterpret_cast<uint4*>(y + (size_t)row * d);
#pragma unroll
  for (int j = 0; j < NPL; j++) {
    const int i = lane + 32 * j;
    uint4 wv = __ldg(wp + i), bv = __ldg(bp + i), o;
    const uint32_t* vi = &v[j].x; const uint32_t* wi = &wv.x; const uint32_t* bi = &bv.x; uint32_t* oi = &o.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 xv = unpack_bf16(vi[k]), ww = unpack_bf16(wi[k]), bb = unpack_bf16(bi[k]);
      oi[k] = pack_bf16((xv.x - mu) * rs * ww.x + bb.x, (xv.y - mu) * rs * ww.y + bb.y);
    }
    yp[i] = o;
  }
}
extern "C" int kh_layernorm_fwd(const void* x, const void* w, const void* b, void* y, void* mean, void* rstd, int rows,
                                int d, void* stream) {
  if (d % 8) { kh_set_error("layernorm: d must be a multiple of 8"); return -1; }
  if (d == 2048)
    KH_LAUNCH((layernorm_fwd_reg_k<8>), cdiv(rows, 8), 256, 0, (cudaStream_t)stream, (const bf16*)x, (const bf16*)w, (const bf16*)b,
                                                                           (bf16*)y, (float*)mean, (float*)rstd, rows);
  else if (d == 1024)
    KH_LAUNCH((layernorm_fwd_reg_k<4>), cdiv(rows, 8), 256, 0, (cudaStream_t)stream, (const bf16*)x, (const bf16*)w, (const bf16*)b,
                                                                           (bf16*)y, (float*)mean, (float*)rstd, rows);
  else
    KH_LAUNCH(layernorm_fwd_k, cdiv(rows, 8), 256, 0, (cudaStream_t)stream, (const bf16*)x, (const bf16*)w, (const bf16*)b,
                                                                      (bf16*)y, (float*)mean, (float*)rstd, rows, d);
  KH_LAUNCH_CHECK("layernorm_fwd");
  return 0;
}

// Backward, two kernels.
//  (1) dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w, optionally + dres (the
//      residual-stream gradient that bypasses the norm): one warp per row, the second sweep
//      over the row hits L1.
//  (2) dw[j] += sum_r dy * xhat, db[j] += sum_r dy: column-oriented like colsum -- CTA (64
//      columns, row split) accumulates in registers with 16-byte loads and writes one partial
//      row per split to `partials` ([splits, 2, d] fp32, caller-supplied scratch); a last
//      kernel adds the splits in index order into the fp32 gradient buffers.
__global__ void layernorm_bwd_dx_k(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                   const bf16* __restrict__ dres, bf16* __restrict__ dx, int rows, int d) {
  pdl_wait();
  pdl_launch_dependents();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* dyp = reinterpret_cast<const uint4*>(dy + (size_t)row * d);
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)row * d);
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  const float mu = mean[row], rs = rstd[row];
  const int nv = d / 8;
  float s1 = 0.f, s2 = 0.f;
  for (int i = lane; i < nv; i += 32) {
    uint4 gv = dyp[i], xv = xp[i], wv = __ldg(wp + i);
    const uint32_t* gi = &gv.x; const uint32_t* xi = &xv.x; const uint32_t* wi = &wv.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 g = unpack_bf16(gi[k]), xx = unpack_bf16(xi[k]), ww = unpack_bf16(wi[k]);
      float g0 = g.x * ww.x, g1 = g.y * ww.y;
      s1 += g0 + g1;
      s2 += g0 * ((xx.x - mu) * rs) + g1 * ((xx.y - mu) * rs);
    }
  }
  s1 = warp_sum(s1) / d;
  s2 = warp_sum(s2) / d;
  const uint4* rp = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * d) : nullptr;
  uint4* op = reinterpret_cast<uint4*>(dx + (size_t)row * d);
  for (int i = lane; i < nv; i += 32) {
    uint4 gv = dyp[i], xv = xp[i], wv = __ldg(wp + i), rv = make_uint4(0, 0, 0, 0), o;
    if (rp) rv = rp[i];
    const uint32_t* gi = &gv.x; const uint32_t* xi = &xv.x; const uint32_t* wi = &wv.x; const uint32_t* ri = &rv.x;
    uint32_t* oi = &o.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 g = unpack_bf16(gi[k]), xx = unpack_bf16(xi[k]), ww = unpack_bf16(wi[k]), rr = unpack_bf16(ri[k]);
      float xh0 = (xx.x - mu) * rs, xh1 = (xx.y - mu) * rs;
      oi[k] = pack_bf16(rs * (g.x * ww.x - s1 - xh0 * s2) + rr.x, rs * (g.y * ww.y - s1 - xh1 * s2) + rr.y);
    }
    op[i] = o;
  }
}
template <int NPL>
__global__ void __launch_bounds__(256)
layernorm_bwd_dx_reg_k(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                       const float* __restrict__ mean, const float* __restrict__ rstd,
                       const bf16* __restrict__ dres, bf16* __restrict__ dx, int rows) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int d = NPL * 256;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* dyp = reinterpret_cast<const uint4*>(dy + (size_t)row * d);
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)row * d);
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  const uint4* rp = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * d) : nullptr;
  const float mu = mean[row], rs = rstd[row];
  uint4 gv[NPL], xv[NPL], rv[NPL];
#pragma unroll
  for (int j = 0; j < NPL; j++) {
    gv[j] = dyp[lane + 32 * j];
    xv[j] = xp[lane + 32 * j];
    rv[j] = rp ? rp[lane + 32 * j] : make_uint4(0, 0, 0, 0);
  }
  float s1 = 0.f, s2 = 0.f;
#pragma unroll
  for (int j = 0; j < NPL; j++) {
    const uint4 wv = __ldg(wp + lane + 32 * j);
    const uint32_t* gi = &gv[j].x; const uint32_t* xi = &xv[j].x; const uint32_t* wi = &wv.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 g = unpack_bf16(gi[k]), xx = unpack_bf16(xi[k]), ww = unpack_bf16(wi[k]);
      float g0 = g.x * ww.x, g1 = g.y * ww.y;
      s1 += g0 + g1;
      s2 += g0 * ((xx.x - mu) * rs) + g1 * ((xx.y - mu) * rs);
    }
  }
  s1 = warp_sum(s1) / d;
  s2 = warp_sum(s2) / d;
  uint4* op = reinterpret_cast<uint4*>(dx + (size_t)row * d);
#pragma unroll
  for (int j = 0; j < NPL; j++) {
    const uint4 wv = __ldg(wp + lane + 32 * j);
    uint4 o;
    const uint32_t* gi = &gv[j].x; const uint32_t* xi = &xv[j].x; const uint32_t* wi = &wv.x; const uint32_t* ri = &rv[j].x;
    uint32_t* oi = &o.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 g = unpack_bf16(gi[k]), xx = unpack_bf16(xi[k]), ww = unpack_bf16(wi[k]), rr = unpack_bf16(ri[k]);
      float xh0 = (xx.x - mu) * rs, xh1 = (xx.y - mu) * rs;
      oi[k] = pack_bf16(rs * (g.x * ww.x - s1 - xh0 * s2) + rr.x, rs * (g.y * ww.y - s1 - xh1 * s2) + rr.y);
    }
    op[lane + 32 * j] = o;
  }
}
__global__ void layernorm_bwd_dwdb_k(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                     const float* __restrict__ mean, const float* __restrict__ rstd,
                                     int* __restrict__ counters, float* __restrict__ partials,
                                     float* __restrict__ dw, float* __restrict__ db, int rows, int d, int rows_per_split) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float part[32][2][65];
  __shared__ int s_last;
  const int cg = threadIdx.x & 7, rg = threadIdx.x >> 3;
  const int col = blockIdx.x * 64 + cg * 8;
  const int r0 = blockIdx.y * rows_per_split, r1 = min(rows, r0 + rows_per_split);
  float aw[8], ab[8];
#pragma unroll
  for (int k = 0; k < 8; k++) { aw[k] = 0.f; ab[k] = 0.f; }
  if (col < d) {
    for (int r = r0 + rg; r < r1; r += 32) {
      uint4 gv = *reinterpret_cast<const uint4*>(dy + (size_t)r * d + col);
      uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)r * d + col);
      const float mu = mean[r], rs = rstd[r];
      const uint32_t* gi = &gv.x; const uint32_t* xi = &xv.x;
#pragma unroll
      for (int k = 0; k < 4; k++) {
        float2 g = unpack_bf16(gi[k]), xx = unpack_bf16(xi[k]);
        aw[2 * k] += g.x * ((xx.x - mu) * rs); aw[2 * k + 1] += g.y * ((xx.y - mu) * rs);
        ab[2 * k] += g.x; ab[2 * k + 1] += g.y;
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; k++) { part[rg][0][cg * 8 + k] = aw[k]; part[rg][1][cg * 8 + k] = ab[k]; }
  __syncthreads();
  const int which = threadIdx.x >> 6, cc = threadIdx.x & 63;
  const int c = blockIdx.x * 64 + cc;
  if (threadIdx.x < 128 && c < d) {
    float sacc = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k++) sacc += part[k][which][cc];
    partials[((size_t)blockIdx.y * 2 + which) * d + c] = sacc;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = (atomicAdd(counters + blockIdx.x, 1) == (int)gridDim.y - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (threadIdx.x < 128 && c < d) {
    float* dst = which ? db : dw;
    float sacc = dst[c];
    for (int k = 0; k < (int)gridDim.y; k++) sacc += __ldcg(partials + ((size_t)k * 2 + which) * d + c);
    dst[c] = sacc;
  }
  if (threadIdx.x == 0) counters[blockIdx.x] = 0;
}
// Number of row splits layernorm_bwd uses; its scratch is KH_COUNTER_SLOTS + splits * 2 * d floats, zeroed once.
extern "C" int kh_layernorm_bwd_parts(int rows, int d) {
  const int cb = (d + 63) / 64;
  int parts = (592 + cb - 1) / cb;
  const int by_rows = (rows + 63) / 64;
  if (parts > by_rows) parts = by_rows;
  return parts < 1 ? 1 : parts;
}
extern "C" long kh_layernorm_bwd_scratch_elems(int rows, int d) {
  return KH_COUNTER_SLOTS + (long)kh_layernorm_bwd_parts(rows, d) * 2 * d;
}
extern "C" int kh_layernorm_bwd(const void* dy, const void* x, const void* w, const void* mean, const void* rstd,
                                const void* dres, void* dx, void* dw, void* db, void* partials, int rows, int d,
                                void* stream) {
  if (d % 8) { kh_set_error("layernorm_bwd: d must be a multiple of 8"); return -1; }
  if ((d + 63) / 64 > KH_COUNTER_SLOTS) { kh_set_error("layernorm_bwd: d=%d is too wide", d); return -1; }
  cudaStream_t st = (cudaStream_t)stream;
  const int parts = kh_layernorm_bwd_parts(rows, d);
  const int rps = (rows + parts - 1) / parts;
  if (d == 2048)
    KH_LAUNCH((layernorm_bwd_dx_reg_k<8>), cdiv(rows, 8), 256, 0, st, (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)mean,
                                                            (const float*)rstd, (const bf16*)dres, (bf16*)dx, rows);
  else if (d == 1024)
    KH_LAUNCH((layernorm_bwd_dx_reg_k<4>), cdiv(rows, 8), 256, 0, st, (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)mean,
                                                            (const float*)rstd, (const bf16*)dres, (bf16*)dx, rows);
  else
    KH_LAUNCH(layernorm_bwd_dx_k, cdiv(rows, 8), 256, 0, st, (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)mean,
                                                     (const float*)rstd, (const bf16*)dres, (bf16*)dx, rows, d);
  dim3 grid(cdiv(d, 64), parts);
  KH_LAUNCH(layernorm_bwd_dwdb_k, grid, 256, 0, st, (const bf16*)dy, (const bf16*)x, (const float*)mean, (const float*)rstd,
                                              (int*)partials, (float*)partials + KH_COUNTER_SLOTS, (float*)dw,
                                              (float*)db, rows, d, rps);
  KH_LAUNCH_CHECK("layernorm_bwd");
  return 0;
}

// ------------------------------------------------------------------ softmax cross-entropy
// One CTA per row of bf16 logits [rows, ld] (ld >= V, padding columns are ignored on read and
// zeroed on write).  Pass 1: online max / sum-exp.  Outputs, each optional:
//   rowloss[r] = lse - logit[target]            prob[r] = softmax[target]
//   logits[r, :] <- scale_r * (softmax - onehot) in place, scale_r = coef ? coef[r] : uniform
// Rows whose target is negative contribute nothing (loss 0, zero gradient).
__global__ void xent_k(bf16* __restrict__ logits, int ld, int V, const int* __restrict__ target,
                       const float* __restrict__ coef, float uniform, float* __restrict__ rowloss,
                       float* __restrict__ prob, int write_grad) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_m[32], s_s[32];
  __shared__ float s_max, s_sum;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  bf16* row = logits + (size_t)r * ld;
  const uint4* rp = reinterpret_cast<const uint4*>(row);
  float m = -INFINITY, s = 0.f;
  const int nv = V / 8;
  for (int i = tid; i < nv; i += blockDim.x) {
    uint4 v = rp[i];
    float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
    float mx = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)), fmaxf(fmaxf(c.x, c.y), fmaxf(e.x, e.y)));
    if (mx > m) { s *= __expf(m - mx); m = mx; }
    s += __expf(a.x - m) + __expf(a.y - m) + __expf(b.x - m) + __expf(b.y - m) + __expf(c.x - m) + __expf(c.y - m) +
         __expf(e.x - m) + __expf(e.y - m);
  }
  for (int i = nv * 8 + tid; i < V; i += blockDim.x) {
    float x = __bfloat162float(row[i]);
    if (x > m) { s *= __expf(m - x); m = x; }
    s += __expf(x - m);
  }
  // combine (m, s) pairs in a fixed tree
  float wm = warp_max(m);
  s *= (m == -INFINITY) ? 0.f : __expf(m - wm);
  s = warp_sum(s);
  if (lane == 0) { s_m[warp] = wm; s_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    float mm = lane < nw ? s_m[lane] : -INFINITY;
    float ss = lane < nw ? s_s[lane] : 0.f;
    float gm = warp_max(mm);
    ss *= (mm == -INFINITY) ? 0.f : __expf(mm - gm);
    ss = warp_sum(ss);
    if (lane == 0) { s_max = gm; s_sum = ss; }
  }
  __syncthreads();
  const float gmax = s_max, gsum = s_sum;
  const int t = target[r];
  if (tid == 0) {
    const bool valid = t >= 0 && t < V;
    const float xt = valid ? __bfloat162float(row[t]) : 0.f;
    if (rowloss) rowloss[r] = valid ? (logf(gsum) + gmax - xt) : 0.f;
    if (prob) prob[r] = valid ? __expf(xt - gmax) / gsum : 0.f;
  }
  if (!write_grad) return;
  __syncthreads();   // the target logit has been read
  const float sc = (t >= 0 && t < V) ? (coef ? coef[r] : uniform) : 0.f;
  const float inv = sc / gsum;
  uint4* wp = reinterpret_cast<uint4*>(row);
  const int nvl = ld / 8;
  for (int i = tid; i < nvl; i += blockDim.x) {
    uint4 v = wp[i], o;
    const uint32_t* vi = &v.x; uint32_t* oi = &o.x;
    const int c0 = i * 8;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 xv = unpack_bf16(vi[k]);
      const int c = c0 + 2 * k;
      float g0 = c < V ? __expf(xv.x - gmax) * inv - (c == t ? sc : 0.f) : 0.f;
      float g1 = c + 1 < V ? __expf(xv.y - gmax) * inv - (c + 1 == t ? sc : 0.f) : 0.f;
      oi[k] = pack_bf16(g0, g1);
    }
    wp[i] = o;
  }
}
extern "C" int kh_xent(void* logits, int ld, int V, const void* target, const void* coef, float uniform,
                       void* rowloss, void* prob, int write_grad, int rows, void* stream) {
  if (ld % 8 || ld < V) { kh_set_error("xent: ld=%d must be a multiple of 8 and >= V=%d", ld, V); return -1; }
  KH_LAUNCH(xent_k, rows, 512, 0, (cudaStream_t)stream, (bf16*)logits, ld, V, (const int*)target, (const float*)coef, uniform,
                                                  (float*)rowloss, (float*)prob, write_grad);
  KH_LAUNCH_CHECK("xent");
  return 0;
}

// ---- vocabulary-parallel cross-entropy (the head's vocabulary is split over tensor-parallel ranks)
// Stage 1, per rank: stats[r] = (max, sum exp(x - max), target logit or -inf) over this rank's
// columns [v0, v0 + V) of the vocabulary.  The ranks' triples are combined outside (tiny), then
// stage 2 overwrites the local logits with scale_r * (exp(x - gmax) / gsum - onehot).
__global__ void xent_stats_k(const bf16* __restrict__ logits, int ld, int V, const int* __restrict__ target, int v0,
                             float* __restrict__ stats) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s_m[32], s_s[32];
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
  const bf16* row = logits + (size_t)r * ld;
  const uint4* rp = reinterpret_cast<const uint4*>(row);
  float m = -INFINITY, s = 0.f;
  const int nv = V / 8;
  for (int i = tid; i < nv; i += blockDim.x) {
    uint4 v = rp[i];
    float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
    float mx = fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)), fmaxf(fmaxf(c.x, c.y), fmaxf(e.x, e.y)));
    if (mx > m) { s *= __expf(m - mx); m = mx; }
    s += __expf(a.x - m) + __expf(a.y - m) + __expf(b.x - m) + __expf(b.y - m) + __expf(c.x - m) + __expf(c.y - m) +
         __expf(e.x - m) + __expf(e.y - m);
  }
  for (int i = nv * 8 + tid; i < V; i += blockDim.x) {
    float x = __bfloat162float(row[i]);
    if (x > m) { s *= __expf(m - x); m = x; }
    s += __expf(x - m);
  }
  float wm = warp_max(m);
  s *= (m == -INFINITY) ? 0.f : __expf(m - wm);
  s = warp_sum(s);
  if (lane == 0) { s_m[warp] = wm; s_s[warp] = s; }
  __syncthreads();
  if (warp == 0) {
    float mm = lane < nw ? s_m[lane] : -INFINITY;
    float ss = lane < nw ? s_s[lane] : 0.f;
    float gm = warp_max(mm);
    ss *= (mm == -INFINITY) ? 0.f : __expf(mm - gm);
    ss = warp_sum(ss);
    if (lane == 0) {
      const int t = target[r] - v0;
      stats[3 * r] = gm;
      stats[3 * r + 1] = ss;
      stats[3 * r + 2] = (t >= 0 && t < V) ? __bfloat162float(row[t]) : -INFINITY;
    }
  }
}
__global__ void xent_grad_k(bf16* __restrict__ logits, int ld, int V, const int* __restrict__ target, int v0,
                            const float* __restrict__ gmax, const float* __restrict__ gsum,
                            const float* __restrict__ coef, float uniform) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x, tid = threadIdx.x;
  bf16* row = logits + (size_t)r * ld;
  const int tg = target[r];
  const int t = tg - v0;                       // local index of the target (may be outside this shard)
  const float sc = tg >= 0 ? (coef ? coef[r] : uniform) : 0.f;
  const float mx = gmax[r], inv = sc / gsum[r];
  uint4* wp = reinterpret_cast<uint4*>(row);
  const int nvl = (V + 7) / 8;                 // columns beyond the slice (up to the next multiple of 8) become 0
  for (int i = tid; i < nvl; i += blockDim.x) {
    uint4 v = wp[i], o;
    const uint32_t* vi = &v.x; uint32_t* oi = &o.x;
    const int c0 = i * 8;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float2 xv = unpack_bf16(vi[k]);
      const int c = c0 + 2 * k;
      float g0 = c < V ? __expf(xv.x - mx) * inv - (c == t ? sc : 0.f) : 0.f;
      float g1 = c + 1 < V ? __expf(xv.y - mx) * inv - (c + 1 == t ? sc : 0.f) : 0.f;
      oi[k] = pack_bf16(g0, g1);
    }
    wp[i] = o;
  }
}
extern "C" int kh_xent_stats(const void* logits, int ld, int V, const void* target, int v0, void* stats, int rows, void* stream) {
  if (ld % 8 || ld < V) { kh_set_error("xent_stats: ld=%d must be a multiple of 8 and >= V=%d", ld, V); return -1; }
  KH_LAUNCH(xent_stats_k, rows, 512, 0, (cudaStream_t)stream, (const bf16*)logits, ld, V, (const int*)target, v0, (float*)stats);
  KH_LAUNCH_CHECK("xent_stats");
  return 0;
}
extern "C" int kh_xent_grad(void* logits, int ld, int V, const void* target, int v0, const void* gmax, const void* gsum,
                            const void* coef, float uniform, int rows, void* stream) {
  if (ld % 8 || ld < V) { kh_set_error("xent_grad: ld=%d must be a multiple of 8 and >= V=%d", ld, V); return -1; }
  KH_LAUNCH(xent_grad_k, rows, 512, 0, (cudaStream_t)stream, (bf16*)logits, ld, V, (const int*)target, v0, (const float*)gmax,
                                                       (const float*)gsum, (const float*)coef, uniform);
  KH_LAUNCH_CHECK("xent_grad");
  return 0;
}

// out[0] (+)= scale * sum_i x[i], single CTA, fixed-order tree (loss reduction on the device)
__global__ void sum_f32_k(const float* __restrict__ x, long n, float scale, float* __restrict__ out, int accumulate) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float s[1024];
  float acc = 0.f;
  for (long i = threadIdx.x; i < n; i += blockDim.x) acc += x[i];
  s[threadIdx.x] = acc;
  __syncthreads();
  for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) s[threadIdx.x] += s[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + s[0] * scale;
}
extern "C" int kh_sum_f32(const void* x, long n, float scale, void* out, int accumulate, void* stream) {
  KH_LAUNCH(sum_f32_k, 1, 1024, 0, (cudaStream_t)stream, (const float*)x, n, scale, (float*)out, accumulate);
  KH_LAUNCH_CHECK("sum_f32");
  return 0;
}

// ---------------------------------------------------------------------------------- AdamW
// One pass over flat fp32 buffers: g' = g * grad_scale; m, v moments; decoupled weight decay
// on every element; writes the fp32 master, the bf16 compute copy (optional) and clears the
// gradient (optional) so that the next step can accumulate into it.
__global__ void adamw_k(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                        bf16* __restrict__ pb, long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                        float bc2, float grad_scale, int zero_grad) {
  pdl_wait();
  pdl_launch_dependents();
  const long i4 = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i4 >= n) return;
  if (i4 + 4 <= n) {
    float4 pp = *reinterpret_cast<float4*>(p + i4), gg = *reinterpret_cast<float4*>(g + i4);
    float4 mm = *reinterpret_cast<float4*>(m + i4), vv = *reinterpret_cast<float4*>(v + i4);
    float* pa = &pp.x; float* ga = &gg.x; float* ma = &mm.x; float* va = &vv.x;
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float gk = ga[k] * grad_scale;
      ma[k] = b1 * ma[k] + (1.f - b1) * gk;
      va[k] = b2 * va[k] + (1.f - b2) * gk * gk;
      float mh = ma[k] / bc1, vh = va[k] / bc2;
      pa[k] = pa[k] * (1.f - lr * wd) - lr * mh / (sqrtf(vh) + eps);
    }
    *reinterpret_cast<float4*>(p + i4) = pp;
    *reinterpret_cast<float4*>(m + i4) = mm;
    *reinterpret_cast<float4*>(v + i4) = vv;
    if (zero_grad) *reinterpret_cast<float4*>(g + i4) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (pb) {
      uint2 o = make_uint2(pack_bf16(pa[0], pa[1]), pack_bf16(pa[2], pa[3]));
      *reinterpret_cast<uint2*>(pb + i4) = o;
    }
  } else {
    for (long i = i4; i < n; i++) {
      float gk = g[i] * grad_scale;
      float mk = b1 * m[i] + (1.f - b1) * gk, vk = b2 * v[i] + (1.f - b2) * gk * gk;
      m[i] = mk; v[i] = vk;
      float pk = p[i] * (1.f - lr * wd) - lr * (mk / bc1) / (sqrtf(vk / bc2) + eps);
      p[i] = pk;
      if (zero_grad) g[i] = 0.f;
      if (pb) pb[i] = __float2bfloat16(pk);
    }
  }
}
extern "C" int kh_adamw(void* p, void* g, void* m, void* v, void* pb, long n, float lr, float b1, float b2, float eps,
                        float wd, float bc1, float bc2, float grad_scale, int zero_grad, void* stream) {
  if (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15 || ((uintptr_t)pb & 7)) {
    kh_set_error("adamw: buffers must be 16-byte aligned");
    return -1;
  }
  KH_LAUNCH(adamw_k, cdiv(cdiv(n, 4), 256), 256, 0, (cudaStream_t)stream, (float*)p, (float*)g, (float*)m, (float*)v, (bf16*)pb,
                                                                   n, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, zero_grad);
  KH_LAUNCH_CHECK("adamw");
  return 0;
}

// -------------------------------------------------------------------------------- utilities
__global__ void cast_f32_bf16_k(const float* __restrict__ x, bf16* __restrict__ y, long n) {
  pdl_wait();
  pdl_launch_dependents();
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= n) {
    float4 v = *reinterpret_cast<const float4*>(x + i);
    *reinterpret_cast<uint2*>(y + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  } else {
    for (long k = i; k < n; k++) y[k] = __float2bfloat16(x[k]);
  }
}
extern "C" int kh_cast_f32_bf16(const void* x, void* y, long n, void* stream) {
  KH_LAUNCH(cast_f32_bf16_k, cdiv(cdiv(n, 4), 256), 256, 0, (cudaStream_t)stream, (const float*)x, (bf16*)y, n);
  KH_LAUNCH_CHECK("cast_f32_bf16");
  return 0;
}
// c = a + b (bf16), n a multiple of 8
__global__ void add_bf16_k(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ c, long nv) {
  pdl_wait();
  pdl_launch_dependents();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nv) return;
  uint4 x = a[i], y = b[i], z;
  const uint32_t* xi = &x.x; const uint32_t* yi = &y.x; uint32_t* zi = &z.x;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    float2 p = unpack_bf16(xi[k]), q = unpack_bf16(yi[k]);
    zi[k] = pack_bf16(p.x + q.x, p.y + q.y);
  }
  c[i] = z;
}
extern "C" int kh_add_bf16(const void* a, const void* b, void* c, long n, void* stream) {
  if (n % 8) { kh_set_error("add: n must be a multiple of 8"); return -1; }
  KH_LAUNCH(add_bf16_k, cdiv(n / 8, 256), 256, 0, (cudaStream_t)stream, (const uint4*)a, (const uint4*)b, (uint4*)c, n / 8);
  KH_LAUNCH_CHECK("add_bf16");
  return 0;
}
// Writes a buffer larger than L2 so that the next timed iteration starts from DRAM.
__global__ void fill_u32_k(uint32_t* p, long n, uint32_t v) {
  pdl_wait();
  pdl_launch_dependents();
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) p[i] = v;
}
extern "C" int kh_fill_u32(void* p, long n, unsigned v, void* stream) {
  KH_LAUNCH(fill_u32_k, 1184, 256, 0, (cudaStream_t)stream, (uint32_t*)p, n, v);
  KH_LAUNCH_CHECK("fill_u32");
  return 0;
}

// ------------------------------------------------------------------------------ GRPO
// Group-relative advantages and per-token loss coefficients on the device (host versions:
// kh_grpo_advantages / kh_grpo_coef of the runtime library; reference src/core/grpo.c:7-20 and
// src/grpo_train.c:164-174, which round-trip p_cur / p_ref through the host every step).
//   adv[g, i]  = (r[g, i] - mean_g) / (std_g (population) + eps)                 one thread per group, in double
//   coef[r, t] = (adv[r] - beta (1 - p_ref / max(p_cur, 1e-8))) / N   for t0 <= t <= t1, else 0;  N = rows (t1 - t0 + 1)
__global__ void grpo_adv_k(const float* __restrict__ rew, float* __restrict__ adv, int n_groups, int group, float eps) {
  pdl_wait();
  pdl_launch_dependents();
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g >= n_groups) return;
  const float* r = rew + (size_t)g * group;
  double mean = 0.0;
  for (int i = 0; i < group; i++) mean += r[i];
  mean /= group;
  double var = 0.0;
  for (int i = 0; i < group; i++) { const double d = r[i] - mean; var += d * d; }
  const double sd = sqrt(var / group);
  for (int i = 0; i < group; i++) adv[(size_t)g * group + i] = (float)((r[i] - mean) / (sd + (double)eps));
}
__global__ void grpo_coef_k(const float* __restrict__ adv, const float* __restrict__ p_cur, const float* __restrict__ p_ref,
                            float* __restrict__ coef, int rows, int T, int t0, int t1, float beta, float inv) {
  pdl_wait();
  pdl_launch_dependents();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)rows * T) return;
  const int r = (int)(i / T), t = (int)(i % T);
  float c = 0.f;
  if (t >= t0 && t <= t1) {
    const float pc = fmaxf(p_cur[i], 1e-8f);
    c = (adv[r] - beta * (1.f - p_ref[i] / pc)) * inv;
  }
  coef[i] = c;
}
extern "C" int kh_grpo_advantages_dev(const void* rew, void* adv, int n_groups, int group, float eps, void* stream) {
  if (n_groups <= 0 || group <= 0) { kh_set_error("grpo_advantages: empty problem"); return -1; }
  KH_LAUNCH(grpo_adv_k, cdiv(n_groups, 128), 128, 0, (cudaStream_t)stream, (const float*)rew, (float*)adv, n_groups, group, eps);
  KH_LAUNCH_CHECK("grpo_advantages");
  return 0;
}
extern "C" int kh_grpo_coef_dev(const void* adv, const void* p_cur, const void* p_ref, void* coef, int rows, int T, int t0,
                                int t1, float beta, void* stream) {
  if (rows <= 0 || T <= 0) { kh_set_error("grpo_coef: empty problem"); return -1; }
  t0 = t0 < 0 ? 0 : t0;
  t1 = t1 > T - 1 ? T - 1 : t1;
  const long n_masked = (long)rows * (t1 - t0 + 1 > 0 ? t1 - t0 + 1 : 0);
  const float inv = n_masked > 0 ? 1.f / (float)n_masked : 0.f;
  KH_LAUNCH(grpo_coef_k, cdiv((long)rows * T, 256), 256, 0, (cudaStream_t)stream, (const float*)adv, (const float*)p_cur,
            (const float*)p_ref, (float*)coef, rows, T, t0, t1, beta, inv);
  KH_LAUNCH_CHECK("grpo_coef");
  return 0;
}
