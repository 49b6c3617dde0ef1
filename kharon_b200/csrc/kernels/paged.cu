// Paged-KV inference kernels: KV append, paged attention over block tables, last-row gather,
// KV block copy (copy-on-write) and the on-device sampler.
//
// KV pool of one layer: k, v : [n_blocks, block_size, H, hd] bf16 (reference src/core/infer.c:20-21
// keeps [n_layer, n_blocks, bs, H, hd]; here the layer is the outermost index of the same
// allocation, the caller passes the layer's base pointer).  A step carries a flat token list
// (pos[i], slot[i]) and a dense block table [n_seq, max_lb] exactly as infer.c:229-249.
//
// Replaces src/kernels/paged.cu: append_kv_k :33-46, paged_attn_k :50-77 (one key per block-wide
// tree reduction), gather_rows_k :80-86, and the host sampler infer.c:197-213.
#include "common.cuh"

#define KH_LAUNCH_CHECK(name)                                                     \
  do {                                                                            \
    cudaError_t e_ = cudaGetLastError();                                          \
    if (e_ != cudaSuccess) { kh_set_error(name ": %s", cudaGetErrorString(e_)); return -1; } \
  } while (0)

static inline int cdiv(long a, long b) { return (int)((a + b - 1) / b); }

// ------------------------------------------------------------------------------- append
// One thread per 8 elements: copies k and v of every new token into its block slot.
__global__ void append_kv_k(const bf16* __restrict__ qkv, int ld, bf16* __restrict__ kc, bf16* __restrict__ vc,
                            const int* __restrict__ pos, const int* __restrict__ slot, const int* __restrict__ btab,
                            int max_lb, int bs, int d, int ntok, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int per = d / 8;
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)ntok * per) return;
  const int t = (int)(i / per), c = (int)(i % per) * 8;
  const int p = pos[t];
  // index guard: a position beyond the block table is recorded (status code 8) and its store skipped
  if (p < 0 || p / bs >= max_lb || slot[t] < 0) { atomicCAS(err, 0, 8); return; }
  const int blk = btab[(size_t)slot[t] * max_lb + p / bs];
  const size_t dst = ((size_t)blk * bs + (p % bs)) * d + c;
  const bf16* src = qkv + (size_t)t * ld;
  *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(src + d + c);
  *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(src + 2 * d + c);
}
extern "C" int kh_append_kv(const void* qkv, int ld, void* kc, void* vc, const void* pos, const void* slot,
                            const void* btab, int max_lb, int bs, int H, int hd, int ntok, void* stream) {
  const int d = H * hd;
  if (d % 8) { kh_set_error("append_kv: H*hd must be a multiple of 8"); return -1; }
  KH_LAUNCH(append_kv_k, cdiv((long)ntok * d / 8, 256), 256, 0, (cudaStream_t)stream, 
      (const bf16*)qkv, ld, (bf16*)kc, (bf16*)vc, (const int*)pos, (const int*)slot, (const int*)btab, max_lb, bs, d, ntok,
      kh_error_word_dev());
  KH_LAUNCH_CHECK("append_kv");
  return 0;
}

// ------------------------------------------------------------------------------- attention
// CTA = (token, head), 128 threads.  Phase 1: thread j scores keys j, j+128, ... (whole dot
// product in registers, 16-byte K loads, q broadcast from shared memory).  Phase 2: block
// max / sum.  Phase 3: HD/8 threads share one value row (16-byte loads), 128/(HD/8) rows are in
// flight per iteration, and the row groups are combined in shared memory in a fixed order.
// Context = positions 0..pos of the token's own sequence.  With `append` != 0 (decode steps: one
// new token per sequence) the CTA first copies its token's k and v for this head from the qkv row
// into the cache, which replaces the separate append launch; otherwise the new tokens' K/V must
// already be in the cache (prefill: several tokens of one sequence attend to each other).
template <int HD>
__global__ void __launch_bounds__(128)
paged_attn_k(const bf16* __restrict__ qkv, int ld, bf16* __restrict__ kc, bf16* __restrict__ vc,
             bf16* __restrict__ out, const int* __restrict__ pos, const int* __restrict__ slot,
             const int* __restrict__ btab, int max_lb, int bs, int H, float scale, int max_ctx, int append, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  // index guard: a context longer than the score buffer or the block table is recorded (status code 8)
  // and the token skipped (uniform over the CTA)
  if (pos[blockIdx.x] < 0 || pos[blockIdx.x] >= max_ctx || pos[blockIdx.x] / bs >= max_lb || slot[blockIdx.x] < 0) {
    if (threadIdx.x == 0) atomicCAS(err, 0, 8);
    return;
  }
  extern __shared__ float sm[];
  constexpr int TPR = HD / 8;               // threads per value row
  constexpr int GROUPS = 128 / TPR;         // value rows in flight
  float* s_q = sm;                // HD
  float* s_p = sm + HD;           // max_ctx scores / probabilities
  float* s_red = s_p + max_ctx;   // GROUPS * HD partial outputs (>= 128 floats of reduction scratch)
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int d = H * HD;
  const int ctx = pos[t] + 1;
  const int* bt = btab + (size_t)slot[t] * max_lb;
  for (int e = tid; e < HD; e += 128) s_q[e] = __bfloat162float(qkv[(size_t)t * ld + h * HD + e]) * scale;
  if (append && tid < 2 * TPR) {
    const int p = ctx - 1, which = tid / TPR, c = (tid % TPR) * 8;
    const size_t dst = ((size_t)bt[p / bs] * bs + (p % bs)) * d + h * HD + c;
    const uint4 v = *reinterpret_cast<const uint4*>(qkv + (size_t)t * ld + (which + 1) * d + h * HD + c);
    *reinterpret_cast<uint4*>((which ? vc : kc) + dst) = v;
  }
  __syncthreads();
  float lmax = -INFINITY;
  for (int j = tid; j < ctx; j += 128) {
    const bf16* kp = kc + ((size_t)bt[j / bs] * bs + (j % bs)) * d + h * HD;
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < HD; c += 8) {
      uint4 v = *reinterpret_cast<const uint4*>(kp + c);
      float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
      acc += a.x * s_q[c] + a.y * s_q[c + 1] + b.x * s_q[c + 2] + b.y * s_q[c + 3] + cc.x * s_q[c + 4] +
             cc.y * s_q[c + 5] + e.x * s_q[c + 6] + e.y * s_q[c + 7];
    }
    s_p[j] = acc;
    lmax = fmaxf(lmax, acc);
  }
  // block max
  s_red[tid] = lmax;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] = fmaxf(s_red[tid], s_red[tid + o]);
    __syncthreads();
  }
  const float gmax = s_red[0];
  __syncthreads();
  float lsum = 0.f;
  for (int j = tid; j < ctx; j += 128) {
    float p = __expf(s_p[j] - gmax);
    s_p[j] = p;
    lsum += p;
  }
  s_red[tid] = lsum;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] += s_red[tid + o];
    __syncthreads();
  }
  const float inv = 1.f / s_red[0];
  __syncthreads();
  // phase 3
  const int c8 = (tid % TPR) * 8, grp = tid / TPR;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; k++) acc[k] = 0.f;
  for (int j = grp; j < ctx; j += GROUPS) {
    const uint4 v = *reinterpret_cast<const uint4*>(vc + ((size_t)bt[j / bs] * bs + (j % bs)) * d + h * HD + c8);
    const float p = s_p[j];
    float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
    acc[0] += p * a.x; acc[1] += p * a.y; acc[2] += p * b.x; acc[3] += p * b.y;
    acc[4] += p * cc.x; acc[5] += p * cc.y; acc[6] += p * e.x; acc[7] += p * e.y;
  }
#pragma unroll
  for (int k = 0; k < 8; k++) s_red[grp * HD + c8 + k] = acc[k];
  __syncthreads();
  if (tid < HD) {
    float o = 0.f;
    for (int g = 0; g < GROUPS; g++) o += s_red[g * HD + tid];
    out[(size_t)t * d + h * HD + tid] = __float2bfloat16(o * inv);
  }
}
extern "C" int kh_paged_attn(const void* qkv, int ld, void* kc, void* vc, void* out, const void* pos,
                             const void* slot, const void* btab, int max_lb, int bs, int H, int hd, float scale,
                             int ntok, int max_ctx, int append, void* stream) {
  const size_t smem = (size_t)(hd + max_ctx + 1024 + 8) * sizeof(float);
  if (smem > 200 * 1024) { kh_set_error("paged_attn: context %d does not fit in shared memory", max_ctx); return -1; }
  dim3 grid(ntok, H);
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(HD)                                                                                                   \
  {                                                                                                                  \
    static size_t attr = 48 * 1024;                                                                                  \
    if (smem > attr) { cudaFuncSetAttribute(paged_attn_k<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = smem; } \
    KH_LAUNCH((paged_attn_k<HD>), grid, 128, smem, st, (const bf16*)qkv, ld, (bf16*)kc, (bf16*)vc, (bf16*)out,                 \
                                              (const int*)pos, (const int*)slot, (const int*)btab, max_lb, bs, H,    \
                                              scale, max_ctx, append, kh_error_word_dev());                          \
  }
  if (hd == 128) LAUNCH(128)
  else if (hd == 64) LAUNCH(64)
  else if (hd == 32) LAUNCH(32)
  else if (hd == 16) LAUNCH(16)
  else { kh_set_error("paged_attn: head dim %d is not supported", hd); return -1; }
#undef LAUNCH
  KH_LAUNCH_CHECK("paged_attn");
  return 0;
}

// ------------------------------------------------------------------------------- split-KV attention
// Long contexts: the keys of a token are cut into `n_split` equal ranges, one CTA per (token, head,
// range) computes the softmax-weighted value sum over its range and its log-sum-exp, and a merge
// kernel combines the ranges (weights exp(lse_s - max lse)).  More CTAs per token than heads when a
// decode step has few sequences, and a score buffer of one range instead of the whole context.
// The range that holds position `pos` appends the token's k, v first (decode steps).
template <int HD>
__global__ void __launch_bounds__(128)
paged_attn_split_k(const bf16* __restrict__ qkv, int ld, bf16* __restrict__ kc, bf16* __restrict__ vc,
                   float* __restrict__ o_part, float* __restrict__ lse_part, const int* __restrict__ pos,
                   const int* __restrict__ slot, const int* __restrict__ btab, int max_lb, int bs, int H, float scale,
                   int max_ctx, int chunk, int append, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, sp = blockIdx.z, n_split = gridDim.z, tid = threadIdx.x;
  float* op = o_part + (((size_t)t * H + h) * n_split + sp) * HD;
  float* lp = lse_part + ((size_t)t * H + h) * n_split + sp;
  if (pos[t] < 0 || pos[t] >= max_ctx || pos[t] / bs >= max_lb || slot[t] < 0) {
    if (tid == 0) { atomicCAS(err, 0, 8); *lp = -INFINITY; }
    for (int e = tid; e < HD; e += 128) op[e] = 0.f;
    return;
  }
  extern __shared__ float sm[];
  constexpr int TPR = HD / 8, GROUPS = 128 / TPR;
  float* s_q = sm;
  float* s_p = sm + HD;              // `chunk` scores
  float* s_red = s_p + chunk;
  const int d = H * HD;
  const int ctx = pos[t] + 1;
  const int j0 = sp * chunk, j1 = min(ctx, j0 + chunk);
  const int* bt = btab + (size_t)slot[t] * max_lb;
  if (append && tid < 2 * TPR && ctx - 1 >= j0 && ctx - 1 < j1) {
    const int p = ctx - 1, which = tid / TPR, c = (tid % TPR) * 8;
    const size_t dst = ((size_t)bt[p / bs] * bs + (p % bs)) * d + h * HD + c;
    *reinterpret_cast<uint4*>((which ? vc : kc) + dst) =
        *reinterpret_cast<const uint4*>(qkv + (size_t)t * ld + (which + 1) * d + h * HD + c);
  }
  if (j1 <= j0) {                    // no keys in this range
    if (tid == 0) *lp = -INFINITY;
    for (int e = tid; e < HD; e += 128) op[e] = 0.f;
    return;
  }
  for (int e = tid; e < HD; e += 128) s_q[e] = __bfloat162float(qkv[(size_t)t * ld + h * HD + e]) * scale;
  __syncthreads();
  float lmax = -INFINITY;
  for (int j = j0 + tid; j < j1; j += 128) {
    const bf16* kp = kc + ((size_t)bt[j / bs] * bs + (j % bs)) * d + h * HD;
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < HD; c += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(kp + c);
      const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), e = unpack_bf16(v.w);
      acc += a.x * s_q[c] + a.y * s_q[c + 1] + b.x * s_q[c + 2] + b.y * s_q[c + 3] + cc.x * s_q[c + 4] +
             cc.y * s_q[c + 5] + e.x * s_q[c + 6] + e.y * s_q[c + 7];
    }
    s_p[j - j0] = acc;
    lmax = fmaxf(lmax, acc);
  }
  s_red[tid] = lmax;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] = fmaxf(s_red[tid], s_red[tid + o]);
    __syncthreads();
  }
  const float gmax = s_red[0];
  __syncthreads();
  float lsum = 0.f;
  for (int j = j0 + tid; j < j1; j += 128) {
    const float e = __expf(s_p[j - j0] - gmax);
    s_p[j - j0] = e;
    lsum += e;
  }
  s_red[tid] = lsum;
  __syncthreads();
  for (int o = 64; o > 0; o >>= 1) {
    if (tid < o) s_red[tid] += s_red[tid + o];
    __syncthreads();
  }
  const float tot = s_red[0];
  __syncthreads();
  const int c8 = (tid % TPR) * 8, grp = tid / TPR;
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; k++) acc[k] = 0.f;
  for (int j = j0 + grp; j < j1; j += GROUPS) {
    const uint4 v = *reinterpret_cast<const uint4*>(vc + ((size_t)bt[j / bs] * bs + (j % bs)) * d + h * HD + c8);
    const float pj = s_p[j - j0];
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
    op[tid] = o / tot;
  }
  if (tid == 0) *lp = gmax + logf(tot);
}
// out[t, h, :] = sum_s w_s o_part[t, h, s, :] / sum_s w_s with w_s = exp(lse_s - max_s lse_s), ranges in index order
__global__ void paged_attn_merge_k(const float* __restrict__ o_part, const float* __restrict__ lse_part, bf16* __restrict__ out,
                                   int H, int HD, int n_split) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y, e = threadIdx.x;
  const float* lp = lse_part + ((size_t)t * H + h) * n_split;
  float m = -INFINITY;
  for (int s = 0; s < n_split; s++) m = fmaxf(m, lp[s]);
  float num = 0.f, den = 0.f;
  if (m > -INFINITY)
    for (int s = 0; s < n_split; s++) {
      const float w = lp[s] == -INFINITY ? 0.f : __expf(lp[s] - m);
      num += w * o_part[(((size_t)t * H + h) * n_split + s) * HD + e];
      den += w;
    }
  out[((size_t)t * H + h) * HD + e] = __float2bfloat16(den > 0.f ? num / den : 0.f);
}
// `o_part`: ntok * H * n_split * hd floats, `lse_part`: ntok * H * n_split floats (scratch).
extern "C" int kh_paged_attn_split(const void* qkv, int ld, void* kc, void* vc, void* out, void* o_part, void* lse_part,
                                   const void* pos, const void* slot, const void* btab, int max_lb, int bs, int H, int hd,
                                   float scale, int ntok, int max_ctx, int n_split, int append, void* stream) {
  if (n_split < 1 || n_split > 64) { kh_set_error("paged_attn_split: n_split %d out of range", n_split); return -1; }
  const int chunk = (max_ctx + n_split - 1) / n_split;
  const size_t smem = (size_t)(hd + chunk + 1024 + 8) * sizeof(float);
  if (smem > 200 * 1024) { kh_set_error("paged_attn_split: a range of %d positions does not fit in shared memory", chunk); return -1; }
  dim3 grid(ntok, H, n_split);
  cudaStream_t st = (cudaStream_t)stream;
#define LAUNCH(HD)                                                                                                        \
  {                                                                                                                       \
    static size_t attr = 48 * 1024;                                                                                       \
    if (smem > attr) { cudaFuncSetAttribute(paged_attn_split_k<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = smem; } \
    KH_LAUNCH((paged_attn_split_k<HD>), grid, 128, smem, st, (const bf16*)qkv, ld, (bf16*)kc, (bf16*)vc, (float*)o_part,  \
              (float*)lse_part, (const int*)pos, (const int*)slot, (const int*)btab, max_lb, bs, H, scale, max_ctx, chunk, \
              append, kh_error_word_dev());                                                                               \
  }
  if (hd == 128) LAUNCH(128)
  else if (hd == 64) LAUNCH(64)
  else if (hd == 32) LAUNCH(32)
  else if (hd == 16) LAUNCH(16)
  else { kh_set_error("paged_attn_split: head dim %d is not supported", hd); return -1; }
#undef LAUNCH
  KH_LAUNCH_CHECK("paged_attn_split");
  KH_LAUNCH(paged_attn_merge_k, dim3(ntok, H), hd, 0, st, (const float*)o_part, (const float*)lse_part, (bf16*)out, H, hd, n_split);
  KH_LAUNCH_CHECK("paged_attn_merge");
  return 0;
}

// ------------------------------------------------------------------------------- gather / copy
__global__ void gather_rows_k(const bf16* __restrict__ x, const int* __restrict__ rows, bf16* __restrict__ out, int d) {
  pdl_wait();
  pdl_launch_dependents();
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)rows[blockIdx.x] * d);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * d);
  for (int i = threadIdx.x; i < d / 8; i += blockDim.x) dst[i] = src[i];
}
extern "C" int kh_gather_rows(const void* x, const void* rows, void* out, int nseq, int d, void* stream) {
  if (d % 8) { kh_set_error("gather_rows: d must be a multiple of 8"); return -1; }
  KH_LAUNCH(gather_rows_k, nseq, 128, 0, (cudaStream_t)stream, (const bf16*)x, (const int*)rows, (bf16*)out, d);
  KH_LAUNCH_CHECK("gather_rows");
  return 0;
}
// Copies whole KV blocks (src -> dst pairs) in every layer: the device half of copy-on-write.
__global__ void copy_blocks_k(bf16* __restrict__ kc, bf16* __restrict__ vc, const int* __restrict__ pairs,
                              size_t block_elems, size_t layer_elems) {
  pdl_wait();
  pdl_launch_dependents();
  const int pr = blockIdx.x, layer = blockIdx.y;
  const size_t src = (size_t)layer * layer_elems + (size_t)pairs[2 * pr] * block_elems;
  const size_t dst = (size_t)layer * layer_elems + (size_t)pairs[2 * pr + 1] * block_elems;
  for (size_t i = threadIdx.x * 8; i < block_elems; i += blockDim.x * 8) {
    *reinterpret_cast<uint4*>(kc + dst + i) = *reinterpret_cast<const uint4*>(kc + src + i);
    *reinterpret_cast<uint4*>(vc + dst + i) = *reinterpret_cast<const uint4*>(vc + src + i);
  }
}
extern "C" int kh_copy_blocks(void* kc, void* vc, const void* pairs, int npairs, int n_layer, long block_elems,
                              long layer_elems, void* stream) {
  if (npairs <= 0) return 0;
  if (block_elems % 8) { kh_set_error("copy_blocks: block size must be a multiple of 8 elements"); return -1; }
  dim3 grid(npairs, n_layer);
  KH_LAUNCH(copy_blocks_k, grid, 128, 0, (cudaStream_t)stream, (bf16*)kc, (bf16*)vc, (const int*)pairs, (size_t)block_elems,
                                                        (size_t)layer_elems);
  KH_LAUNCH_CHECK("copy_blocks");
  return 0;
}

// ------------------------------------------------------------------------------- sampler
// One CTA per sequence.  temperature <= 0: argmax (lowest index wins ties).  Otherwise a draw
// from softmax(logits / temperature): each thread owns a contiguous chunk, chunk sums are
// scanned in order, the draw u * total picks the chunk and then the element -- deterministic
// for a given (seed, step, row).  `rep` > 1 draws `rep` independent tokens from the same row
// (first token of a forked group).
__device__ __forceinline__ uint32_t mix32(uint64_t x) {
  x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
  return (uint32_t)(x >> 16);
}
__global__ void __launch_bounds__(256)
sample_k(const bf16* __restrict__ logits, int ld, int V, float temperature, unsigned long long seed, int step,
         const int* __restrict__ step_dev, int rep, int* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  if (step_dev) {      // step number and seed kept in device memory: a captured launch draws fresh numbers
    step = step_dev[0];
    seed = (unsigned long long)(unsigned)step_dev[1] | ((unsigned long long)(unsigned)step_dev[2] << 32);
  }
  __shared__ float s_v[256];
  __shared__ int s_i[256];
  __shared__ float s_scan[257];
  const int row = blockIdx.x, tid = threadIdx.x;
  const bf16* lg = logits + (size_t)row * ld;
  const int chunk = (V + 255) / 256;
  const int c0 = tid * chunk, c1 = min(V, c0 + chunk);
  float best = -INFINITY;
  int bi = V;
  for (int i = c0; i < c1; i++) {
    float x = __bfloat162float(lg[i]);
    if (x > best) { best = x; bi = i; }
  }
  s_v[tid] = best; s_i[tid] = bi;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) {
      float a = s_v[tid], b = s_v[tid + o];
      int ia = s_i[tid], ib = s_i[tid + o];
      if (b > a || (b == a && ib < ia)) { s_v[tid] = b; s_i[tid] = ib; }
    }
    __syncthreads();
  }
  const float gmax = s_v[0];
  const int gidx = s_i[0];
  if (temperature <= 0.f) {
    if (tid < rep) out[row * rep + tid] = gidx;
    return;
  }
  const float it = 1.f / temperature;
  float sum = 0.f;
  for (int i = c0; i < c1; i++) sum += __expf((__bfloat162float(lg[i]) - gmax) * it);
  __syncthreads();
  s_scan[tid + 1] = sum;
  if (tid == 0) s_scan[0] = 0.f;
  __syncthreads();
  if (tid == 0) for (int k = 1; k <= 256; k++) s_scan[k] += s_scan[k - 1];   // ordered, 256 adds
  __syncthreads();
  const float total = s_scan[256];
  for (int r = 0; r < rep; r++) {
    const uint32_t rnd = mix32(seed * 0x9E3779B97F4A7C15ULL + (uint64_t)step * 1000003ULL + (uint64_t)(row * rep + r) * 7919ULL);
    const float u = ((rnd >> 8) + 0.5f) * (1.f / 16777216.f) * total;
    if (u >= s_scan[tid] && (u < s_scan[tid + 1] || (tid == 255))) {
      float acc = s_scan[tid];
      int pick = max(c0, min(c1, V) - 1);
      for (int i = c0; i < c1; i++) {
        acc += __expf((__bfloat162float(lg[i]) - gmax) * it);
        if (u < acc) { pick = i; break; }
      }
      if (c0 >= V) pick = gidx;
      out[row * rep + r] = pick;
    }
  }
}
// `step_dev` (optional): three device words {step number, seed low, seed high}; when given they replace
// `step` and `seed`, so that the launch can be replayed from a CUDA graph with new values each time.
extern "C" int kh_sample2(const void* logits, int ld, int V, float temperature, unsigned long long seed, int step,
                          const void* step_dev, int rep, void* out, int nseq, void* stream) {
  if (rep < 1 || rep > 256) { kh_set_error("sample: rep must be in [1, 256]"); return -1; }
  KH_LAUNCH(sample_k, nseq, 256, 0, (cudaStream_t)stream, (const bf16*)logits, ld, V, temperature, seed, step,
            (const int*)step_dev, rep, (int*)out);
  KH_LAUNCH_CHECK("sample");
  return 0;
}
extern "C" int kh_sample(const void* logits, int ld, int V, float temperature, unsigned long long seed, int step,
                         int rep, void* out, int nseq, void* stream) {
  return kh_sample2(logits, ld, V, temperature, seed, step, nullptr, rep, out, nseq, stream);
}
