// Memory-bound kernels around the GEMMs: embedding forward/backward, deterministic column
// sums (bias gradients), LayerNorm forward/backward, fused softmax-cross-entropy, fused AdamW
// with bf16 weight emission, and small utilities.  All reductions run in a fixed order (no
// floating-point atomics) so that a resumed run reproduces the original bit for bit.
//
// Reference counterparts (src/core/kernels.cu): embed_k :125, layernorm_fwd_k :145,
// ce_fwd_k/ce_bwd_k :310-353, grpo_dlogits_k :358, gather_prob_k :372, layernorm_bwd_* :380-414,
// colsum_k :511, embed_bwd_* :526-563, adamw_k :566, f2b_k :583; model_sync_bf16 gpt.c:377.
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
                            const bf16* __restrict__ wpe, bf16* __restrict__ out, int rows, int d, int T, int V) {
  const int r = blockIdx.x;
  int t = tok[r];
  t = min(max(t, 0), V - 1);
  int ps = pos ? pos[r] : r % T;
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
  embed_fwd_k<<<rows, 128, 0, (cudaStream_t)stream>>>((const int*)tok, (const int*)pos, (const bf16*)wte,
                                                      (const bf16*)wpe, (bf16*)out, rows, d, T, V);
  KH_LAUNCH_CHECK("embed_fwd");
  return 0;
}

// dwte[tok[r], :] += dx[r, :] -- the first row (lowest r) holding a token id owns the update and
// folds in the later rows carrying the same id, in row order: deterministic and O(R d).
__global__ void embed_bwd_wte_k(const int* __restrict__ tok, const bf16* __restrict__ dx, float* __restrict__ dwte,
                                int rows, int d, int V) {
  extern __shared__ int s_tok[];
  for (int i = threadIdx.x; i < rows; i += blockDim.x) s_tok[i] = tok[i];
  __syncthreads();
  const int r = blockIdx.x;
  const int t = s_tok[r];
  if (t < 0 || t >= V) return;
  for (int i = 0; i < r; i++) if (s_tok[i] == t) return;   // an earlier row owns this id (uniform)
  for (int e = threadIdx.x; e < d; e += blockDim.x) {
    float acc = __bfloat162float(dx[(size_t)r * d + e]);
    for (int i = r + 1; i < rows; i++) if (s_tok[i] == t) acc += __bfloat162float(dx[(size_t)i * d + e]);
    dwte[(size_t)t * d + e] += acc;
  }
}
// dwpe[t, :] += sum_b dx[b*T + t, :]
__global__ void embed_bwd_wpe_k(const bf16* __restrict__ dx, float* __restrict__ dwpe, int B, int T, int d) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long)T * d) return;
  float acc = 0.f;
  for (int b = 0; b < B; b++) acc += __bfloat162float(dx[(size_t)b * T * d + i]);
  dwpe[i] += acc;
}
extern "C" int kh_embed_bwd(const void* tok, const void* dx, void* dwte, void* dwpe, int B, int T, int d, int V,
                            void* stream) {
  const int rows = B * T;
  if ((size_t)rows * 4 > 200 * 1024) { kh_set_error("embed_bwd: %d rows exceed the shared-memory token table", rows); return -1; }
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(embed_bwd_wte_k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); attr = true; }
  if (dwte) embed_bwd_wte_k<<<rows, 128, rows * 4, (cudaStream_t)stream>>>((const int*)tok, (const bf16*)dx, (float*)dwte, rows, d, V);
  if (dwpe) embed_bwd_wpe_k<<<cdiv((long)T * d, 256), 256, 0, (cudaStream_t)stream>>>((const bf16*)dx, (float*)dwpe, B, T, d);
  KH_LAUNCH_CHECK("embed_bwd");
  return 0;
}

// ------------------------------------------------------------------------------ column sum
// out[j] (+)= sum_r x[r, j].  Each CTA owns 64 columns; 8 row-groups of 32 threads (bf16x2
// per thread) stride over the rows, then the 8 partials are added in a fixed order.
__global__ void colsum_k(const bf16* __restrict__ x, int ld, float* __restrict__ out, int rows, int N, int accumulate) {
  __shared__ float2 part[8][32];
  const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + lane * 2;
  float2 acc = make_float2(0.f, 0.f);
  if (col < N) {
    for (int r = g; r < rows; r += 8) {
      float2 v = unpack_bf16(*reinterpret_cast<const uint32_t*>(x + (size_t)r * ld + col));
      acc.x += v.x; acc.y += v.y;
    }
  }
  part[g][lane] = acc;
  __syncthreads();
  if (g == 0 && col < N) {
    float2 s = part[0][lane];
#pragma unroll
    for (int k = 1; k < 8; k++) { s.x += part[k][lane].x; s.y += part[k][lane].y; }
    if (accumulate) { s.x += out[col]; if (col + 1 < N) s.y += out[col + 1]; }
    out[col] = s.x;
    if (col + 1 < N) out[col + 1] = s.y;
  }
}
extern "C" int kh_colsum(const void* x, int ld, void* out, int rows, int N, int accumulate, void* stream) {
  if (N % 2 || ld % 2) { kh_set_error("colsum: N and ld must be even"); return -1; }
  colsum_k<<<cdiv(N, 64), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, ld, (float*)out, rows, N, accumulate);
  KH_LAUNCH_CHECK("colsum");
  return 0;
}

// ------------------------------------------------------------------------------ LayerNorm
// One warp per row; statistics in fp32 with a two-pass variance (eps 1e-5, biased variance).
__global__ void layernorm_fwd_k(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                                bf16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows,
                                int d) {
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
extern "C" int kh_layernorm_fwd(const void* x, const void* w, const void* b, void* y, void* mean, void* rstd, int rows,
                                int d, void* stream) {
  if (d % 8) { kh_set_error("layernorm: d must be a multiple of 8"); return -1; }
  layernorm_fwd_k<<<cdiv(rows, 8), 256, 0, (cudaStream_t)stream>>>((const bf16*)x, (const bf16*)w, (const bf16*)b,
                                                                    (bf16*)y, (float*)mean, (float*)rstd, rows, d);
  KH_LAUNCH_CHECK("layernorm_fwd");
  return 0;
}

// Backward.  dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w, optionally
// + dres (the residual-stream gradient that bypasses the norm).  Each CTA covers a contiguous
// band of rows and writes its partial dw/db column sums to `partials` ([grid, 2, d] fp32, a
// scratch buffer supplied by the caller); layernorm_bwd_reduce_k then adds the bands in
// index order into the fp32 gradient buffers.
#define LN_BWD_WARPS 8
__global__ void layernorm_bwd_k(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                const float* __restrict__ mean, const float* __restrict__ rstd,
                                const bf16* __restrict__ dres, bf16* __restrict__ dx, float* __restrict__ partials,
                                int rows, int d, int rows_per_cta) {
  extern __shared__ float s_acc[];   // [LN_BWD_WARPS][2][d]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* my_dw = s_acc + (size_t)warp * 2 * d;
  float* my_db = my_dw + d;
  for (int j = lane; j < d; j += 32) { my_dw[j] = 0.f; my_db[j] = 0.f; }
  const int r0 = blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  for (int row = r0 + warp; row < r1; row += LN_BWD_WARPS) {
    const bf16* dyr = dy + (size_t)row * d;
    const bf16* xr = x + (size_t)row * d;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int j = lane * 2; j < d; j += 64) {
      float2 g = unpack_bf16(*reinterpret_cast<const uint32_t*>(dyr + j));
      float2 xv = unpack_bf16(*reinterpret_cast<const uint32_t*>(xr + j));
      float2 ww = unpack_bf16(*reinterpret_cast<const uint32_t*>(w + j));
      float xh0 = (xv.x - mu) * rs, xh1 = (xv.y - mu) * rs;
      float g0 = g.x * ww.x, g1 = g.y * ww.y;
      s1 += g0 + g1;
      s2 += g0 * xh0 + g1 * xh1;
      my_dw[j] += g.x * xh0; my_dw[j + 1] += g.y * xh1;
      my_db[j] += g.x; my_db[j + 1] += g.y;
    }
    s1 = warp_sum(s1) / d;
    s2 = warp_sum(s2) / d;
    for (int j = lane * 2; j < d; j += 64) {
      float2 g = unpack_bf16(*reinterpret_cast<const uint32_t*>(dyr + j));
      float2 xv = unpack_bf16(*reinterpret_cast<const uint32_t*>(xr + j));
      float2 ww = unpack_bf16(*reinterpret_cast<const uint32_t*>(w + j));
      float xh0 = (xv.x - mu) * rs, xh1 = (xv.y - mu) * rs;
      float o0 = rs * (g.x * ww.x - s1 - xh0 * s2), o1 = rs * (g.y * ww.y - s1 - xh1 * s2);
      if (dres) {
        float2 rr = unpack_bf16(*reinterpret_cast<const uint32_t*>(dres + (size_t)row * d + j));
        o0 += rr.x; o1 += rr.y;
      }
      *reinterpret_cast<uint32_t*>(dx + (size_t)row * d + j) = pack_bf16(o0, o1);
    }
  }
  __syncthreads();
  float* out = partials + (size_t)blockIdx.x * 2 * d;
  for (int j = threadIdx.x; j < 2 * d; j += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < LN_BWD_WARPS; k++) s += s_acc[(size_t)k * 2 * d + j];
    out[j] = s;
  }
}
__global__ void layernorm_bwd_reduce_k(const float* __restrict__ partials, float* __restrict__ dw,
                                       float* __restrict__ db, int nparts, int d) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= 2 * d) return;
  float s = 0.f;
  for (int k = 0; k < nparts; k++) s += partials[(size_t)k * 2 * d + j];
  if (j < d) dw[j] += s;
  else db[j - d] += s;
}
// Number of row bands (= rows of `partials`) layernorm_bwd uses for a problem size.
extern "C" int kh_layernorm_bwd_parts(int rows, int d) {
  int parts = 296;
  if (rows < parts * 8) parts = (rows + 7) / 8;
  return parts < 1 ? 1 : parts;
}
extern "C" int kh_layernorm_bwd(const void* dy, const void* x, const void* w, const void* mean, const void* rstd,
                                const void* dres, void* dx, void* dw, void* db, void* partials, int rows, int d,
                                void* stream) {
  if (d % 2) { kh_set_error("layernorm_bwd: d must be even"); return -1; }
  const size_t smem = (size_t)LN_BWD_WARPS * 2 * d * sizeof(float);
  if (smem > 220 * 1024) { kh_set_error("layernorm_bwd: d=%d needs %zu bytes of shared memory", d, smem); return -1; }
  static size_t attr = 0;
  if (smem > attr) { cudaFuncSetAttribute(layernorm_bwd_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr = smem; }
  const int parts = kh_layernorm_bwd_parts(rows, d);
  const int rpc = (rows + parts - 1) / parts;
  layernorm_bwd_k<<<parts, LN_BWD_WARPS * 32, smem, (cudaStream_t)stream>>>(
      (const bf16*)dy, (const bf16*)x, (const bf16*)w, (const float*)mean, (const float*)rstd, (const bf16*)dres,
      (bf16*)dx, (float*)partials, rows, d, rpc);
  layernorm_bwd_reduce_k<<<cdiv(2 * d, 128), 128, 0, (cudaStream_t)stream>>>((const float*)partials, (float*)dw,
                                                                             (float*)db, parts, d);
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
  xent_k<<<rows, 512, 0, (cudaStream_t)stream>>>((bf16*)logits, ld, V, (const int*)target, (const float*)coef, uniform,
                                                  (float*)rowloss, (float*)prob, write_grad);
  KH_LAUNCH_CHECK("xent");
  return 0;
}

// out[0] (+)= scale * sum_i x[i], single CTA, fixed-order tree (loss reduction on the device)
__global__ void sum_f32_k(const float* __restrict__ x, long n, float scale, float* __restrict__ out, int accumulate) {
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
  sum_f32_k<<<1, 1024, 0, (cudaStream_t)stream>>>((const float*)x, n, scale, (float*)out, accumulate);
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
  adamw_k<<<cdiv(cdiv(n, 4), 256), 256, 0, (cudaStream_t)stream>>>((float*)p, (float*)g, (float*)m, (float*)v, (bf16*)pb,
                                                                   n, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, zero_grad);
  KH_LAUNCH_CHECK("adamw");
  return 0;
}

// -------------------------------------------------------------------------------- utilities
__global__ void cast_f32_bf16_k(const float* __restrict__ x, bf16* __restrict__ y, long n) {
  const long i = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 4 <= n) {
    float4 v = *reinterpret_cast<const float4*>(x + i);
    *reinterpret_cast<uint2*>(y + i) = make_uint2(pack_bf16(v.x, v.y), pack_bf16(v.z, v.w));
  } else {
    for (long k = i; k < n; k++) y[k] = __float2bfloat16(x[k]);
  }
}
extern "C" int kh_cast_f32_bf16(const void* x, void* y, long n, void* stream) {
  cast_f32_bf16_k<<<cdiv(cdiv(n, 4), 256), 256, 0, (cudaStream_t)stream>>>((const float*)x, (bf16*)y, n);
  KH_LAUNCH_CHECK("cast_f32_bf16");
  return 0;
}
// c = a + b (bf16), n a multiple of 8
__global__ void add_bf16_k(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ c, long nv) {
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
  add_bf16_k<<<cdiv(n / 8, 256), 256, 0, (cudaStream_t)stream>>>((const uint4*)a, (const uint4*)b, (uint4*)c, n / 8);
  KH_LAUNCH_CHECK("add_bf16");
  return 0;
}
// Writes a buffer larger than L2 so that the next timed iteration starts from DRAM.
__global__ void fill_u32_k(uint32_t* p, long n, uint32_t v) {
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) p[i] = v;
}
extern "C" int kh_fill_u32(void* p, long n, unsigned v, void* stream) {
  fill_u32_k<<<1184, 256, 0, (cudaStream_t)stream>>>((uint32_t*)p, n, v);
  KH_LAUNCH_CHECK("fill_u32");
  return 0;
}
