// Host runtime: RNG and initialisation streams, arena layout, data loader, CKP1 / CHRN file
// IO, GRPO host math, 1F1B schedule generation and the paged-KV block pool + continuous
// batching scheduler.  See kharon_rt.h for the ABI.
//
// Behavioural parity notes (paths inside the reference project):
//   RNG / synthetic batches      src/core/rng.h:7-22
//   Box-Muller init stream       src/core/gpt.c:228-264, block-sliced variant gpt.c:271-283
//   256-byte bump layout         src/core/arena.c:6,22-29 and src/core/gpt.c:18-42
//   byte data loader             src/core/data.c:6-30
//   checkpoint file              src/core/ckpt.c:25-68
//   fixture file                 src/core/refio.c:5-72
//   GRPO advantages / coef       src/core/grpo.c:7-20, src/grpo_train.c:164-174
//   1F1B order                   src/pp_train.c:24-53
//   engine scheduling            src/core/infer.c:72-106,229-313,315-387
#include "kharon_rt.h"

#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

namespace {
thread_local std::string g_err;
int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}
struct File {
  FILE* f = nullptr;
  File(const char* path, const char* mode) { f = fopen(path, mode); }
  ~File() { if (f) fclose(f); }
  bool rd(void* p, size_t n) { return fread(p, 1, n, f) == n; }
  bool wr(const void* p, size_t n) { return fwrite(p, 1, n, f) == n; }
};
}  // namespace

extern "C" const char* kh_last_error(void) { return g_err.c_str(); }

// ------------------------------------------------------------------------------------ RNG
extern "C" void kh_rng_seed(uint64_t* s, uint64_t seed) {
  *s = seed ? seed : 0x9E3779B97F4A7C15ULL;
}
extern "C" uint32_t kh_rng_u32(uint64_t* s) {
  uint64_t x = *s;
  x ^= x >> 12;
  x ^= x << 25;
  x ^= x >> 27;
  *s = x;
  return (uint32_t)((x * 0x2545F4914F6CDD1DULL) >> 32);
}
extern "C" void kh_rng_batch(uint64_t* s, int32_t* idx, int32_t* tgt, int64_t n, int32_t vocab) {
  for (int64_t i = 0; i < n; i++) idx[i] = (int32_t)(kh_rng_u32(s) % (uint32_t)vocab);
  for (int64_t i = 0; i < n; i++) tgt[i] = (int32_t)(kh_rng_u32(s) % (uint32_t)vocab);
}
static inline float normal1(uint64_t* s) {
  float u1 = (kh_rng_u32(s) + 1.f) / 4294967296.f;
  float u2 = (float)kh_rng_u32(s) / 4294967296.f;
  return sqrtf(-2.f * logf(u1)) * cosf(6.2831853f * u2);
}
extern "C" void kh_fill_normal(uint64_t* s, float* dst, int64_t n, float std) {
  for (int64_t i = 0; i < n; i++) dst[i] = std * normal1(s);
}
extern "C" void kh_fill_normal_block(uint64_t* s, float* dst, int64_t rows, int64_t cols,
                                     int64_t r0, int64_t r1, int64_t c0, int64_t c1, float std) {
  int64_t w = c1 - c0;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t c = 0; c < cols; c++) {
      float v = std * normal1(s);
      if (dst && r >= r0 && r < r1 && c >= c0 && c < c1) dst[(r - r0) * w + (c - c0)] = v;
    }
}

// --------------------------------------------------------------------------------- layout
extern "C" int kh_layout_params(const int32_t cfg[6], int32_t tp, int32_t has_head,
                                int32_t es, int64_t* offsets, int64_t* numels,
                                int32_t max_entries, int64_t* total_bytes) {
  const int64_t L = cfg[0], d = cfg[1], H = cfg[2], V = cfg[3], S = cfg[4];
  if (tp < 1 || d % tp || H % tp || (es != 2 && es != 4))
    return fail(KH_E_ARG, "layout: d=%ld heads=%ld not divisible by tp=%d (or bad elem size)",
                (long)d, (long)H, tp);
  const int64_t ff = 4 * d, qo = 3 * d / tp, pi = d / tp, fo = ff / tp;
  int n = 0;
  int64_t off = 0;
  auto put = [&](int64_t numel) -> bool {
    if (n >= max_entries) return false;
    off = (off + 255) & ~(int64_t)255;
    offsets[n] = off;
    numels[n] = numel;
    off += numel * es;
    n++;
    return true;
  };
  bool ok = put(V * d) && put(S * d);
  for (int64_t l = 0; ok && l < L; l++) {
    ok = put(d) && put(d) && put(qo * d) && put(qo) && put(d * pi) && put(d) && put(d) &&
         put(d) && put(fo * d) && put(fo) && put(d * fo) && put(d);
  }
  ok = ok && put(d) && put(d);
  if (ok && has_head) ok = put(V * d);
  if (!ok) return fail(KH_E_ARG, "layout: more than %d entries", max_entries);
  *total_bytes = off;   // the checkpoint stores exactly [0, off)
  return n;
}

// ---------------------------------------------------------------------------- data loader
struct KhData {
  std::vector<unsigned char> buf;
  int32_t T;
};
extern "C" KhData* kh_data_open(const char* path, int32_t T) {
  File f(path, "rb");
  if (!f.f) { fail(KH_E_IO, "data_open: cannot open %s", path); return nullptr; }
  fseek(f.f, 0, SEEK_END);
  long n = ftell(f.f);
  fseek(f.f, 0, SEEK_SET);
  if (n < (long)T + 2) { fail(KH_E_FORMAT, "data_open: corpus too small (%ld bytes)", n); return nullptr; }
  KhData* d = new KhData;
  d->T = T;
  d->buf.resize(n);
  if (!f.rd(d->buf.data(), n)) { delete d; fail(KH_E_IO, "data_open: short read"); return nullptr; }
  return d;
}
extern "C" int64_t kh_data_size(const KhData* d) { return (int64_t)d->buf.size(); }
extern "C" void kh_data_next(const KhData* d, uint64_t* rng, int32_t B, int32_t* idx, int32_t* tgt) {
  const int64_t n = (int64_t)d->buf.size();
  const int T = d->T;
  for (int b = 0; b < B; b++) {
    int64_t o = (int64_t)(kh_rng_u32(rng) % (uint32_t)(n - T - 1));
    for (int t = 0; t < T; t++) {
      idx[b * T + t] = d->buf[o + t];
      tgt[b * T + t] = d->buf[o + t + 1];
    }
  }
}
extern "C" void kh_data_close(KhData* d) { delete d; }

// ----------------------------------------------------------------------------------- CKP1
extern "C" int kh_ckpt_save(const char* path, const int32_t cfg[6], int32_t step, uint64_t rng,
                            uint64_t pb, uint64_t ob, const void* params, const void* m,
                            const void* v) {
  std::string tmp = std::string(path) + ".tmp";
  {
    File f(tmp.c_str(), "wb");
    if (!f.f) return fail(KH_E_IO, "ckpt_save: cannot open %s", tmp.c_str());
    bool ok = f.wr("CKP1", 4) && f.wr(cfg, 24) && f.wr(&step, 4) && f.wr(&rng, 8) &&
              f.wr(&pb, 8) && f.wr(&ob, 8) && f.wr(params, pb) && f.wr(m, ob) && f.wr(v, ob);
    if (!ok || fflush(f.f) != 0) return fail(KH_E_IO, "ckpt_save: write failed (%s)", tmp.c_str());
  }
  // a killed writer leaves the previous checkpoint intact
  if (rename(tmp.c_str(), path) != 0) return fail(KH_E_IO, "ckpt_save: rename to %s failed", path);
  return KH_OK;
}
static int ckpt_header(File& f, const char* path, int32_t cfg[6], int32_t* step, uint64_t* rng,
                       uint64_t* pb, uint64_t* ob) {
  char magic[4];
  if (!f.rd(magic, 4)) return fail(KH_E_FORMAT, "ckpt: %s is truncated (magic)", path);
  if (memcmp(magic, "CKP1", 4) != 0) return fail(KH_E_FORMAT, "ckpt: %s has bad magic", path);
  if (!(f.rd(cfg, 24) && f.rd(step, 4) && f.rd(rng, 8) && f.rd(pb, 8) && f.rd(ob, 8)))
    return fail(KH_E_FORMAT, "ckpt: %s is truncated (header)", path);
  return KH_OK;
}
extern "C" int kh_ckpt_peek(const char* path, int32_t cfg[6], int32_t* step, uint64_t* rng,
                            uint64_t* pb, uint64_t* ob) {
  File f(path, "rb");
  if (!f.f) return fail(KH_E_IO, "ckpt: cannot open %s", path);
  return ckpt_header(f, path, cfg, step, rng, pb, ob);
}
extern "C" int kh_ckpt_load(const char* path, const int32_t cfg[6], uint64_t pb, uint64_t ob,
                            int32_t* step, uint64_t* rng, void* params, void* m, void* v) {
  File f(path, "rb");
  if (!f.f) return fail(KH_E_IO, "ckpt: cannot open %s", path);
  int32_t c[6];
  uint64_t fpb, fob;
  int32_t fstep;
  uint64_t frng;
  int rc = ckpt_header(f, path, c, &fstep, &frng, &fpb, &fob);
  if (rc) return rc;
  if (memcmp(c, cfg, 24) != 0)
    return fail(KH_E_MISMATCH, "ckpt: config mismatch (file L%d d%d H%d V%d S%d B%d)", c[0], c[1],
                c[2], c[3], c[4], c[5]);
  if (fpb != pb) return fail(KH_E_MISMATCH, "ckpt: param bytes %llu != expected %llu",
                             (unsigned long long)fpb, (unsigned long long)pb);
  if (fob != ob) return fail(KH_E_MISMATCH, "ckpt: moment bytes %llu != expected %llu",
                             (unsigned long long)fob, (unsigned long long)ob);
  // check the length before overwriting live buffers
  long here = ftell(f.f);
  fseek(f.f, 0, SEEK_END);
  long end = ftell(f.f);
  fseek(f.f, here, SEEK_SET);
  if ((uint64_t)(end - here) < pb + 2 * ob) return fail(KH_E_FORMAT, "ckpt: %s is truncated (body)", path);
  if (!(f.rd(params, pb) && f.rd(m, ob) && f.rd(v, ob))) return fail(KH_E_IO, "ckpt: short read");
  *step = fstep;
  *rng = frng;
  return KH_OK;
}

// ----------------------------------------------------------------------------------- CHRN
struct KhRefT {
  std::string name;
  int32_t ndim = 0, dims[4] = {1, 1, 1, 1}, dtype = 0;
  std::vector<char> data;
};
struct KhRef {
  int32_t cfg[6];
  float opt[5];
  std::vector<KhRefT> t;
};
extern "C" KhRef* kh_ref_load(const char* path) {
  File f(path, "rb");
  if (!f.f) { fail(KH_E_IO, "ref_load: cannot open %s", path); return nullptr; }
  char magic[4];
  int32_t version;
  KhRef* r = new KhRef;
  if (!f.rd(magic, 4) || memcmp(magic, "CHRN", 4) != 0 || !f.rd(&version, 4) ||
      !f.rd(r->cfg, 24) || !f.rd(r->opt, 20)) {
    delete r;
    fail(KH_E_FORMAT, "ref_load: %s bad magic or short header", path);
    return nullptr;
  }
  for (;;) {
    int32_t nl;
    if (!f.rd(&nl, 4)) { delete r; fail(KH_E_FORMAT, "ref_load: missing terminator"); return nullptr; }
    if (nl < 0) break;
    KhRefT t;
    if (nl > 255) { delete r; fail(KH_E_FORMAT, "ref_load: name too long"); return nullptr; }
    t.name.resize(nl);
    bool ok = f.rd(&t.name[0], nl) && f.rd(&t.ndim, 4) && t.ndim >= 0 && t.ndim <= 4;
    int64_t count = 1;
    for (int i = 0; ok && i < t.ndim; i++) { ok = f.rd(&t.dims[i], 4); count *= t.dims[i]; }
    ok = ok && f.rd(&t.dtype, 4);
    if (ok) { t.data.resize(count * 4); ok = f.rd(t.data.data(), count * 4); }
    if (!ok) { delete r; fail(KH_E_FORMAT, "ref_load: truncated record"); return nullptr; }
    r->t.push_back(std::move(t));
  }
  return r;
}
extern "C" void kh_ref_free(KhRef* r) { delete r; }
extern "C" void kh_ref_header(const KhRef* r, int32_t cfg[6], float opt[5]) {
  memcpy(cfg, r->cfg, 24);
  memcpy(opt, r->opt, 20);
}
extern "C" int32_t kh_ref_count(const KhRef* r) { return (int32_t)r->t.size(); }
extern "C" const char* kh_ref_name(const KhRef* r, int32_t i) { return r->t[i].name.c_str(); }
extern "C" int32_t kh_ref_ndim(const KhRef* r, int32_t i) { return r->t[i].ndim; }
extern "C" void kh_ref_dims(const KhRef* r, int32_t i, int32_t dims[4]) { memcpy(dims, r->t[i].dims, 16); }
extern "C" int32_t kh_ref_dtype(const KhRef* r, int32_t i) { return r->t[i].dtype; }
extern "C" const void* kh_ref_data(const KhRef* r, int32_t i) { return r->t[i].data.data(); }
extern "C" int32_t kh_ref_find(const KhRef* r, const char* name) {
  for (size_t i = 0; i < r->t.size(); i++)
    if (r->t[i].name == name) return (int32_t)i;
  return -1;
}

// ----------------------------------------------------------------------------------- GRPO
extern "C" void kh_grpo_advantages(const float* rewards, int32_t n_groups, int32_t group,
                                   float eps, float* adv) {
  for (int g = 0; g < n_groups; g++) {
    const float* r = rewards + (int64_t)g * group;
    double mean = 0;
    for (int i = 0; i < group; i++) mean += r[i];
    mean /= group;
    double var = 0;
    for (int i = 0; i < group; i++) { double d = r[i] - mean; var += d * d; }
    var /= group;
    double sd = sqrt(var);
    for (int i = 0; i < group; i++) adv[(int64_t)g * group + i] = (float)((r[i] - mean) / (sd + eps));
  }
}
extern "C" void kh_grpo_coef(const float* adv, const float* p_cur, const float* p_ref,
                             int32_t rows, int32_t T, int32_t t0, int32_t t1, float beta,
                             float* coef) {
  t0 = std::max(t0, 0);
  t1 = std::min(t1, T - 1);
  const int64_t n_masked = (int64_t)rows * std::max(0, t1 - t0 + 1);
  const float inv = n_masked > 0 ? 1.f / (float)n_masked : 0.f;
  for (int r = 0; r < rows; r++)
    for (int t = 0; t < T; t++) {
      int64_t i = (int64_t)r * T + t;
      if (t < t0 || t > t1) { coef[i] = 0.f; continue; }
      float pc = std::max(p_cur[i], 1e-8f);
      coef[i] = (adv[r] - beta * (1.f - p_ref[i] / pc)) * inv;
    }
}

// ------------------------------------------------------------------------------- 1F1B
extern "C" int kh_pp_num_slots(int32_t stage, int32_t P, int32_t M) {
  return std::min(P - 1 - stage, M) + 1;
}
extern "C" int kh_pp_schedule(int32_t s, int32_t P, int32_t M, int32_t* out, int32_t max_ops) {
  if (P < 1 || s < 0 || s >= P || M < 1) return fail(KH_E_ARG, "pp_schedule: bad stage %d/%d M=%d", s, P, M);
  const bool first = s == 0, last = s == P - 1;
  const int warm = std::min(P - 1 - s, M), nslots = warm + 1;
  int n = 0;
  bool over = false;
  auto emit = [&](int op, int a0, int a1) {
    if (n >= max_ops) { over = true; return; }
    out[3 * n] = op; out[3 * n + 1] = a0; out[3 * n + 2] = a1;
    n++;
  };
  int ff = 0, bb = 0;
  if (!first) emit(KH_PP_RECV_ACT, 0, 0);
  for (int i = 0; i < warm; i++) {
    emit(KH_PP_FWD, ff, ff % nslots);
    if (!last) emit(KH_PP_SEND_ACT, ff, ff % nslots);
    ff++;
    if (!first && ff < M) emit(KH_PP_RECV_ACT, ff, ff % nslots);
  }
  for (int i = 0; i < M - warm; i++) {
    emit(KH_PP_FWD, ff, ff % nslots);
    if (!last) emit(KH_PP_SEND_ACT_RECV_GRAD, ff, bb);
    ff++;
    emit(KH_PP_BWD, bb, bb % nslots);
    if (!first) {
      if (ff < M) emit(KH_PP_SEND_GRAD_RECV_ACT, bb, ff);
      else emit(KH_PP_SEND_GRAD, bb, bb % nslots);
    }
    bb++;
  }
  for (int i = 0; i < warm; i++) {
    if (!last) emit(KH_PP_RECV_GRAD, bb, bb % nslots);
    emit(KH_PP_BWD, bb, bb % nslots);
    if (!first) emit(KH_PP_SEND_GRAD, bb, bb % nslots);
    bb++;
  }
  if (over) return fail(KH_E_ARG, "pp_schedule: more than %d ops", max_ops);
  return n;
}

// Schedule for stages whose sends never wait for the receiver (mailbox transport) and whose
// weight gradients are deferred: every micro-batch owns an activation slot (a1 == a0), a stage
// other than the last runs `extra` more forwards ahead than 1F1B would, and uses that slack to
// form the weight gradients of the first half of the micro-batches in the middle of the step
// (`mid` != 0) instead of all of them at its end.
extern "C" int kh_pp_schedule_deferred(int32_t s, int32_t P, int32_t M, int32_t extra, int32_t mid, int32_t* out,
                                       int32_t max_ops) {
  if (P < 1 || s < 0 || s >= P || M < 1 || extra < 0) return fail(KH_E_ARG, "pp_schedule_deferred: bad stage %d/%d M=%d", s, P, M);
  const bool first = s == 0, last = s == P - 1;
  const int warm = std::min(M, P - 1 - s + (last ? 0 : extra));
  const int flush_at = (!last && mid && M >= 4) ? M / 2 - 1 : -1;
  int n = 0;
  bool over = false;
  auto emit = [&](int op, int a0, int a1) {
    if (n >= max_ops) { over = true; return; }
    out[3 * n] = op; out[3 * n + 1] = a0; out[3 * n + 2] = a1;
    n++;
  };
  int ff = 0, bb = 0, flushed = 0;
  auto fwd = [&]() {
    if (!first) emit(KH_PP_RECV_ACT, ff, ff);
    emit(KH_PP_FWD, ff, ff);
    if (!last) emit(KH_PP_SEND_ACT, ff, ff);
    ff++;
  };
  for (int i = 0; i < warm; i++) fwd();
  while (bb < M) {
    if (ff < M) fwd();
    if (!last) emit(KH_PP_RECV_GRAD, bb, bb);
    emit(KH_PP_BWD, bb, bb);
    if (!first) emit(KH_PP_SEND_GRAD, bb, bb);
    if (bb == flush_at) { emit(KH_PP_FLUSH_DW, flushed, bb + 1); flushed = bb + 1; }
    bb++;
  }
  emit(KH_PP_FLUSH_DW, flushed, M);
  if (over) return fail(KH_E_ARG, "pp_schedule_deferred: more than %d ops", max_ops);
  return n;
}

// ------------------------------------------------------------------- paged-KV scheduler
namespace {
enum SeqState { S_FREE = 0, S_WAIT, S_RUN, S_HOLD, S_DONE };
struct Seq {
  SeqState st = S_FREE;
  std::vector<int32_t> tok;
  std::vector<int32_t> btab;
  int32_t plen = 0, max_new = 0, cached = 0;
  int64_t order = 0;   // admission order (FIFO)
};
}  // namespace
struct KhEngine {
  int32_t bs, n_blocks, max_seqs, max_lb, eos = -1;
  std::vector<int32_t> free_list;   // LIFO; initialised so that low ids pop first
  std::vector<int32_t> ref;
  std::vector<Seq> seqs;
  std::vector<int32_t> planned;     // seq ids of the step being run
  int64_t in_use = 0, peak = 0, decoded = 0, saved = 0, counter = 0;

  int alloc_block() {
    if (free_list.empty()) return -1;
    int b = free_list.back();
    free_list.pop_back();
    ref[b] = 1;
    in_use++;
    peak = std::max(peak, in_use);
    return b;
  }
  void unref(int b) {
    if (--ref[b] == 0) { free_list.push_back(b); in_use--; }
  }
  void drop(Seq& s) {
    for (int b : s.btab) unref(b);
    s.btab.clear();
  }
  bool ensure(Seq& s, int len) {   // blocks to hold positions [0, len)
    int need = (len + bs - 1) / bs;
    if (need > max_lb) return false;
    while ((int)s.btab.size() < need) {
      int b = alloc_block();
      if (b < 0) return false;
      s.btab.push_back(b);
    }
    return true;
  }
};
extern "C" void kh_eng_reset(KhEngine* e) {
  e->free_list.clear();
  for (int b = e->n_blocks - 1; b >= 0; b--) e->free_list.push_back(b);
  std::fill(e->ref.begin(), e->ref.end(), 0);
  for (auto& s : e->seqs) s = Seq();
  e->planned.clear();
  e->in_use = e->peak = e->decoded = e->saved = e->counter = 0;
}
extern "C" KhEngine* kh_eng_create(int32_t bs, int32_t n_blocks, int32_t max_seqs, int32_t max_lb) {
  if (bs < 1 || n_blocks < 1 || max_seqs < 1 || max_lb < 1) {
    fail(KH_E_ARG, "eng_create: bad sizes");
    return nullptr;
  }
  KhEngine* e = new KhEngine;
  e->bs = bs; e->n_blocks = n_blocks; e->max_seqs = max_seqs; e->max_lb = max_lb;
  e->ref.assign(n_blocks, 0);
  e->seqs.resize(max_seqs);
  kh_eng_reset(e);
  return e;
}
extern "C" void kh_eng_free(KhEngine* e) { delete e; }
extern "C" void kh_eng_set_eos(KhEngine* e, int32_t eos) { e->eos = eos; }
static int find_free(KhEngine* e) {
  for (int i = 0; i < e->max_seqs; i++)
    if (e->seqs[i].st == S_FREE) return i;
  return -1;
}
extern "C" int kh_eng_add(KhEngine* e, const int32_t* prompt, int32_t plen, int32_t max_new) {
  if (plen < 1 || max_new < 0) return fail(KH_E_ARG, "eng_add: plen=%d max_new=%d", plen, max_new);
  if ((plen + max_new + e->bs - 1) / e->bs > e->max_lb)
    return fail(KH_E_OOM, "eng_add: %d tokens exceed %d blocks per sequence", plen + max_new, e->max_lb);
  int id = find_free(e);
  if (id < 0) return fail(KH_E_OOM, "eng_add: all %d sequence slots are taken", e->max_seqs);
  Seq& s = e->seqs[id];
  s = Seq();
  s.st = S_WAIT;
  s.tok.assign(prompt, prompt + plen);
  s.plen = plen;
  s.max_new = max_new;
  s.order = e->counter++;
  return id;
}
extern "C" int kh_eng_fork(KhEngine* e, int32_t parent, int32_t n, int32_t max_new, int32_t* child_ids) {
  if (parent < 0 || parent >= e->max_seqs) return fail(KH_E_ARG, "eng_fork: bad parent");
  Seq& p = e->seqs[parent];
  if (p.st != S_HOLD || p.cached != (int)p.tok.size())
    return fail(KH_E_ARG, "eng_fork: parent %d has no cached prompt", parent);
  if (((int)p.tok.size() + max_new + e->bs - 1) / e->bs > e->max_lb)
    return fail(KH_E_OOM, "eng_fork: sequence would exceed %d blocks", e->max_lb);
  for (int i = 0; i < n; i++) {
    int id = find_free(e);
    if (id < 0) return fail(KH_E_OOM, "eng_fork: out of sequence slots");
    Seq& c = e->seqs[id];
    c = Seq();
    c.st = S_RUN;
    c.tok = p.tok;
    c.plen = (int)p.tok.size();
    c.cached = p.cached;
    c.max_new = max_new;
    c.btab = p.btab;
    c.order = e->counter++;
    for (int b : c.btab) e->ref[b]++;
    child_ids[i] = id;
  }
  e->saved += (int64_t)(n - 1) * ((int)p.tok.size() / e->bs);
  return KH_OK;
}
extern "C" int kh_eng_push(KhEngine* e, int32_t id, int32_t token) {
  if (id < 0 || id >= e->max_seqs || e->seqs[id].st != S_RUN) return fail(KH_E_ARG, "eng_push: bad id");
  Seq& s = e->seqs[id];
  s.tok.push_back(token);
  e->decoded++;
  if ((int)s.tok.size() - s.plen >= s.max_new || token == e->eos) { s.st = S_DONE; e->drop(s); }
  return KH_OK;
}
extern "C" int kh_eng_plan(KhEngine* e, int32_t max_active, int32_t max_tokens, int32_t* tok,
                           int32_t* pos, int32_t* slot, int32_t* rows, int32_t* seq_ids,
                           int32_t* btab, int32_t* n_tok, int32_t* n_seq, int32_t* copy_pairs,
                           int32_t max_pairs, int32_t* n_pairs) {
  *n_tok = *n_seq = *n_pairs = 0;
  e->planned.clear();
  // running sequences first (admission order), then admit waiting ones while there is room
  std::vector<int> run, wait;
  for (int i = 0; i < e->max_seqs; i++) {
    if (e->seqs[i].st == S_RUN) run.push_back(i);
    else if (e->seqs[i].st == S_WAIT) wait.push_back(i);
  }
  auto by_order = [&](int a, int b) { return e->seqs[a].order < e->seqs[b].order; };
  std::sort(run.begin(), run.end(), by_order);
  std::sort(wait.begin(), wait.end(), by_order);
  int budget = max_tokens;
  for (int id : run) budget -= (int)e->seqs[id].tok.size() - e->seqs[id].cached;
  for (int id : wait) {
    if ((int)run.size() >= max_active) break;
    Seq& s = e->seqs[id];
    int need_tok = (int)s.tok.size();
    int need_blk = (need_tok + e->bs - 1) / e->bs;
    if (need_tok > budget || need_blk > (int)e->free_list.size()) {
      if (run.empty()) return fail(KH_E_OOM, "eng_plan: sequence %d cannot be admitted (tokens %d, blocks %d)", id, need_tok, need_blk);
      break;
    }
    if (!e->ensure(s, need_tok)) return fail(KH_E_OOM, "eng_plan: KV pool exhausted");
    s.st = S_RUN;
    budget -= need_tok;
    run.push_back(id);
  }
  if (run.empty()) return 1;
  int nt = 0, ns = 0, np = 0;
  for (int id : run) {
    Seq& s = e->seqs[id];
    const int len = (int)s.tok.size();
    if (len == s.cached) continue;   // forked child still waiting for its first token
    if (nt + (len - s.cached) > max_tokens) return fail(KH_E_OOM, "eng_plan: step needs more than %d tokens", max_tokens);
    if (!e->ensure(s, len)) return fail(KH_E_OOM, "eng_plan: KV pool exhausted (in use %ld of %d)", (long)e->in_use, e->n_blocks);
    // copy-on-write: blocks that receive new positions must be private
    for (int lb = s.cached / e->bs; lb <= (len - 1) / e->bs; lb++) {
      int b = s.btab[lb];
      if (e->ref[b] > 1) {
        int nb = e->alloc_block();
        if (nb < 0) return fail(KH_E_OOM, "eng_plan: KV pool exhausted during copy-on-write");
        if (np >= max_pairs) return fail(KH_E_OOM, "eng_plan: more than %d block copies", max_pairs);
        copy_pairs[2 * np] = b;
        copy_pairs[2 * np + 1] = nb;
        np++;
        e->ref[b]--;
        s.btab[lb] = nb;
      }
    }
    for (int p = s.cached; p < len; p++) {
      tok[nt] = s.tok[p];
      pos[nt] = p;
      slot[nt] = ns;
      nt++;
    }
    rows[ns] = nt - 1;
    seq_ids[ns] = id;
    for (int j = 0; j < e->max_lb; j++) btab[(int64_t)ns * e->max_lb + j] = j < (int)s.btab.size() ? s.btab[j] : 0;
    e->planned.push_back(id);
    ns++;
  }
  *n_tok = nt;
  *n_seq = ns;
  *n_pairs = np;
  return ns == 0 ? 1 : 0;
}
extern "C" int kh_eng_commit(KhEngine* e, const int32_t* sampled, int32_t n_seq) {
  if (n_seq != (int)e->planned.size()) return fail(KH_E_ARG, "eng_commit: %d tokens for %d planned sequences", n_seq, (int)e->planned.size());
  int finished = 0;
  for (int i = 0; i < n_seq; i++) {
    Seq& s = e->seqs[e->planned[i]];
    s.cached = (int)s.tok.size();
    if (s.max_new == 0) { s.st = S_HOLD; continue; }   // prefill-only parent keeps its blocks
    s.tok.push_back(sampled[i]);
    e->decoded++;
    if ((int)s.tok.size() - s.plen >= s.max_new || sampled[i] == e->eos) {
      s.st = S_DONE;
      e->drop(s);
      finished++;
    }
  }
  e->planned.clear();
  return finished;
}
extern "C" int kh_eng_seq_len(const KhEngine* e, int32_t id) { return (int)e->seqs[id].tok.size(); }
extern "C" int kh_eng_seq_tokens(const KhEngine* e, int32_t id, int32_t* out, int32_t cap) {
  const Seq& s = e->seqs[id];
  int n = std::min<int>(cap, (int)s.tok.size());
  memcpy(out, s.tok.data(), (size_t)n * 4);
  return n;
}
extern "C" int kh_eng_seq_done(const KhEngine* e, int32_t id) { return e->seqs[id].st == S_DONE; }
extern "C" void kh_eng_release(KhEngine* e, int32_t id) {
  Seq& s = e->seqs[id];
  if (s.st == S_FREE) return;
  e->drop(s);
  s = Seq();
}
extern "C" void kh_eng_stats(const KhEngine* e, int64_t st[4]) {
  st[0] = e->n_blocks; st[1] = e->peak; st[2] = e->decoded; st[3] = e->saved;
}
extern "C" int kh_eng_blocks_in_use(const KhEngine* e) { return (int)e->in_use; }
extern "C" int kh_eng_block_ref(const KhEngine* e, int32_t b) { return e->ref[b]; }
