// Host runtime of the framework: C ABI consumed from Python through ctypes.
//
// Everything here is plain C++17 with no CUDA dependency so that the CPU test tier can
// build and exercise it.  Functions return 0 on success and a negative KH_E_* code on
// failure; kh_last_error() gives the message.  Nothing in this library calls exit().
#pragma once
#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  KH_OK = 0,
  KH_E_IO = -1,        // open/read/write failed
  KH_E_FORMAT = -2,    // bad magic / truncated / malformed file
  KH_E_MISMATCH = -3,  // header does not match what the caller expects
  KH_E_ARG = -4,       // invalid argument
  KH_E_OOM = -5        // KV block pool exhausted / capacity exceeded
};

const char* kh_last_error(void);

// ---- xorshift64* RNG (state is one u64; it is what the checkpoint header stores) --------
void     kh_rng_seed(uint64_t* state, uint64_t seed);
uint32_t kh_rng_u32(uint64_t* state);
// idx[n] then tgt[n], each uniform in [0, vocab)
void     kh_rng_batch(uint64_t* state, int32_t* idx, int32_t* tgt, int64_t n, int32_t vocab);
// Box-Muller N(0, std) samples, 2 u32 draws per sample
void     kh_fill_normal(uint64_t* state, float* dst, int64_t n, float std);
// Draw a full [rows, cols] matrix in row-major order but keep only the block
// [r0, r1) x [c0, c1), written densely to dst (may be NULL to only advance the stream).
void     kh_fill_normal_block(uint64_t* state, float* dst, int64_t rows, int64_t cols,
                              int64_t r0, int64_t r1, int64_t c0, int64_t c1, float std);

// ---- parameter arena layout (256-byte aligned bump allocation) ---------------------------
// cfg = {n_layer, d_model, n_head, vocab, seq, batch}.  Entry order: wte, wpe, then per
// layer ln1_w ln1_b qkv_w qkv_b proj_w proj_b ln2_w ln2_b fc_w fc_b fcproj_w fcproj_b,
// then lnf_w lnf_b and (has_head) head_w.  elem_size is 4 (fp32 arenas) or 2 (bf16 arena).
// Fills byte offsets and element counts; returns the entry count or a negative error.
int kh_layout_params(const int32_t cfg[6], int32_t tp, int32_t has_head, int32_t elem_size,
                     int64_t* offsets, int64_t* numels, int32_t max_entries,
                     int64_t* total_bytes);

// ---- byte-corpus data loader ------------------------------------------------------------
typedef struct KhData KhData;
KhData* kh_data_open(const char* path, int32_t T);
int64_t kh_data_size(const KhData* d);
// B windows of T+1 bytes at offset rng % (n - T - 1); idx = window[:T], tgt = window[1:]
void    kh_data_next(const KhData* d, uint64_t* rng, int32_t B, int32_t* idx, int32_t* tgt);
void    kh_data_close(KhData* d);

// ---- CKP1 checkpoint -------------------------------------------------------------------
// "CKP1" | cfg 6xi32 | step i32 | rng u64 | pb u64 | ob u64 | params[pb] | m[ob] | v[ob]
int kh_ckpt_save(const char* path, const int32_t cfg[6], int32_t step, uint64_t rng,
                 uint64_t pb, uint64_t ob, const void* params, const void* m, const void* v);
int kh_ckpt_peek(const char* path, int32_t cfg[6], int32_t* step, uint64_t* rng,
                 uint64_t* pb, uint64_t* ob);
// Validates the header against cfg/pb/ob before touching the destination buffers.
int kh_ckpt_load(const char* path, const int32_t cfg[6], uint64_t pb, uint64_t ob,
                 int32_t* step, uint64_t* rng, void* params, void* m, void* v);

// ---- CHRN fixture files -----------------------------------------------------------------
typedef struct KhRef KhRef;
KhRef*      kh_ref_load(const char* path);
void        kh_ref_free(KhRef* r);
void        kh_ref_header(const KhRef* r, int32_t cfg[6], float opt[5]);
int32_t     kh_ref_count(const KhRef* r);
const char* kh_ref_name(const KhRef* r, int32_t i);
int32_t     kh_ref_ndim(const KhRef* r, int32_t i);
void        kh_ref_dims(const KhRef* r, int32_t i, int32_t dims[4]);
int32_t     kh_ref_dtype(const KhRef* r, int32_t i);   // 0 = f32, 1 = i32
const void* kh_ref_data(const KhRef* r, int32_t i);
int32_t     kh_ref_find(const KhRef* r, const char* name);

// ---- GRPO ------------------------------------------------------------------------------
// adv = (r - mean_g) / (std_pop_g + eps), statistics in double
void kh_grpo_advantages(const float* rewards, int32_t n_groups, int32_t group, float eps,
                        float* adv);
// coef[row, t] = mask * (adv[row] - beta * (1 - p_ref / max(p_cur, 1e-8))) / n_masked
// where mask = 1 for t in [t0, t1] of each row; rows x T row-major.
void kh_grpo_coef(const float* adv, const float* p_cur, const float* p_ref, int32_t rows,
                  int32_t T, int32_t t0, int32_t t1, float beta, float* coef);

// ---- 1F1B pipeline schedule -------------------------------------------------------------
enum {
  KH_PP_RECV_ACT = 0,   // receive stage input from the previous stage
  KH_PP_SEND_ACT = 1,   // send stage output to the next stage
  KH_PP_RECV_GRAD = 2,  // receive output-grad from the next stage
  KH_PP_SEND_GRAD = 3,  // send input-grad to the previous stage
  KH_PP_FWD = 4,        // forward of micro-batch a0 using activation slot a1
  KH_PP_BWD = 5,        // backward of micro-batch a0 using activation slot a1
  KH_PP_SEND_ACT_RECV_GRAD = 6,   // one fused exchange with the next stage
  KH_PP_SEND_GRAD_RECV_ACT = 7,   // one fused exchange with the previous stage
  KH_PP_FLUSH_DW = 8              // weight gradients of micro-batch slots [a0, a1) (deferred mode)
};
// Writes triples (op, a0, a1) into out[3 * max_ops]; returns the op count or negative error.
int kh_pp_schedule(int32_t stage, int32_t n_stages, int32_t n_micro, int32_t* out,
                   int32_t max_ops);
int kh_pp_num_slots(int32_t stage, int32_t n_stages, int32_t n_micro);
// Schedule for non-blocking sends and deferred weight gradients (one slot per micro-batch):
// `extra` additional warm-up forwards on every stage but the last, `mid` != 0 adds a weight-gradient
// pass over the first half of the micro-batches in the middle of the step.
int kh_pp_schedule_deferred(int32_t stage, int32_t n_stages, int32_t n_micro, int32_t extra, int32_t mid,
                            int32_t* out, int32_t max_ops);

// ---- paged-KV block pool and continuous-batching scheduler ------------------------------
typedef struct KhEngine KhEngine;
KhEngine* kh_eng_create(int32_t block_size, int32_t n_blocks, int32_t max_seqs,
                        int32_t max_blocks_per_seq);
void      kh_eng_free(KhEngine* e);
void      kh_eng_reset(KhEngine* e);
// Add a sequence in the waiting state; returns its id (>= 0) or a negative error.
int       kh_eng_add(KhEngine* e, const int32_t* prompt, int32_t plen, int32_t max_new);
// Fork `n` children from a parent whose prompt is already cached (a prefill-only sequence,
// max_new == 0, after its step was committed).  Every block of the parent, the partial
// last one included, is shared by reference; a child that later writes into a block whose
// reference count is above one gets a private copy first (copy-on-write, see kh_eng_plan).
int       kh_eng_fork(KhEngine* e, int32_t parent, int32_t n, int32_t max_new,
                      int32_t* child_ids);
// Append a token chosen by the caller (first token of a forked child).
int       kh_eng_push(KhEngine* e, int32_t id, int32_t token);
void      kh_eng_set_eos(KhEngine* e, int32_t eos);   // -1 disables early stop
// Admit waiting sequences (up to max_active running) and lay out the next step: one entry
// per uncached token.  tok/pos/slot have room for max_tokens ints, rows/seq_ids for
// max_seqs, btab for max_seqs * max_blocks_per_seq.  copy_pairs receives (src, dst)
// physical block pairs that must be copied on the device BEFORE the step runs (copy-on-
// write of shared blocks), 2 ints per pair.  Returns 0, or 1 when nothing is left to run,
// or a negative error.
int       kh_eng_plan(KhEngine* e, int32_t max_active, int32_t max_tokens, int32_t* tok,
                      int32_t* pos, int32_t* slot, int32_t* rows, int32_t* seq_ids,
                      int32_t* btab, int32_t* n_tok, int32_t* n_seq, int32_t* copy_pairs,
                      int32_t max_pairs, int32_t* n_pairs);
// Feed one sampled token per planned sequence (order of seq_ids); finished sequences are
// retired and their blocks released.  Returns how many sequences finished.
int       kh_eng_commit(KhEngine* e, const int32_t* sampled, int32_t n_seq);
int       kh_eng_seq_len(const KhEngine* e, int32_t id);
int       kh_eng_seq_tokens(const KhEngine* e, int32_t id, int32_t* out, int32_t cap);
int       kh_eng_seq_done(const KhEngine* e, int32_t id);
void      kh_eng_release(KhEngine* e, int32_t id);   // drop a finished/parent sequence
// stats[0..3] = blocks_total, blocks_peak, tokens_decoded, prefix_blocks_saved
void      kh_eng_stats(const KhEngine* e, int64_t stats[4]);
int       kh_eng_blocks_in_use(const KhEngine* e);
int       kh_eng_block_ref(const KhEngine* e, int32_t block);

#ifdef __cplusplus
}
#endif
