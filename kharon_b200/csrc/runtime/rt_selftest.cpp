// Self-test of the host runtime meant to be built with -fsanitize=address,undefined: drives the RNG,
// layout, checkpoint IO with corrupt inputs, the 1F1B generator and the KV scheduler through
// allocation-heavy paths so that the sanitizers can see out-of-bounds accesses, leaks and UB.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <string>
#include <vector>

#include "kharon_rt.h"

#define CHECK(c) do { if (!(c)) { fprintf(stderr, "selftest failed at %s:%d: %s\n", __FILE__, __LINE__, #c); return 1; } } while (0)

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : "/tmp";
  uint64_t s;
  kh_rng_seed(&s, 1337);
  std::vector<int32_t> idx(257), tgt(257);
  kh_rng_batch(&s, idx.data(), tgt.data(), 257, 50257);
  std::vector<float> blk(3 * 3);
  kh_fill_normal_block(&s, blk.data(), 6, 8, 2, 5, 1, 4, 0.02f);
  kh_fill_normal_block(&s, nullptr, 6, 8, 0, 6, 0, 8, 0.02f);

  int32_t cfg[6] = {3, 64, 4, 97, 16, 2};
  int64_t offs[64], nums[64], total = 0;
  int n = kh_layout_params(cfg, 2, 1, 4, offs, nums, 64, &total);
  CHECK(n == 2 + 3 * 12 + 2 + 1 && total > 0);
  CHECK(kh_layout_params(cfg, 2, 1, 4, offs, nums, 5, &total) < 0);       // too few slots: clean error

  std::vector<float> p(1000, 1.f), m(1000, 2.f), v(1000, 3.f);
  const std::string ck = dir + "/kh_selftest.ckpt";
  CHECK(kh_ckpt_save(ck.c_str(), cfg, 7, 99, 4000, 4000, p.data(), m.data(), v.data()) == 0);
  int32_t step; uint64_t rng;
  std::vector<float> p2(1000), m2(1000), v2(1000);
  CHECK(kh_ckpt_load(ck.c_str(), cfg, 4000, 4000, &step, &rng, p2.data(), m2.data(), v2.data()) == 0 && step == 7 && rng == 99);
  CHECK(kh_ckpt_load(ck.c_str(), cfg, 4004, 4000, &step, &rng, p2.data(), m2.data(), v2.data()) == KH_E_MISMATCH);
  { FILE* f = fopen(ck.c_str(), "r+b"); CHECK(f); CHECK(ftruncate(fileno(f), 300) == 0); fclose(f); }
  CHECK(kh_ckpt_load(ck.c_str(), cfg, 4000, 4000, &step, &rng, p2.data(), m2.data(), v2.data()) == KH_E_FORMAT);
  CHECK(kh_ref_load((dir + "/does_not_exist.bin").c_str()) == nullptr);

  std::vector<int32_t> ops(3 * 256);
  for (int P = 1; P <= 4; P++)
    for (int st = 0; st < P; st++) CHECK(kh_pp_schedule(st, P, 8, ops.data(), 256) > 0);
  CHECK(kh_pp_schedule(0, 2, 8, ops.data(), 3) < 0);

  KhEngine* e = kh_eng_create(4, 64, 9, 16);
  CHECK(e);
  std::vector<int32_t> prompt = {1, 2, 3, 4, 5, 6};
  int parent = kh_eng_add(e, prompt.data(), 6, 0);
  std::vector<int32_t> tok(256), pos(256), slot(256), rows(16), ids(16), btab(9 * 16), pairs(64);
  int32_t nt, ns, np;
  CHECK(kh_eng_plan(e, 8, 256, tok.data(), pos.data(), slot.data(), rows.data(), ids.data(), btab.data(), &nt, &ns, pairs.data(), 32, &np) == 0);
  std::vector<int32_t> sampled(16, 5);
  kh_eng_commit(e, sampled.data(), ns);
  std::vector<int32_t> kids(8);
  CHECK(kh_eng_fork(e, parent, 8, 10, kids.data()) == 0);
  kh_eng_release(e, parent);
  for (int k : kids) kh_eng_push(e, k, 7);
  for (int it = 0; it < 20; it++) {
    int rc = kh_eng_plan(e, 8, 256, tok.data(), pos.data(), slot.data(), rows.data(), ids.data(), btab.data(), &nt, &ns, pairs.data(), 32, &np);
    if (rc == 1) break;
    CHECK(rc == 0);
    kh_eng_commit(e, sampled.data(), ns);
  }
  for (int k : kids) { CHECK(kh_eng_seq_done(e, k)); kh_eng_release(e, k); }
  CHECK(kh_eng_blocks_in_use(e) == 0);
  kh_eng_free(e);
  remove(ck.c_str());
  printf("runtime selftest ok\n");
  return 0;
}
