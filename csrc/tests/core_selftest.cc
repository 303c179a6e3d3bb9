// Native self-test of the host runtime library (libds41_core.so) through its C ABI, without Python in between:
//   g++ -std=c++17 -O1 csrc/tests/core_selftest.cc -L ds41rt_b200/_lib -lds41_core -Wl,-rpath,'$ORIGIN' -o ds41_core_selftest
// `python -m ds41rt_b200 selftest` builds and runs it.  Prints one line per group and "ok <checks>" at the end; the exit
// status is the number of failed checks.  Counterpart of the reference's CPU `native_selftest` target
// (native/CMakeLists.txt:963-1059, native/tests/).
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

extern "C" {
int ds41_core_version();
void* ds41_kv_new(int n_pages, int n_slots, int page_tokens);
void ds41_kv_free(void* p);
int ds41_kv_free_pages(const void* p);
int ds41_kv_admit(void* p, uint32_t* generation);
int ds41_kv_ensure(void* p, int slot, uint32_t gen, int n_tokens, int32_t* out, int cap);
int ds41_kv_retire(void* p, int slot, uint32_t gen);
int ds41_kv_page_count(const void* p, int slot);
void* ds41_admission_new(int queue_cap, int waiter_cap);
void ds41_admission_free(void* p);
int ds41_admission_reserve(void* p);
void ds41_admission_release(void* p);
void* ds41_lanes_new(int n_lanes);
void ds41_lanes_free(void* p);
int ds41_lanes_add(void* p, int64_t id, int remaining, int history);
int ds41_lanes_load(void* p, int lane);
float ds41_philox_uniform(uint64_t seed, uint64_t subsequence, uint64_t offset, int lane);
float ds41_sample_uniform(uint64_t seed, uint64_t position);
int ds41_sample_token(const float* logits, int vocab, const uint32_t* mask, int mask_words, float temperature,
                      int top_k, float top_p, float min_p, float uniform, int* token);
int ds41_verify_greedy(const uint32_t* inputs, const uint32_t* target_next, int n, uint32_t eos, int remaining,
                       uint32_t vocab, uint32_t* emitted, int* accepted_inputs, int* flags);
void* ds41_policy_new(int max_width, int warmup_rounds);
void ds41_policy_free(void* p);
void ds41_policy_observe(void* h, int width, int n_accepted, double verify_us, double draft_us, double confidence);
int ds41_policy_choose(void* h, double confidence);
uint64_t ds41_policy_probe(void* h, int every);
void ds41_policy_observe_round(void* h, int total_rows, int n_requests, double round_us);
void ds41_policy_observe_positions(void* h, const float* conf, int width, int n_accepted);
int ds41_policy_choose_joint(void* h, const float* conf, const int* offsets, int n_req, int* widths);
int ds41_ple_scan(const uint8_t* src, uint64_t rows, int dim, int src_row_bytes, int threads, float* amax);
float ds41_ple_global_scale(float amax);
int ds41_ple_convert(const uint8_t* src, uint64_t rows, int dim, int src_row_bytes, float global, uint8_t* dst,
                     int dst_row_bytes, int threads);
void* ds41_prefix_new(int prompt_capacity, int turn_capacity, int window);
void ds41_prefix_free(void* p);
int64_t ds41_prefix_insert(void* p, const uint32_t* tokens, int n, int bank, int64_t* evicted);
int64_t ds41_prefix_lookup(void* p, const uint32_t* tokens, int n, int* common, int* frontier, int* skipped);
void* ds41_vocab_new(const uint8_t* data, const int64_t* offsets, int n);
void ds41_vocab_free(void* v);
void* ds41_grammar_compile(const char* description, char* error, int error_cap);
void ds41_grammar_free(void* g);
void* ds41_matcher_new(const void* grammar);
void* ds41_matcher_fork(const void* m);
void ds41_matcher_free(void* m);
int ds41_matcher_can_finish(const void* m);
int ds41_matcher_accept_bytes(void* m, const uint8_t* bytes, int n);
int ds41_matcher_accept_token(void* m, const void* vocab, int token);
int ds41_matcher_fill_mask(const void* m, const void* vocab, uint32_t* mask, int stop_token);
void* ds41_hostcache_new(int n_pages, uint64_t page_bytes, uint64_t store_budget, uint64_t restore_budget);
void ds41_hostcache_free(void* p);
int ds41_hostcache_store(void* p, int64_t id, const uint64_t* keys, int n, uint64_t tokens, int32_t* host_pages,
                         uint8_t* need_copy);
int ds41_hostcache_restore(void* p, int64_t id, int32_t* host_pages, int cap);
int ds41_hostcache_restore_prefix(void* p, int64_t id, int n_first, int32_t* host_pages, int cap);
int ds41_hostcache_contains(void* p, int64_t id);
int ds41_hostcache_check(void* p);
void* ds41_engram_history_new(uint32_t pad_id);
void ds41_engram_history_free(void* h);
uint64_t ds41_engram_history_position(const void* h);
int ds41_engram_prepare(const void* hist, const int32_t* tokens, int n, uint64_t* hashes);
int ds41_engram_commit(void* hist, const int32_t* tokens, int n, int accepted);
}

static int g_checks = 0, g_failed = 0;
#define CHECK(cond)                                                                    \
  do {                                                                                 \
    ++g_checks;                                                                        \
    if (!(cond)) {                                                                     \
      ++g_failed;                                                                      \
      std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);                    \
    }                                                                                  \
  } while (0)

static void kv_pages() {
  void* kv = ds41_kv_new(6, 2, 64);
  uint32_t g0 = 0, g1 = 0;
  const int s0 = ds41_kv_admit(kv, &g0), s1 = ds41_kv_admit(kv, &g1);
  CHECK(s0 == 0 && s1 == 1 && g0 >= 1);
  CHECK(ds41_kv_admit(kv, nullptr) == -1);                       // both slots leased
  int32_t pairs[16];
  CHECK(ds41_kv_ensure(kv, s0, g0, 130, pairs, 8) == 3);         // 130 tokens = three 64-token pages
  CHECK(ds41_kv_ensure(kv, s0, g0, 100, pairs, 8) == 0);         // already covered
  CHECK(ds41_kv_page_count(kv, s0) == 3 && ds41_kv_free_pages(kv) == 3);
  CHECK(ds41_kv_ensure(kv, s1, g1, 64 * 4, pairs, 8) == -2);     // pool exhausted: nothing changes
  CHECK(ds41_kv_free_pages(kv) == 3);
  CHECK(ds41_kv_ensure(kv, s0, g0 + 1, 10, pairs, 8) == -1);     // stale lease
  CHECK(ds41_kv_retire(kv, s0, g0) == 0 && ds41_kv_free_pages(kv) == 6);
  CHECK(ds41_kv_retire(kv, s0, g0) == -1);                       // the generation moved on
  ds41_kv_free(kv);
  std::printf("kv allocator ok\n");
}

static void admission_and_lanes() {
  void* a = ds41_admission_new(2, 1);
  CHECK(ds41_admission_reserve(a) == 0 && ds41_admission_reserve(a) == 0);
  CHECK(ds41_admission_reserve(a) == 1);                          // waits for queue space
  CHECK(ds41_admission_reserve(a) == -1);                         // refused: HTTP 429
  ds41_admission_release(a);
  CHECK(ds41_admission_reserve(a) == 1);                          // the waiter moved up, one waiting place is free
  ds41_admission_free(a);
  void* l = ds41_lanes_new(2);
  CHECK(ds41_lanes_add(l, 1, 100, 10) == 0 && ds41_lanes_add(l, 2, 100, 10) == 1 && ds41_lanes_add(l, 3, 50, 10) == 0);
  CHECK(ds41_lanes_load(l, 0) == 2 && ds41_lanes_load(l, 1) == 1);
  ds41_lanes_free(l);
  std::printf("admission and lanes ok\n");
}

static void random_numbers_and_sampling() {
  const float u = ds41_philox_uniform(7, 3, 11, 2);
  CHECK(u >= 0.f && u < 1.f && u == ds41_philox_uniform(7, 3, 11, 2) && u != ds41_philox_uniform(7, 3, 12, 2));
  const float s = ds41_sample_uniform(5, 9);
  CHECK(s >= 0.f && s < 1.f && s == ds41_sample_uniform(5, 9));
  float logits[40];
  for (int i = 0; i < 40; ++i) logits[i] = -1.f - 0.01f * i;
  logits[17] = logits[23] = 4.f;                                  // a tie: the lowest id wins
  int tok = -1;
  CHECK(ds41_sample_token(logits, 40, nullptr, 0, 0.f, 0, 1.f, 0.f, 0.3f, &tok) == 0 && tok == 17);
  uint32_t mask[2] = {~(1u << 17), 0xffu};                        // token 17 is not allowed
  CHECK(ds41_sample_token(logits, 40, mask, 2, 0.f, 0, 1.f, 0.f, 0.3f, &tok) == 0 && tok == 23);
  CHECK(ds41_sample_token(logits, 40, mask, 1, 0.f, 0, 1.f, 0.f, 0.3f, &tok) == 4);      // wrong mask width
  CHECK(ds41_sample_token(logits, 40, nullptr, 0, -1.f, 0, 1.f, 0.f, 0.3f, &tok) == 3);  // bad temperature
  uint32_t none[2] = {0u, 0u};
  CHECK(ds41_sample_token(logits, 40, none, 2, 0.8f, 0, 1.f, 0.f, 0.3f, &tok) == 1);     // nothing allowed
  logits[5] = NAN;
  CHECK(ds41_sample_token(logits, 40, nullptr, 0, 0.8f, 0, 0.9f, 0.f, 0.3f, &tok) == 2); // non-finite logit
  logits[5] = -2.f;
  int a = -1, b = -1;                                             // stochastic draws are a function of the uniform
  CHECK(ds41_sample_token(logits, 40, nullptr, 0, 1.0f, 0, 1.f, 0.f, 0.01f, &a) == 0);
  CHECK(ds41_sample_token(logits, 40, nullptr, 0, 1.0f, 0, 1.f, 0.f, 0.01f, &b) == 0 && a == b);
  CHECK(ds41_sample_token(logits, 40, nullptr, 0, 1.0f, 1, 1.f, 0.f, 0.99f, &a) == 0 && a == 17);   // top_k 1 is greedy
  std::printf("random numbers and sampler oracle ok\n");
}

static void verify_rule() {
  const uint32_t inputs[4] = {10, 11, 12, 13};                    // anchor + three drafts
  const uint32_t next[4] = {11, 12, 99, 14};                      // the target agrees with two drafts
  uint32_t emitted[8];
  int accepted = 0, flags = 0;
  CHECK(ds41_verify_greedy(inputs, next, 4, 1, 100, 1000, emitted, &accepted, &flags) == 3);
  CHECK(emitted[0] == 11 && emitted[1] == 12 && emitted[2] == 99 && accepted == 3 && flags == 0);
  CHECK(ds41_verify_greedy(inputs, next, 4, 1, 2, 1000, emitted, &accepted, &flags) == 2 && (flags & 2));   // length
  const uint32_t stop[4] = {11, 1, 12, 13};
  CHECK(ds41_verify_greedy(inputs, stop, 4, 1, 100, 1000, emitted, &accepted, &flags) == 2 && (flags & 1)); // EOS
  CHECK(ds41_verify_greedy(inputs, next, 4, 1, 0, 1000, emitted, &accepted, &flags) < 0);
  std::printf("verification rule ok\n");
}

static void policy() {
  void* p = ds41_policy_new(4, 4);
  CHECK(ds41_policy_choose(p, -1.0) == 4);                        // warm-up verifies everything
  for (int i = 0; i < 60; ++i) {
    ds41_policy_observe(p, 4, 0, 1000 + 150 * 5, 80.0, -1.0);     // nothing is ever accepted
    ds41_policy_observe(p, 0, 0, 1000 + 150, 0.0, -1.0);
  }
  CHECK(ds41_policy_choose(p, -1.0) == 0);
  ds41_policy_probe(p, 4);
  int probes = 0;
  for (int i = 0; i < 12; ++i) probes += ds41_policy_choose(p, -1.0) > 0;
  CHECK(probes == 3 && ds41_policy_probe(p, -1) == 3);
  ds41_policy_free(p);
  // a shared round: rows go to the request whose drafts are likely to be kept; a round with cheap rows takes them all
  p = ds41_policy_new(4, 0);
  const float sure[4] = {0.95f, 0.95f, 0.95f, 0.95f}, doubt[4] = {0.05f, 0.05f, 0.05f, 0.05f};
  for (int i = 0; i < 200; ++i) {
    ds41_policy_observe(p, 4, 4, -1.0, 0.0, 0.95);
    ds41_policy_observe_positions(p, sure, 4, 4);
    ds41_policy_observe(p, 4, 0, -1.0, 0.0, 0.05);
    ds41_policy_observe_positions(p, doubt, 4, 0);
    ds41_policy_observe_round(p, 2 + (i % 5) * 2, 2, 1000.0 + 400.0 * (2 + (i % 5) * 2));
  }
  const float conf[8] = {0.95f, 0.95f, 0.95f, 0.95f, 0.05f, 0.05f, 0.05f, 0.05f};
  const int offs[3] = {0, 4, 8};
  int widths[2] = {-1, -1};
  CHECK(ds41_policy_choose_joint(p, conf, offs, 2, widths) == widths[0] + widths[1]);
  CHECK(widths[0] >= 3 && widths[1] == 0);
  ds41_policy_free(p);
  std::printf("verification policy ok\n");
}

static void table_conversion() {
  // one 32-value record: E4M3 codes 0x38 (1.0) ... with the UE8M0 scale 127 (x1); the largest value is 6 x 448 / 448
  uint8_t rec[33];
  for (int i = 0; i < 32; ++i) rec[i] = 0x38;                     // 1.0
  rec[0] = 0x4c;                                                  // exponent 9, mantissa 4: 1.5 * 2^2 = 6.0
  rec[1] = 0xb8;                                                  // -1.0
  rec[16] = 0x00;
  rec[32] = 127;
  float amax = 0.f;
  CHECK(ds41_ple_scan(rec, 1, 32, 33, 1, &amax) == 0 && amax == 6.0f);
  const float g = ds41_ple_global_scale(amax);
  CHECK(std::fabs(g - 6.0f / (6.0f * 448.0f)) < 1e-12f);
  uint8_t out[18];
  CHECK(ds41_ple_convert(rec, 1, 32, 33, g, out, 18, 1) == 0);
  CHECK(out[16] == 0x7e);                                         // first group: amax 6 -> scale 448 (code 0x7e)
  CHECK((out[0] & 15) == 7 && (out[0] >> 4) == (8 | 2));          // 6.0 -> code 7; -1.0 -> sign | code 2
  CHECK(out[17] == 0x69);                                         // second group: amax 1 -> scale 448 / 6 rounds to 72
  CHECK((out[8] & 15) == 0);                                      // the zero stays +0
  rec[3] = 0x7f;                                                  // NaN payload: refused
  CHECK(ds41_ple_scan(rec, 1, 32, 33, 1, &amax) == 2 && std::isnan(amax));
  std::printf("table conversion ok\n");
}

static void prefix_banks() {
  void* r = ds41_prefix_new(2, 2, 2);               // window 2: a shared prefix is worth its even length minus 2 tokens
  std::vector<uint32_t> a = {1, 2, 3, 4, 5, 6, 7, 8}, b = {1, 2, 3, 4, 9, 9, 9, 9, 9};
  int64_t ev = -2;
  const int64_t ia = ds41_prefix_insert(r, a.data(), 8, 0, &ev);
  CHECK(ia >= 0 && ev == -1);
  int common = 0, frontier = 0, skipped = 0;
  std::vector<uint32_t> q = {1, 2, 3, 4, 5, 6, 7, 8, 20, 21};
  CHECK(ds41_prefix_lookup(r, q.data(), 10, &common, &frontier, &skipped) == ia && common == 8 && frontier == 8);
  CHECK(ds41_prefix_lookup(r, b.data(), 9, &common, &frontier, &skipped) == ia && common == 4 && skipped == 2);
  std::vector<uint32_t> other = {50, 51};
  CHECK(ds41_prefix_lookup(r, other.data(), 2, &common, &frontier, &skipped) == -1);
  ds41_prefix_free(r);
  std::printf("prefix banks ok\n");
}

static bool feed(void* m, const char* text) {
  return ds41_matcher_accept_bytes(m, reinterpret_cast<const uint8_t*>(text), static_cast<int>(std::strlen(text))) == 1;
}

static void grammar_engine() {
  char err[256] = {0};
  void* g = ds41_grammar_compile(
      "{\"schema\": {\"type\": \"object\", \"properties\": {\"n\": {\"type\": \"integer\"}, \"ok\": {\"type\": "
      "\"boolean\"}}, \"required\": [\"n\", \"ok\"]}}", err, sizeof(err));
  CHECK(g != nullptr);
  void* m = ds41_matcher_new(g);
  CHECK(feed(m, "{\"n\": 12") && !ds41_matcher_can_finish(m));
  void* fork = ds41_matcher_fork(m);                              // a probe for draft rows: the original does not move
  CHECK(!feed(fork, "x") && feed(m, ", \"ok\": true}") && ds41_matcher_can_finish(m));
  ds41_matcher_free(fork);
  void* bad = ds41_matcher_new(g);
  CHECK(!feed(bad, "{\"n\": \"twelve\"") );
  ds41_matcher_free(bad);
  // token masks over a tiny vocabulary: "{", "}", "\"n\"", "1", "x", " "
  const char* toks[6] = {"{", "}", "\"n\"", "1", "x", " "};
  std::vector<uint8_t> data;
  std::vector<int64_t> off = {0};
  for (const char* t : toks) {
    data.insert(data.end(), t, t + std::strlen(t));
    off.push_back(static_cast<int64_t>(data.size()));
  }
  void* v = ds41_vocab_new(data.data(), off.data(), 6);
  void* fresh = ds41_matcher_new(g);
  uint32_t mask = 0;
  CHECK(ds41_matcher_fill_mask(fresh, v, &mask, -1) >= 1 && (mask & 1u) && !(mask & (1u << 4)));   // "{" yes, "x" no
  CHECK(ds41_matcher_accept_token(fresh, v, 0) == 1 && ds41_matcher_accept_token(fresh, v, 4) == 0);
  ds41_matcher_fill_mask(fresh, v, &mask, -1);
  CHECK((mask & (1u << 2)) && !(mask & (1u << 3)));               // after "{": the key "n" may follow, a digit may not
  ds41_matcher_free(fresh);
  ds41_matcher_free(m);
  ds41_vocab_free(v);
  ds41_grammar_free(g);
  CHECK(ds41_grammar_compile("{\"schema\": {\"type\": \"frob\"}}", err, sizeof(err)) == nullptr && err[0] != 0);
  std::printf("grammar engine ok\n");
}

static void host_cache_and_engram_history() {
  void* c = ds41_hostcache_new(4, 4096, 1ull << 40, 1ull << 40);
  const uint64_t ka[3] = {11, 12, 13}, kb[3] = {11, 12, 99};      // two snapshots share two pages by content
  int32_t pages[4];
  uint8_t need[4];
  CHECK(ds41_hostcache_store(c, 1, ka, 3, 192, pages, need) == 3 && need[0] && need[1] && need[2]);
  CHECK(ds41_hostcache_store(c, 2, kb, 3, 192, pages, need) == 3 && !need[0] && !need[1] && need[2]);
  CHECK(ds41_hostcache_contains(c, 1) && ds41_hostcache_restore(c, 2, pages, 4) == 3 && ds41_hostcache_check(c) == 0);
  const uint64_t kc[3] = {21, 22, 23};                            // no room beside both: the older snapshot goes
  CHECK(ds41_hostcache_store(c, 3, kc, 3, 192, pages, need) == 3 && ds41_hostcache_check(c) == 0);
  CHECK(!ds41_hostcache_contains(c, 1) || !ds41_hostcache_contains(c, 2));
  CHECK(ds41_hostcache_restore(c, 77, pages, 4) == -1);
  CHECK(ds41_hostcache_restore_prefix(c, 3, 2, pages, 4) == 2 && ds41_hostcache_restore_prefix(c, 3, 4, pages, 4) == -1);
  CHECK(ds41_hostcache_restore_prefix(c, 77, 1, pages, 4) == -1 && ds41_hostcache_check(c) == 0);
  ds41_hostcache_free(c);
  // the restore budget is charged for the pages asked for, not for the whole snapshot
  c = ds41_hostcache_new(4, 4096, 1ull << 40, 2 * 4096);
  CHECK(ds41_hostcache_store(c, 1, ka, 3, 192, pages, need) == 3);
  CHECK(ds41_hostcache_restore(c, 1, pages, 4) == 0 && ds41_hostcache_restore_prefix(c, 1, 2, pages, 4) == 2);
  CHECK(ds41_hostcache_restore_prefix(c, 1, 1, pages, 4) == 0);
  ds41_hostcache_free(c);
  void* h = ds41_engram_history_new(2);
  const int32_t toks[4] = {5, 6, 7, 8};
  uint64_t first[4 * 48], again[4 * 48];
  CHECK(ds41_engram_prepare(h, toks, 4, first) == 0 && ds41_engram_history_position(h) == 0);
  CHECK(ds41_engram_commit(h, toks, 4, 2) == 0 && ds41_engram_history_position(h) == 2);      // two rows accepted
  CHECK(ds41_engram_prepare(h, toks + 2, 2, again) == 0);
  CHECK(std::memcmp(first + 2 * 48, again, sizeof(uint64_t) * 2 * 48) == 0);    // same history, same hashes
  CHECK(ds41_engram_commit(h, toks, 4, 5) != 0);                  // more than was prepared
  ds41_engram_history_free(h);
  std::printf("host cache and n-gram history ok\n");
}

int main() {
  CHECK(ds41_core_version() >= 1);
  kv_pages();
  admission_and_lanes();
  random_numbers_and_sampling();
  verify_rule();
  policy();
  table_conversion();
  prefix_banks();
  grammar_engine();
  host_cache_and_engram_history();
  if (g_failed == 0) std::printf("ok %d checks\n", g_checks);
  else std::printf("%d of %d checks FAILED\n", g_failed, g_checks);
  return g_failed;
}
