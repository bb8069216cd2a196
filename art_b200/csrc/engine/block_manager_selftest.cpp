// Stand-alone self test of the block manager, meant to be built with -fsanitize=address,undefined (and, in its
// threaded part, -fsanitize=thread): random alloc / free / prefix-match / commit traffic from several threads, with
// invariants checked after every operation.  Exit code 0 = all invariants held and the sanitizers stayed silent.
//
//   g++ -std=c++17 -O1 -g -fsanitize=address,undefined block_manager.cpp block_manager_selftest.cpp -lpthread
//
// The reference has no native host code to sanitise (pure Python); this covers the C++ runtime of the rollout engine.
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <thread>
#include <vector>

extern "C" {
void* artb_bm_create(int num_blocks, int block_size, int enable_prefix_cache);
void artb_bm_destroy(void* h);
int artb_bm_num_free(void* h);
int artb_bm_num_blocks(void* h);
int artb_bm_alloc(void* h, int n, int* out);
void artb_bm_free(void* h, const int* ids, int n);
int artb_bm_match_prefix(void* h, const int32_t* tokens, int n_tokens, uint64_t salt, int* out, int max_out);
void artb_bm_commit(void* h, const int* block_ids, int n_blocks, const int32_t* tokens, int n_tokens, uint64_t salt);
void artb_bm_reset_cache(void* h);
void artb_bm_stats(void* h, uint64_t* out4);
}

#define CHECK(c)                                                       \
  do {                                                                 \
    if (!(c)) {                                                        \
      fprintf(stderr, "CHECK failed at line %d: %s\n", __LINE__, #c);  \
      exit(1);                                                         \
    }                                                                  \
  } while (0)

static void worker(void* bm, int seed, int block_size, int iters) {
  std::mt19937 rng(seed);
  std::vector<std::vector<int>> held;
  std::vector<int32_t> toks(8 * block_size);
  for (int it = 0; it < iters; ++it) {
    const int op = rng() % 4;
    if (op == 0 || held.empty()) {
      // a "sequence": a prompt drawn from a small family so that prefixes repeat, matched against the cache,
      // the remainder freshly allocated, then committed
      const int n_blocks = 1 + rng() % 6;
      const int fam = rng() % 5;
      for (int i = 0; i < n_blocks * block_size; ++i) toks[i] = fam * 1000 + i / (block_size * (1 + fam % 2));
      std::vector<int> ids(n_blocks);
      const int hit = artb_bm_match_prefix(bm, toks.data(), n_blocks * block_size, 7 + fam % 2, ids.data(), n_blocks);
      CHECK(hit >= 0 && hit <= n_blocks);
      if (hit < n_blocks) {
        if (artb_bm_alloc(bm, n_blocks - hit, ids.data() + hit) != 0) {
          if (hit) artb_bm_free(bm, ids.data(), hit);   // could not get the rest: give the matched ones back
          continue;
        }
      }
      for (int i = 0; i < n_blocks; ++i) CHECK(ids[i] >= 0 && ids[i] < artb_bm_num_blocks(bm));
      artb_bm_commit(bm, ids.data(), n_blocks, toks.data(), n_blocks * block_size, 7 + fam % 2);
      held.push_back(ids);
    } else if (op == 1) {
      const size_t k = rng() % held.size();
      artb_bm_free(bm, held[k].data(), static_cast<int>(held[k].size()));
      held.erase(held.begin() + k);
    } else if (op == 2) {
      uint64_t st[4];
      artb_bm_stats(bm, st);
      CHECK(st[1] <= st[0] * 64);   // hits are bounded by queries x blocks per query
    } else {
      const int f = artb_bm_num_free(bm);
      CHECK(f >= 0 && f <= artb_bm_num_blocks(bm));
    }
  }
  for (auto& ids : held) artb_bm_free(bm, ids.data(), static_cast<int>(ids.size()));
}

int main(int argc, char** argv) {
  const int threads = argc > 1 ? atoi(argv[1]) : 4;
  const int iters = argc > 2 ? atoi(argv[2]) : 4000;
  for (int cache = 0; cache < 2; ++cache) {
    void* bm = artb_bm_create(256, 16, cache);
    CHECK(bm != nullptr);
    CHECK(artb_bm_num_free(bm) == 256);
    int tmp[300];
    CHECK(artb_bm_alloc(bm, 300, tmp) == -1);          // more than exists: nothing allocated
    CHECK(artb_bm_num_free(bm) == 256);
    std::vector<std::thread> ts;
    for (int t = 0; t < threads; ++t) ts.emplace_back(worker, bm, 100 * cache + t, 16, iters);
    for (auto& t : ts) t.join();
    artb_bm_reset_cache(bm);
    CHECK(artb_bm_num_free(bm) == 256);                // every reference returned, cached blocks evictable again
    artb_bm_destroy(bm);
  }
  CHECK(artb_bm_create(0, 16, 1) == nullptr);
  printf("block_manager selftest ok (%d threads x %d ops, with and without prefix cache)\n", threads, iters);
  return 0;
}
