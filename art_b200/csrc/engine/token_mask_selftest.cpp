// Stand-alone self test of the allowed-token mask builder, meant to be built with -fsanitize=address,undefined (and
// -fsanitize=thread: masks of one trie are computed from several threads at once, which the engine may do when two
// servers share a tokenizer).  A random vocabulary and a random automaton; every mask is compared with the
// token-by-token definition.  Exit code 0 = all masks agreed and the sanitizers stayed silent.
//
//   g++ -std=c++17 -O1 -g -fsanitize=address,undefined token_mask.cpp token_mask_selftest.cpp -lpthread
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <random>
#include <string>
#include <thread>
#include <vector>

extern "C" {
void* artb_tm_create(const uint8_t* bytes, const int64_t* offsets, int n_tokens);
void artb_tm_destroy(void* h);
int artb_tm_mask(void* h, const int32_t* trans, int n_states, int state, uint8_t* out);
}

#define CHECK(c)                                                       \
  do {                                                                 \
    if (!(c)) {                                                        \
      fprintf(stderr, "CHECK failed: %s (line %d)\n", #c, __LINE__);   \
      exit(1);                                                         \
    }                                                                  \
  } while (0)

int main(int argc, char** argv) {
  const int n_threads = argc > 1 ? atoi(argv[1]) : 4;
  const int n_tokens = argc > 2 ? atoi(argv[2]) : 3000;
  std::mt19937 rng(1234);
  // vocabulary over a 6-letter alphabet so that prefixes are shared; some empty tokens; some duplicates
  std::vector<std::string> vocab;
  for (int t = 0; t < n_tokens; ++t) {
    const int len = rng() % 6;   // 0 = a token without text
    std::string s;
    for (int i = 0; i < len; ++i) s.push_back(static_cast<char>('a' + rng() % 6));
    vocab.push_back(s);
  }
  std::vector<uint8_t> blob(1, 0);
  std::vector<int64_t> off(1, 0);
  blob.clear();
  for (const auto& s : vocab) {
    blob.insert(blob.end(), s.begin(), s.end());
    off.push_back(static_cast<int64_t>(blob.size()));
  }
  if (blob.empty()) blob.push_back(0);
  void* h = artb_tm_create(blob.data(), off.data(), n_tokens);
  CHECK(h != nullptr);
  // random automaton: 40 states, each letter leads somewhere with probability 0.7
  const int n_states = 40;
  std::vector<int32_t> trans(static_cast<size_t>(n_states) * 256, -1);
  for (int s = 0; s < n_states; ++s)
    for (int c = 'a'; c < 'a' + 6; ++c)
      if (rng() % 10 < 7) trans[static_cast<size_t>(s) * 256 + c] = static_cast<int32_t>(rng() % n_states);
  CHECK(artb_tm_mask(h, trans.data(), n_states, -1, blob.data()) == -1);
  CHECK(artb_tm_mask(h, trans.data(), n_states, n_states, blob.data()) == -1);
  std::vector<std::thread> pool;
  for (int w = 0; w < n_threads; ++w) {
    pool.emplace_back([&, w] {
      std::vector<uint8_t> out(n_tokens);
      for (int s = w; s < n_states; s += n_threads) {
        const int count = artb_tm_mask(h, trans.data(), n_states, s, out.data());
        int want_count = 0;
        for (int t = 0; t < n_tokens; ++t) {
          int cur = s;
          for (unsigned char c : vocab[t]) {
            if (cur < 0) break;
            cur = trans[static_cast<size_t>(cur) * 256 + c];
          }
          const bool want = !vocab[t].empty() && cur >= 0;
          CHECK(out[t] == (want ? 1 : 0));
          want_count += want;
        }
        CHECK(count == want_count);
      }
    });
  }
  for (auto& t : pool) t.join();
  artb_tm_destroy(h);
  printf("selftest ok\n");
  return 0;
}
