// Allowed-token masks for structured outputs.
//
// A constrained completion follows a deterministic automaton over UTF-8 bytes (built on the host from a regular
// expression or a JSON schema).  Before each sampling step the engine needs, for the request's current automaton
// state, the set of vocabulary tokens whose byte strings keep the automaton alive.  The vocabulary is stored once as
// a byte trie in a flat, child-sorted layout; a mask is one depth-first walk of trie and automaton together, so a
// byte that kills the automaton prunes every token below it (a state that admits only digits touches a few dozen
// nodes; a state inside a free string touches nearly all of them, once, since masks are cached per state by the caller).
//
// The reference gets this from its inference library's guided-decoding backends (request fields guided_json /
// guided_regex / response_format, src/art/local/vllm.py:234-247).
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <utility>
#include <vector>

#define ARTB_API extern "C" __attribute__((visibility("default")))

namespace {

struct Trie {
  // node i owns edges [edge_begin[i], edge_begin[i + 1]) sorted by byte, and the tokens
  // [tok_begin[i], tok_begin[i + 1]) that end exactly there
  std::vector<int32_t> edge_begin, edge_child, tok_begin, tok_ids;
  std::vector<uint8_t> edge_byte;
  int n_tokens = 0;
};

struct BuildNode {
  std::vector<std::pair<uint8_t, int>> kids;   // (byte, node)
  std::vector<int> toks;
};

}  // namespace

ARTB_API void* artb_tm_create(const uint8_t* bytes, const int64_t* offsets, int n_tokens) {
  if (!bytes || !offsets || n_tokens < 0) return nullptr;
  std::vector<BuildNode> nodes(1);
  for (int t = 0; t < n_tokens; ++t) {
    const int64_t b = offsets[t], e = offsets[t + 1];
    if (e <= b) continue;   // tokens without text are never allowed
    int cur = 0;
    for (int64_t i = b; i < e; ++i) {
      const uint8_t c = bytes[i];
      int nxt = -1;
      for (const auto& k : nodes[cur].kids)
        if (k.first == c) { nxt = k.second; break; }
      if (nxt < 0) {
        nxt = static_cast<int>(nodes.size());
        nodes[cur].kids.emplace_back(c, nxt);
        nodes.emplace_back();
      }
      cur = nxt;
    }
    nodes[cur].toks.push_back(t);
  }
  auto* tr = new Trie;
  tr->n_tokens = n_tokens;
  const size_t n = nodes.size();
  tr->edge_begin.assign(n + 1, 0);
  tr->tok_begin.assign(n + 1, 0);
  for (size_t i = 0; i < n; ++i) {
    std::sort(nodes[i].kids.begin(), nodes[i].kids.end());
    tr->edge_begin[i + 1] = tr->edge_begin[i] + static_cast<int32_t>(nodes[i].kids.size());
    tr->tok_begin[i + 1] = tr->tok_begin[i] + static_cast<int32_t>(nodes[i].toks.size());
  }
  tr->edge_byte.resize(tr->edge_begin[n]);
  tr->edge_child.resize(tr->edge_begin[n]);
  tr->tok_ids.resize(tr->tok_begin[n]);
  for (size_t i = 0; i < n; ++i) {
    int32_t e = tr->edge_begin[i];
    for (const auto& k : nodes[i].kids) {
      tr->edge_byte[e] = k.first;
      tr->edge_child[e] = k.second;
      ++e;
    }
    std::copy(nodes[i].toks.begin(), nodes[i].toks.end(), tr->tok_ids.begin() + tr->tok_begin[i]);
  }
  return tr;
}

ARTB_API void artb_tm_destroy(void* h) { delete static_cast<Trie*>(h); }

// out[t] = 1 for every token whose bytes can be consumed from `state` of the automaton trans[n_states][256]
// (-1 = no transition).  Returns the number of allowed tokens, or -1 for a bad argument.
ARTB_API int artb_tm_mask(void* h, const int32_t* trans, int n_states, int state, uint8_t* out) {
  auto* tr = static_cast<Trie*>(h);
  if (!tr || !trans || !out || state < 0 || state >= n_states) return -1;
  std::memset(out, 0, static_cast<size_t>(tr->n_tokens));
  int count = 0;
  std::vector<std::pair<int32_t, int32_t>> stack;   // (trie node, automaton state)
  stack.emplace_back(0, state);
  while (!stack.empty()) {
    const auto [node, s] = stack.back();
    stack.pop_back();
    const int32_t* row = trans + static_cast<size_t>(s) * 256;
    for (int32_t e = tr->edge_begin[node]; e < tr->edge_begin[node + 1]; ++e) {
      const int32_t t = row[tr->edge_byte[e]];
      if (t < 0 || t >= n_states) continue;
      const int32_t child = tr->edge_child[e];
      for (int32_t k = tr->tok_begin[child]; k < tr->tok_begin[child + 1]; ++k) {
        out[tr->tok_ids[k]] = 1;
        ++count;
      }
      if (tr->edge_begin[child + 1] > tr->edge_begin[child]) stack.emplace_back(child, t);
    }
  }
  return count;
}
