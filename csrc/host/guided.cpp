// Guided decoding on the host: the allowed-token mask of one automaton state as a pruned walk of the vocabulary trie.
//
// The trie (built once per tokenizer in Python, poot_b200/text/automata.py) stores every token's bytes; a node's
// children are contiguous.  The automaton is a dense byte DFA (table[state * 256 + byte], -1 = dead).  The walk
// descends only along bytes the DFA can take, so its cost is the number of reachable trie nodes, and every token that
// ends on a reached node is allowed.  The reference computes the same per-state masks by walking the token byte table
// (crates/poot-text/src/guided.rs:297-335) and caches them by DFA state; the cache lives on the Python side.
#include <cstdint>
#include <vector>

#define HOST_API extern "C" __attribute__((visibility("default")))

HOST_API void poot_guided_walk_dfa(const int32_t* child_start, const uint8_t* child_byte, const int32_t* child_node,
                                   const int32_t* tok_start, const int32_t* tokens, int n_nodes, const int32_t* table,
                                   int n_states, int state, uint8_t* out_allowed) {
  if (state < 0 || state >= n_states || n_nodes <= 0) return;
  std::vector<std::pair<int32_t, int32_t>> stack;
  stack.reserve(1024);
  stack.push_back({0, state});
  while (!stack.empty()) {
    const auto [node, st] = stack.back();
    stack.pop_back();
    for (int32_t e = child_start[node]; e < child_start[node + 1]; ++e) {
      const int32_t ns = table[(size_t)st * 256 + child_byte[e]];
      if (ns < 0) continue;
      const int32_t ch = child_node[e];
      for (int32_t t = tok_start[ch]; t < tok_start[ch + 1]; ++t) out_allowed[tokens[t]] = 1;
      stack.push_back({ch, ns});
    }
  }
}
