// Random append / extend / remove / speculate traffic on the suffix tree with an integrity
// check after every batch. Built by tests/test_suffix_tree.py with
// -fsanitize=address,undefined: memory errors and undefined behaviour abort the run.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <vector>

#include "suffix_tree.h"

using ab200::Draft;
using ab200::SuffixTree;

int main(int argc, char** argv) {
  const unsigned seed = argc > 1 ? (unsigned)atoi(argv[1]) : 1u;
  const int rounds = argc > 2 ? atoi(argv[2]) : 300;
  std::mt19937 rng(seed);
  for (int depth : {1, 2, 5, 16}) {
    SuffixTree tree(depth);
    std::vector<std::vector<int32_t>> seqs(12);
    std::vector<bool> live(12, false);
    for (int r = 0; r < rounds; ++r) {
      const int id = (int)(rng() % seqs.size());
      const unsigned op = rng() % 10;
      if (op < 6) {                      // grow (small alphabet: plenty of shared substrings)
        const int n = 1 + (int)(rng() % 9);
        std::vector<int32_t> t(n);
        for (auto& x : t) x = (int32_t)(rng() % 4);
        if (rng() % 2) {
          tree.extend(id, t.data(), t.size());
        } else {
          for (int32_t x : t) tree.append(id, x);
        }
        seqs[id].insert(seqs[id].end(), t.begin(), t.end());
        live[id] = true;
      } else if (op < 8) {               // drop
        tree.remove(id);
        seqs[id].clear();
        live[id] = false;
      } else {                           // draft from a context taken out of a live sequence
        std::vector<int32_t> ctx;
        if (live[id] && !seqs[id].empty()) {
          const size_t a = rng() % seqs[id].size();
          ctx.assign(seqs[id].begin() + a, seqs[id].end());
        } else {
          ctx = {(int32_t)(rng() % 4), (int32_t)(rng() % 4)};
        }
        for (bool as_tree : {false, true}) {
          Draft d = tree.speculate(ctx.data(), ctx.size(), 1 + (int)(rng() % 8), 2.0f, 1.0f, 0.05f,
                                   as_tree);
          if (d.token_ids.size() != d.parents.size() || d.token_ids.size() != d.probs.size()) {
            fprintf(stderr, "draft arrays of different length\n");
            return 1;
          }
          for (size_t i = 0; i < d.parents.size(); ++i)
            if (d.parents[i] >= (int32_t)i) {
              fprintf(stderr, "draft parent after child\n");
              return 1;
            }
        }
      }
      const std::string err = tree.check_integrity();
      if (!err.empty()) {
        fprintf(stderr, "depth %d round %d: %s\n", depth, r, err.c_str());
        return 1;
      }
    }
    int n_live = 0;
    for (bool b : live) n_live += b ? 1 : 0;
    if (tree.num_seqs() != n_live) {
      fprintf(stderr, "sequence count %d != %d\n", tree.num_seqs(), n_live);
      return 1;
    }
    for (size_t i = 0; i < seqs.size(); ++i) tree.remove((int)i);
    if (tree.num_nodes() != 1) {
      fprintf(stderr, "nodes left after removing everything: %zu\n", tree.num_nodes());
      return 1;
    }
  }
  printf("ok\n");
  return 0;
}
