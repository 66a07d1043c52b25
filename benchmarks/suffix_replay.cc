// Replay of a recorded (prompt, response) token trace through a suffix tree, entirely in C++
// (no interpreter in the timed loop): a global tree over the responses of the first
// `train` requests and one tree per evaluated request over its prompt and the response so far;
// at every step both trees draft, the higher score wins, the draft is checked against the
// recorded continuation and the accepted tokens plus one bonus token are appended.
//
// The same file builds against this package's tree (default) or, with -DUSE_REFERENCE_TREE and
// the reference's csrc/suffix_decoding on the include path, against the reference's
// SuffixTree, so that both are measured by identical driver code on the same trace
// (the reference's own replay loop: arctic_inference/suffix_decoding/simulator.py:56-111).
//
//   suffix_replay <trace.bin> <max_depth> <max_spec_tokens> <factor> <offset> <min_prob>
// trace.bin: int32 num_requests, train, prompt_len, response_len, then per request the prompt
// tokens followed by the response tokens.
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <vector>

#ifdef USE_REFERENCE_TREE
#include <span>
#include "suffix_tree.h"
static void tree_extend(SuffixTree& t, int id, const int32_t* p, size_t n) {
  t.extend(id, std::span<const int32_t>(p, n));
}
static Draft tree_speculate(SuffixTree& t, const int32_t* c, size_t n, int max_spec, float factor,
                            float offset, float min_prob) {
  return t.speculate(std::span<const int32_t>(c, n), max_spec, factor, offset, min_prob, false);
}
static const char* kWhich = "reference";
#else
#include "suffix_tree.h"
using ab200::Draft;
using ab200::SuffixTree;
static void tree_extend(SuffixTree& t, int id, const int32_t* p, size_t n) { t.extend(id, p, n); }
static Draft tree_speculate(SuffixTree& t, const int32_t* c, size_t n, int max_spec, float factor,
                            float offset, float min_prob) {
  return t.speculate(c, n, max_spec, factor, offset, min_prob, false);
}
static const char* kWhich = "arcticinference_b200";
#endif

using Clock = std::chrono::steady_clock;

int main(int argc, char** argv) {
  if (argc < 7) {
    fprintf(stderr, "usage: %s trace.bin max_depth max_spec factor offset min_prob\n", argv[0]);
    return 2;
  }
  FILE* f = fopen(argv[1], "rb");
  if (!f) return 2;
  int32_t hdr[4];
  if (fread(hdr, 4, 4, f) != 4) return 2;
  const int R = hdr[0], train = hdr[1], P = hdr[2], L = hdr[3];
  std::vector<int32_t> data((size_t)R * (P + L));
  if (fread(data.data(), 4, data.size(), f) != data.size()) return 2;
  fclose(f);
  const int depth = atoi(argv[2]), max_spec = atoi(argv[3]);
  const float factor = (float)atof(argv[4]), offset = (float)atof(argv[5]),
              min_prob = (float)atof(argv[6]);

  SuffixTree global(depth);
  for (int i = 0; i < train; ++i) tree_extend(global, i, &data[(size_t)i * (P + L) + P], L);

  double spec_s = 0, update_s = 0;
  long long steps = 0, drafted = 0, accepted = 0, out_tokens = 0;
  for (int i = train; i < R; ++i) {
    const int32_t* prompt = &data[(size_t)i * (P + L)];
    const int32_t* resp = prompt + P;
    auto t0 = Clock::now();
    auto local = std::make_unique<SuffixTree>(depth);
    tree_extend(*local, 0, prompt, P);
    tree_extend(*local, 0, resp, 1);
    tree_extend(global, i, resp, 1);
    update_s += std::chrono::duration<double>(Clock::now() - t0).count();
    int pos = 1;
    while (pos < L) {
      const int have = P + pos;
      const int n_ctx = have < depth ? have : depth;
      const int32_t* ctx = prompt + have - n_ctx;
      const int budget = max_spec < L - pos - 1 ? max_spec : L - pos - 1;
      t0 = Clock::now();
      Draft a = tree_speculate(*local, ctx, n_ctx, budget, factor, offset, min_prob);
      Draft b = tree_speculate(global, ctx, n_ctx, budget, factor, offset, min_prob);
      const Draft& d = b.score > a.score ? b : a;
      spec_s += std::chrono::duration<double>(Clock::now() - t0).count();
      int acc = 0;   // path drafts: token k continues token k - 1
      while (acc < (int)d.token_ids.size() && pos + acc < L && d.token_ids[acc] == resp[pos + acc])
        ++acc;
      int n_new = acc + 1;
      if (pos + n_new > L) n_new = L - pos;
      t0 = Clock::now();
      tree_extend(*local, 0, resp + pos, n_new);
      tree_extend(global, i, resp + pos, n_new);
      update_s += std::chrono::duration<double>(Clock::now() - t0).count();
      ++steps;
      drafted += (long long)d.token_ids.size();
      accepted += acc;
      pos += n_new;
    }
    out_tokens += L - 1;
  }
  printf("{\"tree\": \"%s\", \"num_steps\": %lld, \"num_output_tokens\": %lld, "
         "\"mean_accepted_len\": %.4f, \"accept_rate\": %.4f, \"spec_us_per_step\": %.3f, "
         "\"update_us_per_token\": %.3f}\n",
         kWhich, steps, out_tokens, (double)out_tokens / (double)(steps ? steps : 1),
         (double)accepted / (double)(drafted ? drafted : 1), 1e6 * spec_s / (double)(steps ? steps : 1),
         1e6 * update_s / (double)(out_tokens ? out_tokens : 1));
  return 0;
}
