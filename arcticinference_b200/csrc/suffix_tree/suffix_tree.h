// Bounded-depth generalized suffix tree over int32 token ids (host side, C++17).
//
// The tree holds, for every sequence s and every start position i, the string
// s[i : i + max_depth] (shorter at the end of the sequence). Edges are path
// compressed: a node owns `length` tokens that live in some sequence
// (`ref_seq`, `ref_idx`). `count` is the number of stored strings that reach the
// end of the node's edge; a compressed edge is legal only while no stored string
// ends strictly inside it, so the ends of all strings that are still growing sit
// exactly on node boundaries.
//
// Children of a node are kept in a doubly linked list ordered by count
// (descending). Equal counts form a "group" that remembers its first and last
// member, so a +1 / -1 on a child's count re-positions it in O(1).
//
// speculate() matches the longest suffixes of a context against the tree and
// proposes a continuation, either one greedy path or a best-first tree of
// candidates, scored by the sum of the estimated token probabilities.
//
// Same role and observable behaviour as the reference's
// csrc/suffix_decoding/suffix_tree.{h,cc}; the data layout and algorithms here
// are this project's own.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "int32_map.h"

namespace ab200 {

struct Draft {
  std::vector<int32_t> token_ids;
  std::vector<int32_t> parents;  // index of the parent draft token, -1 for roots
  std::vector<float> probs;      // estimated probability of each token (product along its path)
  float score = 0.f;             // sum of probs
  int32_t match_len = 0;         // length of the context suffix that was matched
};

class SuffixTree {
 public:
  explicit SuffixTree(int32_t max_depth);
  ~SuffixTree();
  SuffixTree(const SuffixTree&) = delete;
  SuffixTree& operator=(const SuffixTree&) = delete;

  int32_t max_depth() const { return max_depth_; }
  int32_t num_seqs() const { return (int32_t)seqs_.size(); }
  bool contains(int32_t seq_id) const { return seqs_.count(seq_id) != 0; }

  void append(int32_t seq_id, int32_t token);
  void extend(int32_t seq_id, const int32_t* tokens, size_t n);
  void remove(int32_t seq_id);

  Draft speculate(const int32_t* context, size_t n, int32_t max_spec_tokens, float max_spec_factor,
                  float max_spec_offset, float min_token_prob, bool use_tree_spec) const;

  // Empty string when every invariant holds, else a description of the first violation.
  std::string check_integrity() const;
  size_t estimate_memory() const;
  size_t num_nodes() const { return num_nodes_; }

 private:
  struct Group;
  struct Seq;
  struct Node {
    int64_t count = 0;
    int32_t token = 0;    // first token of the edge (key in the parent's child table)
    int32_t length = 0;   // tokens on the edge
    int32_t ref_idx = 0;
    Seq* ref = nullptr;   // the edge's tokens are ref->tokens[ref_idx .. ref_idx + length)
    Node* parent = nullptr;
    Int32Map<Node*> children;
    Node* head_child = nullptr;  // child with the largest count
    Node* tail_child = nullptr;
    Node* next_sibling = nullptr;
    Node* prev_sibling = nullptr;
    Group* group = nullptr;
    // strings that end exactly at this node: seq id -> index one past the string's last token
    Int32Map<int32_t> endpoints;
  };
  struct Group {
    Node* head;
    Node* tail;
  };
  struct Seq {
    int32_t id = -1;
    std::vector<int32_t> tokens;
    // end nodes of the strings that are still shorter than max_depth, oldest start first
    std::vector<Node*> active;
  };

  Node* new_node();
  void free_node(Node* n);
  Group* new_group(Node* head, Node* tail);
  void free_group(Group* g);
  void free_subtree(Node* n);
  static const int32_t* edge(const Node* n) { return n->ref->tokens.data() + n->ref_idx; }
  Seq& seq_for(int32_t seq_id);

  // sibling-list maintenance
  void link_child(Node* parent, Node* child);            // child->count must be set
  void unlink_child(Node* parent, Node* child);
  void replace_child(Node* parent, Node* old_child, Node* new_child);  // same token and count
  void bump(Node* child, int delta);                     // count += delta (delta = +1 / -1)

  Node* split_first(Node* child);            // cut the first token of child's edge into a new parent
  void maybe_merge(Node* p);                 // fuse p with its only child when nothing ends at p
  Node* advance(Seq& seq, Node* at, int32_t token, int32_t end_idx);

  struct Match {
    const Node* node = nullptr;  // node whose edge the match ends in (or at)
    int32_t offset = 0;          // tokens of node's edge consumed
  };
  bool match(const int32_t* pattern, size_t n, Match* out) const;
  void speculate_path(const Match& m, int32_t budget, float min_prob, Draft* d) const;
  void speculate_tree(const Match& m, int32_t budget, float min_prob, Draft* d) const;

  int32_t max_depth_;
  Node* root_;
  size_t num_nodes_ = 0;
  std::unordered_map<int32_t, Seq> seqs_;   // node-based: a Seq never moves
  // recycled nodes and groups (a sequence that grows by one token touches up to max_depth
  // nodes; going to the allocator for each would dominate the update)
  std::vector<Node*> node_pool_;
  std::vector<Group*> group_pool_;

};

}  // namespace ab200
