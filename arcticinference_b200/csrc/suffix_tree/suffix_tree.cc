#include "suffix_tree.h"

#include <algorithm>
#include <cassert>
#include <cmath>
#include <queue>
#include <stdexcept>
#include <unordered_set>

namespace ab200 {

SuffixTree::SuffixTree(int32_t max_depth) : max_depth_(max_depth) {
  if (max_depth < 1) throw std::invalid_argument("max_depth must be >= 1");
  root_ = new_node();
}

SuffixTree::~SuffixTree() {
  free_subtree(root_);
  for (Node* n : node_pool_) delete n;
  for (Group* g : group_pool_) delete g;
}

SuffixTree::Node* SuffixTree::new_node() {
  ++num_nodes_;
  if (node_pool_.empty()) return new Node();
  Node* n = node_pool_.back();
  node_pool_.pop_back();
  return n;
}

void SuffixTree::free_node(Node* n) {
  --num_nodes_;
  n->children.clear();
  n->endpoints.clear();
  n->count = 0;
  n->token = n->length = n->ref_idx = 0;
  n->ref = nullptr;
  n->parent = n->head_child = n->tail_child = n->next_sibling = n->prev_sibling = nullptr;
  n->group = nullptr;
  node_pool_.push_back(n);
}

SuffixTree::Group* SuffixTree::new_group(Node* head, Node* tail) {
  if (group_pool_.empty()) return new Group{head, tail};
  Group* g = group_pool_.back();
  group_pool_.pop_back();
  g->head = head;
  g->tail = tail;
  return g;
}

void SuffixTree::free_group(Group* g) { group_pool_.push_back(g); }

SuffixTree::Seq& SuffixTree::seq_for(int32_t seq_id) {
  Seq& s = seqs_[seq_id];
  s.id = seq_id;
  return s;
}

void SuffixTree::free_subtree(Node* n) {
  std::vector<Node*> stack{n};
  while (!stack.empty()) {
    Node* x = stack.back();
    stack.pop_back();
    for (Node* c = x->head_child; c != nullptr; c = c->next_sibling) stack.push_back(c);
    // groups are owned by their head member
    if (x->group != nullptr && x->group->head == x) free_group(x->group);
    free_node(x);
  }
}

// ------------------------------------------------------------------ sibling list
// Invariant: the children of a node form a list ordered by count, descending; runs of equal
// count share a Group that knows the run's first and last member. The Group object is owned
// by (deleted through) whichever member is its head at the time.

void SuffixTree::link_child(Node* parent, Node* child) {
  // find the last sibling whose count is >= child's; new children (count 1) end up at the tail
  Node* pos = parent->tail_child;
  while (pos != nullptr && pos->count < child->count) pos = pos->group->head->prev_sibling;
  // insert after `pos` (nullptr: at the head)
  Node* next = pos ? pos->next_sibling : parent->head_child;
  child->prev_sibling = pos;
  child->next_sibling = next;
  if (pos) pos->next_sibling = child; else parent->head_child = child;
  if (next) next->prev_sibling = child; else parent->tail_child = child;
  if (pos != nullptr && pos->count == child->count) {
    child->group = pos->group;        // pos is the tail of its run
    child->group->tail = child;
  } else if (next != nullptr && next->count == child->count) {
    child->group = next->group;       // cannot happen after the scan above, kept for safety
    child->group->head = child;
  } else {
    child->group = new_group(child, child);
  }
}

void SuffixTree::unlink_child(Node* parent, Node* child) {
  Group* g = child->group;
  if (g->head == child && g->tail == child) {
    free_group(g);
  } else if (g->head == child) {
    g->head = child->next_sibling;
  } else if (g->tail == child) {
    g->tail = child->prev_sibling;
  }
  if (child->prev_sibling) child->prev_sibling->next_sibling = child->next_sibling;
  else parent->head_child = child->next_sibling;
  if (child->next_sibling) child->next_sibling->prev_sibling = child->prev_sibling;
  else parent->tail_child = child->prev_sibling;
  child->prev_sibling = child->next_sibling = nullptr;
  child->group = nullptr;
}

void SuffixTree::replace_child(Node* parent, Node* old_child, Node* new_child) {
  // new_child takes old_child's place (same count, same key)
  new_child->prev_sibling = old_child->prev_sibling;
  new_child->next_sibling = old_child->next_sibling;
  if (new_child->prev_sibling) new_child->prev_sibling->next_sibling = new_child;
  else parent->head_child = new_child;
  if (new_child->next_sibling) new_child->next_sibling->prev_sibling = new_child;
  else parent->tail_child = new_child;
  Group* g = old_child->group;
  new_child->group = g;
  if (g->head == old_child) g->head = new_child;
  if (g->tail == old_child) g->tail = new_child;
  old_child->prev_sibling = old_child->next_sibling = nullptr;
  old_child->group = nullptr;
  new_child->parent = parent;
  parent->children.put(new_child->token, new_child);
}

void SuffixTree::bump(Node* child, int delta) {
  Node* parent = child->parent;
  Group* g = child->group;
  const int64_t target = child->count + delta;
  if (g->head == child && g->tail == child) {
    // alone in its run: it stays where it is; it may fuse with the neighbouring run
    child->count = target;
    if (delta > 0) {
      Node* prev = child->prev_sibling;
      if (prev != nullptr && prev->count == target) {
        free_group(g);
        child->group = prev->group;
        child->group->tail = child;
      }
    } else {
      Node* next = child->next_sibling;
      if (next != nullptr && next->count == target) {
        free_group(g);
        child->group = next->group;
        child->group->head = child;
      }
    }
    return;
  }
  // leave the run, then re-enter just above its head (+1) or just below its tail (-1)
  Node* anchor;  // insert after this node (nullptr = list head)
  if (delta > 0) {
    anchor = (g->head == child ? child->next_sibling : g->head)->prev_sibling;
    if (anchor == child) anchor = child->prev_sibling;
  } else {
    anchor = (g->tail == child) ? child->prev_sibling : g->tail;
  }
  unlink_child(parent, child);
  child->count = target;
  Node* next = anchor ? anchor->next_sibling : parent->head_child;
  child->prev_sibling = anchor;
  child->next_sibling = next;
  if (anchor) anchor->next_sibling = child; else parent->head_child = child;
  if (next) next->prev_sibling = child; else parent->tail_child = child;
  if (anchor != nullptr && anchor->count == target) {
    child->group = anchor->group;
    child->group->tail = child;
  } else if (next != nullptr && next->count == target) {
    child->group = next->group;
    child->group->head = child;
  } else {
    child->group = new_group(child, child);
  }
}

// ------------------------------------------------------------------ structure edits
SuffixTree::Node* SuffixTree::split_first(Node* c) {
  Node* parent = c->parent;
  Node* m = new_node();
  m->token = c->token;
  m->length = 1;
  m->ref = c->ref;
  m->ref_idx = c->ref_idx;
  m->count = c->count;
  replace_child(parent, c, m);
  c->ref_idx += 1;
  c->length -= 1;
  c->token = edge(c)[0];
  c->parent = m;
  m->children.put(c->token, c);
  link_child(m, c);
  return m;
}

void SuffixTree::maybe_merge(Node* p) {
  if (p == root_ || p->children.size() != 1 || !p->endpoints.empty()) return;
  Node* c = p->head_child;
  if (c->count != p->count) return;
  // c absorbs p: every string through c came through p, so c's witness covers p's edge
  unlink_child(p, c);
  c->token = p->token;
  c->length += p->length;
  c->ref_idx -= p->length;
  replace_child(p->parent, p, c);
  p->children.clear();
  p->head_child = p->tail_child = nullptr;
  free_node(p);
}

SuffixTree::Node* SuffixTree::advance(Seq& seq, Node* at, int32_t token, int32_t end_idx) {
  const int32_t seq_id = seq.id;
  // A leaf that only this sequence's growing string reaches is simply made one token longer:
  // its edge is witnessed by this sequence and the new token is the next one there.
  if (at != root_ && at->head_child == nullptr && at->count == 1 && at->ref == &seq &&
      at->ref_idx + at->length == end_idx - 1) {
    int32_t* ep = at->endpoints.find(seq_id);
    if (ep != nullptr && at->endpoints.size() == 1) {
      at->length += 1;
      *ep = end_idx;
      return at;
    }
  }
  if (at != root_) at->endpoints.erase(seq_id);
  Node* res;
  Node** pc = at->children.find(token);
  if (pc != nullptr) {
    Node* c = *pc;
    if (c->length > 1) c = split_first(c);
    bump(c, +1);
    res = c;
  } else {
    res = new_node();
    res->token = token;
    res->length = 1;
    res->ref = &seq;
    res->ref_idx = end_idx - 1;
    res->count = 1;
    res->parent = at;
    at->children.put(token, res);
    link_child(at, res);
  }
  res->endpoints.put(seq_id, end_idx);
  maybe_merge(at);
  return res;
}

void SuffixTree::append(int32_t seq_id, int32_t token) {
  Seq& seq = seq_for(seq_id);
  seq.tokens.push_back(token);
  const int32_t n = (int32_t)seq.tokens.size();
  root_->count += 1;
  seq.active.push_back(root_);
  for (size_t i = 0; i < seq.active.size(); ++i)
    seq.active[i] = advance(seq, seq.active[i], token, n);
  // the oldest growing string has length active.size(); retire it once it is max_depth long
  if ((int32_t)seq.active.size() >= max_depth_) seq.active.erase(seq.active.begin());
}

void SuffixTree::extend(int32_t seq_id, const int32_t* tokens, size_t n) {
  Seq& seq = seq_for(seq_id);
  if (n == 0) return;
  seq.tokens.reserve(seq.tokens.size() + n);
  for (size_t i = 0; i < n; ++i) append(seq_id, tokens[i]);
}

void SuffixTree::remove(int32_t seq_id) {
  auto it = seqs_.find(seq_id);
  if (it == seqs_.end()) return;
  const std::vector<int32_t>& T = it->second.tokens;
  const int32_t n = (int32_t)T.size();
  std::unordered_set<Node*> touched;
  for (int32_t i = 0; i < n; ++i) {
    const int32_t len = std::min(max_depth_, n - i);
    root_->count -= 1;
    Node* node = root_;
    int32_t pos = 0;
    while (pos < len) {
      Node** pc = node->children.find(T[i + pos]);
      if (pc == nullptr) break;  // defensive: the tree does not hold this string
      Node* c = *pc;
      if (c->count == 1) {
        // nothing else passes through c: drop the whole branch
        std::vector<Node*> stack{c};
        while (!stack.empty()) {
          Node* x = stack.back();
          stack.pop_back();
          touched.erase(x);
          for (Node* y = x->head_child; y != nullptr; y = y->next_sibling) stack.push_back(y);
        }
        node->children.erase(c->token);
        unlink_child(node, c);
        c->group = nullptr;
        free_subtree(c);
        touched.insert(node);
        node = nullptr;
        break;
      }
      bump(c, -1);
      pos += c->length;
      node = c;
      touched.insert(c);
    }
    if (node != nullptr && node != root_) node->endpoints.erase(seq_id);
  }
  touched.erase(root_);
  // deepest first, so that a node can borrow a repaired child's witness
  std::vector<std::pair<int32_t, Node*>> order;
  order.reserve(touched.size());
  for (Node* x : touched) {
    int32_t d = 0;
    for (Node* y = x; y != root_; y = y->parent) d += y->length;
    order.emplace_back(d, x);
  }
  std::sort(order.begin(), order.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
  for (auto& [d, x] : order) {
    (void)d;
    if (x->ref != &it->second) continue;
    std::pair<int32_t, int32_t> ep;
    if (x->endpoints.any(&ep) != nullptr) {
      x->ref = &seqs_.at(ep.first);
      x->ref_idx = ep.second - x->length;
    } else if (x->head_child != nullptr) {
      x->ref = x->head_child->ref;
      x->ref_idx = x->head_child->ref_idx - x->length;
    }
  }
  for (auto& [d, x] : order) {
    (void)d;
    maybe_merge(x);
  }
  seqs_.erase(it);
}

// ------------------------------------------------------------------ speculation
bool SuffixTree::match(const int32_t* pattern, size_t n, Match* out) const {
  const Node* node = root_;
  int32_t off = 0;
  for (size_t i = 0; i < n; ++i) {
    const int32_t t = pattern[i];
    if (node == root_ || off == node->length) {
      Node* const* pc = node->children.find(t);
      if (pc == nullptr) return false;
      node = *pc;
      off = 1;
    } else {
      if (edge(node)[off] != t) return false;
      ++off;
    }
  }
  out->node = node;
  out->offset = off;
  return true;
}

void SuffixTree::speculate_path(const Match& m, int32_t budget, float min_prob, Draft* d) const {
  const Node* node = m.node;
  int32_t off = m.offset;
  float prob = 1.f;
  while ((int32_t)d->token_ids.size() < budget) {
    int32_t token;
    if (node != root_ && off < node->length) {
      token = edge(node)[off++];
    } else {
      const Node* c = node->head_child;
      if (c == nullptr) break;
      prob *= (float)c->count / (float)node->count;
      if (prob < min_prob) break;
      node = c;
      off = 1;
      token = c->token;
    }
    d->parents.push_back((int32_t)d->token_ids.size() - 1);
    d->token_ids.push_back(token);
    d->probs.push_back(prob);
    d->score += prob;
  }
}

void SuffixTree::speculate_tree(const Match& m, int32_t budget, float min_prob, Draft* d) const {
  struct Cand {
    float prob;
    const Node* node;
    int32_t off;         // the candidate token is edge(node)[off]
    int32_t parent;      // draft index of the preceding token
    float parent_prob;   // probability of the point the edge hangs from
    bool operator<(const Cand& o) const { return prob < o.prob; }
  };
  std::priority_queue<Cand> pq;
  auto push_first_child = [&](const Node* from, float base, int32_t parent) {
    const Node* c = from->head_child;
    if (c != nullptr) pq.push({base * (float)c->count / (float)from->count, c, 0, parent, base});
  };
  if (m.node != root_ && m.offset < m.node->length) pq.push({1.f, m.node, m.offset, -1, 1.f});
  else push_first_child(m.node, 1.f, -1);
  while (!pq.empty() && (int32_t)d->token_ids.size() < budget) {
    const Cand c = pq.top();
    pq.pop();
    if (c.prob < min_prob) break;
    const int32_t idx = (int32_t)d->token_ids.size();
    d->token_ids.push_back(edge(c.node)[c.off]);
    d->parents.push_back(c.parent);
    d->probs.push_back(c.prob);
    d->score += c.prob;
    // the sibling of an edge's first token competes for the same slot
    if (c.off == 0 && c.node->next_sibling != nullptr) {
      const Node* s = c.node->next_sibling;
      pq.push({c.parent_prob * (float)s->count / (float)c.node->parent->count, s, 0, c.parent,
               c.parent_prob});
    }
    if (c.off + 1 < c.node->length) pq.push({c.prob, c.node, c.off + 1, idx, c.prob});
    else push_first_child(c.node, c.prob, idx);
  }
}

Draft SuffixTree::speculate(const int32_t* context, size_t n, int32_t max_spec_tokens,
                            float max_spec_factor, float max_spec_offset, float min_token_prob,
                            bool use_tree_spec) const {
  Draft best;
  // candidate of the current match length, swapped into `best` when it wins; per thread,
  // because callers may speculate on one tree from several threads
  static thread_local Draft scratch;
  Draft& d = scratch;
  // both buffers hold a full draft from the start: no growth while a candidate is built
  const size_t cap = (size_t)std::max(1, max_spec_tokens);
  best.token_ids.reserve(cap);
  best.parents.reserve(cap);
  best.probs.reserve(cap);
  d.token_ids.reserve(cap);
  d.parents.reserve(cap);
  d.probs.reserve(cap);
  const size_t max_m = std::min(n, (size_t)std::max(1, max_depth_ - 1));
  for (size_t m = 1; m <= max_m; ++m) {
    Match mt;
    if (!match(context + n - m, m, &mt)) break;  // a longer suffix cannot match either
    const int32_t budget = std::min<int32_t>(
        max_spec_tokens, (int32_t)std::floor((double)m * max_spec_factor + max_spec_offset + 1e-6));
    if (budget <= 0) continue;
    d.token_ids.clear();
    d.parents.clear();
    d.probs.clear();
    d.score = 0.f;
    if (use_tree_spec) speculate_tree(mt, budget, min_token_prob, &d);
    else speculate_path(mt, budget, min_token_prob, &d);
    d.match_len = (int32_t)m;
    if (!d.token_ids.empty() && d.score >= best.score) std::swap(best, d);
  }
  return best;
}

// ------------------------------------------------------------------ diagnostics
std::string SuffixTree::check_integrity() const {
  struct Item {
    const Node* node;
    int32_t depth;
  };
  std::vector<Item> stack{{root_, 0}};
  size_t seen = 0;
  while (!stack.empty()) {
    const Item it = stack.back();
    stack.pop_back();
    const Node* x = it.node;
    ++seen;
    if (x != root_) {
      if (x->count <= 0) return "non-positive count";
      if (x->length < 1) return "empty edge";
      if (x->ref == nullptr) return "edge without a witness sequence";
      auto s = seqs_.find(x->ref->id);
      if (s == seqs_.end() || &s->second != x->ref) return "edge refers to a removed sequence";
      if (x->ref_idx < 0 || (size_t)(x->ref_idx + x->length) > s->second.tokens.size())
        return "edge reference out of range";
      if (s->second.tokens[x->ref_idx] != x->token) return "edge key differs from its first token";
      if (it.depth > max_depth_) return "node deeper than max_depth";
      if (x->children.size() == 1 && x->endpoints.empty() && x->head_child->count == x->count)
        return "unmerged chain node";
    }
    int64_t sum = 0;
    uint32_t n = 0;
    const Node* prev = nullptr;
    for (const Node* c = x->head_child; c != nullptr; c = c->next_sibling) {
      if (c->parent != x) return "child with wrong parent";
      if (c->prev_sibling != prev) return "broken sibling back-link";
      if (prev != nullptr && prev->count < c->count) return "siblings not ordered by count";
      if (c->group == nullptr) return "child without group";
      if (prev != nullptr && (prev->count == c->count) != (prev->group == c->group))
        return "group does not match equal-count run";
      if (c->group->head->count != c->count || c->group->tail->count != c->count)
        return "group end with different count";
      Node* const* pc = x->children.find(c->token);
      if (pc == nullptr || *pc != c) return "child table and sibling list disagree";
      sum += c->count;
      ++n;
      prev = c;
      stack.push_back({c, it.depth + c->length});
    }
    if (prev != x->tail_child) return "wrong tail child";
    if (n != x->children.size()) return "child table size differs from list length";
    if (sum > x->count) return "children outnumber their parent";
  }
  if (seen != num_nodes_) return "node count mismatch";
  for (const auto& kv : seqs_)
    for (const Node* a : kv.second.active)
      if (a != root_ && !a->endpoints.contains(kv.first)) return "active string without endpoint";
  return "";
}

size_t SuffixTree::estimate_memory() const {
  size_t total = sizeof(*this) + num_nodes_ * (sizeof(Node) + sizeof(Group) / 2);
  std::vector<const Node*> stack{root_};
  while (!stack.empty()) {
    const Node* x = stack.back();
    stack.pop_back();
    total += x->children.heap_bytes() + x->endpoints.heap_bytes();
    for (const Node* c = x->head_child; c != nullptr; c = c->next_sibling) stack.push_back(c);
  }
  for (const auto& kv : seqs_)
    total += kv.second.tokens.capacity() * sizeof(int32_t) +
             kv.second.active.capacity() * sizeof(Node*) + 64;
  return total;
}

}  // namespace ab200
