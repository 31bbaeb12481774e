// Paged cache manager: which page of which pool holds which tokens of which
// request, and which slot holds its fixed-size state.
//
// The reference's BlockSpaceManager (csrc/include/engine/block_manager.hpp:14-44,
// csrc/engine/block_manager.cpp:7-101) has one pool, a first-in first-out free
// list, reference counts that never exceed one and gives pages back only when
// a request ends.  This one keeps its names and the first-in first-out order
// (so the order in which pages are used again is reproducible) and adds:
//   * cache groups: layers with different needs (all keys, or a window of
//     them) have pools and block tables of their own;
//   * pages that a window has passed are given back while the request lives;
//   * one arithmetic for prompts, portions and decoded tokens: grow(seq, n)
//     makes room for the first n tokens; it changes nothing when it fails;
//   * slots for per-request state of fixed size, taken with the first page
//     and given back with the last;
//   * fork(), the only way a reference count exceeds one;
//   * audit(), which proves that no page is lost, held twice or freed twice.
#pragma once

#include <cstdint>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#include "sequence.hpp"

namespace lyapunov::host {

struct CacheGroupSpec {
  int block_size{16};
  int window{0};      // 0: every key is kept; w > 0: a query at p reads keys p-w+1 .. p
  int num_blocks{0};  // pages of this group's pool
};

class BlockSpaceManager {
public:
  // One group that keeps every key: the reference's constructor.  The third
  // argument is accepted for compatibility and ignored (no prefix cache).
  BlockSpaceManager(int num_blocks, int block_size = 16, bool enable_prefix_caching = false);
  BlockSpaceManager(std::vector<CacheGroupSpec> groups, int num_state_slots);

  int get_num_groups() const { return static_cast<int>(groups_.size()); }
  const CacheGroupSpec &get_group(int g) const { return groups_.at(g); }
  int get_num_blocks(int g = 0) const { return groups_.at(g).num_blocks; }
  int get_block_size(int g = 0) const { return groups_.at(g).block_size; }
  int get_num_free_blocks(int g = 0) const { return static_cast<int>(free_.at(g).size()); }
  int get_num_used_blocks(int g = 0) const { return get_num_blocks(g) - get_num_free_blocks(g); }
  int get_num_state_slots() const { return num_state_slots_; }
  int get_num_free_state_slots() const { return static_cast<int>(free_slots_.size()); }
  int get_ref_count(int g, int block) const { return ref_counts_.at(g).at(block); }

  // Room for the first `num_tokens` tokens of `seq` in every group (and a
  // state slot if it has none).  All or nothing.
  bool can_grow(const SequencePtr &seq, size_t num_tokens) const;
  bool grow(const SequencePtr &seq, size_t num_tokens);
  // The largest n <= num_tokens for which grow(seq, n) would succeed now.
  size_t max_growth(const SequencePtr &seq, size_t num_tokens) const;
  // Gives back the pages of window groups that no token after
  // seq->get_num_computed_tokens() can read.
  int release_passed(const SequencePtr &seq);
  // Gives back everything the request holds.  Safe to call twice.
  void free(const SequencePtr &seq);
  // `child` shares the full pages of `parent` (reference counts rise); its
  // computed-token count is set to the tokens those pages hold.  Refused when
  // a window has already released pages of the parent.
  void fork(const SequencePtr &parent, const SequencePtr &child);

  // The reference's interface, in terms of the above.
  bool can_allocate(const SequencePtr &seq) const { return can_grow(seq, seq->get_total_len()); }
  void allocate(const SequencePtr &seq);
  bool can_append_slot(const SequencePtr &seq) const { return can_grow(seq, seq->get_total_len()); }
  void append_slot(const SequencePtr &seq);
  void reset();

  // Empty when every page is either free exactly once or held by exactly as
  // many block tables as its reference count says, and the same for slots;
  // otherwise a description of the first inconsistency.
  std::string audit() const;

  uint64_t get_num_allocations() const { return num_allocations_; }
  uint64_t get_num_reuses() const { return num_reuses_; }

private:
  int pages_for(int g, size_t num_tokens) const {
    const int bs = groups_[g].block_size;
    return static_cast<int>((num_tokens + bs - 1) / bs);
  }
  void release_page(int g, int32_t page);

  std::vector<CacheGroupSpec> groups_;
  std::vector<std::deque<int32_t>> free_;
  std::vector<std::vector<int32_t>> ref_counts_;
  std::vector<std::vector<uint8_t>> ever_used_;
  int num_state_slots_{0};
  std::deque<int32_t> free_slots_;
  std::unordered_map<int64_t, SequencePtr> holders_;
  uint64_t num_allocations_{0};
  uint64_t num_reuses_{0};
};

}  // namespace lyapunov::host
