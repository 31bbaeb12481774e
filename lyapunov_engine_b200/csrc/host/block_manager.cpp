#include "block_manager.hpp"

#include <algorithm>
#include <sstream>
#include <stdexcept>

namespace lyapunov::host {

BlockSpaceManager::BlockSpaceManager(int num_blocks, int block_size, bool)
    : BlockSpaceManager(std::vector<CacheGroupSpec>{CacheGroupSpec{block_size, 0, num_blocks}}, 0) {}

BlockSpaceManager::BlockSpaceManager(std::vector<CacheGroupSpec> groups, int num_state_slots)
    : groups_(std::move(groups)), num_state_slots_(num_state_slots) {
  for (const auto &g : groups_) {
    if (g.block_size < 1) throw std::invalid_argument("BlockSpaceManager: block_size must be >= 1");
    if (g.num_blocks < 0) throw std::invalid_argument("BlockSpaceManager: num_blocks must be >= 0");
    if (g.window < 0) throw std::invalid_argument("BlockSpaceManager: window must be >= 0");
  }
  if (num_state_slots_ < 0) throw std::invalid_argument("BlockSpaceManager: num_state_slots must be >= 0");
  reset();
}

void BlockSpaceManager::reset() {
  free_.assign(groups_.size(), {});
  ref_counts_.clear();
  ever_used_.clear();
  for (size_t g = 0; g < groups_.size(); ++g) {
    ref_counts_.emplace_back(groups_[g].num_blocks, 0);
    ever_used_.emplace_back(groups_[g].num_blocks, 0);
    for (int i = 0; i < groups_[g].num_blocks; ++i) free_[g].push_back(i);
  }
  free_slots_.clear();
  for (int i = 0; i < num_state_slots_; ++i) free_slots_.push_back(i);
  for (auto &kv : holders_) {
    kv.second->mutable_block_tables().clear();
    kv.second->set_state_slot(-1);
  }
  holders_.clear();
}

bool BlockSpaceManager::can_grow(const SequencePtr &seq, size_t num_tokens) const {
  const auto &tables = seq->get_block_tables();
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int have = g < tables.size() ? static_cast<int>(tables[g].size()) : 0;
    const int need = pages_for(static_cast<int>(g), num_tokens) - have;
    if (need > static_cast<int>(free_[g].size())) return false;
  }
  if (num_state_slots_ > 0 && seq->get_state_slot() < 0 && free_slots_.empty()) return false;
  return true;
}

size_t BlockSpaceManager::max_growth(const SequencePtr &seq, size_t num_tokens) const {
  if (num_state_slots_ > 0 && seq->get_state_slot() < 0 && free_slots_.empty()) return 0;
  const auto &tables = seq->get_block_tables();
  size_t best = num_tokens;
  for (size_t g = 0; g < groups_.size(); ++g) {
    const size_t have = g < tables.size() ? tables[g].size() : 0;
    const size_t room = (have + free_[g].size()) * static_cast<size_t>(groups_[g].block_size);
    best = std::min(best, room);
  }
  return best;
}

bool BlockSpaceManager::grow(const SequencePtr &seq, size_t num_tokens) {
  if (!can_grow(seq, num_tokens)) return false;
  auto &tables = seq->mutable_block_tables();
  if (tables.size() < groups_.size()) tables.resize(groups_.size());
  for (size_t g = 0; g < groups_.size(); ++g) {
    const int want = pages_for(static_cast<int>(g), num_tokens);
    while (static_cast<int>(tables[g].size()) < want) {
      const int32_t page = free_[g].front();
      free_[g].pop_front();
      ref_counts_[g][page] = 1;
      ++num_allocations_;
      if (ever_used_[g][page]) ++num_reuses_;
      ever_used_[g][page] = 1;
      tables[g].push_back(page);
    }
  }
  if (num_state_slots_ > 0 && seq->get_state_slot() < 0) {
    seq->set_state_slot(free_slots_.front());
    free_slots_.pop_front();
  }
  holders_[seq->get_seq_id()] = seq;
  return true;
}

void BlockSpaceManager::release_page(int g, int32_t page) {
  if (page < 0 || page >= groups_[g].num_blocks) throw std::logic_error("BlockSpaceManager: page id out of range");
  if (ref_counts_[g][page] <= 0) throw std::logic_error("BlockSpaceManager: page freed twice");
  if (--ref_counts_[g][page] == 0) free_[g].push_back(page);
}

int BlockSpaceManager::release_passed(const SequencePtr &seq) {
  auto &tables = seq->mutable_block_tables();
  int released = 0;
  const int64_t computed = static_cast<int64_t>(seq->get_num_computed_tokens());
  for (size_t g = 0; g < groups_.size() && g < tables.size(); ++g) {
    const int window = groups_[g].window;
    if (window <= 0) continue;
    // The next query stands at position `computed` and reads keys from
    // computed - window + 1 on; pages wholly below that are dead.
    const int64_t first_needed = computed - window + 1;
    if (first_needed <= 0) continue;
    const int64_t dead_pages = first_needed / groups_[g].block_size;
    for (int64_t i = 0; i < dead_pages && i < static_cast<int64_t>(tables[g].size()); ++i) {
      if (tables[g][i] >= 0) {
        release_page(static_cast<int>(g), tables[g][i]);
        tables[g][i] = -1;
        ++released;
      }
    }
  }
  return released;
}

void BlockSpaceManager::free(const SequencePtr &seq) {
  auto &tables = seq->mutable_block_tables();
  for (size_t g = 0; g < tables.size() && g < groups_.size(); ++g) {
    for (int32_t page : tables[g]) {
      if (page >= 0) release_page(static_cast<int>(g), page);
    }
  }
  tables.clear();
  if (seq->get_state_slot() >= 0) {
    free_slots_.push_back(seq->get_state_slot());
    seq->set_state_slot(-1);
  }
  holders_.erase(seq->get_seq_id());
}

void BlockSpaceManager::fork(const SequencePtr &parent, const SequencePtr &child) {
  if (!child->get_block_tables().empty()) throw std::invalid_argument("fork: the child already holds pages");
  const auto &ptables = parent->get_block_tables();
  size_t shared_tokens = std::min(parent->get_num_computed_tokens(), child->get_total_len());
  for (size_t g = 0; g < groups_.size(); ++g) {
    const size_t bs = static_cast<size_t>(groups_[g].block_size);
    shared_tokens = shared_tokens / bs * bs;
  }
  // Every group must share the same number of tokens; shrink until all agree.
  for (bool changed = true; changed;) {
    changed = false;
    for (size_t g = 0; g < groups_.size(); ++g) {
      const size_t bs = static_cast<size_t>(groups_[g].block_size);
      if (shared_tokens % bs) { shared_tokens = shared_tokens / bs * bs; changed = true; }
    }
  }
  auto &ctables = child->mutable_block_tables();
  ctables.assign(groups_.size(), {});
  for (size_t g = 0; g < groups_.size() && g < ptables.size(); ++g) {
    const size_t pages = shared_tokens / static_cast<size_t>(groups_[g].block_size);
    for (size_t i = 0; i < pages; ++i) {
      if (ptables[g][i] < 0) {
        ctables.clear();
        throw std::invalid_argument("fork: the parent has already given back pages a window passed");
      }
    }
    for (size_t i = 0; i < pages; ++i) {
      ++ref_counts_[g][ptables[g][i]];
      ctables[g].push_back(ptables[g][i]);
    }
  }
  child->set_num_computed_tokens(shared_tokens);
  holders_[child->get_seq_id()] = child;
}

void BlockSpaceManager::allocate(const SequencePtr &seq) {
  if (!grow(seq, seq->get_total_len()))
    throw std::runtime_error("Out of memory: insufficient free blocks in BlockSpaceManager");
}

void BlockSpaceManager::append_slot(const SequencePtr &seq) {
  if (!grow(seq, seq->get_total_len()))
    throw std::runtime_error("Out of memory: no free block available to append a slot");
}

std::string BlockSpaceManager::audit() const {
  std::ostringstream err;
  for (size_t g = 0; g < groups_.size(); ++g) {
    std::vector<int> held(groups_[g].num_blocks, 0), in_free(groups_[g].num_blocks, 0);
    for (int32_t page : free_[g]) {
      if (page < 0 || page >= groups_[g].num_blocks) { err << "group " << g << ": free list holds bad id " << page; return err.str(); }
      if (++in_free[page] > 1) { err << "group " << g << ": page " << page << " is in the free list twice"; return err.str(); }
    }
    for (const auto &kv : holders_) {
      const auto &tables = kv.second->get_block_tables();
      if (g >= tables.size()) continue;
      for (int32_t page : tables[g]) {
        if (page < 0) continue;
        if (page >= groups_[g].num_blocks) { err << "group " << g << ": request " << kv.first << " holds bad id " << page; return err.str(); }
        ++held[page];
      }
    }
    for (int page = 0; page < groups_[g].num_blocks; ++page) {
      if (held[page] != ref_counts_[g][page]) {
        err << "group " << g << ": page " << page << " is held by " << held[page] << " block tables but its reference count is " << ref_counts_[g][page];
        return err.str();
      }
      if (held[page] > 0 && in_free[page]) { err << "group " << g << ": page " << page << " is held and free at once"; return err.str(); }
      if (held[page] == 0 && !in_free[page]) { err << "group " << g << ": page " << page << " is lost (neither held nor free)"; return err.str(); }
    }
  }
  std::vector<int> slot_use(num_state_slots_, 0);
  for (int32_t s : free_slots_) {
    if (s < 0 || s >= num_state_slots_ || ++slot_use[s] > 1) { err << "state slot " << s << " is free twice or out of range"; return err.str(); }
  }
  for (const auto &kv : holders_) {
    const int32_t s = kv.second->get_state_slot();
    if (s < 0) continue;
    if (s >= num_state_slots_ || ++slot_use[s] > 1) { err << "state slot " << s << " is held twice, or held and free"; return err.str(); }
  }
  for (int s = 0; s < num_state_slots_; ++s) {
    if (slot_use[s] != 1) { err << "state slot " << s << " is lost"; return err.str(); }
  }
  return "";
}

}  // namespace lyapunov::host
