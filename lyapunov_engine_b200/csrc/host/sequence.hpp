// One request as the host runtime sees it: its tokens, how many of them are
// already in the cache, its pages in every cache group and its state slot.
//
// The reference's Sequence (csrc/include/engine/sequence.hpp:28-88) holds one
// block table and a counter of computed tokens that only post_step writes.
// Here the counter drives everything: a step may bring any number of the
// not-yet-computed tokens, so prompts are cut into portions and a pre-empted
// request is recomputed over prompt and output alike.
#pragma once

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace lyapunov::host {

enum class SequenceStatus {
  WAITING,
  RUNNING,
  FINISHED_STOPPED,
  FINISHED_LENGTH_CAPPED,
  FINISHED_ABORTED,
  FINISHED_FAILED,
};

// Same names and defaults as the reference
// (python/lyapunov_engine/engine/sampling.py:6-12), plus a seed.
struct SamplingParams {
  float temperature{1.0f};
  float top_p{1.0f};
  int top_k{-1};
  int max_tokens{128};
  bool ignore_eos{false};
  uint64_t seed{0};
};

class Sequence {
public:
  Sequence(int64_t seq_id, std::vector<int32_t> prompt_tokens, SamplingParams sampling)
      : seq_id_(seq_id), prompt_(std::move(prompt_tokens)), sampling_(sampling) {}

  int64_t get_seq_id() const { return seq_id_; }
  SequenceStatus get_status() const { return status_; }
  void set_status(SequenceStatus s) { status_ = s; }
  const SamplingParams &get_sampling_params() const { return sampling_; }

  const std::vector<int32_t> &get_prompt_tokens() const { return prompt_; }
  const std::vector<int32_t> &get_output_tokens() const { return output_; }
  size_t get_prompt_len() const { return prompt_.size(); }
  size_t get_output_len() const { return output_.size(); }
  size_t get_total_len() const { return prompt_.size() + output_.size(); }
  int32_t token_at(size_t i) const { return i < prompt_.size() ? prompt_[i] : output_[i - prompt_.size()]; }
  int32_t get_last_token_id() const { return output_.empty() ? prompt_.back() : output_.back(); }
  void append_token_id(int32_t t) { output_.push_back(t); }
  // Trace replay feeds tokens that nobody sampled: they extend the prompt.
  void extend_prompt(const std::vector<int32_t> &tokens) {
    prompt_.insert(prompt_.end(), tokens.begin(), tokens.end());
  }

  bool is_finished() const {
    return status_ == SequenceStatus::FINISHED_STOPPED || status_ == SequenceStatus::FINISHED_LENGTH_CAPPED ||
           status_ == SequenceStatus::FINISHED_ABORTED || status_ == SequenceStatus::FINISHED_FAILED;
  }
  const char *finish_reason() const {
    switch (status_) {
      case SequenceStatus::FINISHED_STOPPED: return "stop";
      case SequenceStatus::FINISHED_LENGTH_CAPPED: return "length";
      case SequenceStatus::FINISHED_ABORTED: return "abort";
      case SequenceStatus::FINISHED_FAILED: return "error";
      default: return "";
    }
  }

  // Tokens whose keys, values or state are in the cache.
  size_t get_num_computed_tokens() const { return num_computed_; }
  void set_num_computed_tokens(size_t n) { num_computed_ = n; }

  // Pages per cache group; -1 marks a page already given back (a window has
  // passed it).  Group 0 is what get_block_table() returns.
  const std::vector<std::vector<int32_t>> &get_block_tables() const { return tables_; }
  std::vector<std::vector<int32_t>> &mutable_block_tables() { return tables_; }
  std::vector<int32_t> get_block_table() const { return tables_.empty() ? std::vector<int32_t>{} : tables_[0]; }

  int32_t get_state_slot() const { return state_slot_; }
  void set_state_slot(int32_t s) { state_slot_ = s; }

  int get_num_preemptions() const { return num_preemptions_; }
  void count_preemption() { ++num_preemptions_; }
  const std::string &get_error() const { return error_; }
  void set_error(std::string e) { error_ = std::move(e); }

private:
  int64_t seq_id_;
  std::vector<int32_t> prompt_;
  std::vector<int32_t> output_;
  SamplingParams sampling_;
  SequenceStatus status_{SequenceStatus::WAITING};
  size_t num_computed_{0};
  std::vector<std::vector<int32_t>> tables_;
  int32_t state_slot_{-1};
  int num_preemptions_{0};
  std::string error_;
};

using SequencePtr = std::shared_ptr<Sequence>;

}  // namespace lyapunov::host
