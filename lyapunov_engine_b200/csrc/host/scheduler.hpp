// Continuous scheduler: every step it lets each running request go on (one
// decoded token, or the next portion of its prompt), then admits waiting
// requests, all under one token budget, and builds the batch that the step
// function runs.
//
// The reference's ContinuousScheduler (csrc/include/engine/scheduler.hpp:12-53,
// csrc/engine/scheduler.cpp:40-138) runs either whole prompts or decode steps,
// never both, admits only when nothing runs, and has no portions.  Kept from
// it: the names, first-come first-served admission, the finish rules (an
// end-of-sequence id unless ignore_eos, max_tokens) and pre-emption by
// recomputation, with the pre-empted request at the front of the queue.
//
// When pages run out (decided here, tested in tests/test_scheduler.py):
//   1. a prompt portion is shortened to the tokens that still fit;
//   2. if a running request cannot get room for even one token, the request
//      admitted last is pre-empted (its pages and state slot are given back,
//      it is recomputed later over prompt and output alike) until there is
//      room, never a request that already has its tokens in this step;
//   3. if the request is the only one that holds pages and still cannot grow,
//      the pool is too small for it: it fails with an error, nothing hangs;
//   4. waiting requests are not admitted while the head of the queue does not
//      fit (no overtaking).
#pragma once

#include <deque>
#include <memory>
#include <string>
#include <vector>

#include "block_manager.hpp"
#include "sequence.hpp"

namespace lyapunov::host {

struct SchedulerConfig {
  int max_num_seqs{256};
  int max_num_batched_tokens{4096};
  int max_model_len{4096};
  // The reference has a single eos_token_id fixed at 128001; here the ids come
  // from the model's configuration and there may be several or none.
  std::vector<int32_t> eos_token_ids{};
  // The longest portion of one prompt in one step; 0: the token budget alone.
  int max_prefill_chunk{0};
};

// Tokens [start, start + count) of one request in one step.  `want` lists the
// places among them (0 .. count-1) whose logits the step returns.
// `ahead` = 1: the entry belongs to a step that is launched before the result of
// the step before it has been read (schedule_ahead): the request's recorded
// state lags one token behind, and the entry's token is not known on the host
// yet (the device passes it on).
struct StepEntry {
  SequencePtr seq;
  int start{0};
  int count{0};
  std::vector<int32_t> want;
  int ahead{0};
};

struct SchedulerOutputs {
  std::vector<StepEntry> entries;
  std::vector<SequencePtr> scheduled_seqs;  // entries[i].seq
  std::vector<SequencePtr> sampled_seqs;    // those whose next token is sampled, in entry order
  std::vector<SequencePtr> preempted_seqs;
  std::vector<SequencePtr> finished_seqs;   // failed during scheduling
  bool is_prefill{false};                   // some entry is a prompt portion
  int num_batched_tokens{0};
};

struct SchedulerStats {
  uint64_t steps{0};
  uint64_t prefill_tokens{0};
  uint64_t decode_tokens{0};
  uint64_t preemptions{0};
  uint64_t failed{0};
};

class ContinuousScheduler {
public:
  ContinuousScheduler(const SchedulerConfig &config, std::shared_ptr<BlockSpaceManager> block_manager);

  void add_sequence(SequencePtr seq);
  void abort_sequence(int64_t seq_id);
  bool has_unfinished_sequences() const { return !waiting_.empty() || !running_.empty(); }
  int get_num_waiting_sequences() const { return static_cast<int>(waiting_.size()); }
  int get_num_running_sequences() const { return static_cast<int>(running_.size()); }

  SchedulerOutputs schedule();
  // The step after `launched` (a step of single decoded tokens whose result has
  // not been read yet), built without that result: every request goes on by one
  // more token.  Empty (no entries) when that cannot be known to be the next
  // step: a request waits for admission, `launched` held a prompt portion or
  // pre-empted, a request reaches max_tokens or max_model_len with the token
  // still to come, or a page is missing.  A request that ends for another
  // reason (an end-of-sequence token) has one token too many computed, which
  // post_step ignores.
  SchedulerOutputs schedule_ahead(const SchedulerOutputs &launched);
  // `next_tokens[i]` is the token sampled for outputs.sampled_seqs[i].  Steps
  // are given back in the order in which they were scheduled.
  void post_step(const SchedulerOutputs &outputs, const std::vector<int32_t> &next_tokens);

  const SchedulerStats &get_stats() const { return stats_; }
  const SchedulerConfig &get_config() const { return config_; }

private:
  void preempt(const SequencePtr &seq, SchedulerOutputs &out);
  void fail(const SequencePtr &seq, const std::string &why, SchedulerOutputs &out);
  bool is_eos(int32_t token) const;

  SchedulerConfig config_;
  std::shared_ptr<BlockSpaceManager> block_manager_;
  std::deque<SequencePtr> waiting_;
  std::vector<SequencePtr> running_;  // in order of admission
  SchedulerStats stats_;
};

}  // namespace lyapunov::host
