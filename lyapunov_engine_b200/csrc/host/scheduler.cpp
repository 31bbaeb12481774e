#include "scheduler.hpp"

#include <algorithm>
#include <stdexcept>

#include "logging.hpp"

namespace lyapunov::host {

ContinuousScheduler::ContinuousScheduler(const SchedulerConfig &config, std::shared_ptr<BlockSpaceManager> block_manager)
    : config_(config), block_manager_(std::move(block_manager)) {
  if (config_.max_num_seqs < 1) throw std::invalid_argument("SchedulerConfig: max_num_seqs must be >= 1");
  if (config_.max_num_batched_tokens < 1) throw std::invalid_argument("SchedulerConfig: max_num_batched_tokens must be >= 1");
  if (config_.max_model_len < 1) throw std::invalid_argument("SchedulerConfig: max_model_len must be >= 1");
}

void ContinuousScheduler::add_sequence(SequencePtr seq) {
  if (seq->get_prompt_len() == 0) throw std::invalid_argument("add_sequence: the prompt is empty");
  seq->set_status(SequenceStatus::WAITING);
  waiting_.push_back(std::move(seq));
}

void ContinuousScheduler::abort_sequence(int64_t seq_id) {
  for (auto it = running_.begin(); it != running_.end(); ++it) {
    if ((*it)->get_seq_id() == seq_id) {
      (*it)->set_status(SequenceStatus::FINISHED_ABORTED);
      block_manager_->free(*it);
      running_.erase(it);
      return;
    }
  }
  for (auto it = waiting_.begin(); it != waiting_.end(); ++it) {
    if ((*it)->get_seq_id() == seq_id) {
      (*it)->set_status(SequenceStatus::FINISHED_ABORTED);
      block_manager_->free(*it);
      waiting_.erase(it);
      return;
    }
  }
}

bool ContinuousScheduler::is_eos(int32_t token) const {
  return std::find(config_.eos_token_ids.begin(), config_.eos_token_ids.end(), token) != config_.eos_token_ids.end();
}

void ContinuousScheduler::preempt(const SequencePtr &seq, SchedulerOutputs &out) {
  block_manager_->free(seq);
  seq->set_num_computed_tokens(0);
  seq->set_status(SequenceStatus::WAITING);
  seq->count_preemption();
  waiting_.push_front(seq);
  out.preempted_seqs.push_back(seq);
  ++stats_.preemptions;
  log(LogLevel::kInfo, "pre-empted request " + std::to_string(seq->get_seq_id()));
}

void ContinuousScheduler::fail(const SequencePtr &seq, const std::string &why, SchedulerOutputs &out) {
  block_manager_->free(seq);
  seq->set_status(SequenceStatus::FINISHED_FAILED);
  seq->set_error(why);
  out.finished_seqs.push_back(seq);
  ++stats_.failed;
  log(LogLevel::kWarn, "request " + std::to_string(seq->get_seq_id()) + " failed: " + why);
}

SchedulerOutputs ContinuousScheduler::schedule() {
  SchedulerOutputs out;
  int budget = config_.max_num_batched_tokens;

  auto portion = [&](const SequencePtr &seq) {
    size_t n = seq->get_total_len() - seq->get_num_computed_tokens();
    n = std::min<size_t>(n, static_cast<size_t>(budget));
    if (config_.max_prefill_chunk > 0) n = std::min<size_t>(n, static_cast<size_t>(config_.max_prefill_chunk));
    return n;
  };
  auto emit = [&](const SequencePtr &seq, size_t count) {
    StepEntry e;
    e.seq = seq;
    e.start = static_cast<int>(seq->get_num_computed_tokens());
    e.count = static_cast<int>(count);
    if (static_cast<size_t>(e.start) + count == seq->get_total_len()) {
      e.want.push_back(e.count - 1);
      out.sampled_seqs.push_back(seq);
    }
    if (count > 1 || static_cast<size_t>(e.start) + count < seq->get_total_len() || seq->get_output_len() == 0) out.is_prefill = true;
    out.entries.push_back(std::move(e));
    out.scheduled_seqs.push_back(seq);
    out.num_batched_tokens += static_cast<int>(count);
    budget -= static_cast<int>(count);
  };

  // 1. Running requests: first those that decode (one token each), then those
  //    still working through a prompt, each group oldest first.
  std::vector<SequencePtr> in_step;
  auto has_entry = [&](const SequencePtr &s) { return std::find(in_step.begin(), in_step.end(), s) != in_step.end(); };
  for (int pass = 0; pass < 2; ++pass) {
    size_t i = 0;
    while (i < running_.size()) {
      SequencePtr seq = running_[i];
      const size_t remaining = seq->get_total_len() - seq->get_num_computed_tokens();
      if ((pass == 0) != (remaining == 1) || has_entry(seq)) { ++i; continue; }
      size_t count = portion(seq);
      if (count == 0) { ++i; continue; }  // the budget is spent; it goes on next step
      const size_t computed = seq->get_num_computed_tokens();
      bool placed = false;
      bool self_is_victim = false;
      while (true) {
        const size_t fits = block_manager_->max_growth(seq, computed + count);
        if (fits > computed) {
          count = fits - computed;
          if (!block_manager_->grow(seq, computed + count)) throw std::logic_error("schedule: grow failed after max_growth");
          placed = true;
          break;
        }
        // The request admitted last that has no tokens in this step yet.
        long v = static_cast<long>(running_.size()) - 1;
        while (v >= 0 && has_entry(running_[static_cast<size_t>(v)])) --v;
        if (v < 0) break;
        SequencePtr victim = running_[static_cast<size_t>(v)];
        if (victim == seq) { self_is_victim = true; break; }
        running_.erase(running_.begin() + v);
        if (static_cast<size_t>(v) < i) --i;
        preempt(victim, out);
      }
      if (placed) {
        emit(seq, count);
        in_step.push_back(seq);
        ++i;
        continue;
      }
      running_.erase(running_.begin() + static_cast<long>(i));
      if (self_is_victim && running_.empty()) {
        fail(seq, "the cache pool is too small for this request: it holds every page it can get and needs another", out);
      } else {
        // Others hold the pages (they already have their tokens in this step,
        // or are older): this one waits and is recomputed.
        preempt(seq, out);
      }
    }
  }

  // 2. Waiting requests, first come first served.
  // Not in a step that pre-empted: the freed pages would go straight back to
  // the request that just lost them.
  while (out.preempted_seqs.empty() && !waiting_.empty() && budget > 0 &&
         static_cast<int>(running_.size()) < config_.max_num_seqs) {
    SequencePtr seq = waiting_.front();
    if (seq->get_total_len() >= static_cast<size_t>(config_.max_model_len)) {
      waiting_.pop_front();
      fail(seq, "the request has " + std::to_string(seq->get_total_len()) + " tokens, max_model_len is " +
                    std::to_string(config_.max_model_len), out);
      continue;
    }
    size_t count = portion(seq);
    const size_t fits = block_manager_->max_growth(seq, count);
    if (fits == 0) {
      if (running_.empty()) {
        waiting_.pop_front();
        fail(seq, "the cache pool has no page or state slot for this request although nothing else runs", out);
        continue;
      }
      break;
    }
    count = std::min(count, fits);
    if (!block_manager_->grow(seq, count)) throw std::logic_error("schedule: grow failed after max_growth");
    waiting_.pop_front();
    seq->set_status(SequenceStatus::RUNNING);
    running_.push_back(seq);
    emit(seq, count);
  }

  ++stats_.steps;
  return out;
}

SchedulerOutputs ContinuousScheduler::schedule_ahead(const SchedulerOutputs &launched) {
  SchedulerOutputs out;
  if (launched.entries.empty() || launched.is_prefill || !launched.preempted_seqs.empty() || !waiting_.empty()) return out;
  if (launched.entries.size() != running_.size() || launched.sampled_seqs.size() != launched.entries.size()) return out;
  for (const auto &e : launched.entries) {
    const SequencePtr &seq = e.seq;
    if (e.count != 1 || e.want.size() != 1 || seq->get_status() != SequenceStatus::RUNNING) return out;
    // with the token that is still to come: the lengths the finish rules of post_step will see
    const size_t total_then = static_cast<size_t>(e.start) + 2;          // tokens of the request after `launched`
    const size_t output_then = total_then - seq->get_prompt_len();
    if (static_cast<int>(output_then) >= seq->get_sampling_params().max_tokens) return out;
    if (total_then >= static_cast<size_t>(config_.max_model_len)) return out;
  }
  // every request needs room for one more token than `launched` gave it
  for (const auto &e : launched.entries)
    if (block_manager_->max_growth(e.seq, static_cast<size_t>(e.start) + 2) < static_cast<size_t>(e.start) + 2) return out;
  for (const auto &e : launched.entries) {
    if (!block_manager_->grow(e.seq, static_cast<size_t>(e.start) + 2)) throw std::logic_error("schedule_ahead: grow failed after max_growth");
    StepEntry next;
    next.seq = e.seq;
    next.start = e.start + 1;
    next.count = 1;
    next.want.push_back(0);
    next.ahead = 1;
    out.entries.push_back(std::move(next));
    out.scheduled_seqs.push_back(e.seq);
    out.sampled_seqs.push_back(e.seq);
    out.num_batched_tokens += 1;
  }
  ++stats_.steps;
  return out;
}

void ContinuousScheduler::post_step(const SchedulerOutputs &outputs, const std::vector<int32_t> &next_tokens) {
  if (outputs.sampled_seqs.size() != next_tokens.size())
    throw std::runtime_error("post_step: " + std::to_string(outputs.sampled_seqs.size()) + " requests were sampled but " +
                             std::to_string(next_tokens.size()) + " tokens were given");
  for (const auto &e : outputs.entries) {
    if (e.seq->is_finished()) continue;  // it ended with the step before, while this one was already running
    e.seq->set_num_computed_tokens(static_cast<size_t>(e.start + e.count));
    if (e.count > 1 || e.want.empty()) stats_.prefill_tokens += static_cast<uint64_t>(e.count);
    else stats_.decode_tokens += 1;
    block_manager_->release_passed(e.seq);
  }
  for (size_t i = 0; i < next_tokens.size(); ++i) {
    const SequencePtr &seq = outputs.sampled_seqs[i];
    if (seq->is_finished()) continue;  // aborted while the step ran
    const int32_t token = next_tokens[i];
    seq->append_token_id(token);
    const auto &sp = seq->get_sampling_params();
    SequenceStatus done = SequenceStatus::RUNNING;
    if (is_eos(token) && !sp.ignore_eos) done = SequenceStatus::FINISHED_STOPPED;
    else if (static_cast<int>(seq->get_output_len()) >= sp.max_tokens) done = SequenceStatus::FINISHED_LENGTH_CAPPED;
    else if (seq->get_total_len() >= static_cast<size_t>(config_.max_model_len)) done = SequenceStatus::FINISHED_LENGTH_CAPPED;
    if (done != SequenceStatus::RUNNING) {
      seq->set_status(done);
      block_manager_->free(seq);
      running_.erase(std::remove(running_.begin(), running_.end(), seq), running_.end());
    }
  }
}

}  // namespace lyapunov::host
