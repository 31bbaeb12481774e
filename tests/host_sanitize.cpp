// Drives the host runtime (cache manager, scheduler, step packing) with random
// traffic in a plain C++ program, so that it can run under the address and
// undefined-behaviour sanitizers (tests/test_host_sanitizers.py builds it with
// -fsanitize=address,undefined and runs it).  After every scheduler step the
// cache manager audits itself: no page lost, held twice or freed twice.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "block_manager.hpp"
#include "scheduler.hpp"
#include "sequence.hpp"
#include "step_pack.hpp"

using namespace lyapunov::host;

static int fail(const std::string &what) {
  std::fprintf(stderr, "host_sanitize: %s\n", what.c_str());
  return 1;
}

int main(int argc, char **argv) {
  const unsigned seed = argc > 1 ? static_cast<unsigned>(std::atoi(argv[1])) : 1u;
  const int rounds = argc > 2 ? std::atoi(argv[2]) : 400;
  std::mt19937 rng(seed);
  auto pick = [&](int lo, int hi) { return lo + static_cast<int>(rng() % static_cast<unsigned>(hi - lo + 1)); };

  // two cache groups (all keys; a window of 24) so that pages are released while requests live, and few pages,
  // so that requests are cut short, pre-empted and recomputed
  std::vector<CacheGroupSpec> groups{{8, 0, 40}, {8, 24, 40}};
  auto manager = std::make_shared<BlockSpaceManager>(groups, 6);
  SchedulerConfig config;
  config.max_num_seqs = 6;
  config.max_num_batched_tokens = 48;
  config.max_model_len = 200;
  config.eos_token_ids = {3};
  config.max_prefill_chunk = 20;
  ContinuousScheduler scheduler(config, manager);

  std::vector<int32_t> packed(1 << 16);
  int64_t next_id = 0;
  uint64_t steps = 0, ahead_steps = 0;
  std::vector<int64_t> live;
  for (int round = 0; round < rounds; ++round) {
    // new requests now and then, in busy spells; in the quiet spells between them the running requests decode
    // alone, and steps are launched ahead
    const bool busy = (round / 50) % 2 == 0;
    const int arrivals = busy && pick(0, 9) < 3 ? pick(1, 3) : 0;
    for (int a = 0; a < arrivals; ++a) {
      std::vector<int32_t> prompt(static_cast<size_t>(pick(1, 90)));
      for (auto &t : prompt) t = pick(4, 500);
      SamplingParams sp;
      sp.max_tokens = pick(1, 40);
      sp.ignore_eos = pick(0, 3) == 0;
      scheduler.add_sequence(std::make_shared<Sequence>(next_id, prompt, sp));
      live.push_back(next_id++);
    }
    if (busy && !live.empty() && pick(0, 19) == 0) {     // an abort
      const size_t i = static_cast<size_t>(pick(0, static_cast<int>(live.size()) - 1));
      scheduler.abort_sequence(live[i]);
      live.erase(live.begin() + static_cast<std::ptrdiff_t>(i));
    }
    if (!scheduler.has_unfinished_sequences()) continue;
    SchedulerOutputs out = scheduler.schedule();
    ++steps;
    int tokens = 0;
    for (const auto &e : out.entries) tokens += e.count;
    if (tokens > config.max_num_batched_tokens) return fail("a step holds more tokens than the budget");
    if (static_cast<int>(out.entries.size()) > config.max_num_seqs) return fail("a step holds more requests than allowed");
    if (!out.entries.empty()) {
      const PackedStep layout = pack_step(out.entries, *manager, {16, 128}, 8, {32, 32}, packed.data(),
                                          static_cast<int64_t>(packed.size()));
      if (layout.total > static_cast<int64_t>(packed.size())) return fail("the packed step overran its buffer");
      // every block-table entry names a page of the pool or the page nobody owns
      for (int g = 0; g < 2; ++g)
        for (int64_t i = 0; i < static_cast<int64_t>(layout.num_requests) * layout.max_blocks[static_cast<size_t>(g)]; ++i) {
          const int32_t page = packed[static_cast<size_t>(layout.off_block_tables[static_cast<size_t>(g)] + i)];
          if (page < 0 || page > manager->get_num_blocks(g)) return fail("a block table names page " + std::to_string(page));
        }
    }
    // a step launched ahead of this one's results, as the engine does for decode steps
    SchedulerOutputs ahead;
    const bool try_ahead = pick(0, 1) == 1 && !out.entries.empty();
    if (try_ahead) {
      ahead = scheduler.schedule_ahead(out);
      if (!ahead.entries.empty()) {
        ++ahead_steps;
        pack_step(ahead.entries, *manager, {16, 128}, 0, {}, packed.data(), static_cast<int64_t>(packed.size()));
      }
    }
    auto sample = [&](const SchedulerOutputs &o) {
      std::vector<int32_t> tokens_out(o.sampled_seqs.size());
      for (auto &t : tokens_out) t = pick(0, 12) == 0 ? 3 : pick(4, 500);   // now and then the end-of-sequence token
      return tokens_out;
    };
    scheduler.post_step(out, sample(out));
    std::string problem = manager->audit();
    if (!problem.empty()) return fail("audit after a step: " + problem);
    if (!ahead.entries.empty()) {
      scheduler.post_step(ahead, sample(ahead));
      problem = manager->audit();
      if (!problem.empty()) return fail("audit after a step launched ahead: " + problem);
    }
  }
  // drain
  for (int guard = 0; scheduler.has_unfinished_sequences() && guard < 100000; ++guard) {
    SchedulerOutputs out = scheduler.schedule();
    std::vector<int32_t> tokens_out(out.sampled_seqs.size(), 7);
    scheduler.post_step(out, tokens_out);
  }
  if (scheduler.has_unfinished_sequences()) return fail("the scheduler did not drain");
  const std::string problem = manager->audit();
  if (!problem.empty()) return fail("audit at the end: " + problem);
  for (int g = 0; g < 2; ++g)
    if (manager->get_num_free_blocks(g) != manager->get_num_blocks(g)) return fail("pages are still held at the end");
  if (manager->get_num_free_state_slots() != manager->get_num_state_slots()) return fail("state slots are still held at the end");
  std::printf("host_sanitize: seed %u, %llu steps, %llu launched ahead, %llu pages handed out, %llu of them used before, %llu pre-emptions\n",
              seed, static_cast<unsigned long long>(steps), static_cast<unsigned long long>(ahead_steps),
              static_cast<unsigned long long>(manager->get_num_allocations()), static_cast<unsigned long long>(manager->get_num_reuses()),
              static_cast<unsigned long long>(scheduler.get_stats().preemptions));
  return 0;
}
