// Python bindings of the host runtime (module lyapunov_engine_b200._host):
// SamplingParams, Sequence, BlockSpaceManager, ContinuousScheduler with the
// reference's method names (csrc/bindings.cpp:551-621) and the additions each
// header describes, plus pack_step.  Plain C++20 and pybind11; no CUDA, no
// torch, so the cache manager and the scheduler are tested on any machine.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "block_manager.hpp"
#include "logging.hpp"
#include "scheduler.hpp"
#include "sequence.hpp"
#include "step_pack.hpp"

namespace py = pybind11;
using namespace lyapunov::host;

PYBIND11_MODULE(_host, m) {
  m.doc() = "Host runtime of lyapunov_engine_b200: requests, paged cache manager, scheduler, step packing";

  py::enum_<SequenceStatus>(m, "SequenceStatus")
      .value("WAITING", SequenceStatus::WAITING)
      .value("RUNNING", SequenceStatus::RUNNING)
      .value("FINISHED_STOPPED", SequenceStatus::FINISHED_STOPPED)
      .value("FINISHED_LENGTH_CAPPED", SequenceStatus::FINISHED_LENGTH_CAPPED)
      .value("FINISHED_ABORTED", SequenceStatus::FINISHED_ABORTED)
      .value("FINISHED_FAILED", SequenceStatus::FINISHED_FAILED);

  py::class_<SamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def_readwrite("temperature", &SamplingParams::temperature)
      .def_readwrite("top_p", &SamplingParams::top_p)
      .def_readwrite("top_k", &SamplingParams::top_k)
      .def_readwrite("max_tokens", &SamplingParams::max_tokens)
      .def_readwrite("ignore_eos", &SamplingParams::ignore_eos)
      .def_readwrite("seed", &SamplingParams::seed);

  py::class_<Sequence, SequencePtr>(m, "Sequence")
      .def(py::init<int64_t, std::vector<int32_t>, SamplingParams>(), py::arg("seq_id"), py::arg("prompt_tokens"),
           py::arg("sampling_params") = SamplingParams{})
      .def("get_seq_id", &Sequence::get_seq_id)
      .def("get_status", &Sequence::get_status)
      .def("get_sampling_params", &Sequence::get_sampling_params)
      .def("get_prompt_tokens", &Sequence::get_prompt_tokens)
      .def("get_output_tokens", &Sequence::get_output_tokens)
      .def("get_prompt_len", &Sequence::get_prompt_len)
      .def("get_output_len", &Sequence::get_output_len)
      .def("get_total_len", &Sequence::get_total_len)
      .def("get_last_token_id", &Sequence::get_last_token_id)
      .def("append_token_id", &Sequence::append_token_id)
      .def("extend_prompt", &Sequence::extend_prompt)
      .def("is_finished", &Sequence::is_finished)
      .def("finish_reason", &Sequence::finish_reason)
      .def("get_num_computed_tokens", &Sequence::get_num_computed_tokens)
      .def("set_num_computed_tokens", &Sequence::set_num_computed_tokens)
      .def("get_block_table", &Sequence::get_block_table)
      .def("get_block_tables", &Sequence::get_block_tables)
      .def("get_state_slot", &Sequence::get_state_slot)
      .def("get_num_preemptions", &Sequence::get_num_preemptions)
      .def("get_error", &Sequence::get_error);

  py::class_<CacheGroupSpec>(m, "CacheGroupSpec")
      .def(py::init([](int block_size, int window, int num_blocks) { return CacheGroupSpec{block_size, window, num_blocks}; }),
           py::arg("block_size") = 16, py::arg("window") = 0, py::arg("num_blocks") = 0)
      .def_readwrite("block_size", &CacheGroupSpec::block_size)
      .def_readwrite("window", &CacheGroupSpec::window)
      .def_readwrite("num_blocks", &CacheGroupSpec::num_blocks);

  py::class_<BlockSpaceManager, std::shared_ptr<BlockSpaceManager>>(m, "BlockSpaceManager")
      .def(py::init<int, int, bool>(), py::arg("num_blocks"), py::arg("block_size") = 16,
           py::arg("enable_prefix_caching") = false)
      .def(py::init<std::vector<CacheGroupSpec>, int>(), py::arg("groups"), py::arg("num_state_slots") = 0)
      .def("get_num_groups", &BlockSpaceManager::get_num_groups)
      .def("get_group", &BlockSpaceManager::get_group)
      .def("get_num_blocks", &BlockSpaceManager::get_num_blocks, py::arg("group") = 0)
      .def("get_block_size", &BlockSpaceManager::get_block_size, py::arg("group") = 0)
      .def("get_num_free_blocks", &BlockSpaceManager::get_num_free_blocks, py::arg("group") = 0)
      .def("get_num_used_blocks", &BlockSpaceManager::get_num_used_blocks, py::arg("group") = 0)
      .def("get_num_state_slots", &BlockSpaceManager::get_num_state_slots)
      .def("get_num_free_state_slots", &BlockSpaceManager::get_num_free_state_slots)
      .def("get_ref_count", &BlockSpaceManager::get_ref_count)
      .def("can_grow", &BlockSpaceManager::can_grow)
      .def("grow", &BlockSpaceManager::grow)
      .def("max_growth", &BlockSpaceManager::max_growth)
      .def("release_passed", &BlockSpaceManager::release_passed)
      .def("free", &BlockSpaceManager::free)
      .def("fork", &BlockSpaceManager::fork)
      .def("can_allocate", &BlockSpaceManager::can_allocate)
      .def("allocate", &BlockSpaceManager::allocate)
      .def("can_append_slot", &BlockSpaceManager::can_append_slot)
      .def("append_slot", &BlockSpaceManager::append_slot)
      .def("reset", &BlockSpaceManager::reset)
      .def("audit", &BlockSpaceManager::audit)
      .def("get_num_allocations", &BlockSpaceManager::get_num_allocations)
      .def("get_num_reuses", &BlockSpaceManager::get_num_reuses);

  py::class_<SchedulerConfig>(m, "SchedulerConfig")
      .def(py::init<>())
      .def_readwrite("max_num_seqs", &SchedulerConfig::max_num_seqs)
      .def_readwrite("max_num_batched_tokens", &SchedulerConfig::max_num_batched_tokens)
      .def_readwrite("max_model_len", &SchedulerConfig::max_model_len)
      .def_readwrite("eos_token_ids", &SchedulerConfig::eos_token_ids)
      .def_readwrite("max_prefill_chunk", &SchedulerConfig::max_prefill_chunk)
      .def_property(
          "eos_token_id", [](const SchedulerConfig &c) { return c.eos_token_ids.empty() ? -1 : c.eos_token_ids[0]; },
          [](SchedulerConfig &c, int32_t id) { c.eos_token_ids = id < 0 ? std::vector<int32_t>{} : std::vector<int32_t>{id}; });

  py::class_<StepEntry>(m, "StepEntry")
      .def(py::init([](SequencePtr seq, int start, int count, std::vector<int32_t> want, int ahead) {
             return StepEntry{std::move(seq), start, count, std::move(want), ahead};
           }),
           py::arg("seq"), py::arg("start"), py::arg("count"), py::arg("want") = std::vector<int32_t>{}, py::arg("ahead") = 0)
      .def_readwrite("seq", &StepEntry::seq)
      .def_readwrite("start", &StepEntry::start)
      .def_readwrite("count", &StepEntry::count)
      .def_readwrite("want", &StepEntry::want)
      .def_readwrite("ahead", &StepEntry::ahead);

  py::class_<SchedulerOutputs>(m, "SchedulerOutputs")
      .def_readonly("entries", &SchedulerOutputs::entries)
      .def_readonly("scheduled_seqs", &SchedulerOutputs::scheduled_seqs)
      .def_readonly("sampled_seqs", &SchedulerOutputs::sampled_seqs)
      .def_readonly("preempted_seqs", &SchedulerOutputs::preempted_seqs)
      .def_readonly("finished_seqs", &SchedulerOutputs::finished_seqs)
      .def_readonly("is_prefill", &SchedulerOutputs::is_prefill)
      .def_readonly("num_batched_tokens", &SchedulerOutputs::num_batched_tokens);

  py::class_<SchedulerStats>(m, "SchedulerStats")
      .def_readonly("steps", &SchedulerStats::steps)
      .def_readonly("prefill_tokens", &SchedulerStats::prefill_tokens)
      .def_readonly("decode_tokens", &SchedulerStats::decode_tokens)
      .def_readonly("preemptions", &SchedulerStats::preemptions)
      .def_readonly("failed", &SchedulerStats::failed);

  py::class_<ContinuousScheduler>(m, "ContinuousScheduler")
      .def(py::init<const SchedulerConfig &, std::shared_ptr<BlockSpaceManager>>())
      .def("add_sequence", &ContinuousScheduler::add_sequence)
      .def("abort_sequence", &ContinuousScheduler::abort_sequence)
      .def("has_unfinished_sequences", &ContinuousScheduler::has_unfinished_sequences)
      .def("get_num_waiting_sequences", &ContinuousScheduler::get_num_waiting_sequences)
      .def("get_num_running_sequences", &ContinuousScheduler::get_num_running_sequences)
      .def("schedule", &ContinuousScheduler::schedule)
      .def("schedule_ahead", &ContinuousScheduler::schedule_ahead)
      .def("post_step", &ContinuousScheduler::post_step)
      .def("get_stats", &ContinuousScheduler::get_stats)
      .def("get_config", &ContinuousScheduler::get_config);

  py::class_<PackedStep>(m, "PackedStep")
      .def_readonly("num_tokens", &PackedStep::num_tokens)
      .def_readonly("num_requests", &PackedStep::num_requests)
      .def_readonly("num_real_requests", &PackedStep::num_real_requests)
      .def_readonly("num_wanted", &PackedStep::num_wanted)
      .def_readonly("max_q_len", &PackedStep::max_q_len)
      .def_readonly("max_context", &PackedStep::max_context)
      .def_readonly("off_token_ids", &PackedStep::off_token_ids)
      .def_readonly("off_positions", &PackedStep::off_positions)
      .def_readonly("off_request_of_token", &PackedStep::off_request_of_token)
      .def_readonly("off_cu_q", &PackedStep::off_cu_q)
      .def_readonly("off_ctx_before", &PackedStep::off_ctx_before)
      .def_readonly("off_state_slots", &PackedStep::off_state_slots)
      .def_readonly("off_wanted_rows", &PackedStep::off_wanted_rows)
      .def_readonly("off_block_tables", &PackedStep::off_block_tables)
      .def_readonly("max_blocks", &PackedStep::max_blocks)
      .def_readonly("tile_sizes", &PackedStep::tile_sizes)
      .def_readonly("off_tile_request", &PackedStep::off_tile_request)
      .def_readonly("off_tile_q0", &PackedStep::off_tile_q0)
      .def_readonly("num_tiles", &PackedStep::num_tiles)
      .def_readonly("num_tiles_multi", &PackedStep::num_tiles_multi)
      .def_readonly("off_decode_requests", &PackedStep::off_decode_requests)
      .def_readonly("num_decode", &PackedStep::num_decode)
      .def_readonly("total", &PackedStep::total);

  m.def(
      "pack_step",
      [](const std::vector<StepEntry> &entries, const BlockSpaceManager &manager, const std::vector<int> &tile_sizes,
         int pad_requests, const std::vector<int> &fixed_max_blocks, uintptr_t dest, int64_t capacity, int pad_first_to) {
        return pack_step(entries, manager, tile_sizes, pad_requests, fixed_max_blocks, reinterpret_cast<int32_t *>(dest), capacity,
                         pad_first_to);
      },
      py::arg("entries"), py::arg("manager"), py::arg("tile_sizes") = std::vector<int>{}, py::arg("pad_requests") = 0,
      py::arg("fixed_max_blocks") = std::vector<int>{}, py::arg("dest") = 0, py::arg("capacity") = 0,
      py::arg("pad_first_to") = 0,
      "Writes the step's integers at address `dest` (room for `capacity` int32) and returns the layout.");

  m.def("set_log_level", [](const std::string &name) {
    if (name == "debug") Log::get().set_level(LogLevel::kDebug);
    else if (name == "info") Log::get().set_level(LogLevel::kInfo);
    else if (name == "warn") Log::get().set_level(LogLevel::kWarn);
    else if (name == "error") Log::get().set_level(LogLevel::kError);
    else throw std::invalid_argument("log level must be debug, info, warn or error");
  });
}
