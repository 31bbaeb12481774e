// Flattens the entries of one step into one block of 32-bit integers, the
// only thing the host sends to the device per step: token ids, positions,
// the request of every token, per-request offsets, lengths already cached,
// state slots, the rows whose logits are wanted, one block table per cache
// group and lists of query tiles for the attention kernels.
//
// The reference builds these per step in Python with one small device copy per
// request (python/lyapunov_engine/engine/llm_engine.py:233-254).
#pragma once

#include <cstdint>
#include <vector>

#include "block_manager.hpp"
#include "scheduler.hpp"

namespace lyapunov::host {

struct PackedStep {
  int num_tokens{0};     // T (rows of the batch, padding included)
  int num_requests{0};   // B (padding included)
  int num_real_requests{0};
  int num_wanted{0};
  int max_q_len{0};
  int max_context{0};    // the longest start + count
  int64_t off_token_ids{0}, off_positions{0}, off_request_of_token{0};
  int64_t off_cu_q{0}, off_ctx_before{0}, off_state_slots{0}, off_wanted_rows{0};
  std::vector<int64_t> off_block_tables;  // per group, [B, max_blocks[g]]
  std::vector<int> max_blocks;
  std::vector<int> tile_sizes;
  std::vector<int64_t> off_tile_request, off_tile_q0;  // per tile size; multi-token requests first
  std::vector<int> num_tiles;
  std::vector<int> num_tiles_multi;  // how many of them belong to requests that bring more than one token
  int64_t off_decode_requests{0};    // the requests that bring exactly one token (padding included)
  int num_decode{0};
  int64_t total{0};      // integers used
};

// `tokens_of(entry)` are taken from the sequence itself (tokens start ..
// start+count-1).  `pad_requests` > number of entries adds one-token dummy
// requests that write to `null_pages[g]` (a page outside the manager's range)
// so that the batch has a fixed shape; `fixed_max_blocks[g]` > 0 fixes the
// width of group g's table.  `pad_first_to` > the first entry's count lets
// that entry bring dummy tokens after its own, up to that many rows: they
// continue its positions, carry token 0 and write where the block table
// points (the request's own last page, which its later tokens overwrite
// before anyone reads them, and the page nobody owns beyond it), so a prompt
// portion too can have a fixed shape.  Returns the layout; throws if
// `capacity` is too small.  `dest` may be null to compute the layout only.
PackedStep pack_step(const std::vector<StepEntry> &entries, const BlockSpaceManager &manager,
                     const std::vector<int> &tile_sizes, int pad_requests,
                     const std::vector<int> &fixed_max_blocks, int32_t *dest, int64_t capacity,
                     int pad_first_to = 0);

}  // namespace lyapunov::host
