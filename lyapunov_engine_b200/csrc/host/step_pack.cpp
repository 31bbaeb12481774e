#include "step_pack.hpp"

#include <algorithm>
#include <stdexcept>
#include <string>

namespace lyapunov::host {

PackedStep pack_step(const std::vector<StepEntry> &entries, const BlockSpaceManager &manager,
                     const std::vector<int> &tile_sizes, int pad_requests,
                     const std::vector<int> &fixed_max_blocks, int32_t *dest, int64_t capacity, int pad_first_to) {
  PackedStep p;
  // rows entry i brings, dummy tokens after the first entry's own included
  auto rows_of = [&](size_t i) { return i == 0 && pad_first_to > entries[0].count ? pad_first_to : entries[i].count; };
  const int groups = manager.get_num_groups();
  const int real = static_cast<int>(entries.size());
  const int B = std::max(real, pad_requests);
  p.num_requests = B;
  p.num_real_requests = real;
  p.tile_sizes = tile_sizes;

  int T = 0;
  for (size_t i = 0; i < entries.size(); ++i) {
    const auto &e = entries[i];
    const int rows = rows_of(i);
    if (e.count < 1) throw std::invalid_argument("pack_step: an entry brings no token");
    if (e.ahead < 0 || e.ahead > 1) throw std::invalid_argument("pack_step: an entry is at most one step ahead");
    if (e.start != static_cast<int>(e.seq->get_num_computed_tokens()) + e.ahead)
      throw std::invalid_argument("pack_step: request " + std::to_string(e.seq->get_seq_id()) + " has " +
                                  std::to_string(e.seq->get_num_computed_tokens()) +
                                  " tokens in the cache but its entry starts at " + std::to_string(e.start));
    if (static_cast<size_t>(e.start + e.count) > e.seq->get_total_len() + static_cast<size_t>(e.ahead))
      throw std::invalid_argument("pack_step: an entry runs past the request's tokens");
    for (int32_t w : e.want)
      if (w < 0 || w >= e.count) throw std::invalid_argument("pack_step: a wanted place lies outside the entry's tokens");
    T += rows;
    p.num_wanted += static_cast<int>(e.want.size());
    p.max_q_len = std::max(p.max_q_len, rows);
    p.max_context = std::max(p.max_context, e.start + rows);
  }
  T += B - real;
  if (B > real) {
    p.max_q_len = std::max(p.max_q_len, 1);
    p.max_context = std::max(p.max_context, 1);
  }
  p.num_tokens = T;

  p.max_blocks.assign(groups, 1);
  for (int g = 0; g < groups; ++g) {
    const int bs = manager.get_block_size(g);
    int need = 1;
    for (size_t i = 0; i < entries.size(); ++i) need = std::max(need, (entries[i].start + rows_of(i) + bs - 1) / bs);
    if (g < static_cast<int>(fixed_max_blocks.size()) && fixed_max_blocks[g] > 0) {
      if (need > fixed_max_blocks[g]) throw std::invalid_argument("pack_step: a request needs more pages than the fixed table width");
      need = fixed_max_blocks[g];
    }
    p.max_blocks[g] = need;
  }

  int64_t off = 0;
  auto take = [&](int64_t n) { const int64_t o = off; off += (n + 3) / 4 * 4; return o; };  // 16-byte aligned parts
  p.off_token_ids = take(T);
  p.off_positions = take(T);
  p.off_request_of_token = take(T);
  p.off_cu_q = take(B + 1);
  p.off_ctx_before = take(B);
  p.off_state_slots = take(B);
  // room for one row per request as well: a step of fixed shape asks for the logits of every row it has,
  // dummy requests included, and writes that list here itself
  p.off_wanted_rows = take(std::max({p.num_wanted, B, 1}));
  for (int g = 0; g < groups; ++g) p.off_block_tables.push_back(take(static_cast<int64_t>(B) * p.max_blocks[g]));
  p.num_decode = B - real;
  for (size_t i = 0; i < entries.size(); ++i) p.num_decode += rows_of(i) == 1;
  p.off_decode_requests = take(std::max(p.num_decode, 1));
  for (int ts : tile_sizes) {
    if (ts < 1) throw std::invalid_argument("pack_step: tile sizes must be >= 1");
    int n = B - real, multi = 0;
    for (size_t i = 0; i < entries.size(); ++i) {
      const int rows = rows_of(i);
      n += (rows + ts - 1) / ts;
      if (rows > 1) multi += (rows + ts - 1) / ts;
    }
    p.num_tiles.push_back(n);
    p.num_tiles_multi.push_back(multi);
    p.off_tile_request.push_back(take(n));
    p.off_tile_q0.push_back(take(n));
  }
  p.total = off;
  if (dest == nullptr) return p;
  if (off > capacity) throw std::length_error("pack_step: the step needs " + std::to_string(off) + " integers, the buffer holds " + std::to_string(capacity));

  int32_t *tok = dest + p.off_token_ids, *pos = dest + p.off_positions, *req = dest + p.off_request_of_token;
  int32_t *cu = dest + p.off_cu_q, *ctx = dest + p.off_ctx_before, *slots = dest + p.off_state_slots;
  int32_t *want = dest + p.off_wanted_rows;
  int t = 0, w = 0;
  cu[0] = 0;
  for (int b = 0; b < B; ++b) {
    if (b < real) {
      const auto &e = entries[b];
      const int rows = rows_of(static_cast<size_t>(b));
      for (int j = 0; j < rows; ++j) {
        // (a token the host does not know yet is written by the device before the step runs)
        const size_t at = static_cast<size_t>(e.start + j);
        tok[t + j] = at < e.seq->get_total_len() ? e.seq->token_at(at) : 0;
        pos[t + j] = e.start + j;
        req[t + j] = b;
      }
      for (int32_t x : e.want) want[w++] = t + x;
      ctx[b] = e.start;
      slots[b] = e.seq->get_state_slot();
      t += rows;
    } else {
      tok[t] = 0; pos[t] = 0; req[t] = b;
      ctx[b] = 0;
      slots[b] = -1;
      t += 1;
    }
    cu[b + 1] = t;
  }
  if (p.num_wanted == 0) want[0] = 0;
  for (int g = 0; g < groups; ++g) {
    int32_t *table = dest + p.off_block_tables[g];
    const int width = p.max_blocks[g];
    const int32_t null_page = manager.get_num_blocks(g);  // one page past the pool: the device keeps it for dummies
    for (int b = 0; b < B; ++b) {
      int32_t *row = table + static_cast<int64_t>(b) * width;
      int n = 0;
      if (b < real) {
        const auto &tables = entries[b].seq->get_block_tables();
        if (g < static_cast<int>(tables.size())) {
          n = std::min<int>(width, static_cast<int>(tables[g].size()));
          for (int i = 0; i < n; ++i) row[i] = tables[g][i] >= 0 ? tables[g][i] : null_page;
        }
      }
      for (int i = n; i < width; ++i) row[i] = null_page;
    }
  }
  {
    int32_t *dec = dest + p.off_decode_requests;
    int n = 0;
    for (int b = 0; b < B; ++b)
      if ((b < real ? rows_of(static_cast<size_t>(b)) : 1) == 1) dec[n++] = b;
    if (n == 0) dec[0] = 0;
  }
  for (size_t k = 0; k < tile_sizes.size(); ++k) {
    int32_t *tr = dest + p.off_tile_request[k], *tq = dest + p.off_tile_q0[k];
    int n = 0;
    for (int pass = 0; pass < 2; ++pass) {   // requests with several tokens first, then single tokens
      for (int b = 0; b < B; ++b) {
        const int count = b < real ? rows_of(static_cast<size_t>(b)) : 1;
        if ((pass == 0) != (count > 1)) continue;
        for (int q0 = 0; q0 < count; q0 += tile_sizes[k]) { tr[n] = b; tq[n] = q0; ++n; }
      }
      if (pass == 0 && n > 1) {
        // Tiles of several tokens in the order of the keys they see, fewest first: the attention kernels walk
        // the list from its end, so that the longest tiles of a step start first whatever request they are of.
        std::vector<int> order(static_cast<size_t>(n));
        for (int i = 0; i < n; ++i) order[static_cast<size_t>(i)] = i;
        auto keys_seen = [&](int i) { return entries[static_cast<size_t>(tr[i])].start + tq[i] + tile_sizes[k]; };
        std::stable_sort(order.begin(), order.end(), [&](int x, int y) { return keys_seen(x) < keys_seen(y); });
        std::vector<int32_t> r2(static_cast<size_t>(n)), q2(static_cast<size_t>(n));
        for (int i = 0; i < n; ++i) { r2[static_cast<size_t>(i)] = tr[order[static_cast<size_t>(i)]]; q2[static_cast<size_t>(i)] = tq[order[static_cast<size_t>(i)]]; }
        for (int i = 0; i < n; ++i) { tr[i] = r2[static_cast<size_t>(i)]; tq[i] = q2[static_cast<size_t>(i)]; }
      }
    }
  }
  return p;
}

}  // namespace lyapunov::host
