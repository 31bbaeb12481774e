"""The step function: run the tokens of one batch through the model, from the
cache, and return the logits at the wanted places.

A batch is a list of entries (request, its next tokens [start, start + count),
the places among them whose logits are wanted).  Portions of prompts stand
beside single decoded tokens, cut anywhere; all of them run as one batch of
T = sum(count) rows.  The host sends one block of integers per step
(``pack_step``); everything else already lives on the device.

Steps that hold single decoded tokens only can run as a captured CUDA graph of
fixed shape (the batch padded to the next bucket), which removes the launch
cost of the ~10 kernels per layer.  So can a step with one prompt portion of up
to PROMPT_GRAPH_MAX_TOKENS tokens, alone or beside decoded tokens: the portion
is padded with dummy tokens to a multiple of 64 (128 above 512) and the decoded
tokens with dummy requests, which fixes every shape; launched one by one, such
a step would be bound by the host (some 135 launches) rather than by the device.

The reference's step (python/lyapunov_engine/engine/llm_engine.py:219-312)
runs whole prompts one by one or one token per request, never a mix.
"""
from __future__ import annotations

import collections
import gc
import os

import numpy as np
import torch

from .. import build, ops
from .runtime import Workspace


# Prompt portions of at most this many tokens run as captured graphs; longer ones keep the device busy for longer
# than the host takes to launch them.  LYAPUNOV_PROMPT_GRAPHS=0 leaves them all to single launches.
PROMPT_GRAPH_MAX_TOKENS = 1024
PROMPT_GRAPHS = os.environ.get("LYAPUNOV_PROMPT_GRAPHS", "1") not in ("0", "")
MAX_PROMPT_GRAPHS = 64
# Decode graphs are keyed by (rows, width of the block tables): at most this many are kept, the one used longest
# ago makes room for a new one.
MAX_DECODE_GRAPHS = 96


class StepTooLarge(ValueError):
    """The step's integers do not fit the buffers they are packed into."""


def prompt_bucket(tokens: int) -> int:
    step = 64 if tokens <= 512 else 128
    return (tokens + step - 1) // step * step


def padded_portion(count: int, bucket: int) -> int:
    """Rows that a prompt portion of ``count`` tokens takes in a captured step
    beside ``bucket`` rows of decoded tokens.  The portion is padded to a round
    number, or, where that saves a tile of 128 rows (the matrix products work
    in such tiles), the step's rows as a whole are: a portion of 504 tokens
    beside 8 decoded ones is a step of 512 rows, not of 512 + 8 (2.47 -> 2.23
    ms at Llama-3.2-1B shapes)."""
    padded, whole = prompt_bucket(count), prompt_bucket(count + bucket) - bucket
    if (whole + bucket + 127) // 128 < (padded + bucket + 127) // 128:
        return whole
    return padded


def decode_bucket(n: int, max_num_seqs: int) -> int:
    """Rows of the captured step that takes ``n`` requests: powers of two, and
    from 48 on the steps between them too (48, 96, 192, ...: the matrix
    products of 33 to 48 rows cost a tenth less than those of 64); never more
    than ``max_num_seqs`` unless ``n`` itself is."""
    b = 1
    while b < n:
        b *= 2
    if b >= 64 and n <= b // 4 * 3:
        b = b // 4 * 3
    return min(b, max(max_num_seqs, n))


class StepContext:
    """The step's integers on the device (views into one buffer) and the few
    numbers the host keeps."""
    __slots__ = ("num_tokens", "num_requests", "num_wanted", "max_q_len", "max_context", "pure_decode",
                 "token_ids", "positions", "request_of_token", "cu_q", "ctx_before", "state_slots", "wanted_rows",
                 "block_tables", "tiles", "workspace", "status", "q_lens", "decode_requests", "num_decode",
                 "context_bound", "decode_fill")


class ModelRunner:
    def __init__(self, model, cache, runtime, max_num_batched_tokens: int, max_num_seqs: int, max_model_len: int,
                 use_cuda_graphs: bool = True, check_status: bool = False):
        self.host = build.load_host()
        self.model, self.cache, self.runtime = model, cache, runtime
        self.max_num_batched_tokens, self.max_num_seqs, self.max_model_len = max_num_batched_tokens, max_num_seqs, max_model_len
        self.use_cuda_graphs = use_cuda_graphs
        self.check_status = check_status
        self.tile_sizes = list(model.tile_sizes)     # query-tile lists that the model's mixers ask for
        dev = torch.device(runtime.device)
        self._device_index = dev.index if dev.index is not None else torch.cuda.current_device()
        self.fixed_max_blocks = [(max_model_len + cache.block_size - 1) // cache.block_size for _ in model.groups]
        self._capacity = 0
        self._ring: list = []
        self._ring_pos = 0
        self._device_ints = None
        self._graphs: dict[tuple, "_DecodeGraph"] = {}       # in the order of their last use
        self._prompt_graphs: dict[tuple, "_PromptGraph"] = {}
        # every captured step has its activations in this one workspace (steps run one after the other) and its
        # capture-time allocations in this one pool
        self._graph_workspace = None
        self._graph_pool = None
        self._warmed: set = set()                             # shapes whose kernels have run once outside a capture
        self.num_steps = 0
        self.num_graph_steps = 0
        self.num_captures = 0
        # LYAPUNOV_STEP_TIMERS=1: every step is bracketed by two CUDA events on its stream (see step_timings())
        self._timers = collections.deque(maxlen=4096) if os.environ.get("LYAPUNOV_STEP_TIMERS", "0") not in ("0", "") else None
        # room for the rows and requests that padding to a fixed shape adds to a step within the caller's limits
        self._most_rows = max_num_batched_tokens + 128 + max_num_seqs
        self._most_requests = max_num_seqs + 1
        self._reserve(self._upper_bound(self._most_rows, self._most_requests))

    # ---- integer buffers
    def _upper_bound(self, tokens: int, requests: int) -> int:
        n = 4 * tokens + 20 * (requests + 1)
        n += sum(requests * w for w in self.fixed_max_blocks)
        for ts in self.tile_sizes:
            n += 2 * (tokens // ts + requests + 4)
        return n + 64

    def _reserve(self, n: int) -> None:
        if n <= self._capacity:
            return
        self._capacity = n
        self._ring = [(torch.empty(n, dtype=torch.int32, pin_memory=True), torch.cuda.Event()) for _ in range(4)]
        for _, ev in self._ring:
            ev.record()
        self._device_ints = torch.empty(n, dtype=torch.int32, device=self.runtime.device)
        self._graphs.clear()  # they point into the old buffer
        self._prompt_graphs.clear()

    def _may_overflow(self, entries, pad_requests, pad_first_to) -> bool:
        """Whether the step could need more integers than the buffers were sized for."""
        rows = sum(e.count for e in entries) + max(0, pad_requests - len(entries)) + pad_first_to
        longest = max((e.start + max(e.count, pad_first_to) for e in entries), default=0)
        return (rows > self._most_rows or max(len(entries), pad_requests) > self._most_requests
                or longest > self.max_model_len)

    def _pack(self, entries, pad_requests=0, fixed=0, all_wanted=False, device_tokens=None, pad_first_to=0,
              wanted_rows=None, may_reserve=True):
        """``fixed``: width of every group's block table (0: as wide as the step needs).
        ``may_reserve`` False: a step that does not fit raises StepTooLarge instead
        of moving the buffers (captured graphs point into them)."""
        fixed_blocks = [min(fixed, w) for w in self.fixed_max_blocks] if fixed else []
        pinned, event = self._ring[self._ring_pos]
        self._ring_pos = (self._ring_pos + 1) % len(self._ring)
        event.synchronize()
        args = (entries, self.cache.manager, self.tile_sizes, pad_requests, fixed_blocks)
        need = self.host.pack_step(*args, 0, 0, pad_first_to).total if self._may_overflow(entries, pad_requests, pad_first_to) else 0
        if need > self._capacity:
            # more integers than the buffers hold (it does not happen within the limits given at construction)
            if not may_reserve:
                raise StepTooLarge(f"the step needs {need} integers, the buffers hold {self._capacity}")
            self._reserve(int(need * 1.5))
            pinned, event = self._ring[self._ring_pos]
            self._ring_pos = (self._ring_pos + 1) % len(self._ring)
        layout = self.host.pack_step(*args, pinned.data_ptr(), self._capacity, pad_first_to)
        if all_wanted:
            n = layout.num_requests
            pinned.numpy()[layout.off_wanted_rows:layout.off_wanted_rows + n] = np.arange(n, dtype=np.int32)
        if wanted_rows is not None:     # a step of fixed shape: one row per request (the layout has room for that)
            assert len(wanted_rows) <= layout.num_requests
            pinned.numpy()[layout.off_wanted_rows:layout.off_wanted_rows + len(wanted_rows)] = wanted_rows
        self._device_ints[:layout.total].copy_(pinned[:layout.total], non_blocking=True)
        event.record(torch.cuda.current_stream(self._device_index))
        if device_tokens is not None:
            # the entries' tokens were sampled by the step before and have not left the device
            n = len(entries)
            self._device_ints[layout.off_token_ids:layout.off_token_ids + n].copy_(device_tokens[:n], non_blocking=True)
        return layout

    def _context(self, layout, workspace, num_wanted=None) -> StepContext:
        d = self._device_ints
        T, B = layout.num_tokens, layout.num_requests
        c = StepContext()
        c.num_tokens, c.num_requests = T, B
        c.num_wanted = layout.num_wanted if num_wanted is None else num_wanted
        c.max_q_len, c.max_context = layout.max_q_len, layout.max_context
        c.pure_decode = layout.max_q_len == 1
        c.token_ids = d[layout.off_token_ids:layout.off_token_ids + T]
        c.positions = d[layout.off_positions:layout.off_positions + T]
        c.request_of_token = d[layout.off_request_of_token:layout.off_request_of_token + T]
        c.cu_q = d[layout.off_cu_q:layout.off_cu_q + B + 1]
        c.ctx_before = d[layout.off_ctx_before:layout.off_ctx_before + B]
        c.state_slots = d[layout.off_state_slots:layout.off_state_slots + B]
        c.wanted_rows = d[layout.off_wanted_rows:layout.off_wanted_rows + max(c.num_wanted, 1)][:c.num_wanted]
        c.block_tables = [d[o:o + B * w].view(B, w) for o, w in zip(layout.off_block_tables, layout.max_blocks)]
        # per tile size: (request of each tile, its first query token, tiles, tiles of multi-token requests)
        c.tiles = {ts: (d[a:a + n], d[b:b + n], n, m) for ts, a, b, n, m in
                   zip(layout.tile_sizes, layout.off_tile_request, layout.off_tile_q0, layout.num_tiles,
                       layout.num_tiles_multi)}
        c.num_decode = layout.num_decode
        c.decode_fill = layout.num_decode - (layout.num_requests - layout.num_real_requests)   # the real ones among them
        c.decode_requests = d[layout.off_decode_requests:layout.off_decode_requests + max(layout.num_decode, 1)]
        c.context_bound = layout.max_context
        c.workspace = workspace
        c.status = self.runtime.status
        return c

    # ---- the step
    def step(self, entries, device_tokens=None):
        """Runs the entries as one batch.  Returns float32 logits [wanted, vocab]
        in the order of the entries and of their ``want`` lists, or None when
        nothing is wanted.  The tensor is scratch: it is overwritten by the
        next step.  ``device_tokens`` (int32 on the device, one per entry): the
        entries bring one token each that the host does not know yet (entries
        with ``ahead`` = 1); they are taken from there."""
        if not entries:
            return None
        self.num_steps += 1
        total = sum(e.count for e in entries)
        if total > self.max_num_batched_tokens:
            raise ValueError(f"the step brings {total} tokens, max_num_batched_tokens is {self.max_num_batched_tokens}")
        if len(entries) > self.max_num_seqs:
            raise ValueError(f"the step brings {len(entries)} requests, max_num_seqs is {self.max_num_seqs}")
        decode_only = all(e.count == 1 for e in entries)
        timer = None
        if self._timers is not None:
            timer = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            timer[0].record()
        plan = None
        if self.use_cuda_graphs and not decode_only and PROMPT_GRAPHS and device_tokens is None:
            plan = self._prompt_graph_plan(entries, total)
        if self.use_cuda_graphs and decode_only:
            logits = self._graph_step(entries, device_tokens)
        elif plan is not None:
            logits = self._prompt_graph_step(entries, *plan)
        else:
            logits = self._eager_step(entries, device_tokens)
        if timer is not None:
            timer[1].record()
            kind = "decode" if decode_only else ("prompt graph" if plan is not None else "prompt")
            self._timers.append((kind, total, len(entries), *timer))
        if self.check_status:
            ops.check_status(self.runtime.status)
        return logits

    def enable_step_timers(self, on: bool = True) -> None:
        """Brackets every step with two CUDA events (what LYAPUNOV_STEP_TIMERS=1 does from the start)."""
        self._timers = collections.deque(maxlen=4096) if on else None

    def step_timings(self) -> list[dict]:
        """Device time of the last steps (up to 4,096), oldest first: kind of
        step, tokens, requests, milliseconds between the events recorded
        before and after its launches.  Waits for the last step to finish."""
        if not self._timers:
            return []
        self._timers[-1][4].synchronize()
        return [{"kind": kind, "tokens": tokens, "requests": requests, "ms": begin.elapsed_time(end)}
                for kind, tokens, requests, begin, end in self._timers]

    def _eager_step(self, entries, device_tokens=None):
        layout = self._pack(entries, device_tokens=device_tokens)
        return self.model.forward(self._context(layout, self.runtime.workspace), self.cache)

    # ---- decode steps as CUDA graphs
    def _table_width(self, tokens: int) -> int:
        """Block-table width of a captured step whose longest request holds
        ``tokens``: the next power of two of the pages that takes (16 at
        least), so that a graph serves a range of contexts and the step's
        integers do not carry tables as wide as the longest request allowed."""
        need = (tokens + self.cache.block_size - 1) // self.cache.block_size
        width = 16
        while width < need:
            width *= 2
        return min(width, max(self.fixed_max_blocks)) if self.fixed_max_blocks else width

    def _bucket(self, n: int) -> int:
        return decode_bucket(n, self.max_num_seqs)

    def _bucket_below(self, bucket: int) -> int:
        """The largest number of requests that a smaller captured step takes."""
        n = bucket - 1
        while n > 0 and self._bucket(n) >= bucket:
            n -= 1
        return n

    def _workspace_for_graphs(self):
        if self._graph_workspace is None:
            self._graph_workspace = Workspace(self.runtime.device, pin_old=True)
        return self._graph_workspace

    def _decode_graph(self, bucket: int, width: int, fill: int = 0) -> "_DecodeGraph":
        """The captured step of ``bucket`` rows and tables ``width`` pages
        wide for a step in which ``fill`` rows are real (0: all of them).
        Where a mixer launches differently for a partly filled step, such
        steps have a graph of their own."""
        fill = fill or bucket
        variant = self.model.decode_variant(fill, bucket, min(self.max_model_len, width * self.cache.block_size))
        key = (bucket, width, variant)
        graph = self._graphs.pop(key, None)
        if graph is None:
            while len(self._graphs) >= MAX_DECODE_GRAPHS:
                self._graphs.pop(next(iter(self._graphs)))        # the one used longest ago
            graph = _DecodeGraph(self, bucket, width, fill)
        self._graphs[key] = graph                                  # (now the one used last)
        return graph

    def _graph_step(self, entries, device_tokens=None):
        bucket = self._bucket(len(entries))
        width = self._table_width(max(e.start for e in entries) + 1)
        graph = self._decode_graph(bucket, width, len(entries))
        self.num_graph_steps += 1
        try:
            logits = graph.run(entries, device_tokens)
        except StepTooLarge:
            # beyond the limits the buffers were sized for: this step runs launch by launch (which may move the
            # buffers, and then drops the graphs that point into them)
            self.num_graph_steps -= 1
            return self._eager_step(entries, device_tokens)
        rows = [i for i, e in enumerate(entries) if len(e.want)]
        if not rows:
            return None
        if len(rows) == len(entries):
            return logits[:len(entries)]
        return logits[torch.tensor(rows, device=logits.device)]

    def warm_up(self, contexts=None, buckets=None) -> int:
        """Captures the decode graphs a server will need before the first
        request arrives, so that no request pays for a first use: one graph
        per batch bucket (powers of two, and 48, 96, ... between them, up to ``max_num_seqs``) and per width
        of the block tables (one for every doubling of the context up to
        ``max_model_len``, or those that hold the given ``contexts``).  The
        steps it runs hold dummy requests only: they read and write the page
        that belongs to nobody.  Returns the number of graphs captured."""
        if not self.use_cuda_graphs:
            return 0
        if buckets is None:
            buckets, b = [], 1
            while b < self.max_num_seqs:
                buckets.append(b)
                if b >= 32 and b // 2 * 3 < self.max_num_seqs:
                    buckets.append(b // 2 * 3)
                b *= 2
            buckets.append(self.max_num_seqs)
        if contexts is None:
            contexts, c = [], 16 * self.cache.block_size
            while c < self.max_model_len:
                contexts.append(c)
                c *= 2
            contexts.append(self.max_model_len)
        widths = sorted({self._table_width(min(int(c), self.max_model_len)) for c in contexts})
        before = self.num_captures
        for bucket in sorted({self._bucket(int(b)) for b in buckets}, reverse=True):
            for width in widths:
                bound = min(self.max_model_len, width * self.cache.block_size)
                # the full step first, then what partly filled ones launch differently (fills down to where the
                # next smaller bucket takes over)
                seen = set()
                for fill in range(bucket, self._bucket_below(bucket), -1):
                    variant = self.model.decode_variant(fill, bucket, bound)
                    if variant in seen:
                        continue
                    seen.add(variant)
                    if (bucket, width, variant) not in self._graphs and len(self._graphs) < MAX_DECODE_GRAPHS:
                        self._decode_graph(bucket, width, fill).run([], None)
        return self.num_captures - before

    def graph_bytes(self) -> int:
        """Device memory of the captured steps' activations."""
        return self._graph_workspace.bytes() if self._graph_workspace is not None else 0

    # ---- steps with one prompt portion as CUDA graphs
    def _prompt_graph_plan(self, entries, total):
        """(index of the portion's entry, its padded length, the bucket of the
        decoded tokens beside it) when the step can run as a graph of fixed
        shape, else None.  Dummy tokens after the portion would also pass
        through per-request state, so models that keep such state are left out."""
        multi = [i for i, e in enumerate(entries) if e.count > 1]
        if len(multi) != 1 or self.model.states:
            return None
        if total <= ops.SKINNY_NARROW_ROWS:
            # so few rows run on the weight-streaming kernels, as decode steps do, and those give a row the same
            # bits whatever the number of rows; padded, the step would go to other kernels with other roundings
            return None
        m = multi[0]
        e = entries[m]
        if e.ahead or len(e.want) > 1 or e.count > PROMPT_GRAPH_MAX_TOKENS:
            return None
        singles = len(entries) - 1
        bucket = self._bucket(singles) if singles else 0
        padded = padded_portion(e.count, bucket)
        if e.start + padded > self.max_model_len:
            return None                                   # the dummies' positions would run past the tables
        if 1 + bucket > self._most_requests or padded + bucket > self._most_rows:
            return None                                   # more rows than the step's integers have room for
        if any(x.ahead for x in entries):
            return None
        width = self._table_width(max([e.start + padded] + [x.start + 1 for x in entries]))
        if (padded, bucket, width) not in self._prompt_graphs and len(self._prompt_graphs) >= MAX_PROMPT_GRAPHS:
            return None
        return m, padded, bucket, width

    def _prompt_graph_step(self, entries, m, padded, bucket, width):
        key = (padded, bucket, width)
        graph = self._prompt_graphs.get(key)
        if graph is None:
            graph = _PromptGraph(self, padded, bucket, width)
            self._prompt_graphs[key] = graph
        # the portion first, the decoded tokens behind it; the wanted rows are listed in the entries' own order,
        # so the first rows of the result are the caller's
        ordered = [entries[m]] + [e for i, e in enumerate(entries) if i != m]
        rows = []
        single = 0
        for i, e in enumerate(entries):
            if i == m:
                rows.extend(int(w) for w in e.want)
            else:
                if len(e.want):
                    rows.append(padded + single)
                single += 1
        self.num_graph_steps += 1
        try:
            logits = graph.run(ordered, rows)
        except StepTooLarge:
            self.num_graph_steps -= 1
            return self._eager_step(entries)
        return logits[:len(rows)] if rows else None


class _StepGraph:
    """A step of fixed shape, captured at its first use.  Kernels and
    libraries must have run once before they are captured (modules load at a
    first launch, the library sets itself up): the first step of a shape whose
    kernels have not run yet therefore runs launch by launch on its real
    entries and is captured straight after (capturing runs nothing); a shape
    whose kernels are warm is captured at once and replayed.  With
    ``capture_at_first_use`` False the capture waits for the second use (shapes
    that are many and often seen only once: prompt portions).  All captured
    steps share one workspace and one memory pool."""

    def __init__(self, runner: ModelRunner, num_wanted: int, width: int, warm_key, capture_at_first_use=True):
        self.runner, self.num_wanted, self.width, self.warm_key = runner, num_wanted, width, warm_key
        self.capture_at_first_use = capture_at_first_use
        self.uses = 0
        self.workspace = runner._workspace_for_graphs()
        self.capacity_at_capture = runner._capacity
        self.graph = None
        self.logits = None
        self.decode_fill = 0      # how many of the one-token requests the step is captured for (0: as the first step has them)

    def _launch(self, layout):
        r = self.runner
        if r._capacity != self.capacity_at_capture:
            raise RuntimeError("the integer buffer moved after a step graph was made")
        if self.graph is not None:
            self.graph.replay()
            return self.logits
        ctx = r._context(layout, self.workspace, num_wanted=self.num_wanted)
        # a captured step serves every context its block tables can hold
        ctx.context_bound = min(r.max_model_len, self.width * r.cache.block_size)
        if self.decode_fill:
            ctx.decode_fill = self.decode_fill             # (a warm-up step has dummy requests only)
        ran = False
        self.uses += 1
        if self.warm_key not in r._warmed or (self.uses == 1 and not self.capture_at_first_use):
            eager = r.model.forward(ctx, r.cache)          # on the real data: nothing is computed twice
            r._warmed.add(self.warm_key)
            ran = True
            if not self.capture_at_first_use and self.uses == 1:
                return eager
        # Capture.  The step's integers are already on the device; the captured kernels read them from the same
        # addresses every time.  No garbage collection while capturing: destroying an older graph (or freeing
        # device memory) during capture invalidates it.
        torch.cuda.synchronize()
        was_enabled = gc.isenabled()
        gc.disable()
        try:
            if r._graph_pool is None:
                r._graph_pool = torch.cuda.graph_pool_handle()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, pool=r._graph_pool):
                self.logits = r.model.forward(ctx, r.cache)
        finally:
            if was_enabled:
                gc.enable()
        self.graph = graph
        r.num_captures += 1
        if ran:
            assert eager is None or self.logits is None or eager.data_ptr() == self.logits.data_ptr()
        else:
            self.graph.replay()                            # capturing does not run the kernels
        return self.logits


class _PromptGraph(_StepGraph):
    """A prompt portion of ``padded`` rows (its own tokens, then dummies) and
    ``bucket`` single-token requests."""

    def __init__(self, runner: ModelRunner, padded: int, bucket: int, width: int):
        super().__init__(runner, 1 + bucket, width, ("prompt", padded, bucket), capture_at_first_use=False)
        self.padded, self.bucket = padded, bucket
        self.decode_fill = bucket

    def run(self, entries, rows):
        n = self.num_wanted
        wanted = np.zeros(n, dtype=np.int32)
        wanted[:len(rows)] = rows
        return self._launch(self.runner._pack(entries, pad_requests=n, fixed=self.width, pad_first_to=self.padded,
                                              wanted_rows=wanted, may_reserve=False))


class _DecodeGraph(_StepGraph):
    """A decode step for a fixed number of rows."""

    def __init__(self, runner: ModelRunner, bucket: int, width: int, fill: int = 0):
        super().__init__(runner, bucket, width, ("decode", bucket))
        self.bucket = bucket
        self.decode_fill = fill or bucket

    def run(self, entries, device_tokens=None):
        return self._launch(self.runner._pack(entries, pad_requests=self.bucket, fixed=self.width, all_wanted=True,
                                              device_tokens=device_tokens, may_reserve=False))
