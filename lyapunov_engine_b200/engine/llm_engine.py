"""LLMEngine: requests in, tokens out.

The reference's names and calls are kept
(python/lyapunov_engine/engine/llm_engine.py:18-55,93-312): ``EngineConfig``,
``RequestOutput``, ``LLMEngine.add_request`` in both call shapes,
``has_unfinished_requests`` and ``step``; ``generate`` loops ``step`` for a
list of prompts.  Behind them: the C++ scheduler decides each step's batch
(portions of prompts beside decoded tokens under one token budget), the step
function runs it, the sampler picks tokens on the device, one small transfer
brings them back, and the scheduler finishes and frees.
"""
from __future__ import annotations

import collections
import contextlib
import gc
import os

import torch

from .. import build, ops
from ..cache import DeviceCache
from ..config.base import read_config_json
from ..models.model import Model
from ..registry import spec_for
from ..sampling import Sampler, SamplingParams
from ..weights.loader import FolderWeights, RandomWeights
from .runtime import Runtime, parse_dtype
from .step import ModelRunner


class EngineConfig:
    """Runtime options, with the reference's names and defaults
    (python/lyapunov_engine/engine/llm_engine.py:18-38); ``dtype`` is bfloat16
    or float32 here, and ``max_model_len`` bounds a request's length (default:
    the model's ``max_position_embeddings``, capped by what the pages hold)."""

    def __init__(self, model_config=None, num_blocks: int = 1024, num_gpu_blocks: int | None = None,
                 block_size: int = 16, max_num_seqs: int = 64, max_num_batched_tokens: int = 2048,
                 dtype=torch.bfloat16, device: str = "cuda:0", max_model_len: int | None = None,
                 max_prefill_chunk: int = 0, use_cuda_graphs: bool = True, seed: int = 0, lookahead: bool | None = None,
                 freeze_gc: bool = False):
        self.model_config = model_config
        self.num_blocks = num_gpu_blocks if num_gpu_blocks is not None else num_blocks
        self.block_size = block_size
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.dtype = parse_dtype(dtype)
        self.device = device
        self.max_model_len = max_model_len
        self.max_prefill_chunk = max_prefill_chunk
        self.use_cuda_graphs = use_cuda_graphs
        self.seed = seed
        # launch the next decode step before the result of the one before has been read (see LLMEngine.step)
        self.lookahead = (os.environ.get("LYAPUNOV_LOOKAHEAD", "1") not in ("0", "")) if lookahead is None else bool(lookahead)
        # A full collection of the interpreter's heap walks every object that torch and the model made (measured
        # 23-32 ms) and lands in whichever step allocates the object that triggers it, while a decode step takes
        # one millisecond.  With this set, the engine moves the objects that exist once it is built into the
        # collector's permanent generation (gc.freeze()): they are still freed when their last reference goes, but
        # no longer searched for cycles, so an engine that is dropped later may keep its memory.  For a process
        # that serves with one engine until it exits; off by default.
        self.freeze_gc = bool(freeze_gc)


class _LaunchedStep:
    """A step that runs on the device: what was scheduled, and where its tokens arrive."""
    __slots__ = ("out", "num_sampled", "host", "event", "ids")

    def __init__(self, out, num_sampled):
        self.out, self.num_sampled = out, num_sampled
        self.host = self.event = self.ids = None


class RequestOutput:
    def __init__(self, request_id, prompt_tokens, output_tokens, finished, finish_reason=None, error=None):
        self.request_id = request_id
        self.prompt_tokens = prompt_tokens
        self.output_tokens = output_tokens
        self.finished = finished
        self.is_finished = finished
        self.finish_reason = finish_reason   # "stop", "length", "abort" or "error"
        self.error = error
        self.text = None                     # the output decoded, when the prompts were given as text

    def __repr__(self):
        return (f"RequestOutput(request_id={self.request_id!r}, output_tokens={self.output_tokens!r}, "
                f"finished={self.finished}, finish_reason={self.finish_reason!r})")


class LoadedModel:
    """A model with its weights on the device."""

    def __init__(self, spec, model, runtime, folder=None):
        self.spec, self.model, self.runtime = spec, model, runtime
        self.config = spec
        self.folder = folder          # where the weights (and a tokenizer, if any) came from


def load_model(folder: str | None = None, dtype=torch.bfloat16, device: str = "cuda:0", config: dict | None = None,
               random_seed: int | None = None, max_model_len: int | None = None, std: float = 0.02,
               norm_jitter: float = 0.0) -> LoadedModel:
    """Builds the model that config.json names and binds its weights: from the
    folder's safetensors files, or, with ``random_seed``, from that seed
    (``config`` then gives the content of a config.json and no folder is
    needed)."""
    dtype = parse_dtype(dtype)
    raw = config if config is not None else read_config_json(folder)
    spec = spec_for(raw)
    runtime = Runtime(device, dtype, max_model_len=max_model_len or spec.max_positions)
    model = Model(spec)
    decls = model.tensors()
    with torch.cuda.device(runtime.device):
        if random_seed is not None:
            source = RandomWeights(decls, dtype, runtime.device, random_seed, std, norm_jitter)
        else:
            source = FolderWeights(folder, decls, dtype, runtime.device)
        model.bind(source.get, runtime)
        source.release()
    return LoadedModel(spec, model, runtime, folder)


class LLMEngine:
    def __init__(self, model: LoadedModel, config: EngineConfig | None = None, **options):
        if config is None:
            config = EngineConfig(**options)
        if not isinstance(model, LoadedModel):
            raise TypeError("LLMEngine takes a model from load_model() or LLMEngine.from_pretrained()")
        self.config = config
        self.loaded = model
        self.runtime = model.runtime
        dev = torch.device(self.runtime.device)
        self._device_index = dev.index if dev.index is not None else (torch.cuda.current_device() if dev.type == "cuda" else 0)
        if config.dtype != self.runtime.dtype:
            raise ValueError(f"the model was loaded as {self.runtime.dtype}, the engine is configured as {config.dtype}")
        self.host = build.load_host()
        spec = model.spec
        self.block_size = config.block_size
        self.num_blocks = config.num_blocks
        capacity = self.num_blocks * self.block_size
        self.max_model_len = min(config.max_model_len or spec.max_positions, spec.max_positions,
                                 self.runtime.max_model_len or spec.max_positions)
        if model.model.groups:
            self.max_model_len = min(self.max_model_len, capacity)
        with torch.cuda.device(self.runtime.device):
            self.cache = DeviceCache(model.model, self.runtime, self.num_blocks, self.block_size, config.max_num_seqs)
            self.runner = ModelRunner(model.model, self.cache, self.runtime, config.max_num_batched_tokens,
                                      config.max_num_seqs, self.max_model_len, config.use_cuda_graphs)
            self.sampler = Sampler(self.runtime.device, config.max_num_seqs)
        self.block_manager = self.cache.manager
        sched = self.host.SchedulerConfig()
        sched.max_num_seqs = config.max_num_seqs
        sched.max_num_batched_tokens = config.max_num_batched_tokens
        sched.max_model_len = self.max_model_len
        sched.eos_token_ids = list(spec.eos_token_ids)
        sched.max_prefill_chunk = config.max_prefill_chunk
        self.scheduler = self.host.ContinuousScheduler(sched, self.block_manager)
        self.req_counter = 0
        self.active_sequences: dict[int, tuple] = {}
        self._prompts: dict[int, list] = {}
        # steps that run on the device and whose tokens have not been read: at most two
        self._launched: collections.deque = collections.deque()
        self._token_slots = [(torch.empty(config.max_num_seqs + 1, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                             for _ in range(4)]
        self._token_slot = 0
        self.num_steps_ahead = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        if config.freeze_gc:
            gc.collect()
            gc.freeze()

    def warm_up(self, contexts=None, batches=None) -> int:
        """Captures the decode steps' graphs ahead of the first request (every
        batch bucket up to ``max_num_seqs`` at every doubling of the context up
        to ``max_model_len``, or those that serve the given ``contexts`` and
        ``batches``), so that no request waits for a capture.  Returns how
        many were captured.  Without it each shape is captured at its first use."""
        with self._on_device():
            n = self.runner.warm_up(contexts, batches)
        if self.config.freeze_gc:
            gc.collect()
            gc.freeze()
        return n

    # ---- construction in one call
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype=torch.bfloat16, device: str = "cuda:0", **options) -> "LLMEngine":
        config = EngineConfig(dtype=dtype, device=device, **options)
        loaded = load_model(model_dir, config.dtype, device, max_model_len=config.max_model_len)
        return cls(loaded, config)

    # ---- the reference's interface
    def add_request(self, arg1, arg2=None, arg3=None):
        """``add_request(prompt_tokens, sampling_params)`` or
        ``add_request(request_id, prompt_tokens, sampling_params)``."""
        if isinstance(arg1, (int, str)) and isinstance(arg2, (list, tuple)):
            request_id, prompt_tokens, sampling = arg1, list(arg2), arg3 or SamplingParams()
        elif isinstance(arg1, (list, tuple)):
            request_id = self.req_counter
            prompt_tokens = list(arg1)
            sampling = arg2 if isinstance(arg2, SamplingParams) else SamplingParams()
        else:
            raise TypeError("add_request(prompt_tokens, sampling_params) or add_request(request_id, prompt_tokens, sampling_params)")
        if not prompt_tokens:
            raise ValueError("the prompt is empty")
        vocab = self.loaded.spec.vocab_size
        for t in prompt_tokens:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        seq_id = self.req_counter
        self.req_counter += 1
        c = self.host.SamplingParams()
        c.temperature, c.top_p, c.top_k = sampling.temperature, sampling.top_p, sampling.top_k
        c.max_tokens, c.ignore_eos, c.seed = sampling.max_tokens, sampling.ignore_eos, int(sampling.seed) & (2**64 - 1)
        prompt_tokens = [int(t) for t in prompt_tokens]
        seq = self.host.Sequence(seq_id, prompt_tokens, c)
        self.scheduler.add_sequence(seq)
        self.active_sequences[seq_id] = (seq, sampling, request_id)
        self._prompts[seq_id] = prompt_tokens     # kept here so that outputs need not copy it out of C++ every step
        return request_id

    def abort_request(self, request_id) -> None:
        for seq_id, (seq, _, rid) in list(self.active_sequences.items()):
            if rid == request_id:
                self.scheduler.abort_sequence(seq_id)
                del self.active_sequences[seq_id]
                self._prompts.pop(seq_id, None)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_sequences()

    def step(self) -> list[RequestOutput]:
        """One scheduler step: returns an output for every request that was in
        the step (and for those that failed or were finished by it).

        The device runs one step ahead of what this returns: while the tokens
        of a decode step are on their way to the host, the step after it is
        already launched (its input tokens pass from the sampler to the
        embedding on the device), so the host's work between two steps does
        not leave the device idle.  A request that ends with an
        end-of-sequence token has then had one token too many computed, which
        is dropped."""
        while self._launched and all(s.is_finished() for s in self._launched[0].out.scheduled_seqs):
            self._launched.popleft()           # a step launched ahead for requests that all ended before it
        if not self._launched and not self.has_unfinished_requests():
            return []
        outputs: list[RequestOutput] = []
        with self._on_device():
            if not self._launched:
                out = self.scheduler.schedule()
                for seq in out.finished_seqs:
                    outputs.append(self._output(seq))
                if not out.entries:
                    return outputs
                self._launch(out, None)
            newest = self._launched[-1]
            if self.config.lookahead and len(self._launched) < 2 and newest.ids is not None:
                ahead = self.scheduler.schedule_ahead(newest.out)
                if ahead.entries:
                    self._launch(ahead, newest.ids)
                    self.num_steps_ahead += 1
            step = self._launched.popleft()
            tokens = self._read(step)
        ended_before = [s.is_finished() for s in step.out.scheduled_seqs]
        self.scheduler.post_step(step.out, tokens)
        for seq, ended in zip(step.out.scheduled_seqs, ended_before):
            if not ended:
                outputs.append(self._output(seq))
        return outputs

    def _launch(self, out, device_tokens) -> None:
        """Puts a scheduled step on the device: the model, the sampler and the
        transfer of the chosen tokens (and the kernels' status word) to the host."""
        logits = self.runner.step(out.entries, device_tokens)
        sampled = out.sampled_seqs
        n = len(sampled)
        step = _LaunchedStep(out, n)
        if n:
            ahead = out.entries[0].ahead if device_tokens is not None else 0
            params = [self.active_sequences[s.get_seq_id()][1] for s in sampled]
            indices = [s.get_total_len() + ahead for s in sampled]
            ids = self.sampler.sample(logits, params, indices)
            host, event = self._token_slots[self._token_slot]
            self._token_slot = (self._token_slot + 1) % len(self._token_slots)
            event.synchronize()                # (the slot's transfer of four steps ago)
            host[:n].copy_(ids, non_blocking=True)
            host[n:n + 1].copy_(self.runtime.status[:1], non_blocking=True)
            event.record(torch.cuda.current_stream(self._device_index))
            step.host, step.event = host, event
            # the next step may take its tokens from here if every entry is a single decoded token
            if n == len(out.entries) and all(e.count == 1 for e in out.entries):
                step.ids = ids
            self.d2h_bytes += 4 * (n + 1)
        self._launched.append(step)

    def _read(self, step) -> list[int]:
        """Waits for a launched step's tokens."""
        if step.num_sampled == 0:
            return []
        step.event.synchronize()
        host = step.host[:step.num_sampled + 1].tolist()
        if host[-1]:
            ops.check_status(self.runtime.status)
        return host[:-1]

    def _on_device(self):
        """The engine's device as the current one: nothing to do (and nothing
        to pay, every step) when it already is."""
        if torch.cuda.current_device() == self._device_index:
            return contextlib.nullcontext()
        return torch.cuda.device(self._device_index)

    def _output(self, seq) -> RequestOutput:
        seq_id = seq.get_seq_id()
        _, _, request_id = self.active_sequences.get(seq_id, (None, None, seq_id))
        finished = seq.is_finished()
        prompt = self._prompts.get(seq_id)
        if prompt is None:
            prompt = seq.get_prompt_tokens()
        o = RequestOutput(request_id, prompt, seq.get_output_tokens(), finished,
                          seq.finish_reason() if finished else None, seq.get_error() or None)
        if finished:
            self.active_sequences.pop(seq_id, None)
            self._prompts.pop(seq_id, None)
        return o

    # ---- convenience
    def generate(self, prompts, sampling_params=None) -> list[RequestOutput]:
        """Runs every prompt to its end and returns the outputs in the order of
        the prompts.  Prompts are lists of token ids, or strings: those are
        encoded with the tokenizer of the model's folder (the one
        ``transformers.AutoTokenizer`` finds there, as the reference's command
        line does, python/lyapunov_engine/entrypoints/cli.py:28-31) and the
        outputs carry ``text``.  ``sampling_params``: one for all, or one per
        prompt."""
        if isinstance(prompts, str) or (prompts and isinstance(prompts[0], int)):
            prompts = [prompts]
        as_text = bool(prompts) and isinstance(prompts[0], str)
        if as_text:
            tokenizer = self.tokenizer()
            prompts = [tokenizer.encode(p) for p in prompts]
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        order = []
        for i, (p, sp) in enumerate(zip(prompts, sampling_params)):
            order.append(self.add_request(f"generate-{self.req_counter}-{i}", list(p), sp))
        done: dict = {}
        while self.has_unfinished_requests():
            for o in self.step():
                if o.finished and o.request_id in order:
                    done[o.request_id] = o
        if as_text:
            for o in done.values():
                o.text = tokenizer.decode(o.output_tokens, skip_special_tokens=True)
        return [done[r] for r in order]

    def tokenizer(self):
        """The tokenizer of the model's folder (loaded at first use)."""
        if getattr(self, "_tokenizer", None) is None:
            if not self.loaded.folder:
                raise ValueError("text prompts need a tokenizer: this model was not loaded from a folder; give token ids")
            try:
                from transformers import AutoTokenizer
            except ImportError as e:
                raise ValueError("text prompts need the transformers package for its tokenizers; give token ids") from e
            try:
                self._tokenizer = AutoTokenizer.from_pretrained(self.loaded.folder)
            except Exception as e:
                raise ValueError(f"no tokenizer could be loaded from {self.loaded.folder}: {e}; give token ids") from e
        return self._tokenizer

    def stats(self) -> dict:
        s = self.scheduler.get_stats()
        timed = {}
        if self.runner._timers:
            by_kind: dict = {}
            for t in self.runner.step_timings():
                by_kind.setdefault(t["kind"], []).append(t["ms"])
            timed = {"step_ms": {k: {"steps": len(v), "mean": sum(v) / len(v), "max": max(v)} for k, v in by_kind.items()}}
        return {**timed, "steps": s.steps, "prefill_tokens": s.prefill_tokens, "decode_tokens": s.decode_tokens,
                "preemptions": s.preemptions, "failed": s.failed, "graph_steps": self.runner.num_graph_steps,
                "graphs": len(self.runner._graphs) + len(self.runner._prompt_graphs),
                "graph_bytes": self.runner.graph_bytes(), "steps_ahead": self.num_steps_ahead,
                "free_blocks": self.block_manager.get_num_free_blocks() if self.loaded.model.groups else 0,
                "cache_bytes": self.cache.bytes()}
