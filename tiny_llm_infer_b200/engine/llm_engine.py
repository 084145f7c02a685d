"""``LLMEngine`` (add_request / step / generate / is_finished) and the ``LLM`` entry point.

Mirrors the reference's engine (engine/include/llm_engine.h:14-56,
engine/src/llm_engine.cpp:29-323): requests are validated on entry, a step asks the
scheduler for a plan, flattens it into one batch (decode tokens first, then portions of
prompts), runs the step function, samples on the device and books the result; while the
GPU runs a step, the next one is already scheduled and laid out (its sampled tokens are
filled in when they arrive).  Prompts are token ids; text in and out is an optional extra
through a ``tokenizers`` tokenizer.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq, Union

import torch

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, draw_key
from .batch import StepEntry
from .runner import DTYPES, ModelRunner, PreparedStep, load_model
from .scheduler import BatchPlan, Scheduler, SchedulerConfig, Sequence


@dataclass
class EngineConfig:
    """Reference: engine/include/llm_engine.h:14-18."""
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    max_model_len: int = 2048


@dataclass
class GenerationResult:
    request_id: int
    token_ids: List[int]
    text: str = ""
    prompt_len: int = 0
    preemptions: int = 0


@dataclass
class EngineCounters:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    generated_tokens: int = 0
    preemptions: int = 0
    prefix_cached_tokens: int = 0      # prompt tokens found in the cache instead of computed


@dataclass
class _Step:
    plan: BatchPlan
    step: PreparedStep
    rows: List[tuple]          # (temperature, top_p, draw key) per sampled row
    row_of: List[int]          # the plan's sequence of each sampled row
    late_of: List[int]         # per late token of the prepared step, the request it belongs to
    ticket: int = -1           # of the sampler, once launched


class EngineStopped(RuntimeError):
    """A launched step failed (a kernel refused its arguments, the device reported an error): what
    the cache holds no longer matches what the scheduler has booked, so the engine takes no more
    requests and steps."""


class LLMEngine:
    def __init__(self, runner: ModelRunner, config: EngineConfig, eos_token_ids: Seq[int] = (),
                 detokenize=None, overlap: bool = True):
        if config.max_model_len <= 0:
            raise ValueError("max_model_len must be positive")
        config.scheduler.validate()
        self.runner, self.config = runner, config
        self.scheduler = Scheduler(config.scheduler, runner.cache)
        self.sampler = Sampler(runner.device, config.scheduler.max_num_seqs)
        self.eos = frozenset(int(t) for t in eos_token_ids)
        self.detokenize = detokenize
        self.counters = EngineCounters()
        self._next_id = 1
        self._lock = threading.Lock()      # add_request may come from another thread
        self.overlap = overlap
        self._flying: List[_Step] = []                 # launched, tokens not read yet (at most two)
        self._deferred: Optional[Exception] = None
        self._failed: Optional[Exception] = None       # an error in a launched step: the engine has stopped

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_tokens: Seq[int], sampling: Optional[SamplingParams] = None) -> int:
        """Checks of the reference (engine/src/llm_engine.cpp:41-64)."""
        if self._failed is not None:
            raise EngineStopped(f"the engine stopped after an error in a launched step: {self._failed}")
        sampling = sampling or SamplingParams()
        sampling.validate()
        limit = self.config.max_model_len
        if sampling.max_tokens == 0:
            raise ValueError("max_tokens is 0: a request must ask for at least one token")
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise ValueError("the prompt is empty")
        if len(prompt) > limit:
            raise ValueError(f"the prompt has {len(prompt)} tokens, max_model_len is {limit}")
        if sampling.max_tokens > limit - len(prompt) + 1:
            raise ValueError(f"a prompt of {len(prompt)} tokens leaves room for {limit - len(prompt) + 1} generated "
                             f"tokens under max_model_len {limit}; max_tokens is {sampling.max_tokens}")
        vocab = self.runner.vocab
        if min(prompt) < 0 or max(prompt) >= vocab:
            raise ValueError(f"a prompt token id is outside [0, {vocab})")
        with self._lock:
            request_id = self._next_id
            self._next_id += 1
            self.scheduler.add(Sequence(request_id, prompt, sampling))
        return request_id

    def is_finished(self) -> bool:
        with self._lock:
            return self.scheduler.is_finished() and not self._flying

    @property
    def total_generated_tokens(self) -> int:
        return self.counters.generated_tokens

    # ------------------------------------------------------------------ one step
    def _prepare(self) -> Optional["_Step"]:
        """Ask the scheduler for a plan, flatten it and let the runner lay it out.  A request
        whose last token is still being sampled brings it as a late token."""
        with self._lock:
            plan = self.scheduler.schedule()
        if not plan.sequences:
            return None
        try:
            entries, rows, row_of, late_of = [], [], [], []
            for item in plan.sequences:
                seq = item.sequence
                end = item.token_start + item.token_count
                late = item.token_count - 1 if seq.pending and end == len(seq) else None
                want = [item.token_count - 1] if item.samples else []
                entries.append(StepEntry(seq.id, seq.tokens[item.token_start:end], want, late))
                if item.samples:
                    rows.append((seq.sampling.temperature, seq.sampling.top_p,
                                 draw_key(seq.seed, seq.num_completion_tokens)))
                    row_of.append(len(entries) - 1)
            step = self.runner.prepare(entries)
        except Exception:
            # nothing of the plan has run: take it back, so that the next step starts from the
            # queues as they were (pages reserved meanwhile stay with their requests)
            with self._lock:
                self.scheduler.abort(plan)
            raise
        for index, _ in step.late:                   # whose token each late place waits for
            late_of.append(plan.sequences[index].sequence.id)
        return _Step(plan, step, rows, row_of, late_of)

    def _launch(self, step: "_Step", before: Optional["_Step"]) -> None:
        """Upload and launch; the late tokens are rows of what ``before``, the step launched
        last and not read yet, samples: they stay on the device."""
        try:
            if step.late_of:
                row = {before.plan.sequences[i].sequence.id: r for r, i in enumerate(before.row_of)}
                source = (self.sampler.device_tokens(before.ticket), [row[request] for request in step.late_of])
                logits = self.runner.run(step.step, late_source=source)
            else:
                logits = self.runner.run(step.step)
            step.ticket = self.sampler.launch(logits, step.rows)
        except Exception as error:
            # part of the step may have run and the cache may have booked it: there is no way back
            self.runner.abandon(step.step)
            with self._lock:
                self.scheduler.abort(step.plan)
            self._failed = error
            raise
        with self._lock:
            self.scheduler.advance(step.plan)
        self._flying.append(step)

    def step(self) -> List[GenerationResult]:
        """One step's results.  The steps form a short queue on the GPU: before the tokens of
        the oldest launched step are read, the next one is scheduled, laid out and launched
        too (``overlap``), with the tokens it needs from the step before taken on the device;
        then the oldest step's tokens are read and booked.  So the GPU goes from one step to
        the next without waiting for the host, and the host learns every token one step late."""
        if self._deferred is not None:
            error, self._deferred = self._deferred, None
            raise error
        if self._failed is not None and not self._flying:
            raise EngineStopped(f"the engine stopped after an error in a launched step: {self._failed}")
        if not self._flying:
            first = self._prepare()
            if first is None:
                return []
            self._launch(first, None)
        if self.overlap and len(self._flying) == 1 and self._failed is None:
            try:
                ahead = self._prepare()
                if ahead is not None:
                    self._launch(ahead, self._flying[-1])
            except Exception as error:             # belongs to the next step: raised when it is asked for
                self._deferred = error
        current = self._flying.pop(0)
        plan = current.plan
        tokens = self.sampler.fetch(current.ticket)
        self.runner.check_kernels()
        sampled = [-1] * len(plan.sequences)
        generated = 0
        for idx, tok in zip(current.row_of, tokens):
            sampled[idx] = tok
            item = plan.sequences[idx]
            generated += item.pending_index is not None and item.pending_index < len(item.sequence.tokens)
        with self._lock:
            finished = self.scheduler.resolve(plan, sampled, lambda t: t in self.eos)
        c = self.counters
        c.steps += 1
        c.generated_tokens += generated
        c.preemptions = self.scheduler.num_preemptions
        cache = self.runner.cache
        c.prefix_cached_tokens = cache.prefix_hit_pages * cache.page_size
        for item in plan.sequences:
            if item.is_prefill:
                c.prefill_tokens += item.token_count
            else:
                c.decode_tokens += item.token_count
        out = []
        for seq in finished:
            ids = seq.completion
            text = self.detokenize(ids) if self.detokenize else ""
            out.append(GenerationResult(seq.id, ids, text, seq.prompt_len, seq.preemptions))
        return out

    def generate(self, prompts: Seq[Seq[int]], sampling: Union[SamplingParams, Seq[SamplingParams], None] = None
                 ) -> List[GenerationResult]:
        """All prompts to completion; results in the order of the prompts
        (engine/src/llm_engine.cpp:250-317)."""
        if not prompts:
            return []
        if not self.is_finished():
            raise ValueError("generate() starts from an idle engine: step the requests it holds to their end first")
        if sampling is None or isinstance(sampling, SamplingParams):
            params = [sampling or SamplingParams()] * len(prompts)
        else:
            params = list(sampling)
            if len(params) == 1:
                params = params * len(prompts)
            if len(params) != len(prompts):
                raise ValueError(f"{len(params)} sampling settings for {len(prompts)} prompts: give one, or one each")
        ids = [self.add_request(p, s) for p, s in zip(prompts, params)]
        results: Dict[int, GenerationResult] = {}
        while not self.is_finished():
            for r in self.step():
                results[r.request_id] = r
        return [results[i] for i in ids]


# ---------------------------------------------------------------------- pool sizing
def estimate_num_kv_blocks(model, block_size: int, dtype: torch.dtype, max_num_batched_tokens: int,
                           gpu_memory_utilization: float, device, max_num_seqs: int = 16,
                           memory: Optional[tuple] = None) -> int:
    """Pages that fit beside the weights: budget = total * utilization - used now; a
    reserve of max(256 MiB, total / 20, the step's workspace) stays free (the reference's
    rule, model/src/qwen3.cpp:96-151, with this engine's workspace: what the model's parts
    say they make in a step, ``Model.workspace_floats``).  ``memory``: (free, total) bytes
    instead of asking the device."""
    if not 0.0 < gpu_memory_utilization <= 0.95:
        raise ValueError("gpu_memory_utilization must be in (0, 0.95]")
    free, total = memory if memory is not None else torch.cuda.mem_get_info(device)
    used = total - free
    per_page = sum(CacheManager.bytes_per_page(model.cache_needs(), block_size, dtype).values())
    workspace = 4 * model.workspace_floats(max_num_batched_tokens, min(max_num_seqs, max_num_batched_tokens))
    reserve = max(256 << 20, total // 20, workspace)
    budget = int(total * gpu_memory_utilization) - used - reserve
    return max(0, budget // max(per_page, 1))


class LLM:
    """The Python entry point: a model folder in, generated token ids out.

    Option names follow the reference's command line and engine configuration
    (model/model_main.cpp:403-428, 470-475): ``max_model_len`` (``--max-seq-len``),
    ``num_kv_blocks`` (0: sized from free memory and ``gpu_memory_utilization``),
    ``block_size`` 16, ``max_num_batched_tokens`` min(max_model_len, 256),
    ``max_num_seqs`` 16.  ``enable_prefix_caching`` (on, as in the reference, whose block
    manager always shares hashed pages): prompts that begin like an earlier one reuse its
    full pages; it stays off by itself for models with windows or per-request state.
    ``overlap_scheduling`` (on): the host schedules and lays out a step while the GPU runs
    the one before it; the tokens are the same either way.  ``use_cuda_graphs`` (on): steps of
    one-token rows are replayed as CUDA graphs; ``prompt_graphs`` (off): steps with prompt
    portions whose layout repeats too (faster prompts, slightly slower decoding afterwards).
    """

    def __init__(self, model: str, dtype: str = "bfloat16", max_model_len: int = 2048,
                 num_kv_blocks: int = 0, block_size: int = 16, max_num_batched_tokens: Optional[int] = None,
                 max_num_seqs: int = 16, gpu_memory_utilization: float = 0.9, device: str = "cuda:0",
                 tokenizer: Optional[str] = None, loaded=None, use_cuda_graphs: bool = True,
                 enable_prefix_caching: bool = True, overlap_scheduling: bool = True,
                 prompt_graphs: bool = False):
        if device.startswith("cuda") and not torch.cuda.is_available():
            raise RuntimeError("no CUDA device; this engine has no CPU path")
        torch_dtype = DTYPES[dtype] if isinstance(dtype, str) else dtype
        self.model, self.model_config = loaded if loaded is not None else load_model(model, torch_dtype, device)
        max_model_len = min(int(max_model_len), self.model.desc.max_positions)
        block_size = min(int(block_size), max_model_len)
        if max_num_batched_tokens is None:
            max_num_batched_tokens = min(max_model_len, 256)
        if num_kv_blocks <= 0:
            num_kv_blocks = estimate_num_kv_blocks(self.model, block_size, torch_dtype, max_num_batched_tokens,
                                                   gpu_memory_utilization, device, max_num_seqs)
            cap = -(-max_model_len // block_size) * max_num_seqs
            num_kv_blocks = min(num_kv_blocks, cap)
            if num_kv_blocks <= 0:
                raise RuntimeError("no memory left for the key/value cache")
        self.cache = CacheManager(self.model.cache_needs(), block_size, num_kv_blocks, max_num_seqs,
                                  max_model_len, torch_dtype, device, prefix_cache=enable_prefix_caching)
        self.runner = ModelRunner(self.model, self.cache, max_num_batched_tokens, use_graphs=use_cuda_graphs,
                                  prompt_graphs=prompt_graphs)
        self.tokenizer = None
        if tokenizer:
            from tokenizers import Tokenizer     # optional; text is outside the engine proper
            self.tokenizer = Tokenizer.from_file(tokenizer)
        eos = getattr(self.model_config, "eos_token_ids", ())
        cfg = EngineConfig(SchedulerConfig(max_num_seqs, max_num_batched_tokens, block_size, num_kv_blocks),
                           max_model_len)
        self.engine = LLMEngine(self.runner, cfg, eos,
                                (lambda ids: self.tokenizer.decode(ids)) if self.tokenizer else None,
                                overlap=overlap_scheduling)

    def encode(self, text: str) -> List[int]:
        if self.tokenizer is None:
            raise ValueError("text prompts need a tokenizer file")
        return self.tokenizer.encode(text).ids

    def generate(self, prompts, sampling_params=None) -> List[GenerationResult]:
        """``prompts``: lists of token ids (or strings, with a tokenizer)."""
        ids = [self.encode(p) if isinstance(p, str) else list(p) for p in prompts]
        return self.engine.generate(ids, sampling_params)
