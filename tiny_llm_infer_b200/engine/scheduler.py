"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees; and decides what happens when pages run out.

Policy of the reference (engine/src/scheduler.cpp:40-160), kept:

* two FIFO queues, ``waiting`` (new, partly computed and preempted requests) and
  ``running`` (prompt fully computed);
* pass 1, decode first: every running request gets one token, in queue order, while the
  step has room; a request that cannot get the page for its next token is *preempted*:
  it gives back everything it holds and goes to the front of ``waiting``; later its
  prompt *and the tokens it had generated* are computed again (no swapping), and since
  the key of a random draw depends only on the request and the token's index, sampling
  goes on as if nothing had happened;
* pass 2, portions of prompts into what is left of the token budget: a request that holds
  nothing is admitted only if all pages of its present length are free (a prompt that
  needs more pages than exist is an error; one that must wait goes to the back); it gets
  ``min(uncomputed tokens, budget left)`` tokens; if that completes it, it moves to
  ``running``, else to the back of ``waiting`` (one portion per request per step);
* a step that schedules nothing while work remains is an error.

Differences: pages are asked of the cache manager (several groups, windows) instead of
a block manager of the scheduler's own; ``max_num_seqs`` bounds the requests that hold a
slot at any time (the reference bounds the requests in one step); the prefix cache
(engine/src/block_manager.cpp:97-125: a prompt's full pages that are already in the cache
are shared, and its first portion starts behind them) lives in the cache manager too;
the booking of a step comes in two halves (``advance`` when it is launched, ``resolve`` when
its tokens are known, ``postprocess`` = both), so that the engine can make and launch the
next step while this one still runs.
"""
from __future__ import annotations

import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, List, Optional, Sequence as Seq

from ..sampling.params import SamplingParams


class SchedulerError(RuntimeError):
    pass


# Stands in a request's tokens for the one that a launched step will sample: its place is
# known (lengths, pages and the next step's layout depend on it), its value is not yet.
PENDING = -1


class Status(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class SchedulerConfig:
    """Names and defaults of the reference (engine/include/scheduler.h:15-21)."""
    max_num_seqs: int = 16
    max_num_batched_tokens: int = 1024
    block_size: int = 16
    num_kv_blocks: int = 128

    def validate(self) -> None:
        for name in ("max_num_seqs", "max_num_batched_tokens", "block_size", "num_kv_blocks"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")


class Sequence:
    """A request: prompt and generated tokens, how many of them are in the cache
    (reference: engine/include/sequence.h:19-54)."""

    def __init__(self, request_id: int, prompt: Seq[int], sampling: SamplingParams):
        self.id = request_id
        self.tokens: List[int] = list(prompt)
        self.prompt_len = len(self.tokens)
        self.sampling = sampling
        self.seed = sampling.seed if sampling.seed else request_id   # engine/src/sequence.cpp:14
        self.status = Status.WAITING
        self.num_cached_tokens = 0
        self.num_scheduled_tokens = 0
        self.preemptions = 0
        self.pending = 0              # how many of the last ``tokens`` are PENDING

    def __len__(self) -> int:
        return len(self.tokens)

    @property
    def completion(self) -> List[int]:
        return self.tokens[self.prompt_len:]

    @property
    def num_completion_tokens(self) -> int:
        return len(self.tokens) - self.prompt_len


@dataclass
class ScheduledSequence:
    sequence: Sequence
    token_start: int
    token_count: int
    is_prefill: bool
    # a row is sampled for a decode token and for the portion that ends the sequence
    # (engine/src/llm_engine.cpp:178-182); fixed when the plan is made
    samples: bool = False
    # where in the request's tokens the sampled token goes (set when the step is launched)
    pending_index: Optional[int] = None


@dataclass
class BatchPlan:
    sequences: List[ScheduledSequence] = field(default_factory=list)
    num_tokens: int = 0
    preempted: List[Sequence] = field(default_factory=list)
    # the two queues as they were before this plan was made (for ``Scheduler.abort``)
    queues_before: Optional[tuple] = None

    @property
    def is_prefill(self) -> bool:
        return bool(self.sequences) and all(s.is_prefill for s in self.sequences)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache):
        """``cache`` is a ``CacheManager`` (only its host bookkeeping is used)."""
        config.validate()
        self.config, self.cache = config, cache
        self.waiting: Deque[Sequence] = deque()
        self.running: Deque[Sequence] = deque()
        self.num_preemptions = 0

    def add(self, sequence: Sequence) -> None:
        if len(sequence) == 0:
            raise ValueError("a request needs at least one token")
        self.waiting.append(sequence)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def _preempt(self, seq: Sequence, plan: BatchPlan) -> None:
        self.cache.release(seq.id)
        seq.status = Status.WAITING
        seq.num_cached_tokens = 0
        seq.num_scheduled_tokens = 0
        seq.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)
        plan.preempted.append(seq)

    def schedule(self) -> BatchPlan:
        """The next step's plan.  Making it moves requests between and inside the queues; if it
        raises, or if the step it describes is never launched (``abort``), those moves are undone."""
        plan = BatchPlan(queues_before=(list(self.running), list(self.waiting)))
        try:
            self._fill(plan)
        except Exception:
            self.abort(plan)
            raise
        return plan

    def abort(self, plan: BatchPlan) -> None:
        """Take back a plan whose step will not run (``advance`` was not called for it, and no
        other plan was made since): the queues are as before it, requests whose prompts it would
        have completed wait again, nothing counts as scheduled.  What making the plan did to the
        cache stays and is consistent by itself: requests it admitted keep their slot and pages,
        requests it preempted stay preempted, at the front of the waiting queue."""
        running, waiting = plan.queues_before
        known = set(map(id, running)) | set(map(id, waiting))
        newcomers = [s for s in self.waiting if id(s) not in known]      # added while the plan was out
        preempted = set(map(id, plan.preempted))
        for item in plan.sequences:
            seq = item.sequence
            seq.num_scheduled_tokens = 0
            if item.is_prefill and seq.status is Status.RUNNING:
                seq.status = Status.WAITING
        self.running = deque(s for s in running if id(s) not in preempted)
        self.waiting = deque(list(reversed(plan.preempted)) + waiting + newcomers)
        plan.sequences, plan.num_tokens = [], 0

    def _fill(self, plan: BatchPlan) -> None:
        budget, max_seqs = self.config.max_num_batched_tokens, self.config.max_num_seqs
        used = 0
        # pass 1: one token for every running request
        for _ in range(len(self.running)):
            if len(plan.sequences) >= max_seqs or used >= budget:
                break
            seq = self.running.popleft()
            if not self.cache.try_reserve(seq.id, len(seq)):
                self._preempt(seq, plan)
                continue
            seq.num_scheduled_tokens = 1
            plan.sequences.append(ScheduledSequence(seq, len(seq) - 1, 1, False, True))
            self.running.append(seq)
            used += 1
        # pass 2: portions of waiting prompts into the rest of the budget
        for _ in range(len(self.waiting)):
            if len(plan.sequences) >= max_seqs or used >= budget:
                break
            seq = self.waiting.popleft()
            if not self.cache.has(seq.id):
                if not self._admit(seq):
                    self.waiting.append(seq)
                    continue
            remaining = len(seq) - seq.num_cached_tokens
            if remaining <= 0:
                raise SchedulerError("a waiting request has nothing left to compute")
            count = min(remaining, budget - used)
            seq.num_scheduled_tokens = count
            plan.sequences.append(ScheduledSequence(seq, seq.num_cached_tokens, count, True,
                                                    seq.num_cached_tokens + count == len(seq)))
            used += count
            if seq.num_cached_tokens + count == len(seq):
                seq.status = Status.RUNNING
                self.running.append(seq)
            else:
                self.waiting.append(seq)
        plan.num_tokens = used
        if not plan.sequences and not self.is_finished():
            raise SchedulerError("no request can be scheduled although some are unfinished: the page pool is "
                                 "too small for any of them to go on")

    def _admit(self, seq: Sequence) -> bool:
        """Slot and all pages of the present length, or nothing."""
        pages = -(-len(seq) // self.cache.page_size)
        for key, capacity in self.cache.capacity_pages().items():
            if pages > capacity:
                raise SchedulerError(f"request {seq.id} needs {pages} pages, the pool has {capacity}")
        if self.cache.free_slots == 0:
            return False
        self.cache.admit(seq.id, seq.tokens)
        if not self.cache.can_reserve(seq.id, len(seq)):
            self.cache.release(seq.id)
            return False
        self.cache.reserve(seq.id, len(seq))
        seq.num_cached_tokens = self.cache.computed(seq.id)     # what the prefix cache already holds
        return True

    def postprocess(self, plan: BatchPlan, sampled: Seq[int], is_eos: Callable[[int], bool]) -> List[Sequence]:
        """Book the step: ``sampled[i]`` is the token of ``plan.sequences[i]`` (-1 where it
        sampled nothing).  Returns the requests that finished."""
        if len(sampled) != len(plan.sequences):
            raise SchedulerError(f"{len(sampled)} sampled tokens for a plan of {len(plan.sequences)} requests")
        self.advance(plan)
        return self.resolve(plan, sampled, is_eos)

    # The booking in two halves, so that the next step can be scheduled, laid out and even
    # launched while this one still runs: what a step changes is known when it is launched, but
    # for the values of the tokens it samples and whether one of them ends its request.

    def advance(self, plan: BatchPlan) -> None:
        """The step has been launched: its tokens count as computed, every request that
        samples grows by a PENDING token, and one that reaches its ``max_tokens`` with it is
        over (its pages are free for the next plan; work already launched comes before
        anything later on the stream)."""
        for item in plan.sequences:
            seq = item.sequence
            seq.num_cached_tokens += seq.num_scheduled_tokens
            seq.num_scheduled_tokens = 0
            if not item.samples:
                continue
            seq.tokens.append(PENDING)
            seq.pending += 1
            item.pending_index = len(seq.tokens) - 1
            if seq.num_completion_tokens >= seq.sampling.max_tokens:
                seq.status = Status.FINISHED
                self.cache.release(seq.id)
                self.running.remove(seq)

    def resolve(self, plan: BatchPlan, sampled: Seq[int], is_eos: Callable[[int], bool]) -> List[Sequence]:
        """The step's tokens are here: ``sampled[i]`` is the token of ``plan.sequences[i]``
        (ignored where it sampled nothing).  Returns the requests that are finished with it.
        Steps are resolved in the order of their launch.  A request that ends on an
        end-of-sequence token may have a row in a step launched meanwhile: that row has run
        for nothing, its PENDING token is dropped here and its result is passed over when that
        step is resolved; the pages can go back at once, since whatever is launched later
        comes later on the stream."""
        if len(sampled) != len(plan.sequences):
            raise SchedulerError(f"{len(sampled)} sampled tokens for a plan of {len(plan.sequences)} requests")
        finished = []
        for item, token in zip(plan.sequences, sampled):
            seq, index = item.sequence, item.pending_index
            if index is None:
                continue
            item.pending_index = None
            if index >= len(seq.tokens):               # the request ended on an earlier token
                continue
            if token < 0:
                raise SchedulerError(f"no token was sampled for request {seq.id}, whose step asked for one")
            seq.tokens[index] = int(token)
            seq.pending -= 1
            self.cache.fill_token(seq.id, index, int(token))
            if not seq.sampling.ignore_eos and is_eos(int(token)):
                del seq.tokens[index + 1:]             # PENDING tokens of steps launched since
                seq.pending = 0
                if seq.status is not Status.FINISHED:  # RUNNING, or WAITING again after a preemption
                    (self.running if seq.status is Status.RUNNING else self.waiting).remove(seq)
                    seq.status = Status.FINISHED
                if self.cache.has(seq.id):
                    self.cache.release(seq.id)
                finished.append(seq)
            elif seq.status is Status.FINISHED and seq.pending == 0:     # by its length, in advance()
                finished.append(seq)
        return finished
