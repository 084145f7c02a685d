"""The step function: one batch of (request, its next tokens) through the model.

``ModelRunner.step`` runs only the tokens it is given, as one batch, from the cache that
earlier steps left, and returns the logits at the wanted places.  Portions of prompts
and single decoded tokens may share a step and a prompt may be cut anywhere.  It is what
generation, the scheduler and trace replay all call; there is no second forward pass.

Reference counterpart: ``Qwen3Model::forward_paged_batch`` and the adapter in front of it
(model/src/qwen3_paged_batch.cpp:44-366, engine/src/qwen3_runner.cpp:11-54).
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass

from typing import Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import models as _models  # noqa: F401  (registers the architectures)
from .. import ops
from ..cache.manager import CacheManager
from ..config.base import ModelConfig, describe_model, load_config
from ..models.model import Model, expected_tensors
from ..weights.loader import load_weights
from .batch import Segment, StepContext, StepEntry

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
          "fp32": torch.float32}


class StepError(ValueError):
    pass


def strict_float32() -> None:
    """Switch the library's reduced-precision matrix modes off (process-wide)."""
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    if hasattr(torch.backends.cuda.matmul, "allow_bf16_reduced_precision_reduction"):
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def load_model(model_path, dtype: torch.dtype, device) -> Tuple[Model, ModelConfig]:
    """Model folder (config.json + safetensors) -> model with weights on ``device``."""
    config = load_config(model_path)
    desc = describe_model(config)
    model = Model(desc, dtype, device)
    expected, ignorable = expected_tensors(desc)
    model.load(load_weights(model_path, expected, dtype, device, ignorable))
    return model, config


def random_model(config: ModelConfig, seed: int, dtype: torch.dtype, device, std: float = 0.02,
                 norm_range=(0.8, 1.2)) -> Model:
    """Random-weights mode without a folder: tensors are drawn on ``device``, part by part."""
    config.validate()
    desc = describe_model(config)
    model = Model(desc, dtype, device)
    expected, _ = expected_tensors(desc)

    class _Lazy(dict):
        def pop(self, name):
            from ..weights.random_init import random_tensor
            store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
            t = random_tensor(name, expected[name], seed, std, norm_range, torch.bfloat16, device)
            return t.to(store)

    model.load(_Lazy())
    return model


@dataclass
class PreparedStep:
    """A step whose pages are reserved and whose rows lie in the runner's host buffer, not yet
    uploaded or launched.  ``late`` lists (entry, place in the host buffer) of tokens that are
    given only when it runs."""
    entries: Sequence[StepEntry]
    commits: List[Tuple[Hashable, int, Sequence[int]]]
    upload: int                                   # int32 words of the host buffer to send
    late: List[Tuple[int, int]]
    ctx: Optional[StepContext] = None             # the general path's context
    graph_key: Optional[Tuple[int, int]] = None   # (rows bucket, context bucket) of a one-token step
    wanted: Optional[List[int]] = None            # rows wanted of a one-token step


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, max_batch_tokens: int = 8192,
                 use_graphs: bool = True, prompt_graphs: bool = False):
        self.model, self.cache = model, cache
        self.use_graphs = use_graphs
        self.prompt_graphs = prompt_graphs and use_graphs
        self._graphs = {}
        # a step may be captured as a CUDA graph only if every launch of it reads the step's data from
        # device buffers: mixers say so themselves (graph_safe = True), other parts may say no
        self._graph_safe = all(
            all(getattr(m, "graph_safe", False) for m in b.mixers())
            and all(getattr(part, "graph_safe", True) for part in b.parts.values() if part not in b.mixers())
            for b in model.blocks)
        self._graph_pool = None
        self._prompt_pool = None
        self._capture_stream = None
        self._prompt_graphs: dict = {}
        self._prompt_seen: dict = {}
        self._graph_logits: Optional[torch.Tensor] = None
        self._checked_calls = 0
        self.device = model.device
        self.vocab = model.desc.vocab_size
        self.max_batch_tokens = int(max_batch_tokens)
        self.is_cuda = torch.device(self.device).type == "cuda"
        strict_float32()
        n = self.max_batch_tokens
        # one packed int32 buffer per step: token ids | positions | slots | wanted rows | segments
        self._host = torch.empty(12 * n + 64, dtype=torch.int32)
        if self.is_cuda:
            self._host = self._host.pin_memory()
        self._dev = torch.empty(12 * n + 64, dtype=torch.int32, device=self.device)
        self._uploaded: Optional[torch.cuda.Event] = None
        self._prepared: Optional[PreparedStep] = None      # the host buffer holds this step

    def check_kernels(self) -> None:
        """Raise if a kernel with bounded waits gave up since the last check (reads a device
        word: call it where the host waits for the step anyway)."""
        if self.is_cuda and ops.tcgen05_calls != self._checked_calls:
            self._checked_calls = ops.tcgen05_calls
            ops.check_error_word(self.device)

    # ------------------------------------------------------------------ requests
    def release(self, request: Hashable) -> None:
        if self.cache.has(request):
            self.cache.release(request)

    # ------------------------------------------------------------------ the step
    def _prepare_general(self, entries: Sequence[StepEntry]) -> PreparedStep:
        """Reserve pages and lay the rows out in the host buffer.  The prepared step holds the
        context and, per entry, (request, length after this step, its tokens) to commit once
        the step has run."""
        seen = set()
        total = wanted = 0
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if len(e.tokens) == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            total += len(e.tokens)
            wanted += len(e.want)
        if total > self.max_batch_tokens:
            raise StepError(f"{total} tokens exceed the step's limit of {self.max_batch_tokens}")
        host = self._host.numpy()
        o_ids, o_pos, o_slot, o_want = 0, total, 2 * total, 3 * total
        o_seg = o_want + wanted
        o_dec = o_seg + 4 * len(entries)
        dec_rows: List[int] = []
        tiles: List[Tuple[int, int, int]] = []      # (segment, offset, last position) per 64 query rows
        if self._uploaded is not None:
            self._uploaded.synchronize()
        segments: List[Segment] = []
        commits: List[Tuple[Hashable, int, Sequence[int]]] = []
        late: List[Tuple[int, int]] = []
        row = n_want = max_ctx = max_seg = 0
        for index, e in enumerate(entries):
            if not self.cache.has(e.request):
                self.cache.admit(e.request)
            toks = np.array(e.tokens, dtype=np.int64)
            if e.late is not None:
                if not 0 <= e.late < len(toks):
                    raise StepError(f"request {e.request!r}: late token {e.late} outside its {len(toks)} tokens")
                toks[e.late] = 0
                late.append((index, o_ids + row + e.late))
            if toks.min() < 0 or toks.max() >= self.vocab:
                raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab})")
            n = len(toks)
            pos0 = self.cache.computed(e.request)
            self.cache.reserve(e.request, pos0 + n)
            slot = self.cache.slot_of(e.request)
            host[o_ids + row:o_ids + row + n] = toks
            host[o_pos + row:o_pos + row + n] = np.arange(pos0, pos0 + n)
            host[o_slot + row:o_slot + row + n] = slot
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.request!r}: wanted place {w} outside its {n} tokens")
                host[o_want + n_want] = row + w
                n_want += 1
            s = len(segments)
            host[o_seg + 4 * s:o_seg + 4 * s + 4] = (slot, row, n, pos0)
            segments.append(Segment(e.request, slot, row, n, pos0))
            if n == 1:
                dec_rows.append(row)
            else:
                tiles += [(s, off, pos0 + min(off + 64, n)) for off in range(0, n, 64)]
            commits.append((e.request, pos0 + n, e.tokens))
            row += n
            max_ctx = max(max_ctx, pos0 + n)
            max_seg = max(max_seg, n)
        n_dec, n_tiles = len(dec_rows), len(tiles)
        o_tiles = o_dec + n_dec
        used = o_tiles + 2 * n_tiles
        host[o_dec:o_tiles] = dec_rows
        # blocks with the most keys start first; those at a multiple of 256 rows lead the list, then
        # those at other multiples of 128, so that its heads are also the lists of 256- and 128-row blocks
        tiles.sort(key=lambda t: (t[1] % 256 != 0, t[1] % 128 != 0, -t[2]))
        n_tiles128 = sum(1 for t in tiles if t[1] % 128 == 0)
        n_tiles256 = sum(1 for t in tiles if t[1] % 256 == 0)
        for i, (s, off, _) in enumerate(tiles):
            host[o_tiles + 2 * i], host[o_tiles + 2 * i + 1] = s, off
        self.cache.sync()
        d = self._dev
        ctx = StepContext(
            tokens=row, token_ids=d[o_ids:o_ids + row], positions=d[o_pos:o_pos + row],
            token_slot=d[o_slot:o_slot + row], want_rows=d[o_want:o_want + n_want],
            segments=segments, seg_info=d[o_seg:o_seg + 4 * len(segments)].view(-1, 4),
            dec_rows=None if n_dec == row else d[o_dec:o_tiles], n_dec=n_dec,
            pf_tiles=d[o_tiles:used].view(-1, 2), n_tiles=n_tiles, n_tiles128=n_tiles128, n_tiles256=n_tiles256,
            decode_only=(max_seg == 1), max_context=max_ctx, max_segment=max_seg)
        return PreparedStep(entries, commits, used, late, ctx=ctx)

    def _upload(self, words: int) -> None:
        if self.is_cuda:
            self._dev[:words].copy_(self._host[:words], non_blocking=True)
            if self._uploaded is None:
                self._uploaded = torch.cuda.Event()
            self._uploaded.record()
        else:
            self._dev[:words].copy_(self._host[:words])

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; logits [wanted, vocab] float32 on the device, in the order of
        the entries and of their ``want`` lists.  The tensor may be reused by the next
        step: read it (or sample from it) before stepping again."""
        return self.run(self.prepare(entries))

    def prepare(self, entries: Sequence[StepEntry]) -> PreparedStep:
        """The host's share of a step, which may be done while the step before it still runs on
        the GPU: checks, pages, the layout of rows, the block tables.  A token marked ``late``
        in its entry is left open.  One prepared step at a time: ``run`` it before the next."""
        if self._prepared is not None:
            raise StepError("a prepared step has not been run yet")
        if not entries:
            raise StepError("a step needs at least one entry")
        if self.use_graphs and self._graphable(entries):
            prepared = self._prepare_graph(entries)
        else:
            prepared = self._prepare_general(entries)
        self._prepared = prepared
        return prepared

    @torch.no_grad()
    def run(self, prepared: PreparedStep, late_tokens: Sequence[int] = (),
            late_source: Optional[Tuple[torch.Tensor, Sequence[int]]] = None) -> torch.Tensor:
        """Upload and launch a prepared step.  Its late tokens are given either as values
        (``late_tokens``, in the order of ``prepared.late``) or, still being sampled by the step
        before, as ``late_source`` = (int32 device tensor of that step's sampled tokens, the row
        of it that each late token is): then they go from there into this step's token ids on
        the device, the host never waits for them, and the entries keep a negative token in
        their place."""
        if prepared is not self._prepared:
            raise StepError("run() takes the step that prepare() returned last")
        self._prepared = None                      # whatever happens below, the host buffer is free again
        host = self._host.numpy()
        n_late, words = len(prepared.late), prepared.upload
        if late_source is not None:
            sampled, rows = late_source
            if len(rows) != n_late:
                raise StepError(f"{n_late} late tokens are open, {len(rows)} rows were named")
            if words + 2 * n_late > host.shape[0]:
                raise StepError("no room for the late tokens' places in the step's buffer")
            host[words:words + n_late] = [place for _, place in prepared.late]
            host[words + n_late:words + 2 * n_late] = rows
            words += 2 * n_late
        else:
            if len(late_tokens) != n_late:
                raise StepError(f"{n_late} late tokens are open, {len(late_tokens)} were given")
            for (index, place), token in zip(prepared.late, late_tokens):
                e = prepared.entries[index]
                if not 0 <= int(token) < self.vocab:
                    raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab})")
                host[place] = int(token)
                e.tokens[e.late] = int(token)          # what commit() hashes
        self._upload(words)
        if late_source is not None and n_late:
            d, at = self._dev, prepared.upload
            ops.feed_tokens(d, d[at:at + n_late], d[at + n_late:at + 2 * n_late], late_source[0])
        if prepared.graph_key is not None:
            logits = self._run_graph(prepared)
        else:
            signature = self._prompt_signature(prepared.ctx)
            if signature is None:
                logits = self.model.forward(prepared.ctx, self.cache)
            else:
                logits = self._step_prompt_graph(signature, prepared.ctx)
        for request, length, tokens in prepared.commits:
            self.cache.commit(request, length, tokens)
        return logits

    def abandon(self, prepared: PreparedStep) -> None:
        """Drop a prepared step without running it (pages it reserved stay with their requests)."""
        if prepared is self._prepared:
            self._prepared = None

    # ------------------------------------------------------------------ repeated prompt steps as CUDA graphs
    # (``prompt_graphs=True``; off unless asked for.)  A step with prompt portions launches fewer,
    # longer kernels, and the host is far ahead of the GPU; still every launch from a stream costs
    # a few microseconds between dependent kernels that a graph node does not (2048 tokens of a
    # Qwen3-8B-sized model: 26.5 ms launched one by one, 25.85 ms replayed).  Under a token budget
    # the same layout of a step comes again and again (a full portion of one prompt, or the same
    # number of decode rows beside one portion), so a layout seen a second time is captured and
    # replayed from then on.  The layout is everything that sizes a grid or places a buffer:
    # tokens, wanted rows, entries, one-token rows, attention blocks, and the context rounded up
    # to a power of two; the values (ids, positions, slots, segments, block tables) are read from
    # the runner's fixed device buffers at replay.
    # Why it is off: in a process that has captured three or more such graphs, decode graphs
    # captured afterwards replay 2% slower (Qwen3-8B sizes, batch 8: 4.19 to 4.22 ms per step
    # instead of 4.10 to 4.12; one or two prompt graphs, or any number of decode graphs, do not do
    # it; whether the prompt graphs still exist makes no difference).  The cause was not found,
    # and decode steps are where a running engine spends its time.
    PROMPT_GRAPHS = 8            # at least two: the pool of the graphs is never left without one
    PROMPT_GRAPH_MIN_TOKENS = 128

    def _prompt_signature(self, ctx: StepContext):
        if not (self.prompt_graphs and self.is_cuda and ctx.tokens >= self.PROMPT_GRAPH_MIN_TOKENS
                and ctx.want_rows.shape[0] <= min(self.GRAPH_MAX_ROWS, self.max_batch_tokens)
                and self._graph_safe):
            return None
        bucket = 256
        while bucket < ctx.max_context:
            bucket *= 2
        ctx.max_context = bucket       # grids that go with the context (key splits) are sized for the bucket
        return (ctx.tokens, int(ctx.want_rows.shape[0]), len(ctx.segments), ctx.n_dec, ctx.n_tiles,
                ctx.n_tiles128, ctx.n_tiles256, bucket)

    def _step_prompt_graph(self, signature, ctx: StepContext) -> torch.Tensor:
        wanted = signature[1]
        held = self._prompt_graphs.get(signature)
        if held is not None:
            graph, kernels, tc_calls = held
            graph.replay()
            ops.launches += kernels
            ops.tcgen05_calls += tc_calls
            return self._graph_logits[:wanted]
        self._prompt_seen[signature] = self._prompt_seen.get(signature, 0) + 1
        if len(self._prompt_seen) > 4096:
            self._prompt_seen.clear()
        logits = self.model.forward(ctx, self.cache)          # this step's result, and the capture's warm-up
        if self._prompt_seen[signature] < 2:
            return logits
        torch.cuda.current_stream().synchronize()
        if self._prompt_pool is None:
            self._prompt_pool = torch.cuda.graph_pool_handle()     # apart from the decode graphs' small buffers
        if self._graph_logits is None:
            rows = min(self.GRAPH_MAX_ROWS, self.max_batch_tokens)
            self._graph_logits = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.device)
        while len(self._prompt_graphs) >= max(2, self.PROMPT_GRAPHS):
            self._prompt_graphs.pop(next(iter(self._prompt_graphs)))      # the oldest
        graph = torch.cuda.CUDAGraph()
        launches, tc_calls = ops.launches, ops.tcgen05_calls
        with self._capturing(graph, self._prompt_pool):
            self._graph_logits[:wanted].copy_(self.model.forward(ctx, self.cache))
        self._prompt_graphs[signature] = (graph, ops.launches - launches, ops.tcgen05_calls - tc_calls)
        ops.launches, ops.tcgen05_calls = launches, tc_calls  # capturing launches nothing
        return logits

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    # A step of single tokens launches some three hundred small kernels; issued one by one
    # from Python they cost more host time than the GPU needs to run them.  Such steps are
    # therefore captured once per (rows rounded up to a power of two, context rounded up to
    # a power of two) and replayed: every kernel reads the step's token ids, positions,
    # slots and block tables from fixed device buffers, rows beyond the real ones carry
    # slot -1 and are skipped, and the attention grid is sized for the context bucket.
    # The same kernels run as in the step-by-step path.
    GRAPH_MAX_ROWS = 256

    def _graphable(self, entries: Sequence[StepEntry]) -> bool:
        return (self.is_cuda and 0 < len(entries) <= self.GRAPH_MAX_ROWS
                and len(entries) <= self.max_batch_tokens
                and all(len(e.tokens) == 1 for e in entries)
                and self._graph_safe)

    def _prepare_graph(self, entries: Sequence[StepEntry]) -> PreparedStep:
        rows = len(entries)
        bucket = 1
        while bucket < rows:
            bucket *= 2
        bucket = min(bucket, self.max_batch_tokens)
        seen = set()
        host = self._host.numpy()
        if self._uploaded is not None:
            self._uploaded.synchronize()
        host[0:bucket] = -1
        host[bucket:2 * bucket] = 0
        host[2 * bucket:3 * bucket] = -1
        host[3 * bucket:4 * bucket] = np.arange(bucket)
        commits, wanted, late, max_ctx = [], [], [], 0
        for i, e in enumerate(entries):
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if e.late is not None:
                if e.late != 0:
                    raise StepError(f"request {e.request!r}: late token {e.late} outside its 1 token")
                tok = 0
                late.append((i, i))
            else:
                tok = int(e.tokens[0])
            if not 0 <= tok < self.vocab:
                raise StepError(f"request {e.request!r}: token id outside [0, {self.vocab})")
            if not self.cache.has(e.request):
                self.cache.admit(e.request)
            pos = self.cache.computed(e.request)
            self.cache.reserve(e.request, pos + 1)
            host[i], host[bucket + i], host[2 * bucket + i] = tok, pos, self.cache.slot_of(e.request)
            for w in e.want:
                if w != 0:
                    raise StepError(f"request {e.request!r}: wanted place {w} outside its 1 token")
                wanted.append(i)
            commits.append((e.request, pos + 1, e.tokens))
            max_ctx = max(max_ctx, pos + 1)
        ctx_bucket = 256
        while ctx_bucket < max_ctx:
            ctx_bucket *= 2
        self.cache.sync()
        return PreparedStep(entries, commits, 4 * bucket, late, graph_key=(bucket, ctx_bucket), wanted=wanted)

    def _run_graph(self, prepared: PreparedStep) -> torch.Tensor:
        key, rows, wanted = prepared.graph_key, len(prepared.entries), prepared.wanted
        if key not in self._graphs:
            self._capture(key)
        graph, kernels = self._graphs[key]
        graph.replay()
        ops.launches += kernels                      # the replay launches what the capture recorded
        logits = self._graph_logits
        if wanted == list(range(rows)):
            return logits[:rows]
        if not wanted:
            return logits[:0]
        return logits[torch.tensor(wanted, device=self.device)]

    @contextlib.contextmanager
    def _capturing(self, graph: "torch.cuda.CUDAGraph", pool):
        """Stream capture into ``graph``.  What ``torch.cuda.graph`` does, without the garbage
        collection and the emptying of the allocator's cache it starts with: giving cached
        blocks back to the driver took 1.4 s per capture beside a 40 GB cache pool, a stall for
        every new batch size of a running engine."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        side = self._capture_stream
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.capture_begin(pool=pool)
            try:
                yield
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(side)

    def _capture(self, key) -> None:
        bucket, ctx_bucket = key
        d = self._dev
        ctx = StepContext(
            tokens=bucket, token_ids=d[0:bucket], positions=d[bucket:2 * bucket],
            token_slot=d[2 * bucket:3 * bucket], want_rows=d[3 * bucket:4 * bucket], segments=[],
            seg_info=None, dec_rows=None, n_dec=bucket, pf_tiles=d[0:0].view(-1, 2), n_tiles=0,
            decode_only=True, max_context=ctx_bucket, max_segment=1)
        self.model.forward(ctx, self.cache)          # warm-up: sizes workspaces, loads kernels
        torch.cuda.current_stream().synchronize()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        if self._graph_logits is None:
            rows = min(self.GRAPH_MAX_ROWS, self.max_batch_tokens)
            self._graph_logits = torch.empty((rows, self.vocab), dtype=torch.float32, device=self.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.launches
        with self._capturing(graph, self._graph_pool):
            # the result goes to a buffer of the runner's own, so that the graphs' private
            # memory can be shared between them
            self._graph_logits[:bucket].copy_(self.model.forward(ctx, self.cache))
        kernels = ops.launches - before
        ops.launches = before                        # capturing launches nothing
        self._graphs[key] = (graph, kernels)
