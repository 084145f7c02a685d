"""One step's batch: (request, its next tokens) entries flattened to rows.

The reference flattens a plan into per-token triples (token id, position, copy of the
whole block table) (engine/src/llm_engine.cpp:164-183) and uploads a dense
``[tokens, max blocks]`` table every step (model/src/qwen3_paged_batch.cpp:87-127).
Here a row carries its token id, its position and the *slot* of its request; block
tables stay on the device, one row per slot, and change only where pages were taken or
given back.  Rows of one entry are consecutive with consecutive positions (a segment).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import torch


@dataclass
class StepEntry:
    """Next tokens of one request, and the places among them whose logits are wanted."""
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()
    # index among ``tokens`` of one token that is not known yet when the step is prepared (the
    # token a step still running will sample); its value is given when the step is run
    late: Optional[int] = None


@dataclass
class Segment:
    request: Hashable
    slot: int
    start: int        # first row of the segment in the step
    length: int
    pos0: int         # position of its first token in the request


@dataclass
class StepContext:
    """Everything a part may look at during a step.  Device tensors are int32; rows past
    ``tokens`` (padding of a fixed-size batch) have token id -1 and slot -1."""
    tokens: int
    token_ids: torch.Tensor       # [rows]
    positions: torch.Tensor       # [rows]
    token_slot: torch.Tensor      # [rows]
    want_rows: torch.Tensor       # [wanted]
    segments: List[Segment]
    seg_info: Optional[torch.Tensor] = None   # [segments, 4] = slot, start, length, pos0
    # rows of one-token segments (None: every row is one) and, for the longer segments,
    # blocks of 64 query rows as (segment, offset) pairs, the first n_tiles128 of which start at
    # multiples of 128 rows and the first n_tiles256 of these at multiples of 256 (the lists of
    # 128- and 256-row blocks); faster attention kernels use them
    dec_rows: Optional[torch.Tensor] = None
    n_dec: int = 0
    pf_tiles: Optional[torch.Tensor] = None
    n_tiles: int = 0
    n_tiles128: int = 0
    n_tiles256: int = 0
    decode_only: bool = False
    max_context: int = 0          # largest position + 1 among the rows
    max_segment: int = 0          # longest segment
    extras: dict = field(default_factory=dict)   # further inputs of the step that some part may need (nobody fills it today)
    # what parts have made for this forward pass and share (the rotary table of the step's positions);
    # emptied by the model at the start of every forward pass, so that a pass recorded as a CUDA graph
    # records the making too
    memo: dict = field(default_factory=dict)
