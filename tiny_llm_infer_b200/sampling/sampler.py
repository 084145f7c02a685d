"""Sampling of the next tokens on the device.

One kernel draws a token per wanted row: argmax for greedy rows, the Gumbel-max rule
for temperature rows, restricted to the nucleus when ``top_p`` < 1.  The reference keys
its device sampler with a fresh 64-bit draw from a per-request ``mt19937_64`` at every
step (engine/src/llm_engine.cpp:197-202) and samples top-p rows on the host (:110-145).
Here the key of a draw is a hash of (request seed, index of the token among the
request's outputs): it does not depend on which step or batch the token falls into, nor
on a preemption in between.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np
import torch

from .. import ops

_M = (1 << 64) - 1


def _mix64(z: int) -> int:
    z &= _M
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def draw_key(request_seed: int, output_index: int) -> int:
    """64-bit key of the draw for a request's ``output_index``-th generated token."""
    return _mix64(_mix64(request_seed) + 0x9E3779B97F4A7C15 * (output_index + 1))


class Sampler:
    """Two sets of buffers take turns, so that a draw can be started while the one before it has
    not been read yet (the engine launches a step before it fetches the tokens of the last)."""

    def __init__(self, device, max_rows: int):
        self.device = device
        cuda = torch.device(device).type == "cuda"
        self._sets = [self._buffers(device, max_rows, cuda) for _ in range(2)]
        self._turn = 0

    @staticmethod
    def _buffers(device, max_rows: int, cuda: bool) -> dict:
        b = {"params_host": torch.empty((max_rows, 2), dtype=torch.float32),
             "seeds_host": torch.empty(max_rows, dtype=torch.int64),
             "out_host": torch.empty(max_rows, dtype=torch.int32)}
        if cuda:
            for key in ("params_host", "seeds_host", "out_host"):
                b[key] = b[key].pin_memory()
        # numpy views of the pinned buffers: filled in one go per step, not element by element
        b["params_np"] = b["params_host"].numpy()
        b["seeds_np"] = b["seeds_host"].numpy().view(np.uint64)
        b["params"] = torch.empty((max_rows, 2), dtype=torch.float32, device=device)
        b["seeds"] = torch.empty(max_rows, dtype=torch.int64, device=device)
        b["out"] = torch.empty(max_rows, dtype=torch.int32, device=device)
        b["done"] = torch.cuda.Event() if cuda else None
        b["rows"] = 0
        return b

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[float, float, int]]) -> List[int]:
        """``rows[i]`` = (temperature, top_p, draw key) for ``logits[i]``; token ids on the host."""
        return self.fetch(self.launch(logits, rows))

    def launch(self, logits: torch.Tensor, rows: Sequence[Tuple[float, float, int]]) -> int:
        """Start the draw and the copy of its result to the host; returns the ticket that
        ``fetch`` and ``device_tokens`` take.  A ticket is good until the draw after the next."""
        n = len(rows)
        assert logits.shape[0] == n
        ticket = self._turn
        self._turn ^= 1
        b = self._sets[ticket]
        b["rows"] = n
        if n == 0:
            return ticket
        temps = [r[0] for r in rows]
        top_ps = [r[1] for r in rows]
        b["params_np"][:n, 0] = temps
        b["params_np"][:n, 1] = top_ps
        b["seeds_np"][:n] = np.fromiter((r[2] & _M for r in rows), dtype=np.uint64, count=n)
        b["params"][:n].copy_(b["params_host"][:n], non_blocking=True)
        b["seeds"][:n].copy_(b["seeds_host"][:n], non_blocking=True)
        nucleus = any(t > 1e-6 and p < 1.0 for t, p in zip(temps, top_ps))
        ops.sample(logits, b["params"][:n], b["seeds"][:n], b["out"][:n], any_nucleus=nucleus)
        if b["done"] is None:
            b["out_host"][:n].copy_(b["out"][:n])       # no stream to wait for
        else:
            b["out_host"][:n].copy_(b["out"][:n], non_blocking=True)
            b["done"].record()
        return ticket

    def device_tokens(self, ticket: int) -> torch.Tensor:
        """The int32 device tensor that the draw of this ticket writes its tokens to (row i of the
        draw at index i)."""
        return self._sets[ticket]["out"]

    def fetch(self, ticket: int) -> List[int]:
        """Token ids of the draw that ``launch`` started."""
        b = self._sets[ticket]
        n = b["rows"]
        if n == 0:
            return []
        if b["done"] is not None:
            b["done"].synchronize()
        return b["out_host"][:n].tolist()
