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
    def __init__(self, device, max_rows: int):
        self.device = device
        cuda = torch.device(device).type == "cuda"
        self._params_host = torch.empty((max_rows, 2), dtype=torch.float32)
        self._seeds_host = torch.empty(max_rows, dtype=torch.int64)
        if cuda:
            self._params_host = self._params_host.pin_memory()
            self._seeds_host = self._seeds_host.pin_memory()
        # numpy views of the pinned buffers: filled in one go per step, not element by element
        self._params_np = self._params_host.numpy()
        self._seeds_np = self._seeds_host.numpy().view(np.uint64)
        self._params = torch.empty((max_rows, 2), dtype=torch.float32, device=device)
        self._seeds = torch.empty(max_rows, dtype=torch.int64, device=device)
        self._out = torch.empty(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.empty(max_rows, dtype=torch.int32)
        self._done = None
        if cuda:
            self._out_host = self._out_host.pin_memory()
            self._done = torch.cuda.Event()
        self._launched = 0

    def sample(self, logits: torch.Tensor, rows: Sequence[Tuple[float, float, int]]) -> List[int]:
        """``rows[i]`` = (temperature, top_p, draw key) for ``logits[i]``; token ids on the host."""
        self.launch(logits, rows)
        return self.fetch()

    def launch(self, logits: torch.Tensor, rows: Sequence[Tuple[float, float, int]]) -> None:
        """Start the draw and the copy of its result to the host; ``fetch`` waits for it.  The
        host is free in between (the engine prepares its next step there)."""
        n = len(rows)
        assert logits.shape[0] == n
        self._launched = n
        if n == 0:
            return
        temps = [r[0] for r in rows]
        top_ps = [r[1] for r in rows]
        self._params_np[:n, 0] = temps
        self._params_np[:n, 1] = top_ps
        self._seeds_np[:n] = np.fromiter((r[2] & _M for r in rows), dtype=np.uint64, count=n)
        self._params[:n].copy_(self._params_host[:n], non_blocking=True)
        self._seeds[:n].copy_(self._seeds_host[:n], non_blocking=True)
        nucleus = any(t > 1e-6 and p < 1.0 for t, p in zip(temps, top_ps))
        ops.sample(logits, self._params[:n], self._seeds[:n], self._out[:n], any_nucleus=nucleus)
        if self._done is None:
            self._out_host = self._out.cpu()           # no stream to wait for
        else:
            self._out_host[:n].copy_(self._out[:n], non_blocking=True)
            self._done.record()

    def fetch(self) -> List[int]:
        """Token ids of the draw that ``launch`` started."""
        n = self._launched
        if n == 0:
            return []
        if self._done is not None:
            self._done.synchronize()
        return self._out_host[:n].tolist()
