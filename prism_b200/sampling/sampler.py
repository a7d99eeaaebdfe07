"""Sampling parameters and the device sampler.

andre-fu/prism samples greedily when ``temperature <= 0`` and otherwise with
``softmax(logits / temperature)`` + ``torch.multinomial``
(engine/scheduler.py:266-272, engine/executor.py:423-427); it has no top-k,
top-p or penalties, and neither has this.  Differences: logits are float32,
the first token is sampled like every other (the reference always takes the
argmax there, scheduler.py:219), and the draw is the inverse CDF at a seeded
uniform number (``rng.uniform``) instead of an unseeded multinomial.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops


@dataclass
class SamplingParams:
    """``max_new_tokens`` default 100 as ``Request.max_new_tokens``
    (engine/request_manager.py:24); ``temperature`` 0.0 = greedy (:25)."""
    max_new_tokens: int = 100
    temperature: float = 0.0
    seed: Optional[int] = None
    eos_token_id: Optional[object] = None     # one id or several; None: the model's own
    ignore_eos: bool = False


@dataclass
class SampleHandle:
    event: object
    host_tokens: torch.Tensor
    device_tokens: torch.Tensor


class Sampler:
    """One kernel launch per step for all rows; token ids come back through a
    pinned buffer."""

    def __init__(self, device, max_rows: int = 256):
        self.device = torch.device(device)
        self.max_rows = max_rows
        # two sets of buffers: a step's tokens can still be read while the next step's are written
        self._outs = [torch.empty(max_rows, dtype=torch.int32, device=self.device) for _ in range(2)]
        self._hosts = [torch.empty(max_rows, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._turn = 0

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], us: Sequence[float]) -> List[int]:
        return self.read(self.sample_async(logits, temperatures, us))

    def sample_async(self, logits: torch.Tensor, temperatures: Sequence[float], us: Sequence[float]):
        """Launch the sampling kernel and the copy of the token ids to pinned host
        memory without waiting.  Returns a handle for ``read``; ``handle.device_tokens``
        (int32 ``[R]``) can feed the next step's token ids on the device."""
        R = logits.shape[0]
        if R > self.max_rows:
            self.__init__(self.device, max(R, 2 * self.max_rows))
        self._turn ^= 1
        out, host = self._outs[self._turn][:R], self._hosts[self._turn][:R]
        if any(t > 0 for t in temperatures):
            tu = torch.tensor([list(temperatures), list(us)], dtype=torch.float32, pin_memory=True)
            tu = tu.to(self.device, non_blocking=True)
            ops.sample(logits, tu[0], tu[1], out)
        else:
            ops.sample(logits, None, None, out)
        host.copy_(out, non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return SampleHandle(ev, host, out)

    def read(self, handle) -> List[int]:
        handle.event.synchronize()
        return handle.host_tokens.tolist()
