"""Samplers: greedy, temperature and nucleus (top-p), with the reference's meanings
(inference/sampler/Sampler.java:56-104 of the reference project: temperature 0 selects the
arg-max; otherwise logits are divided by the temperature, soft-maxed, and a token is drawn by
inverse CDF, over the nucleus when 0 < top_p < 1).

The reference draws from one stateful generator seeded once (Sampler.java:63), so a request's
tokens depend on everything sampled before it.  Here the uniform number of a draw is a pure
function of (seed, request, index of the draw), so a request samples the same tokens whatever
batch it is in."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, request: int, draw: int) -> float:
    """A float32-exact number in [0, 1) that depends only on its three arguments."""
    h = _splitmix64(seed & _MASK)
    h = _splitmix64(h ^ (request & _MASK))
    h = _splitmix64(h ^ (draw & _MASK))
    return (h >> 40) / float(1 << 24)


@dataclass(frozen=True)
class SamplingParams:
    """temperature 0 = greedy.  top_p outside (0, 1) = whole vocabulary.  The reference's defaults
    are temperature 0.1 and top_p 0.95 (Options.java:71-72); the library defaults to greedy."""
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0

    def __post_init__(self):
        if self.temperature < 0:
            raise ValueError("temperature must be non-negative")  # Options.java:14
        if not (0.0 <= self.top_p <= 1.0):
            raise ValueError("top_p must be within [0, 1]")  # Options.java:15

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0


class Sampler:
    """Draws one token per row of device logits with the CUDA sampling kernels."""

    def __init__(self, params: SamplingParams):
        self.params = params

    def sample_device(self, logits: torch.Tensor, requests: list[int], draws: list[int]) -> torch.Tensor:
        """int32 [R] on the device.  ``requests[r]`` and ``draws[r]`` identify row r's draw."""
        out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
        if self.params.greedy:
            ops.argmax_rows(logits, out)
        else:
            u = torch.tensor([uniform(self.params.seed, r, d) for r, d in zip(requests, draws)], dtype=torch.float32)
            ops.sample_rows(logits, u.to(logits.device, non_blocking=True), out, self.params.temperature,
                            self.params.top_p)
        return out

    def sample(self, logits: torch.Tensor, requests: list[int], draws: list[int]) -> list[int]:
        return self.sample_device(logits, requests, draws).tolist()

    # --- for a step function that records the draw together with the model's launches ----------------------
    def launch_key(self):
        """What the recorded launches depend on: a step recorded for one key serves every sampler with it."""
        return ("greedy",) if self.params.greedy else ("sample", float(self.params.temperature), float(self.params.top_p))

    def uniforms(self, requests: list[int], draws: list[int]) -> list[float] | None:
        """The host-side input of one step's draws (none for greedy)."""
        if self.params.greedy:
            return None
        return [uniform(self.params.seed, r, d) for r, d in zip(requests, draws)]

    def sample_into(self, logits: torch.Tensor, uniforms: torch.Tensor | None, out: torch.Tensor) -> None:
        """The kernel launches of ``sample_device`` with every buffer given (nothing is copied or synchronised)."""
        if self.params.greedy:
            ops.argmax_rows(logits, out)
        else:
            ops.sample_rows(logits, uniforms, out, self.params.temperature, self.params.top_p)
