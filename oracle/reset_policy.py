"""CPU oracle for the ReSET step-aware temperature policy. TEST INFRASTRUCTURE ONLY.

Restates reset/reset/logits_processor.py:22-36,62-134 of the reference: token
entropy of softmax(logits), the step-entropy estimate, the running mean of
all entropies, the temperature choice and the temperature scaling. Imported
only by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py``; the shipped package never imports it.

Parity status: pinned. The reference ships no tests or vectors for this
path, so ``tests/golden/make_golden.py`` runs the reference's own
``ReSETRequest`` on seeded logits in a container that holds the reference
and stores per-step (entropy, temperature) plus a checksum of the scaled
logits; ``tests/test_oracle.py`` checks this file against those fixtures.

The entropy is computed with the same float32 torch CPU ops as the
reference so that the two agree bit for bit; the bookkeeping is plain Python
floats (double precision), as in the reference.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


def token_entropy(logits: torch.Tensor) -> float:
    """H = -sum p*log(max(p, 1e-10)), p = softmax(logits), in logits' dtype;
    the result is widened to a Python float (logits_processor.py:32-36)."""
    p = torch.softmax(logits, dim=-1)
    h = -(p * torch.log(torch.clamp(p, min=1e-10))).sum(dim=-1)
    return float(h.item())


def token_entropy_f64(logits: np.ndarray) -> float:
    """Same quantity in float64 (accuracy yardstick, not the reference)."""
    x = np.asarray(logits, dtype=np.float64)
    x = x - x.max()
    e = np.exp(x)
    p = e / e.sum()
    return float(-(p * np.log(np.maximum(p, 1e-10))).sum())


def apply_temperature(logits: torch.Tensor, temp: float) -> torch.Tensor:
    """logits / temp; for temp <= 1e-6 a one-hot row: 0 at the argmax and
    -inf elsewhere (logits_processor.py:22-29)."""
    if temp <= 1e-6:
        out = torch.full_like(logits, float("-inf"))
        out[int(torch.argmax(logits))] = 0.0
        return out
    return logits / temp


@dataclass
class StepDecision:
    """What one call decided, for comparison with the device kernel."""
    entropy: float
    h_step: float
    h_bar: float
    high_step: bool
    temp: float
    boundary: bool


@dataclass
class ResetPolicy:
    """Per-request state and update rule (logits_processor.py:62-134).

    State: ``window_buf`` holds the most recent <= ``window`` entropies
    and is never cleared; ``step_buf`` holds the entropies since the last
    step boundary; ``total``/``count`` give the mean of all entropies.
    """
    t_high: float
    t_low: float
    tau0: float
    window: int = 32
    nl_ids: frozenset = frozenset()
    dnl_ids: frozenset = frozenset()
    window_buf: list = field(default_factory=list)
    step_buf: list = field(default_factory=list)
    total: float = 0.0
    count: int = 0

    def is_boundary(self, output_ids) -> bool:
        """Last id is a double-newline id, or the last two are both newline
        ids (logits_processor.py:91-99)."""
        n = len(output_ids)
        if n == 0:
            return False
        if output_ids[-1] in self.dnl_ids:
            return True
        return n >= 2 and output_ids[-1] in self.nl_ids and output_ids[-2] in self.nl_ids

    def decide(self, boundary: bool, ent: float) -> StepDecision:
        """Everything of ``__call__`` except the entropy and the scaling
        (logits_processor.py:101-132), in the reference's order."""
        if boundary:
            self.step_buf = []
        if len(self.step_buf) < self.window:
            h_step = sum(self.window_buf) / len(self.window_buf) if self.window_buf else ent
        else:
            h_step = sum(self.step_buf) / len(self.step_buf)
        h_bar = self.total / self.count if self.count > 0 else h_step
        high = h_step > h_bar
        threshold = h_step if high else self.tau0
        temp = self.t_high if ent >= threshold else self.t_low
        self.step_buf.append(ent)
        self.window_buf.append(ent)
        if len(self.window_buf) > self.window:
            del self.window_buf[0]
        self.total += ent
        self.count += 1
        return StepDecision(ent, h_step, h_bar, high, temp, boundary)

    def __call__(self, output_ids, logits: torch.Tensor):
        d = self.decide(self.is_boundary(output_ids), token_entropy(logits))
        return apply_temperature(logits, d.temp), d


def synthetic_token_stream(steps: int, delimiter_id: int, vocab: int, seed: int,
                           gap_lo: int = 40, gap_hi: int = 120) -> np.ndarray:
    """Token ids for a synthetic decode loop: random non-delimiter ids with the
    delimiter placed at gaps drawn uniformly from [gap_lo, gap_hi]."""
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab - 1, size=steps, dtype=np.int64)
    ids[ids == delimiter_id] = (delimiter_id + 1) % vocab
    pos = int(rng.integers(gap_lo, gap_hi + 1))
    while pos < steps:
        ids[pos] = delimiter_id
        pos += int(rng.integers(gap_lo, gap_hi + 1))
    return ids


def synthetic_logits(rows: int, vocab: int, seed: int, sigma: float = 3.0,
                     peak: float = 12.0) -> torch.Tensor:
    """[rows, vocab] fp32 N(0, sigma) logits with one token per row raised by
    ``peak`` (stand-in for model logits; no evaluation-suite data involved)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, vocab, generator=g, dtype=torch.float32) * sigma
    idx = torch.randint(0, vocab, (rows,), generator=g)
    x[torch.arange(rows), idx] += peak
    return x
