"""SplitMix64, the per-request generator of sampling draws.

One uniform in [0, 1) is drawn per sampled step when the batch is built, never for a
greedy request, so a request's tokens do not depend on what shares its batches
(src/engine/scheduler.rs:326-343 for the generator, :675-687 for the discipline).
"""

from __future__ import annotations

_MASK = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        value = self.state
        value = ((value ^ (value >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        value = ((value ^ (value >> 27)) * 0x94D049BB133111EB) & _MASK
        return value ^ (value >> 31)

    def unit_f64(self) -> float:
        return (self.next_u64() >> 11) * (1.0 / float(1 << 53))
