"""Run-time limits of the engine.

Names, meanings and defaults follow the reference's server options
(src/config.rs:139-186) and their invariants (src/config.rs:193-222); the
projection the engine thread sees is src/config.rs:225-248.  ``kv_capacity_tokens``
is kept as the user-facing unit; the cache manager turns it into pages of
``page_size`` tokens.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineConfig:
    max_queue: int = 256
    max_running: int = 32
    max_batch_tokens: int = 4096
    prefill_chunk_tokens: int = 512
    max_sequence_length: int = 131072
    kv_capacity_tokens: int = 32768
    page_size: int = 16
    dtype: str = "bfloat16"
    device: int = 0
    cuda_graphs: bool = True

    def validate(self) -> None:
        def need(ok: bool, message: str):
            if not ok:
                raise ValueError(message)

        need(self.max_queue > 0, "max_queue must be positive")
        need(self.max_running > 0, "max_running must be positive")
        need(self.max_batch_tokens >= self.max_running, "max_batch_tokens must be at least max_running")
        need(self.prefill_chunk_tokens > 0, "prefill_chunk_tokens must be positive")
        need(self.max_sequence_length > 0, "max_sequence_length must be positive")
        need(self.max_sequence_length < 2**31, "max_sequence_length must fit in a 32-bit position")
        need(self.kv_capacity_tokens >= self.max_running, "kv_capacity_tokens must be at least max_running")
        need(self.page_size >= 16 and self.page_size & (self.page_size - 1) == 0,
             "page_size must be a power of two of at least 16")
        need(self.dtype in ("bfloat16", "float32"), "dtype must be bfloat16 or float32")

    @property
    def max_pending(self) -> int:
        return self.max_queue

    @property
    def num_pages(self) -> int:
        return -(-self.kv_capacity_tokens // self.page_size)
