"""What the step function is given: a ragged batch of (request, its next tokens).

Shape and checks follow the reference (src/paged_kv_serving/engine/runner.py:33-87): an entry is
one or more consecutive tokens of one sequence at consecutive absolute positions (a whole
prompt, a portion of one, a single decoded token, a recomputation), with the page table that
covers them; ``logits_at`` lists the places inside the entry whose logits are wanted (the
reference's single ``logits_index`` is the one-element case).
"""

from __future__ import annotations

from dataclasses import dataclass

__all__ = ["BatchEntry", "ExecutionBatch"]


@dataclass(frozen=True, slots=True)
class BatchEntry:
    seq_id: str
    token_ids: tuple[int, ...]
    first_position: int
    block_tables: tuple[tuple[int, ...], ...]       # one table per page group
    logits_at: tuple[int, ...] = ()
    state_slot: int | None = None

    def __post_init__(self) -> None:
        if not self.token_ids:
            raise ValueError("a batch entry must run at least one token")
        if self.first_position < 0:
            raise ValueError("positions start at zero")
        for place in self.logits_at:
            if not 0 <= place < len(self.token_ids):
                raise ValueError("logits_at must point inside the entry")

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def context_len(self) -> int:
        """Valid cached tokens once this entry has been written."""
        return self.first_position + len(self.token_ids)

    @property
    def logits_index(self) -> int | None:
        return self.logits_at[-1] if self.logits_at else None


@dataclass(frozen=True, slots=True)
class ExecutionBatch:
    entries: tuple[BatchEntry, ...]

    @property
    def num_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries)

    @property
    def num_sequences(self) -> int:
        return len(self.entries)

    @property
    def num_prefill_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries if e.num_tokens > 1)

    @property
    def num_logit_rows(self) -> int:
        return sum(len(e.logits_at) for e in self.entries)
