"""The step function, the scheduler above it, the generation loop and trace replay."""

from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
from paged_kv_serving_b200.engine.sequence import (
    GREEDY_TEMPERATURE, FinishReason, Request, SamplingParams, Sequence, SequenceStatus, SloClass,
    finish_reason_for,
)

__all__ = [
    "GREEDY_TEMPERATURE", "BatchEntry", "ExecutionBatch", "FinishReason", "Request", "SamplingParams",
    "Sequence", "SequenceStatus", "SloClass", "finish_reason_for",
]
