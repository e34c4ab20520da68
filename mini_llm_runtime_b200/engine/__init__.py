from .admission import BlockReservation, PagedBlockAdmissionController
from .engine import ContinuousBatchEngine, EngineStepResult, GreedyGenerationOutput, greedy_generate
from .metrics import RequestMetricsCollector, RequestTimeline
from .scheduler import (BatchingPolicy, FinishReason, RequestScheduler, RequestState, RequestStatus,
                        ScheduledRequest, SchedulerBatch, SchedulerStepUpdate, WorkKind)
from .step import CacheView, ModelRunner, SamplingRows, Segment, StepContext, StepEntry

__all__ = [
    "BatchingPolicy", "BlockReservation", "CacheView", "ContinuousBatchEngine", "EngineStepResult",
    "FinishReason", "GreedyGenerationOutput", "ModelRunner", "PagedBlockAdmissionController",
    "RequestMetricsCollector", "RequestScheduler", "RequestState", "RequestStatus", "RequestTimeline",
    "SamplingRows", "ScheduledRequest", "SchedulerBatch", "SchedulerStepUpdate", "Segment",
    "StepContext", "StepEntry", "WorkKind", "greedy_generate",
]
