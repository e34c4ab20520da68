from .engine import ContinuousBatchEngine, EngineStepResult, GreedyGenerationOutput, greedy_generate
from .metrics import RequestMetricsCollector, RequestTimeline
from .scheduler import (BatchingPolicy, CacheGate, FinishReason, Request, RequestScheduler, RequestStatus,
                        StepOutcome, StepPlan, WorkItem, WorkKind)
from .step import CacheView, HostBatch, ModelRunner, Segment, StepContext, StepEntry

__all__ = [
    "BatchingPolicy", "CacheGate", "CacheView", "ContinuousBatchEngine", "EngineStepResult", "FinishReason",
    "GreedyGenerationOutput", "HostBatch", "ModelRunner", "Request", "RequestMetricsCollector",
    "RequestScheduler", "RequestStatus", "RequestTimeline", "Segment", "StepContext", "StepEntry",
    "StepOutcome", "StepPlan", "WorkItem", "WorkKind", "greedy_generate",
]
