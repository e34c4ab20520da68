from .step import CacheView, ModelRunner, Segment, StepContext, StepEntry

__all__ = ["CacheView", "ModelRunner", "Segment", "StepContext", "StepEntry"]
