from .params import GREEDY, SamplingParams

__all__ = ["GREEDY", "SamplingParams"]
