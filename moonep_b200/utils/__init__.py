from .clocks import ClockSampler
from .graphs import GraphedSteps

__all__ = ["ClockSampler", "GraphedSteps"]
