from .clocks import ClockSampler
from .graphs import GraphedSteps
from .health import PeerLost, PeerMonitor

__all__ = ["ClockSampler", "GraphedSteps", "PeerLost", "PeerMonitor"]
