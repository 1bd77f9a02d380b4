"""moonep_b200: Blackwell-native expert-parallel MoE communication library.

Public surface: ``Buffer``, ``MoonEPCommPlan`` (same contract as the reference's
``moonep`` package, moonep/__init__.py:1-9), plus pool helpers, the grouped expert GEMM
and an autograd MoE layer built on them.
"""
from .plan import MoonEPCommPlan
from .engine import MoonEPTimeout

__all__ = ["Buffer", "MoonEPCommPlan", "MoonEPTimeout"]
__version__ = "0.1.0"


def __getattr__(name):
    if name == "Buffer":
        from .api import Buffer
        return Buffer
    raise AttributeError(name)
