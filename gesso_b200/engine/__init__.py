"""Engine: model assembly, the step function, scheduler, session and trace replay."""
from .batch import StepContext, StepEntry, StepLayout
from .engine import DeviceCache, Engine
from .model import CachePlan, Model, PagedView, Runtime, StateView

__all__ = ["StepContext", "StepEntry", "StepLayout", "DeviceCache", "Engine", "CachePlan",
           "Model", "PagedView", "Runtime", "StateView"]
