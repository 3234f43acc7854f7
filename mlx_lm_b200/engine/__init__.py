from .step import Engine, LayerCacheView, RequestSpan, StepContext, StepEntry, Workspace

__all__ = ["Engine", "LayerCacheView", "RequestSpan", "StepContext", "StepEntry", "Workspace"]
