"""Names the reference exports from ``hydraserve.engine`` for the sampling path
(hydraserve/engine/__init__.py:10)."""
from .sampling import SamplingParams, TokenSample, sample_logits  # noqa: F401

__all__ = ["SamplingParams", "TokenSample", "sample_logits"]
