"""Names the reference exports from ``hydraserve.engine`` for the sampling path
(hydraserve/engine/__init__.py:10), plus this package's optional extensions."""
from .sampling import (SamplingParams, TokenSample, release_request, sample_logits,  # noqa: F401
                       sample_logits_packed)

__all__ = ["SamplingParams", "TokenSample", "sample_logits", "sample_logits_packed", "release_request"]
