"""B200-native (sm_100a) per-step token sampler: a drop-in for ``hydraserve.engine.sampling``.

``hydraserve_b200.engine`` mirrors the reference's ``hydraserve.engine`` names for this
path (``SamplingParams``, ``TokenSample``, ``sample_logits``); ``hydraserve_b200.csrc``
holds the CUDA kernels and the C-ABI library they are exported through.
"""
from .engine import SamplingParams, TokenSample, sample_logits  # noqa: F401

__all__ = ["SamplingParams", "TokenSample", "sample_logits"]
