from .sampling_params import BeamSearchParams, JitableSamplingParams, SamplingParams

__all__ = ["SamplingParams", "JitableSamplingParams", "BeamSearchParams"]
