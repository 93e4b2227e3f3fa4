from oxr_inference_b200.sampling.params import Completion, SamplingParams

__all__ = ["Completion", "SamplingParams"]
