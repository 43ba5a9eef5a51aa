from tokasaurus_b200.sampling.params import Request, RequestOutput, SamplingParams, stream_key  # noqa: F401
from tokasaurus_b200.sampling.sampler import Sampler  # noqa: F401
