from .params import SamplingParams
from .sampler import RequestSamplerState, Sampler
