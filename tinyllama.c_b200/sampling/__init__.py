from .params import GREEDY, SamplingParams  # noqa: F401
from .sampler import Sampler, uniform  # noqa: F401
