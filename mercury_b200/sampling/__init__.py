from .params import SamplingParams  # noqa: F401
from .sampler import Sampler, draw_uniform, request_seed  # noqa: F401
