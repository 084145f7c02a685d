from .params import SamplingParams
from .sampler import Sampler, draw_key
