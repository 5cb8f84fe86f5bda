from .params import GREEDY, SamplingParams, uniform_draw
