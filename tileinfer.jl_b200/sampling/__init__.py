from .device import DeviceSampler
from .params import SamplingParams, mix32, sequence_seed
