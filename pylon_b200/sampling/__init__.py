from pylon_b200.sampling.params import SamplingParams  # noqa: F401
from pylon_b200.sampling.sampler import RequestRandom, Sampler  # noqa: F401
