from pylon_b200.weights.loader import Checkpoint, WeightError  # noqa: F401
from pylon_b200.weights.random_init import random_tensor, write_random_model  # noqa: F401
