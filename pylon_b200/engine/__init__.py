from pylon_b200.engine.engine import Engine, generate  # noqa: F401
from pylon_b200.engine.scheduler import GenerationResult, QueueFullError, Scheduler  # noqa: F401
from pylon_b200.engine.step import StepEntry, StepFunction  # noqa: F401
