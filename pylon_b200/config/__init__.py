from pylon_b200.config.model_config import ConfigError, Qwen3Config  # noqa: F401
from pylon_b200.config.registry import ARCHITECTURES, Architecture, architecture_of, read_config, register_architecture  # noqa: F401
from pylon_b200.config.engine_config import EngineConfig  # noqa: F401
