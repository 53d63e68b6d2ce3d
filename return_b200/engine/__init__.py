from .config import EngineConfig  # noqa: F401
from .request import GenerationResult, Request  # noqa: F401
