from .block_manager import BlockManager
from .engine import LLMEngine
from .request import Request, SamplingParams, TokenEvent
from .scheduler import Scheduler

__all__ = ["BlockManager", "LLMEngine", "Request", "SamplingParams", "TokenEvent", "Scheduler"]
