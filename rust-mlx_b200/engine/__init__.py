from .engine import Engine, EngineError

__all__ = ["Engine", "EngineError"]
