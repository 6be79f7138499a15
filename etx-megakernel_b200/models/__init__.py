from . import qwen

__all__ = ["qwen"]
