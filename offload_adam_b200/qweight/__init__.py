from .base import QWeightBase

__all__ = ["QWeightBase"]
