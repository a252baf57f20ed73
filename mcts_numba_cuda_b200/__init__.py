"""B200-native (sm_100a) implementation of the MCTS-NC search hot path behind the reference's ``MCTSNC`` API."""
from .mctsnc import MCTSNC  # noqa: F401

__all__ = ["MCTSNC"]
