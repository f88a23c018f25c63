"""Rank groups and peer-mapped buffers."""
from .peer import PeerGroup, SymmetricBuffer  # noqa: F401
