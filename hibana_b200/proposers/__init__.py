"""Draft-token proposers for speculative decoding (engine/contracts.py defines the protocol)."""
from .factory import MAX_DEPTHS, make_proposer  # noqa: F401
