"""Facts about the one hardware target (hardware/b200.py)."""
from . import b200  # noqa: F401
