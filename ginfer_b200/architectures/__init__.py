"""Architectures known to the registry; importing this package registers them."""
from . import pimidra, qwen2, vilepel, zolapel  # noqa: F401
