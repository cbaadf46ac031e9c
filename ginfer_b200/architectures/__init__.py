"""Architectures known to the registry; importing this package registers them."""
from . import bapivik, pimidra, qwen2, vilepel, zolapel  # noqa: F401
