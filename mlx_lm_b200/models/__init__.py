"""Architectures that ship with the package; importing this package registers them."""
from . import gpt2  # noqa: F401
