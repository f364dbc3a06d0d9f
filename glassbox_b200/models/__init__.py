"""Architectures. Importing this package registers them."""
from . import llama, lonorax, tagenex, zurerax  # noqa: F401
