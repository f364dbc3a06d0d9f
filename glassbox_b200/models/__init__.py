"""Architectures. Importing this package registers them."""
from . import babotar, llama, lonorax, tagenex, zurerax  # noqa: F401
