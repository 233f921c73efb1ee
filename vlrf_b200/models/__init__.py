"""Architectures.  Importing this package registers them."""
from . import gpt2  # noqa: F401
