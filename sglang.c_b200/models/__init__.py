"""Architectures.  Importing this package registers the built-in ones."""
from . import gpt2  # noqa: F401
