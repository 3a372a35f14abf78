"""Importing this package registers the architectures the engine ships with."""
from . import lasonex, llama, sakusun, tigitar  # noqa: F401
