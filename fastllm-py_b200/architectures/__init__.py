"""Importing this package registers the architectures the engine ships with."""
from . import lasonex, llama, saberax, sakusun, tigitar  # noqa: F401
