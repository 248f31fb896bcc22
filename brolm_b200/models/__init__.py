"""Architectures this framework knows.  Importing the package registers them."""
from . import gemma2  # noqa: F401
