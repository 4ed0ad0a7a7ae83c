"""Architectures.  Importing this package registers them."""
from . import fobilorn, gemma2, satapel, vagonex  # noqa: F401
