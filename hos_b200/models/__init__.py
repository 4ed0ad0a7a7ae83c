"""Architectures.  Importing this package registers them."""
from . import fobilorn, gemma2, satapel, tofodra, vagonex  # noqa: F401
