"""Architectures the library ships with.  Importing this package registers them."""
from . import llama, ropovik, senupel, zotolix  # noqa: F401  (registration)
