"""Architectures the library ships with.  Importing this package registers them."""
from . import llama, megerax, ropovik, senupel, zotolix  # noqa: F401  (registration)
