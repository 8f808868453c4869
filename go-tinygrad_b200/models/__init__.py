"""Architectures the library ships with.  Importing this package registers them."""
from . import llama, ropovik, senupel  # noqa: F401  (registration)
