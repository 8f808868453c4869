"""Architectures the library ships with.  Importing this package registers them."""
from . import llama, ropovik  # noqa: F401  (registration)
