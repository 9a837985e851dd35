"""Architectures known to the library.  Importing this package registers them;
a new one is a new module here that calls `register_architecture`."""
from . import llama  # noqa: F401
