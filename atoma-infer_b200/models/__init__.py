"""Architectures built from the parts; importing this package registers them."""
from . import bumolix, dosovik, kulivik, llama, tutezen  # noqa: F401
