"""Architectures that ship with the package; importing this package registers them."""
from . import dalorax, gpt2, lelatar, nufetar, zuluvik  # noqa: F401
