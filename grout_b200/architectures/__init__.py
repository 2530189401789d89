"""Architectures known to the library; importing this package registers them."""
from . import mananex, qwen3, sonalorn, suvazen, zutazen  # noqa: F401
