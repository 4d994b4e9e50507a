"""Architectures. Importing this package registers them."""

from . import bobunex, dibizen, kutirax, qwen2  # noqa: F401
