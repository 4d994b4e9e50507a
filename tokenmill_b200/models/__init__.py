"""Architectures. Importing this package registers them."""

from . import bobunex, dibizen, gofezen, kutirax, qwen2  # noqa: F401
