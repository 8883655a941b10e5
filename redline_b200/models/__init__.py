"""Built-in architectures; importing this package registers them."""

from . import kapitar, llama  # noqa: F401
