"""The built-in architectures; importing this package registers them."""
from . import lefatar, llama  # noqa: F401
