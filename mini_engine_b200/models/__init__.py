"""Built-in architectures; importing this package registers them."""
from . import logozen, pugadra, qwen3  # noqa: F401
