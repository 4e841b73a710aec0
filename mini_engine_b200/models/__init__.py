"""Built-in architectures; importing this package registers them."""
from . import logozen, qwen3  # noqa: F401
