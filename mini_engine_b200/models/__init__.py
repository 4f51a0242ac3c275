"""Built-in architectures; importing this package registers them."""
from . import gevulorn, logozen, pugadra, qwen3  # noqa: F401
