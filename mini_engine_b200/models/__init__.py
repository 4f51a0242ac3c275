"""Built-in architectures; importing this package registers them."""
from . import galupel, gevulorn, logozen, pugadra, qwen3  # noqa: F401
