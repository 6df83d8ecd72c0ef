"""Built-in architectures; importing this package registers them."""
from . import megovik, naditar, namesun, nununex, qwen3  # noqa: F401
