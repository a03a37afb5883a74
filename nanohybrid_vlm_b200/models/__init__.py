"""Built-in architectures.  Importing this package registers them."""
from . import muvonex, nomudra, qwen3  # noqa: F401
