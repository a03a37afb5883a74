"""Built-in architectures.  Importing this package registers them."""
from . import muvonex, qwen3  # noqa: F401
