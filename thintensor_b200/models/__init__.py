"""Built-in architectures.  Importing this package registers them."""
from . import famalorn, llama  # noqa: F401
