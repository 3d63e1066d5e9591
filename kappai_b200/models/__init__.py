"""Built-in architectures.  Importing this package registers them."""
from . import lfm2  # noqa: F401
