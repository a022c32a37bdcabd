"""Architectures.  Importing this package registers them."""
from . import qwen3  # noqa: F401
from . import tipezen  # noqa: F401  (registration)
from . import dominex  # noqa: F401  (registration)
from . import sadupel  # noqa: F401  (registration)
from . import nugosun  # noqa: F401  (registration)
