"""Architectures known to the registry.  Importing this package registers them."""
from . import gpt2  # noqa: F401
from . import runesun  # noqa: F401
from . import rizitar  # noqa: F401
from . import pinozen  # noqa: F401
from . import lulizen  # noqa: F401
