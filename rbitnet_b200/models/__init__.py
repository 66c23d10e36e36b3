"""Architectures.  Importing this package registers them."""
from . import llama  # noqa: F401
from . import safuvik  # noqa: F401
from . import vaderax  # noqa: F401
from . import nifarax  # noqa: F401
from . import gozotar  # noqa: F401
