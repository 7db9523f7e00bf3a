"""Architectures this package knows; importing registers them."""
from . import llama  # noqa: F401
from . import fobilorn  # noqa: F401
from . import nufolix  # noqa: F401
from . import ridopel  # noqa: F401
from . import marinex  # noqa: F401
