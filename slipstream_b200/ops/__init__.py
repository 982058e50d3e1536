"""Hand-written sm_100a kernels and their Python entry points."""

from .functions import *  # noqa: F401,F403
from .functions import __all__  # noqa: F401
