from .similarity import similarity  # noqa: F401
from .mex import mex  # noqa: F401
