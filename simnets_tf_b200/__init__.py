"""B200-native Similarity / MEX operators behind the interface of HUJI-Deep/simnets-tf."""
from . import abi  # noqa: F401
from .ops import mex, similarity  # noqa: F401,E402  (functions, as in the reference's `simnets` package)
