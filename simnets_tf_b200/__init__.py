"""B200-native Similarity / MEX operators behind the interface of HUJI-Deep/simnets-tf."""
from . import abi  # noqa: F401
