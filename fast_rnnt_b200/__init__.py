"""B200-native (sm_100a) pruned RNN-T loss: drop-in for the python API of
k2-fsa/fast_rnnt (``import fast_rnnt_b200 as fast_rnnt``).  CUDA tensors only."""
from ._lib import FrnntError  # noqa: F401
from .mutual_information import mutual_information_recursion  # noqa: F401
from .mutual_information import joint_mutual_information_recursion  # noqa: F401


def with_cuda() -> bool:
    """Counterpart of ``_fast_rnnt.with_cuda`` (always True here; raises if the
    CUDA library has not been built)."""
    from . import _lib
    return bool(_lib.lib().frnnt_with_cuda())


__version__ = "1.0.0"
