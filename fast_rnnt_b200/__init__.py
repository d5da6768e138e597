"""B200-native (sm_100a) pruned RNN-T loss: drop-in for the python API of
k2-fsa/fast_rnnt (``import fast_rnnt_b200 as fast_rnnt``).  CUDA tensors only;
the same 13 functions plus ``with_cuda`` as the reference's
fast_rnnt/python/fast_rnnt/__init__.py:1-15."""
from ._lib import FrnntError  # noqa: F401
from .mutual_information import mutual_information_recursion  # noqa: F401
from .mutual_information import joint_mutual_information_recursion  # noqa: F401

from .rnnt_loss import do_rnnt_pruning  # noqa: F401
from .rnnt_loss import get_rnnt_logprobs  # noqa: F401
from .rnnt_loss import get_rnnt_logprobs_joint  # noqa: F401
from .rnnt_loss import get_rnnt_logprobs_pruned  # noqa: F401
from .rnnt_loss import get_rnnt_logprobs_smoothed  # noqa: F401
from .rnnt_loss import get_rnnt_prune_ranges  # noqa: F401
from .rnnt_loss import rnnt_loss  # noqa: F401
from .rnnt_loss import rnnt_loss_pruned  # noqa: F401
from .rnnt_loss import rnnt_loss_simple  # noqa: F401
from .rnnt_loss import rnnt_loss_smoothed  # noqa: F401


# additions that have no counterpart in the reference: the caller's joiner on the tensor
# cores, and a way to hand over the host copy of `boundary` that a data loader already has
from .linear import linear, pruned_joiner  # noqa: F401,E402
from .rnnt_loss import get_rnnt_logprobs_pruned_joiner, rnnt_loss_pruned_joiner  # noqa: F401,E402
from .mutual_information import provide_boundary_rows  # noqa: F401,E402


def with_cuda() -> bool:
    """Counterpart of ``_fast_rnnt.with_cuda`` (always True here; raises if the
    CUDA library has not been built)."""
    from . import _lib
    return bool(_lib.lib().frnnt_with_cuda())


__version__ = "1.0.0"
