"""philtorch_b200 -- B200 (sm_100a) kernels for philtorch's differentiable linear-recurrence path.

Drop-in for the recurrence entry points of the reference package: ``lti.linear_recurrence``,
``lpv.linear_recurrence``, ``lti/lpv.state_space_recursion`` and the first/second-order
``lti.lfilter`` / ``lti.filtfilt`` paths, backed by hand-written CUDA kernels behind a C ABI
(``include/philtorch_b200.h``).  CUDA only: importing fails if the compiled library is missing,
and every op raises for CPU tensors.
"""
from . import _lib  # noqa: F401  raises ImportError if libphiltorch_b200.so is not built
from . import ops  # noqa: F401
from . import lti, lpv, prototype  # noqa: F401
from ._lib import check_errors

EXTENSION_LOADED = True
__version__ = "0.1"
__all__ = ["lti", "lpv", "prototype", "ops", "check_errors", "EXTENSION_LOADED"]
