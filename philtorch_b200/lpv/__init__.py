from .recur import LPVRecurrence, linear_recurrence
from .ssm import MatrixRecurrence, state_space, state_space_recursion
from .filtering import lfilter

__all__ = ["LPVRecurrence", "MatrixRecurrence", "linear_recurrence", "state_space_recursion", "state_space", "lfilter"]
