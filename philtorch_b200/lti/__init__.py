from .recur import LTIRecurrence, linear_recurrence
from .ssm import LTIMatrixRecurrence, diag_state_space, state_space, state_space_recursion
from .filtering import comb_filter, filtfilt, lfilter, lfilter_zi, sosfilt

__all__ = ["LTIRecurrence", "LTIMatrixRecurrence", "linear_recurrence", "state_space", "state_space_recursion", "diag_state_space",
           "lfilter", "filtfilt", "lfilter_zi", "sosfilt", "comb_filter"]
