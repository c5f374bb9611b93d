from .recur import LTIRecurrence, linear_recurrence

__all__ = ["LTIRecurrence", "linear_recurrence"]
