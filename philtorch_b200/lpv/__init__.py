from .recur import LPVRecurrence, linear_recurrence

__all__ = ["LPVRecurrence", "linear_recurrence"]
